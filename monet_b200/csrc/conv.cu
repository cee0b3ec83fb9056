// Host side of the tensor-core convolutions: validation, tiling, tap tables,
// tensor maps, workspace accounting and the three C-ABI passes.
//
// Data layout.  Activations are NHWC fp32 (torch.channels_last), filters are
// [K][R][S][C] fp32 (a channels_last weight), gradients alike.  C and K must be
// multiples of 4 (16-byte TMA strides).
//
// Passes
//   fprop  y = conv(x, w) + bias        implicit GEMM, A = x, B = w
//   dgrad  dx = conv^T(dy, w)           implicit GEMM per stride phase, A = dy,
//                                       B = filter transposed to [C][R][S][K]
//                                       in the workspace
//   wgrad  dw = x (*) dy, db = sum dy   see conv_wgrad.cuh
#include "conv_gemm.cuh"
#include "conv_gemm_halo.cuh"
#include "conv_gemm_pair.cuh"
#include "conv_wgrad.cuh"
#include "conv_wgrad_halo.cuh"

#include <cstring>
#include <atomic>
#include <mutex>

namespace mb {


namespace {

// ------------------------------------------------------- driver entry point
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  });
  return fn;
}

// fp32 tensor map, 128-byte swizzle, zero fill.  dims/strides innermost first;
// strides[i] is the byte stride of dims[i+1].
int encode_map(const char* who, CUtensorMap* m, const void* base, int rank, const cuuint64_t* dims,
               const cuuint64_t* strides, const cuuint32_t* box, CUtensorMapSwizzle swizzle) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return fail(MB_ERR_LAUNCH, "%s: cuTensorMapEncodeTiled is not available", who);
  cuuint32_t ones[5] = {1, 1, 1, 1, 1};
  CUresult r = fn(m, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, rank, const_cast<void*>(base), dims, strides,
                  box, ones, CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS)
    return fail(MB_ERR_INVALID_ARGUMENT,
                "%s: tensor map rejected (CUresult %d; rank %d dims %llu %llu %llu %llu box %u %u %u %u)",
                who, static_cast<int>(r), rank, (unsigned long long)dims[0],
                (unsigned long long)dims[1], (unsigned long long)(rank > 2 ? dims[2] : 0),
                (unsigned long long)(rank > 3 ? dims[3] : 0), box[0], box[1], rank > 2 ? box[2] : 0,
                rank > 3 ? box[3] : 0);
  return MB_OK;
}

// NHWC activation view {C, Wv, Hv, Nv} with byte strides of w / h / n.
int encode_act(const char* who, CUtensorMap* m, const float* base, int C, long long Wv, long long Hv,
               long long Nv, long long sw_b, long long sh_b, long long sn_b, int bw, int bh, int bn,
               CUtensorMapSwizzle swizzle = CU_TENSOR_MAP_SWIZZLE_128B) {
  cuuint64_t dims[4] = {(cuuint64_t)C, (cuuint64_t)Wv, (cuuint64_t)Hv, (cuuint64_t)Nv};
  cuuint64_t strides[3] = {(cuuint64_t)sw_b, (cuuint64_t)sh_b, (cuuint64_t)sn_b};
  cuuint32_t box[4] = {(cuuint32_t)kChunkK, (cuuint32_t)bw, (cuuint32_t)bh, (cuuint32_t)bn};
  return encode_map(who, m, base, 4, dims, strides, box, swizzle);
}

// The same view with the channels split into chunks of 32: {32, Wv, Hv, Nv, C/32}, box
// {32, bw, bh, bn, chunks}.  One copy lands `chunks` boxes of bw*bh*bn rows back to back in
// shared memory, which is the operand layout of the backward-filter kernel.  C % 32 == 0.
int encode_act_chunked(const char* who, CUtensorMap* m, const float* base, int C, long long Wv,
                       long long Hv, long long Nv, long long sw_b, long long sh_b, long long sn_b,
                       int bw, int bh, int bn, int chunks, CUtensorMapSwizzle swizzle) {
  cuuint64_t dims[5] = {(cuuint64_t)kChunkK, (cuuint64_t)Wv, (cuuint64_t)Hv, (cuuint64_t)Nv,
                        (cuuint64_t)(C / kChunkK)};
  cuuint64_t strides[4] = {(cuuint64_t)sw_b, (cuuint64_t)sh_b, (cuuint64_t)sn_b,
                           (cuuint64_t)kChunkK * 4};
  cuuint32_t box[5] = {(cuuint32_t)kChunkK, (cuuint32_t)bw, (cuuint32_t)bh, (cuuint32_t)bn,
                       (cuuint32_t)chunks};
  return encode_map(who, m, base, 5, dims, strides, box, swizzle);
}

// Filter view {Cin, taps, Kout} of a [Kout][taps][Cin] array; box {32, 1, rows}.
int encode_filter(const char* who, CUtensorMap* m, const float* base, int Cin, int taps, int Kout,
                  int rows) {
  cuuint64_t dims[3] = {(cuuint64_t)Cin, (cuuint64_t)taps, (cuuint64_t)Kout};
  cuuint64_t strides[2] = {(cuuint64_t)Cin * 4, (cuuint64_t)Cin * taps * 4};
  cuuint32_t box[3] = {(cuuint32_t)kChunkK, 1, (cuuint32_t)rows};
  return encode_map(who, m, base, 3, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
}

// The filter of a backward-data pass read in place: w is [K][taps][C] and the GEMM reduces over
// K, so a tile of `cols` output columns (input channels of the convolution) x 32 k is MN-major:
// view {32, K, taps, C/32}, box {32, 32, 1, cols/32} = cols/32 boxes of [32 k rows][32 columns].
int encode_filter_mn(const char* who, CUtensorMap* m, const float* w, int K, int taps, int C, int cols) {
  cuuint64_t dims[4] = {(cuuint64_t)kChunkK, (cuuint64_t)K, (cuuint64_t)taps, (cuuint64_t)(C / kChunkK)};
  cuuint64_t strides[3] = {(cuuint64_t)taps * C * 4, (cuuint64_t)C * 4, (cuuint64_t)kChunkK * 4};
  cuuint32_t box[4] = {(cuuint32_t)kChunkK, (cuuint32_t)kChunkK, 1, (cuuint32_t)(cols / kChunkK)};
  return encode_map(who, m, w, 4, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B);
}

// ------------------------------------------------------------------- tiling
struct TileShape { int bw, bh, bn; };

// Pixels per tile along w/h/n with bw*bh*bn <= 128, maximising the fraction
// of MMA rows that land on real output pixels.
TileShape pick_tile(int N, int P, int Q) {
  TileShape best{1, 1, 1};
  double best_u = -1.0;
  const int wsplit = (Q + kTileM - 1) / kTileM;
  const int bw = (Q + wsplit - 1) / wsplit;
  for (int bh = 1; bh <= P && bw * bh <= kTileM; ++bh) {
    int bn = 1;
    if (bh == P) {
      bn = kTileM / (bw * bh);
      if (bn > N) bn = N;
      if (bn < 1) bn = 1;
    }
    const double tiles = static_cast<double>((Q + bw - 1) / bw) * ((P + bh - 1) / bh) * ((N + bn - 1) / bn);
    const double u = static_cast<double>(N) * P * Q / (tiles * kTileM);
    if (u > best_u + 1e-9) {
      best_u = u;
      best = TileShape{bw, bh, bn};
    }
  }
  return best;
}

int round_up(int v, int m) { return (v + m - 1) / m * m; }

// Tile width along N and pipeline depth for `kout` output channels.
void pick_bn_stages(int kout, long long m_tiles, int* BN, int* stages, size_t* smem,
                    size_t extra_bytes = 0) {
  int bn = round_up(kout < 256 ? kout : 256, 32);   // whole 32-column chunks for the TMA-store epilogue
  // Narrower tiles only while twice as many still fit in one wave (SMs would sit idle
  // otherwise).  An M = 128 MMA costs about the same for 64 and 128 columns and only 1.6 times as
  // much for 256, and every tile streams the whole K extent of the activation again, so with
  // more than one wave the wide tile wins even when the last wave is half empty (measured:
  // 3x3/2 512->512 at 14x14, 184 wide tiles on 148 SMs 0.13 ms, 736 narrow ones 0.27 ms).
  auto tiles = [&](int b) { return m_tiles * ((kout + b - 1) / b); };
  while (bn > 64 && bn % 64 == 0 && tiles(bn / 2) <= num_sms()) bn /= 2;
  const size_t stage = kAStageBytes + static_cast<size_t>(bn) * 128;
  const size_t staging = 2 * kAStageBytes;            // TMA-store epilogue buffers
  int st = static_cast<int>((220 * 1024 - 2048 - staging - extra_bytes) / stage);
  if (st > 8) st = 8;
  if (st < 2) st = 2;
  *BN = bn;
  *stages = st;
  *smem = 512 + 1024 + stage * st + staging + extra_bytes;
}

long long* g_conv_prof = nullptr;   // diagnostics: device buffer for cycle counters (or null)

struct GemmLaunch {
  CUtensorMap a[4];
  CUtensorMap b;
  CUtensorMap out;
  GemmParams p;
  size_t smem;
  int grid;
};

// Opt a kernel in to 227 KB of dynamic shared memory.  Function attributes belong to a device,
// so what is remembered is one bit per (kernel, device): a process that drives several GPUs sets
// the attribute on each, and a failed attempt is not remembered.
template <class Kernel>
int raise_smem_limit(const char* who, Kernel kernel, std::atomic<unsigned long long>& done) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess)
    return fail(MB_ERR_LAUNCH, "%s: no current CUDA device", who);
  const unsigned long long bit = dev < 64 ? (1ull << dev) : 0ull;
  if (bit && (done.load(std::memory_order_acquire) & bit)) return MB_OK;
  cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
  if (e != cudaSuccess)
    return fail(MB_ERR_LAUNCH, "%s: cannot raise the shared-memory limit: %s", who, cudaGetErrorString(e));
  if (bit) done.fetch_or(bit, std::memory_order_release);
  return MB_OK;
}

int launch_gemm(const char* who, GemmLaunch& L, cudaStream_t st) {
  static std::atomic<unsigned long long> done_plain{0}, done_stats{0};
  if (int rc = raise_smem_limit(who, conv_gemm_kmajor<false>, done_plain)) return rc;
  if (int rc = raise_smem_limit(who, conv_gemm_kmajor<true>, done_stats)) return rc;
  // output view {Kout, Q, P, N} with the tile's box: the epilogue stores whole tiles with TMA
  {
    GemmParams& p = L.p;
    const long long e = 4;
    long long sw = p.out_sw * e, sh = p.out_sh * e, sn = p.out_sn * e;
    if (sh == 0) sh = sw * p.Q;
    if (sn == 0) sn = sh * p.P;
    p.tma_store = (p.BN % 32 == 0 && sw % 16 == 0 && sh % 16 == 0 && sn % 16 == 0) ? 1 : 0;
    if (p.tma_store) {
      int rc = encode_act(who, &L.out, p.out, p.Kout, p.Q, p.P, p.Nimg, sw, sh, sn, p.bw, p.bh, p.bn);
      if (rc) return rc;
    } else {
      L.out = L.b;
    }
  }
  L.p.prof = g_conv_prof;
  if (L.p.stats && !L.p.tma_store)
    return fail(MB_ERR_UNSUPPORTED, "%s: output statistics need the TMA-store epilogue", who);
  // warps 6-13 exist only when the per-channel sums of the output are wanted
  if (L.p.stats)
    conv_gemm_kmajor<true><<<L.grid, 448, L.smem, st>>>(L.a[0], L.a[1], L.a[2], L.a[3], L.b, L.out, L.p);
  else
    conv_gemm_kmajor<false><<<L.grid, 192, L.smem, st>>>(L.a[0], L.a[1], L.a[2], L.a[3], L.b, L.out, L.p);
  return after_launch(who);
}


// ----------------------------------------------------------- halo kernel (stride 1, many taps)
struct HaloTap { int dh, dw, btap; };

// Runs out = sum_t shift(in, dh_t, dw_t) * filter[:, btap_t, :] with the halo kernel.
// Returns MB_ERR_UNSUPPORTED (without setting an error message the caller must keep) when the
// geometry does not fit, so that the caller can fall back to the per-tap kernel.
int run_halo(const char* who, const float* in, int Cin, int Win, int Hin, const float* filt, int T,
             float* out, int Kout, int Qo, int Po, int N, const HaloTap* taps, int ntaps,
             const float* bias, cudaStream_t st, bool filter_mn = false,
             const long long* in_strides = nullptr) {
  // in_strides: byte strides {pixel, row, image} of `in` when it is not a dense NHWC tensor (the
  // overlapping-window view of a few-channel input); Cin is then the length of a window
  if (ntaps < 2 || ntaps > kMaxTaps) return MB_ERR_UNSUPPORTED;
  int min_dh = taps[0].dh, max_dh = taps[0].dh, min_dw = taps[0].dw, max_dw = taps[0].dw;
  for (int t = 1; t < ntaps; ++t) {
    if (taps[t].dh < min_dh) min_dh = taps[t].dh;
    if (taps[t].dh > max_dh) max_dh = taps[t].dh;
    if (taps[t].dw < min_dw) min_dw = taps[t].dw;
    if (taps[t].dw > max_dw) max_dw = taps[t].dw;
  }
  const int halo_h = max_dh - min_dh, halo_w = max_dw - min_dw;
  // 64 output columns, a full 3x3 grid of taps one row above to one row below, rows that fit an
  // M = 128 tile with their halo: two output rows per GEMM row (conv_gemm_pair.cuh)
  if (!in_strides && ntaps == 9 && Kout == 64 && halo_h == 2 && halo_w == 2 && min_dh == -1 && Hin >= 2 && Po >= 2) {
    PairParams q;
    std::memset(&q, 0, sizeof(q));
    bool grid3 = true;
    for (int t = 0; t < 9 && grid3; ++t) {
      const int r = taps[t].dh - min_dh, c = taps[t].dw - min_dw;
      grid3 = r >= 0 && r < 3 && c >= 0 && c < 3 && q.btap[r][c] == 0;
      if (grid3) q.btap[r][c] = static_cast<short>(taps[t].btap + 1);      // +1: 0 marks "not seen yet"
    }
    for (int r = 0; r < 3; ++r)
      for (int c = 0; c < 3; ++c) q.btap[r][c] = static_cast<short>(q.btap[r][c] - 1);
    if (grid3) {
      const int pairs = (Po + 1) / 2;
      q.bias = bias; q.Kout = Kout; q.kchunks = (Cin + kChunkK - 1) / kChunkK;
      // whole rows in a tile when they fit; else the column tiling with the most useful MMA rows
      q.tiles_w = 1; q.bw = Qo;
      if (Qo + 2 > kTileM) {
        double best = 0.0;
        for (int bw = 14; bw <= kTileM - 2; ++bw) {
          const int tw = (Qo + bw - 1) / bw, j = kTileM / (bw + 2);
          const double eff = static_cast<double>(j) * Qo / (static_cast<double>(kTileM) * tw);
          if (eff > best + 1e-9) { best = eff; q.tiles_w = tw; q.bw = bw; }
        }
        q.bw = (Qo + q.tiles_w - 1) / q.tiles_w;          // balanced
      }
      q.Wh = q.bw + 2;
      const int jmax = kTileM / q.Wh;
      q.MT = pairs > jmax ? 2 : 1;                       // two M tiles share every filter tile
      q.tiles_h = (pairs + jmax * q.MT - 1) / (jmax * q.MT);
      q.J = (pairs + q.tiles_h * q.MT - 1) / (q.tiles_h * q.MT);
      q.Hb = q.MT * q.J + 1;
      q.box_rows = q.Wh * q.Hb;
      q.a_half = (q.box_rows * 128 + 1023) / 1024 * 1024;
      q.out_rows = q.Wh * q.J;
      q.org_w = min_dw;
      q.rows_even = (Po + 1) / 2; q.rows_odd = Po / 2;
      q.b_mn = filter_mn ? 1 : 0;
      q.prof = g_conv_prof;
      q.a_stages = 2;
      const size_t budget = 222 * 1024 - 2048;
      const size_t staging = (static_cast<size_t>(q.out_rows) * 128 + 1023) / 1024 * 1024;
      const size_t fixed = 2 * 2 * static_cast<size_t>(q.a_half) + staging;
      const long long items = static_cast<long long>(q.tiles_h) * q.tiles_w * N;
      if (fixed + 5 * 8192 <= budget && items <= 0x7fffffffLL) {
        q.b_stages = 3;                                    // the three filter slots of a filter column
        q.num_items = static_cast<int>(items);
        const size_t smem = 512 + 1024 + fixed + 5 * 8192;
        const long long C4 = static_cast<long long>(Cin) * 4, K4 = static_cast<long long>(Kout) * 4;
        CUtensorMap me, mo_in, mb2, moe, moo;
        int rc = encode_act(who, &me, in, Cin, Win, (Hin + 1) / 2, N, C4, 2 * C4 * Win, C4 * Win * Hin, q.Wh, q.Hb, 1);
        if (rc) return rc;
        rc = encode_act(who, &mo_in, in + static_cast<long long>(Win) * Cin, Cin, Win, Hin / 2, N, C4, 2 * C4 * Win,
                        C4 * Win * Hin, q.Wh, q.Hb, 1);
        if (rc) return rc;
        rc = filter_mn ? encode_filter_mn(who, &mb2, filt, Cin, T, Kout, 64) : encode_filter(who, &mb2, filt, Cin, T, Kout, 64);
        if (rc) return rc;
        const int sbw = q.tiles_w == 1 ? q.Wh : q.bw, sbh = q.tiles_w == 1 ? q.J : 1;   // store box
        rc = encode_act(who, &moe, out, Kout, Qo, (Po + 1) / 2, N, K4, 2 * K4 * Qo, K4 * Qo * Po, sbw, sbh, 1);
        if (rc) return rc;
        rc = encode_act(who, &moo, out + static_cast<long long>(Qo) * Kout, Kout, Qo, Po / 2, N, K4, 2 * K4 * Qo,
                        K4 * Qo * Po, sbw, sbh, 1);
        if (rc) return rc;
        static std::atomic<unsigned long long> pair_smem_done{0};
        if (int rc2 = raise_smem_limit(who, conv_gemm_pair, pair_smem_done)) return rc2;
        const int grid = q.num_items < num_sms() ? q.num_items : num_sms();
        conv_gemm_pair<<<grid, 192, smem, st>>>(me, mo_in, mb2, moe, moo, q);
        return after_launch("conv_gemm_pair");
      }
    }
  }
  // Geometry of one candidate: the map cut into `tw` column tiles.  Returns the fraction of MMA
  // rows that are real output pixels, or 0 when the candidate does not fit (TMA box limits, two
  // accumulators, shared memory).
  const size_t budget = 222 * 1024 - 2048;
  auto plan = [&](int tw, HaloParams& p) -> double {
    std::memset(&p, 0, sizeof(p));
    const int rows_cap = 2 * kTileM;
    p.tiles_w = tw;
    p.bw = (Qo + tw - 1) / tw;
    p.Wh = p.bw + halo_w;
    p.row_stores = (tw > 1 && halo_w > 0) ? 1 : 0;     // without a column halo the tile is the store box
    p.Po = Po;
    if (p.Wh > 256) return 0.0;
    if (tw == 1 && (Po + halo_h) * p.Wh <= rows_cap) {        // whole (padded) images, several per super-tile
      p.Hb = Po + halo_h;
      p.bn = rows_cap / (p.Hb * p.Wh);
      if (p.bn > N) p.bn = N;
      p.bh = Po;
      p.tiles_h = 1;
      p.Hout = p.bn > 1 ? p.Hb : p.bh;
    } else {
      p.bn = 1;
      const int bh_max = rows_cap / p.Wh;
      if (bh_max < 1) return 0.0;
      p.tiles_h = (Po + bh_max - 1) / bh_max;
      p.bh = (Po + p.tiles_h - 1) / p.tiles_h;
      p.Hb = p.bh + halo_h;
      p.Hout = p.bh;
    }
    if (p.Hb > 256) return 0.0;
    p.tiles_n = (N + p.bn - 1) / p.bn;
    p.box_rows = p.Wh * p.Hb * p.bn;
    p.out_rows = p.Wh * p.Hout * p.bn;
    const int span = ((p.bn - 1) * p.Hb + p.bh) * p.Wh;
    p.MT = ((span > p.out_rows ? span : p.out_rows) + kTileM - 1) / kTileM;
    if (p.MT > 2) return 0.0;
    const int max_off = halo_h * p.Wh + halo_w;
    int need_rows = p.MT * kTileM + max_off;
    if (need_rows < p.box_rows) need_rows = p.box_rows;
    p.a_rows_alloc = (need_rows + 7) / 8 * 8;
    p.BN = Kout >= 256 ? 256 : round_up(Kout, 32);
    const size_t a_slot = static_cast<size_t>(p.a_rows_alloc) * 128;
    const size_t staging = (static_cast<size_t>(p.out_rows) * 128 + 1023) / 1024 * 1024;
    if (2 * a_slot + staging + 2 * static_cast<size_t>(p.BN) * 128 > budget) {
      if (p.BN != 256 || 2 * a_slot + staging + 2 * static_cast<size_t>(128) * 128 > budget) return 0.0;
      p.BN = 128;                                   // narrower filter tiles leave room for the halo box
    }
    return static_cast<double>(Qo) * Po * N /
           (static_cast<double>(p.tiles_w) * p.tiles_h * p.tiles_n * p.MT * kTileM);
  };
  // One column tile (the whole row in the box) unless that does not fit or wastes more than 30 %
  // of the MMA rows and a tiling recovers at least 15 points: maps wider than a TMA box (256
  // pixels), and wide maps whose single output row already spills into a second accumulator.
  HaloParams p;
  double eff = plan(1, p);
  if (halo_w == 0) {
    // taps that differ in their row only: column tiles cost nothing (no halo columns), and a
    // narrow tile can be tall, which is what saves input traffic (bh + halo_h rows are fetched
    // for bh rows of output).  Take the tiling with the most useful work per fetched row.
    HaloParams q;
    double best = eff > 0.0 ? eff * p.bh / (p.bh + halo_h) : 0.0;
    int best_tw = 1;
    for (int tw = 2; tw <= (Qo + 7) / 8; ++tw) {
      const double e = plan(tw, q);
      const double score = e > 0.0 ? e * q.bh / (q.bh + halo_h) : 0.0;
      if (score > best + 1e-9) { best = score; best_tw = tw; }
    }
    eff = plan(best_tw, p);
  } else if (eff < 0.7) {
    HaloParams q;
    double best = eff;
    int best_tw = 1;
    for (int tw = 2; tw <= (Qo + 7) / 8; ++tw) {
      const double e = plan(tw, q);
      if (e > best + 1e-9) { best = e; best_tw = tw; }
    }
    if (best_tw > 1 && (eff == 0.0 || best >= eff + 0.15)) eff = plan(best_tw, p);
    else if (eff > 0.0) eff = plan(1, p);
  }
  if (eff == 0.0) return MB_ERR_UNSUPPORTED;
  p.bias = bias;
  p.Kout = Kout;
  p.tiles_c = (Kout + p.BN - 1) / p.BN;
  if (p.BN == 256) {
    // 128-column tiles when they fill the SMs' rounds better: an M = 128 MMA takes about 140
    // cycles with 256 columns and 86 with 128 in this kernel, and a round costs its MMAs
    const long long pix_items = static_cast<long long>(p.tiles_h) * p.tiles_w * p.tiles_n;
    const long long rounds256 = (pix_items * p.tiles_c + num_sms() - 1) / num_sms();
    const int tiles128 = (Kout + 127) / 128;
    const long long rounds128 = (pix_items * tiles128 + num_sms() - 1) / num_sms();
    if (rounds128 * 86 < rounds256 * 140) {
      p.BN = 128;
      p.tiles_c = tiles128;
    }
  }
  p.kchunks = (Cin + kChunkK - 1) / kChunkK;
  p.num_taps = ntaps;
  p.org_w = min_dw; p.org_h = min_dh;
  for (int t = 0; t < ntaps; ++t) {
    p.tap_off[t] = static_cast<short>((taps[t].dh - min_dh) * p.Wh + (taps[t].dw - min_dw));
    p.btap[t] = static_cast<unsigned char>(taps[t].btap);
  }
  p.acc_bufs = 2 * p.MT * p.BN <= 512 ? 2 : 1;
  p.prof = g_conv_prof;
  p.a_stages = 2;
  const size_t a_slot = static_cast<size_t>(p.a_rows_alloc) * 128, b_slot = static_cast<size_t>(p.BN) * 128;
  const size_t staging = (static_cast<size_t>(p.out_rows) * 128 + 1023) / 1024 * 1024;
  if (2 * a_slot + staging + 2 * b_slot > budget) return MB_ERR_UNSUPPORTED;
  int bs = static_cast<int>((budget - 2 * a_slot - staging) / b_slot);
  if (bs > 16) bs = 16;
  p.b_stages = bs;
  const long long items = static_cast<long long>(p.tiles_h) * p.tiles_w * p.tiles_n * p.tiles_c;
  if (items > 0x7fffffffLL) return MB_ERR_UNSUPPORTED;
  p.num_items = static_cast<int>(items);
  const size_t smem = 512 + 1024 + 2 * a_slot + bs * b_slot + staging;

  CUtensorMap ma, mb_, mo;
  const long long C4 = static_cast<long long>(Cin) * 4, K4 = static_cast<long long>(Kout) * 4;
  int rc = in_strides ? encode_act(who, &ma, in, Cin, Win, Hin, N, in_strides[0], in_strides[1], in_strides[2],
                                   p.Wh, p.Hb, p.bn)
                      : encode_act(who, &ma, in, Cin, Win, Hin, N, C4, C4 * Win, C4 * Win * Hin, p.Wh, p.Hb, p.bn);
  if (rc) return rc;
  p.b_mn = filter_mn ? 1 : 0;
  rc = filter_mn ? encode_filter_mn(who, &mb_, filt, Cin, T, Kout, p.BN)
                 : encode_filter(who, &mb_, filt, Cin, T, Kout, p.BN);
  if (rc) return rc;
  rc = p.row_stores ? encode_act(who, &mo, out, Kout, Qo, Po, N, K4, K4 * Qo, K4 * Qo * Po, p.bw, 1, 1)
                    : encode_act(who, &mo, out, Kout, Qo, Po, N, K4, K4 * Qo, K4 * Qo * Po, p.Wh, p.Hout, p.bn);
  if (rc) return rc;
  static std::atomic<unsigned long long> smem_done{0};
  if (int rc = raise_smem_limit(who, conv_gemm_halo, smem_done)) return rc;
  const int grid = p.num_items < num_sms() ? p.num_items : num_sms();
  conv_gemm_halo<<<grid, 192, smem, st>>>(ma, mb_, mo, p);
  return after_launch("conv_gemm_halo");
}

int floordiv(int a, int b) { return (a >= 0) ? a / b : -((-a + b - 1) / b); }
int posmod(int a, int b) { return a - floordiv(a, b) * b; }

int validate(const char* who, const mb_conv_desc* d) {
  if (!d) return fail(MB_ERR_INVALID_ARGUMENT, "%s: null descriptor", who);
  if (d->N <= 0 || d->C <= 0 || d->H <= 0 || d->W <= 0 || d->K <= 0 || d->R <= 0 || d->S <= 0)
    return fail(MB_ERR_INVALID_ARGUMENT, "%s: bad extent", who);
  if (d->stride_h <= 0 || d->stride_w <= 0 || d->dil_h <= 0 || d->dil_w <= 0 || d->pad_h < 0 || d->pad_w < 0)
    return fail(MB_ERR_INVALID_ARGUMENT, "%s: bad stride / dilation / padding", who);
  const int P = (d->H + 2 * d->pad_h - d->dil_h * (d->R - 1) - 1) / d->stride_h + 1;
  const int Q = (d->W + 2 * d->pad_w - d->dil_w * (d->S - 1) - 1) / d->stride_w + 1;
  if (P <= 0 || Q <= 0 || P != d->P || Q != d->Q)
    return fail(MB_ERR_INVALID_ARGUMENT, "%s: output extent %dx%d does not match the geometry (%dx%d)",
                who, d->P, d->Q, P, Q);
  if (d->groups != 1)
    return fail(MB_ERR_UNSUPPORTED, "%s: groups=%d (grouped convolution runs the depthwise kernels)", who, d->groups);
  if (d->C % 4 || d->K % 4)
    return fail(MB_ERR_UNSUPPORTED, "%s: C=%d and K=%d must be multiples of 4", who, d->C, d->K);
  if (d->R * d->S > kMaxTaps)
    return fail(MB_ERR_UNSUPPORTED, "%s: %dx%d filter has more than %d taps", who, d->R, d->S, kMaxTaps);
  if (d->stride_h > 2 || d->stride_w > 2)
    return fail(MB_ERR_UNSUPPORTED, "%s: stride above 2", who);
  return MB_OK;
}

bool is_pointwise(const mb_conv_desc* d) {
  return d->R == 1 && d->S == 1 && d->stride_h == 1 && d->stride_w == 1 && d->pad_h == 0 && d->pad_w == 0;
}

__global__ void __launch_bounds__(256) transpose_filter(const float* __restrict__ w,
                                                        float* __restrict__ wt, int K, int T, int C) {
  // wt[c][t][k] = w[k][t][c]
  const size_t total = static_cast<size_t>(K) * T * C;
  for (size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<size_t>(gridDim.x) * blockDim.x) {
    const int k = static_cast<int>(i % K);
    const size_t r = i / K;
    const int t = static_cast<int>(r % T);
    const int c = static_cast<int>(r / T);
    wt[i] = __ldg(w + (static_cast<size_t>(k) * T + t) * C + c);
  }
}

}  // namespace
}  // namespace mb

namespace mb {

// Shared head and tail of the wgrad entry points.  `prepare` zeroes dw (variant 0) or checks
// the partial-sum workspace (variant 1) and says where the kernel writes; `finish` reduces the
// partials and computes the bias gradient.
int wgrad_prepare(const char* who, int variant, int splits, bool all_taps_written, float* dw,
                  size_t dw_elems, void* workspace, size_t workspace_bytes, cudaStream_t st,
                  float** out, long long* split_stride) {
  if (variant == 0) {
    if (cudaMemsetAsync(dw, 0, dw_elems * sizeof(float), st) != cudaSuccess)
      return fail(MB_ERR_LAUNCH, "%s: memset failed", who);
    *out = dw;
    *split_stride = 0;
    return MB_OK;
  }
  const size_t need = static_cast<size_t>(splits) * dw_elems * sizeof(float);
  if (!workspace || workspace_bytes < need || !aligned(workspace, 16))
    return fail(MB_ERR_WORKSPACE, "%s: workspace of %zu bytes needed, %zu given", who, need,
                workspace ? workspace_bytes : size_t(0));
  if (!all_taps_written && cudaMemsetAsync(workspace, 0, need, st) != cudaSuccess)
    return fail(MB_ERR_LAUNCH, "%s: memset failed", who);
  *out = static_cast<float*>(workspace);
  *split_stride = static_cast<long long>(dw_elems);
  return MB_OK;
}

int wgrad_finish(const char* who, int variant, int splits, const float* dy, float* dw,
                 size_t dw_elems, float* dbias, const mb_conv_desc* d, const void* workspace,
                 cudaStream_t st) {
  int rc;
  if (variant == 1) {
    wgrad_reduce_splits<<<grid_for(dw_elems, 256, 8), 256, 0, st>>>(static_cast<const float*>(workspace), dw, dw_elems, splits);
    rc = after_launch("conv_wgrad_reduce");
    if (rc) return rc;
  }
  if (dbias) {
    if (cudaMemsetAsync(dbias, 0, static_cast<size_t>(d->K) * sizeof(float), st) != cudaSuccess)
      return fail(MB_ERR_LAUNCH, "%s: memset failed", who);
    const size_t pixels = static_cast<size_t>(d->N) * d->P * d->Q;
    int chunks = static_cast<int>((pixels + 2047) / 2048);
    const int cap = 4 * num_sms() / ((d->K + 31) / 32) + 1;
    if (chunks > cap) chunks = cap;
    dim3 grid((d->K + 31) / 32, chunks);
    bias_grad_kernel<<<grid, 256, 0, st>>>(dy, dbias, pixels, d->K);
    rc = after_launch("conv_bias_grad");
    if (rc) return rc;
  }
  return MB_OK;
}

int wgrad_launch(const char* who, wg::Plan& pl, const CUtensorMap& mdy, const CUtensorMap* mx,
                 const float* dy, float* dw, size_t dw_elems, float* dbias, const mb_conv_desc* d,
                 int variant, void* workspace, size_t workspace_bytes, cudaStream_t st) {
  WgradParams& p = pl.p;
  int rc = wgrad_prepare(who, variant, p.splits, p.ntaps >= p.T, dw, dw_elems, workspace,
                         workspace_bytes, st, &p.out, &p.split_stride);
  if (rc) return rc;
  static std::atomic<unsigned long long> smem_done{0};
  if (int rc = raise_smem_limit(who, conv_wgrad_tcgen05, smem_done)) return rc;
  p.prof = g_conv_prof;
  conv_wgrad_tcgen05<<<pl.grid, 192, pl.smem, st>>>(mdy, mx[0], mx[1], mx[2], mx[3], p);
  rc = after_launch("conv_wgrad_tcgen05");
  if (rc) return rc;
  return wgrad_finish(who, variant, p.splits, dy, dw, dw_elems, dbias, d, workspace, st);
}

// Multi-tap filters: the halo kernel (one x box per tile, taps by descriptor offset), one
// launch per stride phase.
int wgrad_run_halo(const char* who, wgh::Launches& hl, const float* x, const float* dy, float* dw,
                   float* dbias, const mb_conv_desc* d, int variant, void* workspace,
                   size_t workspace_bytes, cudaStream_t st) {
  const CUtensorMapSwizzle kWg = CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B;
  const size_t dw_elems = static_cast<size_t>(d->K) * d->R * d->S * d->C;
  float* out = nullptr;
  long long split_stride = 0;
  int covered = 0;
  for (int i = 0; i < hl.n; ++i) covered += hl.plan[i].p.ntaps;
  int rc = wgrad_prepare(who, variant, hl.plan[0].p.splits, covered >= d->R * d->S, dw, dw_elems, workspace,
                         workspace_bytes, st, &out, &split_stride);
  if (rc) return rc;
  static std::atomic<unsigned long long> smem_done{0};
  if (int rc = raise_smem_limit(who, conv_wgrad_halo_tcgen05, smem_done)) return rc;
  const long long K4 = static_cast<long long>(d->K) * 4, C4 = static_cast<long long>(d->C) * 4;
  for (int i = 0; i < hl.n; ++i) {
    WgHaloParams& p = hl.plan[i].p;
    p.out = out;
    p.split_stride = split_stride;
    const int a = hl.phase_a[i], b = hl.phase_b[i];
    CUtensorMap mdy, mx;
    rc = encode_act(who, &mdy, dy, d->K, d->Q, d->P, d->N, K4, K4 * d->Q, K4 * d->Q * d->P,
                    p.row_loads ? p.bw : p.Wh, p.row_loads ? 1 : p.bh, 1, kWg);
    if (rc) return rc;
    const long long Wv = (d->W - b + d->stride_w - 1) / d->stride_w;
    const long long Hv = (d->H - a + d->stride_h - 1) / d->stride_h;
    rc = encode_act(who, &mx, x + (static_cast<long long>(a) * d->W + b) * d->C, d->C, Wv, Hv, d->N,
                    C4 * d->stride_w, C4 * d->W * d->stride_h, C4 * d->W * d->H, p.Wh, p.bhB, 1, kWg);
    if (rc) return rc;
    conv_wgrad_halo_tcgen05<<<hl.plan[i].grid, 192, hl.plan[i].smem, st>>>(mdy, mx, p);
    rc = after_launch("conv_wgrad_halo_tcgen05");
    if (rc) return rc;
  }
  return wgrad_finish(who, variant, hl.plan[0].p.splits, dy, dw, dw_elems, dbias, d, workspace, st);
}

int wgrad_run(const char* who, const float* x, const float* dy, float* dw, float* dbias,
              const mb_conv_desc* d, int variant, void* workspace, size_t workspace_bytes,
              cudaStream_t st) {
  const CUtensorMapSwizzle kWg = CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B;   // MN-major TF32 operands
  {
    wgh::Launches hl;
    if (wgh::make_plans(d, variant, &hl))
      return wgrad_run_halo(who, hl, x, dy, dw, dbias, d, variant, workspace, workspace_bytes, st);
  }
  wg::Plan pl;
  if (!wg::make_plan(d, variant, &pl))
    return fail(MB_ERR_UNSUPPORTED, "%s: geometry not supported by the tensor-core kernel", who);
  WgradParams& p = pl.p;
  const size_t dw_elems = static_cast<size_t>(d->K) * d->R * d->S * d->C;
  int rc;
  CUtensorMap mdy, mx[4];
  const long long K4 = static_cast<long long>(d->K) * 4, C4 = static_cast<long long>(d->C) * 4;
  auto act = [&](CUtensorMap* m, const float* base, int Cn, long long Wv, long long Hv, long long Nv,
                 long long sw_b, long long sh_b, long long sn_b, int chunks) {
    if (p.chunked)
      return encode_act_chunked(who, m, base, Cn, Wv, Hv, Nv, sw_b, sh_b, sn_b, p.bw, p.bh, p.bn,
                                chunks, kWg);
    return encode_act(who, m, base, Cn, Wv, Hv, Nv, sw_b, sh_b, sn_b, p.bw, p.bh, p.bn, kWg);
  };
  if (pl.flat) {
    const long long pixels = static_cast<long long>(d->N) * d->P * d->Q;
    rc = act(&mdy, dy, d->K, pixels, 1, 1, K4, K4 * pixels, K4 * pixels, p.KA);
    if (rc) return rc;
    rc = act(&mx[0], x, d->C, pixels, 1, 1, C4, C4 * pixels, C4 * pixels, p.U);
    if (rc) return rc;
    mx[1] = mx[2] = mx[3] = mx[0];
  } else {
    rc = act(&mdy, dy, d->K, d->Q, d->P, d->N, K4, K4 * d->Q, K4 * d->Q * d->P, p.KA);
    if (rc) return rc;
    int first = -1;
    for (int mi = 0; mi < d->stride_h * d->stride_w; ++mi) {
      if (!pl.map_used[mi]) continue;
      const int a = mi / d->stride_w, b = mi % d->stride_w;
      const long long Wv = (d->W - b + d->stride_w - 1) / d->stride_w;
      const long long Hv = (d->H - a + d->stride_h - 1) / d->stride_h;
      rc = act(&mx[mi], x + (static_cast<long long>(a) * d->W + b) * d->C, d->C, Wv, Hv, d->N,
               C4 * d->stride_w, C4 * d->W * d->stride_h, C4 * d->W * d->H, p.U);
      if (rc) return rc;
      if (first < 0) first = mi;
    }
    for (int mi = 0; mi < 4; ++mi)
      if (mi >= d->stride_h * d->stride_w || !pl.map_used[mi]) mx[mi] = mx[first];
  }
  return wgrad_launch(who, pl, mdy, mx, dy, dw, dw_elems, dbias, d, variant, workspace, workspace_bytes, st);
}

// ------------------------------------------------------------- few-channel convolutions
// A convolution with C <= 4 input channels (the network input) would waste 7/8 of every
// 32-channel operand row.  Instead the input is copied once into a zero-padded NHWC buffer
// with 4 channels, xp[N][Hp][Wp][4]; the 8 pixels x 4 channels to the right of any pixel
// are then 32 contiguous floats, i.e. one whole operand row holding filter columns
// s = 0..7 of filter row r.  A tensor map whose pixel stride (stride_w * 16 bytes) is smaller
// than its 128-byte rows exposes exactly those overlapping windows, so the GEMM K dimension
// becomes (r) x (s, c) = R x 32 and the generic kernels run with R "taps" and one chunk.
bool smallc_ok(const mb_conv_desc* d) {
  return d && d->groups == 1 && d->C <= 4 && d->S <= 8 && d->dil_w == 1 && d->dil_h == 1 &&
         d->stride_h >= 1 && d->stride_h <= 2 && d->stride_w >= 1 && d->stride_w <= 2 &&
         d->K % 4 == 0 && d->R <= kMaxTaps;
}
int smallc_Hp(const mb_conv_desc* d) { return d->H + 2 * d->pad_h; }
int smallc_Wp(const mb_conv_desc* d) {
  int need = d->stride_w * (d->Q - 1) + 8;           // last window must stay inside the row
  const int full = d->W + 2 * d->pad_w;
  if (need < full) need = full;
  return (need + 3) / 4 * 4;
}

// Window view of phase `a` (rows a, a+stride_h, ...) of the padded input.
int encode_smallc(const char* who, CUtensorMap* m, const float* xp, const mb_conv_desc* d, int a,
                  int bw, int bh, int bn, CUtensorMapSwizzle sw) {
  const long long Hp = smallc_Hp(d), Wp = smallc_Wp(d);
  const long long Hv = (Hp - a + d->stride_h - 1) / d->stride_h;
  return encode_act(who, m, xp + static_cast<long long>(a) * Wp * 4, 32, d->Q, Hv, d->N,
                    16LL * d->stride_w, 16LL * Wp * d->stride_h, 16LL * Wp * Hp, bw, bh, bn, sw);
}

__global__ void __launch_bounds__(256) smallc_pack_input(const float* __restrict__ x,
                                                         float* __restrict__ xp, int C, int H, int W,
                                                         int ph, int pw, int Hp, int Wp,
                                                         size_t total) {
  // one thread per padded pixel: reads the C planes of the NCHW input, writes 4 floats
  for (size_t t = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; t < total;
       t += static_cast<size_t>(gridDim.x) * blockDim.x) {
    const int wq = static_cast<int>(t % Wp);
    size_t r = t / Wp;
    const int hq = static_cast<int>(r % Hp);
    const size_t n = r / Hp;
    const int h = hq - ph, w = wq - pw;
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
    if (h >= 0 && h < H && w >= 0 && w < W) {
      const float* src = x + (n * C * H + h) * static_cast<size_t>(W) + w;
      const size_t plane = static_cast<size_t>(H) * W;
      v.x = __ldg(src);
      if (C > 1) v.y = __ldg(src + plane);
      if (C > 2) v.z = __ldg(src + 2 * plane);
      if (C > 3) v.w = __ldg(src + 3 * plane);
    }
    reinterpret_cast<float4*>(xp)[t] = v;
  }
}

// one thread per (image, phase-row, padded column): both row phases of up to 4 channels
__global__ void __launch_bounds__(256) smallc2_pack_input(const float* __restrict__ x,
                                                          float* __restrict__ xp2, int C, int H, int W,
                                                          int ph, int pw, int Hp2, int Wp,
                                                          size_t total) {
  for (size_t t = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; t < total;
       t += static_cast<size_t>(gridDim.x) * blockDim.x) {
    const int wq = static_cast<int>(t % Wp);
    size_t r = t / Wp;
    const int hh = static_cast<int>(r % Hp2);
    const size_t n = r / Hp2;
    const int w = wq - pw;
    const size_t plane = static_cast<size_t>(H) * W;
    float4 v[2];
#pragma unroll
    for (int phase = 0; phase < 2; ++phase) {
      const int h = 2 * hh + phase - ph;
      v[phase] = make_float4(0.f, 0.f, 0.f, 0.f);
      if (h >= 0 && h < H && w >= 0 && w < W) {
        const float* src = x + (n * C * H + h) * static_cast<size_t>(W) + w;
        v[phase].x = __ldg(src);
        if (C > 1) v[phase].y = __ldg(src + plane);
        if (C > 2) v[phase].z = __ldg(src + 2 * plane);
        if (C > 3) v[phase].w = __ldg(src + 3 * plane);
      }
    }
    reinterpret_cast<float4*>(xp2)[2 * t] = v[0];
    reinterpret_cast<float4*>(xp2)[2 * t + 1] = v[1];
  }
}

}  // namespace mb

using namespace mb;

extern "C" {

int mb_conv_num_variants(int pass) {
  switch (pass) {
    case MB_CONV_FPROP: return 1;
    case MB_CONV_DGRAD: return 1;
    case MB_CONV_WGRAD: return 2;
    default: return 0;
  }
}

size_t mb_conv_workspace_bytes(int pass, int variant, const mb_conv_desc* d) {
  if (!d || variant < 0 || variant >= mb_conv_num_variants(pass)) return 0;
  if (pass == MB_CONV_DGRAD)   // the filter is read in place when its tiles are whole 32-channel groups
    return d->C % 32 == 0 ? 0 : static_cast<size_t>(d->K) * d->R * d->S * d->C * sizeof(float);
  if (pass == MB_CONV_WGRAD) return wgrad_workspace_bytes(d, variant);
  return 0;
}

int mb_conv_device_status(int reset) {
  int v = 0;
  if (cudaMemcpyFromSymbol(&v, g_conv_status, sizeof(int)) != cudaSuccess) return -1;
  if (reset && v != 0) {
    int z = 0;
    cudaMemcpyToSymbol(g_conv_status, &z, sizeof(int));
  }
  return v;
}

static int fprop_impl(const char* who, const float* x, const float* w, const float* bias, float* y,
                      const mb_conv_desc* d, int variant, void* workspace, size_t workspace_bytes,
                      void* stream, float* stats, const float* stats_shift, int* stats_rows) {
  int rc = validate(who, d);
  if (rc) return rc;
  if (variant < 0 || variant >= mb_conv_num_variants(MB_CONV_FPROP))
    return fail(MB_ERR_UNSUPPORTED, "%s: no variant %d", who, variant);
  if (!x || !w || !y) return fail(MB_ERR_INVALID_ARGUMENT, "%s: null pointer", who);
  if (!aligned(x, 16) || !aligned(w, 16) || !aligned(y, 16) || !aligned(bias, 16))
    return fail(MB_ERR_INVALID_ARGUMENT, "%s: pointers must be 16-byte aligned", who);
  (void)workspace; (void)workspace_bytes;

  if (d->stride_h == 1 && d->stride_w == 1 && d->R * d->S > 1) {
    // the halo kernels have no statistics warps: the caller falls back to the plain pair
    if (stats) return fail(MB_ERR_UNSUPPORTED, "%s: no output statistics for stride-1 multi-tap filters", who);
    HaloTap taps[kMaxTaps];
    int nt = 0;
    for (int r = 0; r < d->R; ++r)
      for (int s = 0; s < d->S; ++s)
        taps[nt++] = HaloTap{r * d->dil_h - d->pad_h, s * d->dil_w - d->pad_w, r * d->S + s};
    rc = run_halo(who, x, d->C, d->W, d->H, w, d->R * d->S, y, d->K, d->Q, d->P, d->N, taps, nt, bias,
                  as_stream(stream));
    if (rc != MB_ERR_UNSUPPORTED) return rc;
  }
  GemmLaunch L;
  std::memset(&L.p, 0, sizeof(L.p));
  GemmParams& p = L.p;
  p.out = y;
  p.bias = bias;
  p.Kout = d->K;
  p.kchunks = (d->C + kChunkK - 1) / kChunkK;
  const long long C4 = static_cast<long long>(d->C) * 4;
  TileShape ts;
  if (is_pointwise(d)) {
    const long long pixels = static_cast<long long>(d->N) * d->H * d->W;
    if (pixels > 0x7fffffffLL) return fail(MB_ERR_UNSUPPORTED, "%s: more than 2^31 pixels", who);
    ts = TileShape{kTileM, 1, 1};
    p.Nimg = 1; p.P = 1; p.Q = static_cast<int>(pixels);
    p.out_sn = 0; p.out_sh = 0; p.out_sw = d->K;
    rc = encode_act(who, &L.a[0], x, d->C, pixels, 1, 1, C4, C4 * pixels, C4 * pixels, ts.bw, 1, 1);
    if (rc) return rc;
    L.a[1] = L.a[2] = L.a[3] = L.a[0];
    p.num_taps = 1;
    p.taps.dh[0] = p.taps.dw[0] = 0;
    p.taps.map[0] = 0;
    p.taps.btap[0] = 0;
  } else {
    ts = pick_tile(d->N, d->P, d->Q);
    p.Nimg = d->N; p.P = d->P; p.Q = d->Q;
    p.out_sw = d->K;
    p.out_sh = static_cast<long long>(d->Q) * d->K;
    p.out_sn = p.out_sh * d->P;
    bool have[4] = {false, false, false, false};
    int nt = 0;
    for (int r = 0; r < d->R; ++r) {
      const int oh = r * d->dil_h - d->pad_h;
      const int a = posmod(oh, d->stride_h), dh = (oh - a) / d->stride_h;
      for (int s = 0; s < d->S; ++s) {
        const int ow = s * d->dil_w - d->pad_w;
        const int b = posmod(ow, d->stride_w), dw = (ow - b) / d->stride_w;
        if (a >= d->H || b >= d->W) continue;   // this phase of the input is empty
        const int mi = a * d->stride_w + b;
        have[mi] = true;
        p.taps.dh[nt] = static_cast<short>(dh);
        p.taps.dw[nt] = static_cast<short>(dw);
        p.taps.map[nt] = static_cast<unsigned char>(mi);
        p.taps.btap[nt] = static_cast<unsigned char>(r * d->S + s);
        ++nt;
      }
    }
    p.num_taps = nt;
    int first = -1;
    for (int mi = 0; mi < d->stride_h * d->stride_w; ++mi) {
      if (!have[mi]) continue;
      const int a = mi / d->stride_w, b = mi % d->stride_w;
      const long long Wv = (d->W - b + d->stride_w - 1) / d->stride_w;
      const long long Hv = (d->H - a + d->stride_h - 1) / d->stride_h;
      rc = encode_act(who, &L.a[mi], x + (static_cast<long long>(a) * d->W + b) * d->C, d->C, Wv, Hv,
                      d->N, C4 * d->stride_w, C4 * d->W * d->stride_h, C4 * d->W * d->H, ts.bw, ts.bh,
                      ts.bn);
      if (rc) return rc;
      if (first < 0) first = mi;
    }
    if (first < 0) return fail(MB_ERR_INVALID_ARGUMENT, "%s: no filter tap touches the input", who);
    for (int mi = 0; mi < 4; ++mi)
      if (mi >= d->stride_h * d->stride_w || !have[mi]) L.a[mi] = L.a[first];
  }
  p.bw = ts.bw; p.bh = ts.bh; p.bn = ts.bn;
  p.tiles_w = (p.Q + ts.bw - 1) / ts.bw;
  p.tiles_h = (p.P + ts.bh - 1) / ts.bh;
  const long long tiles_n = (p.Nimg + ts.bn - 1) / ts.bn;
  const long long m_tiles = static_cast<long long>(p.tiles_w) * p.tiles_h * tiles_n;
  pick_bn_stages(d->K, m_tiles, &p.BN, &p.stages, &L.smem,
                 stats ? kAStageBytes + (static_cast<size_t>(3) * d->K + 128) * sizeof(float) : 0);
  p.tiles_c = (d->K + p.BN - 1) / p.BN;
  const long long tiles = m_tiles * p.tiles_c;
  if (tiles > 0x7fffffffLL) return fail(MB_ERR_UNSUPPORTED, "%s: too many tiles", who);
  p.num_tiles = static_cast<int>(tiles);
  rc = encode_filter(who, &L.b, w, d->C, d->R * d->S, d->K, p.BN);
  if (rc) return rc;
  L.grid = p.num_tiles < num_sms() ? p.num_tiles : num_sms();
  p.stats = stats;
  p.stats_shift = stats_shift;
  if (stats_rows) *stats_rows = L.grid;
  return launch_gemm("conv_fprop_tcgen05", L, as_stream(stream));
}

int mb_conv2d_fprop(const float* x, const float* w, const float* bias, float* y,
                    const mb_conv_desc* d, int variant, void* workspace, size_t workspace_bytes,
                    void* stream) {
  return fprop_impl("mb_conv2d_fprop", x, w, bias, y, d, variant, workspace, workspace_bytes, stream,
                    nullptr, nullptr, nullptr);
}

size_t mb_conv_bnstats_bytes(const mb_conv_desc* d) {
  if (!d || d->K <= 0) return 0;
  return static_cast<size_t>(2) * num_sms() * d->K * sizeof(float);
}

int mb_conv2d_fprop_bnstats(const float* x, const float* w, const float* bias, float* y,
                            const mb_conv_desc* d, int variant, void* workspace,
                            size_t workspace_bytes, const float* shift, float* partials,
                            size_t partials_bytes, int* partial_rows, void* stream) {
  const char* who = "mb_conv2d_fprop_bnstats";
  if (!partials || !partial_rows) return fail(MB_ERR_INVALID_ARGUMENT, "%s: null pointer", who);
  if (partials_bytes < mb_conv_bnstats_bytes(d))
    return fail(MB_ERR_WORKSPACE, "%s: %zu bytes needed for the partial sums, %zu given", who,
                mb_conv_bnstats_bytes(d), partials_bytes);
  if (d && d->K % 32)
    return fail(MB_ERR_UNSUPPORTED, "%s: output channels must be a multiple of 32", who);
  *partial_rows = 0;
  return fprop_impl(who, x, w, bias, y, d, variant, workspace, workspace_bytes, stream, partials, shift,
                    partial_rows);
}

int mb_conv2d_dgrad(const float* dy, const float* w, float* dx, const mb_conv_desc* d, int variant,
                    void* workspace, size_t workspace_bytes, void* stream) {
  const char* who = "mb_conv2d_dgrad";
  int rc = validate(who, d);
  if (rc) return rc;
  if (variant < 0 || variant >= mb_conv_num_variants(MB_CONV_DGRAD))
    return fail(MB_ERR_UNSUPPORTED, "%s: no variant %d", who, variant);
  if (!dy || !w || !dx) return fail(MB_ERR_INVALID_ARGUMENT, "%s: null pointer", who);
  if (!aligned(dy, 16) || !aligned(w, 16) || !aligned(dx, 16))
    return fail(MB_ERR_INVALID_ARGUMENT, "%s: pointers must be 16-byte aligned", who);
  const size_t need = mb_conv_workspace_bytes(MB_CONV_DGRAD, variant, d);
  if (need && (!workspace || workspace_bytes < need || !aligned(workspace, 16)))
    return fail(MB_ERR_WORKSPACE, "%s: workspace of %zu bytes needed, %zu given", who, need,
                workspace ? workspace_bytes : size_t(0));
  cudaStream_t st = as_stream(stream);
  const int T = d->R * d->S;
  // The GEMM reduces over K.  With whole 32-channel groups of C the filter tile is taken MN-major
  // straight from w = [K][R*S][C]; otherwise w is first transposed to [C][R*S][K] in the workspace.
  const bool filter_mn = need == 0;
  const float* wt = w;
  if (!filter_mn) {
    float* t = static_cast<float*>(workspace);
    const size_t total = static_cast<size_t>(d->K) * T * d->C;
    transpose_filter<<<grid_for(total, 256, 8), 256, 0, st>>>(w, t, d->K, T, d->C);
    rc = after_launch("conv_transpose_filter");
    if (rc) return rc;
    wt = t;
  }
  if (d->stride_h == 1 && d->stride_w == 1 && T > 1) {
    HaloTap taps[kMaxTaps];
    int nt = 0;
    for (int r = 0; r < d->R; ++r)
      for (int s = 0; s < d->S; ++s)
        taps[nt++] = HaloTap{d->pad_h - r * d->dil_h, d->pad_w - s * d->dil_w, r * d->S + s};
    rc = run_halo(who, dy, d->K, d->Q, d->P, wt, T, dx, d->C, d->W, d->H, d->N, taps, nt, nullptr, st,
                  filter_mn);
    if (rc != MB_ERR_UNSUPPORTED) return rc;
  }
  const long long K4 = static_cast<long long>(d->K) * 4;
  const int sh = d->stride_h, sw = d->stride_w;
  // a phase of dx that no filter tap reaches is zero: clear dx first if there is one
  bool any_empty = false;
  for (int a = 0; a < sh && a < d->H; ++a)
    for (int b = 0; b < sw && b < d->W; ++b) {
      int cnt = 0;
      for (int r = 0; r < d->R; ++r)
        for (int s = 0; s < d->S; ++s)
          if (!posmod(a + d->pad_h - r * d->dil_h, sh) && !posmod(b + d->pad_w - s * d->dil_w, sw)) ++cnt;
      if (!cnt) any_empty = true;
    }
  if (any_empty &&
      cudaMemsetAsync(dx, 0, static_cast<size_t>(d->N) * d->H * d->W * d->C * sizeof(float), st) != cudaSuccess)
    return fail(MB_ERR_LAUNCH, "%s: memset failed", who);
  for (int a = 0; a < sh; ++a) {
    for (int b = 0; b < sw; ++b) {
      if (a >= d->H || b >= d->W) continue;
      GemmLaunch L;
      std::memset(&L.p, 0, sizeof(L.p));
      GemmParams& p = L.p;
      int nt = 0;
      // dx[h = i*sh + a] takes dy[(h + pad - r*dil) / sh] for the taps where that is exact
      for (int r = 0; r < d->R; ++r) {
        const int oh = a + d->pad_h - r * d->dil_h;
        if (posmod(oh, sh)) continue;
        for (int s = 0; s < d->S; ++s) {
          const int ow = b + d->pad_w - s * d->dil_w;
          if (posmod(ow, sw)) continue;
          p.taps.dh[nt] = static_cast<short>(floordiv(oh, sh));
          p.taps.dw[nt] = static_cast<short>(floordiv(ow, sw));
          p.taps.map[nt] = 0;
          p.taps.btap[nt] = static_cast<unsigned char>(r * d->S + s);
          ++nt;
        }
      }
      const int Hv = (d->H - a + sh - 1) / sh, Wv = (d->W - b + sw - 1) / sw;
      if (nt == 0) continue;
      p.num_taps = nt;
      p.out = dx + (static_cast<long long>(a) * d->W + b) * d->C;
      p.bias = nullptr;
      p.Kout = d->C;
      p.kchunks = (d->K + kChunkK - 1) / kChunkK;
      TileShape ts;
      const bool flat = is_pointwise(d);
      if (flat) {
        const long long pixels = static_cast<long long>(d->N) * d->H * d->W;
        if (pixels > 0x7fffffffLL) return fail(MB_ERR_UNSUPPORTED, "%s: more than 2^31 pixels", who);
        ts = TileShape{kTileM, 1, 1};
        p.Nimg = 1; p.P = 1; p.Q = static_cast<int>(pixels);
        p.out_sw = d->C;
        rc = encode_act(who, &L.a[0], dy, d->K, pixels, 1, 1, K4, K4 * pixels, K4 * pixels, ts.bw, 1, 1);
      } else {
        ts = pick_tile(d->N, Hv, Wv);
        p.Nimg = d->N; p.P = Hv; p.Q = Wv;
        p.out_sw = static_cast<long long>(sw) * d->C;
        p.out_sh = static_cast<long long>(sh) * d->W * d->C;
        p.out_sn = static_cast<long long>(d->H) * d->W * d->C;
        rc = encode_act(who, &L.a[0], dy, d->K, d->Q, d->P, d->N, K4, K4 * d->Q, K4 * d->Q * d->P,
                        ts.bw, ts.bh, ts.bn);
      }
      if (rc) return rc;
      L.a[1] = L.a[2] = L.a[3] = L.a[0];
      p.bw = ts.bw; p.bh = ts.bh; p.bn = ts.bn;
      p.tiles_w = (p.Q + ts.bw - 1) / ts.bw;
      p.tiles_h = (p.P + ts.bh - 1) / ts.bh;
      const long long tiles_n = (p.Nimg + ts.bn - 1) / ts.bn;
      const long long m_tiles = static_cast<long long>(p.tiles_w) * p.tiles_h * tiles_n;
      pick_bn_stages(d->C, m_tiles, &p.BN, &p.stages, &L.smem);
      p.tiles_c = (d->C + p.BN - 1) / p.BN;
      const long long tiles = m_tiles * p.tiles_c;
      if (tiles > 0x7fffffffLL) return fail(MB_ERR_UNSUPPORTED, "%s: too many tiles", who);
      p.num_tiles = static_cast<int>(tiles);
      p.b_mn = filter_mn ? 1 : 0;
      rc = filter_mn ? encode_filter_mn(who, &L.b, wt, d->K, T, d->C, p.BN)
                     : encode_filter(who, &L.b, wt, d->K, T, d->C, p.BN);
      if (rc) return rc;
      L.grid = p.num_tiles < num_sms() ? p.num_tiles : num_sms();
      rc = launch_gemm("conv_dgrad_tcgen05", L, st);
      if (rc) return rc;
    }
  }
  return MB_OK;
}

int mb_conv2d_wgrad(const float* x, const float* dy, float* dw, float* dbias,
                    const mb_conv_desc* d, int variant, void* workspace, size_t workspace_bytes,
                    void* stream) {
  const char* who = "mb_conv2d_wgrad";
  int rc = validate(who, d);
  if (rc) return rc;
  if (variant < 0 || variant >= mb_conv_num_variants(MB_CONV_WGRAD))
    return fail(MB_ERR_UNSUPPORTED, "%s: no variant %d", who, variant);
  if (!x || !dy || !dw) return fail(MB_ERR_INVALID_ARGUMENT, "%s: null pointer", who);
  if (!aligned(x, 16) || !aligned(dy, 16) || !aligned(dw, 16))
    return fail(MB_ERR_INVALID_ARGUMENT, "%s: pointers must be 16-byte aligned", who);
  return wgrad_run(who, x, dy, dw, dbias, d, variant, workspace, workspace_bytes, as_stream(stream));
}


int mb_conv_smallc_geometry(const mb_conv_desc* d, int* Hp, int* Wp) {
  if (!smallc_ok(d)) return MB_ERR_UNSUPPORTED;
  if (Hp) *Hp = smallc_Hp(d);
  if (Wp) *Wp = smallc_Wp(d);
  return MB_OK;
}

int mb_conv_smallc_pack_input(const float* x_nchw, float* xp, const mb_conv_desc* d, void* stream) {
  const char* who = "mb_conv_smallc_pack_input";
  if (!smallc_ok(d)) return fail(MB_ERR_UNSUPPORTED, "%s: not a few-channel geometry", who);
  if (!x_nchw || !xp || !aligned(xp, 16)) return fail(MB_ERR_INVALID_ARGUMENT, "%s: bad pointer", who);
  const int Hp = smallc_Hp(d), Wp = smallc_Wp(d);
  const size_t total = static_cast<size_t>(d->N) * Hp * Wp;
  smallc_pack_input<<<grid_for(total, 256, 8), 256, 0, as_stream(stream)>>>(
      x_nchw, xp, d->C, d->H, d->W, d->pad_h, d->pad_w, Hp, Wp, total);
  return after_launch("conv_smallc_pack_input");
}

int mb_conv2d_fprop_smallc(const float* xp, const float* wp, const float* bias, float* y,
                           const mb_conv_desc* d, void* stream) {
  const char* who = "mb_conv2d_fprop_smallc";
  if (!smallc_ok(d)) return fail(MB_ERR_UNSUPPORTED, "%s: not a few-channel geometry", who);
  if (!xp || !wp || !y) return fail(MB_ERR_INVALID_ARGUMENT, "%s: null pointer", who);
  if (!aligned(xp, 16) || !aligned(wp, 16) || !aligned(y, 16) || !aligned(bias, 16))
    return fail(MB_ERR_INVALID_ARGUMENT, "%s: pointers must be 16-byte aligned", who);
  if (d->stride_h == 1 && d->stride_w == 1 && d->R >= 2) {
    // stride 1 (the first layer of VGG-16 and of the UNet): the taps are the R filter rows of
    // one window column, so the many-tap kernel fetches each window row once per tile with its
    // R - 1 halo rows instead of once per tap (VGG's 3 -> 64 layer on 224x224: 1.0 -> 0.6 ms, packing included)
    HaloTap taps[kMaxTaps];
    for (int t = 0; t < d->R; ++t) taps[t] = HaloTap{t, 0, t};
    const long long Hp = smallc_Hp(d), Wp = smallc_Wp(d);
    const long long strides[3] = {16LL, 16LL * Wp, 16LL * Wp * Hp};
    const int rc = run_halo(who, xp, 32, d->Q, static_cast<int>(Hp), wp, d->R, y, d->K, d->Q, d->P, d->N, taps,
                            d->R, bias, as_stream(stream), false, strides);
    if (rc != MB_ERR_UNSUPPORTED) return rc;
  }
  GemmLaunch L;
  std::memset(&L.p, 0, sizeof(L.p));
  GemmParams& p = L.p;
  p.out = y; p.bias = bias; p.Kout = d->K; p.kchunks = 1;
  const TileShape ts = pick_tile(d->N, d->P, d->Q);
  p.Nimg = d->N; p.P = d->P; p.Q = d->Q;
  p.out_sw = d->K;
  p.out_sh = static_cast<long long>(d->Q) * d->K;
  p.out_sn = p.out_sh * d->P;
  for (int r = 0; r < d->R; ++r) {
    p.taps.dh[r] = static_cast<short>(r / d->stride_h);
    p.taps.dw[r] = 0;
    p.taps.map[r] = static_cast<unsigned char>(r % d->stride_h);
    p.taps.btap[r] = static_cast<unsigned char>(r);
  }
  p.num_taps = d->R;
  int rc;
  for (int a = 0; a < 4; ++a) {
    const int src = a < d->stride_h && a < d->R ? a : 0;
    rc = encode_smallc(who, &L.a[a], xp, d, src, ts.bw, ts.bh, ts.bn, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc) return rc;
  }
  p.bw = ts.bw; p.bh = ts.bh; p.bn = ts.bn;
  p.tiles_w = (p.Q + ts.bw - 1) / ts.bw;
  p.tiles_h = (p.P + ts.bh - 1) / ts.bh;
  const long long m_tiles = static_cast<long long>(p.tiles_w) * p.tiles_h * ((p.Nimg + ts.bn - 1) / ts.bn);
  pick_bn_stages(d->K, m_tiles, &p.BN, &p.stages, &L.smem);
  p.tiles_c = (d->K + p.BN - 1) / p.BN;
  const long long tiles = m_tiles * p.tiles_c;
  if (tiles > 0x7fffffffLL) return fail(MB_ERR_UNSUPPORTED, "%s: too many tiles", who);
  p.num_tiles = static_cast<int>(tiles);
  rc = encode_filter(who, &L.b, wp, 32, d->R, d->K, p.BN);
  if (rc) return rc;
  L.grid = p.num_tiles < num_sms() ? p.num_tiles : num_sms();
  return launch_gemm("conv_fprop_smallc_tcgen05", L, as_stream(stream));
}

// ---- few-channel input, stride 2: both row phases in one buffer, forward on the halo kernel.
// xp2[N][Hp2][Wp][2][4]: padded pixel (2*hh + phase, w) of image n, channel c, at float
// ((n*Hp2 + hh)*Wp + w)*8 + phase*4 + c.  The 64 floats that start at pixel (hh, 2q) are the
// window of output column q for filter rows 2*dh and 2*dh + 1 (dh = hh - p): 8 input columns x
// 2 phases x 4 channels, i.e. two 32-float operand chunks.  The GEMM therefore has
// ceil(R/2) "taps" that differ only in their row and 2 chunks each, which is the halo
// kernel's interface: the window rows a tile needs are fetched once (bh + ceil(R/2) - 1 rows
// for bh output rows) instead of once per filter row, and the filter tiles are 8 per tile
// instead of one per filter row and tile.
int mb_conv_smallc2_geometry(const mb_conv_desc* d, int* Hp2, int* Wp) {
  if (!smallc_ok(d) || d->stride_h != 2 || d->stride_w != 2 || d->R > 8 || d->R < 3)
    return MB_ERR_UNSUPPORTED;
  const int taps = (d->R + 1) / 2;
  int hp = (d->H + 2 * d->pad_h + 1) / 2;
  if (hp < d->P + taps - 1) hp = d->P + taps - 1;
  int wp = 2 * (d->Q - 1) + 8;
  if (wp < d->W + 2 * d->pad_w) wp = d->W + 2 * d->pad_w;
  if (Hp2) *Hp2 = hp;
  if (Wp) *Wp = (wp + 1) / 2 * 2;
  return MB_OK;
}

int mb_conv_smallc2_pack_input(const float* x_nchw, float* xp2, const mb_conv_desc* d, void* stream) {
  const char* who = "mb_conv_smallc2_pack_input";
  int Hp2, Wp;
  if (mb_conv_smallc2_geometry(d, &Hp2, &Wp)) return fail(MB_ERR_UNSUPPORTED, "%s: not a stride-2 few-channel geometry", who);
  if (!x_nchw || !xp2 || !aligned(xp2, 32)) return fail(MB_ERR_INVALID_ARGUMENT, "%s: bad pointer", who);
  const size_t total = static_cast<size_t>(d->N) * Hp2 * Wp;
  smallc2_pack_input<<<grid_for(total, 256, 8), 256, 0, as_stream(stream)>>>(
      x_nchw, xp2, d->C, d->H, d->W, d->pad_h, d->pad_w, Hp2, Wp, total);
  return after_launch("conv_smallc2_pack_input");
}

int mb_conv2d_fprop_smallc2(const float* xp2, const float* wp2, const float* bias, float* y,
                            const mb_conv_desc* d, void* stream) {
  const char* who = "mb_conv2d_fprop_smallc2";
  int Hp2, Wp;
  if (mb_conv_smallc2_geometry(d, &Hp2, &Wp)) return fail(MB_ERR_UNSUPPORTED, "%s: not a stride-2 few-channel geometry", who);
  if (!xp2 || !wp2 || !y) return fail(MB_ERR_INVALID_ARGUMENT, "%s: null pointer", who);
  if (!aligned(xp2, 16) || !aligned(wp2, 16) || !aligned(y, 16) || !aligned(bias, 16))
    return fail(MB_ERR_INVALID_ARGUMENT, "%s: pointers must be 16-byte aligned", who);
  const int T = (d->R + 1) / 2;
  HaloTap taps[4];
  for (int t = 0; t < T; ++t) taps[t] = HaloTap{t, 0, t};
  const long long strides[3] = {64LL, 32LL * Wp, 32LL * Wp * Hp2};
  int rc = run_halo(who, xp2, 64, d->Q, Hp2, wp2, T, y, d->K, d->Q, d->P, d->N, taps, T, bias, as_stream(stream),
                    false, strides);
  if (rc == MB_ERR_UNSUPPORTED) return fail(MB_ERR_UNSUPPORTED, "%s: geometry does not fit the halo kernel", who);
  return rc;
}

size_t mb_conv_smallc_wgrad_workspace_bytes(const mb_conv_desc* d, int variant) {
  if (!smallc_ok(d) || variant != 1) return 0;
  wg::Plan pl;
  if (!wg::make_plan(d, variant, &pl, true)) return 0;
  return static_cast<size_t>(pl.p.splits) * d->K * d->R * 32 * sizeof(float);
}

int mb_conv2d_wgrad_smallc(const float* xp, const float* dy, float* dwp, float* dbias,
                           const mb_conv_desc* d, int variant, void* workspace,
                           size_t workspace_bytes, void* stream) {
  const char* who = "mb_conv2d_wgrad_smallc";
  if (!smallc_ok(d)) return fail(MB_ERR_UNSUPPORTED, "%s: not a few-channel geometry", who);
  if (variant < 0 || variant > 1) return fail(MB_ERR_UNSUPPORTED, "%s: no variant %d", who, variant);
  if (!xp || !dy || !dwp) return fail(MB_ERR_INVALID_ARGUMENT, "%s: null pointer", who);
  if (!aligned(xp, 16) || !aligned(dy, 16) || !aligned(dwp, 16))
    return fail(MB_ERR_INVALID_ARGUMENT, "%s: pointers must be 16-byte aligned", who);
  const CUtensorMapSwizzle kWg = CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B;
  wg::Plan pl;
  if (!wg::make_plan(d, variant, &pl, true))
    return fail(MB_ERR_UNSUPPORTED, "%s: geometry not supported by the tensor-core kernel", who);
  WgradParams& p = pl.p;
  CUtensorMap mdy, mx[4];
  const long long K4 = static_cast<long long>(d->K) * 4;
  int rc = encode_act(who, &mdy, dy, d->K, d->Q, d->P, d->N, K4, K4 * d->Q, K4 * d->Q * d->P, p.bw,
                      p.bh, p.bn, kWg);
  if (rc) return rc;
  for (int a = 0; a < 4; ++a) {
    const int src = a < d->stride_h && a < d->R ? a : 0;
    rc = encode_smallc(who, &mx[a], xp, d, src, p.bw, p.bh, p.bn, kWg);
    if (rc) return rc;
  }
  const size_t dw_elems = static_cast<size_t>(d->K) * d->R * 32;
  return wgrad_launch(who, pl, mdy, mx, dy, dwp, dw_elems, dbias, d, variant, workspace,
                      workspace_bytes, as_stream(stream));
}


int mb_conv_debug_counters(long long* device_buffer) {
  g_conv_prof = device_buffer;
  return MB_OK;
}

}  // extern "C"
