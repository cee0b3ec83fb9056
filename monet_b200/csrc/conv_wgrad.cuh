// Backward-weight convolution on tcgen05: dw[k][tap][c] = sum over output
// pixels of dy[pixel][k] * x[pixel shifted by the tap][c].
//
// The reduction runs over PIXELS, so both operands are "MN-major" for the MMA:
// a TMA box {32 channels, pixels...} lands in shared memory as rows of one
// pixel x 32 channels (128 bytes).  For 32-bit MN-major operands the MMA only
// accepts the 128-byte swizzle with a 32-byte base, so the wgrad tensor maps
// use SWIZZLE_128B_ATOM_32B; four pixel rows form a 512-byte atom and one
// K = 8 step consumes two of them.  Boxes of 32 channels sit back to back in
// the slot, which is exactly the descriptor's leading-dimension stride, so ONE
// MMA spans up to four dy boxes (M = 128) and up to eight x boxes (N = 256).
//
//   A    = dy tile : KA boxes of 32 output channels (KA = 4 or 8 -> one or
//                    two M = 128 halves)
//   B_u            : one box of 32 input channels of x, shifted by the filter
//                    tap of "unit" u = (tap, 32-channel chunk); eight units
//                    form one N = 256 half
//   D[mh][nh]      : 128 x 256 fp32 accumulators in tensor memory, at most two
//                    (KA = 8 with up to 8 units, or KA = 4 with up to 16)
//
// One CTA owns a work item (KA boxes of output channels, a group of U units, a
// range of pixel tiles), so the CTA tile is 256 x 256 or 128 x 512 and each
// operand byte fetched from L2 feeds 64 / 51 flop.  The pixel range is a split
// of the reduction; partial results are combined either with red.global.add
// (variant 0, dw zeroed first) or through a workspace of per-split partials
// and a deterministic reduction kernel (variant 1).
//
// Pixel boxes always hold a multiple of 8 rows, and rows outside the image are
// zero-filled by TMA in dy, so padding rows contribute nothing.
#pragma once
#include "conv_gemm.cuh"

namespace mb {

struct WgradParams {
  float* out;               // dw, or the partial-sum workspace
  long long split_stride;   // elements between the partials of two splits (0: atomics into dw)
  int K, C, T;              // output channels, input channels, filter taps R*S
  int ntaps;                // taps that touch the input at all
  int cchunks;              // ceil(C / 32)
  int units, U, groups;     // units in total, per CTA, groups of units
  int KA, k_tiles;          // dy boxes (of 32 channels) per CTA: 4 or 8
  int splits;
  int bw, bh, bn, rows;     // pixel box, rows = bw*bh*bn (multiple of 8)
  int tiles_w, tiles_h;
  int pix_tiles;            // total pixel tiles
  int stages;
  int use_atomics;
  int chunked;              // 1: the maps are 5-d {32, w, h, n, chunk}: one copy brings all the
                            //    32-channel boxes of an operand; units are ordered tap-major
  long long* prof;          // optional: cycle counters written by CTA 0 (diagnostics), or null
  Taps taps;
};

__global__ void __launch_bounds__(192, 1)
conv_wgrad_tcgen05(const __grid_constant__ CUtensorMap mapDy, const __grid_constant__ CUtensorMap mapX0,
                   const __grid_constant__ CUtensorMap mapX1, const __grid_constant__ CUtensorMap mapX2,
                   const __grid_constant__ CUtensorMap mapX3, const __grid_constant__ WgradParams p) {
  using namespace sm100;
  extern __shared__ uint8_t smem_raw[];
  uint64_t* full = reinterpret_cast<uint64_t*>(smem_raw);
  uint64_t* empty = full + 16;
  uint64_t* acc_full = empty + 16;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_full + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  const uint32_t slots0 = (smem_u32(smem_raw) + 512u + 1023u) & ~1023u;
  uint8_t* slots_ptr = smem_raw + (slots0 - smem_u32(smem_raw));

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  // work item
  int wi = blockIdx.x;
  const int split = wi % p.splits;
  wi /= p.splits;
  const int group = wi % p.groups;
  const int kt = wi / p.groups;
  const int k0 = kt * p.KA * 32;
  const int u0 = group * p.U;
  const int nu = (p.units - u0) < p.U ? (p.units - u0) : p.U;
  int ka = (p.K - k0 + 31) / 32;          // dy boxes that exist for this CTA
  if (ka > p.KA) ka = p.KA;
  const int mh_n = (ka + 3) / 4;          // M = 128 halves in use
  const int nh_n = (nu + 7) / 8;          // N = 256 halves in use
  const int NH = (p.U + 7) / 8;           // accumulator grid is [KA/4][NH]
  const int per = (p.pix_tiles + p.splits - 1) / p.splits;
  const int t_begin = split * per;
  const int t_end = (t_begin + per) < p.pix_tiles ? (t_begin + per) : p.pix_tiles;
  const int n_iter = t_end > t_begin ? t_end - t_begin : 0;

  const uint32_t box_bytes = static_cast<uint32_t>(p.rows) * 128u;
  const uint32_t a_bytes = static_cast<uint32_t>(p.KA) * box_bytes;     // fixed slot layout
  const uint32_t stage_bytes = a_bytes + static_cast<uint32_t>(p.U) * box_bytes;
  // a 5-d copy always delivers its whole box (chunks past the tensor arrive as zeros)
  const uint32_t tx_bytes = static_cast<uint32_t>(p.chunked ? p.KA + p.U : ka + nu) * box_bytes;
  const uint32_t tmem_cols = 256u * (p.KA / 4) * NH;                     // 256 or 512

  if (threadIdx.x == 0) {
    for (int s = 0; s < p.stages; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    mbar_init(&acc_full[0], 1);
    *abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 5) {
    tmem_alloc(tmem_slot, tmem_cols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const bool prof = p.prof != nullptr && blockIdx.x == 0;

  if (warp == 4) {
    // ------------------------------------------------------------ TMA producer
    // One lane per box: lane j < ka loads dy box j, lane ka + u loads x box u, so the ka + nu
    // (up to 20) copies of a stage are issued by one warp instruction instead of one after
    // the other by a single thread.  Lane 0 owns the barriers.
    if (n_iter > 0) {
      if (lane == 0) {
        prefetch_tensormap(&mapDy);
        prefetch_tensormap(&mapX0);
      }
      bool is_a = lane < ka;
      bool is_b = lane >= ka && lane < ka + nu;
      const CUtensorMap* my_map = &mapDy;
      int my_c = k0 + 32 * lane, my_dw = 0, my_dh = 0;
      uint32_t my_off = static_cast<uint32_t>(lane) * box_bytes;
      if (p.chunked) {
        // lane 0: every dy box of the stage; lane 1: every x box (one tap, U consecutive chunks)
        is_a = lane == 0;
        is_b = lane == 1;
        my_c = k0 / 32;
        my_off = 0;
        if (is_b) {
          const int ti = u0 / p.cchunks;
          const int mi = p.taps.map[ti];
          my_map = mi == 0 ? &mapX0 : mi == 1 ? &mapX1 : mi == 2 ? &mapX2 : &mapX3;
          my_c = u0 - ti * p.cchunks;
          my_dw = p.taps.dw[ti];
          my_dh = p.taps.dh[ti];
          my_off = a_bytes;
        }
      } else if (is_b) {
        const int u = lane - ka;
        const int unit = u0 + u;
        const int cc = unit / p.ntaps, ti = unit - cc * p.ntaps;
        const int mi = p.taps.map[ti];
        my_map = mi == 0 ? &mapX0 : mi == 1 ? &mapX1 : mi == 2 ? &mapX2 : &mapX3;
        my_c = cc * 32;
        my_dw = p.taps.dw[ti];
        my_dh = p.taps.dh[ti];
        my_off = a_bytes + static_cast<uint32_t>(u) * box_bytes;
      }
      detail::Ring ring{0, 0u, p.stages};
      uint32_t armed[16];
      for (int s = 0; s < 16; ++s) armed[s] = 0;
      bool ok = true;
      long long w_empty = 0, w_issue = 0;
      int wt = t_begin % p.tiles_w;
      int rr = t_begin / p.tiles_w;
      int ht = rr % p.tiles_h;
      int nt = rr / p.tiles_h;
      for (int t = t_begin; t < t_end; ++t) {
        const int q0 = wt * p.bw, p0 = ht * p.bh, n0 = nt * p.bn;
        const long long tw0 = prof ? clock64() : 0;
        if (lane == 0) {
          ok = mbar_wait(&empty[ring.stage], ring.phase ^ 1u, abort_flag);
          if (ok) {
            mbar_arrive_expect_tx(&full[ring.stage], tx_bytes);
            armed[ring.stage] = 1u + ring.phase;
          }
        }
        ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
        if (!ok) break;
        const long long tw1 = prof ? clock64() : 0;
        w_empty += tw1 - tw0;
        if (is_a || is_b) {
          uint8_t* slot = slots_ptr + static_cast<size_t>(ring.stage) * stage_bytes;
          if (p.chunked)
            tma_load_5d(my_map, slot + my_off, &full[ring.stage], 0, q0 + my_dw, p0 + my_dh, n0, my_c);
          else
            tma_load_4d(my_map, slot + my_off, &full[ring.stage], my_c, q0 + my_dw, p0 + my_dh, n0);
        }
        ring.advance();
        if (++wt == p.tiles_w) {
          wt = 0;
          if (++ht == p.tiles_h) { ht = 0; ++nt; }
        }
        if (prof) w_issue += clock64() - tw1;
      }
      if (prof && lane == 0) { p.prof[1] = w_empty; p.prof[2] = w_issue; }
      if (!ok && lane == 0) {
        *abort_flag = 1;
        atomicCAS(&g_conv_status, 0, 11);
        for (int s = 0; s < p.stages; ++s) {
          if (!armed[s]) continue;
          const long long t0 = clock64();
          while (!mbar_try_wait(&full[s], armed[s] - 1u) && clock64() - t0 < 20000000LL) {
          }
        }
      }
    }
  } else if (warp == 5) {
    if (lane == 0 && n_iter > 0) {
      detail::Ring ring{0, 0u, p.stages};
      bool ok = true;
      const int ksteps = p.rows / 8;
      long long w_full = 0, w_mma = 0;
      const long long tk0 = prof ? clock64() : 0;
      for (int it = 0; it < n_iter; ++it) {
        const long long tf0 = prof ? clock64() : 0;
        if (!mbar_wait(&full[ring.stage], ring.phase, abort_flag)) {
          ok = false;
          break;
        }
        const long long tf1 = prof ? clock64() : 0;
        w_full += tf1 - tf0;
        tc_fence_after();
        const uint32_t a_addr = slots0 + static_cast<uint32_t>(ring.stage) * stage_bytes;
        for (int mh = 0; mh < mh_n; ++mh) {
          // 32-channel boxes are box_bytes apart (LBO), 4-pixel atoms 512 bytes apart (SBO)
          const uint64_t da = smem_desc(a_addr + mh * 4u * box_bytes, box_bytes, 512, kSwizzle128BBase32B);
          for (int nh = 0; nh < nh_n; ++nh) {
            const int n_units = (nu - 8 * nh) < 8 ? (nu - 8 * nh) : 8;
            const uint32_t idesc = idesc_tf32(kTileM, 32 * n_units, 1, 1);
            const uint64_t db = smem_desc(a_addr + a_bytes + nh * 8u * box_bytes, box_bytes, 512,
                                          kSwizzle128BBase32B);
            const uint32_t d_tmem = tmem_base + 256u * (mh * NH + nh);
            for (int k = 0; k < ksteps; ++k)   // 8 pixels = 1024 bytes (two atoms) per step
              mma_tf32(d_tmem, da + 64u * k, db + 64u * k, idesc, (it | k) != 0 ? 1u : 0u);
          }
        }
        mma_commit(&empty[ring.stage]);
        ring.advance();
        if (prof) w_mma += clock64() - tf1;
      }
      if (prof) { p.prof[0] = clock64() - tk0; p.prof[3] = w_full; p.prof[4] = w_mma; p.prof[5] = n_iter; }
      if (ok) {
        mma_commit(&acc_full[0]);
      } else {
        *abort_flag = 1;
        atomicCAS(&g_conv_status, 0, 12);
      }
    }
  } else if (n_iter > 0 || !p.use_atomics) {
    // epilogue: thread = output channel row, 32 input channels per unit
    const long long te0 = prof ? clock64() : 0;
    bool got = n_iter > 0 ? mbar_wait(&acc_full[0], 0, abort_flag) : true;
    got = __all_sync(0xffffffffu, got);
    const long long te1 = prof ? clock64() : 0;
    if (got) {
      tc_fence_after();
      float* base = p.out + static_cast<long long>(split) * p.split_stride;
      for (int mh = 0; mh < mh_n; ++mh) {
        const int k = k0 + mh * 128 + warp * 32 + lane;
        for (int u = 0; u < nu; ++u) {
          const int unit = u0 + u;
          int cc, ti;
          if (p.chunked) {
            ti = unit / p.cchunks;
            cc = unit - ti * p.cchunks;
          } else {
            cc = unit / p.ntaps;
            ti = unit - cc * p.ntaps;
          }
          float v[32];
          if (n_iter > 0) {
            tmem_ld32(tmem_base + (static_cast<uint32_t>(warp * 32) << 16) +
                          256u * (mh * NH + (u >> 3)) + 32u * (u & 7), v);
            tmem_ld_wait();
          } else {
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] = 0.f;
          }
          if (k < p.K) {
            float* dst = base + (static_cast<long long>(k) * p.T + p.taps.btap[ti]) * p.C + cc * 32;
            const int left = p.C - cc * 32;
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              if (4 * j < left) {
                if (p.use_atomics) {
                  asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(dst + 4 * j),
                               "f"(v[4 * j]), "f"(v[4 * j + 1]), "f"(v[4 * j + 2]), "f"(v[4 * j + 3])
                               : "memory");
                } else {
                  *reinterpret_cast<float4*>(dst + 4 * j) =
                      make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
                }
              }
            }
          }
        }
      }
    } else if (lane == 0) {
      *abort_flag = 1;
      atomicCAS(&g_conv_status, 0, 13);
    }
    if (prof && threadIdx.x == 0) { p.prof[6] = te1 - te0; p.prof[7] = clock64() - te1; }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 5) tmem_dealloc(tmem_base, tmem_cols);
}

// out[i] = sum over splits of part[s][i]; also used for the bias gradient.
__global__ void __launch_bounds__(256) wgrad_reduce_splits(const float* __restrict__ part,
                                                           float* __restrict__ out, size_t n,
                                                           int splits) {
  for (size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n;
       i += static_cast<size_t>(gridDim.x) * blockDim.x) {
    float s = 0.f;
    for (int j = 0; j < splits; ++j) s += __ldg(part + static_cast<size_t>(j) * n + i);
    out[i] = s;
  }
}

// db[k] = sum over pixels of dy[pixel][k]; dy is [pixels][K].  grid = (K/32 column
// groups, row chunks); partial sums are combined with atomics into a zeroed db.
__global__ void __launch_bounds__(256) bias_grad_kernel(const float* __restrict__ dy,
                                                        float* __restrict__ db, size_t pixels,
                                                        int K) {
  __shared__ float red[8][33];
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  const int k = blockIdx.x * 32 + tx;
  const size_t per = (pixels + gridDim.y - 1) / gridDim.y;
  const size_t r0 = blockIdx.y * per;
  const size_t r1 = (r0 + per) < pixels ? (r0 + per) : pixels;
  float s = 0.f;
  if (k < K)
    for (size_t r = r0 + ty; r < r1; r += 8) s += __ldg(dy + r * K + k);
  red[ty][tx] = s;
  __syncthreads();
  if (ty == 0 && k < K) {
    for (int j = 1; j < 8; ++j) s += red[j][tx];
    atomicAdd(db + k, s);
  }
}

namespace wg {

struct Plan {
  WgradParams p;
  size_t smem;
  int grid;
  int map_used[4];
  bool flat;
};

inline int posmod_(int a, int b) { int m = a % b; return m < 0 ? m + b : m; }

// Fills tap table, pixel box, unit grouping and split count.  Returns false if
// the geometry is not supported.
// `smallc`: the few-channel layout where one "tap" is a whole filter row r and its 32
// "channels" are the (s, c) pairs of a spatially pre-padded 4-channel input (see
// mb_conv2d_wgrad_smallc); the gradient then has the shape [K][R][32].
inline bool make_plan(const mb_conv_desc* d, int variant, Plan* pl, bool smallc = false) {
  WgradParams& p = pl->p;
  memset(&p, 0, sizeof(p));
  for (int i = 0; i < 4; ++i) pl->map_used[i] = 0;
  p.K = d->K; p.C = smallc ? 32 : d->C; p.T = smallc ? d->R : d->R * d->S;
  p.cchunks = (p.C + 31) / 32;
  const bool flat = !smallc && d->R == 1 && d->S == 1 && d->stride_h == 1 && d->stride_w == 1 &&
                    d->pad_h == 0 && d->pad_w == 0;
  pl->flat = flat;
  int nt = 0;
  if (smallc) {
    for (int r = 0; r < d->R; ++r) {     // the input is pre-padded: row r of the window is r itself
      const int a = r % d->stride_h;
      pl->map_used[a] = 1;
      p.taps.dh[nt] = static_cast<short>(r / d->stride_h);
      p.taps.dw[nt] = 0;
      p.taps.map[nt] = static_cast<unsigned char>(a);
      p.taps.btap[nt] = static_cast<unsigned char>(r);
      ++nt;
    }
  }
  for (int r = 0; !smallc && r < d->R; ++r) {
    const int oh = r * d->dil_h - d->pad_h;
    const int a = posmod_(oh, d->stride_h), dh = (oh - a) / d->stride_h;
    for (int s = 0; s < d->S; ++s) {
      const int ow = s * d->dil_w - d->pad_w;
      const int b = posmod_(ow, d->stride_w), dw = (ow - b) / d->stride_w;
      if (a >= d->H || b >= d->W) continue;
      const int mi = a * d->stride_w + b;
      pl->map_used[mi] = 1;
      p.taps.dh[nt] = static_cast<short>(dh);
      p.taps.dw[nt] = static_cast<short>(dw);
      p.taps.map[nt] = static_cast<unsigned char>(mi);
      p.taps.btap[nt] = static_cast<unsigned char>(r * d->S + s);
      ++nt;
    }
  }
  if (nt == 0) return false;
  p.ntaps = nt;
  p.units = nt * p.cchunks;
  // CTA tile: 256 x 256 when there are more than 128 output channels, else 128 x 512
  p.KA = d->K > 128 ? 8 : 4;
  const int u_max = p.KA == 8 ? 8 : 16;
  p.groups = (p.units + u_max - 1) / u_max;
  p.U = (p.units + p.groups - 1) / p.groups;
  p.groups = (p.units + p.U - 1) / p.U;
  // chunked form: whole 32-channel chunks on both operands, and every group of units is one
  // tap with U consecutive chunks (units ordered tap-major), so that one 5-d copy per operand
  // fills a stage
  p.chunked = 0;
  if (!smallc && d->C % 32 == 0 && d->K % 32 == 0) {
    int U = p.cchunks < u_max ? p.cchunks : u_max;
    while (p.cchunks % U) --U;
    if (U >= 2 || p.cchunks == 1) {
      p.chunked = 1;
      p.U = U;
      p.groups = p.units / U;
    }
  }
  p.k_tiles = (d->K + 32 * p.KA - 1) / (32 * p.KA);
  // pixel box: rows multiple of 8, slot = (KA + U) * rows * 128 bytes; two slots of large
  // boxes when every box is a copy of its own (the copy engine takes ~70 cycles per copy,
  // whatever its size), three slots when one copy per operand fills a slot
  const int boxes = p.KA + p.U;
  int max_rows = static_cast<int>((212 * 1024 / (p.chunked ? 3 : 2)) / (boxes * 128)) / 8 * 8;
  if (max_rows > 128) max_rows = 128;
  if (max_rows < 8) return false;
  if (flat) {
    const long long pixels = static_cast<long long>(d->N) * d->P * d->Q;
    if (pixels > 0x7fffffffLL) return false;
    p.bw = max_rows > 64 ? 64 : max_rows; p.bh = 1; p.bn = 1;
    p.tiles_w = static_cast<int>((pixels + p.bw - 1) / p.bw);
    p.tiles_h = 1;
    p.pix_tiles = p.tiles_w;
  } else {
    // exhaustive search over boxes {bw, bh, bn}: highest fraction of real pixels per
    // loaded row, larger boxes on ties; bh may exceed P (rows past the image are zero)
    double best = -1.0;
    const int cap = max_rows < 64 ? max_rows : 64;
    for (int bn = 1; bn <= 4 && bn <= d->N; ++bn)
      for (int bh = 1; bh <= d->P + 7 && bh <= 64; ++bh)
        for (int bw = 1; bw <= d->Q && bw <= 128; ++bw) {
          const int rows = bw * bh * bn;
          if (rows % 8 || rows > cap) continue;
          if (bn > 1 && bh < d->P) continue;       // several images only with whole images
          const double tiles = static_cast<double>((d->Q + bw - 1) / bw) * ((d->P + bh - 1) / bh) *
                               ((d->N + bn - 1) / bn);
          const double score = static_cast<double>(d->N) * d->P * d->Q / (tiles * rows) + 1e-3 * rows / 128.0;
          if (score > best) {
            best = score;
            p.bw = bw; p.bh = bh; p.bn = bn;
          }
        }
    if (best < 0) return false;
    p.tiles_w = (d->Q + p.bw - 1) / p.bw;
    p.tiles_h = (d->P + p.bh - 1) / p.bh;
    const long long tiles = static_cast<long long>(p.tiles_w) * p.tiles_h * ((d->N + p.bn - 1) / p.bn);
    if (tiles > 0x7fffffffLL) return false;
    p.pix_tiles = static_cast<int>(tiles);
  }
  p.rows = p.bw * p.bh * p.bn;
  const size_t stage = static_cast<size_t>(boxes) * p.rows * 128;
  int st = static_cast<int>((216 * 1024) / stage);
  if (st > 8) st = 8;
  if (st < 2) return false;
  p.stages = st;
  pl->smem = 512 + 1024 + stage * st;
  // splits: one wave of CTAs (every extra CTA adds a full tile of atomics / partials to
  // combine), at least 4 pixel tiles per split
  const int items = p.k_tiles * p.groups;
  int splits = num_sms() / items;
  const int max_splits = (p.pix_tiles + 3) / 4;
  if (splits > max_splits) splits = max_splits;
  if (splits < 1) splits = 1;
  if (variant == 1 && splits > 64) splits = 64;
  p.splits = splits;
  p.use_atomics = variant == 0;
  pl->grid = items * splits;
  return true;
}

}  // namespace wg

// Defined in conv.cu (needs the tensor-map helpers).
int wgrad_run(const char* who, const float* x, const float* dy, float* dw, float* dbias,
              const mb_conv_desc* d, int variant, void* workspace, size_t workspace_bytes,
              cudaStream_t st);

}  // namespace mb
