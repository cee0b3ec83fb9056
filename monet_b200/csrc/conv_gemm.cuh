// Implicit-GEMM convolution on the 5th-generation tensor cores (tcgen05, TF32
// inputs, fp32 accumulation in tensor memory), operands fetched by TMA.
//
//   D[pixel, out_channel] = sum over taps t, channel chunks kc of
//                           A_t[pixel, 32 ch] * B_t[out_channel, 32 ch]^T
//
// A is an NHWC activation seen through up to four 4-D tensor maps (one per
// stride phase); a tap is (map, dh, dw, filter tap) and its A tile is the TMA
// box {32 channels, bw, bh, bn pixels} at {kc*32, q0+dw, p0+dh, n0}: halo and
// padding come from TMA's out-of-bounds zero fill, so there is no im2col
// buffer and no per-element index arithmetic.  B is a [out_channel][tap][ch]
// filter.  Forward convolution and backward-data are both instances of this
// kernel (backward-data uses the gradient as A and the transposed filter).
//
// Persistent CTAs (one per SM), 192 threads, three roles:
//   warp 4   TMA producer: fills a ring of `stages` {A,B} slots
//   warp 5   MMA issuer  : one thread issues tcgen05.mma (M=128, N=BN, K=8),
//                          commits free the slots and publish the accumulator
//   warps 6-13 statistics: only when the output's per-channel sums are wanted: they walk the
//                          columns of every staged chunk while the epilogue moves on
//   warps 0-3 epilogue   : tcgen05.ld of a double-buffered accumulator, bias,
//                          128-byte-per-thread stores, overlapped with the
//                          next tile's main loop
// Every mbarrier wait is bounded; on a time-out the CTA records a status code
// in g_conv_status, frees its tensor memory and exits.
#pragma once
#include "common.cuh"
#include "sm100.cuh"

namespace mb {

constexpr int kMaxTaps = 64;
constexpr int kTileM = 128;
constexpr int kChunkK = 32;                     // fp32 per 128-byte swizzle row
constexpr int kAStageBytes = kTileM * 128;      // 16 KiB

struct Taps {
  short dh[kMaxTaps];
  short dw[kMaxTaps];
  unsigned char map[kMaxTaps];
  unsigned char btap[kMaxTaps];
};

struct GemmParams {
  float* out;
  const float* bias;            // may be null
  long long out_sn, out_sh, out_sw;   // element strides of the output pixel grid
  int Nimg, P, Q;               // output pixel grid
  int bn, bh, bw;               // pixels per tile along n / h / w
  int tiles_h, tiles_w, tiles_c;
  int num_tiles;
  int Kout;                     // GEMM N extent (output channels)
  int BN;                       // tile width along N (multiple of 16, <= 256)
  int kchunks;                  // ceil(input channels / 32)
  int num_taps;
  int stages;
  int tma_store;                // epilogue stages tiles in shared memory and stores them with TMA
  int b_mn;                     // 1: the filter tile is MN-major, [32-column group][32 k rows][32 columns]
                                //    straight from a [k][tap][n] filter (backward-data without a transpose)
  long long* prof;              // optional: cycle counters written by CTA 0 (diagnostics), or null
  float* stats;                 // optional: per-CTA partial sums [2][gridDim.x][Kout] of the output
                                // (sum of (y - shift) and of (y - shift)^2 per channel), or null;
                                // needs tma_store and a launch with 448 threads (warps 6-13 do it)
  const float* stats_shift;     // [Kout] shift used in those sums, or null for zero
  Taps taps;
};

// Status word written by kernels that gave up waiting (0 = healthy).
static __device__ int g_conv_status = 0;

namespace detail {

struct Ring {
  int stage;
  uint32_t phase;
  int stages;
  __device__ __forceinline__ void advance() {
    if (++stage == stages) {
      stage = 0;
      phase ^= 1u;
    }
  }
};

}  // namespace detail

// kStats: the instantiation with the statistics warps (448 threads); the plain one has none of
// their code and keeps the 192-thread launch bound.
template <bool kStats>
__global__ void __launch_bounds__(kStats ? 448 : 192, 1)
conv_gemm_kmajor(const __grid_constant__ CUtensorMap mapA0, const __grid_constant__ CUtensorMap mapA1,
                 const __grid_constant__ CUtensorMap mapA2, const __grid_constant__ CUtensorMap mapA3,
                 const __grid_constant__ CUtensorMap mapB, const __grid_constant__ CUtensorMap mapOut,
                 const __grid_constant__ GemmParams p) {
  using namespace sm100;
  extern __shared__ uint8_t smem_raw[];
  // control block first, then 1024-byte aligned operand slots
  uint64_t* full = reinterpret_cast<uint64_t*>(smem_raw);          // [stages]
  uint64_t* empty = full + 16;                                      // [stages]
  uint64_t* acc_full = empty + 16;                                  // [2]
  uint64_t* acc_empty = acc_full + 2;                               // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  volatile int* epi_ok = abort_flag + 1;                            // [4], one per epilogue warp
  uint64_t* stat_full = reinterpret_cast<uint64_t*>(smem_raw + 320);   // [3] staged chunk ready for the statistics warps
  uint64_t* stat_empty = stat_full + 3;                               // [3] statistics warps are done with the buffer
  // staging buffers of the TMA-store epilogue: a third one when statistics warps read them too,
  // so that those warps have two chunk periods to finish with a buffer
  constexpr int nbuf = kStats ? 3 : 2;
  const uint32_t slots0 = (smem_u32(smem_raw) + 512u + 1023u) & ~1023u;
  const uint32_t b_stage_bytes = static_cast<uint32_t>(p.BN) * 128u;
  const uint32_t stage_bytes = kAStageBytes + b_stage_bytes;
  uint8_t* slots_ptr = smem_raw + (slots0 - smem_u32(smem_raw));
  // two 16 KiB staging buffers for the TMA-store epilogue sit behind the operand slots
  uint8_t* stage_out = slots_ptr + static_cast<size_t>(p.stages) * stage_bytes;
  float* s_stats = reinterpret_cast<float*>(stage_out + 3 * kAStageBytes);   // [2][Kout] when p.stats
  int* row_dec = reinterpret_cast<int*>(s_stats + 2 * p.Kout);               // [128] when p.stats
  float* s_shift = reinterpret_cast<float*>(row_dec + kTileM);               // [Kout] when p.stats: the shift, read once

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // two accumulators of BN columns; the epilogue reads whole 32-column groups, so the
  // allocation must also cover the round-up of the second accumulator's last group
  uint32_t tmem_cols = 32;
  while (tmem_cols < static_cast<uint32_t>(p.BN + (p.BN + 31) / 32 * 32)) tmem_cols <<= 1;

  if (threadIdx.x == 0) {
    for (int s = 0; s < p.stages; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&acc_full[a], 1);
      mbar_init(&acc_empty[a], 128);
    }
    for (int a = 0; a < 3; ++a) {
      mbar_init(&stat_full[a], 1);
      mbar_init(&stat_empty[a], 8);      // one arrival per statistics warp
    }
    *abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 5) {
    tmem_alloc(tmem_slot, tmem_cols);
    tmem_relinquish();
  }
  if (kStats) {
    // per-CTA sums start at zero; row_dec[m] = (w, h, n) of tile row m packed 10 bits each, or
    // -1 for rows past the pixel box (the same for every tile of this launch)
    for (int i = threadIdx.x; i < 2 * p.Kout; i += blockDim.x) s_stats[i] = 0.f;
    for (int i = threadIdx.x; i < p.Kout; i += blockDim.x) s_shift[i] = p.stats_shift ? __ldg(p.stats_shift + i) : 0.f;
    for (int m = threadIdx.x; m < kTileM; m += blockDim.x) {
      const int wi = m % p.bw, hi = (m / p.bw) % p.bh, ni = m / (p.bw * p.bh);
      row_dec[m] = m < p.bn * p.bh * p.bw ? (wi | (hi << 10) | (ni << 20)) : -1;
    }
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  const int box_rows = p.bn * p.bh * p.bw;
  const uint32_t tx_bytes = static_cast<uint32_t>(box_rows) * 128u + b_stage_bytes;
  const int kblocks = p.num_taps * p.kchunks;

  auto decode = [&](int tile, int& c0, int& q0, int& p0, int& n0) {
    const int ct = tile % p.tiles_c;
    int r = tile / p.tiles_c;
    const int wt = r % p.tiles_w;
    r /= p.tiles_w;
    const int ht = r % p.tiles_h;
    const int nt = r / p.tiles_h;
    c0 = ct * p.BN;
    q0 = wt * p.bw;
    p0 = ht * p.bh;
    n0 = nt * p.bn;
  };

  if (warp == 4) {
    // ------------------------------------------------------------ TMA producer
    // Lane 0 owns the barriers and copies the activation tile, lane 1 copies the filter tile:
    // the two copies of a stage leave in one warp instruction.
    {
      if (lane == 0) {
        prefetch_tensormap(&mapA0);
        prefetch_tensormap(&mapB);
      }
      detail::Ring ring{0, 0u, p.stages};
      uint32_t armed[16];   // per slot: 0 = never armed, else 1 + parity of the last arming
      for (int s = 0; s < 16; ++s) armed[s] = 0;
      bool ok = true;
      for (int tile = blockIdx.x; ok && tile < p.num_tiles; tile += gridDim.x) {
        int c0, q0, p0, n0;
        decode(tile, c0, q0, p0, n0);
        for (int t = 0; ok && t < p.num_taps; ++t) {
          const int mi = p.taps.map[t];
          const CUtensorMap* ma = mi == 0 ? &mapA0 : mi == 1 ? &mapA1 : mi == 2 ? &mapA2 : &mapA3;
          const int cw = q0 + p.taps.dw[t], ch = p0 + p.taps.dh[t], bt = p.taps.btap[t];
          for (int kc = 0; kc < p.kchunks; ++kc) {
            if (lane == 0) {
              ok = mbar_wait(&empty[ring.stage], ring.phase ^ 1u, abort_flag);
              if (ok) {
                mbar_arrive_expect_tx(&full[ring.stage], tx_bytes);
                armed[ring.stage] = 1u + ring.phase;
              }
            }
            ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
            if (!ok) break;
            uint8_t* slot = slots_ptr + static_cast<size_t>(ring.stage) * stage_bytes;
            if (lane == 0)
              tma_load_4d(ma, slot, &full[ring.stage], kc * kChunkK, cw, ch, n0);
            else if (lane == 1) {
              if (p.b_mn)
                tma_load_4d(&mapB, slot + kAStageBytes, &full[ring.stage], 0, kc * kChunkK, bt, c0 / 32);
              else
                tma_load_3d(&mapB, slot + kAStageBytes, &full[ring.stage], kc * kChunkK, bt, c0);
            }
            ring.advance();
          }
        }
      }
      if (!ok && lane == 0) {
        *abort_flag = 1;
        atomicCAS(&g_conv_status, 0, 1);
        // copies already issued still write this CTA's shared memory: give each armed
        // slot a bounded time to complete before the CTA is allowed to exit
        for (int s = 0; s < p.stages; ++s) {
          if (!armed[s]) continue;
          const long long t0 = clock64();
          while (!mbar_try_wait(&full[s], armed[s] - 1u) && clock64() - t0 < 20000000LL) {
          }
        }
      }
    }
  } else if (warp == 5) {
    // -------------------------------------------------------------- MMA issuer
    if (lane == 0) {
      const uint32_t idesc = idesc_tf32(kTileM, p.BN, 0, p.b_mn);
      const uint32_t b_step = p.b_mn ? 64u : 2u;   // 8 k: 8 rows of 128 bytes, or 32 bytes along a row
      detail::Ring ring{0, 0u, p.stages};
      bool ok = true;
      int it = 0;
      const bool prof = p.prof != nullptr && blockIdx.x == 0;
      long long w_acc = 0, w_full = 0;
      const long long tk0 = prof ? clock64() : 0;
      for (int tile = blockIdx.x; ok && tile < p.num_tiles; tile += gridDim.x, ++it) {
        const int acc = it & 1;
        const uint32_t acc_phase = (it >> 1) & 1u;
        const long long ta0 = prof ? clock64() : 0;
        if (!mbar_wait(&acc_empty[acc], acc_phase ^ 1u, abort_flag)) {
          ok = false;
          break;
        }
        if (prof) w_acc += clock64() - ta0;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(acc * p.BN);
        for (int kb = 0; kb < kblocks; ++kb) {
          const long long tf0 = prof ? clock64() : 0;
          if (!mbar_wait(&full[ring.stage], ring.phase, abort_flag)) {
            ok = false;
            break;
          }
          if (prof) w_full += clock64() - tf0;
          tc_fence_after();
          const uint32_t a_addr = slots0 + static_cast<uint32_t>(ring.stage) * stage_bytes;
          const uint64_t da = smem_desc_sw128(a_addr, 16, 1024);
          const uint32_t b_addr = a_addr + kAStageBytes;
          const uint64_t db = p.b_mn ? smem_desc(b_addr, 4096, 512, kSwizzle128BBase32B)
                                     : smem_desc_sw128(b_addr, 16, 1024);
#pragma unroll
          for (int k = 0; k < 4; ++k)   // 4 x K=8 per 32-channel chunk, 32 bytes apart
            mma_tf32(d_tmem, da + 2u * k, db + b_step * k, idesc, (kb | k) != 0 ? 1u : 0u);
          mma_commit(&empty[ring.stage]);
          ring.advance();
        }
        if (ok) mma_commit(&acc_full[acc]);
      }
      if (prof) { p.prof[0] = clock64() - tk0; p.prof[1] = w_acc; p.prof[2] = w_full; p.prof[3] = it; }
      if (!ok) {
        *abort_flag = 1;
        atomicCAS(&g_conv_status, 0, 2);
      }
    }
  } else if (warp < 4) {
    // ---------------------------------------------------------------- epilogue
    bool ok = true;
    int it = 0;
    int bsel = 0;                 // staging buffer of the next 32-column chunk ...
    uint32_t bphase = 0;          // ... and how many times (mod 2) the buffers have gone round
    for (int tile = blockIdx.x; ok && tile < p.num_tiles; tile += gridDim.x, ++it) {
      const int acc = it & 1;
      const uint32_t acc_phase = (it >> 1) & 1u;
      int c0, q0, p0, n0;
      decode(tile, c0, q0, p0, n0);
      const int m = warp * 32 + lane;
      const int wi = m % p.bw, hi = (m / p.bw) % p.bh, ni = m / (p.bw * p.bh);
      const bool valid = m < box_rows && (n0 + ni) < p.Nimg && (p0 + hi) < p.P && (q0 + wi) < p.Q;
      float* orow = p.out + (n0 + ni) * p.out_sn + (p0 + hi) * p.out_sh + (q0 + wi) * p.out_sw + c0;
      // all four epilogue warps must agree before the warp-collective tensor-memory loads and
      // the named barriers of the store path: every warp always reaches this barrier
      const bool got = mbar_wait(&acc_full[acc], acc_phase, abort_flag);
      const bool warp_ok = __all_sync(0xffffffffu, got);
      if (lane == 0) epi_ok[warp] = warp_ok ? 1 : 0;
      named_barrier(1, 128);
      if (!(epi_ok[0] && epi_ok[1] && epi_ok[2] && epi_ok[3])) {
        ok = false;
        break;
      }
      named_barrier(1, 128);      // flags are read before the next tile overwrites them
      tc_fence_after();
      const uint32_t t_row = tmem_base + (static_cast<uint32_t>(warp * 32) << 16) +
                             static_cast<uint32_t>(acc * p.BN);
      if (p.tma_store) {
        // Each thread owns one output pixel row.  Writing it straight to global memory would
        // touch 32 different cache lines per warp instruction; instead the 128 x 32 chunk is
        // laid out in shared memory in the 128-byte swizzle and one TMA store writes whole
        // lines (and clips what lies outside the tensor).
        for (int col = 0; col < p.BN && c0 + col < p.Kout; col += 32) {
          float v[32];
          tmem_ld32(t_row + col, v);
          tmem_ld_wait();
          uint8_t* buf = stage_out + static_cast<size_t>(bsel) * kAStageBytes;
          if (threadIdx.x == 0) {
            // the store that last read `buf` is done ...
            if (kStats) tma_store_wait_read<2>(); else tma_store_wait_read<1>();
            // ... and so are the statistics warps (first use of a buffer passes at once)
            if (kStats && !mbar_wait_spin(&stat_empty[bsel], bphase ^ 1u, abort_flag)) {
              *abort_flag = 1;
              atomicCAS(&g_conv_status, 0, 4);
            }
          }
          named_barrier(1, 128);
          float4* rowp = reinterpret_cast<float4*>(buf + m * 128);
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            float4 o = make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
            if (p.bias && c0 + col + 4 * j < p.Kout) {
              const float4 b = __ldg(reinterpret_cast<const float4*>(p.bias + c0 + col + 4 * j));
              o.x += b.x; o.y += b.y; o.z += b.z; o.w += b.w;
            }
            rowp[j ^ (m & 7)] = o;
          }
          fence_async_smem();
          named_barrier(1, 128);
          if (threadIdx.x == 0) {
            tma_store_4d(&mapOut, buf, c0 + col, q0, p0, n0);
            tma_store_commit();
            if (kStats) mbar_arrive(&stat_full[bsel]);   // staged chunk visible to warps 6-13
          }
          if (++bsel == nbuf) {      // (a counter, not chunk number % nbuf: a runtime modulo here
            bsel = 0;                //  sat on every chunk's critical path)
            bphase ^= 1u;
          }
        }
      } else {
        for (int col = 0; col < p.BN && c0 + col < p.Kout; col += 32) {
          float v[32];
          tmem_ld32(t_row + col, v);
          tmem_ld_wait();
          if (valid) {
            // columns of this tile that exist: bounded by the tile width and by Kout
            const int left = min(p.Kout - (c0 + col), p.BN - col);
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              if (j * 4 < left) {
                float4 o = make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
                if (p.bias) {
                  const float4 b = __ldg(reinterpret_cast<const float4*>(p.bias + c0 + col + 4 * j));
                  o.x += b.x; o.y += b.y; o.z += b.z; o.w += b.w;
                }
                *reinterpret_cast<float4*>(orow + col + 4 * j) = o;
              }
            }
          }
        }
      }
      tc_fence_before();
      mbar_arrive(&acc_empty[acc]);
    }
    if (p.tma_store && threadIdx.x == 0) tma_store_wait_read<0>();   // staging must outlive the stores
    if (!ok && lane == 0) {
      *abort_flag = 1;
      atomicCAS(&g_conv_status, 0, 3);
    }
  } else if (kStats) {
    // ------------------------------------------------------------- statistics (warps 6-13)
    // Warp w owns columns 4w .. 4w+3 of every staged 32-column chunk, all 128 rows: lane l sums
    // column 4w + (l & 3) over the 16 rows of group l >> 2 (rows visited in a per-group rotated
    // order so that the eight groups read different banks of the swizzled staging buffer), three
    // shuffles combine the groups, and lanes 0-3 add the totals to the CTA's sums in shared
    // memory.  Every column of the output belongs to one fixed thread, so those sums need no
    // atomics (a float atomicAdd on shared memory is a compare-and-swap loop and cost more than
    // the whole walk).  Sums are taken around stats_shift; halo / padding rows are masked.
    // Eight warps rather than four: the walk is bound by one warp's instruction latency, and the
    // epilogue thread waits for it before it reuses a staging buffer.
    const int sw = warp - 6;
    const int cl = lane & 3, grp = lane >> 2;
    const int c = 4 * sw + cl, r0 = 16 * grp;
    const int t = static_cast<int>(threadIdx.x) - 192;
    int row_off8[8];         // byte offset, inside a block of 8 rows, of the j-th row this lane visits
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int r7 = (j + grp) & 7;
      row_off8[j] = r7 * 128 + (((c >> 2) ^ r7) << 4);
    }
    bool ok = true;
    int chunk_no = 0;
    for (int tile = blockIdx.x; ok && tile < p.num_tiles; tile += gridDim.x) {
      int c0, q0, p0, n0;
      decode(tile, c0, q0, p0, n0);
      uint32_t mask = 0;     // bit i: the i-th row this lane visits is a real output pixel
#pragma unroll 4
      for (int i = 0; i < 16; ++i) {
        const int dec = row_dec[r0 + (i & ~7) + ((i + grp) & 7)];
        const bool valid = dec >= 0 && q0 + (dec & 0x3ff) < p.Q && p0 + ((dec >> 10) & 0x3ff) < p.P &&
                           n0 + (dec >> 20) < p.Nimg;
        mask |= (valid ? 1u : 0u) << i;
      }
      // the shift of the next chunk is fetched while this one is walked
      float kk = c0 + c < p.Kout ? s_shift[c0 + c] : 0.f;
      for (int col = 0; col < p.BN && c0 + col < p.Kout; col += 32) {
        const int b = chunk_no % 3;
        const int kn = c0 + col + 32 + c;
        const float kk_next = (col + 32 < p.BN && kn < p.Kout) ? s_shift[kn] : 0.f;
        int got = 1;
        // (try_wait, which parks the lane, not a spin: eight spinning warps would take issue slots
        //  and shared-memory cycles from the epilogue warps; three staging buffers hide the wake-up)
        if (lane == 0) got = mbar_wait(&stat_full[b], (chunk_no / 3) & 1u, abort_flag) ? 1 : 0;
        got = __shfl_sync(0xffffffffu, got, 0);
        if (!got) {
          ok = false;
          break;
        }
        const uint8_t* buf = stage_out + static_cast<size_t>(b) * kAStageBytes;
        const int k = c0 + col + c;
        // the byte offset of row-in-block j for this lane is fixed for the whole kernel (row_off8),
        // so a load costs one address add per 8 rows; two independent chains per sum for ILP
        const uint8_t* colp = buf + r0 * 128 + ((c & 3) << 2);
        float s1a = 0.f, s1b = 0.f, s2a = 0.f, s2b = 0.f;
        if (mask == 0xffffu) {                     // the common case: every row is a real pixel
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const uint8_t* pj = colp + row_off8[j];
            const float d0 = *reinterpret_cast<const float*>(pj) - kk;
            const float d1 = *reinterpret_cast<const float*>(pj + 1024) - kk;
            s1a += d0; s2a = fmaf(d0, d0, s2a);
            s1b += d1; s2b = fmaf(d1, d1, s2b);
          }
        } else {
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const uint8_t* pj = colp + row_off8[j];
            const float v0 = *reinterpret_cast<const float*>(pj);
            const float v1 = *reinterpret_cast<const float*>(pj + 1024);
            const float d0 = ((mask >> j) & 1u) ? v0 - kk : 0.f;
            const float d1 = ((mask >> (8 + j)) & 1u) ? v1 - kk : 0.f;
            s1a += d0; s2a = fmaf(d0, d0, s2a);
            s1b += d1; s2b = fmaf(d1, d1, s2b);
          }
        }
        float s1 = s1a + s1b, s2 = s2a + s2b;
        __syncwarp();                              // every lane has read its column
        if (lane == 0) mbar_arrive(&stat_empty[b]);
#pragma unroll
        for (int x = 4; x <= 16; x <<= 1) {
          s1 += __shfl_xor_sync(0xffffffffu, s1, x);
          s2 += __shfl_xor_sync(0xffffffffu, s2, x);
        }
        if (grp == 0 && k < p.Kout) {              // the one thread that owns column k
          s_stats[k] += s1;
          s_stats[p.Kout + k] += s2;
        }
        kk = kk_next;
        ++chunk_no;
      }
    }
    const bool all_ok = __all_sync(0xffffffffu, ok);
    if (!all_ok && lane == 0) {
      *abort_flag = 1;
      atomicCAS(&g_conv_status, 0, 5);
    }
    named_barrier(2, 256);                       // every statistics warp has added its share
    if (*abort_flag == 0) {
      // this CTA's row of the partial sums: [0][blockIdx.x][k] and [1][blockIdx.x][k]
      float* g1 = p.stats + static_cast<size_t>(blockIdx.x) * p.Kout;
      float* g2 = p.stats + (static_cast<size_t>(gridDim.x) + blockIdx.x) * p.Kout;
      for (int i = t; i < p.Kout; i += 256) {
        g1[i] = s_stats[i];
        g2[i] = s_stats[p.Kout + i];
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 5) tmem_dealloc(tmem_base, tmem_cols);
}

}  // namespace mb
