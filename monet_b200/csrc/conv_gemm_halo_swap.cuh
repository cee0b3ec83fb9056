// Stride-1 multi-tap forward / backward-data for layers with FEW output channels
// (64 < Kout <= 128): the same halo scheme as conv_gemm_halo.cuh with the operand roles swapped.
//
// An M = 128 MMA takes about as long with 64 columns as with 256 (its A tile of 128 rows is
// fetched from shared memory either way), so with Kout = 64 as the N extent three quarters of
// the tensor pipe's time is wasted.  Here the FILTER tile is the A operand (M = output
// channels, rows past Kout are don't-care) and the ACTIVATION halo box is the B operand
// (N = up to 256 pixels, taps = descriptor row offsets as before): half the MMAs for
// Kout = 128.  (Each of them is slower than an MMA whose 256-row operand starts on a 1024-byte
// swizzle atom - the taps start at arbitrary rows - so the measured gain is 22 % for 128
// channels and nothing for 64; the host side uses this kernel for 65..128 channels only.)
//
// The accumulator then holds D[channel][pixel]: lane = output channel, column = pixel.  The
// epilogue needs no transposition through shared memory: thread (channel k) reads 32 pixels
// of its lane, and for every pixel the 32 lanes of a warp write 32 consecutive channels, i.e.
// one whole 128-byte line of the NHWC output per store instruction.  Pixel -> output offset
// comes from a 256-entry table in shared memory rebuilt per work item (-1 = halo row, skipped).
//
// Roles as in conv_gemm.cuh: warp 4 TMA producer, warp 5 MMA issuer, warps 0-3 epilogue
// (only the warps whose 32 lanes hold real channels work).  All mbarrier waits are bounded.
#pragma once
#include "conv_gemm_halo.cuh"

namespace mb {

struct HaloSwapParams {
  float* out;                // NHWC output, Kout channels per pixel
  const float* bias;         // [Kout] or null
  int Kout;                  // <= 128, multiple of 32
  int Q, P, Nimg;            // output extent
  int kchunks, num_taps;
  int Wh, Hb, bn;            // halo box (pixels); box_rows = Wh*Hb*bn
  int box_rows;
  int a_rows_alloc;          // rows reserved per halo slot (>= ncols + largest tap offset)
  int ncols;                 // MMA N: 128 or 256 pixel columns per work item
  int out_rows;              // pixel rows of an item that can be real outputs: Wh*Hout*bn
  int Hout, bh;
  int tiles_h, tiles_n, num_items;
  int org_w, org_h;
  int act_stages, f_stages;
  int f_mn;                  // 1: filter tiles are MN-major boxes [32-ch group][32 k rows][32 ch]
                             //    straight from a [k][tap][ch] filter (backward-data)
  short tap_off[kMaxTaps];
  unsigned char btap[kMaxTaps];
};

__global__ void __launch_bounds__(192, 1)
conv_gemm_halo_swapped(const __grid_constant__ CUtensorMap mapAct, const __grid_constant__ CUtensorMap mapF,
                       const __grid_constant__ HaloSwapParams p) {
  using namespace sm100;
  extern __shared__ uint8_t smem_raw[];
  uint64_t* act_full = reinterpret_cast<uint64_t*>(smem_raw);      // [4]
  uint64_t* act_empty = act_full + 4;                               // [4]
  uint64_t* f_full = act_empty + 4;                                 // [16]
  uint64_t* f_empty = f_full + 16;                                  // [16]
  uint64_t* acc_full = f_empty + 16;                                // [2]
  uint64_t* acc_empty = acc_full + 2;                               // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  volatile int* epi_ok = abort_flag + 1;                            // [4]
  const uint32_t base0 = (smem_u32(smem_raw) + 512u + 1023u) & ~1023u;
  uint8_t* base_ptr = smem_raw + (base0 - smem_u32(smem_raw));
  const uint32_t act_slot = static_cast<uint32_t>(p.a_rows_alloc) * 128u;
  const uint32_t f_slot = static_cast<uint32_t>(p.Kout) * 128u;
  const uint32_t act_region = act_slot * p.act_stages;
  // the MMA always reads 128 filter rows: one spare tile behind the ring keeps that inside
  // the allocation (those rows land in accumulator lanes nobody reads)
  const uint32_t f_region = f_slot * p.f_stages + 16384u;
  int* row_off = reinterpret_cast<int*>(base_ptr + act_region + f_region);   // [256]

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t acc_cols = static_cast<uint32_t>(p.ncols);
  const uint32_t tmem_cols = 2 * acc_cols < 32 ? 32 : 2 * acc_cols;           // 256 or 512

  if (threadIdx.x == 0) {
    for (int s = 0; s < p.act_stages; ++s) { mbar_init(&act_full[s], 1); mbar_init(&act_empty[s], 1); }
    for (int s = 0; s < p.f_stages; ++s) { mbar_init(&f_full[s], 1); mbar_init(&f_empty[s], 1); }
    for (int a = 0; a < 2; ++a) { mbar_init(&acc_full[a], 1); mbar_init(&acc_empty[a], 128); }
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

  auto decode = [&](int item, int& p0, int& n0) {
    const int ht = item % p.tiles_h;
    const int nt = item / p.tiles_h;
    p0 = ht * p.bh;
    n0 = nt * p.bn;
  };

  if (warp == 4) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      prefetch_tensormap(&mapAct);
      prefetch_tensormap(&mapF);
      detail::Ring ra{0, 0u, p.act_stages}, rf{0, 0u, p.f_stages};
      uint32_t armed_a[4] = {0, 0, 0, 0}, armed_f[16];
      for (int s = 0; s < 16; ++s) armed_f[s] = 0;
      bool ok = true;
      for (int item = blockIdx.x; ok && item < p.num_items; item += gridDim.x) {
        int p0, n0;
        decode(item, p0, n0);
        for (int kc = 0; ok && kc < p.kchunks; ++kc) {
          if (!mbar_wait(&act_empty[ra.stage], ra.phase ^ 1u, abort_flag)) { ok = false; break; }
          mbar_arrive_expect_tx(&act_full[ra.stage], static_cast<uint32_t>(p.box_rows) * 128u);
          armed_a[ra.stage] = 1u + ra.phase;
          tma_load_4d(&mapAct, base_ptr + static_cast<size_t>(ra.stage) * act_slot, &act_full[ra.stage],
                      kc * kChunkK, p.org_w, p0 + p.org_h, n0);
          ra.advance();
          for (int t = 0; t < p.num_taps; ++t) {
            if (!mbar_wait(&f_empty[rf.stage], rf.phase ^ 1u, abort_flag)) { ok = false; break; }
            mbar_arrive_expect_tx(&f_full[rf.stage], f_slot);
            armed_f[rf.stage] = 1u + rf.phase;
            uint8_t* dst = base_ptr + act_region + static_cast<size_t>(rf.stage) * f_slot;
            if (p.f_mn)
              tma_load_4d(&mapF, dst, &f_full[rf.stage], 0, kc * kChunkK, p.btap[t], 0);
            else
              tma_load_3d(&mapF, dst, &f_full[rf.stage], kc * kChunkK, p.btap[t], 0);
            rf.advance();
          }
        }
      }
      if (!ok) {
        *abort_flag = 1;
        atomicCAS(&g_conv_status, 0, 41);
        for (int s = 0; s < p.act_stages; ++s) {
          if (!armed_a[s]) continue;
          const long long t0 = clock64();
          while (!mbar_try_wait(&act_full[s], armed_a[s] - 1u) && clock64() - t0 < 20000000LL) {
          }
        }
        for (int s = 0; s < p.f_stages; ++s) {
          if (!armed_f[s]) continue;
          const long long t0 = clock64();
          while (!mbar_try_wait(&f_full[s], armed_f[s] - 1u) && clock64() - t0 < 20000000LL) {
          }
        }
      }
    }
  } else if (warp == 5) {
    // -------------------------------------------------------------- MMA issuer
    if (lane == 0) {
      const uint32_t idesc = idesc_tf32(kTileM, p.ncols, p.f_mn, 0);
      const uint32_t a_step = p.f_mn ? 64u : 2u;
      detail::Ring ra{0, 0u, p.act_stages}, rf{0, 0u, p.f_stages};
      bool ok = true;
      int it = 0;
      for (int item = blockIdx.x; ok && item < p.num_items; item += gridDim.x, ++it) {
        const int acc = it & 1;
        const uint32_t acc_phase = (it >> 1) & 1u;
        if (!mbar_wait(&acc_empty[acc], acc_phase ^ 1u, abort_flag)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(acc) * acc_cols;
        for (int kc = 0; ok && kc < p.kchunks; ++kc) {
          if (!mbar_wait(&act_full[ra.stage], ra.phase, abort_flag)) { ok = false; break; }
          const uint32_t act_addr = base0 + static_cast<uint32_t>(ra.stage) * act_slot;
          for (int t = 0; t < p.num_taps; ++t) {
            if (!mbar_wait(&f_full[rf.stage], rf.phase, abort_flag)) { ok = false; break; }
            tc_fence_after();
            const uint32_t f_addr = base0 + act_region + static_cast<uint32_t>(rf.stage) * f_slot;
            const uint64_t da = p.f_mn ? smem_desc(f_addr, 4096, 512, kSwizzle128BBase32B)
                                       : smem_desc_sw128(f_addr, 16, 1024);
            // pixel rows of this tap: `tap_off` rows into the halo box
            const uint64_t db = smem_desc_sw128(act_addr + static_cast<uint32_t>(p.tap_off[t]) * 128u, 16, 1024);
            const uint32_t first = (kc | t) == 0 ? 0u : 1u;
#pragma unroll
            for (int k = 0; k < 4; ++k)
              mma_tf32(d_tmem, da + a_step * k, db + 2u * k, idesc, (first | k) != 0 ? 1u : 0u);
            mma_commit(&f_empty[rf.stage]);
            rf.advance();
          }
          if (ok) mma_commit(&act_empty[ra.stage]);
          ra.advance();
        }
        if (ok) mma_commit(&acc_full[acc]);
      }
      if (!ok) {
        *abort_flag = 1;
        atomicCAS(&g_conv_status, 0, 42);
      }
    }
  } else {
    // ---------------------------------------------------------------- epilogue
    bool ok = true;
    int it = 0;
    const int k = warp * 32 + lane;                  // this thread's output channel
    const bool warp_has_channels = warp * 32 < p.Kout;
    const float bias = (p.bias && k < p.Kout) ? __ldg(p.bias + k) : 0.f;
    for (int item = blockIdx.x; ok && item < p.num_items; item += gridDim.x, ++it) {
      const int acc = it & 1;
      const uint32_t acc_phase = (it >> 1) & 1u;
      int p0, n0;
      decode(item, p0, n0);
      const bool got = mbar_wait(&acc_full[acc], acc_phase, abort_flag);
      const bool warp_ok = __all_sync(0xffffffffu, got);
      if (lane == 0) epi_ok[warp] = warp_ok ? 1 : 0;
      named_barrier(1, 128);
      if (!(epi_ok[0] && epi_ok[1] && epi_ok[2] && epi_ok[3])) { ok = false; break; }
      // pixel column m of the accumulator -> element offset of that pixel in the output,
      // or -1 when the column is a halo / padding row
      for (int m = threadIdx.x; m < p.ncols; m += 128) {
        const int wi = m % p.Wh, hi = (m / p.Wh) % p.Hout, ni = m / (p.Wh * p.Hout);
        const bool valid = m < p.out_rows && wi < p.Q && hi < p.bh && p0 + hi < p.P && n0 + ni < p.Nimg;
        row_off[m] = valid ? ((n0 + ni) * p.P + (p0 + hi)) * p.Q + wi : -1;
      }
      named_barrier(1, 128);      // table complete; also orders the epi_ok reads before the next item
      tc_fence_after();
      if (warp_has_channels) {
        const uint32_t t_row = tmem_base + (static_cast<uint32_t>(warp * 32) << 16) +
                               static_cast<uint32_t>(acc) * acc_cols;
        for (int col = 0; col < p.ncols; col += 32) {
          float v[32];
          tmem_ld32(t_row + col, v);
          tmem_ld_wait();
          if (k < p.Kout) {
#pragma unroll
            for (int j = 0; j < 32; ++j) {
              const int off = row_off[col + j];       // same for the whole warp
              if (off >= 0) p.out[static_cast<size_t>(off) * p.Kout + k] = v[j] + bias;
            }
          }
        }
      }
      tc_fence_before();
      mbar_arrive(&acc_empty[acc]);
      named_barrier(1, 128);      // nobody rebuilds the table while another warp still reads it
    }
    if (!ok && lane == 0) {
      *abort_flag = 1;
      atomicCAS(&g_conv_status, 0, 43);
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 5) tmem_dealloc(tmem_base, tmem_cols);
}

}  // namespace mb
