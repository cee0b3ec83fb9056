// Forward / backward-data convolution for stride-1 filters with several taps:
// the activation tile is fetched ONCE per 32-channel chunk together with its
// halo, and every filter tap reads it through a shared-memory descriptor that
// starts a few 128-byte rows further on.  (conv_gemm.cuh re-fetches a shifted
// tile per tap, which makes 3x3 layers bound by the TMA fill rate.)
//
// Pixels are indexed in "halo-width" order inside the box {32 ch, Wh, Hb, bn}:
//     row = (image * Hb + h) * Wh + w,   Wh = Q + halo_w,   Hb = rows + halo_h
// The output pixel of GEMM row m is the pixel at box row m; for tap t the
// operand row is m + off_t with off_t = dh_t * Wh + dw_t (tap offsets measured
// from the box origin).  Rows whose w >= Q (or h beyond the image) are
// computed and thrown away: the TMA store clips them because they lie outside
// the output tensor.
//
// A CTA works on super-tiles of up to 256 GEMM rows (two M = 128 accumulators
// sharing every filter tile), so a filter tile fetched from L2 feeds twice the
// rows.  Two rings: one of halo boxes (per channel chunk), one of filter tiles
// (per chunk and tap).  Roles as in conv_gemm.cuh.
#pragma once
#include <type_traits>

#include "conv_gemm.cuh"

namespace mb {

struct HaloParams {
  const float* bias;
  int Kout, BN, tiles_c;
  int kchunks, num_taps;
  int Wh, Hb, bn;            // halo box (pixels); rows = Wh*Hb*bn
  int box_rows;              // Wh*Hb*bn
  int a_rows_alloc;          // rows reserved per halo slot (>= MT*128 + largest tap offset)
  int MT;                    // M = 128 accumulators per super-tile (1 or 2)
  int out_rows;              // rows of the staging/store box: Wh*Hout*bn
  int Hout;                  // height of the store box (bh, or Hb when bn > 1)
  int bh;                    // output rows per super-tile
  int tiles_h, tiles_n;      // super-tiles along h and n
  int tiles_w, bw;           // super-tiles along w and their output width (tiles_w == 1: bw == Q)
  int row_stores;            // 1: the store box is one output row of bw pixels (w-tiled maps)
  int Po;                    // output height (row stores skip rows past it)
  int num_items;             // super-tiles * tiles_c
  int org_w, org_h;          // input coordinates of the box origin relative to the output pixel
  int a_stages, b_stages;
  int acc_bufs;              // 1 or 2 accumulator sets in tensor memory
  int b_mn;                  // 1: MN-major filter tiles (see GemmParams)
  long long* prof;           // optional: 16 cycle counters written by CTA 0 (diagnostics), or null
  short tap_off[kMaxTaps];   // operand row offset of each tap
  unsigned char btap[kMaxTaps];
};

__global__ void __launch_bounds__(192, 1)
conv_gemm_halo(const __grid_constant__ CUtensorMap mapA, const __grid_constant__ CUtensorMap mapB,
               const __grid_constant__ CUtensorMap mapOut, const __grid_constant__ HaloParams p) {
  using namespace sm100;
  extern __shared__ uint8_t smem_raw[];
  uint64_t* a_full = reinterpret_cast<uint64_t*>(smem_raw);        // [4]
  uint64_t* a_empty = a_full + 4;                                   // [4]
  uint64_t* b_full = a_empty + 4;                                   // [16]
  uint64_t* b_empty = b_full + 16;                                  // [16]
  uint64_t* acc_full = b_empty + 16;                                // [2]
  uint64_t* acc_empty = acc_full + 2;                               // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  volatile int* epi_ok = abort_flag + 1;                            // [4]
  const uint32_t base0 = (smem_u32(smem_raw) + 512u + 1023u) & ~1023u;
  uint8_t* base_ptr = smem_raw + (base0 - smem_u32(smem_raw));
  const uint32_t a_slot_bytes = static_cast<uint32_t>(p.a_rows_alloc) * 128u;
  const uint32_t b_slot_bytes = static_cast<uint32_t>(p.BN) * 128u;
  const uint32_t a_region = a_slot_bytes * p.a_stages;
  const uint32_t b_region = b_slot_bytes * p.b_stages;
  uint8_t* stage_out = base_ptr + a_region + b_region;              // out_rows * 128 bytes

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t acc_cols = static_cast<uint32_t>(p.MT * p.BN);
  uint32_t tmem_cols = 32;
  while (tmem_cols < acc_cols * p.acc_bufs) tmem_cols <<= 1;

  if (threadIdx.x == 0) {
    for (int s = 0; s < p.a_stages; ++s) { mbar_init(&a_full[s], 1); mbar_init(&a_empty[s], 1); }
    for (int s = 0; s < p.b_stages; ++s) { mbar_init(&b_full[s], 1); mbar_init(&b_empty[s], 1); }
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

  const bool prof = p.prof != nullptr && blockIdx.x == 0;
  auto timed_wait = [&](uint64_t* bar, uint32_t parity, long long& acc_cycles) {
    if (!prof) return mbar_wait(bar, parity, abort_flag);
    const long long t0 = clock64();
    const bool r = mbar_wait(bar, parity, abort_flag);
    acc_cycles += clock64() - t0;
    return r;
  };
  auto decode = [&](int item, int& c0, int& w0, int& p0, int& n0) {
    const int ct = item % p.tiles_c;
    int r = item / p.tiles_c;
    const int wt = r % p.tiles_w;
    r /= p.tiles_w;
    const int ht = r % p.tiles_h;
    const int nt = r / p.tiles_h;
    c0 = ct * p.BN;
    w0 = wt * p.bw;
    p0 = ht * p.bh;
    n0 = nt * p.bn;
  };

  if (warp == 4) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      prefetch_tensormap(&mapA);
      prefetch_tensormap(&mapB);
      detail::Ring ra{0, 0u, p.a_stages}, rb{0, 0u, p.b_stages};
      uint32_t armed_a[4] = {0, 0, 0, 0}, armed_b[16];
      for (int s = 0; s < 16; ++s) armed_b[s] = 0;
      bool ok = true;
      long long w_ae = 0, w_be = 0;
      for (int item = blockIdx.x; ok && item < p.num_items; item += gridDim.x) {
        int c0, w0, p0, n0;
        decode(item, c0, w0, p0, n0);
        for (int kc = 0; ok && kc < p.kchunks; ++kc) {
          if (!timed_wait(&a_empty[ra.stage], ra.phase ^ 1u, w_ae)) { ok = false; break; }
          mbar_arrive_expect_tx(&a_full[ra.stage], static_cast<uint32_t>(p.box_rows) * 128u);
          armed_a[ra.stage] = 1u + ra.phase;
          tma_load_4d(&mapA, base_ptr + static_cast<size_t>(ra.stage) * a_slot_bytes, &a_full[ra.stage],
                      kc * kChunkK, w0 + p.org_w, p0 + p.org_h, n0);
          ra.advance();
          for (int t = 0; t < p.num_taps; ++t) {
            if (!timed_wait(&b_empty[rb.stage], rb.phase ^ 1u, w_be)) { ok = false; break; }
            mbar_arrive_expect_tx(&b_full[rb.stage], b_slot_bytes);
            armed_b[rb.stage] = 1u + rb.phase;
            uint8_t* b_dst = base_ptr + a_region + static_cast<size_t>(rb.stage) * b_slot_bytes;
            if (p.b_mn)
              tma_load_4d(&mapB, b_dst, &b_full[rb.stage], 0, kc * kChunkK, p.btap[t], c0 / 32);
            else
              tma_load_3d(&mapB, b_dst, &b_full[rb.stage], kc * kChunkK, p.btap[t], c0);
            rb.advance();
          }
        }
      }
      if (prof) { p.prof[4] = w_ae; p.prof[5] = w_be; }
      if (!ok) {
        *abort_flag = 1;
        atomicCAS(&g_conv_status, 0, 31);
        for (int s = 0; s < p.a_stages; ++s) {
          if (!armed_a[s]) continue;
          const long long t0 = clock64();
          while (!mbar_try_wait(&a_full[s], armed_a[s] - 1u) && clock64() - t0 < 20000000LL) {
          }
        }
        for (int s = 0; s < p.b_stages; ++s) {
          if (!armed_b[s]) continue;
          const long long t0 = clock64();
          while (!mbar_try_wait(&b_full[s], armed_b[s] - 1u) && clock64() - t0 < 20000000LL) {
          }
        }
      }
    }
  } else if (warp == 5) {
    // -------------------------------------------------------------- MMA issuer
    if (lane == 0) {
      const uint32_t idesc = idesc_tf32(kTileM, p.BN, 0, p.b_mn);
      const uint32_t b_step = p.b_mn ? 64u : 2u;
      detail::Ring ra{0, 0u, p.a_stages}, rb{0, 0u, p.b_stages};
      bool ok = true;
      int it = 0;
      long long w_af = 0, w_bf = 0, w_acc = 0;
      const long long t_start = prof ? clock64() : 0;
      // 3x3 filters (every layer of the networks measured) and the 7x7 stem: the tap loop is
      // unrolled with the tap offsets in registers, descriptors advance by their low word only and barriers are
      // addressed by integer, so that few scalar instructions sit between two MMAs -- with
      // the generic loop below the issuing thread, not the tensor pipe, set the pace.
      auto issue_unrolled = [&](auto taps_c, auto mt_c) {
        constexpr int TAPS = decltype(taps_c)::value;
        constexpr int MTC = decltype(mt_c)::value;
        uint32_t tap16[TAPS];                               // tap offsets in 16-byte units
#pragma unroll
        for (int t = 0; t < TAPS; ++t) tap16[t] = static_cast<uint32_t>(p.tap_off[t]) * 8u;
        const uint64_t da0 = smem_desc_sw128(base0, 16, 1024);
        const uint64_t db0 = p.b_mn ? smem_desc(base0 + a_region, 4096, 512, kSwizzle128BBase32B)
                                    : smem_desc_sw128(base0 + a_region, 16, 1024);
        const uint32_t a_hi = static_cast<uint32_t>(da0 >> 32), a_lo0 = static_cast<uint32_t>(da0);
        const uint32_t b_hi = static_cast<uint32_t>(db0 >> 32), b_lo0 = static_cast<uint32_t>(db0);
        const uint32_t a_stage16 = a_slot_bytes >> 4, b_stage16 = b_slot_bytes >> 4;
        const uint32_t bs1 = b_step, bs2 = 2u * b_step, bs3 = 3u * b_step;
        const uint32_t a_full_u = smem_u32(a_full), a_empty_u = smem_u32(a_empty);
        const uint32_t b_full_u = smem_u32(b_full), b_empty_u = smem_u32(b_empty);
        const uint32_t bn = static_cast<uint32_t>(p.BN);
        for (int item = blockIdx.x; ok && item < p.num_items; item += gridDim.x, ++it) {
          const int acc = p.acc_bufs == 2 ? (it & 1) : 0;
          const uint32_t acc_phase = p.acc_bufs == 2 ? ((it >> 1) & 1u) : (it & 1u);
          if (!timed_wait(&acc_empty[acc], acc_phase ^ 1u, w_acc)) { ok = false; break; }
          tc_fence_after();
          const uint32_t d_base = tmem_base + static_cast<uint32_t>(acc) * acc_cols;
          for (int kc = 0; ok && kc < p.kchunks; ++kc) {
            {
              const long long t0 = prof ? clock64() : 0;
              if (!mbar_wait_u32(a_full_u + 8u * ra.stage, ra.phase, abort_flag)) { ok = false; break; }
              if (prof) w_af += clock64() - t0;
            }
            const uint32_t a_lo = a_lo0 + static_cast<uint32_t>(ra.stage) * a_stage16;
#pragma unroll
            for (int t = 0; t < TAPS; ++t) {
              {
                const long long t0 = prof ? clock64() : 0;
                if (!mbar_wait_u32(b_full_u + 8u * rb.stage, rb.phase, abort_flag)) { ok = false; break; }
                if (prof) w_bf += clock64() - t0;
              }
              tc_fence_after();
              const uint32_t b_lo = b_lo0 + static_cast<uint32_t>(rb.stage) * b_stage16;
#pragma unroll
              for (int mt = 0; mt < MTC; ++mt) {
                const uint32_t al = a_lo + static_cast<uint32_t>(mt * kTileM * 8) + tap16[t];
                const uint32_t dt = d_base + static_cast<uint32_t>(mt) * bn;
                if (t == 0)
                  mma_tf32(dt, pack64(al, a_hi), pack64(b_lo, b_hi), idesc, kc != 0 ? 1u : 0u);
                else
                  mma_tf32_acc(dt, pack64(al, a_hi), pack64(b_lo, b_hi), idesc);
                mma_tf32_acc(dt, pack64(al + 2u, a_hi), pack64(b_lo + bs1, b_hi), idesc);
                mma_tf32_acc(dt, pack64(al + 4u, a_hi), pack64(b_lo + bs2, b_hi), idesc);
                mma_tf32_acc(dt, pack64(al + 6u, a_hi), pack64(b_lo + bs3, b_hi), idesc);
              }
              mma_commit_u32(b_empty_u + 8u * rb.stage);
              rb.advance();
            }
            if (ok) mma_commit_u32(a_empty_u + 8u * ra.stage);
            ra.advance();
          }
          if (ok) mma_commit(&acc_full[acc]);
        }
      };
      if (p.num_taps == 9 && p.MT == 2)
        issue_unrolled(std::integral_constant<int, 9>{}, std::integral_constant<int, 2>{});
      else if (p.num_taps == 9 && p.MT == 1)
        issue_unrolled(std::integral_constant<int, 9>{}, std::integral_constant<int, 1>{});
      else if (p.num_taps == 3 && p.MT == 2)      // 3x3 on a few-channel input: one tap per filter row
        issue_unrolled(std::integral_constant<int, 3>{}, std::integral_constant<int, 2>{});
      else if (p.num_taps == 3 && p.MT == 1)
        issue_unrolled(std::integral_constant<int, 3>{}, std::integral_constant<int, 1>{});
      else if (p.num_taps == 4 && p.MT == 2)      // the 7x7 stride-2 stem: four row taps per phase pair
        issue_unrolled(std::integral_constant<int, 4>{}, std::integral_constant<int, 2>{});
      else if (p.num_taps == 4 && p.MT == 1)
        issue_unrolled(std::integral_constant<int, 4>{}, std::integral_constant<int, 1>{});
      else
      for (int item = blockIdx.x; ok && item < p.num_items; item += gridDim.x, ++it) {
        const int acc = p.acc_bufs == 2 ? (it & 1) : 0;
        const uint32_t acc_phase = p.acc_bufs == 2 ? ((it >> 1) & 1u) : (it & 1u);
        if (!timed_wait(&acc_empty[acc], acc_phase ^ 1u, w_acc)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_base = tmem_base + static_cast<uint32_t>(acc) * acc_cols;
        for (int kc = 0; ok && kc < p.kchunks; ++kc) {
          if (!timed_wait(&a_full[ra.stage], ra.phase, w_af)) { ok = false; break; }
          const uint32_t a_addr = base0 + static_cast<uint32_t>(ra.stage) * a_slot_bytes;
          for (int t = 0; t < p.num_taps; ++t) {
            if (!timed_wait(&b_full[rb.stage], rb.phase, w_bf)) { ok = false; break; }
            tc_fence_after();
            const uint32_t b_addr = base0 + a_region + static_cast<uint32_t>(rb.stage) * b_slot_bytes;
            const uint64_t db = p.b_mn ? smem_desc(b_addr, 4096, 512, kSwizzle128BBase32B)
                                       : smem_desc_sw128(b_addr, 16, 1024);
            const uint32_t first = (kc | t) == 0 ? 0u : 1u;
            for (int mt = 0; mt < p.MT; ++mt) {
              // operand rows of this tap: (mt*128 + off) rows into the halo box
              const uint64_t da = smem_desc_sw128(a_addr + static_cast<uint32_t>(mt * kTileM + p.tap_off[t]) * 128u, 16, 1024);
              const uint32_t d_tmem = d_base + static_cast<uint32_t>(mt * p.BN);
#pragma unroll
              for (int k = 0; k < 4; ++k)
                mma_tf32(d_tmem, da + 2u * k, db + b_step * k, idesc, (first | k) != 0 ? 1u : 0u);
            }
            mma_commit(&b_empty[rb.stage]);
            rb.advance();
          }
          if (ok) mma_commit(&a_empty[ra.stage]);
          ra.advance();
        }
        if (ok) mma_commit(&acc_full[acc]);
      }
      if (prof) { p.prof[0] = clock64() - t_start; p.prof[1] = w_af; p.prof[2] = w_bf; p.prof[3] = w_acc; p.prof[8] = it; }
      if (!ok) {
        *abort_flag = 1;
        atomicCAS(&g_conv_status, 0, 32);
      }
    }
  } else {
    // ---------------------------------------------------------------- epilogue
    bool ok = true;
    int it = 0;
    long long w_full = 0, t_store = 0;
    for (int item = blockIdx.x; ok && item < p.num_items; item += gridDim.x, ++it) {
      const int acc = p.acc_bufs == 2 ? (it & 1) : 0;
      const uint32_t acc_phase = p.acc_bufs == 2 ? ((it >> 1) & 1u) : (it & 1u);
      int c0, w0, p0, n0;
      decode(item, c0, w0, p0, n0);
      const bool got = timed_wait(&acc_full[acc], acc_phase, w_full);
      const long long t_e0 = prof ? clock64() : 0;
      const bool warp_ok = __all_sync(0xffffffffu, got);
      if (lane == 0) epi_ok[warp] = warp_ok ? 1 : 0;
      named_barrier(1, 128);
      if (!(epi_ok[0] && epi_ok[1] && epi_ok[2] && epi_ok[3])) { ok = false; break; }
      named_barrier(1, 128);
      tc_fence_after();
      const uint32_t t_row = tmem_base + (static_cast<uint32_t>(warp * 32) << 16) +
                             static_cast<uint32_t>(acc) * acc_cols;
      for (int col = 0; col < p.BN && c0 + col < p.Kout; col += 32) {
        if (threadIdx.x == 0) tma_store_wait_read<0>();   // the previous store has read the staging
        named_barrier(1, 128);
        for (int mt = 0; mt < p.MT; ++mt) {
          float v[32];
          tmem_ld32(t_row + static_cast<uint32_t>(mt * p.BN + col), v);
          tmem_ld_wait();
          const int m = mt * kTileM + warp * 32 + lane;
          if (m < p.out_rows) {
            float4* rowp = reinterpret_cast<float4*>(stage_out + static_cast<size_t>(m) * 128);
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              float4 o = make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
              if (p.bias && c0 + col + 4 * j < p.Kout) {
                const float4 b = __ldg(reinterpret_cast<const float4*>(p.bias + c0 + col + 4 * j));
                o.x += b.x; o.y += b.y; o.z += b.z; o.w += b.w;
              }
              rowp[j ^ (m & 7)] = o;
            }
          }
        }
        fence_async_smem();
        named_barrier(1, 128);
        if (threadIdx.x == 0) {
          if (!p.row_stores) {
            tma_store_4d(&mapOut, stage_out, c0 + col, w0, p0, n0);
          } else {
            // w-tiled map: the halo columns of this tile are real pixels of the next one, so
            // only the bw pixels the tile owns are stored, one output row at a time (the
            // staging rows keep the halo pitch Wh; the tensor map clips the ragged last tile)
            for (int h = 0; h < p.bh && p0 + h < p.Po; ++h)
              tma_store_4d(&mapOut, stage_out + static_cast<size_t>(h) * p.Wh * 128, c0 + col, w0, p0 + h, n0);
          }
          tma_store_commit();
        }
      }
      tc_fence_before();
      mbar_arrive(&acc_empty[acc]);
      if (prof) t_store += clock64() - t_e0;
    }
    if (prof && threadIdx.x == 0) { p.prof[6] = w_full; p.prof[7] = t_store; }
    if (threadIdx.x == 0) tma_store_wait_read<0>();
    if (!ok && lane == 0) {
      *abort_flag = 1;
      atomicCAS(&g_conv_status, 0, 33);
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 5) tmem_dealloc(tmem_base, tmem_cols);
}

}  // namespace mb
