// 3x3 stride-1 forward / backward-data for layers with 64 output columns (ResNet-50's layer1,
// the first blocks of VGG-16 and of the UNet), two output rows per GEMM row.
//
// With 64 output channels the MMAs of conv_gemm_halo.cuh are 64 columns wide and cost the same
// ~76 cycles as 128-column ones.  Here a GEMM row is a PAIR of vertically adjacent output pixels
// (rows 2j and 2j+1 of the map, same column): accumulator columns 0-63 hold the even row's
// channels, columns 64-127 the odd row's.  Both rows read the same input rows, one filter row
// apart:
//     out(2j)   = in(2j-1) * F[0] + in(2j) * F[1] + in(2j+1) * F[2]
//     out(2j+1) =                   in(2j) * F[0] + in(2j+1) * F[1] + in(2j+2) * F[2]
// so an MMA whose A operand is one input row position and whose B operand is the 128-column
// tile [F[r] | F[r-1]] feeds both.  Four row positions (2j-1 .. 2j+2) x three filter columns
// = 12 MMAs of 128 columns per 32-channel chunk replace 2 x 9 MMAs of 64 columns: a third
// fewer instructions for the same work.
//
// For the A operand the rows of one position must be contiguous, so the input is read through
// two tensor maps, the even rows (E) and the odd rows (O) of the map (row stride 2 * W * C):
// the box {32 ch, Wh, J+1 rows} of each holds, in halo-width pixel order, what the J row pairs
// of a tile need.  Position 2j-1 is O[j-1], 2j is E[j], 2j+1 is O[j], 2j+2 is E[j+1]: two start
// rows in each box, plus the filter column as in conv_gemm_halo.cuh.  The output goes out
// through two maps as well (even and odd rows).
//
// Filter tiles.  The 128-column tile of position pos is [F[pos] | F[pos-1]] with F[3] = F[-1] = 0.
// The three 64-column tiles of a filter column sit in five consecutive 8 KB slots
//     [ 0 | F[2] | F[1] | F[0] | 0 ]
// whose first and last are zeroed once and never written: the tile of position pos is the pair
// of slots starting at slot 3 - pos, so each filter tile is fetched once per (chunk, filter
// column) and serves two positions.  Positions run 3, 2, 1, 0; a slot is handed back to the
// producer after the second position that reads it, which leaves its refill two positions
// (16 MMAs) to land.
#pragma once
#include <type_traits>

#include "conv_gemm.cuh"

namespace mb {

struct PairParams {
  const float* bias;
  int Kout;                 // 64
  int kchunks;
  int Wh, J, Hb;            // box width (Q + 2), row pairs per M = 128 tile, box height MT * J + 1
  int MT;                   // M tiles per work item (1 or 2): they share every filter tile, which
                            // halves the filter traffic from L2 (with one tile the kernel was bound
                            // by it: 24 composite tiles of 16 KB per 224 output pixels)
  int box_rows;             // Wh * Hb
  int a_half;               // bytes reserved per parity box (multiple of 1024)
  int out_rows;             // Wh * J
  int tiles_h, num_items;   // tiles along the row pairs; tiles_w * tiles_h * N work items
  int tiles_w, bw;          // column tiles and the output columns each owns (tiles_w == 1: bw == Q);
                            // with several, a tile stores its bw columns row by row (the two halo
                            // columns of its box are real pixels of the neighbouring tile)
  int a_stages, b_stages;
  int org_w;                // input column of box column 0 relative to the output column
  int rows_even, rows_odd;  // output rows of each parity (row stores skip rows past them)
  int b_mn;                 // 1: MN-major filter tiles (backward-data reads the filter in place)
  short btap[3][3];         // filter tap of grid position (row, column)
  long long* prof;          // optional: cycle counters of CTA 0's MMA thread (diagnostics), or null
};

__global__ void __launch_bounds__(192, 1)
conv_gemm_pair(const __grid_constant__ CUtensorMap mapE, const __grid_constant__ CUtensorMap mapO,
               const __grid_constant__ CUtensorMap mapB, const __grid_constant__ CUtensorMap mapOutE,
               const __grid_constant__ CUtensorMap mapOutO, const __grid_constant__ PairParams p) {
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
  const uint32_t a_slot_bytes = 2u * static_cast<uint32_t>(p.a_half);
  constexpr uint32_t kBHalf = 64u * 128u;                           // 64 columns x 32 k
  const uint32_t a_region = a_slot_bytes * p.a_stages;
  const uint32_t b_region = 5u * kBHalf;
  uint8_t* stage_out = base_ptr + a_region + b_region;              // out_rows * 128 bytes

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t kAccCols = 128u * static_cast<uint32_t>(p.MT);     // columns of one accumulator set
  const uint32_t kTmemCols = 2u * kAccCols;                         // two sets (256 or 512)

  if (threadIdx.x == 0) {
    for (int s = 0; s < p.a_stages; ++s) { mbar_init(&a_full[s], 1); mbar_init(&a_empty[s], 1); }
    for (int s = 0; s < 3; ++s) { mbar_init(&b_full[s], 1); mbar_init(&b_empty[s], 1); }
    for (int a = 0; a < 2; ++a) { mbar_init(&acc_full[a], 1); mbar_init(&acc_empty[a], 128); }
    *abort_flag = 0;
    fence_barrier_init();
  }
  // the two zero filter slots
  for (uint32_t i = threadIdx.x; i < 2u * kBHalf / 16u; i += blockDim.x) {
    const uint32_t slot = i < kBHalf / 16u ? 0u : 4u, j = i < kBHalf / 16u ? i : i - kBHalf / 16u;
    reinterpret_cast<float4*>(base_ptr + a_region + slot * kBHalf)[j] = make_float4(0.f, 0.f, 0.f, 0.f);
  }
  fence_async_smem();
  if (warp == 5) {
    tmem_alloc(tmem_slot, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 4) {
    // ------------------------------------------------------------ TMA producers
    // Lane 0 copies the input boxes, lane 1 the filter tiles.  One thread doing both issued the
    // boxes of a chunk only after the last filter tile of the previous one, i.e. when the MMAs
    // were about to need them (13 % of the issuing thread's time went into that wait).
    if (lane == 0) {
      prefetch_tensormap(&mapE);
      prefetch_tensormap(&mapO);
      detail::Ring ra{0, 0u, p.a_stages};
      uint32_t armed_a[4] = {0, 0, 0, 0};
      bool ok = true;
      for (int item = blockIdx.x; ok && item < p.num_items; item += gridDim.x) {
        const int wt = item % p.tiles_w, ht = (item / p.tiles_w) % p.tiles_h, n0 = item / (p.tiles_w * p.tiles_h);
        const int j0 = ht * p.J * p.MT;                   // first row pair of the work item
        const int w0 = wt * p.bw + p.org_w;               // input column of box column 0
        for (int kc = 0; ok && kc < p.kchunks; ++kc) {
          if (!mbar_wait(&a_empty[ra.stage], ra.phase ^ 1u, abort_flag)) { ok = false; break; }
          mbar_arrive_expect_tx(&a_full[ra.stage], 2u * static_cast<uint32_t>(p.box_rows) * 128u);
          armed_a[ra.stage] = 1u + ra.phase;
          uint8_t* slot = base_ptr + static_cast<size_t>(ra.stage) * a_slot_bytes;
          // E box: input rows 2*j0, 2*j0+2, ...; O box: rows 2*j0-1, 2*j0+1, ... (O row index j0-1)
          tma_load_4d(&mapE, slot, &a_full[ra.stage], kc * kChunkK, w0, j0, n0);
          tma_load_4d(&mapO, slot + p.a_half, &a_full[ra.stage], kc * kChunkK, w0, j0 - 1, n0);
          ra.advance();
        }
      }
      if (!ok) {
        *abort_flag = 1;
        atomicCAS(&g_conv_status, 0, 41);
        for (int s = 0; s < p.a_stages; ++s) {
          if (!armed_a[s]) continue;
          const long long t0 = clock64();
          while (!mbar_try_wait(&a_full[s], armed_a[s] - 1u) && clock64() - t0 < 20000000LL) {
          }
        }
      }
    } else if (lane == 1) {
      prefetch_tensormap(&mapB);
      uint32_t armed_b[3] = {0, 0, 0};
      uint32_t gphase = 0;                                 // parity of the filter-column group
      bool ok = true;
      for (int item = blockIdx.x; ok && item < p.num_items; item += gridDim.x) {
        for (int kc = 0; ok && kc < p.kchunks; ++kc) {
          for (int sx = 0; ok && sx < 3; ++sx) {
            for (int i = 0; i < 3; ++i) {                  // slot 1 + i holds filter row 2 - i
              if (!mbar_wait(&b_empty[i], gphase ^ 1u, abort_flag)) { ok = false; break; }
              mbar_arrive_expect_tx(&b_full[i], kBHalf);
              armed_b[i] = 1u + gphase;
              uint8_t* b_dst = base_ptr + a_region + static_cast<size_t>(1 + i) * kBHalf;
              const int tap = p.btap[2 - i][sx];
              if (p.b_mn)
                tma_load_4d(&mapB, b_dst, &b_full[i], 0, kc * kChunkK, tap, 0);
              else
                tma_load_3d(&mapB, b_dst, &b_full[i], kc * kChunkK, tap, 0);
            }
            gphase ^= 1u;
          }
        }
      }
      if (!ok) {
        *abort_flag = 1;
        atomicCAS(&g_conv_status, 0, 44);
        for (int s = 0; s < 3; ++s) {
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
      const uint32_t idesc = idesc_tf32(kTileM, 128, 0, p.b_mn);
      const uint32_t b_step = p.b_mn ? 64u : 2u;
      detail::Ring ra{0, 0u, p.a_stages};
      uint32_t gphase = 0;                                 // parity of the filter-column group
      bool ok = true;
      int it = 0;
      const uint64_t da0 = smem_desc_sw128(base0, 16, 1024);
      const uint64_t db0 = p.b_mn ? smem_desc(base0 + a_region, 4096, 512, kSwizzle128BBase32B)
                                  : smem_desc_sw128(base0 + a_region, 16, 1024);
      const uint32_t a_hi = static_cast<uint32_t>(da0 >> 32), a_lo0 = static_cast<uint32_t>(da0);
      const uint32_t b_hi = static_cast<uint32_t>(db0 >> 32), b_lo0 = static_cast<uint32_t>(db0);
      const uint32_t a_stage16 = a_slot_bytes >> 4, half16 = static_cast<uint32_t>(p.a_half) >> 4;
      const uint32_t wh16 = static_cast<uint32_t>(p.Wh) * 8u;        // one box row of pixels, in 16-byte units
      const uint32_t tile16 = wh16 * static_cast<uint32_t>(p.J);     // the J box rows of one M tile
      const uint32_t a_full_u = smem_u32(a_full), a_empty_u = smem_u32(a_empty);
      const uint32_t b_full_u = smem_u32(b_full), b_empty_u = smem_u32(b_empty);
      const bool prof = p.prof != nullptr && blockIdx.x == 0;
      long long w_af = 0, w_bf = 0, w_acc = 0;
      const long long t_start = prof ? clock64() : 0;
      // MT is a compile-time constant inside: with a run-time loop over the M tiles the issuing
      // thread needed 118 cycles per MMA and set the pace instead of the tensor pipe
      auto issue = [&](auto mt_c) {
      constexpr int MTC = decltype(mt_c)::value;
      for (int item = blockIdx.x; ok && item < p.num_items; item += gridDim.x, ++it) {
        const int acc = it & 1;
        const uint32_t acc_phase = (it >> 1) & 1u;
        {
          const long long t0 = prof ? clock64() : 0;
          if (!mbar_wait(&acc_empty[acc], acc_phase ^ 1u, abort_flag)) { ok = false; break; }
          if (prof) w_acc += clock64() - t0;
        }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(acc) * kAccCols;
        for (int kc = 0; ok && kc < p.kchunks; ++kc) {
          {
            const long long t0 = prof ? clock64() : 0;
            if (!mbar_wait_u32(a_full_u + 8u * ra.stage, ra.phase, abort_flag)) { ok = false; break; }
            if (prof) w_af += clock64() - t0;
          }
          const uint32_t a_lo = a_lo0 + static_cast<uint32_t>(ra.stage) * a_stage16;
#pragma unroll
          for (int sx = 0; sx < 3; ++sx) {
#pragma unroll
            for (int pp = 0; pp < 4; ++pp) {
              // positions run 3, 2, 1, 0: position 0 = O[j-1], 1 = E[j], 2 = O[j], 3 = E[j+1] (the O box
              // starts at row index j0 - 1); its filter tile is the slot pair starting at slot pp
              const int pos = 3 - pp;
              const uint32_t a_pos = a_lo + ((pos & 1) ? 0u : half16) + ((pos >= 2) ? wh16 : 0u);
              if (pp < 3) {                                   // slot 1 + pp arrives for this position
                const long long t0 = prof ? clock64() : 0;
                if (!mbar_wait_u32(b_full_u + 8u * pp, gphase, abort_flag)) { ok = false; break; }
                if (prof) w_bf += clock64() - t0;
                tc_fence_after();
              }
              const uint32_t b_lo = b_lo0 + static_cast<uint32_t>(pp) * (kBHalf >> 4);
#pragma unroll
              for (int mt = 0; mt < MTC; ++mt) {
                const uint32_t al = a_pos + static_cast<uint32_t>(sx) * 8u + static_cast<uint32_t>(mt) * tile16;
                const uint32_t dt = d_tmem + 128u * static_cast<uint32_t>(mt);
                if (pp == 0 && sx == 0)
                  mma_tf32(dt, pack64(al, a_hi), pack64(b_lo, b_hi), idesc, kc != 0 ? 1u : 0u);
                else
                  mma_tf32_acc(dt, pack64(al, a_hi), pack64(b_lo, b_hi), idesc);
                mma_tf32_acc(dt, pack64(al + 2u, a_hi), pack64(b_lo + b_step, b_hi), idesc);
                mma_tf32_acc(dt, pack64(al + 4u, a_hi), pack64(b_lo + 2u * b_step, b_hi), idesc);
                mma_tf32_acc(dt, pack64(al + 6u, a_hi), pack64(b_lo + 3u * b_step, b_hi), idesc);
              }
              if (pp >= 1) mma_commit_u32(b_empty_u + 8u * (pp - 1));   // slot pp has had both its readers
            }
            if (!ok) break;
            gphase ^= 1u;
          }
          if (ok) mma_commit_u32(a_empty_u + 8u * ra.stage);
          ra.advance();
        }
        if (ok) mma_commit(&acc_full[acc]);
      }
      };
      if (p.MT == 2) issue(std::integral_constant<int, 2>{});
      else issue(std::integral_constant<int, 1>{});
      if (prof) { p.prof[0] = clock64() - t_start; p.prof[1] = w_af; p.prof[2] = w_bf; p.prof[3] = w_acc; p.prof[8] = it; }
      if (!ok) {
        *abort_flag = 1;
        atomicCAS(&g_conv_status, 0, 42);
      }
    }
  } else {
    // ---------------------------------------------------------------- epilogue
    bool ok = true;
    int it = 0;
    for (int item = blockIdx.x; ok && item < p.num_items; item += gridDim.x, ++it) {
      const int acc = it & 1;
      const uint32_t acc_phase = (it >> 1) & 1u;
      const int wt = item % p.tiles_w, ht = (item / p.tiles_w) % p.tiles_h, n0 = item / (p.tiles_w * p.tiles_h);
      const int j0 = ht * p.J * p.MT;
      const bool got = mbar_wait(&acc_full[acc], acc_phase, abort_flag);
      const bool warp_ok = __all_sync(0xffffffffu, got);
      if (lane == 0) epi_ok[warp] = warp_ok ? 1 : 0;
      named_barrier(1, 128);
      if (!(epi_ok[0] && epi_ok[1] && epi_ok[2] && epi_ok[3])) { ok = false; break; }
      named_barrier(1, 128);
      tc_fence_after();
      const uint32_t t_row = tmem_base + (static_cast<uint32_t>(warp * 32) << 16) + static_cast<uint32_t>(acc) * kAccCols;
      // column blocks 0, 1: even output rows, channels 0-31 and 32-63; blocks 2, 3: odd rows
      for (int cbm = 0; cbm < 4 * p.MT; ++cbm) {
        const int mt = cbm >> 2, cb = cbm & 3;
        const int ch0 = (cb & 1) * 32;
        if (threadIdx.x == 0) tma_store_wait_read<0>();   // the previous store has read the staging
        named_barrier(1, 128);
        float v[32];
        tmem_ld32(t_row + static_cast<uint32_t>(mt * 128 + cb * 32), v);
        tmem_ld_wait();
        const int m = warp * 32 + lane;
        if (m < p.out_rows) {
          float4* rowp = reinterpret_cast<float4*>(stage_out + static_cast<size_t>(m) * 128);
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            float4 o = make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
            if (p.bias) {
              const float4 b = __ldg(reinterpret_cast<const float4*>(p.bias + ch0 + 4 * j));
              o.x += b.x; o.y += b.y; o.z += b.z; o.w += b.w;
            }
            rowp[j ^ (m & 7)] = o;
          }
        }
        fence_async_smem();
        named_barrier(1, 128);
        if (threadIdx.x == 0) {
          const CUtensorMap* mo = cb < 2 ? &mapOutE : &mapOutO;
          if (p.tiles_w == 1) {
            tma_store_4d(mo, stage_out, ch0, 0, j0 + mt * p.J, n0);
          } else {
            const int nrows = cb < 2 ? p.rows_even : p.rows_odd;
            for (int jj = 0; jj < p.J && j0 + mt * p.J + jj < nrows; ++jj)
              tma_store_4d(mo, stage_out + static_cast<size_t>(jj) * p.Wh * 128, ch0, wt * p.bw, j0 + mt * p.J + jj, n0);
          }
          tma_store_commit();
        }
      }
      tc_fence_before();
      mbar_arrive(&acc_empty[acc]);
    }
    if (threadIdx.x == 0) tma_store_wait_read<0>();
    if (!ok && lane == 0) {
      *abort_flag = 1;
      atomicCAS(&g_conv_status, 0, 43);
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 5) tmem_dealloc(tmem_base, kTmemCols);
}

}  // namespace mb
