// Backward-weight for filters with several taps (3x3, 5x5, dilated, and - one
// launch per stride phase - strided ones): the input tile is fetched ONCE with
// its halo and every filter tap reads it through a shifted shared-memory
// descriptor.
//
// Both operands are laid out in "halo-width" pixel order: a pixel row index is
//     i = h * Wh + w,   Wh = Q + (S-1)*dil_w   (output width plus the halo)
// The dy box {32 ch, Wh, bh} is loaded at w = 0, so its columns w >= Q are
// out of bounds and arrive as zeros; the x box {32 ch, Wh, bh + (R-1)*dil_h}
// is loaded at (-pad_w, p0 - pad_h).  For tap (r, s) the input pixel paired
// with dy row i is simply x row i + r*dil_h*Wh + s*dil_w: a start-address
// offset of whole 128-byte rows, which the address-based swizzle of the MMA
// accepts unchanged.  The S taps of one filter row are dil_w rows apart, which
// is a legal leading-dimension stride, so ONE MMA (N = 32*S) covers a filter
// row and writes the accumulators of its S taps side by side.
//
// Stride 2: the input is seen as four phase tensors x[:, a::2, b::2]; the taps
// whose (row, column) parity selects phase (a, b) form a small stride-1 filter
// on that tensor, so each phase is one launch of this kernel with its own tap
// list, all adding into the same dw.
//
// Compared with fetching one shifted x box per tap this cuts the x traffic
// from R*S boxes to (bh + halo)/bh boxes per tile.
//
// Wide maps (a row with its halo does not fit a slot, or is wider than a TMA box): the map is
// cut into column tiles of bw pixels.  The x box of a tile still carries its halo columns, but
// the dy columns beyond bw belong to the next tile and must not be summed twice, so dy is
// copied one image row at a time ({32 ch, bw, 1} boxes landing Wh rows apart) into a slot
// that was zeroed once: the columns a tile does not own stay zero for the whole kernel.
//
// Work item: (128 output channels, one 32-channel chunk of x, a range of pixel
// tiles); tensor memory holds the R*S accumulators of 128 x 32.  Rows that pad
// a box up to a multiple of 8 (the MMA's K step) are zeroed once at kernel
// start and never written again.
#pragma once
#include <cmath>

#include "conv_wgrad.cuh"

namespace mb {

struct WgHaloParams {
  float* out;
  long long split_stride;
  int K, C, T;              // output channels, input channels, taps R*S of the whole filter
  int ntaps;                // taps handled by this launch (accumulators in tensor memory)
  int ngroups;              // MMA groups: runs of taps that are `tap_col_pitch` rows apart
  int tap_col_pitch;        // rows between neighbouring taps of a group
  short grp_off[16];        // first operand row offset of each group
  unsigned char grp_n[16];  // taps in the group (N = 32 * grp_n)
  unsigned char grp_first[16];  // index of the group's first tap among this launch's taps
  unsigned char btap[16];   // filter tap (r*S + s) of each of this launch's taps
  int cchunks, k_tiles, splits;
  int Wh, bh;               // box width (pixels incl. halo) and output rows per tile
  int tiles_w, bw;          // column tiles and the dy columns each owns (tiles_w == 1: bw == Q)
  int row_loads;            // 1: dy arrives one image row per copy ({32 ch, bw, 1}), so that the
                            //    Wh - bw columns a tile does not own stay zero (column tiles)
  int a_boxes;              // dy boxes allocated per stage (2..4)
  int rowsA, rowsA_alloc;   // dy box rows (Wh*bh) and its allocation (multiple of 8)
  int rowsB, rowsB_alloc;   // x box rows (Wh*(bh+(R-1)*dil_h)) and its allocation
  int bhB;                  // x box height
  int tiles_h, pix_tiles;
  int org_h, org_w;         // x box origin relative to the dy box origin (in x-view pixels)
  int stages;
  int use_atomics;
  // Filter-row mode (frows > 0; layers with 128 or more input channels, stride 1, dilation 1): a
  // CTA owns ONE filter row and `gch` 32-channel chunks of x.  Its x boxes start at that filter
  // row (no halo rows), the chunks sit back to back, and one MMA per tap s spans all chunks
  // (N = 32 * chunks, leading-dimension stride = one x box) at the operand offset of s rows.
  int frows, S;             // filter rows R (0: mode off) and taps per row
  int gch, cgroups;         // chunks per CTA and ceil(cchunks / gch)
  // Stacked mode (3x3, stride 1, K <= 64): the lower half of the M = 128 operand, which 64 output
  // channels leave empty, holds the same dy channels one image row further down.  An MMA at
  // the x offset of filter row r then yields filter row r in accumulator rows 0-63 and filter
  // row r - 1 in rows 64-127, so offsets r = 1 and r = 3 cover the three filter rows with two
  // MMAs per K step instead of three (rows 0-63 of the second are not used).  Tiles start one
  // row above the map so that both halves see every dy row once.
  int stack;
};

__global__ void __launch_bounds__(192, 1)
conv_wgrad_halo_tcgen05(const __grid_constant__ CUtensorMap mapDy, const __grid_constant__ CUtensorMap mapX,
                        const __grid_constant__ WgHaloParams p) {
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

  const bool rowmode = p.frows > 0;
  int wi = blockIdx.x;
  const int split = wi % p.splits;
  wi /= p.splits;
  int cc, kt, frow = 0, nch = 1;          // first chunk, k tile, filter row, chunks of this CTA
  if (rowmode) {
    cc = (wi % p.cgroups) * p.gch;
    wi /= p.cgroups;
    frow = wi % p.frows;
    kt = wi / p.frows;
    nch = (p.cchunks - cc) < p.gch ? (p.cchunks - cc) : p.gch;
  } else {
    cc = wi % p.cchunks;
    kt = wi / p.cchunks;
  }
  const int xrow = (rowmode && p.stack) ? 1 + 2 * frow : frow;   // x box row offset of this CTA
  const int k0 = kt * kTileM;
  int ka = (p.K - k0 + 31) / 32;
  if (ka > 4) ka = 4;
  const int per = (p.pix_tiles + p.splits - 1) / p.splits;
  const int t_begin = split * per;
  const int t_end = (t_begin + per) < p.pix_tiles ? (t_begin + per) : p.pix_tiles;
  const int n_iter = t_end > t_begin ? t_end - t_begin : 0;

  // Shared memory: the dy boxes of all stages first, then the x boxes.  An MMA always spans
  // four dy boxes (M = 128); with fewer allocated (K <= 96) the rows of the missing ones are
  // read from whatever follows -- the next stage's dy boxes or the x region, which the host
  // sizes to cover them -- and land in accumulator rows that are never stored.
  const uint32_t a_box = static_cast<uint32_t>(p.rowsA_alloc) * 128u;
  const uint32_t a_bytes = static_cast<uint32_t>(p.a_boxes) * a_box;
  const uint32_t b_box = static_cast<uint32_t>(p.rowsB_alloc) * 128u;
  const uint32_t b_bytes = b_box * static_cast<uint32_t>(rowmode ? p.gch : 1);
  const uint32_t b_region = static_cast<uint32_t>(p.stages) * a_bytes;
  const int ndy = p.stack ? 2 * ka : ka;   // dy boxes copied per stage
  const uint32_t tx_bytes =
      static_cast<uint32_t>((p.row_loads ? ndy * p.bh * p.bw : ndy * p.rowsA) + nch * p.rowsB) * 128u;
  uint32_t tmem_cols = 32;
  while (tmem_cols < 32u * (rowmode ? p.S * p.gch : p.ntaps)) tmem_cols <<= 1;

  if (threadIdx.x == 0) {
    for (int s = 0; s < p.stages; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    mbar_init(&acc_full[0], 1);
    *abort_flag = 0;
    fence_barrier_init();
  }
  // zero every slot once: the rows that pad a box up to a multiple of 8 and, with column tiles,
  // the columns of a dy row that belong to the neighbouring tile are never written by TMA
  {
    float4* z = reinterpret_cast<float4*>(slots_ptr);
    const uint32_t n16 = static_cast<uint32_t>(p.stages) * (a_bytes + b_bytes) / 16u;
    for (uint32_t i = threadIdx.x; i < n16; i += blockDim.x) z[i] = make_float4(0.f, 0.f, 0.f, 0.f);
  }
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // visible to the tensor core
  if (warp == 5) {
    tmem_alloc(tmem_slot, tmem_cols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 4) {
    // TMA producer: lanes 0..ka-1 copy the dy boxes, lane ka the x box, in one warp instruction;
    // lane 0 owns the barriers
    if (n_iter > 0) {
      if (lane == 0) {
        prefetch_tensormap(&mapDy);
        prefetch_tensormap(&mapX);
      }
      detail::Ring ring{0, 0u, p.stages};
      uint32_t armed[16];
      for (int s = 0; s < 16; ++s) armed[s] = 0;
      bool ok = true;
      int wt = t_begin % p.tiles_w, ht = (t_begin / p.tiles_w) % p.tiles_h, n0 = t_begin / (p.tiles_w * p.tiles_h);
      for (int t = t_begin; t < t_end; ++t) {
        const int p0 = ht * p.bh - (p.stack ? 1 : 0), w0 = wt * p.bw;
        if (lane == 0) {
          ok = mbar_wait(&empty[ring.stage], ring.phase ^ 1u, abort_flag);
          if (ok) {
            mbar_arrive_expect_tx(&full[ring.stage], tx_bytes);
            armed[ring.stage] = 1u + ring.phase;
          }
        }
        ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
        if (!ok) break;
        uint8_t* slot_a = slots_ptr + static_cast<size_t>(ring.stage) * a_bytes;
        uint8_t* slot_b = slots_ptr + b_region + static_cast<size_t>(ring.stage) * b_bytes;
        if (!p.row_loads) {
          if (lane < ndy) {
            // stacked: copies ka.. go to boxes 2.. and start one image row further down
            const int half = lane / ka, j = lane - half * ka;
            tma_load_4d(&mapDy, slot_a + (2 * half + j) * a_box, &full[ring.stage], k0 + 32 * j, 0, p0 + half, n0);
          } else if (lane < ndy + nch) {
            tma_load_4d(&mapX, slot_b + (lane - ndy) * b_box, &full[ring.stage], (cc + lane - ndy) * 32, p.org_w,
                        p0 + p.org_h + xrow, n0);
          }
        } else {
          // one copy per (dy box, image row): row h of a box starts h * Wh rows in, and Wh is a
          // multiple of 8 rows, so every copy lands on a whole swizzle atom
          const int nrow = ndy * p.bh;
          for (int l = lane; l < nrow + nch; l += 32) {
            if (l < nrow) {
              const int d = l / p.bh, h = l - d * p.bh;
              const int half = d / ka, j = d - half * ka;
              tma_load_4d(&mapDy, slot_a + (2 * half + j) * a_box + static_cast<size_t>(h) * p.Wh * 128,
                          &full[ring.stage], k0 + 32 * j, w0, p0 + half + h, n0);
            } else {
              tma_load_4d(&mapX, slot_b + (l - nrow) * b_box, &full[ring.stage], (cc + l - nrow) * 32,
                          w0 + p.org_w, p0 + p.org_h + xrow, n0);
            }
          }
        }
        ring.advance();
        if (++wt == p.tiles_w) {
          wt = 0;
          if (++ht == p.tiles_h) { ht = 0; ++n0; }
        }
      }
      if (!ok && lane == 0) {
        *abort_flag = 1;
        atomicCAS(&g_conv_status, 0, 21);
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
      const int ksteps = p.rowsA_alloc / 8;
      for (int it = 0; it < n_iter; ++it) {
        if (!mbar_wait(&full[ring.stage], ring.phase, abort_flag)) {
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t a_addr = slots0 + static_cast<uint32_t>(ring.stage) * a_bytes;
        const uint32_t b_addr = slots0 + b_region + static_cast<uint32_t>(ring.stage) * b_bytes;
        const uint64_t da = smem_desc(a_addr, a_box, 512, kSwizzle128BBase32B);
        if (rowmode) {
          // one MMA per tap of the filter row, N = all chunks of this CTA (LBO = one x box)
          const uint32_t idesc = idesc_tf32(kTileM, 32 * nch, 1, 1);
          for (int sx = 0; sx < p.S; ++sx) {
            const uint64_t db = smem_desc(b_addr + static_cast<uint32_t>(sx * p.tap_col_pitch) * 128u, b_box, 512,
                                          kSwizzle128BBase32B);
            const uint32_t d_tmem = tmem_base + 32u * static_cast<uint32_t>(sx * p.gch);
            for (int k = 0; k < ksteps; ++k)
              mma_tf32(d_tmem, da + 64u * k, db + 64u * k, idesc, (it | k) != 0 ? 1u : 0u);
          }
        } else
        for (int g = 0; g < p.ngroups; ++g) {
          // the taps of a group are tap_col_pitch rows apart, which is the descriptor's LBO
          const uint32_t idesc = idesc_tf32(kTileM, 32 * p.grp_n[g], 1, 1);
          const uint64_t db = smem_desc(b_addr + static_cast<uint32_t>(p.grp_off[g]) * 128u,
                                        static_cast<uint32_t>(p.tap_col_pitch) * 128u, 512,
                                        kSwizzle128BBase32B);
          const uint32_t d_tmem = tmem_base + 32u * p.grp_first[g];
          for (int k = 0; k < ksteps; ++k)
            mma_tf32(d_tmem, da + 64u * k, db + 64u * k, idesc, (it | k) != 0 ? 1u : 0u);
        }
        mma_commit(&empty[ring.stage]);
        ring.advance();
      }
      if (ok) {
        mma_commit(&acc_full[0]);
      } else {
        *abort_flag = 1;
        atomicCAS(&g_conv_status, 0, 22);
      }
    }
  } else if (n_iter > 0 || !p.use_atomics) {
    bool got = n_iter > 0 ? mbar_wait(&acc_full[0], 0, abort_flag) : true;
    got = __all_sync(0xffffffffu, got);
    if (got) {
      tc_fence_after();
      float* base = p.out + static_cast<long long>(split) * p.split_stride;
      // stacked: accumulator rows 64-127 (warps 2, 3) are output channels 0-63 again
      const int k = k0 + (p.stack ? (warp & 1) : warp) * 32 + lane;
      const int n_units = rowmode ? p.S * nch : (p.stack ? 2 * p.S : p.ntaps);
      for (int u = 0; u < n_units; ++u) {
        // unit -> accumulator column block, filter tap and 32-channel chunk
        const int sx = rowmode ? u / nch : 0, cj = rowmode ? u - sx * nch : 0;
        const int t = rowmode ? sx * p.gch + cj : u;
        int tap = rowmode ? p.btap[(p.stack ? 0 : frow) * p.S + sx] : p.btap[p.stack ? 0 : u];
        if (rowmode && p.stack) {
          // x offset of filter row 1 (frow 0): rows 0-63 -> filter row 1, rows 64-127 -> row 0;
          // offset of "row 3" (frow 1): rows 64-127 -> filter row 2, rows 0-63 unused
          const int frow_of = warp < 2 ? (frow == 0 ? 1 : -1) : (frow == 0 ? 0 : 2);
          if (frow_of < 0) continue;
          tap = p.btap[frow_of * p.S + sx];
        } else if (p.stack) {
          // block 0 (x offset of filter row 1): rows 0-63 -> filter row 1, rows 64-127 -> row 0;
          // block 1 (offset of "row 3"): rows 64-127 -> filter row 2, rows 0-63 unused
          const int blk = u / p.S, sc = u - blk * p.S;
          const int frow_of = warp < 2 ? (blk == 0 ? 1 : -1) : (blk == 0 ? 0 : 2);
          if (frow_of < 0) continue;
          tap = p.btap[frow_of * p.S + sc];
        }
        const int cu = cc + cj;
        float v[32];
        if (n_iter > 0) {
          tmem_ld32(tmem_base + (static_cast<uint32_t>(warp * 32) << 16) + 32u * t, v);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] = 0.f;
        }
        if (k < p.K) {
          float* dst = base + (static_cast<long long>(k) * p.T + tap) * p.C + cu * 32;
          const int left = p.C - cu * 32;
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
    } else if (lane == 0) {
      *abort_flag = 1;
      atomicCAS(&g_conv_status, 0, 23);
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 5) tmem_dealloc(tmem_base, tmem_cols);
}

namespace wgh {

struct Plan {
  WgHaloParams p;
  size_t smem;
  int grid;
  int items;      // work items before the pixel split: grid = items * splits
};

struct Tap { int dh, dw, btap; };   // x pixel = dy pixel + (dh, dw) in the x view; filter tap index

// One launch: dy grid P x Q (x N images), an x view, and the taps that read that view.
// `taps` must be sorted by (dh, dw).  Returns false when the geometry does not fit.
// `frows` > 0 asks for the filter-row mode (the taps must then be the full frows x S grid at
// dilation 1): a CTA takes one filter row and up to 16 / S chunks of x.
inline bool plan_launch(int K, int C, int T, int N, int P, int Q, const Tap* taps, int ntaps,
                        int variant, Plan* pl, int frows = 0, int S = 0) {
  if (ntaps < 1 || ntaps > 16) return false;
  WgHaloParams& p = pl->p;
  memset(&p, 0, sizeof(p));
  p.K = K; p.C = C; p.T = T; p.ntaps = ntaps;
  int min_dh = taps[0].dh, max_dh = taps[0].dh, min_dw = taps[0].dw, max_dw = taps[0].dw;
  for (int t = 1; t < ntaps; ++t) {
    if (taps[t].dh < min_dh) min_dh = taps[t].dh;
    if (taps[t].dh > max_dh) max_dh = taps[t].dh;
    if (taps[t].dw < min_dw) min_dw = taps[t].dw;
    if (taps[t].dw > max_dw) max_dw = taps[t].dw;
  }
  // stacked mode: a full 3x3 grid of taps at dilation 1 and at most 64 output channels
  bool stack = (frows == 0 || (frows == 3 && S == 3)) && K <= 64 && ntaps == 9;
  for (int t = 0; stack && t < 9; ++t)
    stack = taps[t].dh == min_dh + t / 3 && taps[t].dw == min_dw + t % 3;
  p.stack = stack ? 1 : 0;
  // in filter-row mode the x boxes of a CTA start at its filter row: no halo rows; in stacked
  // mode the second MMA reads at the offset of a fourth filter row
  const int halo_h = frows > 0 ? 0 : (stack ? 3 : max_dh - min_dh), halo_w = max_dw - min_dw;
  p.org_h = min_dh; p.org_w = min_dw;
  p.cchunks = (C + 31) / 32;
  p.k_tiles = (K + kTileM - 1) / kTileM;
  // filter-row mode stacked: the two x offsets (filter rows 1 and "3") are the work items
  p.frows = (frows > 0 && stack) ? 2 : frows; p.S = S; p.gch = 1; p.cgroups = p.cchunks;
  if (frows > 0) {
    if (S < 1 || S > 16 || frows * S != ntaps) return false;
    const int gmax = 16 / S;                       // 512 accumulator columns / (32 * S)
    p.cgroups = (p.cchunks + gmax - 1) / gmax;
    p.gch = (p.cchunks + p.cgroups - 1) / p.cgroups;
  }
  const int xb = p.gch;                            // x boxes per stage
  // dy boxes per stage: all four of an M = 128 MMA unless the whole of K fits in fewer
  p.a_boxes = (p.k_tiles > 1 || K > 96 || stack) ? 4 : (K > 64 ? 3 : 2);
  auto sizes = [&](int Wh, int bh, int* ra, int* raa, int* rb, int* rba) {
    *ra = Wh * bh;
    *raa = (*ra + 7) / 8 * 8;
    *rb = Wh * (bh + halo_h);
    // the last tap of the last (padding) dy row reads up to raa + halo rows + halo columns
    const int reach = *raa + halo_h * Wh + halo_w;
    *rba = ((reach > *rb ? reach : *rb) + 7) / 8 * 8;
  };
  // largest tile height whose stage fits a slot of 108 KiB (two slots: larger tiles beat a
  // third, smaller slot -- measured); 0 when not even one row fits
  auto fit_bh = [&](int Wh, bool rows) {
    for (int bh = P; bh >= 1; --bh) {
      if (bh + halo_h > 256) continue;
      if (rows && p.a_boxes * bh + xb > 32) continue;       // one copy per lane of the producer warp
      int ra, raa, rb, rba;
      sizes(Wh, bh, &ra, &raa, &rb, &rba);
      if (static_cast<size_t>(p.a_boxes * raa + xb * rba) * 128 <= 108 * 1024) return bh;
    }
    return 0;
  };
  // Whole rows in a box when that fits (Wh = Q + halo).  Otherwise -- maps wider than a TMA box
  // or than a slot -- the map is cut into column tiles of bw pixels: dy is copied row by row so
  // that the Wh - bw columns a tile does not own stay zero and add nothing to the sums; Wh is
  // rounded up to 8 rows so that every row copy starts on a swizzle atom.
  p.tiles_w = 1; p.bw = Q; p.row_loads = 0;
  p.Wh = Q + halo_w;
  int best_bh = p.Wh <= 256 ? fit_bh(p.Wh, false) : 0;
  if (!best_bh) {
    if (C % 4 != 0 || K % 4 != 0) return false;           // row copies need 16-byte pixel strides
    double best = 0.0;
    for (int tw = 2; tw <= (Q + 7) / 8; ++tw) {
      const int bw = (Q + tw - 1) / tw;
      const int Wh = (bw + halo_w + 7) / 8 * 8;
      if (Wh > 256) continue;
      const int bh0 = fit_bh(Wh, true);
      if (!bh0) continue;
      const int th = (P + bh0 - 1) / bh0, bh = (P + th - 1) / th;
      // MMA rows that are real pixels, times a penalty for refetching the halo rows of x
      const double eff = static_cast<double>(Q) * P / (static_cast<double>(tw) * th * Wh * bh);
      const double score = eff * std::sqrt(static_cast<double>(bh) / (bh + halo_h));
      if (score > best + 1e-9) {
        best = score; best_bh = bh0;
        p.tiles_w = tw; p.bw = bw; p.Wh = Wh; p.row_loads = 1;
      }
    }
    if (!best_bh) return false;
  }
  const int Pt = P + (stack ? 1 : 0);              // stacked tiles start one row above the map
  p.tiles_h = (Pt + best_bh - 1) / best_bh;
  p.bh = (Pt + p.tiles_h - 1) / p.tiles_h;         // balanced tiles
  p.bhB = p.bh + halo_h;
  sizes(p.Wh, p.bh, &p.rowsA, &p.rowsA_alloc, &p.rowsB, &p.rowsB_alloc);
  // column pitch: smallest positive dw difference inside a row of taps
  int pitch = 0;
  for (int t = 1; t < ntaps; ++t)
    if (taps[t].dh == taps[t - 1].dh && (pitch == 0 || taps[t].dw - taps[t - 1].dw < pitch))
      pitch = taps[t].dw - taps[t - 1].dw;
  if (pitch <= 0) pitch = 1;
  p.tap_col_pitch = pitch;
  int ng = 0;
  for (int t = 0; t < ntaps; ++t) {
    p.btap[t] = static_cast<unsigned char>(taps[t].btap);
    const bool extend = ng > 0 && taps[t].dh == taps[t - 1].dh && taps[t].dw - taps[t - 1].dw == pitch &&
                        p.grp_n[ng - 1] < 8;
    if (extend) {
      ++p.grp_n[ng - 1];
    } else {
      if (ng >= 16) return false;
      p.grp_off[ng] = static_cast<short>((taps[t].dh - min_dh) * p.Wh + (taps[t].dw - min_dw));
      p.grp_n[ng] = 1;
      p.grp_first[ng] = static_cast<unsigned char>(t);
      ++ng;
    }
  }
  p.ngroups = ng;
  if (stack && frows == 0) {
    // two MMAs per K step: at the x offsets of filter rows 1 and "3", three taps wide each
    p.S = 3;
    p.ngroups = 2;
    for (int g = 0; g < 2; ++g) {
      p.grp_off[g] = static_cast<short>((1 + 2 * g) * p.Wh);
      p.grp_n[g] = 3;
      p.grp_first[g] = static_cast<unsigned char>(3 * g);
    }
  }
  const long long tiles = static_cast<long long>(p.tiles_w) * p.tiles_h * N;
  if (tiles > 0x7fffffffLL) return false;
  p.pix_tiles = static_cast<int>(tiles);
  const size_t stage = static_cast<size_t>(p.a_boxes * p.rowsA_alloc + xb * p.rowsB_alloc) * 128;
  int st = static_cast<int>((216 * 1024) / stage);
  if (st > 8) st = 8;
  if (st < 2) return false;
  p.stages = st;
  pl->smem = 512 + 1024 + stage * st;
  const int items = frows > 0 ? p.k_tiles * p.frows * p.cgroups : p.k_tiles * p.cchunks;
  // one wave of CTAs: the kernel is bound by MMA issue, a second wave would only repeat the
  // set-up and double the number of partial results to combine
  int splits = num_sms() / items;
  const int max_splits = (p.pix_tiles + 3) / 4;
  if (splits > max_splits) splits = max_splits;
  if (splits < 1) splits = 1;
  if (variant == 1 && splits > 64) splits = 64;
  p.splits = splits;
  p.use_atomics = variant == 0;
  pl->items = items;
  pl->grid = items * splits;
  return true;
}

// The launches of a whole convolution: one for stride 1, one per non-empty stride phase
// otherwise.  `phase[i]` says which input phase (a, b) launch i reads.
struct Launches {
  int n;
  Plan plan[4];
  int phase_a[4], phase_b[4];
};

// The halo kernel saves shared-memory fill (x is fetched once instead of once per tap) but
// its MMAs are only 32 * S columns wide, which is below the tensor pipe's floor of ~76 cycles
// per instruction.  With 128 or more input channels the per-tap kernel of conv_wgrad.cuh
// (256-column MMAs, one 5-d copy per operand and stage) is faster on every map size measured
// (28x28: equal, 14x14 and 7x7: 1.3-1.8x, stride 2: 2x); with fewer channels it would be bound
// by the 9-fold refetch of x, so those layers (64 channels on 56x56 maps) stay here.
inline bool eligible(const mb_conv_desc* d) {
  if (d->groups != 1 || d->R * d->S <= 1 || d->R * d->S > 16) return false;
  const bool per_tap_ok = d->C % 32 == 0 && d->K % 32 == 0 && d->C >= 128;
  if (per_tap_ok) return false;
  if (d->stride_h == 1 && d->stride_w == 1) return true;
  return d->stride_h <= 2 && d->stride_w <= 2 && d->Q >= 24 && d->P >= 24;
}

// Filter-row mode: stride 1, dilation 1, whole 32-channel chunks, at least 128 input channels.
// Where it is used is a matter of measurement against the per-tap kernel of conv_wgrad.cuh
// (batch 176 VGG-16 and batch 11 UNet layers, all 3x3): that kernel's 256 x 256 tile needs 2 KB
// of operands per pixel from L2 and is starved by it on most layers, this mode needs 1 KB for
// three quarters of the work but issues 128-column MMAs and pads every row to Wh.  It wins for
// 128 input channels on every map (1.43 -> 1.18 ms on 112x112, 0.46 -> 0.35 on 208x304) and for
// 256 / 512 input channels unless K = 256 -- where the per-tap kernel has one M = 256 tile, its
// best case (0.93 against 1.39 ms) -- or the map is small or the work items leave SMs idle.
inline bool row_mode_ok(const mb_conv_desc* d) {
  if (!(d->groups == 1 && d->R * d->S > 1 && d->R * d->S <= 16 && d->stride_h == 1 && d->stride_w == 1 &&
        d->dil_h == 1 && d->dil_w == 1 && d->C % 32 == 0 && d->K % 4 == 0 && d->C >= 128))
    return false;
  if (d->C == 128) return true;
  return d->C <= 512 && d->K != 256 && static_cast<long long>(d->P) * d->Q >= 700;
}

inline bool make_plans(const mb_conv_desc* d, int variant, Launches* L) {
  if (row_mode_ok(d)) {
    Tap taps[16];
    int nt = 0;
    for (int r = 0; r < d->R; ++r)
      for (int s = 0; s < d->S; ++s) taps[nt++] = Tap{r - d->pad_h, s - d->pad_w, r * d->S + s};
    L->n = 1;
    L->phase_a[0] = L->phase_b[0] = 0;
    // only when its work items fill the SMs: k tiles x filter rows x chunk groups x pixel splits
    if (plan_launch(d->K, d->C, d->R * d->S, d->N, d->P, d->Q, taps, nt, variant, &L->plan[0], d->R, d->S) &&
        L->plan[0].grid * 100 >= num_sms() * 85)
      return true;
  }
  if (!eligible(d)) return false;
  L->n = 0;
  for (int a = 0; a < d->stride_h; ++a)
    for (int b = 0; b < d->stride_w; ++b) {
      if (a >= d->H || b >= d->W) continue;
      Tap taps[16];
      int nt = 0;
      for (int r = 0; r < d->R; ++r) {
        const int oh = r * d->dil_h - d->pad_h;
        if (((oh % d->stride_h) + d->stride_h) % d->stride_h != a) continue;
        for (int s = 0; s < d->S; ++s) {
          const int ow = s * d->dil_w - d->pad_w;
          if (((ow % d->stride_w) + d->stride_w) % d->stride_w != b) continue;
          taps[nt++] = Tap{(oh - a) / d->stride_h, (ow - b) / d->stride_w, r * d->S + s};
        }
      }
      if (nt == 0) continue;
      if (!plan_launch(d->K, d->C, d->R * d->S, d->N, d->P, d->Q, taps, nt, variant, &L->plan[L->n]))
        return false;
      L->phase_a[L->n] = a;
      L->phase_b[L->n] = b;
      ++L->n;
    }
  if (L->n == 0) return false;
  if (variant == 1) {
    // the deterministic variant sums per-split partials: every launch must use the same split
    // count and together they must write every tap
    for (int i = 1; i < L->n; ++i)
      if (L->plan[i].p.splits != L->plan[0].p.splits) {
        const int s0 = L->plan[0].p.splits < L->plan[i].p.splits ? L->plan[0].p.splits : L->plan[i].p.splits;
        for (int j = 0; j < L->n; ++j) {
          L->plan[j].p.splits = s0;
          L->plan[j].grid = L->plan[j].items * s0;
        }
      }
  }
  return true;
}

}  // namespace wgh

// Workspace of the deterministic variant: one partial dw per split of whichever kernel runs.
inline size_t wgrad_workspace_bytes(const mb_conv_desc* d, int variant) {
  if (variant != 1 || d->groups != 1) return 0;
  const size_t dw_bytes = static_cast<size_t>(d->K) * d->R * d->S * d->C * sizeof(float);
  wgh::Launches hl;
  if (wgh::make_plans(d, variant, &hl)) return hl.plan[0].p.splits * dw_bytes;
  wg::Plan pl;
  if (!wg::make_plan(d, variant, &pl)) return 0;
  return pl.p.splits * dw_bytes;
}

}  // namespace mb
