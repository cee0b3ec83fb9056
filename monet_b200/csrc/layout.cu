// Layout conversion between the reference's NCHW activations and the NHWC
// (torch.channels_last) form the tensor-core convolutions consume, plus global
// average pooling forward/backward.
#include "common.cuh"

namespace mb {
namespace {

// Per image: transpose a [rows, cols] matrix into [cols, rows] through a padded
// 32x32 shared-memory tile; both the loads and the stores are coalesced.
__global__ void __launch_bounds__(256) transpose_batched(const float* __restrict__ x,
                                                         float* __restrict__ y, int rows,
                                                         int cols) {
  __shared__ float tile[32][33];
  const size_t img = static_cast<size_t>(blockIdx.z) * rows * cols;
  const int c0 = blockIdx.x * 32, r0 = blockIdx.y * 32;
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  for (int i = ty; i < 32; i += 8) {
    const int r = r0 + i, c = c0 + tx;
    if (r < rows && c < cols) tile[i][tx] = __ldg(x + img + static_cast<size_t>(r) * cols + c);
  }
  __syncthreads();
  for (int i = ty; i < 32; i += 8) {
    const int c = c0 + i, r = r0 + tx;
    if (r < rows && c < cols) y[img + static_cast<size_t>(c) * rows + r] = tile[tx][i];
  }
}

int transpose(const char* who, const float* x, float* y, int N, int rows, int cols, void* stream) {
  if (N < 0 || rows <= 0 || cols <= 0) return fail(MB_ERR_INVALID_ARGUMENT, "%s: bad extent", who);
  if (N == 0) return MB_OK;
  if (!x || !y) return fail(MB_ERR_INVALID_ARGUMENT, "%s: null pointer", who);
  if (N > 65535 || (rows + 31) / 32 > 65535)
    return fail(MB_ERR_UNSUPPORTED, "%s: extent exceeds the grid limits", who);
  dim3 grid((cols + 31) / 32, (rows + 31) / 32, N);
  transpose_batched<<<grid, 256, 0, as_stream(stream)>>>(x, y, rows, cols);
  return after_launch(who);
}

// NCHW -> NHWC with the channel count padded to Cp (zeros): one thread per pixel reads the
// C planes (coalesced across the warp) and writes Cp contiguous floats.  For the few-channel
// network input (C = 3 -> 4), which the tensor-core convolution needs 16-byte aligned.
__global__ void __launch_bounds__(256) nchw_to_nhwc_pad(const float* __restrict__ x,
                                                        float* __restrict__ y, int C, int Cp,
                                                        size_t HW, size_t total_pixels) {
  for (size_t t = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; t < total_pixels;
       t += static_cast<size_t>(gridDim.x) * blockDim.x) {
    const size_t n = t / HW, i = t - n * HW;
    const float* src = x + n * C * HW + i;
    float* dst = y + t * Cp;
    for (int c0 = 0; c0 < Cp; c0 += 4) {
      float4 v;
      v.x = (c0 + 0 < C) ? __ldg(src + (c0 + 0) * HW) : 0.f;
      v.y = (c0 + 1 < C) ? __ldg(src + (c0 + 1) * HW) : 0.f;
      v.z = (c0 + 2 < C) ? __ldg(src + (c0 + 2) * HW) : 0.f;
      v.w = (c0 + 3 < C) ? __ldg(src + (c0 + 3) * HW) : 0.f;
      *reinterpret_cast<float4*>(dst + c0) = v;
    }
  }
}

// NHWC global average pool: thread = (n, 4 channels), loop over HW rows.
__global__ void __launch_bounds__(256) gap_fwd_nhwc(const float* __restrict__ x,
                                                    float* __restrict__ y, int N, int C, int HW) {
  const int cg = C / 4;
  const int t = blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= N * cg) return;
  const int n = t / cg, g = t - n * cg;
  const float* p = x + static_cast<size_t>(n) * HW * C + g * 4;
  float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
  for (int i = 0; i < HW; ++i) {
    const float4 v = __ldg(reinterpret_cast<const float4*>(p + static_cast<size_t>(i) * C));
    s.x += v.x; s.y += v.y; s.z += v.z; s.w += v.w;
  }
  const float inv = 1.f / HW;
  *reinterpret_cast<float4*>(y + static_cast<size_t>(n) * C + g * 4) =
      make_float4(s.x * inv, s.y * inv, s.z * inv, s.w * inv);
}

// Generic: one warp per (n, c); element (n, c, i) at n*sn + c*sc + i*si.
__global__ void __launch_bounds__(256) gap_fwd_generic(const float* __restrict__ x,
                                                       float* __restrict__ y, int planes, int C,
                                                       int HW, size_t sn, size_t sc, size_t si) {
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  if (warp >= planes) return;
  const int n = warp / C, c = warp - n * C;
  const float* p = x + n * sn + c * sc;
  float s = 0.f;
  for (int i = lane; i < HW; i += 32) s += __ldg(p + i * si);
  s = warp_sum(s);
  if (lane == 0) y[warp] = s / HW;
}

__global__ void __launch_bounds__(256) gap_bwd(const float* __restrict__ dy, float* __restrict__ dx,
                                               size_t total, int C, int HW, int nhwc) {
  const float inv = 1.f / HW;
  for (size_t e = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; e < total;
       e += static_cast<size_t>(gridDim.x) * blockDim.x) {
    size_t plane;
    if (nhwc) {
      const size_t c = e % C, n = e / (static_cast<size_t>(C) * HW);
      plane = n * C + c;
    } else {
      plane = e / HW;
    }
    dx[e] = __ldg(dy + plane) * inv;
  }
}

// Concatenation along one axis, seen as a row copy: with everything before the axis folded
// into `rows` and everything from the axis on into a row, piece i is the column range
// [begin[i], begin[i+1]) of every row of the whole tensor.  One launch serves all pieces, in
// either direction (forward: pieces -> whole; backward: whole -> pieces, the split of the
// gradient).  V floats per thread per access.
struct CatPieces {
  float* ptr[MB_CAT_MAX_PIECES];
  int begin[MB_CAT_MAX_PIECES + 1];
  int n;
};

template <int V, bool kToPieces>
__global__ void __launch_bounds__(256) cat_rows(float* __restrict__ whole, CatPieces P,
                                                size_t rows, int width) {
  const size_t wv = static_cast<size_t>(width / V), total = rows * wv;
  for (size_t t = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; t < total;
       t += static_cast<size_t>(gridDim.x) * blockDim.x) {
    const size_t r = t / wv;
    const int c = static_cast<int>(t - r * wv) * V;
    int i = 0;
#pragma unroll
    for (int k = 1; k < MB_CAT_MAX_PIECES; ++k)
      if (k < P.n && c >= P.begin[k]) i = k;
    const int w = P.begin[i + 1] - P.begin[i];
    float* piece = P.ptr[i] + r * w + (c - P.begin[i]);
    float* big = whole + r * width + c;
    if (V == 4) {
      if (kToPieces) *reinterpret_cast<float4*>(piece) = __ldg(reinterpret_cast<const float4*>(big));
      else *reinterpret_cast<float4*>(big) = __ldg(reinterpret_cast<const float4*>(piece));
    } else {
      if (kToPieces) *piece = __ldg(big);
      else *big = __ldg(piece);
    }
  }
}

}  // namespace
}  // namespace mb

using namespace mb;

extern "C" {

int mb_nchw_to_nhwc(const float* x, float* y, int N, int C, int H, int W, void* stream) {
  if (H <= 0 || W <= 0) return fail(MB_ERR_INVALID_ARGUMENT, "mb_nchw_to_nhwc: bad extent");
  return transpose("mb_nchw_to_nhwc", x, y, N, C, H * W, stream);
}

int mb_nhwc_to_nchw(const float* x, float* y, int N, int C, int H, int W, void* stream) {
  if (H <= 0 || W <= 0) return fail(MB_ERR_INVALID_ARGUMENT, "mb_nhwc_to_nchw: bad extent");
  return transpose("mb_nhwc_to_nchw", x, y, N, H * W, C, stream);
}

int mb_nchw_to_nhwc_pad(const float* x, float* y, int N, int C, int H, int W, int Cp,
                        void* stream) {
  if (N < 0 || C <= 0 || H <= 0 || W <= 0 || Cp < C || Cp % 4)
    return fail(MB_ERR_INVALID_ARGUMENT, "mb_nchw_to_nhwc_pad: bad extent (Cp must be a multiple of 4, >= C)");
  if (N == 0) return MB_OK;
  if (!x || !y || !aligned(y, 16)) return fail(MB_ERR_INVALID_ARGUMENT, "mb_nchw_to_nhwc_pad: bad pointer");
  const size_t HW = static_cast<size_t>(H) * W, total = HW * N;
  nchw_to_nhwc_pad<<<grid_for(total, 256, 8), 256, 0, as_stream(stream)>>>(x, y, C, Cp, HW, total);
  return after_launch("nchw_to_nhwc_pad");
}

int mb_cat_rows(float* whole, float* const* pieces, const int* widths, int n_pieces, size_t rows,
                int to_pieces, void* stream) {
  if (n_pieces < 1 || n_pieces > MB_CAT_MAX_PIECES || !pieces || !widths)
    return fail(MB_ERR_INVALID_ARGUMENT, "mb_cat_rows: 1..%d pieces", MB_CAT_MAX_PIECES);
  CatPieces P;
  P.n = n_pieces;
  P.begin[0] = 0;
  bool vec = aligned(whole, 16);
  for (int i = 0; i < n_pieces; ++i) {
    if (widths[i] <= 0) return fail(MB_ERR_INVALID_ARGUMENT, "mb_cat_rows: empty piece %d", i);
    if (rows && !pieces[i]) return fail(MB_ERR_INVALID_ARGUMENT, "mb_cat_rows: null piece %d", i);
    P.ptr[i] = pieces[i];
    P.begin[i + 1] = P.begin[i] + widths[i];
    vec = vec && widths[i] % 4 == 0 && aligned(pieces[i], 16);
  }
  for (int i = n_pieces; i < MB_CAT_MAX_PIECES; ++i) { P.ptr[i] = nullptr; P.begin[i + 1] = P.begin[n_pieces]; }
  if (rows == 0) return MB_OK;
  if (!whole) return fail(MB_ERR_INVALID_ARGUMENT, "mb_cat_rows: null pointer");
  const int width = P.begin[n_pieces];
  cudaStream_t st = as_stream(stream);
  const size_t items = rows * static_cast<size_t>(vec ? width / 4 : width);
  const int grid = grid_for(items, 256, 8);
  if (vec) {
    if (to_pieces) cat_rows<4, true><<<grid, 256, 0, st>>>(whole, P, rows, width);
    else cat_rows<4, false><<<grid, 256, 0, st>>>(whole, P, rows, width);
  } else {
    if (to_pieces) cat_rows<1, true><<<grid, 256, 0, st>>>(whole, P, rows, width);
    else cat_rows<1, false><<<grid, 256, 0, st>>>(whole, P, rows, width);
  }
  return after_launch("cat_rows");
}

int mb_global_avgpool_fwd(const float* x, float* y, int N, int C, int HW, int layout,
                          void* stream) {
  if (N < 0 || C <= 0 || HW <= 0) return fail(MB_ERR_INVALID_ARGUMENT, "mb_global_avgpool_fwd: bad extent");
  if (N == 0) return MB_OK;
  if (!x || !y) return fail(MB_ERR_INVALID_ARGUMENT, "mb_global_avgpool_fwd: null pointer");
  cudaStream_t st = as_stream(stream);
  if (layout == MB_NHWC && C % 4 == 0 && aligned(x, 16) && aligned(y, 16)) {
    const int threads = N * (C / 4);
    gap_fwd_nhwc<<<(threads + 255) / 256, 256, 0, st>>>(x, y, N, C, HW);
    return after_launch("gap_fwd_nhwc");
  }
  const int planes = N * C;
  const size_t sn = static_cast<size_t>(C) * HW;
  if (layout == MB_NHWC)
    gap_fwd_generic<<<(planes + 7) / 8, 256, 0, st>>>(x, y, planes, C, HW, sn, 1, C);
  else
    gap_fwd_generic<<<(planes + 7) / 8, 256, 0, st>>>(x, y, planes, C, HW, sn, HW, 1);
  return after_launch("gap_fwd_generic");
}

int mb_global_avgpool_bwd(const float* dy, float* dx, int N, int C, int HW, int layout,
                          void* stream) {
  if (N < 0 || C <= 0 || HW <= 0) return fail(MB_ERR_INVALID_ARGUMENT, "mb_global_avgpool_bwd: bad extent");
  if (N == 0) return MB_OK;
  if (!dy || !dx) return fail(MB_ERR_INVALID_ARGUMENT, "mb_global_avgpool_bwd: null pointer");
  const size_t total = static_cast<size_t>(N) * C * HW;
  gap_bwd<<<grid_for(total, 256, 8), 256, 0, as_stream(stream)>>>(dy, dx, total, C, HW, layout == MB_NHWC);
  return after_launch("gap_bwd");
}

}  // extern "C"
