// Depthwise convolution (groups == C, one filter per channel; MobileNetV2's 3x3 layers),
// NHWC, fp32 FMA.  These layers move 8 bytes per output element for ~18 flops, so they are
// HBM-bound and run as vectorised SIMT kernels rather than on the tensor cores:
//   forward        thread = output pixel x 4 channels, R*S float4 taps
//   backward-data  thread = input pixel x 4 channels, gathers the taps that reach it
//   backward-filter per-channel reduction over all pixels: each CTA accumulates its share of
//                  rows in registers, combines over its row lanes in shared memory and adds
//                  the result to dw with atomics (dw zeroed first)
// Filters are given as [R*S][C] (channel innermost).  Replaces the ATen depthwise kernels
// the reference defers to (conv.cpp:704-726).
#include "common.cuh"

namespace mb {
namespace {

struct DwP {
  int N, C, H, W, P, Q, R, S, sh, sw, ph, pw, dh, dw;
};

constexpr int kMaxDwTaps = 25;

__global__ void __launch_bounds__(256) dw_fprop(const float* __restrict__ x, const float* __restrict__ w,
                                                const float* __restrict__ bias, float* __restrict__ y,
                                                DwP p, size_t total) {
  const int cg = p.C / 4;
  for (size_t t = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; t < total;
       t += static_cast<size_t>(gridDim.x) * blockDim.x) {
    const int g = static_cast<int>(t % cg);
    size_t pix = t / cg;
    const int q = static_cast<int>(pix % p.Q);
    pix /= p.Q;
    const int pp = static_cast<int>(pix % p.P);
    const int n = static_cast<int>(pix / p.P);
    float4 acc = bias ? __ldg(reinterpret_cast<const float4*>(bias) + g) : make_float4(0.f, 0.f, 0.f, 0.f);
    const float* xn = x + static_cast<size_t>(n) * p.H * p.W * p.C + g * 4;
    for (int r = 0; r < p.R; ++r) {
      const int h = pp * p.sh - p.ph + r * p.dh;
      if (h < 0 || h >= p.H) continue;
      for (int s = 0; s < p.S; ++s) {
        const int ww = q * p.sw - p.pw + s * p.dw;
        if (ww < 0 || ww >= p.W) continue;
        const float4 a = __ldg(reinterpret_cast<const float4*>(xn + (static_cast<size_t>(h) * p.W + ww) * p.C));
        const float4 f = __ldg(reinterpret_cast<const float4*>(w + static_cast<size_t>(r * p.S + s) * p.C) + g);
        acc.x = fmaf(a.x, f.x, acc.x); acc.y = fmaf(a.y, f.y, acc.y);
        acc.z = fmaf(a.z, f.z, acc.z); acc.w = fmaf(a.w, f.w, acc.w);
      }
    }
    reinterpret_cast<float4*>(y)[t] = acc;
  }
}

__global__ void __launch_bounds__(256) dw_dgrad(const float* __restrict__ dy, const float* __restrict__ w,
                                                float* __restrict__ dx, DwP p, size_t total) {
  const int cg = p.C / 4;
  for (size_t t = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; t < total;
       t += static_cast<size_t>(gridDim.x) * blockDim.x) {
    const int g = static_cast<int>(t % cg);
    size_t pix = t / cg;
    const int ww = static_cast<int>(pix % p.W);
    pix /= p.W;
    const int h = static_cast<int>(pix % p.H);
    const int n = static_cast<int>(pix / p.H);
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    const float* dn = dy + static_cast<size_t>(n) * p.P * p.Q * p.C + g * 4;
    for (int r = 0; r < p.R; ++r) {
      const int hn = h + p.ph - r * p.dh;
      if (hn < 0 || hn % p.sh) continue;
      const int pp = hn / p.sh;
      if (pp >= p.P) continue;
      for (int s = 0; s < p.S; ++s) {
        const int wn = ww + p.pw - s * p.dw;
        if (wn < 0 || wn % p.sw) continue;
        const int q = wn / p.sw;
        if (q >= p.Q) continue;
        const float4 a = __ldg(reinterpret_cast<const float4*>(dn + (static_cast<size_t>(pp) * p.Q + q) * p.C));
        const float4 f = __ldg(reinterpret_cast<const float4*>(w + static_cast<size_t>(r * p.S + s) * p.C) + g);
        acc.x = fmaf(a.x, f.x, acc.x); acc.y = fmaf(a.y, f.y, acc.y);
        acc.z = fmaf(a.z, f.z, acc.z); acc.w = fmaf(a.w, f.w, acc.w);
      }
    }
    reinterpret_cast<float4*>(dx)[t] = acc;
  }
}


// ---------------------------------------------------------------- 3x3 specialisations
// MobileNetV2's depthwise layers are all 3x3, dilation 1, stride 1 or 2.  With the filter
// shape and the stride fixed at compile time the tap loops unroll, the divisions by the
// stride disappear, and one thread produces kTw consecutive output pixels of a row: the
// 3 x ((kTw-1)*STRIDE + 3) input columns it needs are loaded once and shared by its outputs
// (4.5 instead of 9 loads per output at stride 1).  A warp still walks the channel groups
// first, so every load instruction covers contiguous runs of 4*32 channels.
constexpr int kTw = 4;
constexpr unsigned kRowBlock = 8;

__device__ __forceinline__ void fma4(float4& acc, const float4& a, const float4& f) {
  acc.x = fmaf(a.x, f.x, acc.x); acc.y = fmaf(a.y, f.y, acc.y);
  acc.z = fmaf(a.z, f.z, acc.z); acc.w = fmaf(a.w, f.w, acc.w);
}

// y[n][pp][q] = sum_{r,s} x[n][pp*STRIDE - ph + r][q*STRIDE - pw + s] * f[r][s]   (FLIP: f[2-r][2-s])
// `p.H, p.W` are the extents of the tensor read, `p.P, p.Q` of the tensor written, so the same
// kernel is the stride-1 backward-data pass when it reads dy with the flipped filter and the
// padding 2 - pad.
template <int STRIDE, bool FLIP>
__global__ void __launch_bounds__(256, 3) dw3x3_tiled(const float* __restrict__ x, const float* __restrict__ w,
                                                   const float* __restrict__ bias, float* __restrict__ y,
                                                   DwP p, int qtiles, size_t total) {
  constexpr int kCols = (kTw - 1) * STRIDE + 3;
  const int cg = p.C / 4;
  // 32-bit index arithmetic (the host sends larger problems to the generic kernel): the three
  // 64-bit divisions per work item of the first version were a quarter of its instructions,
  // and the kernel is bound by instruction issue, not by memory (ncu: ALU pipe 62 %, issue
  // slots 67 % busy, DRAM 40 %)
  const unsigned total32 = static_cast<unsigned>(total), ucg = static_cast<unsigned>(cg),
                 uqt = static_cast<unsigned>(qtiles), uP = static_cast<unsigned>(p.P);
  // Work items are ordered channel group, then kRowBlock output rows, then column tile: the
  // threads of a CTA then hold vertically adjacent tiles, whose windows share two of their three
  // input rows, at the same time, so that L1 can serve the overlap (in row-major order the rows
  // of a window were fetched by three different SMs and L2 delivered 3.3x the input).  Worth
  // 5 % at stride 2, nothing measurable at stride 1.
  const unsigned uPB = (uP + kRowBlock - 1) / kRowBlock;
  for (unsigned t = blockIdx.x * blockDim.x + threadIdx.x; t < total32; t += gridDim.x * blockDim.x) {
    const unsigned r1 = t / ucg;
    const int g = static_cast<int>(t - r1 * ucg);
    const unsigned r2 = r1 / kRowBlock, rl = r1 - r2 * kRowBlock;
    const unsigned r3 = r2 / uqt;
    const int qt = static_cast<int>(r2 - r3 * uqt);
    const unsigned n_u = r3 / uPB;
    const int pp = static_cast<int>((r3 - n_u * uPB) * kRowBlock + rl);
    if (pp >= p.P) continue;                    // the last row block of a map may be ragged
    const int n = static_cast<int>(n_u);
    const int q0 = qt * kTw;
    float4 f[9];
#pragma unroll
    for (int i = 0; i < 9; ++i)
      f[i] = __ldg(reinterpret_cast<const float4*>(w + static_cast<size_t>(FLIP ? 8 - i : i) * p.C) + g);
    float4 acc[kTw];
    const float4 b0 = bias ? __ldg(reinterpret_cast<const float4*>(bias) + g) : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int j = 0; j < kTw; ++j) acc[j] = b0;
    const float* xn = x + static_cast<size_t>(n) * p.H * p.W * p.C + g * 4;
    const int w0 = q0 * STRIDE - p.pw;
    const int h0 = pp * STRIDE - p.ph;
    if (h0 >= 0 && h0 + 2 < p.H && w0 >= 0 && w0 + kCols <= p.W) {
      // the whole 3 x kCols window lies inside the map (most tiles): no bounds tests, no zero
      // fill, one base pointer and two strides
      const float4* xb = reinterpret_cast<const float4*>(xn + (static_cast<size_t>(h0) * p.W + w0) * p.C);
      const size_t rstep = static_cast<size_t>(p.W) * cg;
#pragma unroll
      for (int r = 0; r < 3; ++r) {
        float4 col[kCols];
#pragma unroll
        for (int c = 0; c < kCols; ++c) col[c] = __ldg(xb + r * rstep + static_cast<size_t>(c) * cg);
#pragma unroll
        for (int j = 0; j < kTw; ++j)
#pragma unroll
          for (int sidx = 0; sidx < 3; ++sidx) fma4(acc[j], col[j * STRIDE + sidx], f[r * 3 + sidx]);
      }
    } else
#pragma unroll
    for (int r = 0; r < 3; ++r) {
      const int h = h0 + r;
      if (h < 0 || h >= p.H) continue;
      const float* xr = xn + static_cast<size_t>(h) * p.W * p.C;
      float4 col[kCols];
#pragma unroll
      for (int c = 0; c < kCols; ++c) {
        const int ww = w0 + c;
        col[c] = (ww >= 0 && ww < p.W) ? __ldg(reinterpret_cast<const float4*>(xr + static_cast<size_t>(ww) * p.C))
                                       : make_float4(0.f, 0.f, 0.f, 0.f);
      }
#pragma unroll
      for (int j = 0; j < kTw; ++j)
#pragma unroll
        for (int sidx = 0; sidx < 3; ++sidx) fma4(acc[j], col[j * STRIDE + sidx], f[r * 3 + sidx]);
    }
    float4* yo = reinterpret_cast<float4*>(y + ((static_cast<size_t>(n) * p.P + pp) * p.Q + q0) * p.C) + g;
#pragma unroll
    for (int j = 0; j < kTw; ++j)
      if (q0 + j < p.Q) yo[static_cast<size_t>(j) * cg] = acc[j];
  }
}

// Stride-2 backward-data, 3x3: thread = input pixel x 4 channels; only the taps whose parity
// matches reach an output pixel (2.25 of 9 on average), selected without divisions.
__global__ void __launch_bounds__(256) dw3x3s2_dgrad(const float* __restrict__ dy, const float* __restrict__ w,
                                                     float* __restrict__ dx, DwP p, size_t total) {
  const int cg = p.C / 4;
  const unsigned total32 = static_cast<unsigned>(total), ucg = static_cast<unsigned>(cg),
                 uW = static_cast<unsigned>(p.W), uH = static_cast<unsigned>(p.H);
  for (unsigned t = blockIdx.x * blockDim.x + threadIdx.x; t < total32; t += gridDim.x * blockDim.x) {
    const unsigned r1 = t / ucg;
    const int g = static_cast<int>(t - r1 * ucg);
    const unsigned r2 = r1 / uW;
    const int ww = static_cast<int>(r1 - r2 * uW);
    const unsigned n_u = r2 / uH;
    const int h = static_cast<int>(r2 - n_u * uH);
    const int n = static_cast<int>(n_u);
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    const float* dn = dy + static_cast<size_t>(n) * p.P * p.Q * p.C + g * 4;
#pragma unroll
    for (int r = 0; r < 3; ++r) {
      const int hn = h + p.ph - r;
      if (hn < 0 || (hn & 1)) continue;
      const int pp = hn >> 1;
      if (pp >= p.P) continue;
#pragma unroll
      for (int sidx = 0; sidx < 3; ++sidx) {
        const int wn = ww + p.pw - sidx;
        if (wn < 0 || (wn & 1)) continue;
        const int q = wn >> 1;
        if (q >= p.Q) continue;
        const float4 a = __ldg(reinterpret_cast<const float4*>(dn + (static_cast<size_t>(pp) * p.Q + q) * p.C));
        const float4 f = __ldg(reinterpret_cast<const float4*>(w + static_cast<size_t>(r * 3 + sidx) * p.C) + g);
        fma4(acc, a, f);
      }
    }
    reinterpret_cast<float4*>(dx)[t] = acc;
  }
}

// Stride-2 backward-data, 3x3, padding 1 (every stride-2 depthwise layer of MobileNetV2): a thread
// owns a 2x2 input quad x 4 channels.  With h = 2p - 1 + r the even input rows are reached by
// r = 1 only (p = a) and the odd ones by r = 2 (p = a) and r = 0 (p = a + 1), likewise for the
// columns, so the quad (rows 2a, 2a+1; columns 2b, 2b+1) needs exactly the four output pixels
// (a..a+1, b..b+1): four gradient loads, nine FMAs and four stores with no parity tests, where
// the per-pixel kernel above spends most of its instructions on them (0.80 -> 0.31 ms on
// 272 x 96 x 112 x 112, 0.83 of the HBM copy rate).
__global__ void __launch_bounds__(256) dw3x3s2p1_dgrad_quad(const float* __restrict__ dy,
                                                            const float* __restrict__ w,
                                                            float* __restrict__ dx, DwP p, unsigned total) {
  const unsigned cg = p.C / 4, H2 = (p.H + 1) / 2, W2 = (p.W + 1) / 2;
  for (unsigned t = blockIdx.x * blockDim.x + threadIdx.x; t < total; t += gridDim.x * blockDim.x) {
    const unsigned r1 = t / cg, g = t - r1 * cg;
    const unsigned r2 = r1 / W2, b = r1 - r2 * W2;
    const unsigned n = r2 / H2, a = r2 - n * H2;
    float4 f[9];
#pragma unroll
    for (int i = 0; i < 9; ++i) f[i] = __ldg(reinterpret_cast<const float4*>(w + static_cast<size_t>(i) * p.C) + g);
    const float4* dn = reinterpret_cast<const float4*>(dy + static_cast<size_t>(n) * p.P * p.Q * p.C) + g;
    const float4 z = make_float4(0.f, 0.f, 0.f, 0.f);
    const bool a1 = a + 1 < static_cast<unsigned>(p.P), b1 = b + 1 < static_cast<unsigned>(p.Q);
    const size_t o00 = (static_cast<size_t>(a) * p.Q + b) * cg;
    const float4 d00 = __ldg(dn + o00);
    const float4 d01 = b1 ? __ldg(dn + o00 + cg) : z;
    const float4 d10 = a1 ? __ldg(dn + o00 + static_cast<size_t>(p.Q) * cg) : z;
    const float4 d11 = (a1 && b1) ? __ldg(dn + o00 + static_cast<size_t>(p.Q) * cg + cg) : z;
    float4 x00 = z, x01 = z, x10 = z, x11 = z;
    fma4(x00, d00, f[4]);
    fma4(x01, d00, f[5]); fma4(x01, d01, f[3]);
    fma4(x10, d00, f[7]); fma4(x10, d10, f[1]);
    fma4(x11, d00, f[8]); fma4(x11, d01, f[6]); fma4(x11, d10, f[2]); fma4(x11, d11, f[0]);
    const unsigned h = 2 * a, ww = 2 * b;
    float4* out = reinterpret_cast<float4*>(dx) + ((static_cast<size_t>(n) * p.H + h) * p.W + ww) * cg + g;
    const bool w1 = ww + 1 < static_cast<unsigned>(p.W);
    out[0] = x00;
    if (w1) out[cg] = x01;
    if (h + 1 < static_cast<unsigned>(p.H)) {
      out[static_cast<size_t>(p.W) * cg] = x10;
      if (w1) out[static_cast<size_t>(p.W) * cg + cg] = x11;
    }
  }
}

// block = (tx channel groups of 4) x (ty row lanes); grid = (row chunks, channel slabs).
// A "row" is one output pixel.  TAPS = R*S is a template parameter so that the per-tap
// accumulators live in registers.
template <int TAPS, int SW>
__global__ void __launch_bounds__(256) dw_wgrad(const float* __restrict__ x, const float* __restrict__ dy,
                                                float* __restrict__ dwt, float* __restrict__ db, DwP p,
                                                size_t pixels, int chunks, int tx_n, int ty_n) {
  extern __shared__ float sm[];   // [ty_n][tx_n][4]
  const int tx = threadIdx.x % tx_n, ty = threadIdx.x / tx_n;
  const int g = blockIdx.y * tx_n + tx;
  const bool live = g * 4 < p.C;
  float4 acc[TAPS];
  float4 accb = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
  for (int t = 0; t < TAPS; ++t) acc[t] = make_float4(0.f, 0.f, 0.f, 0.f);
  if (live) {
    const size_t per = (pixels + chunks - 1) / chunks;
    const size_t r0 = static_cast<size_t>(blockIdx.x) * per;
    const size_t r1 = (r0 + per) < pixels ? (r0 + per) : pixels;
    for (size_t row = r0 + ty; row < r1; row += ty_n) {
      const int q = static_cast<int>(row % p.Q);
      size_t rr = row / p.Q;
      const int pp = static_cast<int>(rr % p.P);
      const int n = static_cast<int>(rr / p.P);
      const float4 d = __ldg(reinterpret_cast<const float4*>(dy + row * p.C) + g);
      accb.x += d.x; accb.y += d.y; accb.z += d.z; accb.w += d.w;
      const float* xn = x + static_cast<size_t>(n) * p.H * p.W * p.C + g * 4;
#pragma unroll
      for (int t = 0; t < TAPS; ++t) {
        const int r = t / SW, s = t - r * SW;        // SW = filter width, compile time
        const int h = pp * p.sh - p.ph + r * p.dh, ww = q * p.sw - p.pw + s * p.dw;
        if (h < 0 || h >= p.H || ww < 0 || ww >= p.W) continue;
        const float4 a = __ldg(reinterpret_cast<const float4*>(xn + (static_cast<size_t>(h) * p.W + ww) * p.C));
        acc[t].x = fmaf(a.x, d.x, acc[t].x); acc[t].y = fmaf(a.y, d.y, acc[t].y);
        acc[t].z = fmaf(a.z, d.z, acc[t].z); acc[t].w = fmaf(a.w, d.w, acc[t].w);
      }
    }
  }
  // combine the row lanes of each channel group, one tap at a time (unrolled: a dynamic index
  // would push the accumulators out of registers into local memory)
  float4* mine = reinterpret_cast<float4*>(sm) + ty * tx_n + tx;
#pragma unroll
  for (int t = 0; t <= TAPS; ++t) {
    *mine = t < TAPS ? acc[t] : accb;
    __syncthreads();
    if (ty == 0 && live && (t < TAPS || db)) {
      float4 s = *mine;
      for (int j = 1; j < ty_n; ++j) {
        const float4 o = reinterpret_cast<float4*>(sm)[j * tx_n + tx];
        s.x += o.x; s.y += o.y; s.z += o.z; s.w += o.w;
      }
      float* dst = t < TAPS ? dwt + static_cast<size_t>(t) * p.C + g * 4 : db + g * 4;
      atomicAdd(dst + 0, s.x); atomicAdd(dst + 1, s.y); atomicAdd(dst + 2, s.z); atomicAdd(dst + 3, s.w);
    }
    __syncthreads();
  }
}


// 3x3 backward-filter with the same row tiling: a lane takes kTw consecutive output pixels of a
// row, loads their dy values and the 3 x ((kTw-1)*STRIDE + 3) input columns once, and updates the
// nine per-tap accumulators for all of them (5.5 instead of 10 loads per pixel at stride 1).
template <int STRIDE>
__global__ void __launch_bounds__(256) dw3x3_wgrad(const float* __restrict__ x, const float* __restrict__ dy,
                                                   float* __restrict__ dwt, float* __restrict__ db, DwP p,
                                                   int qtiles, size_t tiles, int chunks, int tx_n, int ty_n) {
  constexpr int kCols = (kTw - 1) * STRIDE + 3;
  extern __shared__ float sm[];   // [ty_n][tx_n][4]
  const int tx = threadIdx.x % tx_n, ty = threadIdx.x / tx_n;
  const int g = blockIdx.y * tx_n + tx;
  const bool live = g * 4 < p.C;
  float4 acc[9];
  float4 accb = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
  for (int t = 0; t < 9; ++t) acc[t] = make_float4(0.f, 0.f, 0.f, 0.f);
  if (live) {
    const size_t per = (tiles + chunks - 1) / chunks;
    const size_t t0 = static_cast<size_t>(blockIdx.x) * per;
    const size_t t1 = (t0 + per) < tiles ? (t0 + per) : tiles;
    for (size_t tile = t0 + ty; tile < t1; tile += ty_n) {
      const unsigned ut = static_cast<unsigned>(tile);        // the host checks tiles < 2^31
      const unsigned r1 = ut / static_cast<unsigned>(qtiles);
      const int qt = static_cast<int>(ut - r1 * static_cast<unsigned>(qtiles));
      const unsigned n_u = r1 / static_cast<unsigned>(p.P);
      const int pp = static_cast<int>(r1 - n_u * static_cast<unsigned>(p.P));
      const int n = static_cast<int>(n_u);
      const int q0 = qt * kTw;
      float4 d[kTw];
      const float4* dr = reinterpret_cast<const float4*>(dy + ((static_cast<size_t>(n) * p.P + pp) * p.Q + q0) * p.C) + g;
      const int cgs = p.C / 4;
      const float* xn = x + static_cast<size_t>(n) * p.H * p.W * p.C + g * 4;
      const int w0 = q0 * STRIDE - p.pw;
      const int h0 = pp * STRIDE - p.ph;
      if (q0 + kTw <= p.Q && h0 >= 0 && h0 + 2 < p.H && w0 >= 0 && w0 + kCols <= p.W) {
        // the tile and its 3 x kCols window lie inside the maps (most tiles): no bounds tests
#pragma unroll
        for (int j = 0; j < kTw; ++j) {
          d[j] = __ldg(dr + static_cast<size_t>(j) * cgs);
          accb.x += d[j].x; accb.y += d[j].y; accb.z += d[j].z; accb.w += d[j].w;
        }
        const float4* xb = reinterpret_cast<const float4*>(xn + (static_cast<size_t>(h0) * p.W + w0) * p.C);
        const size_t rstep = static_cast<size_t>(p.W) * cgs;
#pragma unroll
        for (int r = 0; r < 3; ++r) {
          float4 col[kCols];
#pragma unroll
          for (int c = 0; c < kCols; ++c) col[c] = __ldg(xb + r * rstep + static_cast<size_t>(c) * cgs);
#pragma unroll
          for (int j = 0; j < kTw; ++j)
#pragma unroll
            for (int sidx = 0; sidx < 3; ++sidx) fma4(acc[r * 3 + sidx], col[j * STRIDE + sidx], d[j]);
        }
        continue;
      }
#pragma unroll
      for (int j = 0; j < kTw; ++j) {
        d[j] = (q0 + j < p.Q) ? __ldg(dr + static_cast<size_t>(j) * cgs) : make_float4(0.f, 0.f, 0.f, 0.f);
        accb.x += d[j].x; accb.y += d[j].y; accb.z += d[j].z; accb.w += d[j].w;
      }
#pragma unroll
      for (int r = 0; r < 3; ++r) {
        const int h = h0 + r;
        if (h < 0 || h >= p.H) continue;
        const float* xr = xn + static_cast<size_t>(h) * p.W * p.C;
        float4 col[kCols];
#pragma unroll
        for (int c = 0; c < kCols; ++c) {
          const int ww = w0 + c;
          col[c] = (ww >= 0 && ww < p.W) ? __ldg(reinterpret_cast<const float4*>(xr + static_cast<size_t>(ww) * p.C))
                                         : make_float4(0.f, 0.f, 0.f, 0.f);
        }
#pragma unroll
        for (int j = 0; j < kTw; ++j)
#pragma unroll
          for (int sidx = 0; sidx < 3; ++sidx) fma4(acc[r * 3 + sidx], col[j * STRIDE + sidx], d[j]);
      }
    }
  }
  // combine the row lanes of each channel group, one tap at a time (unrolled: a dynamic index
  // would push the accumulators out of registers into local memory)
  float4* mine = reinterpret_cast<float4*>(sm) + ty * tx_n + tx;
#pragma unroll
  for (int t = 0; t <= 9; ++t) {
    *mine = t < 9 ? acc[t] : accb;
    __syncthreads();
    if (ty == 0 && live && (t < 9 || db)) {
      float4 sum = *mine;
      for (int j = 1; j < ty_n; ++j) {
        const float4 o = reinterpret_cast<float4*>(sm)[j * tx_n + tx];
        sum.x += o.x; sum.y += o.y; sum.z += o.z; sum.w += o.w;
      }
      float* dst = t < 9 ? dwt + static_cast<size_t>(t) * p.C + g * 4 : db + g * 4;
      atomicAdd(dst + 0, sum.x); atomicAdd(dst + 1, sum.y); atomicAdd(dst + 2, sum.z); atomicAdd(dst + 3, sum.w);
    }
    __syncthreads();
  }
}

int check(const char* who, const mb_conv_desc* d, DwP* p) {
  if (!d) return fail(MB_ERR_INVALID_ARGUMENT, "%s: null descriptor", who);
  if (d->groups != d->C || d->K != d->C)
    return fail(MB_ERR_UNSUPPORTED, "%s: only groups == C == K (one filter per channel)", who);
  if (d->C % 4) return fail(MB_ERR_UNSUPPORTED, "%s: C=%d must be a multiple of 4", who, d->C);
  if (d->R * d->S > kMaxDwTaps) return fail(MB_ERR_UNSUPPORTED, "%s: more than %d taps", who, kMaxDwTaps);
  const int P = (d->H + 2 * d->pad_h - d->dil_h * (d->R - 1) - 1) / d->stride_h + 1;
  const int Q = (d->W + 2 * d->pad_w - d->dil_w * (d->S - 1) - 1) / d->stride_w + 1;
  if (P != d->P || Q != d->Q || P <= 0 || Q <= 0)
    return fail(MB_ERR_INVALID_ARGUMENT, "%s: output extent does not match the geometry", who);
  *p = DwP{d->N, d->C, d->H, d->W, d->P, d->Q, d->R, d->S, d->stride_h, d->stride_w, d->pad_h,
           d->pad_w, d->dil_h, d->dil_w};
  return MB_OK;
}

}  // namespace
}  // namespace mb

using namespace mb;

extern "C" {

int mb_depthwise_fprop(const float* x, const float* w_tc, const float* bias, float* y,
                       const mb_conv_desc* d, void* stream) {
  DwP p;
  int rc = check("mb_depthwise_fprop", d, &p);
  if (rc) return rc;
  if (!x || !w_tc || !y || !aligned(x, 16) || !aligned(w_tc, 16) || !aligned(y, 16) || !aligned(bias, 16))
    return fail(MB_ERR_INVALID_ARGUMENT, "mb_depthwise_fprop: null or misaligned pointer");
  if (p.R == 3 && p.S == 3 && p.dh == 1 && p.dw == 1 && p.sh == p.sw && (p.sh == 1 || p.sh == 2) &&
      static_cast<size_t>(p.N) * (p.P + kRowBlock) * ((p.Q + kTw - 1) / kTw) * (p.C / 4) < 0x7fffffffull) {
    const int qtiles = (p.Q + kTw - 1) / kTw;
    const size_t total = static_cast<size_t>(p.N) * ((p.P + kRowBlock - 1) / kRowBlock * kRowBlock) * qtiles * (p.C / 4);
    const int grid = grid_for(total, 256, 8);
    if (p.sh == 1)
      dw3x3_tiled<1, false><<<grid, 256, 0, as_stream(stream)>>>(x, w_tc, bias, y, p, qtiles, total);
    else
      dw3x3_tiled<2, false><<<grid, 256, 0, as_stream(stream)>>>(x, w_tc, bias, y, p, qtiles, total);
    return after_launch("depthwise_fprop_3x3");
  }
  const size_t total = static_cast<size_t>(p.N) * p.P * p.Q * (p.C / 4);
  dw_fprop<<<grid_for(total, 256, 8), 256, 0, as_stream(stream)>>>(x, w_tc, bias, y, p, total);
  return after_launch("depthwise_fprop");
}

int mb_depthwise_dgrad(const float* dy, const float* w_tc, float* dx, const mb_conv_desc* d,
                       void* stream) {
  DwP p;
  int rc = check("mb_depthwise_dgrad", d, &p);
  if (rc) return rc;
  if (!dy || !w_tc || !dx || !aligned(dy, 16) || !aligned(w_tc, 16) || !aligned(dx, 16))
    return fail(MB_ERR_INVALID_ARGUMENT, "mb_depthwise_dgrad: null or misaligned pointer");
  if (p.R == 3 && p.S == 3 && p.dh == 1 && p.dw == 1 && p.sh == 1 && p.sw == 1 && p.ph <= 2 && p.pw <= 2 &&
      static_cast<size_t>(p.N) * (p.H + kRowBlock) * ((p.W + kTw - 1) / kTw) * (p.C / 4) < 0x7fffffffull) {
    // stride 1: a forward pass over dy with the flipped filter and padding 2 - pad
    DwP b = p;
    b.H = p.P; b.W = p.Q; b.P = p.H; b.Q = p.W;
    b.ph = 2 - p.ph; b.pw = 2 - p.pw;
    const int qtiles = (b.Q + kTw - 1) / kTw;
    const size_t total = static_cast<size_t>(b.N) * ((b.P + kRowBlock - 1) / kRowBlock * kRowBlock) * qtiles * (b.C / 4);
    dw3x3_tiled<1, true><<<grid_for(total, 256, 8), 256, 0, as_stream(stream)>>>(dy, w_tc, nullptr, dx, b,
                                                                                 qtiles, total);
    return after_launch("depthwise_dgrad_3x3");
  }
  const size_t total = static_cast<size_t>(p.N) * p.H * p.W * (p.C / 4);
  if (p.R == 3 && p.S == 3 && p.dh == 1 && p.dw == 1 && p.sh == 2 && p.sw == 2 && p.ph == 1 && p.pw == 1 &&
      total < 0x7fffffffull) {
    const size_t quads = static_cast<size_t>(p.N) * ((p.H + 1) / 2) * ((p.W + 1) / 2) * (p.C / 4);
    dw3x3s2p1_dgrad_quad<<<grid_for(quads, 256, 8), 256, 0, as_stream(stream)>>>(dy, w_tc, dx, p,
                                                                               static_cast<unsigned>(quads));
    return after_launch("depthwise_dgrad_3x3s2_quad");
  }
  if (p.R == 3 && p.S == 3 && p.dh == 1 && p.dw == 1 && p.sh == 2 && p.sw == 2 && total < 0x7fffffffull) {
    dw3x3s2_dgrad<<<grid_for(total, 256, 8), 256, 0, as_stream(stream)>>>(dy, w_tc, dx, p, total);
    return after_launch("depthwise_dgrad_3x3s2");
  }
  dw_dgrad<<<grid_for(total, 256, 8), 256, 0, as_stream(stream)>>>(dy, w_tc, dx, p, total);
  return after_launch("depthwise_dgrad");
}

int mb_depthwise_wgrad(const float* x, const float* dy, float* dw_tc, float* dbias,
                       const mb_conv_desc* d, void* stream) {
  const char* who = "mb_depthwise_wgrad";
  DwP p;
  int rc = check(who, d, &p);
  if (rc) return rc;
  if (!x || !dy || !dw_tc || !aligned(x, 16) || !aligned(dy, 16))
    return fail(MB_ERR_INVALID_ARGUMENT, "%s: null or misaligned pointer", who);
  cudaStream_t st = as_stream(stream);
  const int taps = p.R * p.S;
  if (p.R != p.S) return fail(MB_ERR_UNSUPPORTED, "%s: square filters only", who);
  if (cudaMemsetAsync(dw_tc, 0, static_cast<size_t>(taps) * p.C * sizeof(float), st) != cudaSuccess ||
      (dbias && cudaMemsetAsync(dbias, 0, static_cast<size_t>(p.C) * sizeof(float), st) != cudaSuccess))
    return fail(MB_ERR_LAUNCH, "%s: memset failed", who);
  const int groups = p.C / 4;
  int tx = 1;
  while (tx < groups && tx < 64) tx <<= 1;
  const int ty = 256 / tx;
  const int slabs = (groups + tx - 1) / tx;
  const size_t pixels = static_cast<size_t>(p.N) * p.P * p.Q;
  int chunks = static_cast<int>((pixels + ty * 8 - 1) / (static_cast<size_t>(ty) * 8));
  const int cap = num_sms() * 4 / slabs > 0 ? num_sms() * 4 / slabs : 1;
  if (chunks > cap) chunks = cap;
  if (chunks < 1) chunks = 1;
  const size_t smem = 256 * sizeof(float4);
  if (taps == 9 && p.dh == 1 && p.dw == 1 && p.sh == p.sw && (p.sh == 1 || p.sh == 2) &&
      static_cast<size_t>(p.N) * p.P * ((p.Q + kTw - 1) / kTw) < 0x7fffffffull) {
    const int qtiles = (p.Q + kTw - 1) / kTw;
    const size_t tiles = static_cast<size_t>(p.N) * p.P * qtiles;
    int tchunks = static_cast<int>((tiles + ty * 2 - 1) / (static_cast<size_t>(ty) * 2));
    if (tchunks > cap) tchunks = cap;
    if (tchunks < 1) tchunks = 1;
    dim3 tgrid(tchunks, slabs);
    if (p.sh == 1)
      dw3x3_wgrad<1><<<tgrid, 256, smem, st>>>(x, dy, dw_tc, dbias, p, qtiles, tiles, tchunks, tx, ty);
    else
      dw3x3_wgrad<2><<<tgrid, 256, smem, st>>>(x, dy, dw_tc, dbias, p, qtiles, tiles, tchunks, tx, ty);
    return after_launch("depthwise_wgrad_3x3");
  }
  dim3 grid(chunks, slabs);
  switch (taps) {
    case 1: dw_wgrad<1, 1><<<grid, 256, smem, st>>>(x, dy, dw_tc, dbias, p, pixels, chunks, tx, ty); break;
    case 9: dw_wgrad<9, 3><<<grid, 256, smem, st>>>(x, dy, dw_tc, dbias, p, pixels, chunks, tx, ty); break;
    case 25: dw_wgrad<25, 5><<<grid, 256, smem, st>>>(x, dy, dw_tc, dbias, p, pixels, chunks, tx, ty); break;
    default: return fail(MB_ERR_UNSUPPORTED, "%s: %dx%d filters (1x1, 3x3 and 5x5 are built)", who, p.R, p.S);
  }
  return after_launch("depthwise_wgrad");
}

}  // extern "C"
