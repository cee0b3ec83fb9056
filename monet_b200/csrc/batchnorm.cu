// Batch normalisation for training: statistics + normalise forward (optionally
// in place), cached-statistics forward, and a backward that works either from
// the stored INPUT x or from the stored OUTPUT y (so x never has to be kept).
//
// Every pass is "reduce per channel, then a pure element-wise sweep":
//
//   reduce   grid = (row chunks S) x (channel slabs); each CTA reduces its rows
//            with 128-bit loads, a shared-memory stage over the row lanes, and
//            writes one partial per channel to the workspace  ws[2][S][C].
//            Many CTAs per channel: a 64-channel layer still fills 148 SMs
//            (the reference runs one CTA per channel, lrbn.cu:228-232).
//   finalize 32 channels x 32 stripes per CTA sum the S partials (fp64 at the end)
//            and write the per-channel constants the sweep needs.
//   sweep    element-wise, 128-bit, grid-stride.
//
// Forward statistics are accumulated around a per-channel shift K = the first
// element of the channel, so var = E[(x-K)^2] - E[x-K]^2 does not cancel
// catastrophically when |mean| >> std.
//
// Both backward flavours reduce S1 = sum(dy) and S2 = sum(dy * xhat):
//   from input : xhat = (x - mean) * invstd
//   from output: xhat = (y - beta) / gamma          (lrbn.cu:153-175)
// and then   dx = (dy - xhat*S2/M - S1/M) * invstd * gamma,  dgamma = S2,
// dbeta = S1  (lrbn.cu:176-208 written in terms of xhat).
//
// Fused forms (one sweep instead of two or three element-wise passes):
//   forward   y = act(bn(x) [+ residual]),  act = ReLU or identity
//   backward  through y = relu(bn(x)) from the stored INPUT x: the ReLU gate z > 0 is
//             re-evaluated from x with exactly the forward's expression
//             z = fma(x - mean, invstd*gamma, beta), so no mask and no output is kept and
//             dy is gated on the fly in both the reduce and the sweep.
//   backward  through y = relu(bn(x) + r) from x and y: the reduce pass also forms the gated
//             gradient d = (dy1 [+ dy2]) * (y > 0), writes it (it is the residual's gradient)
//             and sums it, so the separate ReLU-backward pass disappears.
#include <cstdlib>
#include "common.cuh"

#include <mutex>

namespace mb {
namespace {

constexpr int kBlock = 256;

struct Geometry {
  int C, HW, N;
  size_t M;      // N*HW, elements per channel
  int tx, ty;    // NHWC block shape: tx channel groups x ty rows
  int slabs;     // NHWC: channel slabs of tx*4 channels
  int S;         // chunks per channel
  int vec;       // NHWC: 4 if C % 4 == 0 else 1
};

int pow2ceil(int v) {
  int p = 1;
  while (p < v) p <<= 1;
  return p;
}

Geometry make_geometry(const mb_bn_desc* d) {
  Geometry g;
  g.C = d->C;
  g.HW = d->HW;
  g.N = d->N;
  g.M = static_cast<size_t>(d->N) * d->HW;
  if (d->layout == MB_NHWC) {
    g.vec = (d->C % 4 == 0) ? 4 : 1;
    int groups = d->C / g.vec;
    g.tx = pow2ceil(groups < kBlock ? groups : kBlock);
    g.ty = kBlock / g.tx;
    g.slabs = (groups + g.tx - 1) / g.tx;
    size_t rows_per_cta_min = static_cast<size_t>(g.ty) * 8;
    size_t want = (g.M + rows_per_cta_min - 1) / rows_per_cta_min;
    // one wave: 4 CTAs of 256 threads are resident per SM at the kernels' register use
    size_t cap = static_cast<size_t>(num_sms()) * 4 / g.slabs;
    if (cap < 1) cap = 1;
    g.S = static_cast<int>(want < cap ? want : cap);   // at most 592 partials per channel
  } else {
    g.vec = 1;
    g.tx = g.ty = 0;
    g.slabs = 1;
    size_t want = (g.M + 4095) / 4096;
    size_t cap = static_cast<size_t>(num_sms()) * 8 / (d->C > 0 ? d->C : 1);
    if (cap < 1) cap = 1;
    g.S = static_cast<int>(want < cap ? want : cap);
  }
  if (g.S < 1) g.S = 1;
  return g;
}

// workspace: partials [2][S][C] floats, then constants [2][C] floats
size_t ws_floats(const Geometry& g) { return (2 * static_cast<size_t>(g.S) + 2) * g.C; }

enum { kFwd = 0, kBwd = 1, kBwdRelu = 2, kFwdRes = 3, kBwdGate = 4 };

// ------------------------------------------- programmatic dependent launch
// A batch-norm call is a chain of two or three short kernels (reduce, finalize, sweep), 138 times
// per ResNet-50 step.  The dependent ones are launched with programmatic stream serialization:
// they may become resident while their predecessor is still running and block in
// `griddepcontrol.wait` (which returns once the predecessor grid has completed and its writes
// are visible) before they touch memory, so the launch latency of each link overlaps the tail of
// the previous one.  A kernel launched without the attribute sees `wait` as a no-op; a
// predecessor that never triggers releases its dependents when it exits.
// The chain stops at the batch-norm kernels on purpose: launching the tensor-core kernels
// and the reduce kernel the same way (trigger at entry, wait after the prologue) made the
// eagerly launched ResNet-50 step 1.3 % faster but the same step replayed from a CUDA graph
// 1.2 % slower (29.55 against 29.20 ms, same GPU, alternating runs), and the replay is what
// a training loop runs.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

template <typename... KArgs, typename... Args>
cudaError_t launch_dependent(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                             cudaStream_t st, Args... args) {
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

// ------------------------------------------------------------- NHWC reduce
// MODE kFwd: a = x;          accumulates (x-K), (x-K)^2
// MODE kBwd: a = dy, b = v;  accumulates dy, dy*(v-p0)*p1
// MODE kBwdRelu: a = dy, b = x, p0 = mean, p1 = invstd; dy is first gated by
//                fma(x-mean, invstd*gamma, beta) > 0
// MODE kBwdGate: a = dy1, a2 = dy2 or null, act = y, b = x, p0 = mean, p1 = invstd;
//                d = (dy1 + dy2) * (y > 0) is written to dout (may alias a) and summed
template <int MODE, int VEC>
__global__ void __launch_bounds__(kBlock) bn_reduce_nhwc(const float* __restrict__ a,
                                                         const float* __restrict__ b,
                                                         const float* __restrict__ p0v,
                                                         const float* __restrict__ p1v,
                                                         int p1_is_gamma,
                                                         const float* __restrict__ gv,
                                                         const float* __restrict__ bv,
                                                         float* __restrict__ ws,
                                                         int C, size_t M, int S, int tx_n,
                                                         int ty_n, const float* a2 = nullptr,
                                                         const float* act = nullptr,
                                                         float* dout = nullptr,
                                                         float act_hi = __builtin_huge_valf()) {
  extern __shared__ float sm[];  // [ty_n][tx_n][2*VEC]
  pdl_trigger();                 // the finalize kernel may take its seats; it waits for this grid
  const int tx = threadIdx.x % tx_n, ty = threadIdx.x / tx_n;
  const int c0 = (blockIdx.y * tx_n + tx) * VEC;
  const bool live = c0 < C;
  float s1[VEC], s2[VEC], p0[VEC], p1[VEC], pg[VEC], pb[VEC];
#pragma unroll
  for (int k = 0; k < VEC; ++k) {
    s1[k] = s2[k] = 0.f;
    p0[k] = 0.f;
    p1[k] = 1.f;
    pg[k] = pb[k] = 0.f;
  }
  if (live) {
#pragma unroll
    for (int k = 0; k < VEC; ++k) {
      if (MODE == kFwd) {
        p0[k] = __ldg(a + c0 + k);  // shift K = first row of the channel
      } else {
        p0[k] = __ldg(p0v + c0 + k);
        float t = __ldg(p1v + c0 + k);
        p1[k] = p1_is_gamma ? 1.f / t : t;
        if (MODE == kBwdRelu) {
          pg[k] = t * __ldg(gv + c0 + k);
          pb[k] = __ldg(bv + c0 + k);
        }
      }
    }
    const size_t rows_per = (M + S - 1) / S;
    const size_t r0 = static_cast<size_t>(blockIdx.x) * rows_per;
    size_t r1 = r0 + rows_per;
    if (r1 > M) r1 = M;
    size_t r = r0 + ty;
    if (VEC == 4) {
      // four rows in flight per thread
      for (; r + 3 * static_cast<size_t>(ty_n) < r1; r += 4 * static_cast<size_t>(ty_n)) {
        float4 u[4], w[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const size_t off = (r + i * static_cast<size_t>(ty_n)) * C + c0;
          u[i] = __ldcs(reinterpret_cast<const float4*>(a + off));
          if (MODE != kFwd) w[i] = __ldcs(reinterpret_cast<const float4*>(b + off));
          if (MODE == kBwdGate) {
            const float4 y4 = __ldcs(reinterpret_cast<const float4*>(act + off));
            if (a2) {
              const float4 v2 = __ldcs(reinterpret_cast<const float4*>(a2 + off));
              u[i].x += v2.x; u[i].y += v2.y; u[i].z += v2.z; u[i].w += v2.w;
            }
            u[i].x = y4.x > 0.f ? u[i].x : 0.f;
            u[i].y = y4.y > 0.f ? u[i].y : 0.f;
            u[i].z = y4.z > 0.f ? u[i].z : 0.f;
            u[i].w = y4.w > 0.f ? u[i].w : 0.f;
            *reinterpret_cast<float4*>(dout + off) = u[i];
          }
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float uu[4] = {u[i].x, u[i].y, u[i].z, u[i].w};
          const float ww[4] = {w[i].x, w[i].y, w[i].z, w[i].w};
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            if (MODE == kFwd) {
              const float dlt = uu[k] - p0[k];
              s1[k] += dlt;
              s2[k] = fmaf(dlt, dlt, s2[k]);
            } else {
              float d = uu[k];
              if (MODE == kBwdRelu) {
                const float z = fmaf(ww[k] - p0[k], pg[k], pb[k]);
                d = (z > 0.f && z < act_hi) ? d : 0.f;
              }
              s1[k] += d;
              s2[k] = fmaf(d, (ww[k] - p0[k]) * p1[k], s2[k]);
            }
          }
        }
      }
    }
    for (; r < r1; r += ty_n) {
      const size_t off = r * C + c0;
#pragma unroll
      for (int k = 0; k < VEC; ++k) {
        float uu = __ldg(a + off + k);
        if (MODE == kBwdGate) {
          if (a2) uu += __ldg(a2 + off + k);
          uu = __ldg(act + off + k) > 0.f ? uu : 0.f;
          dout[off + k] = uu;
        }
        if (MODE == kFwd) {
          const float dlt = uu - p0[k];
          s1[k] += dlt;
          s2[k] = fmaf(dlt, dlt, s2[k]);
        } else {
          const float ww = __ldg(b + off + k);
          float d = uu;
          if (MODE == kBwdRelu) {
            const float z = fmaf(ww - p0[k], pg[k], pb[k]);
            d = (z > 0.f && z < act_hi) ? d : 0.f;
          }
          s1[k] += d;
          s2[k] = fmaf(d, (ww - p0[k]) * p1[k], s2[k]);
        }
      }
    }
  }
  float* mine = sm + (static_cast<size_t>(ty) * tx_n + tx) * 2 * VEC;
#pragma unroll
  for (int k = 0; k < VEC; ++k) {
    mine[k] = s1[k];
    mine[VEC + k] = s2[k];
  }
  __syncthreads();
  if (ty == 0 && live) {
    for (int j = 1; j < ty_n; ++j) {
      const float* o = sm + (static_cast<size_t>(j) * tx_n + tx) * 2 * VEC;
#pragma unroll
      for (int k = 0; k < VEC; ++k) {
        s1[k] += o[k];
        s2[k] += o[VEC + k];
      }
    }
    float* w1 = ws + static_cast<size_t>(blockIdx.x) * C + c0;
    float* w2 = ws + (static_cast<size_t>(S) + blockIdx.x) * C + c0;
#pragma unroll
    for (int k = 0; k < VEC; ++k) {
      w1[k] = s1[k];
      w2[k] = s2[k];
    }
  }
}

// ------------------------------------------------------------- NCHW reduce
// grid (C, S); a chunk is a range of the channel's N*HW elements.
template <int MODE>
__global__ void __launch_bounds__(kBlock) bn_reduce_nchw(const float* __restrict__ a,
                                                         const float* __restrict__ b,
                                                         const float* __restrict__ p0v,
                                                         const float* __restrict__ p1v,
                                                         int p1_is_gamma,
                                                         const float* __restrict__ gv,
                                                         const float* __restrict__ bv,
                                                         float* __restrict__ ws,
                                                         int C, int HW, size_t M, int S,
                                                         const float* a2 = nullptr,
                                                         const float* act = nullptr,
                                                         float* dout = nullptr,
                                                         float act_hi = __builtin_huge_valf()) {
  __shared__ float red[2][kBlock / 32];
  const int c = blockIdx.x;
  float p0, p1 = 1.f, pg = 0.f, pb = 0.f;
  if (MODE == kFwd) {
    p0 = __ldg(a + static_cast<size_t>(c) * HW);
  } else {
    p0 = __ldg(p0v + c);
    float t = __ldg(p1v + c);
    p1 = p1_is_gamma ? 1.f / t : t;
    if (MODE == kBwdRelu) {
      pg = t * __ldg(gv + c);
      pb = __ldg(bv + c);
    }
  }
  const size_t per = (M + S - 1) / S;
  const size_t j0 = static_cast<size_t>(blockIdx.y) * per;
  size_t j1 = j0 + per;
  if (j1 > M) j1 = M;
  float s1 = 0.f, s2 = 0.f;
  for (size_t j = j0 + threadIdx.x; j < j1; j += kBlock) {
    const size_t n = j / HW;
    const size_t off = (n * C + c) * HW + (j - n * HW);
    float u = __ldg(a + off);
    if (MODE == kBwdGate) {
      if (a2) u += __ldg(a2 + off);
      u = __ldg(act + off) > 0.f ? u : 0.f;
      dout[off] = u;
    }
    if (MODE == kFwd) {
      const float dlt = u - p0;
      s1 += dlt;
      s2 = fmaf(dlt, dlt, s2);
    } else {
      const float w = __ldg(b + off);
      float d = u;
      if (MODE == kBwdRelu) {
        const float z = fmaf(w - p0, pg, pb);
        d = (z > 0.f && z < act_hi) ? d : 0.f;
      }
      s1 += d;
      s2 = fmaf(d, (w - p0) * p1, s2);
    }
  }
  s1 = warp_sum(s1);
  s2 = warp_sum(s2);
  if ((threadIdx.x & 31) == 0) {
    red[0][threadIdx.x >> 5] = s1;
    red[1][threadIdx.x >> 5] = s2;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int i = 1; i < kBlock / 32; ++i) {
      s1 += red[0][i];
      s2 += red[1][i];
    }
    ws[static_cast<size_t>(blockIdx.y) * C + c] = s1;
    ws[(static_cast<size_t>(S) + blockIdx.y) * C + c] = s2;
  }
}

// ---------------------------------------------------------------- finalize
// block = 32 channels (lanes) x 32 chunk stripes (warps).  Every thread sums its stripe
// of the S partials with four independent loads in flight (the loop is latency-bound:
// one dependent chain over all S partials costs tens of microseconds), then the 32
// stripes of a channel are combined in fp64 through shared memory.
constexpr int kFinStripes = 32;
template <int MODE>
__global__ void __launch_bounds__(32 * kFinStripes) bn_finalize(
    const float* __restrict__ ws_part, float* __restrict__ ws_const,
    const float* __restrict__ first_elems, size_t first_stride, int C, size_t M, int S, float eps,
    float momentum, float* __restrict__ running_mean, float* __restrict__ running_var,
    float* __restrict__ out0, float* __restrict__ out1) {
  __shared__ double red[2][kFinStripes][33];
  pdl_wait();                    // the partial sums are complete and visible
  pdl_trigger();                 // the sweep may take its seats
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  const int c = blockIdx.x * 32 + tx;
  float a1[4] = {0.f, 0.f, 0.f, 0.f}, a2[4] = {0.f, 0.f, 0.f, 0.f};
  if (c < C) {
    const float* p1 = ws_part + c;
    const float* p2 = ws_part + static_cast<size_t>(S) * C + c;
    int s = ty;
    for (; s + 3 * kFinStripes < S; s += 4 * kFinStripes) {
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        a1[j] += __ldg(p1 + static_cast<size_t>(s + j * kFinStripes) * C);
        a2[j] += __ldg(p2 + static_cast<size_t>(s + j * kFinStripes) * C);
      }
    }
    for (; s < S; s += kFinStripes) {
      a1[0] += __ldg(p1 + static_cast<size_t>(s) * C);
      a2[0] += __ldg(p2 + static_cast<size_t>(s) * C);
    }
  }
  red[0][ty][tx] = (static_cast<double>(a1[0]) + a1[1]) + (static_cast<double>(a1[2]) + a1[3]);
  red[1][ty][tx] = (static_cast<double>(a2[0]) + a2[1]) + (static_cast<double>(a2[2]) + a2[3]);
  __syncthreads();
  if (ty == 0 && c < C) {
    double s1 = 0.0, s2 = 0.0;
    for (int j = 0; j < kFinStripes; ++j) {
      s1 += red[0][j][tx];
      s2 += red[1][j][tx];
    }
    const double m = static_cast<double>(M);
    if (MODE == kFwd) {
      const double K = first_elems ? static_cast<double>(first_elems[static_cast<size_t>(c) * first_stride]) : 0.0;
      const double e1 = s1 / m;
      double var = s2 / m - e1 * e1;
      if (var < 0.0) var = 0.0;
      const double mean = K + e1;
      out0[c] = static_cast<float>(mean);                                   // save_mean
      out1[c] = static_cast<float>(1.0 / sqrt(var + static_cast<double>(eps)));  // save_invstd
      if (running_mean) running_mean[c] = (1.f - momentum) * running_mean[c] + momentum * static_cast<float>(mean);
      if (running_var) {
        const double unbiased = M > 1 ? var * m / (m - 1.0) : var;
        running_var[c] = (1.f - momentum) * running_var[c] + momentum * static_cast<float>(unbiased);
      }
    } else {
      out0[c] = static_cast<float>(s2);  // dgamma
      out1[c] = static_cast<float>(s1);  // dbeta
      ws_const[c] = static_cast<float>(s1 / m);
      ws_const[C + c] = static_cast<float>(s2 / m);
    }
  }
}

// ------------------------------------------------------------------- sweeps
// MODE kFwd:     out = act((a - mean)*(invstd*gamma) + beta)
// MODE kFwdRes:  out = act((a - mean)*(invstd*gamma) + beta + b),  b = residual
// MODE kBwd:     out = (a - xhat*k2 - k1)*(invstd*gamma),  a = dy, xhat = (b-p0)*p1
// MODE kBwdRelu: as kBwd with b = x, p0 = mean, p1 = invstd and a gated by
//                fma(x-mean, invstd*gamma, beta) > 0
struct SweepConst {
  const float* gamma;
  const float* beta;    // fwd
  const float* mean;    // fwd
  const float* invstd;
  const float* p0v;     // bwd
  const float* p1v;     // bwd
  int p1_is_gamma;
  const float* k12;     // bwd: [2][C]
  int relu;             // fwd modes: clamp the result at zero
  float act_hi;         // upper clamp of the activation (+inf: ReLU, 6: ReLU6)
};

template <int MODE>
__device__ __forceinline__ void load_const(const SweepConst& k, int c, int C, float& q0, float& q1,
                                           float& q2, float& q3, float& q4, float& q5) {
  q5 = 0.f;
  if (MODE == kFwd || MODE == kFwdRes) {
    q0 = __ldg(k.mean + c);
    q1 = __ldg(k.invstd + c) * __ldg(k.gamma + c);
    q2 = __ldg(k.beta + c);
    q3 = q4 = 0.f;
  } else {
    q0 = __ldg(k.p0v + c);
    float t = __ldg(k.p1v + c);
    q1 = k.p1_is_gamma ? 1.f / t : t;
    q2 = __ldg(k.k12 + c);      // S1/M
    q3 = __ldg(k.k12 + C + c);  // S2/M
    q4 = __ldg(k.invstd + c) * __ldg(k.gamma + c);
    if (MODE == kBwdRelu) q5 = __ldg(k.beta + c);
  }
}

template <int MODE>
__device__ __forceinline__ float sweep1(float a, float b, float q0, float q1, float q2, float q3,
                                        float q4, float q5, int relu, float hi) {
  if (MODE == kFwd || MODE == kFwdRes) {
    float z = fmaf(a - q0, q1, q2);
    if (MODE == kFwdRes) z += b;
    return relu ? (z > 0.f ? fminf(z, hi) : (z != z ? z : 0.f)) : z;   // NaN passes through, as in ReLU
  }
  if (MODE == kBwdRelu) {
    const float z = fmaf(b - q0, q4, q5);
    a = (z > 0.f && z < hi) ? a : 0.f;
  }
  const float xhat = (b - q0) * q1;
  return (a - xhat * q3 - q2) * q4;
}

template <int MODE, int VEC>
__global__ void __launch_bounds__(kBlock) bn_sweep_nhwc(const float* a, const float* b, float* out,
                                                        SweepConst k, int C, size_t M, int tx_n,
                                                        int ty_n) {
  pdl_wait();                    // the constants of the finalize kernel are complete and visible
  const int tx = threadIdx.x % tx_n, ty = threadIdx.x / tx_n;
  const int c0 = (blockIdx.y * tx_n + tx) * VEC;
  if (c0 >= C) return;
  float q0[VEC], q1[VEC], q2[VEC], q3[VEC], q4[VEC], q5[VEC];
#pragma unroll
  for (int i = 0; i < VEC; ++i) load_const<MODE>(k, c0 + i, C, q0[i], q1[i], q2[i], q3[i], q4[i], q5[i]);
  const int relu = k.relu;
  const float hi = k.act_hi;
  const size_t step = static_cast<size_t>(gridDim.x) * ty_n;
  size_t r = static_cast<size_t>(blockIdx.x) * ty_n + ty;
  if (VEC == 4) {
    for (; r + 3 * step < M; r += 4 * step) {
      float4 u[4], w[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const size_t off = (r + i * step) * C + c0;
        u[i] = *reinterpret_cast<const float4*>(a + off);
        if (MODE != kFwd) w[i] = *reinterpret_cast<const float4*>(b + off);
      }
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        float4 o;
        o.x = sweep1<MODE>(u[i].x, w[i].x, q0[0], q1[0], q2[0], q3[0], q4[0], q5[0], relu, hi);
        o.y = sweep1<MODE>(u[i].y, w[i].y, q0[1], q1[1], q2[1], q3[1], q4[1], q5[1], relu, hi);
        o.z = sweep1<MODE>(u[i].z, w[i].z, q0[2], q1[2], q2[2], q3[2], q4[2], q5[2], relu, hi);
        o.w = sweep1<MODE>(u[i].w, w[i].w, q0[3], q1[3], q2[3], q3[3], q4[3], q5[3], relu, hi);
        *reinterpret_cast<float4*>(out + (r + i * step) * C + c0) = o;
      }
    }
  }
  for (; r < M; r += step) {
    const size_t off = r * C + c0;
#pragma unroll
    for (int i = 0; i < VEC; ++i) {
      const float u = a[off + i];
      const float w = MODE != kFwd ? b[off + i] : 0.f;
      out[off + i] = sweep1<MODE>(u, w, q0[i], q1[i], q2[i], q3[i], q4[i], q5[i], relu, hi);
    }
  }
}

// grid (planes = N*C, chunks of HW)
template <int MODE>
__global__ void __launch_bounds__(kBlock) bn_sweep_nchw(const float* a, const float* b, float* out,
                                                        SweepConst k, int C, int HW) {
  const int c = blockIdx.x % C;
  float q0, q1, q2, q3, q4, q5;
  load_const<MODE>(k, c, C, q0, q1, q2, q3, q4, q5);
  const size_t base = static_cast<size_t>(blockIdx.x) * HW;
  for (int i = blockIdx.y * kBlock + threadIdx.x; i < HW; i += gridDim.y * kBlock) {
    const float u = a[base + i];
    const float w = MODE != kFwd ? b[base + i] : 0.f;
    out[base + i] = sweep1<MODE>(u, w, q0, q1, q2, q3, q4, q5, k.relu, k.act_hi);
  }
}

// activation code of the fused entries: 0 none, 1 ReLU, 2 ReLU6
float act_upper(int act) { return act == 2 ? 6.f : __builtin_huge_valf(); }

int check(const char* who, const mb_bn_desc* d) {
  if (!d) return fail(MB_ERR_INVALID_ARGUMENT, "%s: null descriptor", who);
  if (d->N <= 0 || d->C <= 0 || d->HW <= 0)
    return fail(MB_ERR_INVALID_ARGUMENT, "%s: bad extent N=%d C=%d HW=%d", who, d->N, d->C, d->HW);
  if (d->layout != MB_NCHW && d->layout != MB_NHWC)
    return fail(MB_ERR_INVALID_ARGUMENT, "%s: bad layout %d", who, d->layout);
  return MB_OK;
}

template <int MODE>
int run_reduce(const char* who, const mb_bn_desc* d, const Geometry& g, const float* a,
               const float* b, const float* p0v, const float* p1v, int p1_is_gamma, float* ws,
               cudaStream_t st, const float* gv = nullptr, const float* bv = nullptr,
               const float* a2 = nullptr, const float* act = nullptr, float* dout = nullptr,
               float act_hi = __builtin_huge_valf()) {
  if (d->layout == MB_NHWC) {
    dim3 grid(g.S, g.slabs);
    const size_t smem = static_cast<size_t>(kBlock) * 2 * g.vec * sizeof(float);
    if (g.vec == 4)
      bn_reduce_nhwc<MODE, 4><<<grid, kBlock, smem, st>>>(a, b, p0v, p1v, p1_is_gamma, gv, bv, ws, g.C, g.M, g.S, g.tx, g.ty, a2, act, dout, act_hi);
    else
      bn_reduce_nhwc<MODE, 1><<<grid, kBlock, smem, st>>>(a, b, p0v, p1v, p1_is_gamma, gv, bv, ws, g.C, g.M, g.S, g.tx, g.ty, a2, act, dout, act_hi);
  } else {
    dim3 grid(g.C, g.S);
    bn_reduce_nchw<MODE><<<grid, kBlock, 0, st>>>(a, b, p0v, p1v, p1_is_gamma, gv, bv, ws, g.C, g.HW, g.M, g.S, a2, act, dout, act_hi);
  }
  return after_launch(who);
}

template <int MODE>
int run_sweep(const char* who, const mb_bn_desc* d, const Geometry& g, const float* a,
              const float* b, float* out, const SweepConst& k, cudaStream_t st) {
  if (d->layout == MB_NHWC) {
    size_t want = (g.M + static_cast<size_t>(g.ty) * 4 - 1) / (static_cast<size_t>(g.ty) * 4);
    size_t cap = static_cast<size_t>(num_sms()) * 8 / g.slabs;
    if (cap < 1) cap = 1;
    dim3 grid(static_cast<unsigned>(want < cap ? want : cap), g.slabs);
    if (grid.x < 1) grid.x = 1;
    if (g.vec == 4)
      launch_dependent(bn_sweep_nhwc<MODE, 4>, grid, dim3(kBlock), 0, st, a, b, out, k, g.C, g.M, g.tx, g.ty);
    else
      launch_dependent(bn_sweep_nhwc<MODE, 1>, grid, dim3(kBlock), 0, st, a, b, out, k, g.C, g.M, g.tx, g.ty);
  } else {
    const size_t planes = static_cast<size_t>(g.N) * g.C;
    if (planes > 0x7fffffffULL) return fail(MB_ERR_UNSUPPORTED, "%s: N*C too large", who);
    int ychunks = (g.HW + kBlock * 4 - 1) / (kBlock * 4);
    if (ychunks > 65535) ychunks = 65535;
    dim3 grid(static_cast<unsigned>(planes), ychunks);
    bn_sweep_nchw<MODE><<<grid, kBlock, 0, st>>>(a, b, out, k, g.C, g.HW);
  }
  return after_launch(who);
}

int check_alignment(const char* who, const mb_bn_desc* d, const void* p0, const void* p1,
                    const void* p2) {
  if (d->layout == MB_NHWC && d->C % 4 == 0 &&
      !(aligned(p0, 16) && aligned(p1, 16) && aligned(p2, 16)))
    return fail(MB_ERR_INVALID_ARGUMENT, "%s: activation pointers must be 16-byte aligned", who);
  return MB_OK;
}

int bwd_common(const char* who, const float* dy, const float* v, const float* gamma,
               const float* p0v, const float* p1v, int p1_is_gamma, const float* invstd, float* dx,
               float* dgamma, float* dbeta, const mb_bn_desc* d, void* workspace,
               size_t workspace_bytes, void* stream, const float* relu_beta = nullptr,
               float act_hi = __builtin_huge_valf()) {
  int rc = check(who, d);
  if (rc) return rc;
  if (!dy || !v || !gamma || !p0v || !p1v || !invstd || !dx || !dgamma || !dbeta)
    return fail(MB_ERR_INVALID_ARGUMENT, "%s: null pointer", who);
  rc = check_alignment(who, d, dy, v, dx);
  if (rc) return rc;
  Geometry g = make_geometry(d);
  if (!workspace || workspace_bytes < ws_floats(g) * sizeof(float))
    return fail(MB_ERR_WORKSPACE, "%s: workspace of %zu bytes needed, %zu given", who,
                ws_floats(g) * sizeof(float), workspace ? workspace_bytes : size_t(0));
  float* ws = static_cast<float*>(workspace);
  float* ws_const = ws + 2 * static_cast<size_t>(g.S) * g.C;
  cudaStream_t st = as_stream(stream);
  if (relu_beta)
    rc = run_reduce<kBwdRelu>("bn_relu_bwd_reduce", d, g, dy, v, p0v, p1v, 0, ws, st, gamma, relu_beta,
                              nullptr, nullptr, nullptr, act_hi);
  else
    rc = run_reduce<kBwd>("bn_bwd_reduce", d, g, dy, v, p0v, p1v, p1_is_gamma, ws, st);
  if (rc) return rc;
  launch_dependent(bn_finalize<kBwd>, dim3((g.C + 31) / 32), dim3(32 * kFinStripes), 0, st, ws, ws_const, nullptr, 0, g.C, g.M, g.S, 0.f,
                                                    0.f, nullptr, nullptr, dgamma, dbeta);
  rc = after_launch("bn_bwd_finalize");
  if (rc) return rc;
  SweepConst k{gamma, relu_beta, nullptr, invstd, p0v, p1v, p1_is_gamma, ws_const, 0, act_hi};
  if (relu_beta) return run_sweep<kBwdRelu>("bn_relu_bwd_sweep", d, g, dy, v, dx, k, st);
  return run_sweep<kBwd>("bn_bwd_sweep", d, g, dy, v, dx, k, st);
}

}  // namespace
}  // namespace mb

using namespace mb;

extern "C" {

size_t mb_bn_workspace_bytes(const mb_bn_desc* d) {
  if (!d || d->N <= 0 || d->C <= 0 || d->HW <= 0) return 0;
  return ws_floats(make_geometry(d)) * sizeof(float);
}

static int fwd_train_impl(const char* who, const float* x, const float* residual, int relu,
                          const float* gamma, const float* beta, float* running_mean,
                          float* running_var, float* y, float* save_mean, float* save_invstd,
                          const mb_bn_desc* d, void* workspace, size_t workspace_bytes,
                          void* stream) {
  int rc = check(who, d);
  if (rc) return rc;
  if (!x || !gamma || !beta || !y || !save_mean || !save_invstd)
    return fail(MB_ERR_INVALID_ARGUMENT, "%s: null pointer", who);
  rc = check_alignment(who, d, x, y, residual ? residual : y);
  if (rc) return rc;
  Geometry g = make_geometry(d);
  if (!workspace || workspace_bytes < ws_floats(g) * sizeof(float))
    return fail(MB_ERR_WORKSPACE, "%s: workspace of %zu bytes needed, %zu given", who,
                ws_floats(g) * sizeof(float), workspace ? workspace_bytes : size_t(0));
  float* ws = static_cast<float*>(workspace);
  cudaStream_t st = as_stream(stream);
  rc = run_reduce<kFwd>("bn_fwd_reduce", d, g, x, nullptr, nullptr, nullptr, 0, ws, st);
  if (rc) return rc;
  const size_t first_stride = d->layout == MB_NHWC ? 1 : static_cast<size_t>(d->HW);
  launch_dependent(bn_finalize<kFwd>, dim3((g.C + 31) / 32), dim3(32 * kFinStripes), 0, st, ws, nullptr, x, first_stride, g.C, g.M, g.S,
                                                    d->eps, d->momentum, running_mean,
                                                    running_var, save_mean, save_invstd);
  rc = after_launch("bn_fwd_finalize");
  if (rc) return rc;
  SweepConst k{gamma, beta, save_mean, save_invstd, nullptr, nullptr, 0, nullptr, relu ? 1 : 0, act_upper(relu)};
  if (residual) return run_sweep<kFwdRes>("bn_act_fwd_sweep", d, g, x, residual, y, k, st);
  return run_sweep<kFwd>("bn_fwd_sweep", d, g, x, nullptr, y, k, st);
}

static int fwd_apply_impl(const char* who, const float* x, const float* residual, int relu,
                          const float* gamma, const float* beta, const float* mean,
                          const float* invstd, float* y, const mb_bn_desc* d, void* stream) {
  int rc = check(who, d);
  if (rc) return rc;
  if (!x || !gamma || !beta || !mean || !invstd || !y)
    return fail(MB_ERR_INVALID_ARGUMENT, "%s: null pointer", who);
  rc = check_alignment(who, d, x, y, residual ? residual : y);
  if (rc) return rc;
  Geometry g = make_geometry(d);
  SweepConst k{gamma, beta, mean, invstd, nullptr, nullptr, 0, nullptr, relu ? 1 : 0, act_upper(relu)};
  if (residual) return run_sweep<kFwdRes>("bn_act_fwd_sweep", d, g, x, residual, y, k, as_stream(stream));
  return run_sweep<kFwd>("bn_fwd_sweep", d, g, x, nullptr, y, k, as_stream(stream));
}

int mb_bn_fwd_train(const float* x, const float* gamma, const float* beta, float* running_mean,
                    float* running_var, float* y, float* save_mean, float* save_invstd,
                    const mb_bn_desc* d, void* workspace, size_t workspace_bytes, void* stream) {
  return fwd_train_impl("mb_bn_fwd_train", x, nullptr, 0, gamma, beta, running_mean, running_var, y,
                        save_mean, save_invstd, d, workspace, workspace_bytes, stream);
}

int mb_bn_fwd_apply(const float* x, const float* gamma, const float* beta, const float* mean,
                    const float* invstd, float* y, const mb_bn_desc* d, void* stream) {
  return fwd_apply_impl("mb_bn_fwd_apply", x, nullptr, 0, gamma, beta, mean, invstd, y, d, stream);
}

int mb_bn_act_fwd_train(const float* x, const float* residual, int relu, const float* gamma,
                        const float* beta, float* running_mean, float* running_var, float* y,
                        float* save_mean, float* save_invstd, const mb_bn_desc* d, void* workspace,
                        size_t workspace_bytes, void* stream) {
  return fwd_train_impl("mb_bn_act_fwd_train", x, residual, relu, gamma, beta, running_mean,
                        running_var, y, save_mean, save_invstd, d, workspace, workspace_bytes, stream);
}

int mb_bn_act_fwd_apply(const float* x, const float* residual, int relu, const float* gamma,
                        const float* beta, const float* mean, const float* invstd, float* y,
                        const mb_bn_desc* d, void* stream) {
  return fwd_apply_impl("mb_bn_act_fwd_apply", x, residual, relu, gamma, beta, mean, invstd, y, d,
                        stream);
}

int mb_bn_act_fwd_train_partials(const float* x, const float* residual, int relu, const float* gamma,
                                 const float* beta, float* running_mean, float* running_var,
                                 float* y, float* save_mean, float* save_invstd,
                                 const mb_bn_desc* d, const float* partials, int partial_rows,
                                 const float* shift, void* stream) {
  const char* who = "mb_bn_act_fwd_train_partials";
  int rc = check(who, d);
  if (rc) return rc;
  if (!x || !gamma || !beta || !y || !save_mean || !save_invstd || !partials || partial_rows <= 0)
    return fail(MB_ERR_INVALID_ARGUMENT, "%s: null pointer or no partial sums", who);
  rc = check_alignment(who, d, x, y, residual ? residual : y);
  if (rc) return rc;
  Geometry g = make_geometry(d);
  cudaStream_t st = as_stream(stream);
  // the statistics pass over x is replaced by the sums its producer left: finalize over
  // `partial_rows` rows of [2][rows][C], taken around `shift` (null: zero)
  launch_dependent(bn_finalize<kFwd>, dim3((g.C + 31) / 32), dim3(32 * kFinStripes), 0, st, partials, nullptr, shift, 1, g.C, g.M, partial_rows, d->eps, d->momentum, running_mean,
      running_var, save_mean, save_invstd);
  rc = after_launch("bn_fwd_finalize");
  if (rc) return rc;
  SweepConst k{gamma, beta, save_mean, save_invstd, nullptr, nullptr, 0, nullptr, relu ? 1 : 0, act_upper(relu)};
  if (residual) return run_sweep<kFwdRes>("bn_act_fwd_sweep", d, g, x, residual, y, k, st);
  return run_sweep<kFwd>("bn_fwd_sweep", d, g, x, nullptr, y, k, st);
}

int mb_bn_add_relu_bwd(const float* dy1, const float* dy2, const float* y, const float* x,
                       const float* gamma, const float* save_mean, const float* save_invstd,
                       float* d, float* dx, float* dgamma, float* dbeta, const mb_bn_desc* desc,
                       void* workspace, size_t workspace_bytes, void* stream) {
  const char* who = "mb_bn_add_relu_bwd";
  int rc = check(who, desc);
  if (rc) return rc;
  if (!dy1 || !y || !x || !gamma || !save_mean || !save_invstd || !d || !dx || !dgamma || !dbeta)
    return fail(MB_ERR_INVALID_ARGUMENT, "%s: null pointer", who);
  rc = check_alignment(who, desc, dy1, y, x);
  if (!rc) rc = check_alignment(who, desc, d, dx, dy2 ? dy2 : dy1);
  if (rc) return rc;
  Geometry g = make_geometry(desc);
  if (!workspace || workspace_bytes < ws_floats(g) * sizeof(float))
    return fail(MB_ERR_WORKSPACE, "%s: workspace of %zu bytes needed, %zu given", who,
                ws_floats(g) * sizeof(float), workspace ? workspace_bytes : size_t(0));
  float* ws = static_cast<float*>(workspace);
  float* ws_const = ws + 2 * static_cast<size_t>(g.S) * g.C;
  cudaStream_t st = as_stream(stream);
  rc = run_reduce<kBwdGate>("bn_add_relu_bwd_reduce", desc, g, dy1, x, save_mean, save_invstd, 0, ws,
                            st, nullptr, nullptr, dy2, y, d);
  if (rc) return rc;
  launch_dependent(bn_finalize<kBwd>, dim3((g.C + 31) / 32), dim3(32 * kFinStripes), 0, st, ws, ws_const, nullptr, 0, g.C, g.M, g.S, 0.f,
                                                    0.f, nullptr, nullptr, dgamma, dbeta);
  rc = after_launch("bn_bwd_finalize");
  if (rc) return rc;
  SweepConst k{gamma, nullptr, nullptr, save_invstd, save_mean, save_invstd, 0, ws_const, 0, __builtin_huge_valf()};
  return run_sweep<kBwd>("bn_bwd_sweep", desc, g, d, x, dx, k, st);
}

int mb_bn_act_bwd_from_input(const float* dy, const float* x, const float* gamma, const float* beta,
                             const float* save_mean, const float* save_invstd, int act, float* dx,
                             float* dgamma, float* dbeta, const mb_bn_desc* d, void* workspace,
                             size_t workspace_bytes, void* stream) {
  if (act != 1 && act != 2)
    return fail(MB_ERR_INVALID_ARGUMENT, "mb_bn_act_bwd_from_input: activation must be 1 (ReLU) or 2 (ReLU6)");
  if (!beta) return fail(MB_ERR_INVALID_ARGUMENT, "mb_bn_act_bwd_from_input: null pointer");
  return bwd_common("mb_bn_act_bwd_from_input", dy, x, gamma, save_mean, save_invstd, 0, save_invstd,
                    dx, dgamma, dbeta, d, workspace, workspace_bytes, stream, beta, act_upper(act));
}

int mb_bn_relu_bwd_from_input(const float* dy, const float* x, const float* gamma,
                              const float* beta, const float* save_mean, const float* save_invstd,
                              float* dx, float* dgamma, float* dbeta, const mb_bn_desc* d,
                              void* workspace, size_t workspace_bytes, void* stream) {
  if (!beta) return fail(MB_ERR_INVALID_ARGUMENT, "mb_bn_relu_bwd_from_input: null pointer");
  return bwd_common("mb_bn_relu_bwd_from_input", dy, x, gamma, save_mean, save_invstd, 0,
                    save_invstd, dx, dgamma, dbeta, d, workspace, workspace_bytes, stream, beta);
}

int mb_bn_bwd_from_output(const float* dy, const float* y, const float* gamma, const float* beta,
                          const float* save_invstd, float* dx, float* dgamma, float* dbeta,
                          const mb_bn_desc* d, void* workspace, size_t workspace_bytes,
                          void* stream) {
  return bwd_common("mb_bn_bwd_from_output", dy, y, gamma, beta, gamma, 1, save_invstd, dx, dgamma,
                    dbeta, d, workspace, workspace_bytes, stream);
}

int mb_bn_bwd_from_input(const float* dy, const float* x, const float* gamma,
                         const float* save_mean, const float* save_invstd, float* dx,
                         float* dgamma, float* dbeta, const mb_bn_desc* d, void* workspace,
                         size_t workspace_bytes, void* stream) {
  return bwd_common("mb_bn_bwd_from_input", dy, x, gamma, save_mean, save_invstd, 0, save_invstd,
                    dx, dgamma, dbeta, d, workspace, workspace_bytes, stream);
}


// ---- statistics scratch that lives inside the library -----------------------------------
// 2 Mi floats = 8 MiB per GPU that loads the library, held until the process exits.
constexpr size_t kStaticScratchFloats = size_t(2) << 20;
static __device__ __align__(256) float g_bn_static_scratch[kStaticScratchFloats];

namespace {
constexpr int kMaxDevices = 64;
std::mutex g_scratch_mutex;
float* g_scratch_ptr[kMaxDevices] = {};   // device address of the array, per device ordinal
}  // namespace

// Same result as mb_bn_fwd_train, for hosts that must not allocate while a step runs: the
// statistics scratch is the array above instead of a caller-provided workspace.
//
// Who needs it.  MONeT executes a schedule whose every byte was planned by its solver under a
// fixed memory budget, and serving / training loops built that way often hand the whole
// device to one pool up front.  In such a host a kernel that asks for "a few more megabytes"
// at run time either cannot get them (the pool owns the device) or breaks the plan it runs
// under, and cudaMalloc / cudaFree would also stall every stream of the device.  This entry
// point therefore calls no cudaMalloc, cudaFree or any allocating library routine.
//
// Set-up.  `g_bn_static_scratch` names a host-side handle, not a device address; the first
// call on each device (with that device current) resolves it with cudaGetSymbolAddress and
// caches the pointer.  Make that first call before starting any stream capture.
//
// Limits.  Shapes whose scratch need (mb_bn_workspace_bytes) exceeds 8 MiB are rejected with
// MB_ERR_WORKSPACE.  All calls on a device share the one array: it keeps whatever the last
// call left there (nothing in it has to start at zero - every partial sum that is read is
// written first by the same call), and two calls that overlap on the GPU, e.g. on different
// streams, race on it.  Serialise them, or use mb_bn_fwd_train with separate workspaces.
int mb_bn_fwd_train_noalloc(const float* x, const float* gamma, const float* beta,
                            float* running_mean, float* running_var, float* y, float* save_mean,
                            float* save_invstd, const mb_bn_desc* d, void* stream) {
  const char* who = "mb_bn_fwd_train_noalloc";
  int rc = check(who, d);
  if (rc) return rc;
  const size_t need = mb_bn_workspace_bytes(d);
  if (need == 0 || need > kStaticScratchFloats * sizeof(float))
    return fail(MB_ERR_WORKSPACE,
                "%s: this shape needs %zu bytes of scratch, the built-in array holds %zu; use "
                "mb_bn_fwd_train with a workspace of your own",
                who, need, kStaticScratchFloats * sizeof(float));
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess || dev < 0 || dev >= kMaxDevices)
    return fail(MB_ERR_LAUNCH, "%s: cannot identify the current device: %s", who, cudaGetErrorString(e));
  float* scratch = nullptr;
  {
    std::lock_guard<std::mutex> lock(g_scratch_mutex);
    if (!g_scratch_ptr[dev]) {
      void* p = nullptr;
      e = cudaGetSymbolAddress(&p, g_bn_static_scratch);
      if (e != cudaSuccess || !p)
        return fail(MB_ERR_LAUNCH, "%s: cudaGetSymbolAddress failed: %s", who, cudaGetErrorString(e));
      g_scratch_ptr[dev] = static_cast<float*>(p);
    }
    scratch = g_scratch_ptr[dev];
  }
  return mb_bn_fwd_train(x, gamma, beta, running_mean, running_var, y, save_mean, save_invstd, d,
                         scratch, kStaticScratchFloats * sizeof(float), stream);
}

}  // extern "C"
