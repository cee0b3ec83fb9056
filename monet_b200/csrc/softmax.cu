// Softmax / log-softmax forward and backward, and the fused
// log-softmax + NLL loss forward+backward that touches the logits once.
//
// Tensor view: [outer, classes, inner], reduction over `classes`.
//   inner == 1 : one warp per row; rows up to 1024 classes live in registers
//                (one global read, one global write per element).
//   inner  > 1 : one thread per (outer, inner) position, walking the class
//                axis with stride `inner` (coalesced across the warp).
#include "common.cuh"

namespace mb {
namespace {

constexpr int kWarpsPerBlock = 8;
constexpr int kRegCols = 32;  // 32 lanes x 32 registers = 1024 classes

// ---- row kernels (inner == 1) ------------------------------------------------
// KIND 0: softmax fwd, 1: log-softmax fwd, 2: softmax bwd, 3: log-softmax bwd,
// KIND 4: fused cross-entropy fwd+bwd.
template <int KIND, bool IN_REGS>
__global__ void __launch_bounds__(kWarpsPerBlock * 32) softmax_rows(
    const float* __restrict__ a, const float* __restrict__ b, const int64_t* __restrict__ labels,
    float* __restrict__ out, float* __restrict__ loss_rows, size_t rows, int classes,
    float grad_scale) {
  const int lane = threadIdx.x & 31;
  const size_t warp = static_cast<size_t>(blockIdx.x) * kWarpsPerBlock + (threadIdx.x >> 5);
  const size_t nwarps = static_cast<size_t>(gridDim.x) * kWarpsPerBlock;
  for (size_t r = warp; r < rows; r += nwarps) {
    const float* ar = a + r * classes;
    const float* br = b ? b + r * classes : nullptr;
    float* outr = out + r * classes;
    float va[IN_REGS ? kRegCols : 1], vb[IN_REGS ? kRegCols : 1];
    if (IN_REGS) {
#pragma unroll
      for (int k = 0; k < kRegCols; ++k) {
        const int i = k * 32 + lane;
        va[k] = i < classes ? __ldg(ar + i) : 0.f;
        if (KIND == 2 || KIND == 3) vb[k] = i < classes ? __ldg(br + i) : 0.f;
      }
    }
    auto A = [&](int k, int i) { return IN_REGS ? va[k] : __ldg(ar + i); };
    auto B = [&](int k, int i) { return IN_REGS ? vb[k] : __ldg(br + i); };
    const int ncols = (classes + 31) / 32;

    if (KIND == 0 || KIND == 1 || KIND == 4) {
      float mx = -INFINITY;
      if (IN_REGS) {
#pragma unroll
        for (int k = 0; k < kRegCols; ++k)
          if (k * 32 + lane < classes) mx = fmaxf(mx, va[k]);
      } else {
        for (int k = 0; k < ncols; ++k)
          if (k * 32 + lane < classes) mx = fmaxf(mx, A(k, k * 32 + lane));
      }
      mx = warp_max(mx);
      float sum = 0.f;
      if (IN_REGS) {
        // softmax and the fused loss keep exp(x - max) in the register that held x: one expf
        // per element instead of two (log-softmax needs x itself again)
#pragma unroll
        for (int k = 0; k < kRegCols; ++k)
          if (k * 32 + lane < classes) {
            const float e = expf(va[k] - mx);
            if (KIND != 1) va[k] = e;
            sum += e;
          }
      } else {
        for (int k = 0; k < ncols; ++k)
          if (k * 32 + lane < classes) sum += expf(A(k, k * 32 + lane) - mx);
      }
      sum = warp_sum(sum);
      const float lse = mx + logf(sum);
      const float inv = 1.f / sum;
      int label = -1;
      if (KIND == 4) {
        label = static_cast<int>(labels[r]);
        if (lane == 0) {
          const bool ok = label >= 0 && label < classes;
          loss_rows[r] = ok ? lse - __ldg(ar + label) : 0.f;
        }
      }
      auto emit = [&](int k, int i) {
        const float x = A(k, i);
        const float e = (IN_REGS && KIND != 1) ? x : expf(x - mx);     // x already holds the exponential
        float o;
        if (KIND == 0) o = e * inv;
        else if (KIND == 1) o = x - lse;
        else o = (e * inv - (i == label ? 1.f : 0.f)) * grad_scale;
        outr[i] = o;
      };
      if (IN_REGS) {
#pragma unroll
        for (int k = 0; k < kRegCols; ++k)
          if (k * 32 + lane < classes) emit(k, k * 32 + lane);
      } else {
        for (int k = 0; k < ncols; ++k)
          if (k * 32 + lane < classes) emit(k, k * 32 + lane);
      }
    } else {
      // a = dy, b = y (softmax output or log-softmax output)
      float dot = 0.f;
      if (IN_REGS) {
#pragma unroll
        for (int k = 0; k < kRegCols; ++k)
          if (k * 32 + lane < classes) dot += (KIND == 2) ? va[k] * vb[k] : va[k];
      } else {
        for (int k = 0; k < ncols; ++k) {
          const int i = k * 32 + lane;
          if (i < classes) dot += (KIND == 2) ? A(k, i) * B(k, i) : A(k, i);
        }
      }
      dot = warp_sum(dot);
      auto emit = [&](int k, int i) {
        const float dyv = A(k, i), yv = B(k, i);
        outr[i] = (KIND == 2) ? yv * (dyv - dot) : dyv - expf(yv) * dot;
      };
      if (IN_REGS) {
#pragma unroll
        for (int k = 0; k < kRegCols; ++k)
          if (k * 32 + lane < classes) emit(k, k * 32 + lane);
      } else {
        for (int k = 0; k < ncols; ++k)
          if (k * 32 + lane < classes) emit(k, k * 32 + lane);
      }
    }
  }
}

// ---- strided kernels (inner > 1) ---------------------------------------------
template <int KIND>
__global__ void __launch_bounds__(256) softmax_strided(
    const float* __restrict__ a, const float* __restrict__ b, const int64_t* __restrict__ labels,
    float* __restrict__ out, float* __restrict__ loss_rows, size_t outer, int classes,
    size_t inner, float grad_scale) {
  const size_t total = outer * inner;
  for (size_t t = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; t < total;
       t += static_cast<size_t>(gridDim.x) * blockDim.x) {
    const size_t o = t / inner, in = t - o * inner;
    const size_t base = o * classes * inner + in;
    if (KIND == 0 || KIND == 1 || KIND == 4) {
      float mx = -INFINITY;
      for (int c = 0; c < classes; ++c) mx = fmaxf(mx, __ldg(a + base + c * inner));
      float sum = 0.f;
      for (int c = 0; c < classes; ++c) sum += expf(__ldg(a + base + c * inner) - mx);
      const float lse = mx + logf(sum), inv = 1.f / sum;
      int label = -1;
      if (KIND == 4) {
        label = static_cast<int>(labels[t]);
        const bool ok = label >= 0 && label < classes;
        loss_rows[t] = ok ? lse - __ldg(a + base + static_cast<size_t>(label) * inner) : 0.f;
      }
      for (int c = 0; c < classes; ++c) {
        const float x = __ldg(a + base + c * inner);
        float v;
        if (KIND == 0) v = expf(x - mx) * inv;
        else if (KIND == 1) v = x - lse;
        else v = (expf(x - mx) * inv - (c == label ? 1.f : 0.f)) * grad_scale;
        out[base + c * inner] = v;
      }
    } else {
      float dot = 0.f;
      for (int c = 0; c < classes; ++c) {
        const float dyv = __ldg(a + base + c * inner);
        dot += (KIND == 2) ? dyv * __ldg(b + base + c * inner) : dyv;
      }
      for (int c = 0; c < classes; ++c) {
        const float dyv = __ldg(a + base + c * inner), yv = __ldg(b + base + c * inner);
        out[base + c * inner] = (KIND == 2) ? yv * (dyv - dot) : dyv - expf(yv) * dot;
      }
    }
  }
}

template <int KIND>
int dispatch(const char* who, const float* a, const float* b, const int64_t* labels, float* out,
             float* loss_rows, size_t outer, int classes, size_t inner, float grad_scale,
             void* stream) {
  if (classes <= 0) return fail(MB_ERR_INVALID_ARGUMENT, "%s: classes must be positive", who);
  if (outer == 0 || inner == 0) return MB_OK;
  if (!a || !out) return fail(MB_ERR_INVALID_ARGUMENT, "%s: null pointer", who);
  cudaStream_t st = as_stream(stream);
  if (inner == 1) {
    const int grid = grid_for(outer, kWarpsPerBlock, 8);
    if (classes <= 32 * kRegCols)
      softmax_rows<KIND, true><<<grid, kWarpsPerBlock * 32, 0, st>>>(a, b, labels, out, loss_rows, outer, classes, grad_scale);
    else
      softmax_rows<KIND, false><<<grid, kWarpsPerBlock * 32, 0, st>>>(a, b, labels, out, loss_rows, outer, classes, grad_scale);
  } else {
    const int grid = grid_for(outer * inner, 256, 8);
    softmax_strided<KIND><<<grid, 256, 0, st>>>(a, b, labels, out, loss_rows, outer, classes, inner, grad_scale);
  }
  return after_launch(who);
}

}  // namespace
}  // namespace mb

using namespace mb;

extern "C" {

int mb_softmax_fwd(const float* x, float* y, size_t outer, int classes, size_t inner,
                   int log_softmax, void* stream) {
  return log_softmax ? dispatch<1>("log_softmax_fwd", x, nullptr, nullptr, y, nullptr, outer, classes, inner, 0.f, stream)
                     : dispatch<0>("softmax_fwd", x, nullptr, nullptr, y, nullptr, outer, classes, inner, 0.f, stream);
}

int mb_softmax_bwd(const float* dy, const float* y, float* dx, size_t outer, int classes,
                   size_t inner, int log_softmax, void* stream) {
  if (outer && inner && !y) return fail(MB_ERR_INVALID_ARGUMENT, "mb_softmax_bwd: null pointer");
  return log_softmax ? dispatch<3>("log_softmax_bwd", dy, y, nullptr, dx, nullptr, outer, classes, inner, 0.f, stream)
                     : dispatch<2>("softmax_bwd", dy, y, nullptr, dx, nullptr, outer, classes, inner, 0.f, stream);
}

int mb_softmax_ce_fwd_bwd(const float* logits, const int64_t* labels, float* loss_rows,
                          float* dlogits, size_t outer, int classes, size_t inner,
                          float grad_scale, void* stream) {
  if (outer && inner && (!labels || !loss_rows))
    return fail(MB_ERR_INVALID_ARGUMENT, "mb_softmax_ce_fwd_bwd: null pointer");
  return dispatch<4>("softmax_ce_fwd_bwd", logits, nullptr, labels, dlogits, loss_rows, outer, classes, inner, grad_scale, stream);
}

}  // extern "C"
