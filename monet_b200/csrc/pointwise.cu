// Memory-bound element-wise operators: ReLU (+1-bit mask), hardtanh, residual
// add, and the stand-alone bit / nibble packers.
//
// One scheme for all of them: a thread owns GROUPS of 8 consecutive fp32
// elements, moved with one 256-bit load and one 256-bit store, which is also
// exactly one byte of a 1-bit mask.  A warp instruction therefore covers 1 KiB
// of contiguous activations.  Grids are persistent (a multiple of the 148 SMs)
// and grid-stride.  When a pointer is not 32-byte aligned, or for the last
// n % 8 elements, the same functor runs its scalar form.
#include "common.cuh"

namespace mb {
namespace {

constexpr int kThreads = 256;
constexpr int kCtasPerSm = 8;

template <class Op>
__global__ void __launch_bounds__(kThreads) group_kernel(Op op, size_t full_groups, int tail,
                                                         bool vectorised) {
  const size_t stride = static_cast<size_t>(gridDim.x) * kThreads;
  size_t g = static_cast<size_t>(blockIdx.x) * kThreads + threadIdx.x;
  if (vectorised) {
    // two groups in flight per thread
    for (; g + stride < full_groups; g += 2 * stride) {
      op.vec2(g, g + stride);
    }
    if (g < full_groups) op.vec(g);
  } else {
    for (; g < full_groups; g += stride) op.scalar(g, 8);
  }
  if (tail && blockIdx.x == 0 && threadIdx.x == 0) op.scalar(full_groups, tail);
}

template <class Op>
int launch_groups(const char* name, Op op, size_t n, bool vectorised, void* stream) {
  if (n == 0) return MB_OK;
  const size_t full = n / 8;
  const int tail = static_cast<int>(n % 8);
  const int grid = grid_for(full, kThreads * 2, kCtasPerSm);
  group_kernel<Op><<<grid, kThreads, 0, as_stream(stream)>>>(op, full, tail, vectorised);
  return after_launch(name);
}

__device__ __forceinline__ float relu1(float x) { return x > 0.f ? x : (x != x ? x : 0.f); }

// ---------------------------------------------------------------- ReLU fwd
struct ReluFwd {
  const float* x;
  float* y;
  uint8_t* mask;  // may be null
  __device__ __forceinline__ uint32_t apply(f8& a) const {
    uint32_t bits = 0;
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      bits |= (a.v[k] > 0.f ? 1u : 0u) << (7 - k);
      a.v[k] = relu1(a.v[k]);
    }
    return bits;
  }
  __device__ __forceinline__ void vec(size_t g) const {
    f8 a = ld8(x + g * 8);
    uint32_t b = apply(a);
    st8(y + g * 8, a);
    if (mask) mask[g] = static_cast<uint8_t>(b);
  }
  __device__ __forceinline__ void vec2(size_t g0, size_t g1) const {
    f8 a = ld8(x + g0 * 8);
    f8 c = ld8(x + g1 * 8);
    uint32_t b0 = apply(a), b1 = apply(c);
    st8(y + g0 * 8, a);
    st8(y + g1 * 8, c);
    if (mask) {
      mask[g0] = static_cast<uint8_t>(b0);
      mask[g1] = static_cast<uint8_t>(b1);
    }
  }
  __device__ __forceinline__ void scalar(size_t g, int count) const {
    uint32_t bits = 0;
    for (int k = 0; k < count; ++k) {
      float v = x[g * 8 + k];
      bits |= (v > 0.f ? 1u : 0u) << (7 - k);
      y[g * 8 + k] = relu1(v);
    }
    if (mask) mask[g] = static_cast<uint8_t>(bits);
  }
};

// ------------------------------------------------------- ReLU bwd from mask
struct ReluBwdMask {
  const float* dy;
  const uint8_t* mask;
  float* dx;
  __device__ __forceinline__ void apply(f8& a, uint32_t bits) const {
#pragma unroll
    for (int k = 0; k < 8; ++k) a.v[k] = (bits >> (7 - k)) & 1u ? a.v[k] : 0.f;
  }
  __device__ __forceinline__ void vec(size_t g) const {
    f8 a = ld8(dy + g * 8);
    apply(a, mask[g]);
    st8(dx + g * 8, a);
  }
  __device__ __forceinline__ void vec2(size_t g0, size_t g1) const {
    f8 a = ld8(dy + g0 * 8);
    f8 c = ld8(dy + g1 * 8);
    uint32_t b0 = mask[g0], b1 = mask[g1];
    apply(a, b0);
    apply(c, b1);
    st8(dx + g0 * 8, a);
    st8(dx + g1 * 8, c);
  }
  __device__ __forceinline__ void scalar(size_t g, int count) const {
    uint32_t bits = mask[g];
    for (int k = 0; k < count; ++k) {
      float v = dy[g * 8 + k];
      dx[g * 8 + k] = (bits >> (7 - k)) & 1u ? v : 0.f;
    }
  }
};

// ------------------------------------ gated backward: ReLU-from-act, hardtanh
// dx = (lo < act && act < hi) ? dy : 0;  ReLU uses lo = threshold, hi = +inf.
// With dy2 != null the gradient is dy + dy2: a tensor read by two consumers gets its two
// incoming gradients summed and gated in one pass (16 bytes per element instead of 12 + 12).
struct GateBwd {
  const float* dy;
  const float* dy2;   // may be null
  const float* act;
  float* dx;
  float lo, hi;
  __device__ __forceinline__ void apply(f8& a, const f8& s) const {
#pragma unroll
    for (int k = 0; k < 8; ++k) a.v[k] = (s.v[k] > lo && s.v[k] < hi) ? a.v[k] : 0.f;
  }
  __device__ __forceinline__ void sum(f8& a, const f8& b) const {
#pragma unroll
    for (int k = 0; k < 8; ++k) a.v[k] += b.v[k];
  }
  __device__ __forceinline__ void vec(size_t g) const {
    f8 a = ld8(dy + g * 8);
    f8 s = ld8(act + g * 8);
    if (dy2) {
      f8 b = ld8(dy2 + g * 8);
      sum(a, b);
    }
    apply(a, s);
    st8(dx + g * 8, a);
  }
  __device__ __forceinline__ void vec2(size_t g0, size_t g1) const {
    f8 a = ld8(dy + g0 * 8);
    f8 s = ld8(act + g0 * 8);
    f8 c = ld8(dy + g1 * 8);
    f8 t = ld8(act + g1 * 8);
    if (dy2) {
      f8 b = ld8(dy2 + g0 * 8);
      f8 d = ld8(dy2 + g1 * 8);
      sum(a, b);
      sum(c, d);
    }
    apply(a, s);
    apply(c, t);
    st8(dx + g0 * 8, a);
    st8(dx + g1 * 8, c);
  }
  __device__ __forceinline__ void scalar(size_t g, int count) const {
    for (int k = 0; k < count; ++k) {
      float s = act[g * 8 + k];
      float v = dy[g * 8 + k];
      if (dy2) v += dy2[g * 8 + k];
      dx[g * 8 + k] = (s > lo && s < hi) ? v : 0.f;
    }
  }
};

// ------------------------------------------------------------ hardtanh fwd
struct ClampFwd {
  const float* x;
  float* y;
  float lo, hi;
  __device__ __forceinline__ float f(float v) const {
    return v != v ? v : fminf(fmaxf(v, lo), hi);
  }
  __device__ __forceinline__ void vec(size_t g) const {
    f8 a = ld8(x + g * 8);
#pragma unroll
    for (int k = 0; k < 8; ++k) a.v[k] = f(a.v[k]);
    st8(y + g * 8, a);
  }
  __device__ __forceinline__ void vec2(size_t g0, size_t g1) const {
    f8 a = ld8(x + g0 * 8);
    f8 c = ld8(x + g1 * 8);
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      a.v[k] = f(a.v[k]);
      c.v[k] = f(c.v[k]);
    }
    st8(y + g0 * 8, a);
    st8(y + g1 * 8, c);
  }
  __device__ __forceinline__ void scalar(size_t g, int count) const {
    for (int k = 0; k < count; ++k) y[g * 8 + k] = f(x[g * 8 + k]);
  }
};

// ---------------------------------------------------------- y = a + alpha*b
struct AxpyFwd {
  const float* a;
  const float* b;  // null: y = alpha * a
  float* y;
  float alpha;
  int relu;        // y = relu(a + alpha*b)
  __device__ __forceinline__ void vec(size_t g) const {
    f8 u = ld8(a + g * 8);
    if (b) {
      f8 w = ld8(b + g * 8);
#pragma unroll
      for (int k = 0; k < 8; ++k) u.v[k] = fmaf(alpha, w.v[k], u.v[k]);
    } else {
#pragma unroll
      for (int k = 0; k < 8; ++k) u.v[k] *= alpha;
    }
    if (relu) {
#pragma unroll
      for (int k = 0; k < 8; ++k) u.v[k] = relu1(u.v[k]);
    }
    st8(y + g * 8, u);
  }
  __device__ __forceinline__ void vec2(size_t g0, size_t g1) const {
    vec(g0);
    vec(g1);
  }
  __device__ __forceinline__ void scalar(size_t g, int count) const {
    for (int k = 0; k < count; ++k) {
      size_t i = g * 8 + k;
      const float v = b ? fmaf(alpha, b[i], a[i]) : alpha * a[i];
      y[i] = relu ? relu1(v) : v;
    }
  }
};

// ------------------------------------------------------------ stand-alone packers
// Group = 8 input bytes <-> 1 packed byte (bits) or 4 packed bytes (nibbles).
struct PackBits {
  const uint8_t* in;
  uint8_t* out;
  __device__ __forceinline__ void vec(size_t g) const {
    uint2 w = *reinterpret_cast<const uint2*>(in + g * 8);
    uint32_t bits = 0;
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      bits |= (((w.x >> (8 * k)) & 0xffu) ? 1u : 0u) << (7 - k);
      bits |= (((w.y >> (8 * k)) & 0xffu) ? 1u : 0u) << (3 - k);
    }
    out[g] = static_cast<uint8_t>(bits);
  }
  __device__ __forceinline__ void vec2(size_t g0, size_t g1) const {
    vec(g0);
    vec(g1);
  }
  __device__ __forceinline__ void scalar(size_t g, int count) const {
    uint32_t bits = 0;
    for (int k = 0; k < count; ++k) bits |= (in[g * 8 + k] ? 1u : 0u) << (7 - k);
    out[g] = static_cast<uint8_t>(bits);
  }
};

struct UnpackBits {
  const uint8_t* in;
  uint8_t* out;
  __device__ __forceinline__ void vec(size_t g) const {
    uint32_t bits = in[g];
    uint2 w = make_uint2(0, 0);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      w.x |= ((bits >> (7 - k)) & 1u) << (8 * k);
      w.y |= ((bits >> (3 - k)) & 1u) << (8 * k);
    }
    *reinterpret_cast<uint2*>(out + g * 8) = w;
  }
  __device__ __forceinline__ void vec2(size_t g0, size_t g1) const {
    vec(g0);
    vec(g1);
  }
  __device__ __forceinline__ void scalar(size_t g, int count) const {
    uint32_t bits = in[g];
    for (int k = 0; k < count; ++k) out[g * 8 + k] = (bits >> (7 - k)) & 1u;
  }
};

// Group = 8 unpacked bytes <-> 4 packed bytes.
struct PackNibbles {
  const uint8_t* in;
  uint8_t* out;
  __device__ __forceinline__ void vec(size_t g) const {
    uint2 w = *reinterpret_cast<const uint2*>(in + g * 8);
    uint32_t r = 0;
#pragma unroll
    for (int k = 0; k < 2; ++k) {
      uint32_t hi = (w.x >> (16 * k)) & 0xffu, lo = (w.x >> (16 * k + 8)) & 0xffu;
      r |= (((hi << 4) | lo) & 0xffu) << (8 * k);
      hi = (w.y >> (16 * k)) & 0xffu;
      lo = (w.y >> (16 * k + 8)) & 0xffu;
      r |= (((hi << 4) | lo) & 0xffu) << (8 * (k + 2));
    }
    *reinterpret_cast<uint32_t*>(out + g * 4) = r;
  }
  __device__ __forceinline__ void vec2(size_t g0, size_t g1) const {
    vec(g0);
    vec(g1);
  }
  __device__ __forceinline__ void scalar(size_t g, int count) const {
    for (int k = 0; k < count; k += 2) {
      uint32_t hi = in[g * 8 + k];
      uint32_t lo = (k + 1 < count) ? in[g * 8 + k + 1] : 0u;
      out[g * 4 + k / 2] = static_cast<uint8_t>((hi << 4) | lo);
    }
  }
};

struct UnpackNibbles {
  const uint8_t* in;
  uint8_t* out;
  __device__ __forceinline__ void vec(size_t g) const {
    uint32_t r = *reinterpret_cast<const uint32_t*>(in + g * 4);
    uint2 w = make_uint2(0, 0);
#pragma unroll
    for (int k = 0; k < 2; ++k) {
      uint32_t b = (r >> (8 * k)) & 0xffu;
      w.x |= ((b >> 4) & 15u) << (16 * k);
      w.x |= (b & 15u) << (16 * k + 8);
      b = (r >> (8 * (k + 2))) & 0xffu;
      w.y |= ((b >> 4) & 15u) << (16 * k);
      w.y |= (b & 15u) << (16 * k + 8);
    }
    *reinterpret_cast<uint2*>(out + g * 8) = w;
  }
  __device__ __forceinline__ void vec2(size_t g0, size_t g1) const {
    vec(g0);
    vec(g1);
  }
  __device__ __forceinline__ void scalar(size_t g, int count) const {
    for (int k = 0; k < count; ++k) {
      uint32_t b = in[g * 4 + k / 2];
      out[g * 8 + k] = (k & 1) ? (b & 15u) : ((b >> 4) & 15u);
    }
  }
};

inline bool null_arg(const void* p) { return p == nullptr; }

}  // namespace
}  // namespace mb

using namespace mb;

extern "C" {

int mb_relu_fwd(const float* x, float* y, size_t n, void* stream) {
  if (n && (null_arg(x) || null_arg(y))) return fail(MB_ERR_INVALID_ARGUMENT, "mb_relu_fwd: null pointer");
  bool v = aligned(x, 32) && aligned(y, 32);
  return launch_groups("relu_fwd", ReluFwd{x, y, nullptr}, n, v, stream);
}

int mb_relu_fwd_mask(const float* x, float* y, uint8_t* mask, size_t n, void* stream) {
  if (n && (null_arg(x) || null_arg(y) || null_arg(mask)))
    return fail(MB_ERR_INVALID_ARGUMENT, "mb_relu_fwd_mask: null pointer");
  bool v = aligned(x, 32) && aligned(y, 32);
  return launch_groups("relu_fwd_mask", ReluFwd{x, y, mask}, n, v, stream);
}

int mb_relu_bwd_mask(const float* dy, const uint8_t* mask, float* dx, size_t n, void* stream) {
  if (n && (null_arg(dy) || null_arg(dx) || null_arg(mask)))
    return fail(MB_ERR_INVALID_ARGUMENT, "mb_relu_bwd_mask: null pointer");
  bool v = aligned(dy, 32) && aligned(dx, 32);
  return launch_groups("relu_bwd_mask", ReluBwdMask{dy, mask, dx}, n, v, stream);
}

int mb_relu_bwd_act(const float* dy, const float* act, float threshold, float* dx, size_t n,
                    void* stream) {
  if (n && (null_arg(dy) || null_arg(dx) || null_arg(act)))
    return fail(MB_ERR_INVALID_ARGUMENT, "mb_relu_bwd_act: null pointer");
  bool v = aligned(dy, 32) && aligned(dx, 32) && aligned(act, 32);
  return launch_groups("relu_bwd_act", GateBwd{dy, nullptr, act, dx, threshold, __builtin_huge_valf()}, n,
                       v, stream);
}

int mb_hardtanh_fwd(const float* x, float* y, float lo, float hi, size_t n, void* stream) {
  if (n && (null_arg(x) || null_arg(y))) return fail(MB_ERR_INVALID_ARGUMENT, "mb_hardtanh_fwd: null pointer");
  if (!(lo <= hi)) return fail(MB_ERR_INVALID_ARGUMENT, "mb_hardtanh_fwd: lo > hi");
  bool v = aligned(x, 32) && aligned(y, 32);
  return launch_groups("hardtanh_fwd", ClampFwd{x, y, lo, hi}, n, v, stream);
}

int mb_hardtanh_bwd(const float* dy, const float* act, float lo, float hi, float* dx, size_t n,
                    void* stream) {
  if (n && (null_arg(dy) || null_arg(dx) || null_arg(act)))
    return fail(MB_ERR_INVALID_ARGUMENT, "mb_hardtanh_bwd: null pointer");
  bool v = aligned(dy, 32) && aligned(dx, 32) && aligned(act, 32);
  return launch_groups("hardtanh_bwd", GateBwd{dy, nullptr, act, dx, lo, hi}, n, v, stream);
}

int mb_add_fwd(const float* a, const float* b, float alpha, float* y, size_t n, void* stream) {
  if (n && (null_arg(a) || null_arg(b) || null_arg(y)))
    return fail(MB_ERR_INVALID_ARGUMENT, "mb_add_fwd: null pointer");
  bool v = aligned(a, 32) && aligned(b, 32) && aligned(y, 32);
  return launch_groups("add_fwd", AxpyFwd{a, b, y, alpha, 0}, n, v, stream);
}

int mb_add_relu_fwd(const float* a, const float* b, float alpha, float* y, size_t n, void* stream) {
  if (n && (null_arg(a) || null_arg(b) || null_arg(y)))
    return fail(MB_ERR_INVALID_ARGUMENT, "mb_add_relu_fwd: null pointer");
  bool v = aligned(a, 32) && aligned(b, 32) && aligned(y, 32);
  return launch_groups("add_relu_fwd", AxpyFwd{a, b, y, alpha, 1}, n, v, stream);
}

int mb_relu_bwd_act2(const float* dy1, const float* dy2, const float* act, float threshold,
                     float* dx, size_t n, void* stream) {
  if (n && (null_arg(dy1) || null_arg(dy2) || null_arg(dx) || null_arg(act)))
    return fail(MB_ERR_INVALID_ARGUMENT, "mb_relu_bwd_act2: null pointer");
  bool v = aligned(dy1, 32) && aligned(dy2, 32) && aligned(dx, 32) && aligned(act, 32);
  return launch_groups("relu_bwd_act2", GateBwd{dy1, dy2, act, dx, threshold, __builtin_huge_valf()},
                       n, v, stream);
}

int mb_scale(const float* x, float alpha, float* y, size_t n, void* stream) {
  if (n && (null_arg(x) || null_arg(y))) return fail(MB_ERR_INVALID_ARGUMENT, "mb_scale: null pointer");
  bool v = aligned(x, 32) && aligned(y, 32);
  return launch_groups("scale", AxpyFwd{x, nullptr, y, alpha, 0}, n, v, stream);
}

int mb_pack_bits(const uint8_t* in, uint8_t* out, size_t n, void* stream) {
  if (n && (null_arg(in) || null_arg(out))) return fail(MB_ERR_INVALID_ARGUMENT, "mb_pack_bits: null pointer");
  return launch_groups("pack_bits", PackBits{in, out}, n, aligned(in, 8), stream);
}

int mb_unpack_bits(const uint8_t* in, uint8_t* out, size_t n, void* stream) {
  if (n && (null_arg(in) || null_arg(out))) return fail(MB_ERR_INVALID_ARGUMENT, "mb_unpack_bits: null pointer");
  return launch_groups("unpack_bits", UnpackBits{in, out}, n, aligned(out, 8), stream);
}

int mb_unpack_multiply(const uint8_t* in, const float* v, float* out, size_t n, void* stream) {
  return mb_relu_bwd_mask(v, in, out, n, stream);
}

int mb_pack_nibbles(const uint8_t* in, uint8_t* out, size_t n, void* stream) {
  if (n && (null_arg(in) || null_arg(out))) return fail(MB_ERR_INVALID_ARGUMENT, "mb_pack_nibbles: null pointer");
  return launch_groups("pack_nibbles", PackNibbles{in, out}, n, aligned(in, 8) && aligned(out, 4), stream);
}

int mb_unpack_nibbles(const uint8_t* in, uint8_t* out, size_t n, void* stream) {
  if (n && (null_arg(in) || null_arg(out))) return fail(MB_ERR_INVALID_ARGUMENT, "mb_unpack_nibbles: null pointer");
  return launch_groups("unpack_nibbles", UnpackNibbles{in, out}, n, aligned(in, 4) && aligned(out, 8), stream);
}

}  // extern "C"
