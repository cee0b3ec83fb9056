// Shared host/device helpers for libmonet_b200 (sm_100a only).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>
#include <stddef.h>
#include "../../include/monet_b200.h"

namespace mb {

// SM count of the current device (cudaDevAttrMultiProcessorCount, cached per device; 148 on a
// B200, which is also the answer when no device can be queried, e.g. a workspace-size call on a
// machine without a GPU).  Grids of grid-stride and persistent kernels are sized from it.
int num_sms();

// Records a printf-style message for mb_last_error() and returns `code`.
int fail(int code, const char* fmt, ...);
// Counts the launch, then turns cudaGetLastError() into a status.
int after_launch(const char* kernel_name);

inline cudaStream_t as_stream(void* s) { return reinterpret_cast<cudaStream_t>(s); }

inline bool aligned(const void* p, size_t a) { return (reinterpret_cast<uintptr_t>(p) & (a - 1)) == 0; }

// Grid for a grid-stride kernel over `work_items` items handled `per_block`
// at a time: enough CTAs to cover the work, capped at `waves` CTAs per SM.
inline int grid_for(size_t work_items, size_t per_block, int ctas_per_sm) {
  size_t need = (work_items + per_block - 1) / per_block;
  size_t cap = static_cast<size_t>(num_sms()) * ctas_per_sm;
  if (need < 1) need = 1;
  return static_cast<int>(need < cap ? need : cap);
}

// Decompose a flat work-item index t = (rest * d1 + i1) * d0 + i0.  Indices below 2^32 take
// 32-bit divisions: a 64-bit division costs several times as many instructions, and the
// stencil kernels (pooling, depthwise) are bound by instruction issue rather than by memory.
__device__ __forceinline__ void split3(size_t t, int d0, int d1, int& i0, int& i1, int& rest) {
  if (t <= 0xffffffffull) {
    const unsigned u = static_cast<unsigned>(t), ud0 = static_cast<unsigned>(d0), ud1 = static_cast<unsigned>(d1);
    const unsigned r1 = u / ud0, r2 = r1 / ud1;
    i0 = static_cast<int>(u - r1 * ud0);
    i1 = static_cast<int>(r1 - r2 * ud1);
    rest = static_cast<int>(r2);
  } else {
    const size_t r1 = t / d0, r2 = r1 / d1;
    i0 = static_cast<int>(t - r1 * d0);
    i1 = static_cast<int>(r1 - r2 * d1);
    rest = static_cast<int>(r2);
  }
}

// ---- 256-bit global accesses (8 floats per thread per instruction) --------
struct f8 { float v[8]; };

__device__ __forceinline__ f8 ld8_stream(const float* p) {
  f8 r;
  asm volatile("ld.global.nc.L1::no_allocate.v8.f32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
               : "=f"(r.v[0]), "=f"(r.v[1]), "=f"(r.v[2]), "=f"(r.v[3]), "=f"(r.v[4]),
                 "=f"(r.v[5]), "=f"(r.v[6]), "=f"(r.v[7])
               : "l"(p));
  return r;
}
// Same, through the coherent path: for buffers the kernel may also write
// (in-place operation), where the read-only path is not allowed.
__device__ __forceinline__ f8 ld8(const float* p) {
  f8 r;
  asm volatile("ld.global.L1::no_allocate.v8.f32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
               : "=f"(r.v[0]), "=f"(r.v[1]), "=f"(r.v[2]), "=f"(r.v[3]), "=f"(r.v[4]),
                 "=f"(r.v[5]), "=f"(r.v[6]), "=f"(r.v[7])
               : "l"(p)
               : "memory");
  return r;
}
__device__ __forceinline__ void st8(float* p, const f8& r) {
  asm volatile("st.global.v8.f32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"l"(p), "f"(r.v[0]),
               "f"(r.v[1]), "f"(r.v[2]), "f"(r.v[3]), "f"(r.v[4]), "f"(r.v[5]), "f"(r.v[6]),
               "f"(r.v[7])
               : "memory");
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

}  // namespace mb
