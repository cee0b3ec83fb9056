// Max-pool forward writing values + packed 4-bit window-local argmax in one
// pass, and the backward that gathers straight from the nibbles (no unpacked
// index tensor, no memset of dx).
//
// Index semantics (maxpool.cu:38-70 of the reference): the stored index of a
// window's maximum at tap (i, j) is i*kw + j, counted from the UNCLIPPED window
// origin (ph*sh - pad, pw*sw - pad); strict '>' so the first maximum wins, and a
// NaN always wins.  A window whose taps are all -inf keeps the index of its
// first in-bounds tap (PyTorch's behaviour; the reference stores a truncated
// global offset there, which does not fit a nibble).
#include "common.cuh"

namespace mb {
namespace {

struct PoolP {
  int N, C, H, W, P, Q, kh, kw, sh, sw, ph, pw, dh, dw;
};

__device__ __forceinline__ bool better(float v, float best) { return v > best || v != v; }

// ---------------------------------------------------------------- NHWC fwd
// One thread = one output pixel x 8 channels: per tap two 128-bit loads, then a
// 256-bit value store and one 32-bit nibble store.  Consecutive threads walk the
// channel groups first, so a warp reads contiguous runs of C floats.
// KH/KW > 0 fix the window at compile time (dilation 1) so that the tap loops unroll.
template <int KH, int KW>
__global__ void __launch_bounds__(256) maxpool_fwd_nhwc8(const float* __restrict__ x,
                                                         float* __restrict__ y,
                                                         uint32_t* __restrict__ nib, PoolP p,
                                                         size_t total) {
  const int cg = p.C / 8;
  const int kh = KH ? KH : p.kh, kw = KW ? KW : p.kw;
  const int dh = KH ? 1 : p.dh, dw = KW ? 1 : p.dw;
  for (size_t t = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; t < total;
       t += static_cast<size_t>(gridDim.x) * blockDim.x) {
    int g, q, rest;
    split3(t, cg, p.Q, g, q, rest);
    const int n = rest / p.P, pp = rest - n * p.P;
    const int h0 = pp * p.sh - p.ph, w0 = q * p.sw - p.pw;
    float best[8];
    uint32_t idx[8];
    bool first = true;
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      best[k] = -INFINITY;
      idx[k] = 0;
    }
    const float* xn = x + static_cast<size_t>(n) * p.H * p.W * p.C + g * 8;
    if (KH > 0 && KW > 0) {
      // Compile-time window: every tap is loaded first, from a clamped (always valid) address,
      // and only then compared.  With the loads behind the bounds tests the compiler issued
      // them one by one and the kernel waited on each (long-scoreboard stalls, 0.6 of the HBM
      // roofline); issued together they overlap.
      float4 va[KH * KW > 0 ? KH * KW : 1], vb[KH * KW > 0 ? KH * KW : 1];
      bool ok[KH * KW > 0 ? KH * KW : 1];
#pragma unroll
      for (int i = 0; i < KH; ++i) {
        const int h = h0 + i;
        const int hc = h < 0 ? 0 : (h >= p.H ? p.H - 1 : h);
#pragma unroll
        for (int j = 0; j < KW; ++j) {
          const int w = w0 + j;
          const int wc = w < 0 ? 0 : (w >= p.W ? p.W - 1 : w);
          const float4* src =
              reinterpret_cast<const float4*>(xn + (static_cast<size_t>(hc) * p.W + wc) * p.C);
          va[i * KW + j] = __ldg(src);
          vb[i * KW + j] = __ldg(src + 1);
          ok[i * KW + j] = h == hc && w == wc;
        }
      }
#pragma unroll
      for (int tap = 0; tap < KH * KW; ++tap) {
        if (!ok[tap]) continue;
        const float4 a = va[tap], b = vb[tap];
        const float v[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          if (first) idx[k] = tap;
          if (better(v[k], best[k])) {
            best[k] = v[k];
            idx[k] = tap;
          }
        }
        first = false;
      }
    } else {
      for (int i = 0; i < kh; ++i) {
        const int h = h0 + i * dh;
        if (h < 0 || h >= p.H) continue;
        for (int j = 0; j < kw; ++j) {
          const int w = w0 + j * dw;
          if (w < 0 || w >= p.W) continue;
          const uint32_t local = i * kw + j;
          const float4* src =
              reinterpret_cast<const float4*>(xn + (static_cast<size_t>(h) * p.W + w) * p.C);
          const float4 a = __ldg(src), b = __ldg(src + 1);
          const float v[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
#pragma unroll
          for (int k = 0; k < 8; ++k) {
            if (first) idx[k] = local;
            if (better(v[k], best[k])) {
              best[k] = v[k];
              idx[k] = local;
            }
          }
          first = false;
        }
      }
    }
    f8 out;
#pragma unroll
    for (int k = 0; k < 8; ++k) out.v[k] = best[k];
    st8(y + t * 8, out);
    if (nib) {
      // element e = t*8+k -> byte e/2, even e in the high nibble
      uint32_t r = 0;
#pragma unroll
      for (int k = 0; k < 4; ++k) r |= (((idx[2 * k] << 4) | idx[2 * k + 1]) & 0xffu) << (8 * k);
      nib[t] = r;
    }
  }
}

// ---------------------------------------------------------------- NHWC bwd
// One thread = one INPUT pixel x 8 channels; loops over the windows covering it.
// KH/KW/SH/SW > 0 fix the window and stride at compile time (dilation 1): the tap loops
// unroll and the divisions by the stride become shifts; 0 takes them from `p`.
template <int KH, int KW, int SH, int SW>
__global__ void __launch_bounds__(256) maxpool_bwd_nhwc8(const float* __restrict__ dy,
                                                         const uint32_t* __restrict__ nib,
                                                         float* __restrict__ dx, PoolP p,
                                                         size_t total) {
  const int cg = p.C / 8;
  const int kh = KH ? KH : p.kh, kw = KW ? KW : p.kw;
  const int sh = SH ? SH : p.sh, sw = SW ? SW : p.sw;
  const int dh = KH ? 1 : p.dh, dw = KW ? 1 : p.dw;
  for (size_t t = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; t < total;
       t += static_cast<size_t>(gridDim.x) * blockDim.x) {
    int g, w, rest;
    split3(t, cg, p.W, g, w, rest);
    const int n = rest / p.H, h = rest - n * p.H;
    float acc[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) acc[k] = 0.f;
    // windows pp with pp*sh - ph + i*dh == h for some tap i in [0, kh)
#pragma unroll
    for (int i = 0; i < kh; ++i) {
      const int hn = h + p.ph - i * dh;
      if (hn < 0 || hn % sh) continue;
      const int pp = hn / sh;
      if (pp >= p.P) continue;
#pragma unroll
      for (int j = 0; j < kw; ++j) {
        const int wn = w + p.pw - j * dw;
        if (wn < 0 || wn % sw) continue;
        const int q = wn / sw;
        if (q >= p.Q) continue;
        const uint32_t local = i * kw + j;
        const size_t o = ((static_cast<size_t>(n) * p.P + pp) * p.Q + q) * cg + g;
        const uint32_t r = __ldg(nib + o);
        const float4* src = reinterpret_cast<const float4*>(dy + o * 8);
        const float4 a = __ldg(src), b = __ldg(src + 1);
        const float v[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          const uint32_t byte = (r >> (8 * (k / 2))) & 0xffu;
          const uint32_t stored = (k & 1) ? (byte & 15u) : (byte >> 4);
          if (stored == local) acc[k] += v[k];
        }
      }
    }
    f8 out;
#pragma unroll
    for (int k = 0; k < 8; ++k) out.v[k] = acc[k];
    st8(dx + t * 8, out);
  }
}

// ------------------------------------------- NHWC, 3x3 window, stride 2, pad 1
// The pooling of the ResNet stem, backward.  Windows overlap by one row and one column: a 2x2
// input quad (rows 2a, 2a+1; columns 2b, 2b+1) is covered by the windows (a, a+1) x (b, b+1)
// only, so a thread that owns a quad serves four pixels with four (gradient, nibble-word)
// loads (1 load per pixel instead of 2.25) and its stores are two 64-byte runs: 0.26 -> 0.13 ms
// on 184 x 64 x 112 x 112.  (The same sharing in the forward -- 2x2 outputs from one 5x5 patch,
// with 8 or with 4 channels per thread -- measured slower than one output per thread, 0.26 and
// 0.24 against 0.19 ms: the forward is read-dominated and L2 already absorbs the overlap, while
// the quad's registers cost occupancy.)
__global__ void __launch_bounds__(256) maxpool_bwd_3x3s2p1_quad(const float* __restrict__ dy,
                                                                const uint32_t* __restrict__ nib,
                                                                float* __restrict__ dx, PoolP p,
                                                                size_t total) {
  const int cg = p.C / 8, H2 = (p.H + 1) / 2, W2 = (p.W + 1) / 2;
  for (size_t t = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; t < total;
       t += static_cast<size_t>(gridDim.x) * blockDim.x) {
    int g, b, rest;
    split3(t, cg, W2, g, b, rest);
    const int n = rest / H2, a = rest - n * H2;
    float acc[2][2][8];
#pragma unroll
    for (int u = 0; u < 2; ++u)
#pragma unroll
      for (int v = 0; v < 2; ++v)
#pragma unroll
        for (int k = 0; k < 8; ++k) acc[u][v][k] = 0.f;
    // window (a + wu, b + wv) starts at row 2(a+wu) - 1, column 2(b+wv) - 1: quad pixel (u, v)
    // (row 2a + u, column 2b + v) is its tap (1 + u - 2 wu, 1 + v - 2 wv) when that is in 0..2
#pragma unroll
    for (int wu = 0; wu < 2; ++wu) {
      const int pp = a + wu;
      if (pp >= p.P) continue;
#pragma unroll
      for (int wv = 0; wv < 2; ++wv) {
        const int q = b + wv;
        if (q >= p.Q) continue;
        const size_t o = ((static_cast<size_t>(n) * p.P + pp) * p.Q + q) * cg + g;
        const uint32_t w32 = __ldg(nib + o);
        const float4* src = reinterpret_cast<const float4*>(dy + o * 8);
        const float4 fa = __ldg(src), fb = __ldg(src + 1);
        const float val[8] = {fa.x, fa.y, fa.z, fa.w, fb.x, fb.y, fb.z, fb.w};
#pragma unroll
        for (int u = wu; u < 2; ++u) {            // wu == 1 reaches row u = 1 only (tap row 0)
          const int i = 1 + u - 2 * wu;
#pragma unroll
          for (int v = wv; v < 2; ++v) {
            const int j = 1 + v - 2 * wv;
            const uint32_t local = i * 3 + j;
#pragma unroll
            for (int k = 0; k < 8; ++k) {
              const uint32_t byte = (w32 >> (8 * (k / 2))) & 0xffu;
              const uint32_t stored = (k & 1) ? (byte & 15u) : (byte >> 4);
              if (stored == local) acc[u][v][k] += val[k];
            }
          }
        }
      }
    }
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      const int h = 2 * a + u;
      if (h >= p.H) continue;
#pragma unroll
      for (int v = 0; v < 2; ++v) {
        const int w = 2 * b + v;
        if (w >= p.W) continue;
        f8 out;
#pragma unroll
        for (int k = 0; k < 8; ++k) out.v[k] = acc[u][v][k];
        st8(dx + (((static_cast<size_t>(n) * p.H + h) * p.W + w) * cg + g) * 8, out);
      }
    }
  }
}

// ------------------------------------------------- generic (NCHW or NHWC) fwd
// One thread = two consecutive output elements (one packed byte).
template <bool NHWC>
__global__ void __launch_bounds__(256) maxpool_fwd_generic(const float* __restrict__ x,
                                                           float* __restrict__ y,
                                                           uint8_t* __restrict__ nib, PoolP p,
                                                           size_t total_out) {
  const size_t pairs = (total_out + 1) / 2;
  for (size_t t = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; t < pairs;
       t += static_cast<size_t>(gridDim.x) * blockDim.x) {
    uint32_t packed = 0;
    for (int s = 0; s < 2; ++s) {
      const size_t e = 2 * t + s;
      if (e >= total_out) break;
      int n, c, pp, q;
      size_t r = e;
      if (NHWC) {
        c = static_cast<int>(r % p.C); r /= p.C;
        q = static_cast<int>(r % p.Q); r /= p.Q;
        pp = static_cast<int>(r % p.P);
        n = static_cast<int>(r / p.P);
      } else {
        q = static_cast<int>(r % p.Q); r /= p.Q;
        pp = static_cast<int>(r % p.P); r /= p.P;
        c = static_cast<int>(r % p.C);
        n = static_cast<int>(r / p.C);
      }
      const int h0 = pp * p.sh - p.ph, w0 = q * p.sw - p.pw;
      float best = -INFINITY;
      uint32_t idx = 0;
      bool first = true;
      for (int i = 0; i < p.kh; ++i) {
        const int h = h0 + i * p.dh;
        if (h < 0 || h >= p.H) continue;
        for (int j = 0; j < p.kw; ++j) {
          const int w = w0 + j * p.dw;
          if (w < 0 || w >= p.W) continue;
          const size_t off = NHWC ? ((static_cast<size_t>(n) * p.H + h) * p.W + w) * p.C + c
                                  : ((static_cast<size_t>(n) * p.C + c) * p.H + h) * p.W + w;
          const float v = __ldg(x + off);
          const uint32_t local = i * p.kw + j;
          if (first) { idx = local; first = false; }
          if (better(v, best)) { best = v; idx = local; }
        }
      }
      y[e] = best;
      packed |= (idx & 15u) << (s == 0 ? 4 : 0);
    }
    if (nib) nib[t] = static_cast<uint8_t>(packed);
  }
}

template <bool NHWC>
__global__ void __launch_bounds__(256) maxpool_bwd_generic(const float* __restrict__ dy,
                                                           const uint8_t* __restrict__ nib,
                                                           float* __restrict__ dx, PoolP p,
                                                           size_t total_in) {
  for (size_t e = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; e < total_in;
       e += static_cast<size_t>(gridDim.x) * blockDim.x) {
    int n, c, h, w;
    size_t r = e;
    if (NHWC) {
      c = static_cast<int>(r % p.C); r /= p.C;
      w = static_cast<int>(r % p.W); r /= p.W;
      h = static_cast<int>(r % p.H);
      n = static_cast<int>(r / p.H);
    } else {
      w = static_cast<int>(r % p.W); r /= p.W;
      h = static_cast<int>(r % p.H); r /= p.H;
      c = static_cast<int>(r % p.C);
      n = static_cast<int>(r / p.C);
    }
    float acc = 0.f;
    for (int i = 0; i < p.kh; ++i) {
      const int hn = h + p.ph - i * p.dh;
      if (hn < 0 || hn % p.sh) continue;
      const int pp = hn / p.sh;
      if (pp >= p.P) continue;
      for (int j = 0; j < p.kw; ++j) {
        const int wn = w + p.pw - j * p.dw;
        if (wn < 0 || wn % p.sw) continue;
        const int q = wn / p.sw;
        if (q >= p.Q) continue;
        const size_t o = NHWC ? ((static_cast<size_t>(n) * p.P + pp) * p.Q + q) * p.C + c
                              : ((static_cast<size_t>(n) * p.C + c) * p.P + pp) * p.Q + q;
        const uint32_t byte = __ldg(nib + (o >> 1));
        const uint32_t stored = (o & 1) ? (byte & 15u) : (byte >> 4);
        if (stored == static_cast<uint32_t>(i * p.kw + j)) acc += __ldg(dy + o);
      }
    }
    dx[e] = acc;
  }
}

int check_desc(const char* who, const mb_pool_desc* d, PoolP* p) {
  if (!d) return fail(MB_ERR_INVALID_ARGUMENT, "%s: null descriptor", who);
  if (d->N < 0 || d->C <= 0 || d->H <= 0 || d->W <= 0 || d->P <= 0 || d->Q <= 0)
    return fail(MB_ERR_INVALID_ARGUMENT, "%s: bad extent N=%d C=%d H=%d W=%d P=%d Q=%d", who, d->N,
                d->C, d->H, d->W, d->P, d->Q);
  if (d->kh <= 0 || d->kw <= 0 || d->sh <= 0 || d->sw <= 0 || d->dh <= 0 || d->dw <= 0 ||
      d->ph < 0 || d->pw < 0)
    return fail(MB_ERR_INVALID_ARGUMENT, "%s: bad window parameters", who);
  if (d->kh * d->kw > 16)
    return fail(MB_ERR_UNSUPPORTED, "%s: window %dx%d does not fit a 4-bit index", who, d->kh, d->kw);
  if (d->layout != MB_NCHW && d->layout != MB_NHWC)
    return fail(MB_ERR_INVALID_ARGUMENT, "%s: bad layout %d", who, d->layout);
  // every window must contain at least one in-bounds tap
  if ((d->P - 1) * d->sh - d->ph >= d->H || (d->Q - 1) * d->sw - d->pw >= d->W)
    return fail(MB_ERR_INVALID_ARGUMENT, "%s: output extent too large for the input", who);
  *p = PoolP{d->N, d->C, d->H, d->W, d->P, d->Q, d->kh, d->kw, d->sh, d->sw, d->ph, d->pw, d->dh, d->dw};
  return MB_OK;
}

}  // namespace
}  // namespace mb

using namespace mb;

extern "C" {

int mb_pool_out_size(int in, int k, int s, int p, int d, int ceil_mode) {
  if (s <= 0) return -1;
  long num = static_cast<long>(in) + 2L * p - static_cast<long>(d) * (k - 1) - 1 + (ceil_mode ? s - 1 : 0);
  long out = (num >= 0 ? num / s : -((-num + s - 1) / s)) + 1;
  if (ceil_mode && (out - 1) * s >= static_cast<long>(in) + p) --out;  // last window must start inside
  return static_cast<int>(out);
}

int mb_maxpool2d_fwd(const float* x, float* y, uint8_t* nibbles, const mb_pool_desc* d,
                     void* stream) {
  PoolP p;
  int rc = check_desc("mb_maxpool2d_fwd", d, &p);
  if (rc) return rc;
  const size_t total_out = static_cast<size_t>(p.N) * p.C * p.P * p.Q;
  if (total_out == 0) return MB_OK;
  if (!x || !y) return fail(MB_ERR_INVALID_ARGUMENT, "mb_maxpool2d_fwd: null pointer");
  if (d->layout == MB_NHWC && p.C % 8 == 0 && aligned(x, 16) && aligned(y, 32) &&
      aligned(nibbles, 4)) {
    const size_t total = total_out / 8;
    uint32_t* nw = reinterpret_cast<uint32_t*>(nibbles);
    const int grid = grid_for(total, 256, 8);
    const bool unit_dil = p.dh == 1 && p.dw == 1;
    if (unit_dil && p.kh == 3 && p.kw == 3)
      maxpool_fwd_nhwc8<3, 3><<<grid, 256, 0, as_stream(stream)>>>(x, y, nw, p, total);
    else if (unit_dil && p.kh == 2 && p.kw == 2)
      maxpool_fwd_nhwc8<2, 2><<<grid, 256, 0, as_stream(stream)>>>(x, y, nw, p, total);
    else
      maxpool_fwd_nhwc8<0, 0><<<grid, 256, 0, as_stream(stream)>>>(x, y, nw, p, total);
    return after_launch("maxpool_fwd_nhwc8");
  }
  const size_t pairs = (total_out + 1) / 2;
  if (d->layout == MB_NHWC)
    maxpool_fwd_generic<true><<<grid_for(pairs, 256, 8), 256, 0, as_stream(stream)>>>(x, y, nibbles, p, total_out);
  else
    maxpool_fwd_generic<false><<<grid_for(pairs, 256, 8), 256, 0, as_stream(stream)>>>(x, y, nibbles, p, total_out);
  return after_launch("maxpool_fwd_generic");
}

int mb_maxpool2d_bwd(const float* dy, const uint8_t* nibbles, float* dx, const mb_pool_desc* d,
                     void* stream) {
  PoolP p;
  int rc = check_desc("mb_maxpool2d_bwd", d, &p);
  if (rc) return rc;
  const size_t total_in = static_cast<size_t>(p.N) * p.C * p.H * p.W;
  if (total_in == 0) return MB_OK;
  if (!dy || !dx || !nibbles) return fail(MB_ERR_INVALID_ARGUMENT, "mb_maxpool2d_bwd: null pointer");
  if (d->layout == MB_NHWC && p.C % 8 == 0 && aligned(dy, 16) && aligned(dx, 32) &&
      aligned(nibbles, 4)) {
    const size_t total = total_in / 8;
    const uint32_t* nw = reinterpret_cast<const uint32_t*>(nibbles);
    const int grid = grid_for(total, 256, 8);
    const bool unit_dil = p.dh == 1 && p.dw == 1;
    if (unit_dil && p.kh == 3 && p.kw == 3 && p.sh == 2 && p.sw == 2 && p.ph == 1 && p.pw == 1) {
      const size_t quads = static_cast<size_t>(p.N) * ((p.H + 1) / 2) * ((p.W + 1) / 2) * (p.C / 8);
      maxpool_bwd_3x3s2p1_quad<<<grid_for(quads, 256, 8), 256, 0, as_stream(stream)>>>(dy, nw, dx, p, quads);
      return after_launch("maxpool_bwd_3x3s2p1_quad");
    }
    if (unit_dil && p.kh == 3 && p.kw == 3 && p.sh == 2 && p.sw == 2)
      maxpool_bwd_nhwc8<3, 3, 2, 2><<<grid, 256, 0, as_stream(stream)>>>(dy, nw, dx, p, total);
    else if (unit_dil && p.kh == 2 && p.kw == 2 && p.sh == 2 && p.sw == 2)
      maxpool_bwd_nhwc8<2, 2, 2, 2><<<grid, 256, 0, as_stream(stream)>>>(dy, nw, dx, p, total);
    else
      maxpool_bwd_nhwc8<0, 0, 0, 0><<<grid, 256, 0, as_stream(stream)>>>(dy, nw, dx, p, total);
    return after_launch("maxpool_bwd_nhwc8");
  }
  if (d->layout == MB_NHWC)
    maxpool_bwd_generic<true><<<grid_for(total_in, 256, 8), 256, 0, as_stream(stream)>>>(dy, nibbles, dx, p, total_in);
  else
    maxpool_bwd_generic<false><<<grid_for(total_in, 256, 8), 256, 0, as_stream(stream)>>>(dy, nibbles, dx, p, total_in);
  return after_launch("maxpool_bwd_generic");
}

}  // extern "C"
