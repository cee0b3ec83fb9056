"""Tensor-level wrappers over the C ABI: allocation (through PyTorch's caching
allocator, so the reference's memory profiler sees every byte), layout detection,
stream selection and argument checking.  CUDA tensors only: a CPU tensor raises.

Layouts.  A logical N x C x H x W activation may be dense NCHW (``is_contiguous()``)
or dense NHWC (``torch.channels_last``).  Element-wise kernels work on the physical
buffer and keep the input's strides; layout-aware kernels (batch norm, pooling) get
the layout flag.  Anything else is first made contiguous.
"""
from __future__ import annotations

import ctypes as C

import torch

from . import _lib
from ._lib import MB_NCHW, MB_NHWC, BnDesc, PoolDesc, check, lib


# torch.cuda.current_stream() costs ~5 us of Python per call (device-index lookups, a Stream
# object); the raw handle of the current stream is one C call.
_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)
_cur_device = getattr(torch._C, "_cuda_getDevice", None)


def _stream() -> int:
    if _raw_stream is not None and _cur_device is not None:
        return _raw_stream(_cur_device())
    return torch.cuda.current_stream().cuda_stream


def _need_cuda(*tensors) -> None:
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise RuntimeError("monet_b200 operators run on CUDA tensors only (no CPU fallback)")
        if t is not None and t.dtype not in (torch.float32, torch.uint8, torch.int64, torch.bool):
            raise RuntimeError(f"monet_b200: unsupported dtype {t.dtype}")


def is_nhwc(t: torch.Tensor) -> bool:
    return (t.dim() == 4 and not t.is_contiguous()
            and t.is_contiguous(memory_format=torch.channels_last))


def dense(t: torch.Tensor) -> torch.Tensor:
    """`t` itself if it is dense NCHW / NHWC, else a contiguous copy."""
    if t.is_contiguous() or is_nhwc(t):
        return t
    return t.contiguous()


def layout_of(t: torch.Tensor) -> int:
    return MB_NHWC if is_nhwc(t) else MB_NCHW


def like(t: torch.Tensor, other: torch.Tensor) -> torch.Tensor:
    """`other` re-laid out, if needed, to share `t`'s physical element order."""
    other = dense(other)
    if other.dim() == 4 and t.dim() == 4 and layout_of(other) != layout_of(t):
        fmt = torch.channels_last if is_nhwc(t) else torch.contiguous_format
        other = other.contiguous(memory_format=fmt)
    return other


def _f32(t: torch.Tensor, name: str) -> None:
    if t.dtype != torch.float32:
        raise RuntimeError(f"monet_b200: {name} must be float32, got {t.dtype}")


# --------------------------------------------------------------------------- ReLU

def relu(x: torch.Tensor, inplace: bool = False) -> torch.Tensor:
    _need_cuda(x); _f32(x, "x")
    xd = dense(x)
    y = xd if (inplace and xd is x) else torch.empty_like(xd)
    check(lib().mb_relu_fwd(xd.data_ptr(), y.data_ptr(), xd.numel(), _stream()), "relu_fwd")
    return y


def relu_mask(x: torch.Tensor, inplace: bool = False):
    """(relu(x), 1-bit mask of x > 0 in physical element order, MSB first)."""
    _need_cuda(x); _f32(x, "x")
    xd = dense(x)
    y = xd if (inplace and xd is x) else torch.empty_like(xd)
    n = xd.numel()
    mask = torch.empty((n + 7) // 8, dtype=torch.uint8, device=x.device)
    check(lib().mb_relu_fwd_mask(xd.data_ptr(), y.data_ptr(), mask.data_ptr(), n, _stream()),
          "relu_fwd_mask")
    return y, mask


def relu_bwd_mask(dy: torch.Tensor, mask: torch.Tensor, inplace: bool = True) -> torch.Tensor:
    _need_cuda(dy, mask); _f32(dy, "dy")
    d = dense(dy)
    n = d.numel()
    if mask.dtype != torch.uint8 or mask.numel() != (n + 7) // 8:
        raise RuntimeError("monet_b200: mask size does not match the gradient")
    dx = d if inplace else torch.empty_like(d)
    check(lib().mb_relu_bwd_mask(d.data_ptr(), mask.data_ptr(), dx.data_ptr(), n, _stream()),
          "relu_bwd_mask")
    return dx


def relu_bwd_act(dy: torch.Tensor, act: torch.Tensor, threshold: float = 0.0,
                 inplace: bool = True) -> torch.Tensor:
    _need_cuda(dy, act); _f32(dy, "dy"); _f32(act, "act")
    a = dense(act)
    d = like(a, dy)
    if d.shape != a.shape:
        raise RuntimeError("monet_b200: gradient and activation shapes differ")
    dx = d if inplace else torch.empty_like(d)
    check(lib().mb_relu_bwd_act(d.data_ptr(), a.data_ptr(), float(threshold), dx.data_ptr(),
                                d.numel(), _stream()), "relu_bwd_act")
    return dx


def relu_bwd_act2(dy1: torch.Tensor, dy2: torch.Tensor, act: torch.Tensor,
                  threshold: float = 0.0) -> torch.Tensor:
    """(dy1 + dy2) gated by act > threshold, written over dy1 (or a dense copy of it)."""
    _need_cuda(dy1, dy2, act); _f32(dy1, "dy1"); _f32(dy2, "dy2"); _f32(act, "act")
    a = dense(act)
    d1 = like(a, dy1)
    d2 = like(a, dy2)
    if d1.shape != a.shape or d2.shape != a.shape:
        raise RuntimeError("monet_b200: gradient and activation shapes differ")
    check(lib().mb_relu_bwd_act2(d1.data_ptr(), d2.data_ptr(), a.data_ptr(), float(threshold),
                                 d1.data_ptr(), d1.numel(), _stream()), "relu_bwd_act2")
    return d1


# ------------------------------------------------------------------------ packing

def pack_bits(flags: torch.Tensor) -> torch.Tensor:
    _need_cuda(flags)
    src = flags.contiguous().view(-1)
    src = src.view(torch.uint8) if src.dtype == torch.bool else src
    n = src.numel()
    out = torch.empty((n + 7) // 8, dtype=torch.uint8, device=flags.device)
    check(lib().mb_pack_bits(src.data_ptr(), out.data_ptr(), n, _stream()), "pack_bits")
    return out


def unpack_bits(packed: torch.Tensor, n: int) -> torch.Tensor:
    _need_cuda(packed)
    out = torch.empty(n, dtype=torch.uint8, device=packed.device)
    check(lib().mb_unpack_bits(packed.data_ptr(), out.data_ptr(), n, _stream()), "unpack_bits")
    return out.view(torch.bool)


def unpack_multiply(packed: torch.Tensor, v: torch.Tensor) -> torch.Tensor:
    return relu_bwd_mask(v, packed, inplace=False)


def pack_nibbles(idx: torch.Tensor) -> torch.Tensor:
    _need_cuda(idx)
    src = idx.contiguous().view(-1)
    n = src.numel()
    out = torch.empty((n + 1) // 2, dtype=torch.uint8, device=idx.device)
    check(lib().mb_pack_nibbles(src.data_ptr(), out.data_ptr(), n, _stream()), "pack_nibbles")
    return out


def unpack_nibbles(packed: torch.Tensor, n: int) -> torch.Tensor:
    _need_cuda(packed)
    out = torch.empty(n, dtype=torch.uint8, device=packed.device)
    check(lib().mb_unpack_nibbles(packed.data_ptr(), out.data_ptr(), n, _stream()),
          "unpack_nibbles")
    return out


# ----------------------------------------------------------------------- hardtanh

def hardtanh(x: torch.Tensor, lo: float, hi: float, inplace: bool = False) -> torch.Tensor:
    _need_cuda(x); _f32(x, "x")
    xd = dense(x)
    y = xd if (inplace and xd is x) else torch.empty_like(xd)
    check(lib().mb_hardtanh_fwd(xd.data_ptr(), y.data_ptr(), float(lo), float(hi), xd.numel(),
                                _stream()), "hardtanh_fwd")
    return y


def hardtanh_bwd(dy: torch.Tensor, act: torch.Tensor, lo: float, hi: float,
                 inplace: bool = False) -> torch.Tensor:
    _need_cuda(dy, act); _f32(dy, "dy"); _f32(act, "act")
    a = dense(act)
    d = like(a, dy)
    dx = d if inplace else torch.empty_like(d)
    check(lib().mb_hardtanh_bwd(d.data_ptr(), a.data_ptr(), float(lo), float(hi), dx.data_ptr(),
                                d.numel(), _stream()), "hardtanh_bwd")
    return dx


# ---------------------------------------------------------------------------- add

def add(a: torch.Tensor, b: torch.Tensor, alpha: float = 1.0, inplace: bool = False):
    _need_cuda(a, b); _f32(a, "a"); _f32(b, "b")
    if a.shape != b.shape:
        raise RuntimeError("monet_b200.add: broadcasting is not supported")
    ad = dense(a)
    bd = like(ad, b)
    y = ad if (inplace and ad is a) else torch.empty_like(ad)
    check(lib().mb_add_fwd(ad.data_ptr(), bd.data_ptr(), float(alpha), y.data_ptr(), ad.numel(),
                           _stream()), "add_fwd")
    return y


def add_relu(a: torch.Tensor, b: torch.Tensor, alpha: float = 1.0, inplace: bool = False):
    """relu(a + alpha * b) in one pass."""
    _need_cuda(a, b); _f32(a, "a"); _f32(b, "b")
    if a.shape != b.shape:
        raise RuntimeError("monet_b200.add_relu: broadcasting is not supported")
    ad = dense(a)
    bd = like(ad, b)
    y = ad if (inplace and ad is a) else torch.empty_like(ad)
    check(lib().mb_add_relu_fwd(ad.data_ptr(), bd.data_ptr(), float(alpha), y.data_ptr(),
                                ad.numel(), _stream()), "add_relu_fwd")
    return y


def add_channel_bias(y: torch.Tensor, bias: torch.Tensor) -> torch.Tensor:
    """y + bias[c], in place on a dense 4-D activation (the cached-statistics batch-norm sweep
    with mean 0, scale 1: one 8 B/element pass)."""
    _need_cuda(y, bias); _f32(y, "y"); _f32(bias, "bias")
    Cc = int(y.shape[1])
    yd = dense(y)
    one = torch.ones(Cc, dtype=y.dtype, device=y.device)
    zero = torch.zeros(Cc, dtype=y.dtype, device=y.device)
    return bn_fwd_apply(yd, one, bias.contiguous(), zero, one, inplace=True)


def scale(x: torch.Tensor, alpha: float) -> torch.Tensor:
    _need_cuda(x); _f32(x, "x")
    xd = dense(x)
    y = torch.empty_like(xd)
    check(lib().mb_scale(xd.data_ptr(), float(alpha), y.data_ptr(), xd.numel(), _stream()),
          "scale")
    return y


# ----------------------------------------------------------------------- max pool

def _pair(v):
    if isinstance(v, (list, tuple)):
        return (int(v[0]), int(v[0])) if len(v) == 1 else (int(v[0]), int(v[1]))
    return int(v), int(v)


def pool_desc(shape, layout, kernel_size, stride, padding, dilation, ceil_mode) -> PoolDesc:
    kh, kw = _pair(kernel_size)
    sh, sw = _pair(stride) if stride not in (None, [], ()) else (kh, kw)
    ph, pw = _pair(padding)
    dh, dw = _pair(dilation)
    N, Cc, H, W = (int(s) for s in shape)
    L = lib()
    P = L.mb_pool_out_size(H, kh, sh, ph, dh, int(bool(ceil_mode)))
    Q = L.mb_pool_out_size(W, kw, sw, pw, dw, int(bool(ceil_mode)))
    return PoolDesc(N, Cc, H, W, P, Q, kh, kw, sh, sw, ph, pw, dh, dw, layout)


def _out_4d(x: torch.Tensor, N, Cc, P, Q, layout) -> torch.Tensor:
    fmt = torch.channels_last if layout == MB_NHWC else torch.contiguous_format
    return torch.empty((N, Cc, P, Q), dtype=x.dtype, device=x.device, memory_format=fmt)


def maxpool2d(x: torch.Tensor, kernel_size, stride, padding, dilation, ceil_mode,
              with_indices: bool = True):
    """(y, packed 4-bit window-local argmax or None, descriptor)."""
    _need_cuda(x); _f32(x, "x")
    if x.dim() != 4:
        raise RuntimeError("monet_b200.maxpool2d expects a 4-D tensor")
    xd = dense(x)
    d = pool_desc(xd.shape, layout_of(xd), kernel_size, stride, padding, dilation, ceil_mode)
    if d.P <= 0 or d.Q <= 0:
        raise RuntimeError("monet_b200.maxpool2d: empty output")
    y = _out_4d(xd, d.N, d.C, d.P, d.Q, d.layout)
    nib = None
    if with_indices:
        nib = torch.empty((y.numel() + 1) // 2, dtype=torch.uint8, device=x.device)
    check(lib().mb_maxpool2d_fwd(xd.data_ptr(), y.data_ptr(), nib.data_ptr() if nib is not None else None,
                                 C.byref(d), _stream()), "maxpool2d_fwd")
    return y, nib, d


def maxpool2d_bwd(dy: torch.Tensor, nibbles: torch.Tensor, d: PoolDesc) -> torch.Tensor:
    _need_cuda(dy, nibbles); _f32(dy, "dy")
    fmt = torch.channels_last if d.layout == MB_NHWC else torch.contiguous_format
    dyd = dy.contiguous(memory_format=fmt)
    if tuple(dyd.shape) != (d.N, d.C, d.P, d.Q):
        raise RuntimeError("monet_b200.maxpool2d_bwd: gradient shape does not match the forward")
    dx = _out_4d(dyd, d.N, d.C, d.H, d.W, d.layout)
    check(lib().mb_maxpool2d_bwd(dyd.data_ptr(), nibbles.data_ptr(), dx.data_ptr(), C.byref(d),
                                 _stream()), "maxpool2d_bwd")
    return dx


# --------------------------------------------------------------------- batch norm

def bn_desc(x: torch.Tensor, eps: float, momentum: float) -> BnDesc:
    if x.dim() < 2:
        raise RuntimeError("monet_b200 batch norm expects at least 2 dimensions")
    N, Cc = int(x.shape[0]), int(x.shape[1])
    HW = 1
    for s in x.shape[2:]:
        HW *= int(s)
    layout = MB_NHWC if (x.dim() == 4 and is_nhwc(x)) else MB_NCHW
    return BnDesc(N, Cc, HW, layout, float(eps), float(momentum if momentum is not None else 0.1))


def _bn_dense(x: torch.Tensor) -> torch.Tensor:
    if x.dim() == 4:
        return dense(x)
    return x.contiguous()


def _bn_workspace(d: BnDesc, device) -> torch.Tensor:
    nbytes = lib().mb_bn_workspace_bytes(C.byref(d))
    return torch.empty(nbytes, dtype=torch.uint8, device=device)


def bn_fwd_train(x, gamma, beta, running_mean, running_var, momentum, eps, inplace=False):
    """(y, save_mean, save_invstd); updates the running statistics in place."""
    _need_cuda(x, gamma, beta, running_mean, running_var); _f32(x, "x")
    xd = _bn_dense(x)
    d = bn_desc(xd, eps, momentum)
    y = xd if (inplace and xd is x) else torch.empty_like(xd)
    save_mean = torch.empty(d.C, dtype=torch.float32, device=x.device)
    save_invstd = torch.empty(d.C, dtype=torch.float32, device=x.device)
    ws = _bn_workspace(d, x.device)
    check(lib().mb_bn_fwd_train(
        xd.data_ptr(), gamma.data_ptr(), beta.data_ptr(),
        running_mean.data_ptr() if running_mean is not None else None,
        running_var.data_ptr() if running_var is not None else None,
        y.data_ptr(), save_mean.data_ptr(), save_invstd.data_ptr(), C.byref(d),
        ws.data_ptr(), ws.numel(), _stream()), "bn_fwd_train")
    return y, save_mean, save_invstd


def bn_fwd_apply(x, gamma, beta, mean, invstd, eps=1e-5, inplace=False):
    _need_cuda(x, gamma, beta, mean, invstd); _f32(x, "x")
    xd = _bn_dense(x)
    d = bn_desc(xd, eps, 0.0)
    y = xd if (inplace and xd is x) else torch.empty_like(xd)
    check(lib().mb_bn_fwd_apply(xd.data_ptr(), gamma.data_ptr(), beta.data_ptr(), mean.data_ptr(),
                                invstd.data_ptr(), y.data_ptr(), C.byref(d), _stream()),
          "bn_fwd_apply")
    return y


def _bn_bwd(entry, dy, saved, gamma, p, save_invstd, inplace):
    _need_cuda(dy, saved, gamma, p, save_invstd); _f32(dy, "dy"); _f32(saved, "saved activation")
    sd = _bn_dense(saved)
    dyd = like(sd, dy) if sd.dim() == 4 else dy.contiguous()
    if dyd.shape != sd.shape:
        raise RuntimeError("monet_b200 batch norm backward: gradient shape mismatch")
    d = bn_desc(sd, 0.0, 0.0)
    dx = dyd if (inplace and dyd is dy) else torch.empty_like(sd)
    dgamma = torch.empty(d.C, dtype=torch.float32, device=dy.device)
    dbeta = torch.empty(d.C, dtype=torch.float32, device=dy.device)
    ws = _bn_workspace(d, dy.device)
    fn = getattr(lib(), entry)
    check(fn(dyd.data_ptr(), sd.data_ptr(), gamma.data_ptr(), p.data_ptr(),
             save_invstd.data_ptr(), dx.data_ptr(), dgamma.data_ptr(), dbeta.data_ptr(),
             C.byref(d), ws.data_ptr(), ws.numel(), _stream()), entry)
    return dx, dgamma, dbeta


def bn_bwd_from_output(dy, y, gamma, beta, save_invstd, inplace=False):
    """(dx, dgamma, dbeta) from the stored output y; x is never needed."""
    return _bn_bwd("mb_bn_bwd_from_output", dy, y, gamma, beta, save_invstd, inplace)


def bn_bwd_from_input(dy, x, gamma, save_mean, save_invstd, inplace=False):
    return _bn_bwd("mb_bn_bwd_from_input", dy, x, gamma, save_mean, save_invstd, inplace)


def bn_act_fwd_train(x, residual, relu, gamma, beta, running_mean, running_var, momentum, eps,
                     inplace=False):
    """(y, save_mean, save_invstd) with y = act(bn(x) + residual); residual may be None."""
    _need_cuda(x, gamma, beta, running_mean, running_var); _f32(x, "x")
    xd = _bn_dense(x)
    d = bn_desc(xd, eps, momentum)
    rd = None
    if residual is not None:
        _need_cuda(residual); _f32(residual, "residual")
        rd = like(xd, residual) if xd.dim() == 4 else residual.contiguous()
        if rd.shape != xd.shape:
            raise RuntimeError("monet_b200 batch norm: residual shape mismatch")
    y = xd if (inplace and xd is x) else torch.empty_like(xd)
    save_mean = torch.empty(d.C, dtype=torch.float32, device=x.device)
    save_invstd = torch.empty(d.C, dtype=torch.float32, device=x.device)
    ws = _bn_workspace(d, x.device)
    check(lib().mb_bn_act_fwd_train(
        xd.data_ptr(), rd.data_ptr() if rd is not None else None, int(relu),
        gamma.data_ptr(), beta.data_ptr(),
        running_mean.data_ptr() if running_mean is not None else None,
        running_var.data_ptr() if running_var is not None else None,
        y.data_ptr(), save_mean.data_ptr(), save_invstd.data_ptr(), C.byref(d),
        ws.data_ptr(), ws.numel(), _stream()), "bn_act_fwd_train")
    return y, save_mean, save_invstd


def bn_act_fwd_train_partials(x, sums: "ChannelSums", residual, relu, gamma, beta, running_mean,
                              running_var, momentum, eps, inplace=False):
    """bn_act_fwd_train without the statistics pass: `sums` come from the producer of x."""
    _need_cuda(x, gamma, beta, running_mean, running_var); _f32(x, "x")
    xd = _bn_dense(x)
    if xd is not x:
        raise RuntimeError("monet_b200 batch norm: producer sums need the producer's own dense tensor")
    d = bn_desc(xd, eps, momentum)
    if sums.partials.numel() < 2 * sums.rows * d.C:
        raise RuntimeError("monet_b200 batch norm: partial sums do not match the channel count")
    rd = None
    if residual is not None:
        _need_cuda(residual); _f32(residual, "residual")
        rd = like(xd, residual) if xd.dim() == 4 else residual.contiguous()
        if rd.shape != xd.shape:
            raise RuntimeError("monet_b200 batch norm: residual shape mismatch")
    y = xd if inplace else torch.empty_like(xd)
    save_mean = torch.empty(d.C, dtype=torch.float32, device=x.device)
    save_invstd = torch.empty(d.C, dtype=torch.float32, device=x.device)
    check(lib().mb_bn_act_fwd_train_partials(
        xd.data_ptr(), rd.data_ptr() if rd is not None else None, int(relu),
        gamma.data_ptr(), beta.data_ptr(),
        running_mean.data_ptr() if running_mean is not None else None,
        running_var.data_ptr() if running_var is not None else None,
        y.data_ptr(), save_mean.data_ptr(), save_invstd.data_ptr(), C.byref(d),
        sums.partials.data_ptr(), int(sums.rows),
        sums.shift.data_ptr() if sums.shift is not None else None, _stream()),
        "bn_act_fwd_train_partials")
    return y, save_mean, save_invstd


def bn_act_fwd_apply(x, residual, relu, gamma, beta, mean, invstd, inplace=False):
    _need_cuda(x, gamma, beta, mean, invstd); _f32(x, "x")
    xd = _bn_dense(x)
    d = bn_desc(xd, 0.0, 0.0)
    rd = None
    if residual is not None:
        _need_cuda(residual); _f32(residual, "residual")
        rd = like(xd, residual) if xd.dim() == 4 else residual.contiguous()
        if rd.shape != xd.shape:
            raise RuntimeError("monet_b200 batch norm: residual shape mismatch")
    y = xd if (inplace and xd is x) else torch.empty_like(xd)
    check(lib().mb_bn_act_fwd_apply(
        xd.data_ptr(), rd.data_ptr() if rd is not None else None, int(relu),
        gamma.data_ptr(), beta.data_ptr(), mean.data_ptr(), invstd.data_ptr(), y.data_ptr(),
        C.byref(d), _stream()), "bn_act_fwd_apply")
    return y


def bn_relu_bwd_from_input(dy, x, gamma, beta, save_mean, save_invstd, inplace=False, act: int = 1):
    """(dx, dgamma, dbeta) through y = act(bn(x)), gate re-evaluated from x; act 1 = ReLU,
    2 = ReLU6."""
    _need_cuda(dy, x, gamma, beta, save_mean, save_invstd); _f32(dy, "dy"); _f32(x, "x")
    sd = _bn_dense(x)
    dyd = like(sd, dy) if sd.dim() == 4 else dy.contiguous()
    if dyd.shape != sd.shape:
        raise RuntimeError("monet_b200 batch norm backward: gradient shape mismatch")
    d = bn_desc(sd, 0.0, 0.0)
    dx = dyd if (inplace and dyd is dy) else torch.empty_like(sd)
    dgamma = torch.empty(d.C, dtype=torch.float32, device=dy.device)
    dbeta = torch.empty(d.C, dtype=torch.float32, device=dy.device)
    ws = _bn_workspace(d, dy.device)
    check(lib().mb_bn_act_bwd_from_input(
        dyd.data_ptr(), sd.data_ptr(), gamma.data_ptr(), beta.data_ptr(), save_mean.data_ptr(),
        save_invstd.data_ptr(), int(act), dx.data_ptr(), dgamma.data_ptr(), dbeta.data_ptr(),
        C.byref(d), ws.data_ptr(), ws.numel(), _stream()), "bn_act_bwd_from_input")
    return dx, dgamma, dbeta


def bn_add_relu_bwd(dy1, dy2, y, x, gamma, save_mean, save_invstd):
    """(d, dx, dgamma, dbeta) through y = relu(bn(x) + r): d = (dy1 [+ dy2]) * (y > 0) is
    written over dy1 (the gradient of r), dx is the gradient of x."""
    _need_cuda(dy1, y, x, gamma, save_mean, save_invstd); _f32(dy1, "dy1"); _f32(x, "x")
    xd = _bn_dense(x)
    yd = like(xd, y) if xd.dim() == 4 else y.contiguous()
    d1 = like(xd, dy1) if xd.dim() == 4 else dy1.contiguous()
    d2 = None
    if dy2 is not None:
        _need_cuda(dy2); _f32(dy2, "dy2")
        d2 = like(xd, dy2) if xd.dim() == 4 else dy2.contiguous()
    if d1.shape != xd.shape or yd.shape != xd.shape or (d2 is not None and d2.shape != xd.shape):
        raise RuntimeError("monet_b200 batch norm backward: shape mismatch")
    desc = bn_desc(xd, 0.0, 0.0)
    dx = torch.empty_like(xd)
    dgamma = torch.empty(desc.C, dtype=torch.float32, device=x.device)
    dbeta = torch.empty(desc.C, dtype=torch.float32, device=x.device)
    ws = _bn_workspace(desc, x.device)
    check(lib().mb_bn_add_relu_bwd(
        d1.data_ptr(), d2.data_ptr() if d2 is not None else None, yd.data_ptr(), xd.data_ptr(),
        gamma.data_ptr(), save_mean.data_ptr(), save_invstd.data_ptr(), d1.data_ptr(),
        dx.data_ptr(), dgamma.data_ptr(), dbeta.data_ptr(), C.byref(desc), ws.data_ptr(),
        ws.numel(), _stream()), "bn_add_relu_bwd")
    return d1, dx, dgamma, dbeta


# ------------------------------------------------------------------------ softmax

def _split_dim(x: torch.Tensor, dim: int):
    dim = dim % x.dim()
    outer = 1
    for s in x.shape[:dim]:
        outer *= int(s)
    inner = 1
    for s in x.shape[dim + 1:]:
        inner *= int(s)
    return outer, int(x.shape[dim]), inner


def softmax(x: torch.Tensor, dim: int, log: bool = False) -> torch.Tensor:
    _need_cuda(x); _f32(x, "x")
    xc = x.contiguous()
    outer, classes, inner = _split_dim(xc, dim)
    y = torch.empty_like(xc)
    check(lib().mb_softmax_fwd(xc.data_ptr(), y.data_ptr(), outer, classes, inner, int(log),
                               _stream()), "softmax_fwd")
    return y


def softmax_bwd(dy: torch.Tensor, y: torch.Tensor, dim: int, log: bool = False) -> torch.Tensor:
    _need_cuda(dy, y); _f32(dy, "dy"); _f32(y, "y")
    yc, dyc = y.contiguous(), dy.contiguous()
    outer, classes, inner = _split_dim(yc, dim)
    dx = torch.empty_like(yc)
    check(lib().mb_softmax_bwd(dyc.data_ptr(), yc.data_ptr(), dx.data_ptr(), outer, classes,
                               inner, int(log), _stream()), "softmax_bwd")
    return dx


def cross_entropy_fwd_bwd(logits: torch.Tensor, labels: torch.Tensor, grad_scale: float):
    """Per-position losses and d(logits) = (softmax - onehot) * grad_scale in one pass.

    `logits` is [N, classes] or [N, classes, d1, ...]; `labels` int64 of the matching shape.
    For a mean-reduced loss pass grad_scale = 1 / labels.numel().
    """
    _need_cuda(logits, labels); _f32(logits, "logits")
    if labels.dtype != torch.int64:
        raise RuntimeError("monet_b200.cross_entropy: labels must be int64")
    lc, lab = logits.contiguous(), labels.contiguous()
    outer, classes, inner = _split_dim(lc, 1)
    if lab.numel() != outer * inner:
        raise RuntimeError("monet_b200.cross_entropy: label shape does not match the logits")
    loss_rows = torch.empty(lab.shape, dtype=torch.float32, device=logits.device)
    dlogits = torch.empty_like(lc)
    check(lib().mb_softmax_ce_fwd_bwd(lc.data_ptr(), lab.data_ptr(), loss_rows.data_ptr(),
                                      dlogits.data_ptr(), outer, classes, inner,
                                      float(grad_scale), _stream()), "softmax_ce_fwd_bwd")
    return loss_rows, dlogits


# ----------------------------------------------------------------- layout / pooling

def to_nhwc(x: torch.Tensor) -> torch.Tensor:
    """A channels_last tensor with x's values (x itself if it already is one)."""
    _need_cuda(x); _f32(x, "x")
    if x.dim() != 4:
        raise RuntimeError("monet_b200.to_nhwc expects a 4-D tensor")
    if x.is_contiguous(memory_format=torch.channels_last):
        return x
    xc = x.contiguous()
    N, Cc, H, W = (int(s) for s in xc.shape)
    y = torch.empty((N, Cc, H, W), dtype=x.dtype, device=x.device,
                    memory_format=torch.channels_last)
    check(lib().mb_nchw_to_nhwc(xc.data_ptr(), y.data_ptr(), N, Cc, H, W, _stream()),
          "nchw_to_nhwc")
    return y


def to_nchw(x: torch.Tensor) -> torch.Tensor:
    _need_cuda(x); _f32(x, "x")
    if x.dim() != 4:
        raise RuntimeError("monet_b200.to_nchw expects a 4-D tensor")
    if x.is_contiguous():
        return x
    xd = dense(x)
    if not is_nhwc(xd):
        return xd
    N, Cc, H, W = (int(s) for s in xd.shape)
    y = torch.empty((N, Cc, H, W), dtype=x.dtype, device=x.device)
    check(lib().mb_nhwc_to_nchw(xd.data_ptr(), y.data_ptr(), N, Cc, H, W, _stream()),
          "nhwc_to_nchw")
    return y


def _cat_geometry(shapes, dim: int, nhwc: bool):
    """(rows, widths, physical-order flag) of a concatenation along logical axis `dim`."""
    nd = len(shapes[0])
    dim = dim % nd
    order = (0, 2, 3, 1) if nhwc else tuple(range(nd))      # logical axes in physical order
    pos = order.index(dim)
    rows = 1
    for a in order[:pos]:
        rows *= int(shapes[0][a])
    tail = 1
    for a in order[pos + 1:]:
        tail *= int(shapes[0][a])
    for sh in shapes:
        if len(sh) != nd or any(int(sh[a]) != int(shapes[0][a]) for a in range(nd) if a != dim):
            raise RuntimeError("monet_b200.cat: shapes differ outside the concatenation axis")
    return rows, [int(sh[dim]) * tail for sh in shapes], dim


def _cat_call(whole, pieces, widths, rows, to_pieces):
    n = len(pieces)
    if n > _lib.MB_CAT_MAX_PIECES:
        raise RuntimeError(f"monet_b200.cat: at most {_lib.MB_CAT_MAX_PIECES} tensors per call")
    ptrs = (C.c_void_p * n)(*[p.data_ptr() for p in pieces])
    ws = (C.c_int * n)(*widths)
    check(lib().mb_cat_rows(whole.data_ptr(), ptrs, ws, n, rows, int(to_pieces), _stream()), "cat_rows")


def cat(tensors, dim: int) -> torch.Tensor:
    """torch.cat(tensors, dim) in one launch; the result has the first tensor's memory format."""
    tensors = list(tensors)
    _need_cuda(*tensors)
    for t in tensors:
        _f32(t, "cat input")
    first = dense(tensors[0])
    nhwc = is_nhwc(first)
    parts = [first] + [like(first, t) if t.dim() == 4 else t.contiguous() for t in tensors[1:]]
    rows, widths, dim = _cat_geometry([p.shape for p in parts], dim, nhwc)
    shape = list(first.shape)
    shape[dim] = sum(int(p.shape[dim]) for p in parts)
    out = torch.empty(shape, dtype=first.dtype, device=first.device,
                      memory_format=torch.channels_last if nhwc else torch.contiguous_format)
    _cat_call(out, parts, widths, rows, False)
    return out


def cat_bwd(grad: torch.Tensor, sizes, dim: int):
    """The gradient of a concatenation split back into dense pieces of `sizes` along `dim`
    (torch.split + .contiguous() per piece in cat.py:20-29) in one launch."""
    _need_cuda(grad); _f32(grad, "grad")
    g = dense(grad)
    nhwc = is_nhwc(g)
    dim = dim % g.dim()
    shapes = []
    for sz in sizes:
        sh = list(g.shape)
        sh[dim] = int(sz)
        shapes.append(sh)
    if sum(int(s) for s in sizes) != int(g.shape[dim]):
        raise RuntimeError("monet_b200.cat_bwd: sizes do not add up to the gradient's extent")
    rows, widths, dim = _cat_geometry(shapes, dim, nhwc)
    fmt = torch.channels_last if nhwc else torch.contiguous_format
    pieces = [torch.empty(sh, dtype=g.dtype, device=g.device, memory_format=fmt) for sh in shapes]
    _cat_call(g, pieces, widths, rows, True)
    return pieces


def global_avgpool(x: torch.Tensor) -> torch.Tensor:
    _need_cuda(x); _f32(x, "x")
    xd = dense(x)
    N, Cc, H, W = (int(s) for s in xd.shape)
    y = torch.empty((N, Cc, 1, 1), dtype=x.dtype, device=x.device)
    check(lib().mb_global_avgpool_fwd(xd.data_ptr(), y.data_ptr(), N, Cc, H * W, layout_of(xd),
                                      _stream()), "global_avgpool_fwd")
    return y


def global_avgpool_bwd(dy: torch.Tensor, shape, nhwc: bool) -> torch.Tensor:
    _need_cuda(dy); _f32(dy, "dy")
    N, Cc, H, W = (int(s) for s in shape)
    dyc = dy.contiguous()
    fmt = torch.channels_last if nhwc else torch.contiguous_format
    dx = torch.empty((N, Cc, H, W), dtype=dy.dtype, device=dy.device, memory_format=fmt)
    check(lib().mb_global_avgpool_bwd(dyc.data_ptr(), dx.data_ptr(), N, Cc, H * W,
                                      MB_NHWC if nhwc else MB_NCHW, _stream()),
          "global_avgpool_bwd")
    return dx


# -------------------------------------------------------------------- convolution
# Tensor-core passes work on NHWC activations and [K][R][S][C] filters, which is what
# torch.channels_last tensors are physically; other layouts are converted on entry.
# Channel counts that are not multiples of 4 (the 3-channel network input, a 1- or
# 2-class head) are zero-padded to the next multiple of 4 and sliced back.

from ._lib import MB_CONV_DGRAD, MB_CONV_FPROP, MB_CONV_WGRAD, ConvDesc  # noqa: E402


def _pad4(n: int) -> int:
    return (n + 3) // 4 * 4


def conv_desc(x_shape, w_shape, stride, padding, dilation, groups) -> ConvDesc:
    N, Cc, H, W = (int(v) for v in x_shape)
    K, Cg, R, S = (int(v) for v in w_shape)
    sh, sw = _pair(stride); ph, pw = _pair(padding); dh, dw = _pair(dilation)
    P = (H + 2 * ph - dh * (R - 1) - 1) // sh + 1
    Q = (W + 2 * pw - dw * (S - 1) - 1) // sw + 1
    return ConvDesc(N, Cc, H, W, K, R, S, P, Q, sh, sw, ph, pw, dh, dw, int(groups))


def conv_num_variants(conv_pass: int) -> int:
    return lib().mb_conv_num_variants(conv_pass)


def conv_workspace_bytes(conv_pass: int, variant: int, d: ConvDesc) -> int:
    return lib().mb_conv_workspace_bytes(conv_pass, variant, C.byref(d))


def _act_nhwc(x: torch.Tensor) -> torch.Tensor:
    """NHWC activation with a channel count that is a multiple of 4."""
    N, Cc, H, W = (int(v) for v in x.shape)
    Cp = _pad4(Cc)
    if Cp == Cc:
        return to_nhwc(x)
    xc = x.contiguous()
    y = torch.empty((N, Cp, H, W), dtype=x.dtype, device=x.device, memory_format=torch.channels_last)
    check(lib().mb_nchw_to_nhwc_pad(xc.data_ptr(), y.data_ptr(), N, Cc, H, W, Cp, _stream()),
          "nchw_to_nhwc_pad")
    return y


def _filter_krsc(w: torch.Tensor) -> torch.Tensor:
    """[K][R][S][C] filter with K and C padded to multiples of 4 (tiny; torch copies)."""
    K, Cc, R, S = (int(v) for v in w.shape)
    Kp, Cp = _pad4(K), _pad4(Cc)
    if Kp == K and Cp == Cc:
        return w.detach().contiguous(memory_format=torch.channels_last)
    wp = torch.empty((Kp, Cp, R, S), dtype=w.dtype, device=w.device,
                     memory_format=torch.channels_last).zero_()
    wp[:K, :Cc] = w.detach()
    return wp


def _padded_desc(d: ConvDesc) -> ConvDesc:
    return ConvDesc(d.N, _pad4(d.C), d.H, d.W, _pad4(d.K), d.R, d.S, d.P, d.Q, d.stride_h,
                    d.stride_w, d.pad_h, d.pad_w, d.dil_h, d.dil_w, d.groups)


def _workspace(conv_pass: int, variant: int, d: ConvDesc, device) -> torch.Tensor:
    n = conv_workspace_bytes(conv_pass, variant, d)
    return torch.empty(max(n, 16), dtype=torch.uint8, device=device)


def _smallc_geometry(d: ConvDesc):
    """(Hp, Wp) of the padded 4-channel input when the few-channel kernels apply, else None."""
    if d.C > 4 or d.K % 4 or d.groups != 1:
        return None
    hp, wp = C.c_int(0), C.c_int(0)
    if lib().mb_conv_smallc_geometry(C.byref(d), C.byref(hp), C.byref(wp)) != 0:
        return None
    return hp.value, wp.value


def _smallc_input(x: torch.Tensor, d: ConvDesc, geom) -> torch.Tensor:
    xc = x.detach().contiguous()
    xp = torch.empty((d.N, geom[0], geom[1], 4), dtype=x.dtype, device=x.device)
    check(lib().mb_conv_smallc_pack_input(xc.data_ptr(), xp.data_ptr(), C.byref(d), _stream()),
          "conv_smallc_pack_input")
    return xp


class ChannelSums:
    """Per-channel partial sums of a convolution's output, left by its statistics warps for the
    batch norm that follows: `partials` is [2][rows][K] (sum and sum of squares around `shift`)."""

    __slots__ = ("partials", "rows", "shift")

    def __init__(self, partials, rows, shift):
        self.partials, self.rows, self.shift = partials, rows, shift


def conv2d_fprop(x, w, bias, stride, padding, dilation, groups=1, variant: int = 0,
                 stats_shift=None, want_stats: bool = False):
    """y = conv2d(x, w) + bias; y is a channels_last tensor of logical shape N x K x P x Q.

    With ``want_stats`` returns ``(y, ChannelSums or None)``: the sums a following batch norm
    needs, accumulated beside the epilogue around ``stats_shift`` ([K] or None); None when this
    geometry has no such path (few-channel input, K not a multiple of 32, stride-1 multi-tap
    filters)."""
    _need_cuda(x, w, bias); _f32(x, "x"); _f32(w, "w")
    d0 = conv_desc(x.shape, w.shape, stride, padding, dilation, groups)
    geom = _smallc_geometry(d0)
    if want_stats:
        multi_tap_s1 = d0.R * d0.S > 1 and d0.stride_h == 1 and d0.stride_w == 1
        if geom is None and d0.K % 32 == 0 and groups == 1 and not multi_tap_s1:
            d = _padded_desc(d0)
            if d.K == d0.K:
                xa, wk = _act_nhwc(x), _filter_krsc(w)
                b = bias.detach().contiguous() if bias is not None else None
                y = torch.empty((d.N, d.K, d.P, d.Q), dtype=x.dtype, device=x.device,
                                memory_format=torch.channels_last)
                ws = _workspace(MB_CONV_FPROP, variant, d, x.device)
                nbytes = lib().mb_conv_bnstats_bytes(C.byref(d))
                partials = torch.empty(nbytes // 4, dtype=torch.float32, device=x.device)
                rows = C.c_int(0)
                sh = stats_shift.detach() if stats_shift is not None else None
                if sh is not None:
                    _need_cuda(sh); _f32(sh, "stats_shift")
                rc = lib().mb_conv2d_fprop_bnstats(
                    xa.data_ptr(), wk.data_ptr(), b.data_ptr() if b is not None else None,
                    y.data_ptr(), C.byref(d), int(variant), ws.data_ptr(), ws.numel(),
                    sh.data_ptr() if sh is not None else None, partials.data_ptr(), nbytes,
                    C.byref(rows), _stream())
                if rc != 2:      # MB_ERR_UNSUPPORTED: nothing was launched, run the plain pair
                    check(rc, "conv2d_fprop_bnstats")
                    return y, ChannelSums(partials, rows.value, sh)
        return conv2d_fprop(x, w, bias, stride, padding, dilation, groups, variant), None
    if geom is not None:
        if variant != 0:
            raise RuntimeError("monet_b200.conv2d_fprop: no variant %d for a few-channel input" % variant)
        hp2, wp2 = C.c_int(0), C.c_int(0)
        if lib().mb_conv_smallc2_geometry(C.byref(d0), C.byref(hp2), C.byref(wp2)) == 0:
            # stride 2: both row phases in one buffer, forward on the many-tap kernel
            xc = x.detach().contiguous()
            xp2 = torch.empty((d0.N, hp2.value, wp2.value, 8), dtype=x.dtype, device=x.device)
            check(lib().mb_conv_smallc2_pack_input(xc.data_ptr(), xp2.data_ptr(), C.byref(d0), _stream()),
                  "conv_smallc2_pack_input")
            T = (d0.R + 1) // 2
            wpad = torch.zeros((d0.K, 4, 2 * T, 8), dtype=w.dtype, device=w.device)
            wpad[:, :d0.C, :d0.R, :d0.S] = w.detach()
            # (k, c, dh, phase, chunk, s%4) -> (k, dh, chunk, s%4, phase, c)
            wq = wpad.view(d0.K, 4, T, 2, 2, 4).permute(0, 2, 4, 5, 3, 1).contiguous()
            y = torch.empty((d0.N, d0.K, d0.P, d0.Q), dtype=x.dtype, device=x.device,
                            memory_format=torch.channels_last)
            b = bias.detach().contiguous() if bias is not None else None
            check(lib().mb_conv2d_fprop_smallc2(xp2.data_ptr(), wq.data_ptr(),
                                                b.data_ptr() if b is not None else None, y.data_ptr(),
                                                C.byref(d0), _stream()), "conv2d_fprop_smallc2")
            return y
        xp = _smallc_input(x, d0, geom)
        wp = torch.zeros((d0.K, d0.R, 8, 4), dtype=w.dtype, device=w.device)
        wp[:, :, :d0.S, :d0.C] = w.detach().permute(0, 2, 3, 1)
        y = torch.empty((d0.N, d0.K, d0.P, d0.Q), dtype=x.dtype, device=x.device,
                        memory_format=torch.channels_last)
        b = bias.detach().contiguous() if bias is not None else None
        check(lib().mb_conv2d_fprop_smallc(xp.data_ptr(), wp.data_ptr(),
                                           b.data_ptr() if b is not None else None, y.data_ptr(),
                                           C.byref(d0), _stream()), "conv2d_fprop_smallc")
        return y
    d = _padded_desc(d0)
    xa, wk = _act_nhwc(x), _filter_krsc(w)
    b = None
    if bias is not None:
        b = bias.detach().contiguous()
        if d.K != d0.K:
            b = torch.nn.functional.pad(b, (0, d.K - d0.K))
    y = torch.empty((d.N, d.K, d.P, d.Q), dtype=x.dtype, device=x.device,
                    memory_format=torch.channels_last)
    ws = _workspace(MB_CONV_FPROP, variant, d, x.device)
    check(lib().mb_conv2d_fprop(xa.data_ptr(), wk.data_ptr(), b.data_ptr() if b is not None else None,
                                y.data_ptr(), C.byref(d), int(variant), ws.data_ptr(), ws.numel(),
                                _stream()), "conv2d_fprop")
    return y if d.K == d0.K else y[:, :d0.K]


def conv2d_dgrad(dy, w, x_shape, stride, padding, dilation, groups=1, variant: int = 0):
    """dx (channels_last, logical shape x_shape) from dy and the filter."""
    _need_cuda(dy, w); _f32(dy, "dy"); _f32(w, "w")
    d0 = conv_desc(x_shape, w.shape, stride, padding, dilation, groups)
    d = _padded_desc(d0)
    if tuple(dy.shape) != (d0.N, d0.K, d0.P, d0.Q):
        raise RuntimeError("monet_b200.conv2d_dgrad: gradient shape does not match the geometry")
    ga, wk = _act_nhwc(dy), _filter_krsc(w)
    dx = torch.empty((d.N, d.C, d.H, d.W), dtype=dy.dtype, device=dy.device,
                     memory_format=torch.channels_last)
    ws = _workspace(MB_CONV_DGRAD, variant, d, dy.device)
    check(lib().mb_conv2d_dgrad(ga.data_ptr(), wk.data_ptr(), dx.data_ptr(), C.byref(d), int(variant),
                                ws.data_ptr(), ws.numel(), _stream()), "conv2d_dgrad")
    return dx if d.C == d0.C else dx[:, :d0.C]


def conv2d_wgrad(x, dy, w_shape, stride, padding, dilation, groups=1, variant: int = 0,
                 need_bias: bool = False):
    """(dw, db): dw is a channels_last tensor of logical shape w_shape; db = dy.sum((0,2,3))."""
    _need_cuda(x, dy); _f32(x, "x"); _f32(dy, "dy")
    d0 = conv_desc(x.shape, w_shape, stride, padding, dilation, groups)
    d = _padded_desc(d0)
    if tuple(dy.shape) != (d0.N, d0.K, d0.P, d0.Q):
        raise RuntimeError("monet_b200.conv2d_wgrad: gradient shape does not match the geometry")
    geom = _smallc_geometry(d0)
    if geom is not None:
        xp = _smallc_input(x, d0, geom)
        ga = to_nhwc(dy)
        dwp = torch.empty((d0.K, d0.R, 8, 4), dtype=x.dtype, device=x.device)
        db = torch.empty(d0.K, dtype=x.dtype, device=x.device) if need_bias else None
        n = lib().mb_conv_smallc_wgrad_workspace_bytes(C.byref(d0), int(variant))
        ws = torch.empty(max(n, 16), dtype=torch.uint8, device=x.device)
        check(lib().mb_conv2d_wgrad_smallc(xp.data_ptr(), ga.data_ptr(), dwp.data_ptr(),
                                           db.data_ptr() if db is not None else None,
                                           C.byref(d0), int(variant), ws.data_ptr(), ws.numel(),
                                           _stream()), "conv2d_wgrad_smallc")
        return dwp[:, :, :d0.S, :d0.C].permute(0, 3, 1, 2), db
    xa, ga = _act_nhwc(x), _act_nhwc(dy)
    dw = torch.empty((d.K, d.C, d.R, d.S), dtype=x.dtype, device=x.device,
                     memory_format=torch.channels_last)
    db = torch.empty(d.K, dtype=x.dtype, device=x.device) if need_bias else None
    ws = _workspace(MB_CONV_WGRAD, variant, d, x.device)
    check(lib().mb_conv2d_wgrad(xa.data_ptr(), ga.data_ptr(), dw.data_ptr(),
                                db.data_ptr() if db is not None else None, C.byref(d), int(variant),
                                ws.data_ptr(), ws.numel(), _stream()), "conv2d_wgrad")
    if d.K != d0.K or d.C != d0.C:
        dw = dw[:d0.K, :d0.C]
        db = db[:d0.K] if db is not None else None
    return dw, db


# ------------------------------------------------------------------ fully connected
# A fully connected layer is a 1x1 convolution over a 1x1 map: x [N, C] is the NHWC activation
# [N, C, 1, 1] and W [K, C] the filter [K][1][1][C], byte for byte.  The three passes therefore run
# on the same tcgen05 kernels (TF32 operands, fp32 accumulation) as the pointwise convolutions,
# instead of the fp32 SIMT library GEMM the reference calls (linear.py:38,52-60).

def linear_fwd(x: torch.Tensor, w: torch.Tensor, bias) -> torch.Tensor:
    """x @ w.T + bias for x [N, C], w [K, C]."""
    _need_cuda(x, w, bias); _f32(x, "x"); _f32(w, "w")
    if x.dim() != 2 or w.dim() != 2 or x.shape[1] != w.shape[1]:
        raise RuntimeError("monet_b200.linear_fwd expects x [N, C] and w [K, C]")
    N, Cc, K = int(x.shape[0]), int(x.shape[1]), int(w.shape[0])
    y = conv2d_fprop(x.detach().contiguous().view(N, Cc, 1, 1), w.detach().contiguous().view(K, Cc, 1, 1),
                     bias, 1, 0, 1)
    return y.reshape(N, K)


def linear_dgrad(dy: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """dy @ w for dy [N, K], w [K, C]."""
    _need_cuda(dy, w); _f32(dy, "dy"); _f32(w, "w")
    N, K, Cc = int(dy.shape[0]), int(w.shape[0]), int(w.shape[1])
    dx = conv2d_dgrad(dy.contiguous().view(N, K, 1, 1), w.detach().contiguous().view(K, Cc, 1, 1),
                      (N, Cc, 1, 1), 1, 0, 1)
    return dx.reshape(N, Cc)


def linear_wgrad(x: torch.Tensor, dy: torch.Tensor, need_bias: bool = False):
    """(dy.T @ x, dy.sum(0) or None) for x [N, C], dy [N, K]."""
    _need_cuda(x, dy); _f32(x, "x"); _f32(dy, "dy")
    N, Cc, K = int(x.shape[0]), int(x.shape[1]), int(dy.shape[1])
    dw, db = conv2d_wgrad(x.detach().contiguous().view(N, Cc, 1, 1), dy.contiguous().view(N, K, 1, 1),
                          (K, Cc, 1, 1), 1, 0, 1, 1, 0, need_bias)
    return dw.reshape(K, Cc), db


def conv_device_status(reset: bool = True) -> int:
    """0 when no tensor-core kernel has reported a pipeline time-out (synchronises)."""
    return lib().mb_conv_device_status(int(reset))


# ---------------------------------------------------------------------- depthwise
def _dw_filter(w: torch.Tensor) -> torch.Tensor:
    """[C, 1, R, S] -> [R*S][C] (tiny; torch copy)."""
    Cc, _, R, S = w.shape
    return w.detach().reshape(Cc, R * S).t().contiguous()


def depthwise_fprop(x, w, bias, stride, padding, dilation, groups):
    """Depthwise conv2d (groups == channels); NHWC output."""
    _need_cuda(x, w, bias); _f32(x, "x"); _f32(w, "w")
    d = conv_desc(x.shape, (w.shape[0], w.shape[1], w.shape[2], w.shape[3]), stride, padding, dilation, groups)
    if groups != d.C or w.shape[0] != d.C or w.shape[1] != 1:
        raise RuntimeError("monet_b200: grouped convolution is supported only as depthwise (groups == C == K)")
    xa = to_nhwc(x)
    y = torch.empty((d.N, d.K, d.P, d.Q), dtype=x.dtype, device=x.device, memory_format=torch.channels_last)
    b = bias.detach().contiguous() if bias is not None else None
    check(lib().mb_depthwise_fprop(xa.data_ptr(), _dw_filter(w).data_ptr(),
                                   b.data_ptr() if b is not None else None, y.data_ptr(), C.byref(d),
                                   _stream()), "depthwise_fprop")
    return y


def depthwise_bwd(dy, x, w, stride, padding, dilation, groups, need=(True, True, False)):
    """(dx, dw, db) of a depthwise convolution; entries not asked for are None."""
    _need_cuda(dy, x, w); _f32(dy, "dy")
    d = conv_desc(x.shape, w.shape, stride, padding, dilation, groups)
    ga = to_nhwc(dy)
    dx = dw = db = None
    if need[0]:
        dx = torch.empty((d.N, d.C, d.H, d.W), dtype=dy.dtype, device=dy.device,
                         memory_format=torch.channels_last)
        check(lib().mb_depthwise_dgrad(ga.data_ptr(), _dw_filter(w).data_ptr(), dx.data_ptr(),
                                       C.byref(d), _stream()), "depthwise_dgrad")
    if need[1] or need[2]:
        xa = to_nhwc(x)
        dwt = torch.empty((d.R * d.S, d.C), dtype=dy.dtype, device=dy.device)
        db = torch.empty(d.C, dtype=dy.dtype, device=dy.device) if need[2] else None
        check(lib().mb_depthwise_wgrad(xa.data_ptr(), ga.data_ptr(), dwt.data_ptr(),
                                       db.data_ptr() if db is not None else None, C.byref(d),
                                       _stream()), "depthwise_wgrad")
        dw = dwt.t().reshape(d.C, 1, d.R, d.S) if need[1] else None
    return dx, dw, db
