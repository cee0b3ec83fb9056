"""Test infrastructure: a CPU stand-in for ``monet_b200.functional`` built on the oracle.

The operator classes are thin protocol adapters over ``functional`` (which only accepts CUDA
tensors).  To exercise the HOST logic above them on a machine without a GPU -- MONeT's own
``Schedule`` / ``MONeTWrapper`` / ``SolverInfo`` driving the classes, the ILP, the gradient
buckets -- ``patched()`` swaps the tensor-level functions for PyTorch-CPU / oracle
equivalents for the duration of a test.  Never imported by the package.
"""
from __future__ import annotations

import contextlib

import torch
import torch.nn.functional as TF

from monet_b200 import functional as F
from oracle import lm_ops_oracle as oracle


def _relu(x, inplace=False):
    return x.relu_() if inplace else torch.relu(x)


def _relu_mask(x, inplace=False):
    mask = torch.from_numpy(oracle.relu_mask_bytes(x.detach().contiguous()))
    return _relu(x, inplace), mask


def _relu_bwd_mask(dy, mask, inplace=True):
    bits = torch.from_numpy(oracle.unpack_bits(mask.numpy(), dy.numel())).view(dy.shape)
    return dy.mul_(bits) if inplace else dy * bits


def _relu_bwd_act(dy, act, threshold=0.0, inplace=True):
    gate = (act > threshold).to(dy.dtype)
    return dy.mul_(gate) if inplace else dy * gate


def _hardtanh(x, lo, hi, inplace=False):
    return x.clamp_(lo, hi) if inplace else x.clamp(lo, hi)


def _hardtanh_bwd(dy, act, lo, hi, inplace=False):
    return oracle.hardtanh_backward(dy, act, lo, hi)


def _add(a, b, alpha=1.0, inplace=False):
    return a.add_(b, alpha=alpha) if inplace else torch.add(a, b, alpha=alpha)


def _maxpool2d(x, kernel_size, stride, padding, dilation, ceil_mode, with_indices=True):
    y, idx = TF.max_pool2d(x, kernel_size, stride, padding, dilation, bool(ceil_mode), return_indices=True)
    desc = (tuple(x.shape), kernel_size, stride, padding, dilation, bool(ceil_mode))
    return y, (idx if with_indices else None), desc


def _maxpool2d_bwd(dy, idx, desc):
    shape = desc[0]
    dx = torch.zeros(shape[0], shape[1], shape[2] * shape[3], dtype=dy.dtype)
    dx.scatter_add_(2, idx.reshape(shape[0], shape[1], -1), dy.reshape(shape[0], shape[1], -1))
    return dx.view(shape)


def _bn_fwd_train(x, gamma, beta, rm, rv, momentum, eps, inplace=False):
    y, mean, invstd, _, _ = oracle.bn_forward_train(x, gamma.detach(), beta.detach(), rm, rv, momentum, eps)
    if inplace:
        x.copy_(y)
        y = x
    return y, mean, invstd


def _bn_fwd_apply(x, gamma, beta, mean, invstd, eps=1e-5, inplace=False):
    y = oracle.bn_forward_apply(x, gamma.detach(), beta.detach(), mean, invstd)
    if inplace:
        x.copy_(y)
        y = x
    return y


def _bn_bwd_from_output(dy, y, gamma, beta, save_invstd, inplace=False):
    return oracle.bn_backward_from_output(dy, y, gamma.detach(), beta.detach(), save_invstd)


def _bn_bwd_from_input(dy, x, gamma, save_mean, save_invstd, inplace=False):
    c = (1, -1) + (1,) * (x.dim() - 2)
    xhat = (x - save_mean.view(c)) * save_invstd.view(c)
    dims = [d for d in range(x.dim()) if d != 1]
    m = x.numel() / x.shape[1]
    dbeta = dy.sum(dims)
    dgamma = (dy * xhat).sum(dims)
    dx = (dy - dbeta.view(c) / m - xhat * dgamma.view(c) / m) * (gamma.detach() * save_invstd).view(c)
    return dx, dgamma, dbeta


def _conv2d_fprop(x, w, bias, stride, padding, dilation, groups=1, variant=0, stats_shift=None,
                  want_stats=False):
    if variant >= F_conv_num_variants(0):
        raise RuntimeError("no such variant")
    y = oracle.conv_forward(x.detach(), w.detach(), bias.detach() if bias is not None else None,
                            stride, padding, dilation, groups)
    return (y, None) if want_stats else y


def _conv2d_dgrad(dy, w, x_shape, stride, padding, dilation, groups=1, variant=0):
    if variant >= F_conv_num_variants(1):
        raise RuntimeError("no such variant")
    x0 = torch.zeros(x_shape)
    with torch.enable_grad():
        dx, _, _ = oracle.conv_backward(dy, x0, w.detach(), stride, padding, dilation, groups, need=(True, False, False))
    return dx


def _conv2d_wgrad(x, dy, w_shape, stride, padding, dilation, groups=1, variant=0, need_bias=False):
    if variant >= F_conv_num_variants(2):
        raise RuntimeError("no such variant")
    w0 = torch.zeros(w_shape)
    with torch.enable_grad():
        _, dw, db = oracle.conv_backward(dy, x.detach(), w0, stride, padding, dilation, groups,
                                     need=(False, True, need_bias))
    return dw, db


def _depthwise_fprop(x, w, bias, stride, padding, dilation, groups):
    return oracle.conv_forward(x.detach(), w.detach(), bias.detach() if bias is not None else None,
                               stride, padding, dilation, groups)


def _depthwise_bwd(dy, x, w, stride, padding, dilation, groups, need=(True, True, False)):
    with torch.enable_grad():
        return oracle.conv_backward(dy, x.detach(), w.detach(), stride, padding, dilation, groups, need=tuple(need))


def F_conv_num_variants(conv_pass):
    return (1, 1, 2)[conv_pass]


def _global_avgpool(x):
    return x.mean((2, 3), keepdim=True)


def _global_avgpool_bwd(dy, shape, nhwc):
    return oracle.global_avgpool_backward(dy, shape)


def _cross_entropy(logits, labels, grad_scale):
    with torch.enable_grad():
        return oracle.cross_entropy(logits, labels, grad_scale)


_FAKES = {
    "relu": _relu, "relu_mask": _relu_mask, "relu_bwd_mask": _relu_bwd_mask,
    "relu_bwd_act": _relu_bwd_act, "hardtanh": _hardtanh, "hardtanh_bwd": _hardtanh_bwd,
    "add": _add, "scale": lambda x, a: x * a, "maxpool2d": _maxpool2d, "maxpool2d_bwd": _maxpool2d_bwd,
    "bn_fwd_train": _bn_fwd_train, "bn_fwd_apply": _bn_fwd_apply,
    "bn_bwd_from_output": _bn_bwd_from_output, "bn_bwd_from_input": _bn_bwd_from_input,
    "conv2d_fprop": _conv2d_fprop, "conv2d_dgrad": _conv2d_dgrad, "conv2d_wgrad": _conv2d_wgrad,
    "depthwise_fprop": _depthwise_fprop, "depthwise_bwd": _depthwise_bwd,
    "conv_num_variants": F_conv_num_variants, "global_avgpool": _global_avgpool,
    "global_avgpool_bwd": _global_avgpool_bwd, "cross_entropy_fwd_bwd": _cross_entropy,
    "softmax": lambda x, dim, log=False: oracle.softmax_forward(x, dim, log),
    "softmax_bwd": lambda dy, y, dim, log=False: oracle.softmax_backward(dy, y, dim, log),
    "linear_fwd": lambda x, w, b: torch.addmm(b, x, w.t()),
    "linear_wgrad": lambda x, dy, need_bias=False: (dy.t().mm(x), dy.sum(0) if need_bias else None),
    "linear_dgrad": lambda dy, w: dy.mm(w),
    "add_channel_bias": lambda y, b: y.add_(b.view(1, -1, 1, 1)),
    "cat": lambda ts, dim: torch.cat(list(ts), dim),
    "cat_bwd": lambda g, sizes, dim: [p.contiguous() for p in torch.split(g, sizes, dim=dim)],
}


@contextlib.contextmanager
def patched():
    """``monet_b200.functional`` with CPU implementations for the length of the block."""
    saved = {k: getattr(F, k, None) for k in _FAKES}
    try:
        for k, v in _FAKES.items():
            setattr(F, k, v)
        yield F
    finally:
        for k, v in saved.items():
            if v is None:
                delattr(F, k)
            else:
                setattr(F, k, v)
