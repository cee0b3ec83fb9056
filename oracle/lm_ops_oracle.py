"""CPU oracle for the low-memory operator path.  TEST INFRASTRUCTURE ONLY.

Only the tests, ``__graft_entry__.smoke()`` and the ``cpu_baseline`` / ``--impl reference``
legs of ``bench.py`` may import this module; nothing in ``monet_b200`` does.

What it restates.  MONeT's operators are defined as "the PyTorch op, but keeping less for
backward", so the value oracle for each of them is the PyTorch CPU op it replaces
(fp32, autograd for gradients).  The parts PyTorch does not define are restated here from
the reference's sources, function by function:

  mask bytes               pack.cu:22-31 / pack.cpp:6-13      -> relu_mask_bytes
  nibble packing           pack.cu:3-12                       -> pack_nibbles
  window-local argmax      maxpool.cu:26-72                   -> maxpool_local_index (loop form)
                                                                 maxpool_forward (from torch's
                                                                 global indices, vectorised)
  gather backward          maxpool.cu:81-131                  -> maxpool_backward_from_index
  BN backward from output  lrbn.cu:153-208                    -> bn_backward_from_output
  BN saved statistics      lrbn.cpp:32-40 (cuDNN semantics)   -> bn_forward_train
  conv pass split          conv.py:292-325                    -> conv_backward

PARITY UNPINNED by the reference: it ships no tests, golden vectors or known answers for
this path (its only checks print, they do not assert), and its native modules cannot be
built against this PyTorch/CUDA (PyTorch 1.5 internals, cuDNN 7 API).  The oracle is
pinned instead against fixtures generated from PyTorch CPU by tests/golden/make_golden.py,
and its two max-pool forms are checked against each other.
"""
from __future__ import annotations

import numpy as np
import torch
import torch.nn.functional as F


# ------------------------------------------------------------------ ReLU + 1-bit mask

def relu_mask_bytes(x: torch.Tensor) -> np.ndarray:
    """pack_kernel (pack.cu:22-31) applied to (x > 0).view(-1) (relu.py:103-104):
    element 8j+k -> bit 7-k of byte j, ceil(n/8) bytes, tail bits zero."""
    flags = (x.detach().cpu().contiguous().view(-1) > 0).numpy()
    return np.packbits(flags, bitorder="big")


def relu_forward(x: torch.Tensor) -> torch.Tensor:
    return torch.relu(x)


def relu_backward(dy: torch.Tensor, saved: torch.Tensor) -> torch.Tensor:
    """threshold_kernel (lrrelu.cu:4-9): dy where saved > 0 else 0."""
    return torch.where(saved > 0, dy, torch.zeros_like(dy))


def unpack_bits(packed: np.ndarray, n: int) -> np.ndarray:
    """unpack_kernel (pack.cu:32-40)."""
    return np.unpackbits(packed, bitorder="big")[:n].astype(bool)


# ------------------------------------------------------------------ nibble packing

def pack_nibbles(idx: np.ndarray) -> np.ndarray:
    """pack_two_kernel (pack.cu:3-12): out[j] = idx[2j] << 4 | idx[2j+1] (uint8 wrap),
    an odd tail leaves the low nibble 0."""
    idx = np.asarray(idx, dtype=np.uint8).reshape(-1)
    n = idx.size
    padded = np.zeros(((n + 1) // 2) * 2, dtype=np.uint8)
    padded[:n] = idx
    return ((padded[0::2].astype(np.uint16) << 4) | padded[1::2]).astype(np.uint8)


def unpack_nibbles(packed: np.ndarray, n: int) -> np.ndarray:
    """unpack_two_kernel (pack.cu:13-21)."""
    packed = np.asarray(packed, dtype=np.uint8)
    out = np.empty(packed.size * 2, dtype=np.uint8)
    out[0::2] = packed >> 4
    out[1::2] = packed & 15
    return out[:n]


# ------------------------------------------------------------------ max pool

def _pair(v):
    if isinstance(v, (list, tuple)):
        return (int(v[0]), int(v[0])) if len(v) == 1 else (int(v[0]), int(v[1]))
    return int(v), int(v)


def maxpool_local_index(x: torch.Tensor, kernel, stride, padding, dilation=1, ceil_mode=False):
    """Loop restatement of max_pool_forward_nchw (maxpool.cu:26-72) for small inputs.

    Returns (y, idx) with idx[n,c,ph,pw] = i*kw + j of the winning tap counted from the
    unclipped window origin; strict '>' (first maximum wins), a NaN always wins."""
    kh, kw = _pair(kernel); sh, sw = _pair(stride); ph_, pw_ = _pair(padding); dh, dw = _pair(dilation)
    xn = x.detach().cpu().numpy()
    N, C, H, W = xn.shape
    P = F.max_pool2d(x[:1, :1].cpu(), (kh, kw), (sh, sw), (ph_, pw_), (dh, dw), ceil_mode).shape[2]
    Q = F.max_pool2d(x[:1, :1].cpu(), (kh, kw), (sh, sw), (ph_, pw_), (dh, dw), ceil_mode).shape[3]
    y = np.empty((N, C, P, Q), dtype=np.float32)
    idx = np.zeros((N, C, P, Q), dtype=np.uint8)
    for n in range(N):
        for c in range(C):
            for p in range(P):
                for q in range(Q):
                    best, bi, first = -np.inf, 0, True
                    for i in range(kh):
                        h = p * sh - ph_ + i * dh
                        if h < 0 or h >= H:
                            continue
                        for j in range(kw):
                            w = q * sw - pw_ + j * dw
                            if w < 0 or w >= W:
                                continue
                            v = xn[n, c, h, w]
                            if first:
                                bi, first = i * kw + j, False
                            if v > best or np.isnan(v):
                                best, bi = v, i * kw + j
                    y[n, c, p, q] = best
                    idx[n, c, p, q] = bi
    return torch.from_numpy(y), idx


def maxpool_forward(x: torch.Tensor, kernel, stride, padding, dilation=1, ceil_mode=False):
    """(y, local idx uint8 [N,C,P,Q]) from torch's max_pool2d global indices h*W+w:
    local = ((h - (ph*sh - pad_h)) / dh) * kw + (w - (pw*sw - pad_w)) / dw  (maxpool.cu:38-61)."""
    kh, kw = _pair(kernel); sh, sw = _pair(stride); ph_, pw_ = _pair(padding); dh, dw = _pair(dilation)
    xc = x.detach().cpu().contiguous()
    y, g = F.max_pool2d(xc, (kh, kw), (sh, sw), (ph_, pw_), (dh, dw), ceil_mode, return_indices=True)
    W = xc.shape[3]
    P, Q = y.shape[2], y.shape[3]
    h = (g // W).numpy(); w = (g % W).numpy()
    h0 = (np.arange(P) * sh - ph_).reshape(1, 1, P, 1)
    w0 = (np.arange(Q) * sw - pw_).reshape(1, 1, 1, Q)
    local = ((h - h0) // dh) * kw + (w - w0) // dw
    assert local.min() >= 0 and local.max() < kh * kw
    return y, local.astype(np.uint8)


def maxpool_nibbles(local_idx: np.ndarray, nhwc: bool = False) -> np.ndarray:
    """Packed nibbles in the physical element order of y (pool.py:48-50 flattens NCHW)."""
    a = local_idx.transpose(0, 2, 3, 1) if nhwc else local_idx
    return pack_nibbles(np.ascontiguousarray(a).reshape(-1))


def maxpool_backward_from_index(dy: torch.Tensor, local_idx: np.ndarray, in_shape, kernel, stride,
                                padding, dilation=1) -> torch.Tensor:
    """max_pool_backward_nchw (maxpool.cu:81-131) as a scatter-add: every output adds its
    gradient to the input pixel its stored local index points at."""
    kh, kw = _pair(kernel); sh, sw = _pair(stride); ph_, pw_ = _pair(padding); dh, dw = _pair(dilation)
    N, C, H, W = in_shape
    P, Q = local_idx.shape[2], local_idx.shape[3]
    i = (local_idx // kw).astype(np.int64); j = (local_idx % kw).astype(np.int64)
    h = (np.arange(P) * sh - ph_).reshape(1, 1, P, 1) + i * dh
    w = (np.arange(Q) * sw - pw_).reshape(1, 1, 1, Q) + j * dw
    flat = torch.from_numpy(h * W + w).reshape(N, C, P * Q)
    dx = torch.zeros(N, C, H * W, dtype=dy.dtype)
    dx.scatter_add_(2, flat, dy.detach().cpu().contiguous().reshape(N, C, P * Q))
    return dx.reshape(N, C, H, W)


# ------------------------------------------------------------------ batch norm

def bn_forward_train(x, gamma, beta, running_mean, running_var, momentum=0.1, eps=1e-5):
    """(y, save_mean, save_invstd, new_running_mean, new_running_var): F.batch_norm in training
    mode plus the statistics cuDNN saves (lrbn.cpp:32-40): batch mean and 1/sqrt(biased var + eps)."""
    x = x.detach().cpu()
    rm, rv = running_mean.clone().cpu(), running_var.clone().cpu()
    y = F.batch_norm(x, rm, rv, gamma.cpu(), beta.cpu(), True, momentum, eps)
    dims = [0] + list(range(2, x.dim()))
    xd = x.double()
    mean = xd.mean(dims)
    var = xd.var(dims, unbiased=False)
    return y, mean.float(), (1.0 / torch.sqrt(var + eps)).float(), rm, rv


def bn_forward_apply(x, gamma, beta, mean, invstd):
    shape = [1, -1] + [1] * (x.dim() - 2)
    return (x.cpu() - mean.view(shape)) * (invstd * gamma).view(shape) + beta.view(shape)


def bn_backward_from_input(dy, x, gamma, eps=1e-5):
    """(dx, dgamma, dbeta) by autograd through F.batch_norm(training=True)."""
    xr = x.detach().cpu().clone().requires_grad_(True)
    g = gamma.detach().cpu().clone().requires_grad_(True)
    b = torch.zeros_like(g).requires_grad_(True)
    y = F.batch_norm(xr, None, None, g, b, True, 0.0, eps)
    y.backward(dy.detach().cpu())
    return xr.grad, g.grad, b.grad


def bn_backward_from_output(dy, y, gamma, beta, save_invstd):
    """batch_norm_backward_kernel1 (lrbn.cu:153-208), fp64 accumulation:
    c = y - beta; S1 = sum dy; S2 = sum dy*c; dgamma = S2/gamma; dbeta = S1;
    dx = (dy - c*S2/(M*gamma^2) - S1/M) * invstd * gamma."""
    dy, y = dy.detach().cpu().double(), y.detach().cpu().double()
    dims = [0] + list(range(2, y.dim()))
    shape = [1, -1] + [1] * (y.dim() - 2)
    g, b, inv = gamma.double().cpu(), beta.double().cpu(), save_invstd.double().cpu()
    M = y.numel() // y.shape[1]
    c = y - b.view(shape)
    S1 = dy.sum(dims)
    S2 = (dy * c).sum(dims)
    dx = (dy - c * (S2 / (M * g * g)).view(shape) - (S1 / M).view(shape)) * (inv * g).view(shape)
    return dx.float(), (S2 / g).float(), S1.float()


# ------------------------------------------ fused batch norm / add / ReLU forms
# The reference has these only as chains of separate operators; the oracle is that chain.

def bn_act_forward_train(x, residual, relu, gamma, beta, running_mean, running_var,
                         momentum=0.1, eps=1e-5):
    """bn.py forward, then funcs.py add of `residual` (may be None), then relu.py forward."""
    y, mean, invstd, rm, rv = bn_forward_train(x, gamma, beta, running_mean, running_var,
                                               momentum, eps)
    if residual is not None:
        y = y + residual.detach().cpu()
    if relu:
        y = relu_forward(y)
    return y, mean, invstd, rm, rv


def bn_relu_backward_from_input(dy, gate, x, gamma, eps=1e-5):
    """relu.py backward with the given boolean gate (y > 0 of the forward), then batch-norm
    backward from the input."""
    dy = dy.detach().cpu() * gate.detach().cpu().to(dy.dtype)
    return bn_backward_from_input(dy, x, gamma, eps)


def relu_backward_sum2(dy1, dy2, saved):
    """Two incoming gradients summed (schedule.py:296-301), then relu.py backward."""
    return relu_backward(dy1.detach().cpu() + dy2.detach().cpu(), saved)


# ------------------------------------------------------------------ softmax / CE

def softmax_forward(x, dim, log=False):
    return F.log_softmax(x.cpu(), dim) if log else F.softmax(x.cpu(), dim)


def softmax_backward(dy, y, dim, log=False):
    """softmax: y*(dy - sum(dy*y)) (softmax.cpp:17-33); log-softmax: dy - exp(y)*sum(dy)."""
    dy, y = dy.cpu(), y.cpu()
    if log:
        return dy - torch.exp(y) * dy.sum(dim, keepdim=True)
    return y * (dy - (dy * y).sum(dim, keepdim=True))


def cross_entropy(logits, labels, grad_scale):
    """(per-position loss, dlogits) of nn.CrossEntropyLoss(reduction='none'), gradient scaled."""
    lg = logits.detach().cpu().clone().requires_grad_(True)
    loss = F.cross_entropy(lg, labels.cpu(), reduction="none")
    loss.sum().backward()
    return loss.detach(), lg.grad * grad_scale


# ------------------------------------------------------------------ glue

def hardtanh_backward(dy, saved, lo, hi):
    """at::hardtanh_backward (lrhardtanh.cpp:11): zero where saved <= lo or saved >= hi."""
    return torch.where((saved > lo) & (saved < hi), dy, torch.zeros_like(dy))


def add_forward(a, b, alpha):
    return torch.add(a, b, alpha=alpha)


def global_avgpool_backward(dy, shape):
    N, C, H, W = shape
    return (dy.reshape(N, C, 1, 1) / (H * W)).expand(N, C, H, W).contiguous()


# ------------------------------------------------------------------ convolution

def conv_forward(x, w, bias, stride, padding, dilation=1, groups=1):
    """fp32 F.conv2d; the bias is added after the convolution (conv.py:284-285)."""
    y = F.conv2d(x.cpu(), w.cpu(), None, stride, padding, dilation, groups)
    if bias is not None:
        y = y + bias.cpu().view(1, -1, 1, 1)
    return y


def conv_backward(dy, x, w, stride, padding, dilation=1, groups=1, need=(True, True, True)):
    """(dx, dw, db): the three passes SpecificAlgoConvolution.backward runs (conv.py:288-329);
    db = dy.sum([0, 2, 3]) (conv.py:313-314)."""
    xr = x.detach().cpu().clone().requires_grad_(need[0])
    wr = w.detach().cpu().clone().requires_grad_(need[1])
    y = F.conv2d(xr, wr, None, stride, padding, dilation, groups)
    y.backward(dy.detach().cpu())
    db = dy.detach().cpu().sum([0, 2, 3]) if need[2] else None
    return xr.grad, wr.grad, db


# ------------------------------------------------------------------ the stem (BASELINE config 1)

def stem_reference(seed=0, N=4, H=224, W=224):
    """conv7x7/2 (3->64, no bias) -> BN(64, train) -> ReLU -> maxpool 3x3/2 pad 1, forward and
    backward, on the seeded inputs of the CPU-runnable configuration.  Returns a dict of every
    tensor the parity test compares."""
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(N, 3, H, W, generator=g)
    w = torch.empty(64, 3, 7, 7)
    std = (2.0 / (64 * 7 * 7)) ** 0.5          # kaiming_normal_(mode='fan_out', relu)
    w.normal_(0.0, std, generator=g)
    gamma, beta = torch.ones(64), torch.zeros(64)
    P, Q = (H + 6 - 7) // 2 + 1, (W + 6 - 7) // 2 + 1      # conv / BN / ReLU extent
    Pp, Qp = (P + 2 - 3) // 2 + 1, (Q + 2 - 3) // 2 + 1    # pooled extent
    dy = torch.randn(N, 64, Pp, Qp, generator=g)
    xr = x.clone().requires_grad_(True)
    wr = w.clone().requires_grad_(True)
    gr = gamma.clone().requires_grad_(True)
    br = beta.clone().requires_grad_(True)
    c = F.conv2d(xr, wr, None, 2, 3)
    b = F.batch_norm(c, None, None, gr, br, True, 0.1, 1e-5)
    r = torch.relu(b)
    y, gi = F.max_pool2d(r, 3, 2, 1, return_indices=True)
    y.backward(dy)
    _, local = maxpool_forward(r.detach(), 3, 2, 1)
    return dict(x=x, w=w, gamma=gamma, beta=beta, dy=dy, conv=c.detach(), bn=b.detach(),
                relu=r.detach(), y=y.detach(), dx=xr.grad, dw=wr.grad, dgamma=gr.grad,
                dbeta=br.grad, mask=relu_mask_bytes(b.detach()), local_idx=local,
                nibbles=maxpool_nibbles(local))
