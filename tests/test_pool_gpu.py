"""Max-pool parity: values rtol 1e-5, packed window-local argmax nibbles bit-exact,
backward from the nibbles against autograd."""
import numpy as np
import pytest
import torch
import torch.nn.functional as TF

from oracle import lm_ops_oracle as oracle

pytestmark = pytest.mark.gpu

CASES = [
    # N, C, H, W, kernel, stride, padding, dilation, ceil
    (2, 3, 9, 11, 3, 2, 1, 1, False),
    (1, 1, 4, 4, 2, 2, 0, 1, False),
    (2, 8, 13, 13, 3, 2, 1, 1, False),      # C % 8 == 0 -> vector NHWC path
    (2, 16, 12, 10, 2, 2, 0, 1, False),
    (1, 8, 7, 7, 3, 1, 1, 1, False),
    (2, 5, 10, 9, 3, 2, 0, 1, True),        # ceil mode, ragged last window
    (1, 8, 9, 9, (2, 3), (2, 1), (1, 1), 1, False),
    (1, 4, 11, 11, 3, 2, 1, 2, False),      # dilation
    (3, 24, 1, 1, 1, 1, 0, 1, False),
    (2, 8, 6, 6, 4, 4, 0, 1, False),        # 16 taps: the largest window a nibble holds
]


def _check(cuda, x, k, s, p, d, ceil, nhwc):
    from monet_b200 import functional as F
    xg = x.to(cuda)
    if nhwc:
        xg = xg.contiguous(memory_format=torch.channels_last)
    y, nib, desc = F.maxpool2d(xg, k, s, p, d, ceil)
    ref_y, local = oracle.maxpool_forward(x, k, s, p, d, ceil)
    assert y.shape == ref_y.shape
    assert torch.allclose(y.cpu(), ref_y, rtol=1e-5, atol=0, equal_nan=True)
    layout_nhwc = F.is_nhwc(y)
    assert np.array_equal(nib.cpu().numpy(), oracle.maxpool_nibbles(local, nhwc=layout_nhwc))
    g = torch.Generator().manual_seed(1)
    dy = torch.randn(ref_y.shape, generator=g)
    dx = F.maxpool2d_bwd(dy.to(cuda), nib, desc)
    ref_dx = oracle.maxpool_backward_from_index(dy, local, x.shape, k, s, p, d)
    assert torch.allclose(dx.cpu(), ref_dx, rtol=1e-5, atol=1e-6)
    xr = x.clone().requires_grad_(True)
    TF.max_pool2d(xr, k, s, p, d, ceil).backward(dy)
    assert torch.allclose(dx.cpu(), xr.grad, rtol=1e-5, atol=1e-6)


@pytest.mark.parametrize("case", CASES)
@pytest.mark.parametrize("nhwc", [False, True])
def test_maxpool_parity(cuda, case, nhwc):
    N, C, H, W, k, s, p, d, ceil = case
    g = torch.Generator().manual_seed(N * 1000 + C)
    _check(cuda, torch.randn(N, C, H, W, generator=g), k, s, p, d, ceil, nhwc)


@pytest.mark.parametrize("nhwc", [False, True])
def test_maxpool_ties_and_nan(cuda, nhwc):
    """Ties keep the first maximum; a NaN always wins (maxpool.cu:60)."""
    x = torch.zeros(1, 8, 6, 6)
    x[0, 1] = 1.0
    x[0, 2, 2, 2] = float("nan")
    x[0, 3] = float("-inf")
    _check(cuda, x, 3, 2, 1, 1, False, nhwc)


def test_maxpool_loop_restatement_agrees(cuda):
    x = torch.randn(1, 2, 7, 8)
    _, a = oracle.maxpool_local_index(x, 3, 2, 1)
    _, b = oracle.maxpool_forward(x, 3, 2, 1)
    assert np.array_equal(a, b)


@pytest.mark.parametrize("nhwc", [False, True])
def test_maxpool_resnet_stem_size(cuda, nhwc):
    """The 4x64x112x112 -> 56x56 pool of the CPU-runnable configuration, 401 408 nibble bytes."""
    g = torch.Generator().manual_seed(0)
    x = torch.randn(4, 64, 112, 112, generator=g)
    _check(cuda, x, 3, 2, 1, 1, False, nhwc)


def test_pool_ops_protocol(cuda):
    from monet_b200.lm_ops import pool as P
    x = torch.randn(2, 8, 10, 10)
    dy = torch.randn(2, 8, 5, 5)
    xr = x.clone().requires_grad_(True)
    ref = TF.max_pool2d(xr, 3, 2, 1)
    ref.backward(dy)
    op = P.IndicesActMaxPool2D()
    y, nib = op.forward(x.to(cuda), [3, 3], [2, 2], [1, 1], [1, 1], False)
    assert nib.numel() == op.backward_storage.size(tuple(y.shape))
    stored = [nib]
    dx = op.backward(dy.to(cuda), stored)
    assert stored == [] and torch.equal(y.cpu(), ref.detach())
    assert torch.allclose(dx.cpu(), xr.grad, rtol=1e-5, atol=1e-6)
    op = P.SimpleMaxPool2D()
    y = op.forward(x.to(cuda), [3, 3], [2, 2], [1, 1], [1, 1], False)
    stored = [x.to(cuda)]
    dx = op.backward(dy.to(cuda), stored)
    assert stored == [] and torch.equal(y.cpu(), ref.detach())
    assert torch.allclose(dx.cpu(), xr.grad, rtol=1e-5, atol=1e-6)


def test_pool_rejects_big_window(cuda):
    from monet_b200 import functional as F
    with pytest.raises(RuntimeError, match="4-bit"):
        F.maxpool2d(torch.randn(1, 1, 9, 9, device=cuda), 5, 1, 0, 1, False)
