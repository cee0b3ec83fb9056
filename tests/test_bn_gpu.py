"""Batch-norm parity (rtol 1e-5 fp32): training forward and saved statistics, cached-statistics
forward, backward from the stored input and from the stored output."""
import pytest
import torch

from oracle import lm_ops_oracle as oracle

pytestmark = pytest.mark.gpu

RTOL, ATOL = 1e-5, 2e-6
SHAPES = [
    (4, 64, 14, 14), (2, 3, 5, 7), (3, 24, 9, 9), (2, 2048, 7, 7), (1, 8, 1, 1), (5, 96, 3, 3),
    (16, 256, 28, 28), (2, 1, 4, 4), (2, 516, 2, 3),
]


def _data(shape, seed=0, offset=0.0):
    g = torch.Generator().manual_seed(seed)
    C = shape[1]
    x = torch.randn(shape, generator=g) * 1.7 + offset
    gamma = torch.rand(C, generator=g) + 0.5
    beta = torch.randn(C, generator=g)
    rm = torch.randn(C, generator=g)
    rv = torch.rand(C, generator=g) + 0.5
    dy = torch.randn(shape, generator=g)
    return x, gamma, beta, rm, rv, dy


def _fmt(t, nhwc):
    return t.contiguous(memory_format=torch.channels_last) if nhwc and t.dim() == 4 else t


@pytest.mark.parametrize("shape", SHAPES)
@pytest.mark.parametrize("nhwc", [False, True])
@pytest.mark.parametrize("inplace", [False, True])
def test_bn_forward(cuda, shape, nhwc, inplace):
    from monet_b200 import functional as F
    if shape[0] * shape[2] * shape[3] == 1:
        pytest.skip("batch statistics of a single value")
    x, gamma, beta, rm, rv, _ = _data(shape)
    ref_y, ref_mean, ref_invstd, ref_rm, ref_rv = oracle.bn_forward_train(x, gamma, beta, rm, rv, 0.1, 1e-5)
    xg = _fmt(x.to(cuda), nhwc)
    rmg, rvg = rm.to(cuda), rv.to(cuda)
    y, mean, invstd = F.bn_fwd_train(xg, gamma.to(cuda), beta.to(cuda), rmg, rvg, 0.1, 1e-5, inplace=inplace)
    assert (y.data_ptr() == xg.data_ptr()) == inplace
    assert torch.allclose(y.cpu(), ref_y, rtol=RTOL, atol=1e-5)
    assert torch.allclose(mean.cpu(), ref_mean, rtol=RTOL, atol=ATOL)
    assert torch.allclose(invstd.cpu(), ref_invstd, rtol=RTOL, atol=ATOL)
    assert torch.allclose(rmg.cpu(), ref_rm, rtol=RTOL, atol=ATOL)
    assert torch.allclose(rvg.cpu(), ref_rv, rtol=RTOL, atol=ATOL)
    # recompute forward with the cached statistics reproduces y
    y2 = F.bn_fwd_apply(_fmt(x.to(cuda), nhwc), gamma.to(cuda), beta.to(cuda), mean, invstd)
    assert torch.allclose(y2.cpu(), ref_y, rtol=RTOL, atol=1e-5)


@pytest.mark.parametrize("shape", SHAPES)
@pytest.mark.parametrize("nhwc", [False, True])
def test_bn_backward_both_ways(cuda, shape, nhwc):
    from monet_b200 import functional as F
    if shape[0] * shape[2] * shape[3] == 1:
        pytest.skip("batch statistics of a single value")
    x, gamma, beta, rm, rv, dy = _data(shape, seed=1)
    ref_dx, ref_dg, ref_db = oracle.bn_backward_from_input(dy, x, gamma, 1e-5)
    scale = max(1.0, float(ref_dx.abs().max()))
    xg = _fmt(x.to(cuda), nhwc)
    y, mean, invstd = F.bn_fwd_train(xg, gamma.to(cuda), beta.to(cuda), None, None, 0.1, 1e-5)
    dyg = _fmt(dy.to(cuda), nhwc)
    dx, dg, db = F.bn_bwd_from_input(dyg, xg, gamma.to(cuda), mean, invstd)
    assert torch.allclose(dx.cpu(), ref_dx, rtol=RTOL, atol=1e-5 * scale)
    assert torch.allclose(dg.cpu(), ref_dg, rtol=1e-4, atol=1e-4)
    assert torch.allclose(db.cpu(), ref_db, rtol=1e-4, atol=1e-4)
    dx2, dg2, db2 = F.bn_bwd_from_output(dyg, y, gamma.to(cuda), beta.to(cuda), invstd)
    o_dx, o_dg, o_db = oracle.bn_backward_from_output(dy, y.cpu(), gamma, beta, invstd.cpu())
    assert torch.allclose(dx2.cpu(), o_dx, rtol=RTOL, atol=1e-5 * scale)
    assert torch.allclose(dx2.cpu(), ref_dx, rtol=1e-4, atol=1e-4 * scale)
    assert torch.allclose(dg2.cpu(), ref_dg, rtol=1e-4, atol=1e-4)
    assert torch.allclose(db2.cpu(), ref_db, rtol=1e-4, atol=1e-4)


def test_bn_large_mean_does_not_cancel(cuda):
    """|mean| >> std: the shifted accumulation keeps the variance accurate."""
    from monet_b200 import functional as F
    x, gamma, beta, rm, rv, _ = _data((8, 32, 20, 20), seed=3, offset=300.0)
    ref_y, ref_mean, ref_invstd, _, _ = oracle.bn_forward_train(x, gamma, beta, rm, rv)
    for nhwc in (False, True):
        y, mean, invstd = F.bn_fwd_train(_fmt(x.to(cuda), nhwc), gamma.to(cuda), beta.to(cuda), None, None, 0.1, 1e-5)
        assert torch.allclose(invstd.cpu(), ref_invstd, rtol=1e-4)
        assert torch.allclose(y.cpu(), ref_y, rtol=1e-3, atol=1e-3)


@pytest.mark.parametrize("nhwc", [False, True])
def test_bn_stem_size(cuda, nhwc):
    """4x64x112x112, the BN of the CPU-runnable configuration."""
    from monet_b200 import functional as F
    x, gamma, beta, rm, rv, dy = _data((4, 64, 112, 112), seed=0)
    gamma, beta = torch.ones(64), torch.zeros(64)
    ref_y, ref_mean, ref_invstd, _, _ = oracle.bn_forward_train(x, gamma, beta, rm, rv)
    xg = _fmt(x.to(cuda), nhwc)
    y, mean, invstd = F.bn_fwd_train(xg, gamma.to(cuda), beta.to(cuda), rm.to(cuda), rv.to(cuda), 0.1, 1e-5)
    assert torch.allclose(y.cpu(), ref_y, rtol=RTOL, atol=1e-5)
    ref_dx, ref_dg, ref_db = oracle.bn_backward_from_input(dy, x, gamma)
    dx, dg, db = F.bn_bwd_from_output(_fmt(dy.to(cuda), nhwc), y, gamma.to(cuda), beta.to(cuda), invstd)
    assert torch.allclose(dx.cpu(), ref_dx, rtol=RTOL, atol=1e-5)
    assert torch.allclose(dg.cpu(), ref_dg, rtol=1e-4, atol=1e-3)
    assert torch.allclose(db.cpu(), ref_db, rtol=1e-4, atol=1e-3)


def test_bn_ops_protocol(cuda):
    """Both operator classes through the executor's calling convention, including the
    statistics cache that a recomputation reuses (params carried between instances)."""
    from monet_b200.lm_ops import bn as B
    x, gamma, beta, rm, rv, dy = _data((4, 16, 6, 6), seed=5)
    ref_y, _, _, ref_rm, ref_rv = oracle.bn_forward_train(x, gamma, beta, rm, rv)
    ref_dx, ref_dg, ref_db = oracle.bn_backward_from_input(dy, x, gamma)
    for cls in (B.InputActBatchNorm, B.OutputActBatchNorm):
        rmg, rvg = rm.to(cuda), rv.to(cuda)
        args = [x.to(cuda), gamma.to(cuda), beta.to(cuda), rmg, rvg, True, 0.1, 1e-5, True]
        op = cls()
        y = op.forward(*args)
        assert torch.allclose(y.cpu(), ref_y, rtol=RTOL, atol=1e-5)
        assert torch.allclose(rmg.cpu(), ref_rm, rtol=RTOL, atol=ATOL)
        again = cls(); again.params = op.params
        y2 = again.forward(*args)                       # recompute: statistics not updated twice
        assert torch.allclose(y2.cpu(), ref_y, rtol=RTOL, atol=1e-5)
        assert torch.allclose(rmg.cpu(), ref_rm, rtol=RTOL, atol=ATOL)
        if cls is B.InputActBatchNorm:
            stored = [args[0], args[1], args[2], rmg, rvg]
        else:
            stored = [args[1], args[2], rmg, rvg, y]
        out = again.backward(dy.to(cuda), stored)
        assert stored == [] and len(out) == 5 and out[3] is None and out[4] is None
        assert torch.allclose(out[0].cpu(), ref_dx, rtol=1e-4, atol=1e-5)
        assert torch.allclose(out[1].cpu(), ref_dg, rtol=1e-4, atol=1e-4)
        assert torch.allclose(out[2].cpu(), ref_db, rtol=1e-4, atol=1e-4)


def test_bn_workspace_too_small_is_an_error(cuda):
    import ctypes as C
    from monet_b200 import _lib
    d = _lib.BnDesc(4, 16, 36, 0, 1e-5, 0.1)
    x = torch.randn(4, 16, 6, 6, device=cuda)
    v = torch.ones(16, device=cuda)
    rc = _lib.lib().mb_bn_fwd_train(x.data_ptr(), v.data_ptr(), v.data_ptr(), None, None,
                                    x.data_ptr(), v.data_ptr(), v.data_ptr(), C.byref(d), None, 0, None)
    assert rc == 3 and "workspace" in _lib.last_error()
