"""Operator-protocol tests on the GPU for the convolution classes the reference offers besides
the solver-driven one (monet/lm_ops/conv.py:11-39,105-258,288-329), the ``algorithm`` encoding
of the backward passes (schedule.py:123-139), and concatenation (cat.py:5-29)."""
import sys
import types

import pytest
import torch

from oracle import lm_ops_oracle as oracle

pytestmark = pytest.mark.gpu


def _rel(a, ref):
    return float((a.cpu() - ref).abs().max() / ref.abs().max().clamp_min(1e-6))


def _case(cuda, seed=0):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(6, 64, 14, 14, generator=g)
    w = torch.randn(96, 64, 3, 3, generator=g) * 0.06
    b = torch.randn(96, generator=g)
    dy = torch.randn(6, 96, 14, 14, generator=g)
    return x, w, b, dy


CONV_ARGS = ([1, 1], [1, 1], [1, 1], False, [0, 0], 1)


@pytest.mark.parametrize("algorithm", [0, 1, 10, 11, 20, 21, -1])
def test_specific_algo_convolution_decodes_algorithm(cuda, algorithm):
    """convtype = algorithm // 10 (0: weights and bias only, 1: input only, 2: both),
    variant = algorithm % 10; a variant the pass does not have falls back to the default
    (conv.py:279-283,308-312,321-325)."""
    from monet_b200 import lm_ops
    x, w, b, dy = _case(cuda)
    ref_dx, ref_dw, ref_db = oracle.conv_backward(dy, x, w, 1, 1, 1)
    op = lm_ops.list_ops("conv_multiway_newnode", "aten::_convolution")[0]()
    assert type(op).__name__ == "SpecificAlgoConvolution"
    xg = x.to(cuda).requires_grad_(True)
    wg = w.to(cuda).requires_grad_(True)
    bg = b.to(cuda).requires_grad_(True)
    op.algorithm = 0
    y = op.forward(xg, wg, bg, *CONV_ARGS)
    assert _rel(y, oracle.conv_forward(x, w, b, 1, 1, 1)) < 2e-2
    op.algorithm = algorithm
    stored = [xg, wg]
    di, dw, db = op.backward(dy.to(cuda), stored)
    assert stored == []                                   # consumed (schedule.py relies on it)
    convtype = 2 if algorithm < 0 else algorithm // 10
    if convtype in (0, 2):
        assert _rel(dw, ref_dw) < 2e-2 and torch.allclose(db.cpu(), ref_db, rtol=1e-4, atol=1e-3)
    else:
        assert dw is None and db is None
    if convtype in (1, 2):
        assert _rel(di, ref_dx) < 2e-2
    else:
        assert di is None
    # nodel=True keeps the caller's list (the profiler's calls, meminfo.py:156)
    stored = [xg, wg]
    op.backward(dy.to(cuda), stored, nodel=True)
    assert len(stored) == 2
    # the two-step form the executor uses: step t-1 gets (x, w), step t only w
    op.algorithm = 10
    di2, dw2, _ = op.backward(dy.to(cuda), [None, wg])
    assert dw2 is None and _rel(di2, ref_dx) < 2e-2


def test_greedy_convolution_autotunes_under_the_budget(cuda):
    """First forward / backward time every variant and keep the fastest that stays under
    config.budget (conv.py:127-148,178-204,214-242); a budget nothing fits raises."""
    from monet_b200 import lm_ops
    cfg = sys.modules.get("config") or types.ModuleType("config")
    sys.modules["config"] = cfg
    old = getattr(cfg, "budget", None)
    try:
        cfg.budget = 64.0                                  # GB: everything fits
        x, w, b, dy = _case(cuda, 1)
        op = lm_ops.list_ops("normal", "aten::_convolution")[0]()
        assert type(op).__name__ == "GreedyAlgoConvolution"
        xg, wg = x.to(cuda).requires_grad_(True), w.to(cuda).requires_grad_(True)
        y = op.forward(xg, wg, None, *CONV_ARGS)
        assert op.fwd_algo == 0
        assert _rel(y, oracle.conv_forward(x, w, None, 1, 1, 1)) < 2e-2
        di, dw = op.backward(dy.to(cuda), [xg, wg])
        assert op.bwd_wt_algo in (0, 1) and op.bwd_ip_algo == 0
        ref_dx, ref_dw, _ = oracle.conv_backward(dy, x, w, 1, 1, 1)
        assert _rel(di, ref_dx) < 2e-2 and _rel(dw, ref_dw) < 2e-2
        # tuned once: the choices stick
        chosen = (op.fwd_algo, op.bwd_wt_algo, op.bwd_ip_algo)
        op.forward(xg, wg, None, *CONV_ARGS)
        op.backward(dy.to(cuda), [xg, wg])
        assert (op.fwd_algo, op.bwd_wt_algo, op.bwd_ip_algo) == chosen
        cfg.budget = 1e-6                                  # nothing fits
        op2 = lm_ops.list_ops("normal", "aten::_convolution")[0]()
        with pytest.raises(RuntimeError, match="budget"):
            op2.forward(xg, wg, None, *CONV_ARGS)
    finally:
        if old is None:
            if hasattr(cfg, "budget"):
                del cfg.budget
        else:
            cfg.budget = old


def test_pytorch_convolution_default_variant(cuda):
    from monet_b200 import lm_ops
    x, w, b, dy = _case(cuda, 2)
    op = lm_ops.list_ops("none", "aten::_convolution")[0]()
    assert type(op).__name__ == "PytorchConvolution"
    xg, wg, bg = (t.to(cuda).requires_grad_(True) for t in (x, w, b))
    y = op.forward(xg, wg, bg, *CONV_ARGS)
    assert _rel(y, oracle.conv_forward(x, w, b, 1, 1, 1)) < 2e-2
    di, dw, db = op.backward(dy.to(cuda), [xg, wg])
    ref_dx, ref_dw, ref_db = oracle.conv_backward(dy, x, w, 1, 1, 1)
    assert _rel(di, ref_dx) < 2e-2 and _rel(dw, ref_dw) < 2e-2
    assert torch.allclose(db.cpu(), ref_db, rtol=1e-4, atol=1e-3)


@pytest.mark.parametrize("geom", [
    # N, C_in, H, W, C_out, R, stride, pad, output_padding
    (3, 64, 13, 19, 32, 2, 2, 0, 0),      # UNet's 2x2 stride-2 up-convolution
    (2, 128, 7, 7, 64, 2, 2, 0, 0),
    (2, 32, 9, 9, 16, 3, 2, 1, 1),        # 3x3 stride 2 with output padding (doubles the extent)
    (2, 16, 10, 12, 24, 3, 1, 1, 0),      # stride 1
    (2, 64, 6, 6, 2, 2, 2, 0, 0),         # two output channels (padded to 4 inside)
])
def test_transposed_convolution_on_the_convolution_kernels(cuda, geom):
    """Beyond the reference (conv.py:269 asserts `not transposed`): forward = backward-data
    kernel, backward-data = forward kernel, backward-filter with the operands exchanged.  Against
    torch's CPU conv_transpose2d and autograd at the convolution tolerance."""
    from monet_b200 import functional as F
    from monet_b200 import lm_ops
    N, Ci, H, W, Co, R, s, p, op_ = geom
    g = torch.Generator().manual_seed(13)
    x = torch.randn(N, Ci, H, W, generator=g)
    w = torch.randn(Ci, Co, R, R, generator=g) * (Ci * R * R) ** -0.5
    b = torch.randn(Co, generator=g)
    xr, wr, br = (t.clone().requires_grad_(True) for t in (x, w, b))
    ref = torch.nn.functional.conv_transpose2d(xr, wr, br, s, p, op_)
    dy = torch.randn(ref.shape, generator=g)
    ref.backward(dy)
    op = lm_ops.list_ops("conv_multiway_newnode", "aten::_convolution")[0]()
    xg, wg, bg = (t.to(cuda).requires_grad_(True) for t in (x, w, b))
    y = op.forward(xg, wg, bg, [s, s], [p, p], [1, 1], True, [op_, op_], 1)
    assert tuple(y.shape) == tuple(ref.shape)
    assert _rel(y, ref.detach()) < 2e-2
    op.algorithm = 20
    di, dw, db = op.backward(dy.to(cuda), [xg, wg])
    assert _rel(di, xr.grad) < 2e-2, _rel(di, xr.grad)
    assert _rel(dw, wr.grad) < 2e-2, _rel(dw, wr.grad)
    assert torch.allclose(db.cpu(), br.grad, rtol=1e-4, atol=1e-3)
    assert F.conv_device_status() == 0


@pytest.mark.parametrize("nhwc", [False, True])
@pytest.mark.parametrize("shapes,dim", [
    ([(3, 8, 5, 7), (3, 12, 5, 7)], 1),            # UNet's skip concatenation
    ([(2, 3, 4, 6), (2, 5, 4, 6), (2, 1, 4, 6)], 1),   # widths that are not multiples of 4
    ([(2, 4, 3, 8), (2, 4, 5, 8)], 2),
    ([(2, 4, 3, 8), (1, 4, 3, 8)], 0),
    ([(4, 16), (4, 24)], -1),
    ([(3, 8, 5, 7)], 1),
])
def test_cat_forward_and_backward(cuda, shapes, dim, nhwc):
    """Bit-exact against torch.cat / torch.split on the CPU (pure data movement)."""
    from monet_b200 import lm_ops
    g = torch.Generator().manual_seed(5)
    parts = [torch.randn(*s, generator=g) for s in shapes]
    dev = [p.to(cuda) for p in parts]
    if nhwc and len(shapes[0]) == 4:
        dev = [p.contiguous(memory_format=torch.channels_last) for p in dev]
    op = lm_ops.list_ops("conv_multiway_newnode", "aten::cat")[0]()
    y = op.forward(*dev, dim)
    want = torch.cat(parts, dim)
    assert torch.equal(y.cpu(), want)
    gy = torch.randn(want.shape, generator=g)
    gd = gy.to(cuda)
    if nhwc and gy.dim() == 4:
        gd = gd.contiguous(memory_format=torch.channels_last)
    grads = op.backward(gd, [])
    grads = [grads] if torch.is_tensor(grads) else grads
    want_g = torch.split(gy, [s[dim] for s in shapes], dim=dim)
    assert len(grads) == len(parts)
    for a, b in zip(grads, want_g):
        assert torch.equal(a.cpu(), b)
        assert a.is_contiguous() or a.is_contiguous(memory_format=torch.channels_last)


@pytest.mark.parametrize("N,C,K", [(184, 2048, 1000), (8, 512, 10), (176, 25088, 4096), (3, 100, 36)])
def test_addmm_runs_on_the_tensor_core_kernels(cuda, N, C, K):
    """LowMemAddMM (linear.py:25-61): forward, the weight/bias step (algorithm 0), the input
    step (algorithm 10) and both (20), against fp32 CPU matmuls at the convolution tolerance.
    Includes the classifier of ResNet-50 and the 25088 x 4096 layer of VGG-16."""
    from monet_b200 import functional as F
    from monet_b200 import lm_ops
    g = torch.Generator().manual_seed(11)
    x = torch.randn(N, C, generator=g)
    w = torch.randn(K, C, generator=g) * C ** -0.5
    b = torch.randn(K, generator=g)
    dy = torch.randn(N, K, generator=g)
    op = lm_ops.list_ops("conv_multiway_newnode", "aten::addmm")[0]()
    xg, wg, bg = (t.to(cuda).requires_grad_(True) for t in (x, w, b))
    y = op.forward(bg, xg, wg, 1, 1)
    assert tuple(y.shape) == (N, K)
    assert _rel(y, torch.addmm(b, x, w.t())) < 2e-2
    op.algorithm = 0
    db, di, dw = op.backward(dy.to(cuda), [xg, wg], nodel=True)
    assert di is None
    assert _rel(dw, dy.t().mm(x)) < 2e-2
    assert torch.allclose(db.cpu(), dy.sum(0), rtol=1e-4, atol=1e-3)
    op.algorithm = 10
    db, di, dw = op.backward(dy.to(cuda), [None, wg], nodel=True)
    assert dw is None and db is None
    assert _rel(di, dy.mm(w)) < 2e-2
    op.algorithm = 20
    stored = [xg, wg]
    db, di, dw = op.backward(dy.to(cuda), stored)
    assert stored == [] and di is not None and dw is not None
    assert F.conv_device_status() == 0
