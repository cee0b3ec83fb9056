"""Fused batch norm / residual add / ReLU: parity with the chain of separate operators the
reference runs (oracle), bit-exact gates, and the operator classes' storage protocol.

Tolerances: values and gradients rtol 1e-5 fp32 (statistics-derived quantities 1e-4, as in the
unfused batch-norm tests); gates, the two-gradient ReLU backward and add+ReLU are bit-exact."""
import pytest
import torch

from oracle import lm_ops_oracle as oracle

pytestmark = pytest.mark.gpu

RTOL, ATOL = 1e-5, 2e-6
SHAPES = [(4, 64, 14, 14), (2, 3, 5, 7), (3, 24, 9, 9), (2, 2048, 7, 7), (5, 96, 3, 3),
          (16, 256, 28, 28), (2, 1, 4, 4), (2, 516, 2, 3)]


def _data(shape, seed=0):
    g = torch.Generator().manual_seed(seed)
    C = shape[1]
    x = torch.randn(shape, generator=g) * 1.7 + 0.3
    gamma = torch.rand(C, generator=g) + 0.5
    beta = torch.randn(C, generator=g) * 0.5
    rm = torch.randn(C, generator=g)
    rv = torch.rand(C, generator=g) + 0.5
    res = torch.randn(shape, generator=g)
    dy = torch.randn(shape, generator=g)
    return x, gamma, beta, rm, rv, res, dy


def _fmt(t, nhwc):
    return t.contiguous(memory_format=torch.channels_last) if nhwc and t.dim() == 4 else t


@pytest.mark.parametrize("shape", SHAPES)
@pytest.mark.parametrize("nhwc", [False, True])
@pytest.mark.parametrize("with_res,relu", [(False, True), (True, True), (True, False)])
def test_bn_act_forward(cuda, shape, nhwc, with_res, relu):
    from monet_b200 import functional as F
    x, gamma, beta, rm, rv, res, _ = _data(shape)
    r = res if with_res else None
    ref_y, ref_mean, ref_invstd, ref_rm, ref_rv = oracle.bn_act_forward_train(
        x, r, relu, gamma, beta, rm, rv, 0.1, 1e-5)
    xg = _fmt(x.to(cuda), nhwc)
    rg = _fmt(res.to(cuda), nhwc) if with_res else None
    rmg, rvg = rm.to(cuda), rv.to(cuda)
    gg, bg = gamma.to(cuda), beta.to(cuda)
    y, mean, invstd = F.bn_act_fwd_train(xg, rg, relu, gg, bg, rmg, rvg, 0.1, 1e-5)
    assert torch.allclose(y.cpu(), ref_y, rtol=RTOL, atol=1e-5)
    assert torch.allclose(mean.cpu(), ref_mean, rtol=RTOL, atol=ATOL)
    assert torch.allclose(invstd.cpu(), ref_invstd, rtol=RTOL, atol=ATOL)
    assert torch.allclose(rmg.cpu(), ref_rm, rtol=RTOL, atol=ATOL)
    assert torch.allclose(rvg.cpu(), ref_rv, rtol=RTOL, atol=ATOL)
    # identical to the separate operators on the GPU, bit for bit
    z, m2, i2 = F.bn_fwd_train(xg, gg, bg, None, None, 0.1, 1e-5)
    if with_res:
        z = F.add(z, rg, 1.0)
    if relu:
        z = F.relu(z)
    assert torch.equal(y, z)
    assert torch.equal(mean, m2) and torch.equal(invstd, i2)
    # recomputation with the cached statistics reproduces y exactly
    y2 = F.bn_act_fwd_apply(xg, rg, relu, gg, bg, mean, invstd)
    assert torch.equal(y2, y)


@pytest.mark.parametrize("shape", SHAPES)
@pytest.mark.parametrize("nhwc", [False, True])
def test_bn_relu_backward(cuda, shape, nhwc):
    from monet_b200 import functional as F
    x, gamma, beta, rm, rv, _, dy = _data(shape, seed=1)
    xg, dyg = _fmt(x.to(cuda), nhwc), _fmt(dy.to(cuda), nhwc)
    gg, bg = gamma.to(cuda), beta.to(cuda)
    y, mean, invstd = F.bn_act_fwd_train(xg, None, True, gg, bg, None, None, 0.1, 1e-5)
    gate = (y > 0).cpu()
    ref_dx, ref_dg, ref_db = oracle.bn_relu_backward_from_input(dy, gate, x, gamma, 1e-5)
    scale = max(1.0, float(ref_dx.abs().max()))
    dx, dg, db = F.bn_relu_bwd_from_input(dyg, xg, gg, bg, mean, invstd)
    assert torch.allclose(dx.cpu(), ref_dx, rtol=RTOL, atol=1e-5 * scale)
    assert torch.allclose(dg.cpu(), ref_dg, rtol=1e-4, atol=1e-4)
    assert torch.allclose(db.cpu(), ref_db, rtol=1e-4, atol=1e-4)
    # same bits as ReLU backward followed by batch-norm backward: the gate evaluated from x in
    # the backward is the forward's gate
    d = F.relu_bwd_act(dyg, y, 0.0, inplace=False)
    dx2, dg2, db2 = F.bn_bwd_from_input(d, xg, gg, mean, invstd)
    assert torch.equal(dx, dx2) and torch.equal(dg, dg2) and torch.equal(db, db2)
    # in place on the gradient
    dyc = dyg.clone(memory_format=torch.preserve_format)
    dx3, _, _ = F.bn_relu_bwd_from_input(dyc, xg, gg, bg, mean, invstd, inplace=True)
    assert dx3.data_ptr() == dyc.data_ptr() and torch.equal(dx3, dx)


@pytest.mark.parametrize("shape", SHAPES)
@pytest.mark.parametrize("nhwc", [False, True])
def test_bn_relu6(cuda, shape, nhwc):
    """Batch norm + ReLU6 (activation code 2): forward = bn.py then hardtanh.py's clamp to [0, 6],
    backward gate 0 < z < 6 re-evaluated from x; bit-identical to the separate operators."""
    from monet_b200 import functional as F
    x, gamma, beta, rm, rv, _, dy = _data(shape, seed=4)
    gamma = gamma * 4.0                                    # so that a good part exceeds 6
    xg, dyg = _fmt(x.to(cuda), nhwc), _fmt(dy.to(cuda), nhwc)
    gg, bg = gamma.to(cuda), beta.to(cuda)
    ref_y, ref_mean, ref_invstd, _, _ = oracle.bn_forward_train(x, gamma, beta, rm, rv, 0.1, 1e-5)
    ref_y = ref_y.clamp(0.0, 6.0)
    y, mean, invstd = F.bn_act_fwd_train(xg, None, 2, gg, bg, None, None, 0.1, 1e-5)
    assert torch.allclose(y.cpu(), ref_y, rtol=RTOL, atol=1e-5)
    if y.numel() >= 1000:                                  # both clamps are exercised
        assert float((y == 6).float().mean()) > 0.01 and float((y == 0).float().mean()) > 0.01
    z, _, _ = F.bn_fwd_train(xg, gg, bg, None, None, 0.1, 1e-5)
    assert torch.equal(y, F.hardtanh(z, 0.0, 6.0))
    assert torch.equal(F.bn_act_fwd_apply(xg, None, 2, gg, bg, mean, invstd), y)
    gate = ((y > 0) & (y < 6)).cpu()
    ref_dx, ref_dg, ref_db = oracle.bn_relu_backward_from_input(dy, gate, x, gamma, 1e-5)
    scale = max(1.0, float(ref_dx.abs().max()))
    dx, dg, db = F.bn_relu_bwd_from_input(dyg, xg, gg, bg, mean, invstd, act=2)
    assert torch.allclose(dx.cpu(), ref_dx, rtol=RTOL, atol=1e-5 * scale)
    assert torch.allclose(dg.cpu(), ref_dg, rtol=1e-4, atol=1e-4 * max(1.0, float(ref_dg.abs().max())))
    assert torch.allclose(db.cpu(), ref_db, rtol=1e-4, atol=1e-4)
    d = F.hardtanh_bwd(dyg, z, 0.0, 6.0)
    dx2, dg2, db2 = F.bn_bwd_from_input(d, xg, gg, mean, invstd)
    assert torch.equal(dx, dx2) and torch.equal(dg, dg2) and torch.equal(db, db2)


@pytest.mark.parametrize("shape", SHAPES)
@pytest.mark.parametrize("nhwc", [False, True])
@pytest.mark.parametrize("pair", [False, True])
def test_bn_add_relu_backward(cuda, shape, nhwc, pair):
    """Backward through y = relu(bn(x) + r) with the gate folded into the batch-norm reduce."""
    from monet_b200 import functional as F
    x, gamma, beta, rm, rv, res, dy = _data(shape, seed=2)
    xg, rg = _fmt(x.to(cuda), nhwc), _fmt(res.to(cuda), nhwc)
    gg, bg = gamma.to(cuda), beta.to(cuda)
    y, mean, invstd = F.bn_act_fwd_train(xg, rg, True, gg, bg, None, None, 0.1, 1e-5)
    g1, g2 = (dy * 0.3, dy * 0.7) if pair else (dy, None)
    d_ref = oracle.relu_backward_sum2(g1, g2, y.cpu()) if pair else oracle.relu_backward(dy, y.cpu())
    ref_dx, ref_dg, ref_db = oracle.bn_backward_from_input(d_ref, x, gamma, 1e-5)
    scale = max(1.0, float(ref_dx.abs().max()))
    g1g = _fmt(g1.to(cuda), nhwc)
    g2g = _fmt(g2.to(cuda), nhwc) if pair else None
    # the unfused chain on the GPU, for bit equality
    dd = F.relu_bwd_act2(g1g.clone(memory_format=torch.preserve_format), g2g, y) if pair else \
        F.relu_bwd_act(g1g, y, 0.0, inplace=False)
    dx2, dg2, db2 = F.bn_bwd_from_input(dd, xg, gg, mean, invstd)
    d, dx, dg, db = F.bn_add_relu_bwd(g1g, g2g, y, xg, gg, mean, invstd)
    assert d.data_ptr() == g1g.data_ptr()                   # written over the first gradient
    assert torch.equal(d.cpu(), d_ref)
    assert torch.allclose(dx.cpu(), ref_dx, rtol=RTOL, atol=1e-5 * scale)
    assert torch.allclose(dg.cpu(), ref_dg, rtol=1e-4, atol=1e-4)
    assert torch.allclose(db.cpu(), ref_db, rtol=1e-4, atol=1e-4)
    assert torch.equal(dx, dx2) and torch.equal(dg, dg2) and torch.equal(db, db2)


@pytest.mark.parametrize("n", [0, 1, 7, 8, 9, 1000, 4097, 1 << 20, (1 << 20) + 3])
def test_relu_backward_two_gradients_and_add_relu(cuda, n):
    from monet_b200 import functional as F
    g = torch.Generator().manual_seed(n)
    a = torch.randn(n, generator=g)
    b = torch.randn(n, generator=g)
    act = torch.randn(n, generator=g)
    act[::5] = 0.0
    ref = oracle.relu_backward_sum2(a, b, act)
    ag = a.to(cuda)
    out = F.relu_bwd_act2(ag, b.to(cuda), act.to(cuda))
    assert out.data_ptr() == ag.data_ptr()
    assert torch.equal(out.cpu(), ref)
    y = F.add_relu(a.to(cuda), b.to(cuda), 1.0)
    assert torch.equal(y.cpu(), oracle.relu_forward(a + b))
    y = F.add_relu(a.to(cuda), b.to(cuda), 0.5)
    assert torch.allclose(y.cpu(), oracle.relu_forward(a + 0.5 * b), rtol=RTOL, atol=1e-6)


def test_unaligned_views(cuda):
    """Views that start off a 32-byte boundary take the scalar path of the same functor."""
    from monet_b200 import functional as F
    g = torch.Generator().manual_seed(3)
    base = [torch.randn(1003, generator=g).to(cuda) for _ in range(3)]
    a, b, act = (t[1:1001] for t in base)
    ref = oracle.relu_backward_sum2(a.cpu(), b.cpu(), act.cpu())
    assert a.data_ptr() % 32 != 0
    out = F.relu_bwd_act2(a, b, act)
    assert torch.equal(out.cpu(), ref)


def test_fused_operator_classes(cuda):
    """Registry names, storage descriptors, params carried to a recomputing instance."""
    from monet_b200 import lm_ops
    from monet_b200.lm_ops import fused  # noqa: F401
    from monet_b200.lm_ops.base import InputStorage, OutputStorage
    shape = (4, 32, 6, 6)
    x, gamma, beta, rm, rv, res, dy = _data(shape, seed=5)
    cl = torch.channels_last
    xg, rg, dyg = (t.to(cuda).contiguous(memory_format=cl) for t in (x, res, dy))
    gg, bg, rmg, rvg = gamma.to(cuda), beta.to(cuda), rm.to(cuda), rv.to(cuda)

    (cls,) = lm_ops.list_ops("multiway_newnode", "monet::batch_norm_relu")
    op = cls()
    assert isinstance(op.backward_storage, InputStorage) and op.backward_storage.ids == (0, 1, 2, 3, 4)
    y = op.forward(xg, gg, bg, rmg, rvg, True, 0.1, 1e-5, True)
    ref_y, *_ = oracle.bn_act_forward_train(x, None, True, gamma, beta, rm, rv, 0.1, 1e-5)
    assert torch.allclose(y.cpu(), ref_y, rtol=RTOL, atol=1e-5)
    rm_after = rmg.clone()
    again = cls()
    again.params = op.params                      # what the executor does before a recomputation
    y2 = again.forward(xg, gg, bg, rmg, rvg, True, 0.1, 1e-5, True)
    assert torch.equal(y2, y) and torch.equal(rmg, rm_after)   # running statistics untouched
    stored = [xg, gg, bg, rmg, rvg]
    dx, dw, db, n1, n2 = op.backward(dyg.clone(memory_format=torch.preserve_format), stored)
    assert stored == [] and n1 is None and n2 is None
    ref_dx, ref_dg, ref_db = oracle.bn_relu_backward_from_input(dy, (y > 0).cpu(), x, gamma, 1e-5)
    assert torch.allclose(dx.cpu(), ref_dx, rtol=RTOL, atol=1e-5)
    assert torch.allclose(dw.cpu(), ref_dg, rtol=1e-4, atol=1e-4)
    assert torch.allclose(db.cpu(), ref_db, rtol=1e-4, atol=1e-4)

    (cls,) = lm_ops.list_ops("multiway_newnode", "monet::batch_norm_add_relu")
    op = cls()
    kinds = [type(d) for d in op.backward_storage]
    assert kinds == [InputStorage, OutputStorage] and op.accepts_grad_pair
    y = op.forward(xg, gg, bg, rmg, rvg, True, 0.1, 1e-5, True, rg)
    ref_y, *_ = oracle.bn_act_forward_train(x, res, True, gamma, beta, rm, rv, 0.1, 1e-5)
    assert torch.allclose(y.cpu(), ref_y, rtol=RTOL, atol=1e-5)
    g1, g2 = dy * 0.25, dy * 0.75
    stored = [xg, gg, bg, rmg, rvg, y]
    outs = op.backward((g1.to(cuda).contiguous(memory_format=cl), g2.to(cuda).contiguous(memory_format=cl)),
                       stored)
    assert stored == [] and len(outs) == 6
    d_ref = oracle.relu_backward_sum2(g1, g2, y.cpu())
    ref_dx, ref_dg, ref_db = oracle.bn_backward_from_input(d_ref, x, gamma, 1e-5)
    assert torch.equal(outs[5].cpu(), d_ref)                   # gradient of the residual
    assert torch.allclose(outs[0].cpu(), ref_dx, rtol=RTOL, atol=1e-5)
    assert torch.allclose(outs[1].cpu(), ref_dg, rtol=1e-4, atol=1e-4)
    assert torch.allclose(outs[2].cpu(), ref_db, rtol=1e-4, atol=1e-4)

    (cls,) = lm_ops.list_ops("normal", "monet::add_relu")
    op = cls()
    y = op.forward(xg, rg, 1)
    assert torch.equal(y.cpu(), oracle.relu_forward(x + res))
    stored = [y]
    da, db_ = op.backward(dyg.clone(memory_format=torch.preserve_format), stored)
    assert stored == []
    assert torch.equal(da.cpu(), oracle.relu_backward(dy, y.cpu())) and torch.equal(db_, da)


@pytest.mark.parametrize("policy", ["store_all", "low_memory", "budget_10gb"])
def test_fused_network_equals_unfused(cuda, policy):
    """A residual network run with the fused nodes gives the logits of the unfused graph bit for
    bit and the same parameter gradients (up to the unordered atomic sums of the weight
    gradient)."""
    import torchvision
    from monet_b200 import runner
    torch.manual_seed(0)
    model = torchvision.models.resnet18(num_classes=10).to(cuda).to(memory_format=torch.channels_last)
    model.train()
    x = torch.randn(6, 3, 64, 64, device=cuda)
    gout = torch.randn(6, 10, device=cuda)
    state = {k: v.clone() for k, v in model.state_dict().items()}
    results = []
    for fuse in (False, True):
        model.load_state_dict(state)
        for p in model.parameters():
            p.grad = None
        run = runner.Runner(model, getattr(runner, policy), fuse=fuse, channel_sums=False)
        if fuse:
            ops = [n.op for n in run.nodes]
            assert 'aten::relu_' not in ops and 'aten::add' not in ops and 'aten::add_' not in ops
            assert ops.count('monet::batch_norm_add_relu') == 8
        out = run.forward(x)
        run.backward(gout.clone())
        results.append((out.clone(), {k: p.grad.clone() for k, p in model.named_parameters()},
                        {k: v.clone() for k, v in model.state_dict().items() if 'running' in k}))
    (o0, g0, s0), (o1, g1, s1) = results
    assert torch.equal(o0, o1)
    for k in s0:
        assert torch.equal(s0[k], s1[k]), k
    for k in g0:
        scale = float(g0[k].abs().max()) + 1e-12
        assert float((g0[k] - g1[k]).abs().max()) <= 1e-4 * scale, k


def test_mobilenet_fused_equals_unfused(cuda):
    """MobileNetV2 (depthwise convolutions, ReLU6): the graph with batch_norm_relu6 nodes gives
    the logits of the unfused graph bit for bit."""
    import torchvision
    from monet_b200 import runner
    torch.manual_seed(0)
    model = torchvision.models.mobilenet_v2(num_classes=10).to(cuda).to(memory_format=torch.channels_last)
    model.train()
    x = torch.randn(4, 3, 64, 64, device=cuda)
    gout = torch.randn(4, 10, device=cuda)
    state = {k: v.clone() for k, v in model.state_dict().items()}
    results = []
    for fuse in (False, True):
        model.load_state_dict(state)
        for p in model.parameters():
            p.grad = None
        run = runner.Runner(model, runner.low_memory, fuse=fuse, channel_sums=False)
        if fuse:
            assert sum(n.op == 'monet::batch_norm_relu6' for n in run.nodes) == 35
        torch.manual_seed(123)            # the classifier's dropout draws from the global generator
        out = run.forward(x)
        run.backward(gout.clone())
        results.append((out.clone(), {k: p.grad.clone() for k, p in model.named_parameters()}))
    (o0, g0), (o1, g1) = results
    assert torch.equal(o0, o1)
    for k in g0:
        scale = float(g0[k].abs().max()) + 1e-12
        assert float((g0[k] - g1[k]).abs().max()) <= 1e-4 * scale, k


def test_conv_channel_sums(cuda):
    """A convolution whose statistics warps sum its output per channel: the sums (taken around a
    shift) reproduce the batch statistics, and a batch norm fed with them matches the oracle."""
    from monet_b200 import functional as F
    g = torch.Generator().manual_seed(11)
    cl = torch.channels_last
    cases = [((6, 64, 20, 20), (96, 64, 1, 1), 1, 0), ((4, 64, 30, 30), (128, 64, 1, 1), 2, 0),
             ((3, 160, 9, 9), (320, 160, 1, 1), 1, 0), ((4, 32, 15, 15), (32, 32, 3, 3), 2, 1),
             ((184, 64, 14, 14), (256, 64, 1, 1), 1, 0), ((5, 32, 17, 19), (64, 32, 3, 3), 1, 1),
             ((2, 3, 40, 40), (32, 3, 7, 7), 2, 3), ((2, 64, 8, 8), (48, 64, 1, 1), 1, 0),
             ((3, 64, 56, 56), (64, 64, 3, 3), 1, 1), ((7, 32, 14, 14), (256, 32, 3, 3), 1, 1),
             ((5, 64, 7, 7), (512, 64, 3, 3), 1, 1), ((2, 32, 23, 31), (128, 32, 3, 3), 1, 1),
             ((3, 32, 13, 9), (32, 32, 5, 5), 1, 2)]
    for xs, ws, stride, pad in cases:
        x = torch.randn(xs, generator=g)
        w = torch.randn(ws, generator=g) * 0.1
        bias = torch.randn(ws[0], generator=g)
        K = ws[0]
        gamma, beta = torch.rand(K, generator=g) + 0.5, torch.randn(K, generator=g)
        rm, rv = torch.randn(K, generator=g) * 0.3, torch.rand(K, generator=g) + 0.5
        xg = x.to(cuda).contiguous(memory_format=cl) if xs[1] % 4 == 0 else x.to(cuda)
        wg = w.to(cuda).contiguous(memory_format=cl)
        rmg, rvg = rm.to(cuda), rv.to(cuda)
        y, sums = F.conv2d_fprop(xg, wg, bias.to(cuda), stride, pad, 1, 1, 0, stats_shift=rmg,
                                 want_stats=True)
        y_plain = F.conv2d_fprop(xg, wg, bias.to(cuda), stride, pad, 1)
        assert torch.equal(y, y_plain)
        multi_tap_s1 = ws[2] * ws[3] > 1 and stride == 1
        if xs[1] < 4 or K % 32 or multi_tap_s1:
            assert sums is None                 # no such path: the caller runs the plain batch norm
            continue
        assert sums is not None and sums.rows >= 1
        part = sums.partials[:2 * sums.rows * K].view(2, sums.rows, K).double().sum(1).cpu()
        yd = y.double().cpu() - rm.double().view(1, -1, 1, 1)
        assert torch.allclose(part[0], yd.sum((0, 2, 3)), rtol=1e-5, atol=1e-3)
        assert torch.allclose(part[1], (yd * yd).sum((0, 2, 3)), rtol=1e-5, atol=1e-3)
        residual = torch.randn(y.shape, generator=g)
        ref_y, ref_mean, ref_invstd, ref_rm, ref_rv = oracle.bn_act_forward_train(
            y.cpu(), residual, True, gamma, beta, rm, rv, 0.1, 1e-5)
        out, mean, invstd = F.bn_act_fwd_train_partials(
            y, sums, residual.to(cuda).contiguous(memory_format=cl), True, gamma.to(cuda),
            beta.to(cuda), rmg, rvg, 0.1, 1e-5)
        assert torch.allclose(out.cpu(), ref_y, rtol=RTOL, atol=2e-5)
        assert torch.allclose(mean.cpu(), ref_mean, rtol=RTOL, atol=1e-5)
        assert torch.allclose(invstd.cpu(), ref_invstd, rtol=1e-4, atol=1e-5)
        assert torch.allclose(rmg.cpu(), ref_rm, rtol=RTOL, atol=1e-5)
        assert torch.allclose(rvg.cpu(), ref_rv, rtol=1e-4, atol=1e-5)
    assert F.conv_device_status() == 0


def test_network_with_channel_sums(cuda):
    """The whole fused graph with convolution-side statistics against the same graph with the
    batch norms' own statistics pass."""
    import torchvision
    from monet_b200 import runner
    torch.manual_seed(0)
    model = torchvision.models.resnet50(num_classes=10).to(cuda).to(memory_format=torch.channels_last)
    model.train()
    x = torch.randn(8, 3, 64, 64, device=cuda)
    gout = torch.randn(8, 10, device=cuda)
    state = {k: v.clone() for k, v in model.state_dict().items()}
    results = []
    for sums in (False, True):
        model.load_state_dict(state)
        for p in model.parameters():
            p.grad = None
        run = runner.Runner(model, runner.low_memory, fuse=True, channel_sums=sums)
        if sums:
            assert sum(n.sums_from >= 0 for n in run.nodes) == 53
        out = run.forward(x)
        run.backward(gout.clone())
        results.append((out.clone(), {k: p.grad.clone() for k, p in model.named_parameters()},
                        {k: v.clone() for k, v in model.state_dict().items() if 'running' in k}))
    (o0, g0, s0), (o1, g1, s1) = results
    # a 1e-7 difference in a statistic can move an activation across a TF32 truncation boundary
    # of the next convolution, so the two runs differ by TF32 noise (about 1e-3 per layer), not
    # by fp32 rounding; the bar is the convolution tolerance of this library, rtol 2e-2
    assert torch.allclose(o0, o1, rtol=2e-2, atol=2e-2 * float(o0.abs().max()))
    for k in [k for k in s0 if k.startswith('layer1.0.bn1.')]:   # first batch norm fed by a 1x1 convolution
        assert torch.allclose(s0[k], s1[k], rtol=1e-4, atol=1e-5), k
    # gradients: only the classifier's, which see the same TF32 noise as the logits; deeper in
    # the backward chain 50 batch norms over 32..2048 samples amplify that noise without bound
    # (stock PyTorch with TF32 cuDNN differs from fp32 by tens of per cent there as well)
    for k in ('fc.weight', 'fc.bias'):
        scale = float(g0[k].abs().max()) + 1e-12
        assert float((g0[k] - g1[k]).abs().max()) <= 5e-2 * scale, k
