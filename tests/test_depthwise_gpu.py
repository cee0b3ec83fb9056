"""Depthwise convolution (MobileNetV2's 3x3 layers) against the fp32 CPU oracle: fp32 FMA
arithmetic, so the tolerance is rtol 1e-5 (1e-4 on the long filter-gradient reductions)."""
import pytest
import torch

from oracle import lm_ops_oracle as oracle

pytestmark = pytest.mark.gpu

# N, C, H, W, R, stride, pad
CASES = [(2, 32, 14, 14, 3, 1, 1), (3, 96, 15, 13, 3, 2, 1), (2, 144, 7, 7, 3, 1, 1), (1, 8, 9, 9, 5, 1, 2),
         (4, 24, 28, 28, 3, 2, 1), (2, 16, 6, 6, 1, 1, 0),
         (2, 16, 11, 11, 3, 2, 0),      # stride 2 without padding: the per-pixel backward-data kernel
         (1, 40, 30, 34, 3, 1, 1)]      # interior tiles of the row-tiled kernels


@pytest.mark.parametrize("case", CASES)
def test_depthwise_passes(cuda, case):
    from monet_b200 import functional as F
    N, C, H, W, R, s, p = case
    g = torch.Generator().manual_seed(C)
    x = torch.randn(N, C, H, W, generator=g)
    w = torch.randn(C, 1, R, R, generator=g) * 0.3
    b = torch.randn(C, generator=g)
    ref = oracle.conv_forward(x, w, b, s, p, 1, groups=C)
    y = F.depthwise_fprop(x.to(cuda), w.to(cuda), b.to(cuda), s, p, 1, C)
    assert y.shape == ref.shape and torch.allclose(y.cpu(), ref, rtol=1e-5, atol=1e-5)
    dy = torch.randn(ref.shape, generator=g)
    rdx, rdw, rdb = oracle.conv_backward(dy, x, w, s, p, 1, groups=C)
    dx, dw, db = F.depthwise_bwd(dy.to(cuda), x.to(cuda), w.to(cuda), s, p, 1, C, need=(True, True, True))
    assert torch.allclose(dx.cpu(), rdx, rtol=1e-5, atol=1e-5)
    assert torch.allclose(dw.cpu(), rdw, rtol=1e-4, atol=1e-4)
    assert torch.allclose(db.cpu(), rdb, rtol=1e-4, atol=1e-4)


def test_depthwise_through_the_operator(cuda):
    """SpecificAlgoConvolution with is_depthwise set, as the executor does for groups == C."""
    from monet_b200.lm_ops.conv import SpecificAlgoConvolution
    x = torch.randn(2, 32, 10, 10)
    w = torch.randn(32, 1, 3, 3) * 0.3
    dy = torch.randn(2, 32, 10, 10)
    op = SpecificAlgoConvolution()
    op.is_depthwise = True
    xg, wg = x.to(cuda).requires_grad_(True), w.to(cuda).requires_grad_(True)
    y = op.forward(xg, wg, None, [1, 1], [1, 1], [1, 1], False, [0, 0], 32)
    assert torch.allclose(y.cpu(), oracle.conv_forward(x, w, None, 1, 1, 1, groups=32), rtol=1e-5, atol=1e-5)
    op.algorithm = 20
    stored = [xg, wg]
    dx, dw = op.backward(dy.to(cuda), stored)
    rdx, rdw, _ = oracle.conv_backward(dy, x, w, 1, 1, 1, groups=32)
    assert stored == []
    assert torch.allclose(dx.cpu(), rdx, rtol=1e-5, atol=1e-5) and torch.allclose(dw.cpu(), rdw, rtol=1e-4, atol=1e-4)


def test_mobilenet_v2_step_runs(cuda):
    """A MobileNetV2 training step through the operators (ReLU6, depthwise, residual adds)."""
    import copy
    import torchvision
    from monet_b200 import runner
    from monet_b200.lm_ops.softmax import SoftmaxCrossEntropy
    torch.manual_seed(0)
    model = torchvision.models.mobilenet_v2(num_classes=10).train()
    for m in model.modules():
        if isinstance(m, torch.nn.Dropout):
            m.p = 0.0
    x = torch.randn(4, 3, 64, 64)
    labels = torch.randint(0, 10, (4,))
    ref = copy.deepcopy(model)
    out_ref = ref(x)
    gm = copy.deepcopy(model).to(cuda)
    for policy in ("store_all", "low_memory"):
        r = runner.Runner(gm, getattr(runner, policy))
        out = r.forward(x.to(cuda))
        ce = SoftmaxCrossEntropy()
        loss = ce.forward(out, labels.to(cuda))
        r.backward(ce.backward())
        torch.cuda.synchronize()
        rel = float((out.cpu() - out_ref.detach()).norm() / out_ref.norm())
        assert rel < 5e-2, rel
        assert all(p.grad is not None and torch.isfinite(p.grad).all() for p in gm.parameters())
        for p in gm.parameters():
            p.grad = None
