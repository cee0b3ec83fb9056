"""Softmax, log-softmax and the fused cross-entropy forward+backward (rtol 1e-5)."""
import pytest
import torch

from oracle import lm_ops_oracle as oracle

pytestmark = pytest.mark.gpu

SHAPES = [((184, 1000), 1), ((7, 10), 1), ((3, 1), 1), ((5, 1500), 1), ((2, 5000), 1),
          ((2, 2, 9, 13), 1), ((3, 7, 4), 2), ((1, 21, 17, 5), 1)]


@pytest.mark.parametrize("shape,dim", SHAPES)
@pytest.mark.parametrize("log", [False, True])
def test_softmax_fwd_bwd(cuda, shape, dim, log):
    from monet_b200 import functional as F
    g = torch.Generator().manual_seed(len(shape))
    x = torch.randn(shape, generator=g) * 3
    dy = torch.randn(shape, generator=g)
    y = F.softmax(x.to(cuda), dim, log=log)
    ref = oracle.softmax_forward(x, dim, log)
    assert torch.allclose(y.cpu(), ref, rtol=1e-5, atol=1e-6)
    dx = F.softmax_bwd(dy.to(cuda), y, dim, log=log)
    assert torch.allclose(dx.cpu(), oracle.softmax_backward(dy, ref, dim, log), rtol=1e-5, atol=2e-6)


@pytest.mark.parametrize("shape", [(184, 1000), (5, 10), (1, 2), (4, 3000), (2, 2, 9, 13), (1, 2, 40, 33)])
def test_cross_entropy_fused(cuda, shape):
    from monet_b200 import functional as F
    g = torch.Generator().manual_seed(7)
    logits = torch.randn(shape, generator=g) * 2
    lshape = (shape[0],) + tuple(shape[2:])
    labels = torch.randint(0, shape[1], lshape, generator=g)
    count = labels.numel()
    loss, dlogits = F.cross_entropy_fwd_bwd(logits.to(cuda), labels.to(cuda), 1.0 / count)
    ref_loss, ref_d = oracle.cross_entropy(logits, labels, 1.0 / count)
    assert torch.allclose(loss.cpu(), ref_loss, rtol=1e-5, atol=1e-6)
    assert torch.allclose(dlogits.cpu(), ref_d, rtol=1e-5, atol=1e-8)


def test_softmax_ops_protocol(cuda):
    import monet_b200.lm_ops.softmax as S
    x = torch.randn(6, 50)
    dy = torch.randn(6, 50)
    op = S.Softmax()
    y = op.forward(x.to(cuda), 1, None)
    stored = [y]
    dx = op.backward(dy.to(cuda), stored)
    ref = torch.softmax(x, 1)
    assert stored == [] and torch.allclose(y.cpu(), ref, rtol=1e-5, atol=1e-7)
    assert torch.allclose(dx.cpu(), oracle.softmax_backward(dy, ref, 1), rtol=1e-5, atol=1e-6)
    ce = S.SoftmaxCrossEntropy()
    labels = torch.randint(0, 50, (6,))
    loss = ce.forward(x.to(cuda), labels.to(cuda))
    d = ce.backward()
    ref_loss, ref_d = oracle.cross_entropy(x, labels, 1.0 / 6)
    assert torch.allclose(loss.cpu(), ref_loss.mean(), rtol=1e-5)
    assert torch.allclose(d.cpu(), ref_d, rtol=1e-5, atol=1e-8)
