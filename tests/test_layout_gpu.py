"""Layout conversion and global average pooling."""
import pytest
import torch

from oracle import lm_ops_oracle as oracle

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("shape", [(2, 3, 5, 7), (1, 64, 33, 31), (3, 100, 1, 1), (2, 1, 9, 9), (4, 3, 224, 224)])
def test_layout_round_trip(cuda, shape):
    from monet_b200 import functional as F
    x = torch.randn(shape)
    a = F.to_nhwc(x.to(cuda))
    assert a.is_contiguous(memory_format=torch.channels_last) and torch.equal(a.cpu(), x)
    assert torch.equal(a.cpu().permute(0, 2, 3, 1).contiguous(), x.permute(0, 2, 3, 1).contiguous())
    b = F.to_nchw(a)
    assert b.is_contiguous() and torch.equal(b.cpu(), x)


@pytest.mark.parametrize("shape", [(2, 8, 7, 7), (3, 5, 4, 6), (184, 2048, 7, 7)])
@pytest.mark.parametrize("nhwc", [False, True])
def test_global_avgpool(cuda, shape, nhwc):
    from monet_b200.lm_ops.funcs import AdaptiveAvgPool2D
    x = torch.randn(shape)
    xg = x.to(cuda)
    if nhwc:
        xg = xg.contiguous(memory_format=torch.channels_last)
    op = AdaptiveAvgPool2D()
    y = op.forward(xg, [1, 1])
    assert torch.allclose(y.cpu(), x.mean((2, 3), keepdim=True), rtol=1e-5, atol=1e-6)
    dy = torch.randn(shape[0], shape[1], 1, 1)
    dx = op.backward(dy.to(cuda), [])
    assert torch.allclose(dx.cpu(), oracle.global_avgpool_backward(dy, shape), rtol=1e-5, atol=1e-7)


def test_adaptive_avgpool_other_sizes_defer_to_torch(cuda):
    from monet_b200.lm_ops.funcs import AdaptiveAvgPool2D
    x = torch.randn(2, 4, 8, 8)
    op = AdaptiveAvgPool2D()
    y = op.forward(x.to(cuda), [4, 4])
    assert torch.allclose(y.cpu(), torch.nn.functional.adaptive_avg_pool2d(x, 4), atol=1e-6)
    dx = op.backward(torch.ones(2, 4, 4, 4, device=cuda), [])
    assert torch.allclose(dx.cpu(), torch.full((2, 4, 8, 8), 0.25))
