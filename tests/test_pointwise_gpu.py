"""Parity of the element-wise kernels (ReLU and its 1-bit mask, hardtanh, add, packers)
with the CPU oracle: values rtol 1e-5, mask / packed bytes bit-exact."""
import numpy as np
import pytest
import torch

from oracle import lm_ops_oracle as oracle

pytestmark = pytest.mark.gpu

RTOL, ATOL = 1e-5, 1e-6
# sizes: empty, below one group, ragged tails, one warp, large ragged, > L2
SIZES = [0, 1, 7, 8, 9, 63, 255, 256, 1000, 8 * 1024 + 3, 3_211_264, 40_000_003]


def _x(n, seed=0):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(n, generator=g)
    if n > 4:
        x[1] = 0.0
        x[2] = -0.0
        x[3] = float("nan")
    return x


@pytest.mark.parametrize("n", SIZES)
@pytest.mark.parametrize("inplace", [False, True])
def test_relu_fwd_mask(cuda, n, inplace):
    from monet_b200 import functional as F
    x = _x(n)
    xg = x.to(cuda)
    y, mask = F.relu_mask(xg, inplace=inplace)
    torch.cuda.synchronize()
    assert (y.data_ptr() == xg.data_ptr()) == (inplace or n == 0) or n == 0
    ref = oracle.relu_forward(x)
    assert torch.allclose(y.cpu(), ref, rtol=RTOL, atol=ATOL, equal_nan=True)
    assert np.array_equal(mask.cpu().numpy(), oracle.relu_mask_bytes(x))
    y2 = F.relu(x.to(cuda))
    assert torch.allclose(y2.cpu(), ref, rtol=RTOL, atol=ATOL, equal_nan=True)


@pytest.mark.parametrize("n", SIZES)
def test_relu_bwd_mask_and_act(cuda, n):
    from monet_b200 import functional as F
    x, dy = _x(n), _x(n, seed=1)
    ref = oracle.relu_backward(dy, x)
    _, mask = F.relu_mask(x.to(cuda))
    dx = F.relu_bwd_mask(dy.to(cuda), mask, inplace=False)
    assert torch.allclose(dx.cpu(), ref, rtol=RTOL, atol=ATOL, equal_nan=True)
    g = dy.to(cuda)
    dx2 = F.relu_bwd_mask(g, mask, inplace=True)
    assert dx2.data_ptr() == g.data_ptr()
    assert torch.allclose(dx2.cpu(), ref, rtol=RTOL, atol=ATOL, equal_nan=True)
    dx3 = F.relu_bwd_act(dy.to(cuda), x.to(cuda), 0.0, inplace=False)
    assert torch.allclose(dx3.cpu(), ref, rtol=RTOL, atol=ATOL, equal_nan=True)
    # from the OUTPUT: relu(x) > 0 iff x > 0
    dx4 = F.relu_bwd_act(dy.to(cuda), torch.relu(x).to(cuda), 0.0, inplace=False)
    assert torch.allclose(dx4.cpu(), ref, rtol=RTOL, atol=ATOL, equal_nan=True)


def test_relu_unaligned_view(cuda):
    """A view that starts 4 bytes into an allocation takes the scalar path."""
    from monet_b200 import functional as F
    x = _x(1001)
    xg = x.to(cuda)[1:]
    y, mask = F.relu_mask(xg)
    assert torch.allclose(y.cpu(), torch.relu(x[1:]), equal_nan=True)
    assert np.array_equal(mask.cpu().numpy(), oracle.relu_mask_bytes(x[1:]))


def test_relu_mask_channels_last_is_physical_order(cuda):
    from monet_b200 import functional as F
    x = torch.randn(2, 8, 5, 7)
    xg = x.to(cuda).contiguous(memory_format=torch.channels_last)
    y, mask = F.relu_mask(xg)
    assert y.is_contiguous(memory_format=torch.channels_last)
    assert torch.equal(y.cpu(), torch.relu(x))
    phys = x.permute(0, 2, 3, 1).contiguous()
    assert np.array_equal(mask.cpu().numpy(), oracle.relu_mask_bytes(phys))


@pytest.mark.parametrize("n", [0, 5, 8, 1001, 2_000_003])
def test_packers(cuda, n):
    from monet_b200.lm_ops import pack as P
    g = torch.Generator().manual_seed(n)
    flags = torch.rand(n, generator=g) > 0.5
    packed = P.pack(flags.to(cuda))
    assert np.array_equal(packed.cpu().numpy(), np.packbits(flags.numpy(), bitorder="big"))
    assert torch.equal(P.unpack(packed, n).cpu(), flags)
    v = torch.randn(n, generator=g)
    assert torch.equal(P.unpack_multiply(packed, v.to(cuda)).cpu(), v * flags)
    idx = torch.randint(0, 16, (n,), generator=g, dtype=torch.uint8)
    two = P.pack_two(idx.to(cuda))
    assert np.array_equal(two.cpu().numpy(), oracle.pack_nibbles(idx.numpy()))
    assert torch.equal(P.unpack_two(two, n).cpu(), idx)


@pytest.mark.parametrize("n", [0, 9, 1000, 3_000_001])
def test_hardtanh(cuda, n):
    from monet_b200 import functional as F
    x, dy = _x(n) * 4, _x(n, seed=2)
    if n > 8:
        x[5], x[6] = 0.0, 6.0
    y = F.hardtanh(x.to(cuda), 0.0, 6.0)
    ref = torch.nn.functional.hardtanh(x, 0.0, 6.0)
    assert torch.allclose(y.cpu(), ref, rtol=RTOL, atol=ATOL, equal_nan=True)
    refb = oracle.hardtanh_backward(dy, x, 0.0, 6.0)
    dx = F.hardtanh_bwd(dy.to(cuda), x.to(cuda), 0.0, 6.0)
    assert torch.allclose(dx.cpu(), refb, rtol=RTOL, atol=ATOL, equal_nan=True)
    dxo = F.hardtanh_bwd(dy.to(cuda), y, 0.0, 6.0)          # from the output
    assert torch.allclose(dxo.cpu(), refb, rtol=RTOL, atol=ATOL, equal_nan=True)


@pytest.mark.parametrize("n", [0, 3, 1024, 5_000_001])
@pytest.mark.parametrize("alpha", [1.0, -0.5])
def test_add(cuda, n, alpha):
    from monet_b200 import functional as F
    a, b = _x(n), _x(n, seed=3)
    y = F.add(a.to(cuda), b.to(cuda), alpha)
    assert torch.allclose(y.cpu(), oracle.add_forward(a, b, alpha), rtol=RTOL, atol=ATOL, equal_nan=True)
    ag = a.to(cuda)
    y2 = F.add(ag, b.to(cuda), alpha, inplace=True)
    assert y2.data_ptr() == ag.data_ptr()
    assert torch.allclose(y2.cpu(), oracle.add_forward(a, b, alpha), rtol=RTOL, atol=ATOL, equal_nan=True)
    assert torch.allclose(F.scale(a.to(cuda), alpha).cpu(), a * alpha, rtol=RTOL, atol=ATOL, equal_nan=True)


def test_relu_ops_protocol(cuda):
    """The three ReLU operator classes through the executor's calling convention
    (forward(*args) -> tensor or (tensor, intermediate); backward(grad, stored))."""
    from monet_b200.lm_ops import relu as R
    x = torch.randn(4, 16, 9, 9)
    dy = torch.randn(4, 16, 9, 9)
    ref_y, ref_dx = torch.relu(x), oracle.relu_backward(dy, x)
    op = R.InputActReLU()
    y = op.forward(x.to(cuda))
    stored = [x.to(cuda)]
    dx = op.backward(dy.to(cuda), stored)
    assert stored == [] and torch.equal(y.cpu(), ref_y) and torch.equal(dx.cpu(), ref_dx)
    op = R.OutputActReLU(); op.inplace = True
    xg = x.to(cuda)
    y = op.forward(xg)
    assert y.data_ptr() == xg.data_ptr()
    stored = [y]
    dx = op.backward(dy.to(cuda), stored, nodel=True)
    assert len(stored) == 1 and torch.equal(dx.cpu(), ref_dx)
    op = R.BinaryActReLU()
    y, mask = op.forward(x.to(cuda))
    assert mask.numel() == op.backward_storage.size(tuple(y.shape))
    stored = [mask]
    dx = op.backward(dy.to(cuda), stored)
    assert stored == [] and torch.equal(y.cpu(), ref_y) and torch.equal(dx.cpu(), ref_dx)
