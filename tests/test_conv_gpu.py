"""Tensor-core convolution parity: TF32 operands / fp32 accumulation against the fp32 CPU
oracle, rtol 2e-2 (relative to the tensor's scale), for the three passes."""
import pytest
import torch

from oracle import lm_ops_oracle as oracle

pytestmark = pytest.mark.gpu

RTOL = 2e-2

# N, C, H, W, K, R, stride, pad, dilation
CASES = [
    (2, 64, 8, 8, 64, 1, 1, 0, 1),       # pointwise, one tile
    (4, 64, 14, 14, 256, 1, 1, 0, 1),    # pointwise, several N tiles of the filter
    (3, 96, 7, 9, 40, 1, 1, 0, 1),       # channel counts that are not tile multiples
    (2, 64, 12, 12, 64, 3, 1, 1, 1),     # 3x3
    (2, 32, 56, 56, 32, 3, 1, 1, 1),     # 3x3, rows of 56 (two rows per tile)
    (3, 128, 14, 14, 128, 3, 1, 1, 1),
    (5, 64, 7, 7, 96, 3, 1, 1, 1),       # 7x7 maps: two images per tile
    (2, 64, 16, 16, 128, 3, 2, 1, 1),    # 3x3 stride 2
    (2, 64, 15, 15, 64, 3, 2, 1, 1),     # odd extent, stride 2
    (2, 128, 14, 14, 256, 1, 2, 0, 1),   # 1x1 stride 2 (downsample)
    (2, 32, 13, 13, 32, 3, 1, 2, 2),     # dilation 2
    (1, 4, 20, 20, 8, 5, 1, 2, 1),       # 5x5
    (2, 3, 32, 32, 64, 7, 2, 3, 1),      # the stem geometry: few-channel kernels
    (3, 3, 37, 41, 32, 7, 2, 3, 1),      # stem, odd extents
    (2, 1, 20, 20, 16, 5, 1, 2, 1),      # one input channel, stride 1
    (2, 4, 18, 18, 24, 3, 2, 1, 1),      # four input channels
    (2, 16, 9, 9, 2, 1, 1, 0, 1),        # K = 2 padded to 4
    (1, 260, 5, 5, 36, 1, 1, 0, 1),      # C spans several 32-channel chunks with a tail
    (1, 32, 7, 300, 64, 3, 1, 1, 1),     # map wider than a TMA box: column-tiled halo kernel
    (2, 64, 5, 610, 32, 3, 1, 1, 1),     # UNet's 608-wide maps, ragged last column tile
    (1, 32, 9, 257, 40, 5, 1, 2, 1),     # 5x5 on a wide map, odd width
    (2, 64, 9, 224, 64, 3, 1, 1, 1),     # VGG's 224-wide 64-channel layer: a row with halo exceeds a backward-filter slot
    (1, 32, 6, 300, 96, 3, 1, 1, 1),     # wide map, three boxes of output channels
    (1, 32, 50, 520, 32, 3, 2, 1, 1),    # stride 2 on a wide map: column tiles per stride phase
    (2, 256, 10, 12, 96, 3, 1, 1, 1),    # backward-filter by filter row: 8 chunks in two groups, three dy boxes
    (1, 160, 9, 40, 64, 3, 1, 1, 1),     # 5 chunks in one group
    (1, 192, 6, 300, 32, 3, 1, 1, 1),    # filter-row mode with column tiles
    (2, 128, 9, 9, 136, 5, 1, 2, 1),     # 5x5: three chunks at most per CTA, two tiles of output channels
    (3, 128, 12, 20, 64, 3, 1, 1, 1),    # filter-row mode with the stacked dy operand (K <= 64)
    (2, 160, 7, 9, 24, 3, 1, 1, 1),      # the same with one box of output channels and 5 chunks
    (3, 64, 13, 17, 64, 3, 1, 1, 1),     # 64 output channels: two output rows per GEMM row, odd extents
    (2, 96, 9, 30, 64, 3, 1, 1, 1),      # the same with three channel chunks
    (1, 64, 2, 5, 64, 3, 1, 1, 1),       # a single row pair
    (2, 64, 11, 20, 96, 3, 1, 1, 1),     # backward-data has 64 columns here (C = 64), forward 96
    (1, 32, 40, 126, 64, 3, 1, 1, 1),    # the widest row that fits one tile (126 + 2 = 128)
    (1, 64, 9, 300, 64, 3, 1, 1, 1),     # row pairs with column tiles, odd height, ragged last tile
    (2, 32, 6, 127, 64, 3, 1, 1, 1),     # one column too wide for a single tile
]


def _rel_err(a, ref):
    return float((a - ref).abs().max() / ref.abs().max().clamp_min(1e-6))


def _inputs(case, seed=0):
    N, C, H, W, K, R, s, p, dil = case
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(N, C, H, W, generator=g)
    w = torch.randn(K, C, R, R, generator=g) * (2.0 / (C * R * R)) ** 0.5
    b = torch.randn(K, generator=g)
    return x, w, b


@pytest.mark.parametrize("case", CASES)
def test_fprop(cuda, case):
    from monet_b200 import functional as F
    N, C, H, W, K, R, s, p, dil = case
    x, w, b = _inputs(case)
    ref = oracle.conv_forward(x, w, b, s, p, dil)
    y = F.conv2d_fprop(x.to(cuda), w.to(cuda), b.to(cuda), s, p, dil)
    assert F.conv_device_status() == 0
    assert y.shape == ref.shape
    assert _rel_err(y.cpu(), ref) < RTOL, _rel_err(y.cpu(), ref)
    y0 = F.conv2d_fprop(x.to(cuda).contiguous(memory_format=torch.channels_last), w.to(cuda), None, s, p, dil)
    assert _rel_err(y0.cpu(), oracle.conv_forward(x, w, None, s, p, dil)) < RTOL


@pytest.mark.parametrize("case", CASES)
def test_dgrad(cuda, case):
    from monet_b200 import functional as F
    N, C, H, W, K, R, s, p, dil = case
    x, w, _ = _inputs(case, seed=1)
    ref_y = oracle.conv_forward(x, w, None, s, p, dil)
    dy = torch.randn(ref_y.shape, generator=torch.Generator().manual_seed(2))
    ref_dx, _, _ = oracle.conv_backward(dy, x, w, s, p, dil)
    dx = F.conv2d_dgrad(dy.to(cuda), w.to(cuda), x.shape, s, p, dil)
    assert F.conv_device_status() == 0
    assert dx.shape == ref_dx.shape
    assert _rel_err(dx.cpu(), ref_dx) < RTOL, _rel_err(dx.cpu(), ref_dx)


@pytest.mark.parametrize("case", CASES)
@pytest.mark.parametrize("variant", [0, 1])
def test_wgrad(cuda, case, variant):
    from monet_b200 import functional as F
    N, C, H, W, K, R, s, p, dil = case
    x, w, _ = _inputs(case, seed=3)
    ref_y = oracle.conv_forward(x, w, None, s, p, dil)
    dy = torch.randn(ref_y.shape, generator=torch.Generator().manual_seed(4))
    _, ref_dw, ref_db = oracle.conv_backward(dy, x, w, s, p, dil)
    dw, db = F.conv2d_wgrad(x.to(cuda), dy.to(cuda), w.shape, s, p, dil, variant=variant, need_bias=True)
    assert F.conv_device_status() == 0
    assert dw.shape == ref_dw.shape
    assert _rel_err(dw.cpu(), ref_dw) < RTOL, _rel_err(dw.cpu(), ref_dw)
    assert torch.allclose(db.cpu(), ref_db, rtol=1e-4, atol=1e-3)


def test_unsupported_geometry_raises(cuda):
    from monet_b200 import functional as F
    x = torch.randn(1, 8, 9, 9, device=cuda)
    w = torch.randn(8, 8, 3, 3, device=cuda)
    with pytest.raises(RuntimeError, match="stride"):
        F.conv2d_fprop(x, w, None, 3, 1, 1)
    with pytest.raises(RuntimeError, match="variant"):
        F.conv2d_fprop(x, w, None, 1, 1, 1, variant=7)
