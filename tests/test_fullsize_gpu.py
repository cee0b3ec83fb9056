"""Full-size cases of the ResNet-50 batch-184 workload, checked through properties that do not
need the CPU oracle at that size (it would take minutes): round trips, conservation laws,
orthogonality relations and linearity."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_relu_mask_round_trip_at_stem_size(cuda):
    """184 x 64 x 112 x 112 (147.7 M elements, 18.5 MB of mask)."""
    from monet_b200 import functional as F
    g = torch.Generator(device=cuda).manual_seed(0)
    x = torch.randn(184, 64, 112, 112, device=cuda, generator=g).contiguous(memory_format=torch.channels_last)
    y, mask = F.relu_mask(x)
    assert mask.numel() == (x.numel() + 7) // 8
    pos = x.permute(0, 2, 3, 1).reshape(-1) > 0                       # physical order
    assert torch.equal(F.unpack_bits(mask, x.numel()), pos)            # unpack(pack(.)) is the identity
    assert torch.equal(F.pack_bits(pos), mask)                         # both packers agree
    assert torch.equal(y, torch.clamp_min(x, 0))
    dy = torch.randn_like(x)
    dx = F.relu_bwd_mask(dy, mask, inplace=False)
    assert torch.equal(dx, dy * (x > 0))
    assert torch.equal(F.relu_bwd_mask(dx, mask, inplace=False), dx)  # masking is idempotent


def test_maxpool_conservation_at_stem_size(cuda):
    from monet_b200 import functional as F
    g = torch.Generator(device=cuda).manual_seed(1)
    x = torch.randn(184, 64, 112, 112, device=cuda, generator=g).contiguous(memory_format=torch.channels_last)
    y, nib, d = F.maxpool2d(x, 3, 2, 1, 1, False)
    assert nib.numel() == (y.numel() + 1) // 2
    assert int((nib >> 4).max()) <= 8 and int((nib & 15).max()) <= 8   # 3x3 window: indices 0..8
    ones = torch.ones_like(y)
    dx = F.maxpool2d_bwd(ones, nib, d)
    assert float(dx.sum()) == float(y.numel())                         # every output's gradient lands once
    assert float(dx.min()) >= 0 and float(dx.max()) <= 4               # a pixel is in at most 4 windows
    # scattering y back to its argmax positions reproduces x there (a pixel that wins k
    # windows receives k copies of the same maximum)
    up = F.maxpool2d_bwd(y, nib, d)
    hit = dx > 0
    assert torch.allclose(up[hit], (x * dx)[hit], rtol=1e-6, atol=0)


def test_batchnorm_invariants_at_layer1_size(cuda):
    """184 x 256 x 56 x 56: normalised output statistics, and the two orthogonality relations
    every batch-norm input gradient satisfies (sum dx = 0 and sum dx * xhat = 0 per channel)."""
    from monet_b200 import functional as F
    g = torch.Generator(device=cuda).manual_seed(2)
    x = (torch.randn(184, 256, 56, 56, device=cuda, generator=g) * 3 + 5).contiguous(memory_format=torch.channels_last)
    gamma = torch.rand(256, device=cuda, generator=g) + 0.5
    beta = torch.randn(256, device=cuda, generator=g)
    y, mean, invstd = F.bn_fwd_train(x, gamma, beta, None, None, 0.1, 1e-5)
    xhat = (y - beta.view(1, -1, 1, 1)) / gamma.view(1, -1, 1, 1)
    assert float(xhat.mean((0, 2, 3)).abs().max()) < 1e-4
    assert float((xhat.var((0, 2, 3), unbiased=False) - 1).abs().max()) < 1e-3
    dy = torch.randn_like(x)
    for dx, dg, db in (F.bn_bwd_from_output(dy, y, gamma, beta, invstd),
                       F.bn_bwd_from_input(dy, x, gamma, mean, invstd)):
        M = x.numel() / 256
        assert float(dx.sum((0, 2, 3)).abs().max()) / M < 1e-5
        assert float((dx * xhat).sum((0, 2, 3)).abs().max()) / M < 1e-4
        assert torch.allclose(db, dy.sum((0, 2, 3)), rtol=1e-4, atol=1e-2)
        assert torch.allclose(dg, (dy * xhat).sum((0, 2, 3)), rtol=1e-3, atol=5e-2)


@pytest.mark.parametrize("geom", [(64, 56, 64, 3, 1, 1), (256, 14, 1024, 1, 1, 0), (128, 56, 128, 3, 2, 1)])
def test_conv_linearity_and_adjointness_at_layer_size(cuda, geom):
    """Full batch 184.  Forward is linear in x; backward-data is the adjoint of forward
    (<conv(x), dy> = <x, dgrad(dy)>) and backward-filter its derivative in w
    (<conv_w(x), dy> = <w, wgrad(x, dy)>), all within the TF32 tolerance."""
    from monet_b200 import functional as F
    C, H, K, R, s, p = geom
    g = torch.Generator(device=cuda).manual_seed(3)
    cl = torch.channels_last
    x1 = torch.randn(184, C, H, H, device=cuda, generator=g).contiguous(memory_format=cl)
    x2 = torch.randn(184, C, H, H, device=cuda, generator=g).contiguous(memory_format=cl)
    w = (torch.randn(K, C, R, R, device=cuda, generator=g) * (2.0 / (C * R * R)) ** 0.5).contiguous(memory_format=cl)
    y1 = F.conv2d_fprop(x1, w, None, s, p, 1)
    y2 = F.conv2d_fprop(x2, w, None, s, p, 1)
    y12 = F.conv2d_fprop(x1 * 0.5 + x2, w, None, s, p, 1)
    scale = float(y1.abs().max())
    assert float((y12 - (0.5 * y1 + y2)).abs().max()) < 2e-2 * scale
    dy = torch.randn_like(y1)
    dx = F.conv2d_dgrad(dy, w, x1.shape, s, p, 1)
    dw, _ = F.conv2d_wgrad(x1, dy, w.shape, s, p, 1)
    lhs = float((y1.double() * dy.double()).sum())
    assert abs(lhs - float((x1.double() * dx.double()).sum())) < 2e-2 * abs(lhs) + 1e-3 * y1.numel() ** 0.5
    assert abs(lhs - float((w.double() * dw.double()).sum())) < 2e-2 * abs(lhs) + 1e-3 * y1.numel() ** 0.5
    assert F.conv_device_status() == 0
