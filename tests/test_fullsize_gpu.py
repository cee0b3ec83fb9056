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


# The 23 distinct convolution geometries of ResNet-50 (torchvision v1.5 layout) at 224 x 224:
# (C, H, K, R, stride, pad); the GEMM shapes they give at batch 184 are M = 184 * P * Q from
# 9 016 to 2 308 096.
RESNET50_GEOMETRIES = [
    (3, 224, 64, 7, 2, 3),
    (64, 56, 64, 1, 1, 0), (64, 56, 64, 3, 1, 1), (64, 56, 256, 1, 1, 0), (256, 56, 64, 1, 1, 0),
    (256, 56, 128, 1, 1, 0), (128, 56, 128, 3, 2, 1), (128, 28, 512, 1, 1, 0), (256, 56, 512, 1, 2, 0),
    (512, 28, 128, 1, 1, 0), (128, 28, 128, 3, 1, 1),
    (512, 28, 256, 1, 1, 0), (256, 28, 256, 3, 2, 1), (256, 14, 1024, 1, 1, 0), (512, 28, 1024, 1, 2, 0),
    (1024, 14, 256, 1, 1, 0), (256, 14, 256, 3, 1, 1),
    (1024, 14, 512, 1, 1, 0), (512, 14, 512, 3, 2, 1), (512, 7, 2048, 1, 1, 0), (1024, 14, 2048, 1, 2, 0),
    (2048, 7, 512, 1, 1, 0), (512, 7, 512, 3, 1, 1),
]
SAMPLED = (0, 91, 183)


@pytest.mark.parametrize("geom", RESNET50_GEOMETRIES, ids=lambda g: "c%d_h%d_k%d_r%d_s%d" % g[:5])
def test_resnet50_convolutions_at_batch_184_against_the_oracle(cuda, geom):
    """Every convolution geometry of the workload at its real batch, three passes, against the
    fp32 CPU oracle at rtol 2e-2 of the tensor's scale.  The launches are the batch-184 ones
    (tile widths, super-tiles and split counts are chosen from the problem size), the oracle
    runs on three images:

    * fprop and dgrad are independent per image: images 0, 91 and 183 of y and dx are compared
      with the oracle applied to those images alone;
    * wgrad sums over the batch: dy is zero outside the three images, so the batch-184 launch
      (both variants) must reproduce the oracle's dw and db of the 3-image sub-batch."""
    from monet_b200 import functional as F
    from oracle import lm_ops_oracle as oracle
    C, H, K, R, s, p = geom
    N = 184
    g = torch.Generator(device=cuda).manual_seed(7)
    x = torch.randn(N, C, H, H, device=cuda, generator=g)
    if C % 4 == 0:
        x = x.contiguous(memory_format=torch.channels_last)
    w = (torch.randn(K, C, R, R, device=cuda, generator=g) * (2.0 / (C * R * R)) ** 0.5)
    idx = list(SAMPLED)
    xs, ws = x[idx].cpu().contiguous(), w.cpu()

    def err(a, ref):
        return float((a - ref).abs().max() / ref.abs().max().clamp_min(1e-6))

    y = F.conv2d_fprop(x, w, None, s, p, 1)
    ref_y = oracle.conv_forward(xs, ws, None, s, p, 1)
    assert tuple(y.shape) == (N,) + tuple(ref_y.shape[1:])
    assert err(y[idx].cpu(), ref_y) < 2e-2, ("fprop", err(y[idx].cpu(), ref_y))

    dy = torch.randn(y.shape, device=cuda, generator=g).contiguous(memory_format=torch.channels_last)
    dys = dy[idx].cpu().contiguous()
    ref_dx, ref_dw, ref_db = oracle.conv_backward(dys, xs, ws, s, p, 1)
    dx = F.conv2d_dgrad(dy, w, x.shape, s, p, 1)
    assert err(dx[idx].cpu(), ref_dx) < 2e-2, ("dgrad", err(dx[idx].cpu(), ref_dx))
    del dx, y

    mask = torch.zeros(N, 1, 1, 1, device=cuda)
    mask[idx] = 1
    dy_sparse = (dy * mask).contiguous(memory_format=torch.channels_last)
    del dy
    for variant in (0, 1):
        dw, db = F.conv2d_wgrad(x, dy_sparse, w.shape, s, p, 1, variant=variant, need_bias=True)
        assert err(dw.cpu(), ref_dw) < 2e-2, ("wgrad", variant, err(dw.cpu(), ref_dw))
        assert torch.allclose(db.cpu(), ref_db, rtol=1e-4, atol=1e-3)
    assert F.conv_device_status() == 0


# 3x3 layers of VGG-16 (224-wide input) and of the UNet configuration (416 x 608 input) at their
# real spatial extents, with a batch the CPU oracle finishes in seconds: (N, C, H, W, K).  They
# select the column-tiled many-tap kernels, the backward-filter halo kernel with column tiles
# and row-wise dy copies, and the backward-filter-by-filter-row mode (with and without tiles).
WIDE_LAYERS = [(2, 64, 224, 224, 64), (1, 64, 416, 608, 64), (1, 128, 416, 608, 64), (1, 128, 208, 304, 128),
               (2, 128, 112, 112, 128), (2, 512, 28, 28, 512), (1, 256, 52, 76, 512), (1, 64, 208, 304, 128),
               (2, 3, 224, 224, 64), (1, 3, 416, 608, 64)]        # the two networks' first layers (few-channel path)


@pytest.mark.parametrize("layer", WIDE_LAYERS, ids=lambda g: "n%d_c%d_%dx%d_k%d" % g)
def test_vgg_and_unet_layers_at_their_real_extents(cuda, layer):
    from monet_b200 import functional as F
    from oracle import lm_ops_oracle as oracle
    N, C, H, W, K = layer
    g = torch.Generator().manual_seed(C + W)
    x = torch.randn(N, C, H, W, generator=g)
    w = torch.randn(K, C, 3, 3, generator=g) * (2.0 / (C * 9)) ** 0.5
    ref_y = oracle.conv_forward(x, w, None, 1, 1, 1)
    dy = torch.randn(ref_y.shape, generator=g)
    ref_dx, ref_dw, _ = oracle.conv_backward(dy, x, w, 1, 1, 1)

    def err(a, ref):
        return float((a.cpu() - ref).abs().max() / ref.abs().max().clamp_min(1e-6))

    xc = x.to(cuda).contiguous(memory_format=torch.channels_last) if C % 4 == 0 else x.to(cuda)
    dyc = dy.to(cuda).contiguous(memory_format=torch.channels_last)
    wc = w.to(cuda)
    assert err(F.conv2d_fprop(xc, wc, None, 1, 1, 1), ref_y) < 2e-2
    assert err(F.conv2d_dgrad(dyc, wc, x.shape, 1, 1, 1), ref_dx) < 2e-2
    for variant in (0, 1):
        dw, _ = F.conv2d_wgrad(xc, dyc, w.shape, 1, 1, 1, variant=variant)
        assert err(dw, ref_dw) < 2e-2, ("wgrad", variant, err(dw, ref_dw))
    assert F.conv_device_status() == 0


def test_stem_configuration_verbatim(cuda):
    """The CPU-runnable configuration at its stated size: N = 4, 3 x 224 x 224, conv 7x7/2 ->
    BN(train) -> ReLU (1-bit mask) -> max-pool 3x3/2 (4-bit indices), forward and backward through
    the four operator classes; y, dx, dW, dgamma, dbeta against torch CPU, and all 401 408 mask
    bytes and 401 408 index bytes bit-exact against the oracle applied to the tensors the
    operators saw."""
    import numpy as np
    from monet_b200 import functional as F
    from monet_b200 import lm_ops
    from oracle import lm_ops_oracle as oracle
    ref = oracle.stem_reference()                     # N=4, 224 x 224
    mode = "conv_multiway_newnode"
    conv = lm_ops.list_ops(mode, "aten::_convolution")[0]()
    bn = lm_ops.list_ops(mode, "aten::batch_norm")[1]()
    relu = lm_ops.list_ops(mode, "aten::relu")[2]()
    pool = lm_ops.list_ops(mode, "aten::max_pool2d")[1]()
    x = ref["x"].to(cuda).requires_grad_(True)
    w = ref["w"].to(cuda).requires_grad_(True)
    gamma, beta = ref["gamma"].to(cuda), ref["beta"].to(cuda)
    rm, rv = torch.zeros(64, device=cuda), torch.ones(64, device=cuda)
    c = conv.forward(x, w, None, [2, 2], [3, 3], [1, 1], False, [0, 0], 1)
    b = bn.forward(c, gamma, beta, rm, rv, True, 0.1, 1e-5, True)
    r, mask = relu.forward(b)
    y, nib = pool.forward(r, [3, 3], [2, 2], [1, 1], [1, 1], False)
    assert mask.numel() == 401408 and nib.numel() == 401408
    cpu = lambda t: t.detach().cpu().contiguous()       # noqa: E731
    b_cpu, r_cpu = cpu(b), cpu(r)
    d_r = pool.backward(ref["dy"].to(cuda), [nib])
    d_b = relu.backward(d_r.clone(), [mask])
    d_c, dgamma, dbeta, _, _ = bn.backward(d_b, [gamma, beta, rm, rv, b])
    conv.algorithm = 20
    dx, dw = conv.backward(d_c, [x, w])
    torch.cuda.synchronize()
    assert F.conv_device_status() == 0

    def rel(a, t):
        return float((cpu(a) - t).abs().max() / t.abs().max().clamp_min(1e-12))

    # packed formats: bit-exact on the operators' own inputs (NHWC physical order)
    assert np.array_equal(mask.cpu().numpy(), oracle.relu_mask_bytes(b_cpu.permute(0, 2, 3, 1).contiguous()))
    o_y, local = oracle.maxpool_forward(r_cpu, 3, 2, 1)
    assert torch.equal(cpu(y), o_y)
    assert np.array_equal(nib.cpu().numpy(), oracle.maxpool_nibbles(local, nhwc=True))
    # against the all-fp32 torch CPU run of the whole stem.  The chain contains discrete decisions
    # (the ReLU gate and the pooling argmax): where TF32 rounding of the convolution flips one,
    # a gradient is routed to a different pixel, so single elements of dx can differ by their
    # whole size.  The chain is therefore compared in the L2 norm at the convolution tolerance,
    # and the number of flipped decisions is bounded; every operator is held to its own
    # element-wise tolerance on the same inputs below.
    def rel2(a, t):
        return float((cpu(a) - t).norm() / t.norm().clamp_min(1e-12))
    # (measured: 3e-4 for y, 2.1e-2 for dx, which sits behind both kinds of flip)
    for name, got, tol in (("y", y, 2e-2), ("dx", dx, 5e-2), ("dw", dw, 5e-2), ("dgamma", dgamma, 5e-2),
                           ("dbeta", dbeta, 5e-2)):
        assert rel2(got, ref[name]) < tol, (name, rel2(got, ref[name]))
    assert rel(y, ref["y"]) < 2e-2
    flipped_gate = float(((b_cpu > 0) != (ref["bn"] > 0)).float().mean())
    flipped_argmax = float((local != ref["local_idx"]).mean())
    assert flipped_gate < 2e-3 and flipped_argmax < 2e-3, (flipped_gate, flipped_argmax)
    # the convolution's own backward-data and backward-filter on the gradient the GPU chain produced
    o_dx, o_dw, _ = oracle.conv_backward(cpu(d_c), ref["x"], ref["w"], 2, 3)
    assert rel(dx, o_dx) < 2e-2 and rel(dw, o_dw) < 2e-2, (rel(dx, o_dx), rel(dw, o_dw))
    # the fp32 operators against the oracle on the same inputs: rtol 1e-5
    o_b, _, o_inv, _, _ = oracle.bn_forward_train(cpu(c), ref["gamma"], ref["beta"], torch.zeros(64), torch.ones(64))
    assert torch.allclose(b_cpu, o_b, rtol=1e-5, atol=1e-5)
    o_dr = oracle.maxpool_backward_from_index(ref["dy"], local, tuple(r.shape), 3, 2, 1)
    assert torch.allclose(cpu(d_r), o_dr, rtol=1e-5, atol=1e-6)
    assert torch.equal(cpu(d_b), oracle.relu_backward(cpu(d_r), b_cpu))
    o_dc, o_dg, o_db = oracle.bn_backward_from_output(cpu(d_b), b_cpu, ref["gamma"], ref["beta"], o_inv)
    assert torch.allclose(cpu(d_c), o_dc, rtol=1e-5, atol=1e-5)
    assert torch.allclose(cpu(dgamma), o_dg, rtol=1e-4, atol=1e-3) and torch.allclose(cpu(dbeta), o_db, rtol=1e-4, atol=1e-3)
