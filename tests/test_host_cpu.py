"""CPU-only checks: the oracle against committed golden vectors and its own two forms, the
registry's slot order, graph extraction, and that the C-ABI library loads and exports every
symbol the header declares."""
import re
from pathlib import Path

import numpy as np
import pytest
import torch

from oracle import lm_ops_oracle as oracle

ROOT = Path(__file__).resolve().parent.parent
GOLDEN = ROOT / "tests" / "golden" / "lm_ops_golden.npz"


def test_library_exports_every_declared_symbol(built_lib):
    from monet_b200 import _lib
    header = (ROOT / "include" / "monet_b200.h").read_text()
    declared = set(re.findall(r"\b(mb_[a-z0-9_]+)\s*\(", header))
    declared -= {"mb_pool_desc", "mb_bn_desc", "mb_conv_desc"}
    assert declared, "no declarations found"
    assert declared == set(_lib.PROTOTYPES), declared ^ set(_lib.PROTOTYPES)
    handle = _lib.lib()
    for name in declared:
        assert hasattr(handle, name), name
    assert handle.mb_abi_version() >= 1
    assert handle.mb_conv_num_variants(0) >= 1 and handle.mb_conv_num_variants(2) >= 2
    assert handle.mb_pool_out_size(112, 3, 2, 1, 1, 0) == 56
    assert handle.mb_pool_out_size(10, 3, 2, 0, 1, 1) == 5


def test_ops_refuse_cpu_tensors(built_lib):
    from monet_b200 import functional as F
    with pytest.raises(RuntimeError, match="CUDA"):
        F.relu(torch.randn(8))


def test_registry_slot_order():
    import monet_b200.lm_ops as L
    names = lambda mode, op: [c.__name__ for c in L.list_ops(mode, op)]   # noqa: E731
    m = "conv_multiway_newnode"
    assert names(m, "aten::relu") == ["InputActReLU", "OutputActReLU", "BinaryActReLU"]
    assert names(m, "aten::relu_") == ["InputActReLU", "OutputActReLU", "BinaryActReLU"]
    assert names(m, "aten::batch_norm") == ["InputActBatchNorm", "OutputActBatchNorm"]
    assert names(m, "aten::max_pool2d") == ["SimpleMaxPool2D", "IndicesActMaxPool2D"]
    assert names(m, "aten::_convolution") == ["SpecificAlgoConvolution"]
    assert names("normal", "aten::_convolution") == ["GreedyAlgoConvolution"]
    assert names("none", "aten::_convolution") == ["PytorchConvolution"]
    assert names("normal", "aten::relu") == ["InputActReLU"]
    assert names("conv_normal", "aten::relu") == ["OutputActReLU"]
    assert names(m, "aten::hardtanh") == ["InputActHardTanh", "OutputActHardTanh"]
    for mode, table in L.registry.items():
        for op, impls in table.items():
            assert len(impls) <= 3, (mode, op)          # the solver has three slots per op
    assert L.relu.BinaryActReLU.backward_storage.size((4, 64, 112, 112)) == 401408
    assert L.pool.IndicesActMaxPool2D.backward_storage.size((4, 64, 56, 56)) == 401408


def test_install_into_a_foreign_registry():
    import types
    import monet_b200.lm_ops as L
    fake = types.SimpleNamespace(registry={"normal": {"aten::relu": ["stale"]}})
    L.install_into(fake)
    assert fake.registry["normal"]["aten::relu"] == L.list_ops("normal", "aten::relu")


def test_graph_extraction_and_policies():
    import torchvision
    from monet_b200 import runner
    model = torchvision.models.resnet50()
    nodes, out = runner.extract_graph(model)
    ops = [n.op for n in nodes]
    assert ops.count("aten::_convolution") == 53 and ops.count("aten::batch_norm") == 53
    assert ops.count("aten::add") == 16 and nodes[out].op == "aten::addmm"
    r = runner.Runner(model, runner.low_memory)
    bn = [n for n in nodes if n.op == "aten::batch_norm"]
    assert all(r.choices[n.id].impl == 1 for n in bn)
    with pytest.raises(ValueError):
        runner.Runner(model, lambda ns, n: runner.Choice(inplace=(n.op == "aten::_convolution")))


def test_graph_fusion_rewrite():
    """batch_norm -> relu and batch_norm -> add -> relu chains become fused nodes; the rewritten
    graph stays in dependency order and its users lists are consistent."""
    import torchvision
    from monet_b200 import runner
    for make, n_add in ((torchvision.models.resnet50, 16), (torchvision.models.resnet18, 8)):
        nodes, out = runner.extract_graph(make())
        n_relu = sum(n.op.startswith("aten::relu") for n in nodes)
        fused, fout = runner.fuse_graph(nodes, out)
        ops = [n.op for n in fused]
        assert ops.count("monet::batch_norm_add_relu") == n_add
        assert ops.count("monet::batch_norm_relu") == n_relu - n_add
        assert not any(o in ("aten::relu", "aten::relu_", "aten::add", "aten::add_") for o in ops)
        assert fused[fout].op == "aten::addmm"
        users = {n.id: [] for n in fused}
        for i, n in enumerate(fused):
            assert n.id == i
            for a in n.args:
                if a.kind == "node":
                    assert a.value < n.id          # producers come first
                    users[a.value].append(n.id)
        assert all(sorted(users[n.id]) == sorted(n.users) for n in fused)
        far = [n for n in fused if n.op == "monet::batch_norm_add_relu"]
        assert all(len(n.args) == 10 and n.args[9].kind == "node" for n in far)
    # a batch norm whose output has a second reader is left alone
    import torch.nn as nn

    class TwoReaders(nn.Module):
        def __init__(self):
            super().__init__()
            self.c = nn.Conv2d(4, 4, 1)
            self.b = nn.BatchNorm2d(4)
            self.r = nn.ReLU()

        def forward(self, x):
            z = self.b(self.c(x))
            return self.r(z) + z

    nodes, out = runner.extract_graph(TwoReaders())
    fused, _ = runner.fuse_graph(nodes, out)
    assert [n.op for n in fused] == [n.op for n in runner.extract_graph(TwoReaders())[0]]
    r = runner.Runner(torchvision.models.resnet18(), runner.low_memory, fuse=True)
    assert all(r.choices[n.id].recompute for n in r.nodes if n.op == "monet::batch_norm_relu")
    # the 10 GB schedule drops every second block output, never two in a row
    r = runner.Runner(torchvision.models.resnet50(), runner.budget_10gb, fuse=True)
    flags = [r.choices[n.id].recompute for n in r.nodes if n.op == "monet::batch_norm_add_relu"]
    assert flags == [False, True] * 8


def test_oracle_maxpool_forms_agree():
    g = torch.Generator().manual_seed(0)
    x = torch.randn(2, 3, 9, 10, generator=g)
    x[0, 0, 1, 1] = float("nan")
    for k, s, p, d, c in [(3, 2, 1, 1, False), (2, 2, 0, 1, False), (3, 2, 0, 1, True), (3, 1, 1, 2, False)]:
        _, a = oracle.maxpool_local_index(x, k, s, p, d, c)
        _, b = oracle.maxpool_forward(x, k, s, p, d, c)
        assert np.array_equal(a, b)


def test_oracle_bn_from_output_matches_autograd():
    g = torch.Generator().manual_seed(1)
    x = torch.randn(4, 6, 5, 5, generator=g)
    gamma = torch.rand(6, generator=g) + 0.5
    beta = torch.randn(6, generator=g)
    dy = torch.randn(4, 6, 5, 5, generator=g)
    y, mean, invstd, _, _ = oracle.bn_forward_train(x, gamma, beta, torch.zeros(6), torch.ones(6))
    dx, dg, db = oracle.bn_backward_from_output(dy, y, gamma, beta, invstd)
    rx, rg, rb = oracle.bn_backward_from_input(dy, x, gamma)
    assert torch.allclose(dx, rx, atol=1e-5) and torch.allclose(dg, rg, atol=1e-4) and torch.allclose(db, rb, atol=1e-4)


def test_oracle_against_golden_vectors():
    """Fixtures generated once from PyTorch CPU by tests/golden/make_golden.py."""
    z = np.load(GOLDEN)
    x = torch.from_numpy(z["relu_x"])
    assert np.array_equal(oracle.relu_mask_bytes(x), z["relu_mask"])
    assert np.array_equal(oracle.pack_nibbles(z["nib_in"]), z["nib_out"])
    assert np.array_equal(oracle.unpack_nibbles(z["nib_out"], z["nib_in"].size), z["nib_in"])
    px = torch.from_numpy(z["pool_x"])
    y, local = oracle.maxpool_forward(px, 3, 2, 1)
    assert np.array_equal(y.numpy(), z["pool_y"]) and np.array_equal(local, z["pool_local"])
    assert np.array_equal(oracle.maxpool_nibbles(local), z["pool_nibbles"])
    dx = oracle.maxpool_backward_from_index(torch.from_numpy(z["pool_dy"]), local, px.shape, 3, 2, 1)
    assert np.allclose(dx.numpy(), z["pool_dx"], atol=1e-6)
    bx = torch.from_numpy(z["bn_x"])
    y, mean, invstd, rm, rv = oracle.bn_forward_train(
        bx, torch.from_numpy(z["bn_gamma"]), torch.from_numpy(z["bn_beta"]),
        torch.zeros(bx.shape[1]), torch.ones(bx.shape[1]))
    assert np.allclose(y.numpy(), z["bn_y"], atol=1e-5)
    assert np.allclose(mean.numpy(), z["bn_mean"], atol=1e-6) and np.allclose(invstd.numpy(), z["bn_invstd"], rtol=1e-5)
    dx, dg, db = oracle.bn_backward_from_output(torch.from_numpy(z["bn_dy"]), y, torch.from_numpy(z["bn_gamma"]),
                                               torch.from_numpy(z["bn_beta"]), invstd)
    assert np.allclose(dx.numpy(), z["bn_dx"], atol=1e-5) and np.allclose(dg.numpy(), z["bn_dgamma"], atol=1e-4)
    loss, dlog = oracle.cross_entropy(torch.from_numpy(z["ce_logits"]), torch.from_numpy(z["ce_labels"]), 0.25)
    assert np.allclose(loss.numpy(), z["ce_loss"], atol=1e-6) and np.allclose(dlog.numpy(), z["ce_dlogits"], atol=1e-7)
    s = oracle.stem_reference(N=1, H=32, W=32)
    assert np.allclose(s["y"].numpy(), z["stem_y"], atol=1e-5)
    assert np.array_equal(s["mask"], z["stem_mask"]) and np.array_equal(s["nibbles"], z["stem_nibbles"])
    assert np.allclose(s["dw"].numpy(), z["stem_dw"], atol=1e-4)


def test_unet_with_transposed_convolution_through_the_runner_on_cpu():
    """Host logic of the transposed convolution (forward = backward-data kernel, backward-data =
    forward kernel, backward-filter with operands exchanged), concatenation and per-pixel
    cross-entropy: a small UNet through the executor on the CPU stand-in of the tensor-level
    functions, against autograd."""
    import copy
    import sys
    from pathlib import Path
    sys.path.insert(0, str(Path(__file__).resolve().parent))
    import cpu_functional
    import bench
    from monet_b200 import runner
    from monet_b200.lm_ops.softmax import SoftmaxCrossEntropy
    torch.manual_seed(0)
    model = bench._unet(n_classes=2, base=4).train()
    x = torch.randn(2, 3, 32, 48)
    y = torch.randint(0, 2, (2, 32, 48))
    ref = copy.deepcopy(model)
    loss_ref = torch.nn.functional.cross_entropy(ref(x), y)
    loss_ref.backward()
    for policy in (runner.store_all, runner.low_memory):
        m = copy.deepcopy(model)
        run = runner.Runner(m, policy)
        ce = SoftmaxCrossEntropy()
        with cpu_functional.patched():
            loss = ce.forward(run.forward(x), y)
            run.backward(ce.backward())
        assert abs(float(loss) - float(loss_ref.detach())) < 1e-5
        top = max(float(p.grad.abs().max()) for p in ref.parameters())
        for (k, p), (_, q) in zip(m.named_parameters(), ref.named_parameters()):
            err = float((p.grad - q.grad).abs().max())
            assert err < 2e-3 * float(q.grad.abs().max()) + 1e-4 * top, (k, err)


def test_rejected_geometries_say_why(built_lib):
    """Geometries outside the kernels' range return MB_ERR_UNSUPPORTED with a message before
    anything touches the device (no GPU needed: the descriptor is validated first)."""
    import ctypes as C
    from monet_b200 import _lib
    api = _lib.lib()
    one = C.c_void_p(16)          # a non-null, 16-byte aligned stand-in: never dereferenced

    def conv(N, Cc, H, W, K, R, S, s, pad, groups=1):
        P = (H + 2 * pad - (R - 1) - 1) // s + 1
        Q = (W + 2 * pad - (S - 1) - 1) // s + 1
        return _lib.ConvDesc(N, Cc, H, W, K, R, S, P, Q, s, s, pad, pad, 1, 1, groups)

    cases = [
        (conv(1, 32, 16, 16, 32, 3, 3, 3, 1), "stride"),            # stride above 2
        (conv(1, 32, 16, 16, 32, 3, 3, 1, 1, groups=2), "group"),   # grouped, not depthwise
        (conv(1, 32, 20, 20, 32, 9, 9, 1, 4), "taps"),              # more than 64 filter taps
        (conv(1, 30, 16, 16, 32, 3, 3, 1, 1), "multiples of 4"),    # channel count not padded
    ]
    for d, word in cases:
        rc = api.mb_conv2d_fprop(one, one, None, one, C.byref(d), 0, None, 0, None)
        assert rc == 2, (word, rc, _lib.last_error())
        assert word in _lib.last_error(), _lib.last_error()
    d = conv(1, 32, 16, 16, 64, 3, 3, 1, 1, groups=32)              # depthwise with a channel multiplier
    rc = api.mb_depthwise_fprop(one, one, None, one, C.byref(d), None)
    assert rc == 2 and "groups" in _lib.last_error()
    d = conv(1, 32, 16, 16, 32, 3, 3, 1, 1)
    assert api.mb_conv2d_fprop(one, one, None, one, C.byref(d), 7, None, 0, None) == 2   # no such variant
    pd = _lib.PoolDesc(1, 8, 16, 16, 4, 4, 5, 5, 3, 3, 0, 0, 1, 1, _lib.MB_NHWC)          # 25 taps > 4 bits
    assert api.mb_maxpool2d_fwd(one, one, one, C.byref(pd), None) == 2 and "4-bit" in _lib.last_error()
