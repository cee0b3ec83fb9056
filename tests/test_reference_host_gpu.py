"""The drop-in proper: MONeT's own ``MONeTWrapper`` / ``Schedule`` / ``SolverInfo`` / profiler
(``meminfo``, ``computeinfo``) running unmodified over the sm_100a kernels.

The reference's host modules are installed under ``baseline/_ref`` by ``baseline/install_ref.py``
(they travel with the working tree); ``monet_b200.reference_host.activate()`` registers this
package as ``monet.lm_ops``.  Results are compared with this repo's own executor (same kernels,
so near-exact) and with fp32 CPU autograd at the whole-network bar of test_runner_gpu.py."""
import copy
import sys
from pathlib import Path

import numpy as np
import pytest
import torch
import torchvision

sys.path.insert(0, str(Path(__file__).resolve().parent))

from baseline import install_ref  # noqa: E402

pytestmark = [pytest.mark.gpu,
              pytest.mark.skipif(not install_ref.installed(), reason="MONeT host code not installed")]

MODE = "inplace_conv_multiway_newnode"


def _rel(a, ref):
    return float((a - ref).norm() / ref.norm().clamp_min(1e-12))


def _cpu_reference(model, x, labels):
    m = copy.deepcopy(model).cpu().train()
    out = m(x)
    loss = torch.nn.functional.cross_entropy(out, labels)
    loss.backward()
    return out.detach(), float(loss), {k: p.grad.clone() for k, p in m.named_parameters()}


def _tf32_grads(model, x, labels, cuda):
    torch.backends.cudnn.allow_tf32 = True
    try:
        tm = copy.deepcopy(model).to(cuda).train()
        torch.nn.functional.cross_entropy(tm(x.to(cuda)), labels.to(cuda)).backward()
        return {k: p.grad.detach().cpu() for k, p in tm.named_parameters()}
    finally:
        torch.backends.cudnn.allow_tf32 = False


@pytest.mark.parametrize("arch,batch", [("resnet18", 8), ("resnet50", 8)])
def test_monet_wrapper_trains_through_the_kernels(cuda, tmp_path, arch, batch):
    """MONeTWrapper(model, solution.pkl, shape) -> loss.backward(), for a store-all, a low-memory
    and an ILP-solved solution (monet_wrapper.py:7-44, schedule.py:58-311)."""
    from monet_b200 import functional as F
    from monet_b200 import reference_host as rh
    from monet_b200 import runner, solver
    from monet_b200.lm_ops.softmax import SoftmaxCrossEntropy
    ref = rh.activate()
    torch.manual_seed(0)
    model = getattr(torchvision.models, arch)(num_classes=10).train()
    x = torch.randn(batch, 3, 64, 64)
    labels = torch.randint(0, 10, (batch,))
    ref_out, ref_loss, ref_grads = _cpu_reference(model, x, labels)
    tf32 = _tf32_grads(model, x, labels, cuda)

    # this repo's executor on the same operator set (no fused nodes): the near-exact yardstick
    gm = copy.deepcopy(model).to(cuda).train()
    r = runner.Runner(gm, runner.store_all)
    ce = SoftmaxCrossEntropy()
    ce.forward(r.forward(x.to(cuda)), labels.to(cuda))
    r.backward(ce.backward())
    own = {k: p.grad.detach().clone() for k, p in gm.named_parameters()}

    graph, si = rh.build_solver_info(model, batch, arch, MODE, (3, 64, 64), workdir=tmp_path, profile=False)
    solutions = {"store_all": solver.hand_solution(si, "store_all"),
                 "low_memory": solver.hand_solution(si, "low_memory")}
    if arch == "resnet18":
        peak = solver.check_solution(si, solutions["store_all"])["peak_gb"]
        _, si64 = rh.build_solver_info(model, 64, arch, MODE, (3, 64, 64), workdir=tmp_path / "b64", profile=False)
        peak64 = solver.check_solution(si64, solver.hand_solution(si64, "store_all"))["peak_gb"]
        solutions["solved"] = solver.solve(si64, 0.8 * peak64, time_limit=240)
        assert peak > 0
    for kind, sol in solutions.items():
        path = rh.save_solution(si, sol, tmp_path / f"solution_{kind}.pkl")
        wrapped = ref.monet_wrapper.MONeTWrapper(copy.deepcopy(model), str(path), (3, 64, 64)).cuda()
        out = wrapped(x.to(cuda))
        loss = torch.nn.functional.cross_entropy(out, labels.to(cuda))
        loss.backward()
        torch.cuda.synchronize()
        assert F.conv_device_status() == 0
        assert _rel(out.detach().cpu(), ref_out) < 5e-2
        assert abs(float(loss) - ref_loss) < 2e-2 * max(1.0, abs(ref_loss))
        for k, p in wrapped.model.named_parameters():
            assert p.grad is not None, (kind, k)
            ours, theirs = _rel(p.grad.cpu(), ref_grads[k]), _rel(tf32[k], ref_grads[k])
            assert ours < 1.6 * theirs + 2e-2, (kind, k, ours, theirs)
            if kind == "store_all":          # same kernels, same order as this repo's executor
                assert _rel(p.grad, own[k]) < 1e-3 + 0.2 * theirs, (k, _rel(p.grad, own[k]))


class _Tiny(torch.nn.Module):
    def __init__(self):
        super().__init__()
        nn = torch.nn
        self.conv1 = nn.Conv2d(3, 32, 3, 1, 1, bias=False); self.bn1 = nn.BatchNorm2d(32)
        self.relu = nn.ReLU(inplace=True)
        self.pool = nn.MaxPool2d(3, 2, 1)
        self.conv2 = nn.Conv2d(32, 64, 3, 1, 1, bias=False); self.bn2 = nn.BatchNorm2d(64)
        self.avg = nn.AdaptiveAvgPool2d((1, 1))
        self.fc = nn.Linear(64, 10)

    def forward(self, x):
        x = self.pool(self.relu(self.bn1(self.conv1(x))))
        x = self.relu(self.bn2(self.conv2(x)))
        return self.fc(torch.flatten(self.avg(x), 1))


@pytest.mark.parametrize("profiler", ["reference", "events"])
def test_reference_profiler_fills_the_cost_tables(cuda, tmp_path, profiler):
    """SolverInfo.extract with MONeT's own meminfo / computeinfo (meminfo.py:6-396,
    solver_info.py:338-427) over every implementation and convolution variant; then the ILP on
    those measured tables and a step under the resulting schedule."""
    from monet_b200 import functional as F
    from monet_b200 import reference_host as rh
    from monet_b200 import solver
    from monet_b200._lib import MB_CONV_WGRAD
    ref = rh.activate()
    torch.manual_seed(0)
    model = _Tiny().to(cuda).train()
    batch = 32
    graph, si = rh.build_solver_info(model, batch, "tiny", MODE, (3, 32, 32), workdir=tmp_path, profile=True,
                                     profiler=profiler)
    assert (tmp_path / "data" / f"cost_tiny_{batch}_{MODE}.pkl").exists()     # solver_info.py:425-427
    BwdNode = ref.solver_info.BwdNode
    n_conv = 0
    for i, node in si.nodes.items():
        assert len(node.workspace_compute) == len(node.workspace_mem) >= 1, (i, node)
        if isinstance(node, BwdNode) and node.fwd_node.op == "aten::_convolution":
            n_conv += 1
            want = F.conv_num_variants(MB_CONV_WGRAD) if node.bwd_op == "param_grad" else 1
            assert len(node.workspace_compute) == want
            assert all(t > 0 for t in node.workspace_compute)          # every variant ran (none is -1)
            c_in = graph.nodes[node.fwd_node.args[0].index].shape[1]
            if node.bwd_op == "param_grad" and c_in > 4:      # (few-channel inputs take their own kernels)
                # the deterministic variant's scratch shows up in the allocator peak the profiler
                # reads, and is what mb_conv_workspace_bytes declares for it
                shape = [batch if s == -1 else s for s in graph.nodes[node.fwd_node.args[0].index].shape]
                w = graph.nodes[node.fwd_node.args[1].index].shape
                d = F.conv_desc(shape, w, node.fwd_node.args[3].value, node.fwd_node.args[4].value,
                                node.fwd_node.args[5].value, 1)
                d = F._padded_desc(d)
                declared = F.conv_workspace_bytes(MB_CONV_WGRAD, 1, d) - F.conv_workspace_bytes(MB_CONV_WGRAD, 0, d)
                measured = (node.workspace_mem[1] - node.workspace_mem[0]) * 2 ** 20
                assert declared > 0
                assert 0.98 * declared <= measured <= declared + 2 ** 20, (measured, declared)
    assert n_conv == 4            # two convolutions x (param_grad, ip_grad)
    for i in range(si.loss):
        node = si.nodes[i]
        if node.op == "aten::relu_":
            assert len(node.workspace_compute) == 3        # three ReLU implementations profiled
    peak = solver.check_solution(si, solver.hand_solution(si, "store_all"))["peak_gb"]
    sol = solver.solve(si, 0.85 * peak, time_limit=120)
    assert solver.check_solution(si, sol, 0.85 * peak)["violations"] == []
    sched = rh.make_schedule(graph, si, sol)
    x = torch.randn(batch, 3, 32, 32, device=cuda)
    params = list(model.state_dict(keep_vars=True).values())
    out = sched.forward(x, *params)
    sched.backward(torch.ones_like(out))
    torch.cuda.synchronize()
    m2 = copy.deepcopy(model).cpu()
    for p in m2.parameters():
        p.grad = None
    o2 = m2(x.cpu())
    o2.backward(torch.ones_like(o2))
    assert _rel(out.cpu(), o2.detach()) < 2e-2
    for (k, p), (_, q) in zip(model.named_parameters(), m2.named_parameters()):
        assert _rel(p.grad.cpu(), q.grad) < 5e-2, k
