"""MONeT's own host code (Graph.create, SolverInfo, Schedule) driven over this operator library
on the CPU stand-in of the tensor-level functions, and the ILP port.

What is under test is host logic only: the torch-2 graph normalisation, the solver-info tables,
hand-made and solved ``Solution`` objects, and that ``Schedule.forward/backward``
(schedule.py:145-311) with those solutions reproduces autograd through the operator classes'
protocol (tuple returns for intermediates, ``del stored[i]``, ``params`` hand-over, in-place
flags, recomputation)."""
import copy
import sys
from pathlib import Path

import numpy as np
import pytest
import torch
import torchvision

sys.path.insert(0, str(Path(__file__).resolve().parent))

from baseline import install_ref  # noqa: E402

pytestmark = pytest.mark.skipif(not install_ref.installed(),
                                reason="MONeT host code not installed (python baseline/install_ref.py)")

MODE = "inplace_conv_multiway_newnode"      # "complete MONeT" (README.md:138)


@pytest.fixture(scope="module")
def host():
    from monet_b200 import reference_host as rh
    return rh, rh.activate()


def test_normalized_graph_shapes(host):
    rh, ref = host
    g = ref.graph
    gr = g.Graph.create(torchvision.models.resnet18(num_classes=10), (3, 64, 64))
    ops = [n.op for n in gr.nodes if isinstance(n, g.ComputeNode)]
    assert "aten::linear" not in ops and ops.count("aten::addmm") == 1
    assert ops.count("aten::add_") == 8                       # the 8 residual adds; the 20 counters are gone
    for k, n in enumerate(gr.nodes):
        if isinstance(n, g.ComputeNode):
            assert n.id == k and n.has_backward
            for i, rg in n.dependencies:
                if isinstance(gr.nodes[i], g.ComputeNode):
                    assert rg, (n, i)
    fc = gr.nodes[gr._outputs[0]]
    assert fc.op == "aten::addmm" and [type(a).__name__ for a in fc.args] == ["D", "D", "D", "V", "V"]
    assert list(gr.nodes[fc.args[0].index].shape) == [10]        # bias first, as addmm(b, x, W, 1, 1)
    assert list(gr.nodes[fc.args[2].index].shape) == [10, 512]
    # parameters and buffers keep the positions state_dict() has (schedule.py:196 indexes by them)
    sd = list(torchvision.models.resnet18(num_classes=10).state_dict().values())
    params = [n for n in gr.nodes if isinstance(n, g.Param)]
    assert [list(p.shape) for p in params] == [list(t.shape) for t in sd]


def _grads_through_schedule(rh, model, graph, si, sol, x, dy=None):
    import cpu_functional
    sched = rh.make_schedule(graph, si, sol)
    params = list(model.state_dict(keep_vars=True).values())
    for p in model.parameters():
        p.grad = None
    with cpu_functional.patched():
        out = sched.forward(x, *params)
        dy = torch.ones_like(out) if dy is None else dy
        sched.backward(dy)
    return out, {k: p.grad.clone() for k, p in model.named_parameters()}


def _autograd(model, x, dy=None):
    m = copy.deepcopy(model).train()
    for p in m.parameters():
        p.grad = None
    out = m(x)
    out.backward(torch.ones_like(out) if dy is None else dy)
    return out.detach(), {k: p.grad.clone() for k, p in m.named_parameters()}


def _close(got, want, what):
    """Every gradient within 2e-3 of its own scale, or (gradients that are analytically zero,
    such as a bias in front of a batch norm) within 1e-4 of the largest gradient's scale."""
    top = max(float(v.abs().max()) for v in want.values())
    for k in want:
        err = float((got[k] - want[k]).abs().max())
        assert err < 2e-3 * float(want[k].abs().max()) + 1e-4 * top, (what, k, err)


@pytest.mark.parametrize("arch", ["resnet18", "mobilenet_v2", "vgg11_bn"])
def test_schedule_runs_hand_solutions(host, tmp_path, arch):
    from monet_b200 import solver
    rh, ref = host
    torch.manual_seed(0)
    model = getattr(torchvision.models, arch)(num_classes=10).train()
    ref.schedule.disable_dropout(model)
    hw = 32 if arch != "vgg11_bn" else 64
    x = torch.randn(4, 3, hw, hw)
    graph, si = rh.build_solver_info(model, 4, arch, MODE, (3, hw, hw), workdir=tmp_path, profile=False)
    traced = rh.wrap_mobilenet(model)
    want_out, want = _autograd(traced, x)
    for kind in ("store_all", "low_memory"):
        sol = solver.hand_solution(si, kind)
        assert solver.check_solution(si, sol)["violations"] == []
        out, got = _grads_through_schedule(rh, traced, graph, si, sol, x)
        assert torch.allclose(out, want_out, rtol=1e-4, atol=1e-5)
        _close(got, want, kind)


def test_ilp_solution_is_valid_cheaper_and_runs(host, tmp_path):
    from monet_b200 import solver
    rh, ref = host
    torch.manual_seed(0)
    model = torchvision.models.resnet18(num_classes=10).train()
    graph, si = rh.build_solver_info(model, 64, "resnet18", MODE, (3, 64, 64), workdir=tmp_path, profile=False)
    store_all = solver.check_solution(si, solver.hand_solution(si, "store_all"))
    low = solver.check_solution(si, solver.hand_solution(si, "low_memory"))
    assert low["peak_kb"] < store_all["peak_kb"]
    budget = 0.8 * store_all["peak_gb"]
    sol = solver.solve(si, budget, time_limit=240)
    chk = solver.check_solution(si, sol, budget)         # the reference's rows, evaluated literally
    assert chk["violations"] == []
    assert chk["peak_gb"] <= budget
    assert abs(chk["cost"] - sol.runtime_expected) < 1e-6
    assert chk["cost"] <= low["cost"]                     # the optimum beats the hand policy that also fits
    assert sol.r.shape == (len(si.nodes) - si.loss, si.loss + 1) and sol.m.shape[1] == 3
    with pytest.raises(ValueError):                       # cvxpy_solver.py:327-328
        solver.solve(si, 0.3 * store_all["peak_gb"], time_limit=60)
    # pickled the way create_schedule() loads it, then executed
    path = rh.save_solution(si, sol, tmp_path / "solution.pkl")
    si2, sol2 = ref.schedule.load_solution(str(path))
    x = torch.randn(4, 3, 64, 64)
    want_out, want = _autograd(model, x)
    out, got = _grads_through_schedule(rh, model, graph, si2, sol2, x)
    assert torch.allclose(out, want_out, rtol=1e-4, atol=1e-5)
    _close(got, want, "solved")


def test_inplace_table_names_the_overwritten_input(host, tmp_path):
    """aten::add_(a, b): the solver info must say `a` is overwritten (what the executor and the
    operator do), or not offer the choice when `a` is read again later."""
    rh, ref = host
    model = torchvision.models.resnet18(num_classes=10)
    _, si = rh.build_solver_info(model, 2, "resnet18", MODE, (3, 32, 32), workdir=tmp_path, profile=False)
    adds = [v for v in si.inplace_list if si.nodes[v].op == "aten::add_"]
    assert adds
    for v in adds:
        assert si.inplace_list[v] == si.nodes[v].args[0][0]
        assert si.nodes[si.inplace_list[v]].last_used == v


@pytest.mark.parametrize("fname", ["solution_resnet50_184_inplace_conv_multiway_newnode_10.00.pkl",
                                   "solution_resnet50_184_inplace_conv_multiway_newnode_10.00_measured.pkl"])
def test_shipped_schedule_is_valid(host, tmp_path, fname):
    """Each committed 10 GB ResNet-50 schedule still matches the graph this PyTorch traces, and
    satisfies every row of the reference's ILP literally (no budget row above 10 GB)."""
    from monet_b200 import solver
    rh, ref = host
    path = Path(rh.__file__).resolve().parent / "schedules" / fname
    si, sol = ref.schedule.load_solution(str(path))
    chk = solver.check_solution(si, sol, 10.0)
    assert chk["violations"] == [] and chk["peak_gb"] <= 10.0
    graph, fresh = rh.build_solver_info(torchvision.models.resnet50(), 184, "resnet50", MODE, (3, 224, 224),
                                        workdir=tmp_path, profile=False)
    assert len(fresh.nodes) == len(si.nodes) and fresh.loss == si.loss
    assert [n.op for n in fresh.nodes.values()] == [n.op for n in si.nodes.values()]
    assert dict(fresh.inplace_list) == dict(si.inplace_list) and dict(fresh.conv_list) == dict(si.conv_list)
    sched = rh.make_schedule(graph, si, sol)            # init_schedule consumes the uint8 arrays
    assert len(sched._bwd_op) == len(si.nodes) - si.loss
    store_all = solver.check_solution(si, solver.hand_solution(si, "store_all"))
    assert chk["cost"] <= 1.05 * store_all["cost"]
