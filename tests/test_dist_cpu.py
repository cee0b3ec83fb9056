"""World-size-2 gloo checks of the data-parallel paths, on CPU.

* ``monet_b200.dist.GradientBuckets`` driven by ``runner.Runner`` (the arrangement bench.py
  uses): every rank trains its own half of a batch; after the bucketed all-reduce the
  parameter gradients must equal the mean of the two single-rank gradients and replicas stay
  identical after the optimiser step.
* MONeT's own arrangement (examples/dist_training.py:13-29): ``DistributedDataParallel`` around
  the reference's ``MONeTWrapper``-style autograd bridge and ``Schedule``, whose backward hands
  gradients over with ``param.backward(grad)``.

The operators run on the CPU stand-in of ``tests/cpu_functional.py``; no kernels are involved
(they only ever touch local memory), the host logic is what is under test."""
import copy
import os
import socket
import sys
from pathlib import Path

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

sys.path.insert(0, str(Path(__file__).resolve().parent))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


class _Net(torch.nn.Module):
    def __init__(self):
        super().__init__()
        nn = torch.nn
        self.c1 = nn.Conv2d(3, 8, 3, 1, 1, bias=False); self.b1 = nn.BatchNorm2d(8)
        self.r = nn.ReLU(inplace=True)
        self.c2 = nn.Conv2d(8, 8, 3, 1, 1, bias=False); self.b2 = nn.BatchNorm2d(8)
        self.p = nn.AdaptiveAvgPool2d((1, 1))
        self.fc = nn.Linear(8, 5)

    def forward(self, x):
        y = self.r(self.b1(self.c1(x)))
        y = self.r(self.b2(self.c2(y)) + y)
        return self.fc(torch.flatten(self.p(y), 1))


def _data():
    g = torch.Generator().manual_seed(3)
    return torch.randn(8, 3, 12, 12, generator=g), torch.randint(0, 5, (8,), generator=g)


def _worker_buckets(rank, world, port, out):
    import cpu_functional
    from monet_b200 import runner
    from monet_b200.dist import GradientBuckets
    from monet_b200.lm_ops.softmax import SoftmaxCrossEntropy
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    torch.manual_seed(0)
    model = _Net().train()
    x, y = _data()
    xs, ys = x[rank * 4:(rank + 1) * 4], y[rank * 4:(rank + 1) * 4]
    run = runner.Runner(model, runner.store_all)
    buckets = GradientBuckets(list(model.named_parameters()), n_buckets=3)
    buckets.install(run)
    opt = torch.optim.SGD(model.parameters(), lr=0.1)
    ce = SoftmaxCrossEntropy()
    with cpu_functional.patched():
        ce.forward(run.forward(xs), ys)
        run.backward(ce.backward())
    assert buckets.reduced == len(buckets.buckets)
    buckets.wait()
    grads = {k: p.grad.clone() for k, p in model.named_parameters()}
    for k, p in model.named_parameters():        # the gradient IS the bucket view
        assert p.grad.data_ptr() == buckets.views[k].data_ptr()
    opt.step()
    out[rank] = (grads, {k: p.detach().clone() for k, p in model.named_parameters()})
    dist.destroy_process_group()


def test_gradient_buckets_two_ranks():
    from monet_b200.dist import plan_buckets
    assert plan_buckets([10, 10, 10, 10], 2) == [[3, 2], [1, 0]]
    assert plan_buckets([1, 1], 8) == [[1], [0]]
    # the last bucket (nothing left to hide its all-reduce behind) shrinks to the tail fraction
    assert plan_buckets([1, 1, 2, 50, 50, 50, 50], 4, 0.02) == [[6], [5, 4], [3], [2, 1, 0]]
    assert plan_buckets([5, 5], 2, 0.02) == [[1], [0]] and plan_buckets([5], 3, 0.02) == [[0]]
    world, port = 2, _free_port()
    with mp.Manager() as m:
        out = m.dict()
        mp.spawn(_worker_buckets, args=(world, port, out), nprocs=world, join=True)
        (g0, p0), (g1, p1) = out[0], out[1]
    # expected: mean over ranks of each rank's own autograd gradient (batch norm is per rank)
    torch.manual_seed(0)
    model = _Net().train()
    x, y = _data()
    want = {k: torch.zeros_like(p) for k, p in model.named_parameters()}
    for r in range(2):
        m2 = copy.deepcopy(model)
        torch.nn.functional.cross_entropy(m2(x[r * 4:(r + 1) * 4]), y[r * 4:(r + 1) * 4]).backward()
        for k, p in m2.named_parameters():
            want[k] += p.grad / 2
    for k in want:
        assert torch.allclose(g0[k], want[k], rtol=1e-4, atol=1e-6), k
        assert torch.equal(g0[k], g1[k]), k
        assert torch.equal(p0[k], p1[k]), k


def _worker_ddp(rank, world, port, out):
    import cpu_functional
    from monet_b200 import reference_host as rh, solver
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    ref = rh.activate()
    torch.manual_seed(0)
    model = _Net().train()
    x, y = _data()
    xs, ys = x[rank * 4:(rank + 1) * 4], y[rank * 4:(rank + 1) * 4]
    workdir = Path(os.environ["MB_TEST_TMP"]) / f"rank{rank}"
    graph, si = rh.build_solver_info(model, 4, "net", "inplace_conv_multiway_newnode", (3, 12, 12),
                                     workdir=workdir, profile=False)
    sched = rh.make_schedule(graph, si, solver.hand_solution(si, "low_memory"))

    class Wrapped(torch.nn.Module):          # monet_wrapper.py:24-44 without the solution file
        def __init__(self, model, schedule):
            super().__init__()
            self.model, self.schedule = model, [schedule]

        def forward(self, inp):
            inp.requires_grad_(True)
            state = self.state_dict(keep_vars=True)
            return ref.monet_wrapper.MONeTWrapperF.apply(inp, self.schedule[0], list(state.values()))

    ddp = torch.nn.parallel.DistributedDataParallel(Wrapped(model, sched))
    with cpu_functional.patched():
        loss = torch.nn.functional.cross_entropy(ddp(xs), ys)
        loss.backward()
    out[rank] = {k: p.grad.clone() for k, p in model.named_parameters()}
    dist.destroy_process_group()


def test_ddp_over_reference_schedule_two_ranks(tmp_path):
    from baseline import install_ref
    if not install_ref.installed():
        pytest.skip("MONeT host code not installed (python baseline/install_ref.py)")
    world, port = 2, _free_port()
    os.environ["MB_TEST_TMP"] = str(tmp_path)
    with mp.Manager() as m:
        out = m.dict()
        mp.spawn(_worker_ddp, args=(world, port, out), nprocs=world, join=True)
        g0, g1 = out[0], out[1]
    torch.manual_seed(0)
    model = _Net().train()
    x, y = _data()
    want = {k: torch.zeros_like(p) for k, p in model.named_parameters()}
    for r in range(2):
        m2 = copy.deepcopy(model)
        torch.nn.functional.cross_entropy(m2(x[r * 4:(r + 1) * 4]), y[r * 4:(r + 1) * 4]).backward()
        for k, p in m2.named_parameters():
            want[k] += p.grad / 2
    for k in want:
        assert torch.allclose(g0[k], want[k], rtol=1e-4, atol=1e-6), k
        assert torch.equal(g0[k], g1[k]), k
