"""World-size-2 gloo check of the data-parallel arrangement bench.py uses: every rank flattens
its gradients into one bucket, the bucket is all-reduced and averaged, and the parameters see
views of it.  Runs on CPU (no kernels involved: the operators only ever touch local memory)."""
import os
import socket

import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    torch.manual_seed(0)
    params = [torch.nn.Parameter(torch.randn(4, 3)), torch.nn.Parameter(torch.randn(5))]
    flat = torch.zeros(sum(p.numel() for p in params))
    views, off = [], 0
    for p in params:
        views.append(flat[off:off + p.numel()].view(p.shape))
        off += p.numel()
    grads = [torch.full_like(p, float(rank + 1)) for p in params]     # what a backward would hand over
    torch._foreach_copy_(views, grads)
    dist.all_reduce(flat)
    flat.div_(world)
    for p, v in zip(params, views):
        p.grad = v
    torch.optim.SGD(params, lr=0.1).step()
    out[rank] = [p.detach().clone() for p in params] + [flat.clone()]
    dist.destroy_process_group()


def test_gradient_bucket_allreduce_two_ranks():
    world, port = 2, _free_port()
    with mp.Manager() as m:
        out = m.dict()
        mp.spawn(_worker, args=(world, port, out), nprocs=world, join=True)
        r0, r1 = out[0], out[1]
    assert torch.allclose(r0[-1], torch.full_like(r0[-1], 1.5))       # mean of 1 and 2
    for a, b in zip(r0, r1):
        assert torch.equal(a, b)                                       # replicas stay identical
