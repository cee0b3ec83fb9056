"""Data-parallel training over the operators: gradient buckets reduced while the backward runs.

MONeT's only multi-GPU arrangement is data parallelism (examples/dist_training.py:13-29): one
process per GPU, the same schedule on every rank, batch-norm statistics local to a rank, and
one exchange per step -- the mean of the weight gradients -- which ``DistributedDataParallel``
performs from the hooks that fire when ``Schedule.backward`` calls ``param.backward(grad)``
(schedule.py:304-306).  Under the reference's executor that arrangement is used as is
(``DistributedDataParallel(MONeTWrapper(...))``).

``GradientBuckets`` is the same mechanism for ``runner.Runner``: parameters are grouped, in
the order their gradients become ready (last layer first), into a few flat buffers; when the
last gradient of a bucket has been produced the bucket is copied into its flat buffer with
one multi-tensor copy and all-reduced (mean) on a communication stream, so NCCL overlaps the
rest of the backward; ``wait()`` joins the streams before the optimiser.  ``param.grad`` ends
up as a view into the reduced flat buffer, with the parameter's own strides.  Every call is
capturable in a CUDA graph together with the step (NCCL collectives are graph-capturable), so
a replayed step has no eager tail.  No kernel reads another GPU's memory.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence, Tuple

import torch
import torch.distributed as dist


def plan_buckets(sizes: Sequence[int], n_buckets: int, tail_fraction: float = 0.0) -> List[List[int]]:
    """Splits indices 0..len(sizes)-1, taken in REVERSE order, into at most ``n_buckets``
    consecutive groups.  Returns lists of indices, first bucket = the parameters whose
    gradients are ready first.

    With ``tail_fraction`` = 0 the groups have roughly equal total size.  The last group is the
    one nothing can hide: its gradients are complete only when the backward ends, so its
    all-reduce runs while the compute stream waits.  With ``tail_fraction`` > 0 that group is
    cut down to the last parameters holding at most that fraction of all elements (always at
    least one parameter) and the other groups share the rest equally: in a convolutional
    network the first layers have few weights, so the exposed exchange shrinks to a
    latency-bound one."""
    order = list(range(len(sizes) - 1, -1, -1))
    total = float(sum(sizes))
    n_buckets = max(1, min(n_buckets, len(order)))
    tail: List[int] = []
    if tail_fraction > 0.0 and n_buckets >= 2:
        acc = 0.0
        while len(order) > n_buckets - 1 and (not tail or acc + sizes[order[-1]] <= tail_fraction * total):
            acc += sizes[order[-1]]
            tail.insert(0, order.pop())
        n_buckets -= 1
        total -= acc
    target = total / n_buckets
    out: List[List[int]] = [[]]
    acc = 0.0
    for i in order:
        if out[-1] and acc + sizes[i] / 2 > target * len(out) and len(out) < n_buckets:
            out.append([])
        out[-1].append(i)
        acc += sizes[i]
    if tail:
        out.append(tail)
    return out


class GradientBuckets:
    def __init__(self, named_params: Sequence[Tuple[str, torch.Tensor]], n_buckets: int = 4,
                 group=None, overlap: bool = True, tail_fraction: float = 0.02):
        self.params = [(n, p) for n, p in named_params if p.requires_grad]
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.backend = dist.get_backend(group) if dist.is_initialized() else None
        sizes = [p.numel() for _, p in self.params]
        self.buckets = plan_buckets(sizes, n_buckets, tail_fraction)
        self.flat: List[torch.Tensor] = []
        self.views: Dict[str, torch.Tensor] = {}
        self.bucket_of: Dict[str, int] = {}
        for b, idxs in enumerate(self.buckets):
            dev = self.params[idxs[0]][1].device
            flat = torch.zeros(sum(sizes[i] for i in idxs), dtype=torch.float32, device=dev)
            off = 0
            for i in idxs:
                name, p = self.params[i]
                # a view with the parameter's own strides over its slice of the flat buffer
                self.views[name] = flat[off:off + p.numel()].as_strided(p.shape, p.stride()) \
                    if _dense(p) else flat[off:off + p.numel()].view(p.shape)
                self.bucket_of[name] = b
                off += p.numel()
            self.flat.append(flat)
        self._left = [len(idxs) for idxs in self.buckets]
        self._cuda = self.flat[0].is_cuda
        self.overlap = overlap and self._cuda
        self.comm_stream = torch.cuda.Stream() if self.overlap else None
        self._done: List[Optional[torch.cuda.Event]] = [None] * len(self.buckets)
        self.reduced = 0            # buckets reduced since the last wait()

    # ------------------------------------------------------------------ per step
    def install(self, run) -> None:
        """Make ``run`` (a ``runner.Runner``) report finished parameter gradients here."""
        run.on_param_grad = self.ready

    def ready(self, name: str, p: torch.Tensor) -> None:
        b = self.bucket_of.get(name)
        if b is None:
            return
        self._left[b] -= 1
        if self._left[b] == 0:
            self._reduce(b)

    def _reduce(self, b: int) -> None:
        names = [self.params[i][0] for i in self.buckets[b]]
        ps = [self.params[i][1] for i in self.buckets[b]]
        views = [self.views[n] for n in names]
        torch._foreach_copy_(views, [p.grad for p in ps])
        for p, v in zip(ps, views):
            p.grad = v
        flat = self.flat[b]
        if self.world > 1:
            if self.overlap:
                ev = torch.cuda.Event()
                ev.record()
                self.comm_stream.wait_event(ev)
                with torch.cuda.stream(self.comm_stream):
                    self._allreduce_mean(flat)
                    done = torch.cuda.Event()
                    done.record()
                self._done[b] = done
            else:
                self._allreduce_mean(flat)
        self.reduced += 1

    def _allreduce_mean(self, flat: torch.Tensor) -> None:
        if self.backend == "nccl":
            dist.all_reduce(flat, op=dist.ReduceOp.AVG, group=self.group)
        else:
            dist.all_reduce(flat, group=self.group)
            flat.div_(self.world)

    def wait(self) -> None:
        """Call after the backward, before the optimiser: every bucket has been reduced and the
        compute stream has joined the communication stream."""
        for b, left in enumerate(self._left):
            if left != 0:
                if left != len(self.buckets[b]):
                    raise RuntimeError(f"gradient bucket {b} is incomplete: {left} gradients missing")
                raise RuntimeError(f"gradient bucket {b} received no gradients")
        if self.overlap:
            cur = torch.cuda.current_stream()
            for ev in self._done:
                if ev is not None:
                    cur.wait_event(ev)
        self._done = [None] * len(self.buckets)
        self._left = [len(idxs) for idxs in self.buckets]
        self.reduced = 0


def _dense(p: torch.Tensor) -> bool:
    return p.is_contiguous() or (p.dim() == 4 and p.is_contiguous(memory_format=torch.channels_last))


def init_from_env(device: Optional[torch.device] = None):
    """``init_process_group`` from torchrun's environment (env://, as dist_training.py:13-18):
    NCCL on a CUDA device, gloo otherwise.  Returns (rank, world_size)."""
    import os
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    if world > 1 and not dist.is_initialized():
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        if device is not None and device.type == "cuda":
            dist.init_process_group("nccl", device_id=device)
        else:
            dist.init_process_group("gloo")
    return rank, world
