"""A whole training step captured once as a CUDA graph and replayed with one host call.

MONeT's executor is a Python loop: ``Schedule.backward`` re-enters ``Schedule._forward`` once
per backward node, and each entry walks every node of the graph (schedule.py:145-198,
207-311), about 10^5 interpreter iterations per ResNet-50 step.  With kernels that take
tens of microseconds that loop, not the GPU, sets the step time.  ``CapturedStep`` keeps the
executor's public API untouched -- ``MONeTWrapper(model, solution, shape)``, ``loss.backward()``,
``optimizer.step()`` are called exactly as in examples/training.py -- but calls them once,
under ``torch.cuda.graph``; afterwards a step is ``graph.replay()``.  The schedule (what is
kept, dropped, recomputed, run in place) is frozen into the graph, which is what a solved
schedule is anyway: it does not depend on the data.

Requirements, all met by this operator library: no host synchronisation and no
data-dependent Python control flow inside the step, every buffer from PyTorch's allocator.
"""
from __future__ import annotations

from typing import Callable, Sequence

import torch


class CapturedStep:
    """``step_fn(*inputs) -> tensor`` (e.g. the loss), captured after ``warmup`` eager calls.

    ``__call__(*inputs)`` copies the new inputs into the graph's fixed buffers, replays, and
    returns the output tensor (overwritten by the next call)."""

    def __init__(self, step_fn: Callable[..., torch.Tensor], example_inputs: Sequence[torch.Tensor],
                 warmup: int = 3, thread_local_errors: bool = False):
        if not all(t.is_cuda for t in example_inputs):
            raise RuntimeError("CapturedStep needs CUDA tensors")
        self.step_fn = step_fn
        self.static = [t.detach().clone() for t in example_inputs]
        # warm-up on a side stream: first calls tune, fill caches, create optimiser state and
        # raise shared-memory limits -- none of that may happen during capture
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for _ in range(max(warmup, 1)):
                step_fn(*self.static)
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        self.graph = torch.cuda.CUDAGraph()
        kwargs = {"capture_error_mode": "thread_local"} if thread_local_errors else {}
        with torch.cuda.graph(self.graph, **kwargs):
            self.output = step_fn(*self.static)

    def __call__(self, *inputs: torch.Tensor) -> torch.Tensor:
        with torch.no_grad():          # a module may have marked its input as requiring grad
            for dst, src in zip(self.static, inputs):
                if src is not dst:
                    dst.copy_(src, non_blocking=True)
        self.graph.replay()
        return self.output


def training_step(module: torch.nn.Module, criterion, optimizer) -> Callable[..., torch.Tensor]:
    """The step of examples/training.py as a function: zero the gradients (set to None, so that
    a captured backward allocates them inside the graph's pool), forward, loss, backward,
    optimiser."""
    def step(x, y):
        optimizer.zero_grad(set_to_none=True)
        loss = criterion(module(x), y)
        loss.backward()
        optimizer.step()
        return loss.detach()
    return step
