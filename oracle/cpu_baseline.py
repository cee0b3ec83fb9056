"""CPU baseline for the benchmark.  TEST / MEASUREMENT INFRASTRUCTURE ONLY.

The reference has no CPU implementation of its low-memory operators (their CPU branches
return zeros or exit: lrrelu.cpp:16-19, pack.cpp:49-51, lrhardtanh.cpp:12-14), so "the
reference's CPU path" is what its operators are defined against: PyTorch CPU eager running
the same model, loss and optimiser.  Only bench.py (cpu_baseline leg and --impl reference)
may call this.
"""
from __future__ import annotations

import os
import time

import torch
import torchvision


def host_cores() -> int:
    try:
        return len(os.sched_getaffinity(0))
    except AttributeError:
        return os.cpu_count() or 1


def resnet50_train_steps(batch: int, steps: int, warmup: int = 1, threads: int | None = None,
                         seed: int = 0):
    """Times `steps` eager training steps (forward, cross-entropy, backward, SGD with momentum)
    of torchvision ResNet-50 on synthetic N(0,1) images; returns (images/s, ms/step, threads)."""
    threads = threads or host_cores()
    torch.set_num_threads(threads)
    torch.manual_seed(seed)
    model = torchvision.models.resnet50().train()
    opt = torch.optim.SGD(model.parameters(), lr=0.1, momentum=0.9)
    x = torch.randn(batch, 3, 224, 224)
    y = torch.randint(0, 1000, (batch,))
    times = []
    for i in range(warmup + steps):
        t0 = time.perf_counter()
        opt.zero_grad(set_to_none=True)
        loss = torch.nn.functional.cross_entropy(model(x), y)
        loss.backward()
        opt.step()
        float(loss)
        if i >= warmup:
            times.append(time.perf_counter() - t0)
    sec = sum(times) / len(times)
    return batch / sec, sec * 1e3, threads
