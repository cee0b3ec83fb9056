#!/usr/bin/env python
"""Benchmark: ResNet-50 (torchvision v1.5 layout) training step, batch 184 per GPU, fp32
semantics (TF32 tensor-core convolutions), synthetic N(0,1) images and uniform labels,
cross-entropy + SGD(lr 0.1, momentum 0.9), run entirely through the low-memory operators.

  python bench.py [--gpus N] [--steps K] [--warmup W] [--schedule budget_10gb|low_memory|store_all]
  python bench.py --impl reference ...      # PyTorch CPU eager on the host cores

One JSON line on stdout (rank 0).  `value` = images/s with the batch already resident in
HBM; `e2e` = the same step fed from pinned host memory each step, loss read back each step.
Under torchrun every rank trains its own batch (weak scaling) and weight gradients are
all-reduced over NCCL.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

METRIC = "resnet50_bs184_train_images_per_s"
WORKLOAD = "ResNet-50 v1.5, batch 184 per GPU, 3x224x224 fp32, CE + SGD momentum (BASELINE configs[1])"


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--model", default="resnet50", choices=["resnet50", "mobilenet_v2", "unet", "vgg16_bn"],
                    help="BASELINE configs[1..4]; batch, input and schedule default to the config's")
    ap.add_argument("--schedule", default=None, choices=["low_memory", "store_all", "budget_10gb"])
    ap.add_argument("--buckets", type=int, default=4, help="gradient buckets of the data-parallel all-reduce")
    ap.add_argument("--no-comparators", action="store_true",
                    help="skip the unfused-graph and stock-PyTorch-on-this-GPU runs (N = 1 only)")
    ap.add_argument("--no-fuse", action="store_true",
                    help="run batch norm, residual add and ReLU as separate operators, as the "
                         "reference's graph does")
    ap.add_argument("--no-channel-sums", action="store_true",
                    help="batch norms make their own statistics pass instead of taking the sums "
                         "the preceding convolution's statistics warps leave")
    ap.add_argument("--no-cuda-graph", action="store_true",
                    help="time the Python executor's eager launches only (the default also captures "
                         "the step as a CUDA graph and reports the replayed step as `value`)")
    ap.add_argument("--batch", type=int, default=None, help="per-GPU batch (default: the config's)")
    ap.add_argument("--cpu-batch", type=int, default=None,
                    help="images per step of the CPU arm (default: the full batch; an override is echoed in config)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--micro", default=None, choices=sorted(MICRO),
                    help="time ONE operator on one ResNet-50 layer's tensors (for ncu captures)")
    ap.add_argument("--micro-batch", type=int, default=184)
    ap.add_argument("--cudnn", action="store_true",
                    help="with --micro on a convolution pass: also time cuDNN (TF32, benchmark mode) on the same tensors")
    ap.add_argument("--conv-counters", action="store_true",
                    help="with --micro on a stride-1 multi-tap fprop/dgrad: one extra launch with the kernel's own "
                         "cycle counters (CTA 0) switched on, added to the line as `cta0_cycles`")
    return ap.parse_args()


# ------------------------------------------------------------------------ micro cases
# name -> (kind, C, H, K, R, stride, pad): one operator on one layer of the workload
MICRO = {
    "fprop3x3_c64": ("fprop", 64, 56, 64, 3, 1, 1), "dgrad3x3_c64": ("dgrad", 64, 56, 64, 3, 1, 1),
    "wgrad3x3_c64": ("wgrad", 64, 56, 64, 3, 1, 1), "wgrad3x3_c128": ("wgrad", 128, 28, 128, 3, 1, 1),
    "fprop3x3_c128": ("fprop", 128, 28, 128, 3, 1, 1), "dgrad3x3_c128": ("dgrad", 128, 28, 128, 3, 1, 1),
    "fprop3x3_c256": ("fprop", 256, 14, 256, 3, 1, 1), "wgrad3x3_c256": ("wgrad", 256, 14, 256, 3, 1, 1),
    "fprop1x1_c64_k256": ("fprop", 64, 56, 256, 1, 1, 0), "dgrad1x1_c64_k256": ("dgrad", 64, 56, 256, 1, 1, 0),
    "wgrad1x1_c64_k256": ("wgrad", 64, 56, 256, 1, 1, 0), "fprop1x1_c1024_k256": ("fprop", 1024, 14, 256, 1, 1, 0),
    "fprop1x1_c256_k64_sums": ("fprop_sums", 256, 56, 64, 1, 1, 0), "fprop1x1_c64_k256_sums": ("fprop_sums", 64, 56, 256, 1, 1, 0),
    "fprop3x3_c512": ("fprop", 512, 7, 512, 3, 1, 1),
    "fprop3x3s2_c128": ("fprop", 128, 56, 128, 3, 2, 1), "wgrad3x3s2_c128": ("wgrad", 128, 56, 128, 3, 2, 1),
    "stem_fprop": ("fprop", 3, 224, 64, 7, 2, 3), "stem_wgrad": ("wgrad", 3, 224, 64, 7, 2, 3),
    "bn_fwd": ("bn_fwd", 256, 56, 0, 0, 0, 0), "bn_bwd": ("bn_bwd", 256, 56, 0, 0, 0, 0),
    "relu_fwd": ("relu_fwd", 256, 56, 0, 0, 0, 0), "relu_fwd_mask": ("relu_fwd_mask", 256, 56, 0, 0, 0, 0),
    "relu_bwd": ("relu_bwd", 256, 56, 0, 0, 0, 0), "add": ("add", 256, 56, 0, 0, 0, 0),
    "bn_relu_fwd": ("bn_relu_fwd", 256, 56, 0, 0, 0, 0), "bn_add_relu_fwd": ("bn_add_relu_fwd", 256, 56, 0, 0, 0, 0),
    "bn_relu_bwd": ("bn_relu_bwd", 256, 56, 0, 0, 0, 0), "relu_bwd2": ("relu_bwd2", 256, 56, 0, 0, 0, 0),
    "bn_add_relu_bwd": ("bn_add_relu_bwd", 256, 56, 0, 0, 0, 0),
    "maxpool_fwd": ("maxpool_fwd", 64, 112, 0, 0, 0, 0), "maxpool_bwd": ("maxpool_bwd", 64, 112, 0, 0, 0, 0),
    "relu_bwd_mask": ("relu_bwd_mask", 256, 56, 0, 0, 0, 0),
    # not ResNet-50 layers: a MobileNetV2 depthwise layer (use --micro-batch 272), UNet's skip
    # concatenation (--micro-batch 11), VGG-16's first classifier layer (--micro-batch 176), and the
    # fused softmax + cross-entropy on 65 536 rows of 1000 classes (ResNet's own 184 rows are 0.7 MB)
    "dw3x3_fprop": ("dw_fprop", 144, 56, 144, 3, 1, 1), "dw3x3_dgrad": ("dw_dgrad", 144, 56, 144, 3, 1, 1),
    "dw3x3_wgrad": ("dw_wgrad", 144, 56, 144, 3, 1, 1),
    "dw3x3s2_fprop": ("dw_fprop", 96, 112, 96, 3, 2, 1), "dw3x3s2_dgrad": ("dw_dgrad", 96, 112, 96, 3, 2, 1),
    # VGG-16's 512-channel 28x28 layer (--micro-batch 176): backward-filter by filter row
    "wgrad3x3_c512_28": ("wgrad", 512, 28, 512, 3, 1, 1),
    "cat_bwd": ("cat_bwd", 128, 208, 0, 0, 0, 0), "cat_fwd": ("cat_fwd", 128, 208, 0, 0, 0, 0),
    "fc_fwd": ("fc_fwd", 25088, 1, 4096, 1, 1, 0), "fc_dgrad": ("fc_dgrad", 25088, 1, 4096, 1, 1, 0),
    "fc_wgrad": ("fc_wgrad", 25088, 1, 4096, 1, 1, 0),
    "softmax_ce": ("softmax_ce", 1000, 1, 0, 0, 0, 0),
}


def run_micro(args):
    """One operator, `--steps` timed calls after `--warmup`, CUDA events; one JSON line."""
    import torch
    from monet_b200 import functional as F
    kind, Cc, H, K, R, s, p = MICRO[args.micro]
    dev = torch.device("cuda", 0)
    N = args.micro_batch
    torch.manual_seed(0)
    cl = torch.channels_last
    if kind == "softmax_ce":
        rows = 65536
        logits = torch.randn(rows, Cc, device=dev)
        labels = torch.randint(0, Cc, (rows,), device=dev)
        flops, nbytes = 0.0, 8.0 * rows * Cc + 12.0 * rows
        fn = lambda: F.cross_entropy_fwd_bwd(logits, labels, 1.0 / rows)      # noqa: E731
    elif kind.startswith("fc_"):
        xf = torch.randn(N, Cc, device=dev)
        wf = torch.randn(K, Cc, device=dev) * Cc ** -0.5
        bf = torch.randn(K, device=dev)
        dyf = torch.randn(N, K, device=dev)
        flops, nbytes = 2.0 * N * Cc * K, 4.0 * (N * Cc + K * Cc + N * K)
        fn = {"fc_fwd": lambda: F.linear_fwd(xf, wf, bf), "fc_dgrad": lambda: F.linear_dgrad(dyf, wf),
              "fc_wgrad": lambda: F.linear_wgrad(xf, dyf, True)}[kind]
    elif kind.startswith("cat_"):
        W = H * 304 // 208
        parts = [torch.randn(N, Cc // 2, H, W, device=dev).contiguous(memory_format=cl) for _ in range(2)]
        whole = F.cat(parts, 1)
        flops, nbytes = 0.0, 8.0 * whole.numel()
        fn = (lambda: F.cat(parts, 1)) if kind == "cat_fwd" else (lambda: F.cat_bwd(whole, [Cc // 2, Cc // 2], 1))
    elif kind.startswith("dw_"):
        xd = torch.randn(N, Cc, H, H, device=dev).contiguous(memory_format=cl)
        wd = torch.randn(Cc, 1, R, R, device=dev) * 0.2
        yd = F.depthwise_fprop(xd, wd, None, s, p, 1, Cc)
        dyd = torch.randn_like(yd)
        flops, nbytes = 0.0, 4.0 * (xd.numel() + yd.numel())
        fn = {"dw_fprop": lambda: F.depthwise_fprop(xd, wd, None, s, p, 1, Cc),
              "dw_dgrad": lambda: F.depthwise_bwd(dyd, xd, wd, s, p, 1, Cc, need=(True, False, False)),
              "dw_wgrad": lambda: F.depthwise_bwd(dyd, xd, wd, s, p, 1, Cc, need=(False, True, False))}[kind]
    else:
        x = torch.randn(N, Cc, H, H, device=dev)
        x = x.contiguous(memory_format=cl) if Cc % 4 == 0 else x
    if kind in ("softmax_ce",) or kind.startswith(("fc_", "cat_", "dw_")):
        pass
    elif kind in ("fprop", "dgrad", "wgrad", "fprop_sums"):
        w = (torch.randn(K, Cc, R, R, device=dev) * 0.05).contiguous(memory_format=cl)
        y = F.conv2d_fprop(x, w, None, s, p, 1)
        dy = torch.randn_like(y)
        nbytes = 4.0 * (x.numel() + w.numel() + y.numel())
        flops = 2.0 * y.numel() * Cc * R * R
        shift = torch.zeros(K, device=dev)
        fn = {"fprop": lambda: F.conv2d_fprop(x, w, None, s, p, 1),
              "fprop_sums": lambda: F.conv2d_fprop(x, w, None, s, p, 1, 1, 0, stats_shift=shift, want_stats=True),
              "dgrad": lambda: F.conv2d_dgrad(dy, w, x.shape, s, p, 1),
              "wgrad": lambda: F.conv2d_wgrad(x, dy, w.shape, s, p, 1)}[kind]
    else:
        flops = 0.0
        E = float(x.numel())
        g, b = torch.ones(Cc, device=dev), torch.zeros(Cc, device=dev)
        dy = torch.randn_like(x)
        if kind == "bn_fwd":
            nbytes, fn = 12 * E, lambda: F.bn_fwd_train(x, g, b, None, None, 0.1, 1e-5)
        elif kind == "bn_bwd":
            yb, _, iv = F.bn_fwd_train(x, g, b, None, None, 0.1, 1e-5)
            nbytes, fn = 20 * E, lambda: F.bn_bwd_from_output(dy, yb, g, b, iv)
        elif kind == "bn_relu_fwd":
            nbytes, fn = 12 * E, lambda: F.bn_act_fwd_train(x, None, True, g, b, None, None, 0.1, 1e-5)
        elif kind == "bn_add_relu_fwd":
            nbytes, fn = 16 * E, lambda: F.bn_act_fwd_train(x, dy, True, g, b, None, None, 0.1, 1e-5)
        elif kind == "bn_relu_bwd":
            _, mu, iv = F.bn_fwd_train(x, g, b, None, None, 0.1, 1e-5)
            nbytes, fn = 20 * E, lambda: F.bn_relu_bwd_from_input(dy, x, g, b, mu, iv)
        elif kind == "bn_add_relu_bwd":
            yb, mu, iv = F.bn_act_fwd_train(x, dy, True, g, b, None, None, 0.1, 1e-5)
            dy2 = torch.randn_like(x)
            nbytes, fn = 32 * E, lambda: F.bn_add_relu_bwd(dy, dy2, yb, x, g, mu, iv)
        elif kind == "relu_bwd2":
            dy2 = torch.randn_like(x)
            nbytes, fn = 16 * E, lambda: F.relu_bwd_act2(dy, dy2, x)
        elif kind == "relu_fwd":
            nbytes, fn = 8 * E, lambda: F.relu(x)
        elif kind == "relu_fwd_mask":
            nbytes, fn = 8.125 * E, lambda: F.relu_mask(x)
        elif kind == "relu_bwd":
            nbytes, fn = 12 * E, lambda: F.relu_bwd_act(dy, x, 0.0, inplace=False)
        elif kind == "relu_bwd_mask":
            _, rmask = F.relu_mask(x)
            nbytes, fn = 8.125 * E, lambda: F.relu_bwd_mask(dy, rmask, inplace=False)
        elif kind == "add":
            nbytes, fn = 12 * E, lambda: F.add(x, dy, 1.0)
        elif kind == "maxpool_fwd":
            yp, _, _ = F.maxpool2d(x, 3, 2, 1, 1, False)
            nbytes, fn = 4 * E + 4.5 * yp.numel(), lambda: F.maxpool2d(x, 3, 2, 1, 1, False)
        else:
            yp, nib, d = F.maxpool2d(x, 3, 2, 1, 1, False)
            dyp = torch.randn_like(yp)
            nbytes, fn = 4 * E + 4.5 * yp.numel(), lambda: F.maxpool2d_bwd(dyp, nib, d)
    def clock(f):
        for _ in range(max(args.warmup, 1)):
            f()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(args.steps):
            f()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / args.steps

    ms = clock(fn)
    line = {"micro": args.micro, "batch": N, "ms": ms, "algorithmic_GBps": nbytes / ms / 1e6,
            "TFLOPps": flops / ms / 1e9, "conv_status": F.conv_device_status()}
    if args.conv_counters and kind in ("fprop", "dgrad"):
        import ctypes
        from monet_b200 import _lib
        buf = torch.zeros(16, dtype=torch.int64, device=dev)
        _lib.lib().mb_conv_debug_counters(ctypes.c_void_p(buf.data_ptr()))
        fn()
        torch.cuda.synchronize()
        _lib.lib().mb_conv_debug_counters(ctypes.c_void_p(0))
        names = ["mma_thread_total", "mma_wait_input_tile", "mma_wait_filter_tile", "mma_wait_free_accumulator",
                 "producer_wait_input_slot", "producer_wait_filter_slot", "epilogue_wait_result", "epilogue_busy", "work_items"]
        line["cta0_cycles"] = dict(zip(names, buf.tolist()[:9]))
    if args.cudnn and kind in ("fprop", "dgrad", "wgrad"):
        # the library op this pass replaces, on the same tensors: cuDNN, TF32, benchmark mode
        torch.backends.cudnn.allow_tf32 = True
        torch.backends.cudnn.benchmark = True
        xc = x.contiguous(memory_format=cl)
        mask = {"dgrad": [True, False, False], "wgrad": [False, True, False]}.get(kind)
        lib_fn = ((lambda: torch.nn.functional.conv2d(xc, w, None, s, p)) if kind == "fprop" else
                  (lambda: torch.ops.aten.convolution_backward(dy, xc, w, None, [s, s], [p, p], [1, 1], False,
                                                                [0, 0], 1, mask)))
        line["cudnn_ms"] = clock(lib_fn)
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------ reference arm (CPU)
def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from oracle import cpu_baseline
    steps = max(1, min(args.steps, 4))
    batch = args.cpu_batch or args.batch or 184
    ips, ms, threads = cpu_baseline.resnet50_train_steps(batch, steps, warmup=1)
    sample = f"{steps} eager steps of batch {batch} (of 184) on {threads} host threads"
    cfg = {"workload": WORKLOAD, "sample": sample}
    if batch != 184:
        cfg["cpu_batch_override"] = batch
    line = {
        "impl": "reference", "metric": METRIC, "value": ips, "unit": "images/s", "n_gpus": args.gpus,
        "steps": steps, "warmup": 1, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": cfg,
        "cpu_baseline": {"value": ips, "unit": "images/s", "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": ips, "unit": "images/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------- clocks
class ClockSampler:
    """Samples SM clock and throttle reasons with nvidia-smi while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.rows, self.proc = index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "200",
                 "-i", str(self.index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()
        sm, smax, reasons = [], 0.0, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            try:
                sm.append(float(r[1])); smax = max(smax, float(r[2]))
            except (ValueError, IndexError):
                continue
            for name, v in zip(names, r[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": smax or None,
                "reasons": sorted(reasons), "samples": len(sm)}


# ----------------------------------------------------------- algorithmic bytes / flops
def family_costs(runner_obj, batch_shape):
    """Per entry-point family: algorithmic HBM bytes and flops of ONE training step, from the
    graph and the recorded shapes (fp32: 4 bytes per element).

    conv pass: activations in + filter + activations out, 2*N*P*Q*K*C*R*S flops.
    bn train fwd 12 B/el (16 with a residual operand), bn cached-stat fwd 8, bn bwd 20 (also
    when it gates by the recomputed ReLU), relu fwd 8 (+1/8 with mask), relu bwd from a saved
    activation 12 (16 when it also sums two gradients), bn+add+relu bwd 32 (28 with one
    gradient), add 12, batch norm fed with its producer's channel sums 8 (12 with a residual), max-pool 4*E_in + 4.5*E_out
    each way."""
    import numpy as np
    cost = {}

    def add(fam, b, f=0.0):
        c = cost.setdefault(fam, [0.0, 0.0, []])
        c[0] += b; c[1] += f
        c[2].append((b, f))          # per call, for the sum of per-layer floors

    shapes = runner_obj.shapes
    needed = getattr(runner_obj, "_need", {})     # node id -> backward step that reads its output

    def recomputed(n, ch):
        """A node marked recompute is rebuilt only when some backward step reads its output."""
        return ch.recompute and n.id in needed

    emitters = {n.sums_from for n in runner_obj.nodes if getattr(n, "sums_from", -1) >= 0}

    def emits_sums(n):
        """True when this convolution's statistics warps leave the sums for its batch norm."""
        if n.id not in emitters:
            return False
        w = runner_obj._tensors[n.args[1].value]
        stride = n.args[3].value
        multi_tap_s1 = w.shape[2] * w.shape[3] > 1 and stride[0] == 1 and stride[1] == 1
        return w.shape[0] % 32 == 0 and w.shape[1] > 4 and not multi_tap_s1

    for n in runner_obj.nodes:
        out = shapes[n.id]
        e_out = float(np.prod(out))
        a0 = n.args[0]
        in_shape = shapes[a0.value] if a0.kind == 'node' else (batch_shape if a0.kind == 'input' else None)
        e_in = float(np.prod(in_shape)) if in_shape is not None else 0.0
        ch = runner_obj.choices[n.id]
        if n.op == 'aten::_convolution':
            w = runner_obj._tensors[n.args[1].value]
            e_w = float(w.numel())
            byts = 4 * (e_in + e_w + e_out)
            if n.args[8].value > 1:                     # depthwise: bandwidth kernels, no tensor cores
                add("mb_depthwise_fprop", byts)
                add("mb_depthwise_wgrad", byts)
                add("mb_depthwise_dgrad", byts)
                continue
            if n.args[6].value:                         # transposed: forward = dgrad kernel, backward-data = fprop kernel
                fl = 2.0 * e_in * w.shape[1] * w.shape[2] * w.shape[3]
                add("mb_conv2d_dgrad", byts, fl)
                add("mb_conv2d_fprop", byts, fl)
                add("mb_conv2d_wgrad", byts, fl)
                continue
            fl = 2.0 * e_out * w.shape[1] * w.shape[2] * w.shape[3]
            add("mb_conv2d_fprop_bnstats" if emits_sums(n) else "mb_conv2d_fprop", byts, fl)
            add("mb_conv2d_wgrad", byts, fl)
            if a0.kind == 'node':
                add("mb_conv2d_dgrad", byts, fl)
        elif n.op == 'aten::batch_norm':
            src = runner_obj.nodes[n.sums_from] if getattr(n, "sums_from", -1) >= 0 else None
            if src is not None and emits_sums(src):
                add("mb_bn_act_fwd_train_partials", 8 * e_out)
            else:
                add("mb_bn_fwd_train", 12 * e_out)
            add("mb_bn_bwd_from_output" if ch.impl == 1 else "mb_bn_bwd_from_input", 20 * e_out)
        elif n.op in ('monet::batch_norm_relu', 'monet::batch_norm_relu6'):
            src = runner_obj.nodes[n.sums_from] if n.sums_from >= 0 else None
            if src is not None and emits_sums(src):
                add("mb_bn_act_fwd_train_partials", 8 * e_out)
            else:
                add("mb_bn_act_fwd_train", 12 * e_out)
            if recomputed(n, ch):
                add("mb_bn_act_fwd_apply", 8 * e_out)
            add("mb_bn_act_bwd_from_input", 20 * e_out)
        elif n.op == 'monet::batch_norm_add_relu':
            src = runner_obj.nodes[n.sums_from] if n.sums_from >= 0 else None
            if src is not None and emits_sums(src):
                add("mb_bn_act_fwd_train_partials", 12 * e_out)
            else:
                add("mb_bn_act_fwd_train", 16 * e_out)
            if recomputed(n, ch):
                add("mb_bn_act_fwd_apply", 12 * e_out)
            add("mb_bn_add_relu_bwd", (32 if len(n.users) == 2 else 28) * e_out)
        elif n.op in ('aten::relu', 'aten::relu_'):
            add("mb_relu_fwd", 8 * e_out * (2 if recomputed(n, ch) else 1))
            add("mb_relu_bwd_act", 12 * e_out)
        elif n.op in ('aten::add', 'aten::add_'):
            add("mb_add_fwd", 12 * e_out)
        elif n.op in ('aten::hardtanh', 'aten::hardtanh_'):
            add("mb_hardtanh_fwd", 8 * e_out * (2 if recomputed(n, ch) else 1))
            add("mb_hardtanh_bwd", 12 * e_out)
        elif n.op == 'aten::cat':
            add("mb_cat_rows", 16 * e_out)              # forward and backward: read + write each
        elif n.op == 'aten::max_pool2d':
            add("mb_maxpool2d_fwd", 4 * e_in + 4.5 * e_out)
            add("mb_maxpool2d_bwd", 4 * e_in + 4.5 * e_out)
    return cost


# DRAM traffic measured by ncu on one layer per kernel family, as a fraction of that layer's
# algorithmic bytes (profiles/conv_bn_pointwise_kernels_ncu_full.md).  A whole step is too large to
# capture under ncu, and every one of these kernels streams its operands once, so the traffic
# of a step's launches is taken to grow in proportion to their algorithmic bytes.
TRAFFIC_RATIO = {
    "mb_conv2d_fprop": 679.8 / 738.7, "mb_conv2d_fprop_bnstats": 679.8 / 738.7, "mb_conv2d_dgrad": 719.8 / 738.7, "mb_conv2d_wgrad": 742.9 / 738.7,
    "mb_bn_bwd_from_output": 1740.8 / 1772.0, "mb_bn_bwd_from_input": 1740.8 / 1772.0,
    "mb_bn_act_bwd_from_input": (1188.5 + 1743.9) / (1182.0 + 1772.0),
    "mb_bn_act_fwd_train_partials": 1136.9 / 1182.0,
    "mb_bn_add_relu_bwd": (2903.3 + 1743.9) / (2954.0 + 1772.0),
    "mb_bn_fwd_train": 594.7 / 591.0, "mb_bn_act_fwd_train": (594.7 + 1136.9) / (591.0 + 1182.0),
    "mb_relu_fwd": 1136.5 / 1182.0, "mb_relu_bwd_act": 1744.0 / 1772.0, "mb_relu_bwd_act2": 2333.9 / 2363.0,
    "mb_add_fwd": 1743.8 / 1772.0, "mb_maxpool2d_bwd": 710.5 / 756.0,
}


# -------------------------------------------------------------------------- workloads
def _unet(n_classes=2, base=64):
    """UNet of BASELINE configs[3]: 4 down / 4 up levels, double 3x3 conv + BN + ReLU per level,
    2x2 max-pool down, 2x2 stride-2 transposed convolution up, skip concatenation."""
    import torch
    nn = torch.nn

    def double(cin, cout):
        return nn.Sequential(nn.Conv2d(cin, cout, 3, padding=1, bias=False), nn.BatchNorm2d(cout), nn.ReLU(inplace=True),
                             nn.Conv2d(cout, cout, 3, padding=1, bias=False), nn.BatchNorm2d(cout), nn.ReLU(inplace=True))

    class UNet(nn.Module):
        def __init__(self):
            super().__init__()
            c = [base, base * 2, base * 4, base * 8, base * 16]
            self.inc = double(3, c[0])
            self.pool1 = nn.MaxPool2d(2); self.down1 = double(c[0], c[1])
            self.pool2 = nn.MaxPool2d(2); self.down2 = double(c[1], c[2])
            self.pool3 = nn.MaxPool2d(2); self.down3 = double(c[2], c[3])
            self.pool4 = nn.MaxPool2d(2); self.down4 = double(c[3], c[4])
            self.up1 = nn.ConvTranspose2d(c[4], c[3], 2, stride=2); self.conv1 = double(c[4], c[3])
            self.up2 = nn.ConvTranspose2d(c[3], c[2], 2, stride=2); self.conv2 = double(c[3], c[2])
            self.up3 = nn.ConvTranspose2d(c[2], c[1], 2, stride=2); self.conv3 = double(c[2], c[1])
            self.up4 = nn.ConvTranspose2d(c[1], c[0], 2, stride=2); self.conv4 = double(c[1], c[0])
            self.outc = nn.Conv2d(c[0], n_classes, 1)

        def forward(self, x):
            x1 = self.inc(x)
            x2 = self.down1(self.pool1(x1))
            x3 = self.down2(self.pool2(x2))
            x4 = self.down3(self.pool3(x3))
            x5 = self.down4(self.pool4(x4))
            y = self.conv1(torch.cat([x4, self.up1(x5)], 1))
            y = self.conv2(torch.cat([x3, self.up2(y)], 1))
            y = self.conv3(torch.cat([x2, self.up3(y)], 1))
            y = self.conv4(torch.cat([x1, self.up4(y)], 1))
            return self.outc(y)

    return UNet()


# name -> (constructor, batch, input shape, classes, default schedule, description)
def workloads():
    import torchvision
    return {
        "resnet50": (torchvision.models.resnet50, 184, (3, 224, 224), 1000, "budget_10gb",
                     "ResNet-50 v1.5, batch 184 per GPU, 3x224x224 fp32, CE + SGD momentum (BASELINE configs[1])"),
        "mobilenet_v2": (torchvision.models.mobilenet_v2, 272, (3, 224, 224), 1000, "low_memory",
                         "MobileNetV2 1.0, batch 272 per GPU, 3x224x224 fp32, CE + SGD momentum (BASELINE configs[2])"),
        "unet": (_unet, 11, (3, 416, 608), 2, "low_memory",
                 "UNet 4+4 levels base 64, transposed-conv up, batch 11 per GPU, 3x416x608 fp32, per-pixel 2-class CE + SGD momentum (BASELINE configs[3])"),
        "vgg16_bn": (torchvision.models.vgg16_bn, 176, (3, 224, 224), 1000, "low_memory",
                     "VGG-16-BN, batch 176 per GPU, 3x224x224 fp32, CE + SGD momentum (BASELINE configs[4])"),
    }


def measure_tf32_peak(dev, seconds=0.6):
    """Sustained dense TF32 rate of this GPU right now: cuBLAS 8192^3 fp32 matmul with TF32
    allowed, repeated for about `seconds`, CUDA events.  The denominator of the convolutions'
    tensor-pipe fraction (no TF32 figure is in MEASURED_PEAKS.json)."""
    import torch
    old = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = True
    try:
        n = 8192
        a = torch.randn(n, n, device=dev)
        b = torch.randn(n, n, device=dev)
        c = torch.empty(n, n, device=dev)
        for _ in range(3):
            torch.matmul(a, b, out=c)
        torch.cuda.synchronize()
        flop = 2.0 * n ** 3
        reps, best = 20, 0.0
        t_end = time.perf_counter() + seconds
        while True:
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(reps):
                torch.matmul(a, b, out=c)
            e1.record()
            torch.cuda.synchronize()
            best = flop * reps / (e0.elapsed_time(e1) * 1e-3) / 1e12     # last window = sustained
            if time.perf_counter() > t_end:
                break
        return best
    finally:
        torch.backends.cuda.matmul.allow_tf32 = old


def torch_gpu_baseline(make_model, x, y, steps, warmup, pixelwise):
    """Stock PyTorch on the same GPU: eager, channels_last, cuDNN TF32 + benchmark mode, same
    batch, CE + SGD momentum -- what the reference compares itself with
    (examples/check_runtime_original.py:32-56).  Returns (ms per step, peak bytes)."""
    import torch
    old = (torch.backends.cudnn.allow_tf32, torch.backends.cudnn.benchmark, torch.backends.cuda.matmul.allow_tf32)
    torch.backends.cudnn.allow_tf32 = True
    torch.backends.cudnn.benchmark = True
    torch.backends.cuda.matmul.allow_tf32 = True
    try:
        torch.manual_seed(0)
        model = make_model().to(x.device).train().to(memory_format=torch.channels_last)
        opt = torch.optim.SGD(model.parameters(), lr=0.1, momentum=0.9)
        xc = x.contiguous(memory_format=torch.channels_last)
        crit = torch.nn.CrossEntropyLoss()

        def step():
            opt.zero_grad(set_to_none=True)
            loss = crit(model(xc), y)
            loss.backward()
            opt.step()
            return loss

        for _ in range(max(warmup, 3)):
            step()
        torch.cuda.synchronize()
        torch.cuda.reset_peak_memory_stats()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            step()
        e1.record()
        torch.cuda.synchronize()
        ms, peak = e0.elapsed_time(e1) / steps, torch.cuda.max_memory_allocated()
        del model, opt
        torch.cuda.empty_cache()
        return ms, peak
    finally:
        torch.backends.cudnn.allow_tf32, torch.backends.cudnn.benchmark, torch.backends.cuda.matmul.allow_tf32 = old


_SCHEDULES = ROOT / "monet_b200" / "schedules"
SOLVED_10GB = _SCHEDULES / "solution_resnet50_184_inplace_conv_multiway_newnode_10.00_measured.pkl"
if not SOLVED_10GB.exists():        # solved on the bytes-and-flops cost model instead of measured kernel times
    SOLVED_10GB = _SCHEDULES / "solution_resnet50_184_inplace_conv_multiway_newnode_10.00.pkl"


def reference_executor_block(model, params, x, y, B, in_shape, args, timed):
    """The drop-in measured: MONeT's own MONeTWrapper / Schedule (installed under baseline/_ref)
    executing its own solver's solution over these kernels, eagerly and as one captured CUDA
    graph.  Uses the committed 10 GB ILP solution when batch and model match it, else a
    hand-made low-memory solution."""
    import tempfile

    import torch
    try:
        from monet_b200 import graphed, reference_host as rh, solver
        ref = rh.activate()
        with tempfile.TemporaryDirectory() as tmp:
            if SOLVED_10GB.exists() and B == 184:
                sol_file, what = str(SOLVED_10GB), "ILP solution, 10 GB budget (scipy/HiGHS), " + SOLVED_10GB.name
            else:
                graph, si = rh.build_solver_info(model, B, "resnet50", "inplace_conv_multiway_newnode",
                                                 tuple(in_shape), workdir=tmp, profile=False)
                sol_file = str(rh.save_solution(si, solver.hand_solution(si, "low_memory"), tmp + "/solution.pkl"))
                what = "hand-made low-memory solution"
            wrapped = ref.monet_wrapper.MONeTWrapper(model, sol_file, tuple(in_shape))
            opt = torch.optim.SGD(params, lr=0.1, momentum=0.9)
            step = graphed.training_step(wrapped, torch.nn.CrossEntropyLoss(), opt)
            xs = x.clone()
            for _ in range(2):
                step(xs, y)
            torch.cuda.synchronize()
            torch.cuda.reset_peak_memory_stats()
            n = max(2, min(args.steps, 5))
            ms_eager, _ = timed(lambda: step(xs, y), n)
            peak = torch.cuda.max_memory_allocated()
            out = {"solution": what, "eager_ms_per_step": ms_eager, "peak_gb": peak / 2 ** 30,
                   "what": "monet_wrapper.MONeTWrapper + schedule.Schedule from the reference, unmodified, "
                           "the reference's node set (no fused nodes), loss by torch"}
            try:
                cap = graphed.CapturedStep(step, [xs, y], warmup=1)
                for _ in range(2):
                    cap(xs, y)
                ms_g, _ = timed(lambda: cap(xs, y), args.steps)
                out["graphed_ms_per_step"] = ms_g
                out["graphed_images_per_s"] = B / (ms_g * 1e-3)
                del cap
            except Exception as exc:      # noqa: BLE001
                out["graph_error"] = f"{type(exc).__name__}: {exc}"[:300]
                print("reference executor: capture failed:", out["graph_error"], file=sys.stderr, flush=True)
                torch.cuda.synchronize()
            del wrapped, step, opt
            return out
    except Exception as exc:              # noqa: BLE001 - the comparator must not take the bench line down
        return {"unavailable": f"{type(exc).__name__}: {exc}"[:300]}


def _stats(ms_list):
    return {"min": min(ms_list), "median": statistics.median(ms_list), "max": max(ms_list)}


# ----------------------------------------------------------------------------- ours
def run_ours(args):
    import math

    import torch
    import torch.distributed as dist

    from monet_b200 import _lib, build, runner
    from monet_b200 import dist as mbdist
    from monet_b200 import functional as F
    from monet_b200.lm_ops.softmax import SoftmaxCrossEntropy

    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU fallback for the operators)")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    rank, world = mbdist.init_from_env(dev)
    import shutil
    if shutil.which("nvcc") or not _lib.LIB_PATH.exists():
        build.build()                      # incremental: never time a library older than its sources
    api = _lib.lib()

    make_model, default_batch, in_shape, classes, default_schedule, workload = workloads()[args.model]
    B = args.batch or default_batch
    schedule = args.schedule or default_schedule
    pixelwise = args.model == "unet"
    metric = METRIC if args.model == "resnet50" and B == 184 else f"{args.model}_bs{B}_train_images_per_s"

    torch.manual_seed(0)
    ctor = (lambda: make_model()) if args.model == "unet" else (lambda: make_model(num_classes=classes))
    model = ctor().to(dev).train()
    model = model.to(memory_format=torch.channels_last)       # filters as [K][R][S][C]
    params = [p for p in model.parameters()]
    opt = torch.optim.SGD(params, lr=0.1, momentum=0.9)

    def make_runner(fuse, policy_name):
        policy = getattr(runner, policy_name)
        if not fuse and policy_name == "budget_10gb":
            policy = runner.low_memory            # the block-output rule needs the fused block nodes
        return runner.Runner(model, policy, fuse=fuse, channel_sums=not args.no_channel_sums)

    run = make_runner(not args.no_fuse, schedule)
    buckets = None
    if world > 1:
        buckets = mbdist.GradientBuckets(list(model.named_parameters()), n_buckets=args.buckets)
        buckets.install(run)
    ce = SoftmaxCrossEntropy()

    g = torch.Generator(device="cpu").manual_seed(1 + rank)
    x_host = torch.randn(B, *in_shape, generator=g).pin_memory()
    label_shape = (B,) + (tuple(in_shape[1:]) if pixelwise else ())
    y_host = torch.randint(0, classes, label_shape, generator=g).pin_memory()
    x_dev = x_host.to(dev)
    y_dev = y_host.to(dev)
    fixed_bytes = sum(p.numel() * 4 for p in params) * 3 + x_dev.numel() * 4 + y_dev.numel() * 8

    def make_step(run_):
        def step(x, y):
            for p in params:
                p.grad = None              # the backward hands over freshly written gradients
            out = run_.forward(x)
            loss = ce.forward(out, y)
            run_.backward(ce.backward())
            if buckets is not None:
                buckets.wait()             # every bucket was all-reduced on the comm stream meanwhile
            opt.step()
            return loss
        return step

    step = make_step(run)
    # measured before any graph capture (a capture that fails leaves the CUDA generator unusable)
    tf32_measured = measure_tf32_peak(dev) if rank == 0 else None

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, n):
        """n calls of fn(), one CUDA event per step boundary: (mean ms, per-step ms list)."""
        evs = [torch.cuda.Event(enable_timing=True) for _ in range(n + 1)]
        barrier()
        evs[0].record()
        for i in range(n):
            fn()
            evs[i + 1].record()
        barrier()
        per = [evs[i].elapsed_time(evs[i + 1]) for i in range(n)]
        return evs[0].elapsed_time(evs[n]) / n, per

    # ---- warm-up, then a survey of every entry-point family over `survey_steps` eager steps
    fam_events = {}
    stream = torch.cuda.current_stream()
    watch = None

    def before(name):
        if watch is None or name in watch:
            ev = torch.cuda.Event(enable_timing=True)
            ev.record(stream)
            fam_events.setdefault(name, []).append([ev, None])

    def after(name):
        if watch is None or name in watch:
            ev = torch.cuda.Event(enable_timing=True)
            ev.record(stream)
            fam_events[name][-1][1] = ev

    W = max(args.warmup, 3)
    for _ in range(W):
        loss = step(x_dev, y_dev)
    torch.cuda.synchronize()
    survey_steps = 2
    _lib.set_probe(before, after)
    for _ in range(survey_steps):
        loss = step(x_dev, y_dev)
    torch.cuda.synchronize()
    _lib.set_probe()
    survey = {k: sum(a.elapsed_time(b) for a, b in v) / survey_steps for k, v in fam_events.items()}
    survey_calls = {k: len(v) / survey_steps for k, v in fam_events.items()}
    costs = family_costs(run, (B,) + tuple(in_shape))
    dominant = max((k for k in survey if k in costs), key=lambda k: survey[k])
    fam_events.clear()
    watch = {dominant}

    # ---- timed region 1: eager launches, batch resident in HBM
    sampler = ClockSampler(local)
    sampler.start()
    torch.cuda.reset_peak_memory_stats()
    launches0 = api.mb_launch_count()
    _lib.set_probe(before, after)
    ms_eager, per_eager = timed(lambda: step(x_dev, y_dev), args.steps)
    _lib.set_probe()
    launches = api.mb_launch_count() - launches0
    h0 = time.perf_counter()
    loss = step(x_dev, y_dev)              # host time to enqueue one step on an idle GPU
    host_ms = (time.perf_counter() - h0) * 1e3
    barrier()
    ms_dev, per_step = ms_eager, per_eager
    peak = torch.cuda.max_memory_allocated()
    dom_ms = sum(a.elapsed_time(b) for a, b in fam_events[dominant]) / args.steps
    dom_calls = len(fam_events[dominant]) / args.steps

    # ---- timed region 1g: the whole step (forward, loss, backward, bucketed all-reduce,
    # optimiser) replayed from one CUDA graph.  The executor is a Python loop that enqueues a
    # step in ~12 ms; the replay is one host call and launches exactly what the eager step did.
    graph, graph_err, host_replay_ms = None, None, None
    x_st, y_st = x_dev.clone(), y_dev.clone()
    if not args.no_cuda_graph:
        try:
            graph = torch.cuda.CUDAGraph()
            # with NCCL in the step its watchdog thread polls events while this thread captures
            mode = {"capture_error_mode": "thread_local"} if world > 1 else {}
            with torch.cuda.graph(graph, **mode):
                loss_st = step(x_st, y_st)
        except Exception as exc:          # capture refused: keep the eager numbers
            graph, graph_err = None, f"{type(exc).__name__}: {exc}"[:300]
            torch.cuda.synchronize()

    def gstep(x, y):
        if x is not x_st:
            x_st.copy_(x, non_blocking=True)
            y_st.copy_(y, non_blocking=True)
        graph.replay()
        return loss_st

    if graph is not None:
        for _ in range(3):
            loss = gstep(x_st, y_st)
        ms_dev, per_step = timed(lambda: gstep(x_st, y_st), args.steps)
        h0 = time.perf_counter()
        loss = gstep(x_st, y_st)
        host_replay_ms = (time.perf_counter() - h0) * 1e3
        barrier()
    run_step = gstep if graph is not None else step

    # ---- timed region 2: end to end from pinned host memory, loss read back every step.
    # Inputs are double-buffered: the batch of step i+1 crosses PCIe on a copy stream while
    # step i computes; every step's batch is copied inside the timed region.
    copy_stream = torch.cuda.Stream()
    xb = [x_dev, torch.empty_like(x_dev)]
    yb = [y_dev, torch.empty_like(y_dev)]
    ready = [torch.cuda.Event(), torch.cuda.Event()]
    free = [torch.cuda.Event(), torch.cuda.Event()]

    def upload(i):
        k = i % 2
        with torch.cuda.stream(copy_stream):
            copy_stream.wait_event(free[k])          # the step that last read this buffer is done
            xb[k].copy_(x_host, non_blocking=True)
            yb[k].copy_(y_host, non_blocking=True)
            ready[k].record(copy_stream)

    # The loss of every step is copied to pinned host memory and read there, one step behind the
    # launches (as a training loop that logs its loss does): the host reads step i - 1 while step
    # i runs, so the GPU does not idle while the host turns around.
    loss_pin = [torch.zeros((), dtype=torch.float32).pin_memory() for _ in range(2)]
    loss_ev = [torch.cuda.Event(), torch.cuda.Event()]

    def e2e_steps(n):
        last = 0.0
        for k in range(2):
            free[k].record(stream)
        upload(0)
        for i in range(n):
            k = i % 2
            stream.wait_event(ready[k])
            loss_t = run_step(xb[k], yb[k])
            free[k].record(stream)
            loss_pin[k].copy_(loss_t.detach().reshape(()), non_blocking=True)   # device -> host, every step
            loss_ev[k].record(stream)
            if i + 1 < n:
                upload(i + 1)
            if i >= 1:
                loss_ev[1 - k].synchronize()
                last = float(loss_pin[1 - k])
        k = (n - 1) % 2
        loss_ev[k].synchronize()
        last = float(loss_pin[k])
        return last

    e2e_steps(2)                                     # untimed: first use of the copy stream
    barrier()
    w0 = time.perf_counter()
    e0 = torch.cuda.Event(enable_timing=True); e1 = torch.cuda.Event(enable_timing=True)
    e0.record()
    last = e2e_steps(args.steps)
    e1.record()
    barrier()
    ms_e2e = max(e0.elapsed_time(e1), (time.perf_counter() - w0) * 1e3) / args.steps
    clocks = sampler.stop()
    conv_status = F.conv_device_status()

    if world > 1:
        t = torch.tensor([ms_dev, ms_e2e, ms_eager], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms_dev, ms_e2e, ms_eager = float(t[0]), float(t[1]), float(t[2])

    # ---- N > 1: the same replayed step without the gradient exchange, on every rank; the
    # difference is the part of the all-reduce that backward does not hide
    allreduce_exposed = None
    if world > 1 and graph is not None:
        kept, buckets = buckets, None          # `step` reads this variable when it runs
        run.on_param_grad = None
        g_local = None
        try:
            g_local = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g_local, capture_error_mode="thread_local"):
                step(x_st, y_st)
        except Exception:
            g_local = None
            torch.cuda.synchronize()
        ok = torch.tensor([1 if g_local is not None else 0], device=dev)
        dist.all_reduce(ok, op=dist.ReduceOp.MIN)
        if int(ok[0]):
            for _ in range(3):
                g_local.replay()
            ms_local, _ = timed(g_local.replay, args.steps)
            t = torch.tensor([ms_local], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            allreduce_exposed = {"ms_per_step_without_exchange": float(t[0]),
                                 "allreduce_ms_exposed": ms_dev - float(t[0])}
        del g_local
        buckets = kept
        kept.install(run)

    # ---- comparators, rank 0 at N = 1 only (they are about one GPU): the reference's node set
    # (no fused nodes) through the same executor, and stock PyTorch on this GPU
    extras = {}
    if rank == 0 and world == 1 and not args.no_comparators:
        del graph
        graph = None
        torch.cuda.empty_cache()
        if not args.no_fuse:
            run_u = make_runner(False, schedule)
            step_u = make_step(run_u)
            for _ in range(3):
                step_u(x_dev, y_dev)
            torch.cuda.synchronize()
            torch.cuda.reset_peak_memory_stats()
            ms_u_eager, _ = timed(lambda: step_u(x_dev, y_dev), args.steps)
            peak_u = torch.cuda.max_memory_allocated()
            ms_u = ms_u_eager
            try:
                gu = torch.cuda.CUDAGraph()
                with torch.cuda.graph(gu):
                    step_u(x_st, y_st)
                for _ in range(2):
                    gu.replay()
                ms_u, _ = timed(gu.replay, args.steps)
                del gu
            except Exception:
                torch.cuda.synchronize()
            extras["unfused"] = {"ms_per_step": ms_u, "eager_ms_per_step": ms_u_eager, "peak_gb": peak_u / 2 ** 30,
                                 "what": "the reference's node set (batch norm, add, ReLU as separate operators), "
                                         "same schedule family, same executor"}
            del run_u, step_u
            for p in params:
                p.grad = None
            torch.cuda.empty_cache()
        tms, tpeak = torch_gpu_baseline(ctor, x_dev, y_dev, args.steps, W, pixelwise)
        extras["torch_gpu"] = {"ms_per_step": tms, "images_per_s": B / (tms * 1e-3), "peak_gb": tpeak / 2 ** 30,
                               "what": "stock PyTorch eager, channels_last, cuDNN TF32 + benchmark, same batch, CE + SGD"}
        extras["overhead_vs_torch_gpu"] = ms_dev / tms - 1.0
        if "unfused" in extras:
            extras["unfused"]["overhead_vs_torch_gpu"] = extras["unfused"]["ms_per_step"] / tms - 1.0
        if args.model == "resnet50" and not args.no_fuse:
            extras["reference_executor"] = reference_executor_block(model, params, x_dev, y_dev, B, in_shape, args, timed)
            for p in params:
                p.grad = None
            torch.cuda.empty_cache()
    if rank == 0:
        peaks_file = ROOT / "MEASURED_PEAKS.json"
        if peaks_file.exists():
            mp = json.loads(peaks_file.read_text())
            hbm, which = mp["hbm_gbs"], "measured"
        else:
            hbm, which = 6650.0, "fallback"
        tf32 = tf32_measured

        def roof_of(b, f, ms):
            t_hbm, t_tc = b / (hbm * 1e9), f / (tf32 * 1e12)
            if t_hbm >= t_tc:
                r = {"bound": "hbm", "achieved": b / (ms * 1e-3) / 1e9, "peak": hbm, "unit": "GB/s"}
            else:
                r = {"bound": "tensor", "achieved": f / (ms * 1e-3) / 1e12, "peak": tf32, "unit": "TFLOP/s"}
            r["frac"] = r["achieved"] / r["peak"]
            return r

        b, f = costs[dominant][:2]
        roof = roof_of(b, f, dom_ms)
        ratio = TRAFFIC_RATIO.get(dominant)
        roof.update({"traffic": (ratio * b / dom_calls / 1e9) if ratio else None, "traffic_unit": "GB per launch (ncu ratio x algorithmic bytes)",
                     "algorithmic_gb_per_launch": b / dom_calls / 1e9, "kernel": dominant, "launches_per_step": dom_calls,
                     "ms_per_step": dom_ms, "peak_source": which,
                     "note": "entry point timed with CUDA events inside the eager timed region (the graphed "
                             "region replays the same launches); tensor peak = cuBLAS TF32 8192^3 sustained, measured in this run"})
        families = {}
        for k, ms in sorted(survey.items(), key=lambda kv: -kv[1]):
            if k not in costs or ms <= 0:
                continue
            fb, ff, calls = costs[k]
            r = roof_of(fb, ff, ms)
            # sum over the family's calls of each call's own floor (the slower of its bytes at the
            # HBM rate and its flops at the TF32 rate): a family mixes HBM-bound and tensor-bound
            # layers, so this, not the family totals, is what the kernels can be held against
            floor_ms = sum(max(cb / (hbm * 1e9), cf / (tf32 * 1e12)) for cb, cf in calls) * 1e3
            families[k] = {"ms_per_step": round(ms, 3), "calls_per_step": survey_calls[k], "algorithmic_gb": round(fb / 1e9, 3),
                           "gflop": round(ff / 1e9, 1), "bound": r["bound"], "achieved": round(r["achieved"], 1),
                           "unit": r["unit"], "frac": round(r["frac"], 3),
                           "per_call_floor_ms": round(floor_ms, 3), "frac_of_per_call_floor": round(floor_ms / ms, 3)}
        conv_ms = sum(v["ms_per_step"] for k, v in families.items() if k.startswith("mb_conv2d"))
        conv_fl = sum(costs[k][1] for k in families if k.startswith("mb_conv2d"))
        conv_floor = sum(v["per_call_floor_ms"] for k, v in families.items() if k.startswith("mb_conv2d"))
        line = {
            "metric": metric, "value": B * world / (ms_dev * 1e-3), "unit": "images/s",
            "n_gpus": world, "steps": args.steps, "warmup": W, "ms_per_step": ms_dev,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32(tf32 conv)",
            "data": "synthetic",
            "config": {"workload": workload, "schedule": schedule,
                       "fused_bn_add_relu": not args.no_fuse, "global_batch": B * world,
                       "parallelism": f"dp{world}", "l2": "inputs and activations exceed L2 (126 MB) many times over"},
            "peak_gb": peak / 2 ** 30, "activation_peak_gb": (peak - fixed_bytes) / 2 ** 30,
            "loss": last, "loss_finite": math.isfinite(last), "conv_device_status": conv_status,
            "e2e": {"value": B * world / (ms_e2e * 1e-3), "unit": "images/s",
                    "h2d_bytes_per_step": x_host.numel() * 4 + y_host.numel() * 8, "d2h_bytes_per_step": 4,
                    "how": "batch copied from pinned host memory every step (double-buffered on a copy stream), "
                           "loss copied to pinned host memory every step and read there one step behind the launches"},
            "cuda_graph": graph_err is None and not args.no_cuda_graph, "eager_ms_per_step": ms_eager,
            "ms_per_step_stats": _stats(per_step), "eager_ms_per_step_stats": _stats(per_eager),
            "host_enqueue_ms": host_ms, "host_replay_ms": host_replay_ms,
            "gpu_launches": int(launches), "clocks": clocks, "roofline": roof,
            "tf32_peak_measured_tflops": tf32,
            "roofline_families": families,
            "conv_total": {"ms_per_step": round(conv_ms, 3), "tflops": round(conv_fl / (conv_ms * 1e-3) / 1e12, 1) if conv_ms else None,
                           "frac_of_measured_tf32": round(conv_fl / (conv_ms * 1e-3) / 1e12 / tf32, 3) if conv_ms else None,
                           "per_call_floor_ms": round(conv_floor, 3),
                           "frac_of_per_call_floor": round(conv_floor / conv_ms, 3) if conv_ms else None},
        }
        if buckets is not None:
            line["gradient_buckets"] = {"count": len(buckets.buckets), "mb": [round(fl.numel() * 4 / 2 ** 20, 1) for fl in buckets.flat],
                                        "overlap": "all-reduce (mean) per bucket on a communication stream during backward, inside the captured step"}
        if allreduce_exposed is not None:
            line.update(allreduce_exposed)
        line.update(extras)
        if graph_err:
            line["cuda_graph_error"] = graph_err
        if not args.no_cpu_baseline and world == 1 and args.model == "resnet50":
            from oracle import cpu_baseline
            cb = args.cpu_batch or B
            ips, ms, threads = cpu_baseline.resnet50_train_steps(cb, 2, warmup=1)
            line["cpu_baseline"] = {"value": ips, "unit": "images/s", "cores": threads, "kind": "port",
                                    "sample": f"2 eager steps of batch {cb} (of {B}), PyTorch CPU"}
        print(json.dumps(line), flush=True)
    bad = conv_status != 0 or not math.isfinite(last)
    if bad:
        print(f"invalid run: conv_device_status={conv_status}, loss={last}", file=sys.stderr, flush=True)
    if world > 1:
        # Leave without tearing NCCL down: destroying a communicator whose collectives live in a
        # captured graph was seen to block at exit.  Every rank has passed the max-reduction of
        # the timings above, so nobody waits for a peer any more.
        torch.cuda.synchronize()
        sys.stdout.flush()
        sys.stderr.flush()
        os._exit(1 if bad else 0)
    if bad:
        raise SystemExit(1)


def main():
    args = parse()
    if args.micro:
        run_micro(args)
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
