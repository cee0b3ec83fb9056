"""Cost-table producer for MONeT's solver: ``meminfo`` / ``computeinfo`` with the reference's
signatures and return layout (monet/meminfo.py:6-187,191-396), measured the way this library
runs.

``SolverInfo.get_workspace_cost`` (solver_info.py:362-372) calls, for every backward node and
every implementation of its operator,

    fwd_mem, bwd_mem, fwd_mem_recompute = meminfo(n, op, graph, bs, bwd_op, conv_mode, inplace_mode, x, *params)
    fwd_ms,  bwd_ms,  fwd_ms_recompute  = computeinfo(...same...)

with one entry per convolution variant in the ``conv`` modes (``op.algorithm = i``, backward
``algorithm = 10 * type + i``), ``[out of place, in place]`` for operators that have an
``inplace`` attribute in the ``inplace`` modes, and ``[first pass]`` / ``[cached statistics]``
for batch norm; a variant that raises records time -1 / memory 0, which the ILP bans
(cvxpy_solver.py:134-138).  The reference's own functions work unchanged over these operators
and are the default (``reference_host.build_solver_info(profiler="reference")``).  The ones
here differ in how, not in what:

* times come from CUDA events around ``runtime_sample`` calls on the current stream after
  two warm-up calls.  The reference times ``time()`` + ``synchronize`` around 20 calls, which on
  a B200 mostly measures the Python call (tens of microseconds) rather than kernels that
  take as little;
* 4-D activations are created ``channels_last``, the layout every operator here produces
  and the next one therefore receives; with NCHW random inputs each convolution would be
  charged a layout conversion (time and an activation-sized temporary) that never happens
  inside a network;
* a batch norm's two forward entries are both *first* passes (statistics cleared before each
  call), its cached-statistics pass is reported separately; the reference's in-place branch
  (meminfo.py:57-70) measures the second call on warm statistics;
* memory is the allocator's peak over the call minus the outputs, as in the reference, so a
  variant's scratch (allocated through torch by ``functional``) is what
  ``mb_conv_workspace_bytes`` declares.

``install()`` makes ``monet.solver_info`` use them.
"""
from __future__ import annotations

import numpy as np
import torch

RUNTIME_SAMPLE = 20
WARMUP = 2


def _shape(graph, index, bs):
    return [bs if v == -1 else int(v) for v in graph.nodes[index].shape]


def _activation(shape, requires_grad, device):
    t = torch.randn(shape, device=device)
    if t.dim() == 4:
        t = t.contiguous(memory_format=torch.channels_last)
    return t.requires_grad_(bool(requires_grad))


def _arguments(n, graph, bs, bwd_op, params, device):
    """Forward arguments of node n (meminfo.py:12-34): parameters are the model's own tensors,
    activations are random; for the two-step operators (dense convolution, addmm) the
    parameter step sees weights that need gradients and inputs that do not, the input step
    the opposite."""
    mod = __import__("monet.graph", fromlist=["ComputeNode"])
    V, Param = mod.ComputeNode.V, mod.Param
    two_step = (n.op == "aten::_convolution" and not n.is_depthwise) or n.op == "aten::addmm"
    args, meta = [], []
    for a in n.args:
        if isinstance(a, V):
            args.append(a.value)
            meta.append(a.value)
            continue
        src = graph.nodes[a.index]
        if isinstance(src, Param):
            p = params[a.index]
            if two_step:
                p = p.requires_grad_(bwd_op == "param_grad")
            args.append(p)
            meta.append([tuple(p.shape), p.requires_grad, p.device, p.dtype, p])
        else:
            rg = False if (two_step and bwd_op == "param_grad") else a.requires_grad
            shape = _shape(graph, a.index, bs)
            args.append(_activation(shape, rg, device))
            meta.append([shape, rg, device, torch.float32, None])
    return args, meta


def _out_bytes(outs):
    if not isinstance(outs, (tuple, list)):
        outs = [outs]
    return sum(o.numel() * o.element_size() for o in outs if o is not None and torch.is_tensor(o))


def _timed(fn, reset=None):
    """Mean milliseconds of fn() over RUNTIME_SAMPLE calls (CUDA events, current stream)."""
    for _ in range(WARMUP):
        if reset:
            reset()
        out = fn()
        del out
    torch.cuda.synchronize()
    total = 0.0
    if reset is None:
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(RUNTIME_SAMPLE):
            out = fn()
            del out
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / RUNTIME_SAMPLE
    for _ in range(RUNTIME_SAMPLE):
        reset()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        out = fn()
        e1.record()
        del out
        torch.cuda.synchronize()
        total += e0.elapsed_time(e1)
    return total / RUNTIME_SAMPLE


def _peak(fn):
    """(allocator peak over fn() minus its outputs, outputs)."""
    torch.cuda.synchronize()
    torch.cuda.empty_cache()
    torch.cuda.reset_peak_memory_stats()
    m0 = torch.cuda.memory_stats()["allocated_bytes.all.peak"]
    outs = fn()
    torch.cuda.synchronize()
    m1 = torch.cuda.memory_stats()["allocated_bytes.all.peak"]
    return (m1 - m0) - _out_bytes(outs), outs


def _forward_cases(n, op, conv_mode, inplace_mode):
    """[(label, setup)] in the order the tables expect."""
    dense_conv = n.op == "aten::_convolution" and not n.is_depthwise
    if conv_mode and dense_conv:
        return [("algo", i) for i in range(op.n_fwd_algos())]
    if inplace_mode and hasattr(op, "inplace"):
        return [("inplace", False), ("inplace", True)]
    return [("plain", None)]


def _apply_case(op, case, n):
    kind, v = case
    if kind == "algo":
        op.algorithm = v
    elif kind == "inplace":
        op.inplace = v
    if n.is_depthwise:
        op.is_depthwise = True


def _stored_for_backward(op, outs, meta, bwd_op, n, device):
    """The `stored` list the executor would assemble (schedule.py:255-272), from fresh tensors."""
    from . import lm_ops
    outs = outs if isinstance(outs, (tuple, list)) else [outs]
    storage = op.backward_storage
    storage = storage if isinstance(storage, list) else [storage]
    want = []
    for st in storage:
        if isinstance(st, lm_ops.InputStorage):
            want += [meta[i] for i in st.ids]
        elif isinstance(st, lm_ops.OutputStorage):
            want.append(("like", outs[0]))
        elif isinstance(st, lm_ops.IntermediateStorage):
            want.append(("like", outs[-1]))
    two_step = (n.op == "aten::_convolution" and not n.is_depthwise) or n.op == "aten::addmm"
    if two_step and bwd_op == "ip_grad" and want:
        want[0] = None                                   # the input step does not get x (meminfo.py:352-354)

    def make():
        stored = []
        for w in want:
            if w is None:
                stored.append(None)
            elif isinstance(w, tuple):
                stored.append(torch.ones_like(w[1]))
            elif isinstance(w, list):
                if w[4] is not None:
                    stored.append(w[4])                   # a parameter: the model's own tensor
                else:
                    stored.append(_activation(w[0], w[1], device))
            else:
                stored.append(w)
        return stored
    return make


def _backward_cases(n, op, conv_mode, bwd_op):
    dense_conv = n.op == "aten::_convolution" and not n.is_depthwise
    two_step = dense_conv or n.op == "aten::addmm"
    base = 10 if bwd_op == "ip_grad" else 0
    if conv_mode and dense_conv:
        count = op.n_bwd_ip_algos() if bwd_op == "ip_grad" else op.n_bwd_wt_algos()
        return [base + i for i in range(count)]
    return [base] if two_step else [None]


def _run(n, op, graph, bs, bwd_op, conv_mode, inplace_mode, params, want_time):
    device = torch.device("cuda", torch.cuda.current_device())
    args, meta = _arguments(n, graph, bs, bwd_op, params, device)
    is_bn = n.op == "aten::batch_norm"
    fwd, fwd_re, bwd = [], [], []
    outs = None

    def clear_stats():
        if is_bn:
            op.params = None

    def fresh_args():
        # an in-place forward destroys its input: give every call its own copy
        return [a.clone() if (torch.is_tensor(a) and a.dim() == 4 and getattr(op, "inplace", False)
                              and a is args[0]) else a for a in args]

    for case in _forward_cases(n, op, conv_mode, inplace_mode):
        _apply_case(op, case, n)
        try:
            if want_time:
                # (an in-place case is timed on one buffer over and over: the copy that keeps the
                # memory measurement honest must not be inside the timed call)
                fwd.append(_timed(lambda: op.forward(*args), reset=clear_stats if is_bn else None))
            else:
                clear_stats()
                a = fresh_args()
                peak, o = _peak(lambda: op.forward(*a))
                fwd.append(peak)
                del o, a
        except Exception as exc:          # noqa: BLE001 - a variant that cannot run is data, not an error
            print("profiler: forward case", case, "of", n.op, "failed:", exc)
            fwd.append(-1 if want_time else 0)
            torch.cuda.empty_cache()
    if is_bn:
        clear_stats()
        op.inplace = False if hasattr(op, "inplace") else None
        warm = op.forward(*args)           # seeds the cached statistics
        del warm
        if want_time:
            fwd_re.append(_timed(lambda: op.forward(*args)))
        else:
            peak, o = _peak(lambda: op.forward(*args))
            fwd_re.append(peak)
            del o

    if bwd_op is not None:
        # one more forward to have outputs (and op.params) of the right kind for the backward
        if hasattr(op, "inplace"):
            op.inplace = False
        if conv_mode and n.op == "aten::_convolution" and not n.is_depthwise:
            op.algorithm = 0
        clear_stats()
        outs = op.forward(*args)
        first = outs[0] if isinstance(outs, (tuple, list)) else outs
        make_stored = _stored_for_backward(op, outs, meta, bwd_op, n, device)
        grad_shape, like = tuple(first.shape), first
        del outs, first
        single = None
        for alg in _backward_cases(n, op, conv_mode, bwd_op):
            try:
                if alg is not None:
                    op.algorithm = alg
                if n.is_depthwise:
                    op.is_depthwise = True
                if want_time:
                    stored = make_stored()

                    def call():
                        g = torch.ones_like(like)         # backward may overwrite its gradient
                        return op.backward(g, stored, nodel=True)
                    bwd.append(_timed(call))
                    del stored
                else:
                    stored = make_stored()
                    g = torch.ones_like(like)
                    peak, grads = _peak(lambda: op.backward(g, stored))
                    bwd.append(peak)
                    del grads, g, stored
            except Exception as exc:      # noqa: BLE001
                print("profiler: backward case", alg, "of", n.op, "failed:", exc)
                single = exc
                bwd.append(-1 if want_time else 0)
                torch.cuda.empty_cache()
        if single is not None and len(bwd) == 1:
            raise RuntimeError(f"the only backward implementation of {n.op} failed: {single}")
        del like
    clear_stats()
    torch.cuda.empty_cache()
    return fwd, bwd, fwd_re


def computeinfo(n, op, graph, bs, bwd_op, conv_mode, inplace_mode, *args):
    """Run times in milliseconds: (forward per case, backward per case, batch-norm cached-statistics
    forward); -1 marks a case that raised."""
    with torch.no_grad():
        fwd, bwd, fwd_re = _run(n, op, graph, bs, bwd_op, conv_mode, inplace_mode, args, True)
    return (np.array(fwd, dtype="f4"), np.array(bwd, dtype="f4"), np.array(fwd_re, dtype="f4"))


def meminfo(n, op, graph, bs, bwd_op, conv_mode, inplace_mode, *args):
    """Working memory in MB beyond inputs and outputs: (forward per case, backward per case,
    batch-norm cached-statistics forward); 0 for a case that raised."""
    with torch.no_grad():
        fwd, bwd, fwd_re = _run(n, op, graph, bs, bwd_op, conv_mode, inplace_mode, args, False)
    mb = 1024.0 * 1024.0
    return np.array(fwd) / mb, np.array(bwd) / mb, np.array(fwd_re) / mb


def install(ref=None) -> None:
    """Make ``SolverInfo.get_workspace_cost`` (solver_info.py:370-371) call the two functions
    above instead of monet/meminfo.py's."""
    from . import reference_host
    ref = ref or reference_host.activate()
    ref.solver_info.meminfo = meminfo
    ref.solver_info.computeinfo = computeinfo


def uninstall(ref=None) -> None:
    from . import reference_host
    ref = ref or reference_host.activate()
    ref.solver_info.meminfo = ref.meminfo.meminfo
    ref.solver_info.computeinfo = ref.meminfo.computeinfo
