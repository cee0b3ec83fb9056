"""A small executor that drives the low-memory operators the way MONeT's ``Schedule`` does.

MONeT's graph extractor, solver and ``Schedule`` (monet/graph.py, cvxpy_solver.py,
schedule.py) stay what they are; this module exists so that the operator library can be run
and measured on whole networks without them: it extracts a straight-line graph of aten-style
nodes from a torchvision-style ``nn.Module`` with ``torch.fx``, picks one implementation per
node from the registry according to a *policy* (what a solver solution would dictate), and
then executes forward and backward through the operators' own protocol:

* ``op.forward(*aten_args)`` returning a tensor, or ``(tensor, intermediate)`` when the
  operator declares an ``IntermediateStorage``;
* tensors are kept alive only while a later forward node or some operator's
  ``backward_storage`` needs them;
* ``op.backward(grad, stored)`` with ``stored`` ordered like the storage descriptors
  (schedule.py:255-272), gradients returned per tensor argument in argument order;
* outputs of nodes marked *recompute* are dropped after their last forward use and rebuilt
  from their (stored) inputs when a backward needs them (schedule.py:243-246).

Two ready-made policies: ``store_all`` (what stock PyTorch keeps) and ``low_memory``
(in-place output-activated batch norm, ReLU recomputed from its input, 4-bit pooling indices).

``fuse_graph`` optionally rewrites batch_norm -> relu, batch_norm -> add -> relu and
add -> relu chains into the fused nodes of ``lm_ops/fused.py`` before execution.
"""
from __future__ import annotations

import operator
from dataclasses import dataclass, field
from typing import Any, Callable, Dict, List, Optional, Tuple

import torch
import torch.fx
import torch.nn as nn

from . import functional as F
from . import lm_ops
from .lm_ops.base import InputStorage, IntermediateStorage, OutputStorage


# ----------------------------------------------------------------------------- graph
@dataclass
class Arg:
    kind: str            # 'node' | 'param' | 'input' | 'const'
    value: Any


@dataclass
class Node:
    id: int
    op: str                       # aten name, e.g. 'aten::_convolution'
    args: List[Arg]
    module: str = ""              # qualified name of the nn.Module it came from
    users: List[int] = field(default_factory=list)
    sums_from: int = -1           # batch-norm-like node: id of the convolution whose statistics
                                  # warps leave the per-channel sums of this node's input, or -1


def _as_list(v, n=2):
    if isinstance(v, (tuple, list)):
        return [int(x) for x in v]
    return [int(v)] * n


def extract_graph(model: nn.Module) -> Tuple[List[Node], int]:
    """(nodes, id of the output node) for a model made of conv / batch-norm / ReLU / ReLU6 /
    max-pool / adaptive-avg-pool / linear / dropout modules joined by add, flatten and cat."""
    gm = torch.fx.symbolic_trace(model)
    mods = dict(gm.named_modules())
    nodes: List[Node] = []
    env: Dict[str, Arg] = {}

    def ref(a) -> Arg:
        if isinstance(a, torch.fx.Node):
            return env[a.name]
        return Arg('const', a)

    def emit(fx_node, op, args, module=""):
        n = Node(len(nodes), op, args, module)
        nodes.append(n)
        for a in args:
            if a.kind == 'node':
                nodes[a.value].users.append(n.id)
        env[fx_node.name] = Arg('node', n.id)

    out_id = -1
    n_inputs = 0
    for fn in gm.graph.nodes:
        if fn.op == 'placeholder':
            env[fn.name] = Arg('input', n_inputs)
            n_inputs += 1
        elif fn.op == 'call_module':
            m = mods[fn.target]
            x = ref(fn.args[0])
            P = lambda name: Arg('param', f"{fn.target}.{name}")   # noqa: E731
            if isinstance(m, nn.Conv2d):
                bias = P('bias') if m.bias is not None else Arg('const', None)
                emit(fn, 'aten::_convolution',
                     [x, P('weight'), bias, Arg('const', _as_list(m.stride)),
                      Arg('const', _as_list(m.padding)), Arg('const', _as_list(m.dilation)),
                      Arg('const', False), Arg('const', [0, 0]), Arg('const', m.groups)], fn.target)
            elif isinstance(m, nn.ConvTranspose2d):
                bias = P('bias') if m.bias is not None else Arg('const', None)
                emit(fn, 'aten::_convolution',
                     [x, P('weight'), bias, Arg('const', _as_list(m.stride)),
                      Arg('const', _as_list(m.padding)), Arg('const', _as_list(m.dilation)),
                      Arg('const', True), Arg('const', _as_list(m.output_padding)),
                      Arg('const', m.groups)], fn.target)
            elif isinstance(m, nn.BatchNorm2d):
                emit(fn, 'aten::batch_norm',
                     [x, P('weight'), P('bias'), P('running_mean'), P('running_var'),
                      Arg('const', True), Arg('const', m.momentum if m.momentum is not None else 0.1),
                      Arg('const', m.eps), Arg('const', True)], fn.target)
            elif isinstance(m, nn.ReLU):
                emit(fn, 'aten::relu_' if m.inplace else 'aten::relu', [x], fn.target)
            elif isinstance(m, nn.ReLU6):
                emit(fn, 'aten::hardtanh_' if m.inplace else 'aten::hardtanh',
                     [x, Arg('const', 0.0), Arg('const', 6.0)], fn.target)
            elif isinstance(m, nn.MaxPool2d):
                emit(fn, 'aten::max_pool2d',
                     [x, Arg('const', _as_list(m.kernel_size)),
                      Arg('const', _as_list(m.stride if m.stride is not None else m.kernel_size)),
                      Arg('const', _as_list(m.padding)), Arg('const', _as_list(m.dilation)),
                      Arg('const', bool(m.ceil_mode))], fn.target)
            elif isinstance(m, nn.AdaptiveAvgPool2d):
                emit(fn, 'aten::adaptive_avg_pool2d', [x, Arg('const', _as_list(m.output_size))], fn.target)
            elif isinstance(m, nn.Linear):
                if m.bias is None:
                    raise NotImplementedError("linear layer without bias")
                emit(fn, 'aten::addmm', [P('bias'), x, P('weight'), Arg('const', 1), Arg('const', 1)],
                     fn.target)
            elif isinstance(m, nn.Dropout):
                emit(fn, 'aten::dropout', [x, Arg('const', m.p), Arg('const', True)], fn.target)
            else:
                raise NotImplementedError(f"module {type(m).__name__} at {fn.target}")
        elif fn.op == 'call_function':
            if fn.target in (operator.add, torch.add):
                emit(fn, 'aten::add', [ref(fn.args[0]), ref(fn.args[1]), Arg('const', 1)])
            elif fn.target is operator.iadd:
                emit(fn, 'aten::add_', [ref(fn.args[0]), ref(fn.args[1]), Arg('const', 1)])
            elif fn.target is torch.flatten:
                start = fn.args[1] if len(fn.args) > 1 else fn.kwargs.get('start_dim', 0)
                emit(fn, 'aten::flatten', [ref(fn.args[0]), Arg('const', start), Arg('const', -1)])
            elif fn.target is torch.nn.functional.adaptive_avg_pool2d:
                emit(fn, 'aten::adaptive_avg_pool2d', [ref(fn.args[0]), Arg('const', _as_list(fn.args[1]))])
            elif fn.target is torch.cat:
                tensors = [ref(t) for t in fn.args[0]]
                dim = fn.args[1] if len(fn.args) > 1 else fn.kwargs.get('dim', 0)
                emit(fn, 'aten::cat', tensors + [Arg('const', dim)])
            else:
                raise NotImplementedError(f"function {fn.target}")
        elif fn.op == 'output':
            out_id = env[fn.args[0].name].value
        else:
            raise NotImplementedError(f"fx node kind {fn.op}")
    return nodes, out_id


def fuse_graph(nodes: List[Node], out_id: int) -> Tuple[List[Node], int]:
    """Rewrites the element-wise tails of batch norm into fused nodes:

    * ``batch_norm -> relu``                 => ``monet::batch_norm_relu`` (at the batch norm);
    * ``batch_norm -> hardtanh(0, 6)``       => ``monet::batch_norm_relu6``;
    * ``batch_norm -> add(., r) -> relu``    => ``monet::batch_norm_add_relu`` with ``r`` appended
      to the batch-norm arguments, placed where the add was (``r`` may be produced after the
      batch norm, e.g. by a downsample branch);
    * ``add -> relu`` (any other add)        => ``monet::add_relu``.

    A link is fused only when the intermediate value has no other reader, the batch norm is
    in training mode and the add has alpha == 1 and two distinct node operands."""
    by_id = {n.id: n for n in nodes}
    removed = set()
    alias: Dict[int, int] = {}
    relus = ('aten::relu', 'aten::relu_')
    adds = ('aten::add', 'aten::add_')

    def sole_user(n: Node) -> Optional[Node]:
        return by_id[n.users[0]] if len(n.users) == 1 and n.id != out_id else None

    def plain_add(u: Node) -> bool:
        return (u.op in adds and u.args[2].value == 1 and u.args[0].kind == 'node'
                and u.args[1].kind == 'node' and u.args[0].value != u.args[1].value)

    for n in nodes:
        if n.id in removed or n.op != 'aten::batch_norm' or not n.args[5].value:
            continue
        u = sole_user(n)
        if u is None:
            continue
        if u.op in relus:
            n.op = 'monet::batch_norm_relu'
            removed.add(u.id)
            alias[u.id] = n.id
        elif (u.op in ('aten::hardtanh', 'aten::hardtanh_') and float(u.args[1].value) == 0.0
              and float(u.args[2].value) == 6.0):
            n.op = 'monet::batch_norm_relu6'
            removed.add(u.id)
            alias[u.id] = n.id
        elif plain_add(u):
            r = sole_user(u)
            if r is None or r.op not in relus:
                continue
            other = u.args[1] if u.args[0].value == n.id else u.args[0]
            u.op = 'monet::batch_norm_add_relu'
            u.args = list(n.args) + [other]
            u.module = n.module
            removed.add(n.id)
            removed.add(r.id)
            alias[r.id] = u.id
    for n in nodes:
        if n.id in removed or not plain_add(n):
            continue
        r = sole_user(n)
        if r is not None and r.op in relus:
            n.op = 'monet::add_relu'
            removed.add(r.id)
            alias[r.id] = n.id

    kept = [n for n in nodes if n.id not in removed]
    renumber = {n.id: i for i, n in enumerate(kept)}

    def target(i: int) -> int:
        while i in alias:
            i = alias[i]
        return renumber[i]

    out: List[Node] = []
    for n in kept:
        args = [Arg('node', target(a.value)) if a.kind == 'node' else a for a in n.args]
        out.append(Node(renumber[n.id], n.op, args, n.module))
    for n in out:
        for a in n.args:
            if a.kind == 'node':
                out[a.value].users.append(n.id)
    link_channel_sums(out)
    return out, target(out_id)


_BN_LIKE = ('aten::batch_norm', 'monet::batch_norm_relu', 'monet::batch_norm_relu6',
            'monet::batch_norm_add_relu')


def link_channel_sums(nodes: List[Node]) -> None:
    """Marks every training-mode batch-norm-like node whose input is a dense convolution with no
    other reader: that convolution can sum its output per channel beside its epilogue and the
    batch norm skip its statistics pass."""
    for n in nodes:
        if n.op not in _BN_LIKE or not n.args[5].value or n.args[0].kind != 'node':
            continue
        src = nodes[n.args[0].value]
        if (src.op == 'aten::_convolution' and src.users == [n.id] and src.args[8].value == 1
                and not src.args[6].value):
            n.sums_from = src.id


# ---------------------------------------------------------------------------- policy
@dataclass
class Choice:
    impl: int = 0            # index into list_ops(mode, name)
    inplace: bool = False
    recompute: bool = False  # drop the output after the forward, rebuild it in backward
    algorithm: int = -1      # conv / addmm variant


Policy = Callable[[List[Node], Node], Choice]


def store_all(nodes: List[Node], n: Node) -> Choice:
    """What stock PyTorch keeps: batch norm from its input, ReLU in place keeping its output,
    max-pool keeping its input."""
    if n.op in ('aten::relu', 'aten::relu_'):
        return Choice(impl=1, inplace=_sole_user(nodes, n))
    if n.op in ('aten::hardtanh', 'aten::hardtanh_'):
        return Choice(impl=1, inplace=_sole_user(nodes, n))
    return Choice()


def low_memory(nodes: List[Node], n: Node) -> Choice:
    """In-place batch norm that backpropagates from its output, ReLU kept as nothing at all
    (recomputed from the batch-norm output it reads, gated in backward by that same tensor),
    residual add in place, max-pool keeping 4-bit indices."""
    if n.op == 'aten::batch_norm':
        return Choice(impl=1, inplace=_sole_user(nodes, n))
    if n.op in ('aten::relu', 'aten::relu_'):
        return Choice(impl=0, inplace=False, recompute=True)
    if n.op in ('aten::hardtanh', 'aten::hardtanh_'):
        return Choice(impl=0, inplace=False, recompute=True)
    if n.op == 'aten::max_pool2d':
        return Choice(impl=1)
    if n.op in ('monet::batch_norm_relu', 'monet::batch_norm_relu6'):
        return Choice(recompute=True)      # keeps x only; y = relu(bn(x)) is rebuilt from it
    return Choice()


def budget_10gb(nodes: List[Node], n: Node) -> Choice:
    """`low_memory`, and in addition the output of every second residual block
    (``monet::batch_norm_add_relu``) is dropped after the forward and rebuilt in backward from
    its kept batch-norm input and the kept output of the block before it (one 12 B/element
    pass each).  On ResNet-50 at batch 184 this brings the activations under 10 GB."""
    if n.op == 'monet::batch_norm_add_relu':
        index = sum(1 for m in nodes[:n.id] if m.op == 'monet::batch_norm_add_relu')
        return Choice(recompute=(index % 2 == 1))
    return low_memory(nodes, n)


def _sole_user(nodes: List[Node], n: Node) -> bool:
    """True when the first tensor argument is a node output nobody else reads."""
    a = n.args[0]
    return a.kind == 'node' and nodes[a.value].users == [n.id]


# -------------------------------------------------------------------------- executor
def _descriptors(op) -> list:
    bs = op.backward_storage
    if bs is None:
        return []
    return list(bs) if isinstance(bs, (list, tuple)) else [bs]


class Runner:
    """Executes forward and backward of an extracted graph through ``lm_ops``."""

    def __init__(self, model: nn.Module, policy: Policy = store_all,
                 mode: str = "conv_multiway_newnode", input_requires_grad: bool = False,
                 fuse: bool = False, channel_sums: bool = True):
        self.model = model
        self.nodes, self.out_id = extract_graph(model)
        if fuse:
            from .lm_ops import fused  # noqa: F401  (registers the monet:: nodes)
            self.nodes, self.out_id = fuse_graph(self.nodes, self.out_id)
            if not channel_sums:       # batch norms make their own statistics pass
                for n in self.nodes:
                    n.sums_from = -1
        self.mode = mode
        self.input_requires_grad = input_requires_grad
        self.choices = [policy(self.nodes, n) for n in self.nodes]
        self.param_grads: Dict[str, torch.Tensor] = {}
        self.on_param_grad: Optional[Callable[[str, torch.Tensor], None]] = None
        self._param_uses: Dict[str, int] = {}
        for n in self.nodes:
            for a in n.args:
                if a.kind == 'param':
                    self._param_uses[a.value] = self._param_uses.get(a.value, 0) + 1
        self.shapes: Dict[int, tuple] = {}      # node id -> output shape, filled by forward()
        self._tensors = dict(model.state_dict(keep_vars=True))
        self._last_fwd_user = {n.id: (max(n.users) if n.users else -1) for n in self.nodes}
        self._validate()

    # -- helpers ---------------------------------------------------------------
    def _new_op(self, n: Node):
        c = self.choices[n.id]
        impls = lm_ops.list_ops(self.mode, n.op)
        op = impls[min(c.impl, len(impls) - 1)]()
        if hasattr(op, 'inplace'):
            op.inplace = c.inplace
        if c.algorithm >= 0:
            op.algorithm = c.algorithm
        if n.op == 'aten::_convolution':
            w = self._tensors[n.args[1].value]
            groups = n.args[8].value
            op.is_depthwise = groups > 1 and groups == w.shape[0] and w.shape[1] == 1
        return op

    def _validate(self):
        for n in self.nodes:
            c = self.choices[n.id]
            if c.inplace and not _sole_user(self.nodes, n):
                raise ValueError(f"node {n.id} ({n.op}) cannot run in place: its input has other readers")

    def _resolve(self, n: Node, vals, inputs):
        out = []
        for a in n.args:
            if a.kind == 'node':
                t = vals[a.value]
                if t is None:
                    raise RuntimeError(f"node {n.id} ({n.op}) needs the output of node {a.value}, which was dropped")
                out.append(t.requires_grad_(True) if t.is_floating_point() else t)
            elif a.kind == 'param':
                out.append(self._tensors[a.value])
            elif a.kind == 'input':
                t = inputs[a.value]
                out.append(t.requires_grad_(self.input_requires_grad))
            else:
                out.append(a.value)
        return out

    def _needs_for_backward(self) -> Dict[int, int]:
        """node id -> id of the LAST (lowest-numbered) backward step that reads its output."""
        need: Dict[int, int] = {}

        def want(tensor_id, at):
            need[tensor_id] = min(need.get(tensor_id, at), at)

        for n in self.nodes:
            op = self._ops[n.id]
            for d in _descriptors(op):
                if isinstance(d, InputStorage):
                    for i in d.ids:
                        a = n.args[i]
                        if a.kind == 'node':
                            want(a.value, n.id)
                elif isinstance(d, OutputStorage):
                    want(n.id, n.id)
        # a recomputed node is rebuilt from its inputs, which therefore have to survive (or be
        # rebuilt themselves) until then; iterate because recomputed nodes can chain
        changed = True
        while changed:
            changed = False
            for n in self.nodes:
                if self.choices[n.id].recompute and n.id in need:
                    for a in n.args:
                        if a.kind == 'node' and need.get(a.value, len(self.nodes)) > need[n.id]:
                            need[a.value] = need[n.id]
                            changed = True
        return need

    # -- forward ---------------------------------------------------------------
    def forward(self, *inputs: torch.Tensor) -> torch.Tensor:
        self._inputs = inputs
        self._ops = {n.id: self._new_op(n) for n in self.nodes}
        self._need = self._needs_for_backward()
        vals: Dict[int, Optional[torch.Tensor]] = {}
        self._inter: Dict[int, Any] = {}
        with torch.no_grad():
            emitters = {n.sums_from: n for n in self.nodes if n.sums_from >= 0}
            for n in self.nodes:
                op = self._ops[n.id]
                args = self._resolve(n, vals, inputs)
                if n.id in emitters and hasattr(op, 'emit_channel_sums'):
                    rm = emitters[n.id].args[3]
                    op.emit_channel_sums = True
                    op.channel_sums_shift = self._tensors[rm.value] if rm.kind == 'param' else None
                if n.sums_from >= 0:
                    src = self._ops[n.sums_from]
                    op.input_sums = getattr(src, 'channel_sums', None)
                    src.channel_sums = None
                out = op.forward(*args)
                if any(isinstance(d, IntermediateStorage) for d in _descriptors(op)):
                    out, self._inter[n.id] = out
                del args
                vals[n.id] = out
                self.shapes[n.id] = tuple(out.shape)
                if self.choices[n.id].inplace:
                    src = n.args[0]
                    if src.kind == 'node':
                        if src.value in self._need:
                            raise RuntimeError(
                                f"node {n.id} ({n.op}) overwrote the output of node {src.value}, "
                                "which a backward step still needs: invalid policy")
                        vals[src.value] = None        # overwritten
                # drop whatever no later forward node and no backward needs
                for a in n.args:
                    if a.kind != 'node' or vals.get(a.value) is None:
                        continue
                    t = a.value
                    if self._last_fwd_user[t] <= n.id and not self._kept(t):
                        vals[t] = None
        self._vals = vals
        out = vals[self.out_id]
        # the output itself stays; everything else that backward does not need is gone already
        return out

    def _kept(self, t: int) -> bool:
        return t in self._need and not self.choices[t].recompute

    # -- backward --------------------------------------------------------------
    def _value_for_backward(self, t: int) -> torch.Tensor:
        """Output of node t, recomputing it from its inputs when it was dropped."""
        v = self._vals.get(t)
        if v is not None:
            return v
        n = self.nodes[t]
        if not self.choices[t].recompute:
            raise RuntimeError(f"output of node {t} ({n.op}) is needed in backward but was not kept")
        op = self._new_op(n)
        op.inplace = False if hasattr(op, 'inplace') else None
        op.params = getattr(self._ops[t], 'params', None)
        args = []
        for a in n.args:
            if a.kind == 'node':
                args.append(self._value_for_backward(a.value))
            elif a.kind == 'param':
                args.append(self._tensors[a.value])
            elif a.kind == 'input':
                args.append(self._inputs[a.value])
            else:
                args.append(a.value)
        out = op.forward(*args)
        if isinstance(out, tuple):
            out = out[0]
        self._vals[t] = out          # kept until its last backward reader has run (_release)
        return out

    def backward(self, grad_output: torch.Tensor) -> None:
        """Backpropagates `grad_output` from the output node; parameter gradients are left in
        ``self.param_grads`` (and accumulated into ``param.grad``)."""
        # node id -> gradients received so far.  They are summed as they arrive, except that an
        # operator with ``accepts_grad_pair`` is handed two of them unsummed (it folds the sum
        # into its own pass).
        grads: Dict[int, List[torch.Tensor]] = {self.out_id: [grad_output]}
        self.param_grads = {}
        pending_params: Dict[str, int] = {}      # parameter -> backward steps that still owe it a gradient

        def pending():
            for lst in grads.values():
                for o in lst:
                    yield o

        def private(g, own_entries=0):
            """A gradient that may be overwritten: cloned when a pending gradient other than its
            own `own_entries` entries lives in the same buffer."""
            same = sum(1 for o in pending()
                       if o.data_ptr() == g.data_ptr() and o.numel() == g.numel())
            return g.clone() if same > own_entries else g

        with torch.no_grad():
            for n in reversed(self.nodes):
                gl = grads.pop(n.id, None)
                if gl is None:
                    self._release(n.id)
                    continue
                op = self._ops[n.id]
                if len(gl) == 2:
                    g = (private(gl[0]), gl[1])      # the second one is only read
                else:
                    g = private(gl[0])
                del gl
                stored: list = []
                for d in _descriptors(op):
                    if isinstance(d, InputStorage):
                        for i in d.ids:
                            a = n.args[i]
                            if a.kind == 'node':
                                stored.append(self._value_for_backward(a.value))
                            elif a.kind == 'param':
                                stored.append(self._tensors[a.value])
                            elif a.kind == 'input':
                                stored.append(self._inputs[a.value])
                            else:
                                stored.append(a.value)
                    elif isinstance(d, OutputStorage):
                        stored.append(self._value_for_backward(n.id))
                    elif isinstance(d, IntermediateStorage):
                        stored.append(self._inter.pop(n.id))
                if n.op in ('aten::_convolution', 'aten::addmm'):
                    variant = max(self.choices[n.id].algorithm, 0)
                    op.algorithm = 20 + variant          # weight and input gradients in one call
                outs = op.backward(g, stored)
                del stored, g
                self._release(n.id)
                if not isinstance(outs, (tuple, list)):
                    outs = (outs,)
                deps = [a for a in n.args if a.kind in ('node', 'param', 'input')]
                if len(outs) != len(deps):
                    raise RuntimeError(f"node {n.id} ({n.op}) returned {len(outs)} gradients for {len(deps)} tensor arguments")
                for a, gi in zip(deps, outs):
                    if gi is None:
                        continue
                    if a.kind == 'node':
                        have = grads.get(a.value)
                        if have is None:
                            grads[a.value] = [gi]
                        elif len(have) == 1 and getattr(self._ops[a.value], 'accepts_grad_pair', False):
                            have.append(gi)
                        else:
                            have[0] = F.add(private(have[0], own_entries=1), gi, 1.0, inplace=True)
                    elif a.kind == 'param':
                        p = self._tensors[a.value]
                        if not p.requires_grad:
                            continue
                        if a.value in self.param_grads:
                            self.param_grads[a.value] = self.param_grads[a.value] + gi
                        else:
                            self.param_grads[a.value] = gi
                        pending_params[a.value] = pending_params.get(a.value, self._param_uses[a.value]) - 1
                        if pending_params[a.value] == 0:
                            del pending_params[a.value]
                            self._finish_param(a.value)
                del outs
        for name in list(pending_params):
            self._finish_param(name)
        self._vals = {}
        self._inter = {}

    def _finish_param(self, name: str) -> None:
        """The gradient of parameter `name` is complete: hand it to ``param.grad`` (accumulating,
        like ``param.backward(grad)`` in schedule.py:304-306) and tell ``on_param_grad``, which
        is how a data-parallel wrapper learns that a gradient bucket can be reduced while the
        rest of the backward still runs."""
        gi = self.param_grads[name]
        p = self._tensors[name]
        gi = gi.reshape(p.shape) if gi.shape != p.shape else gi
        if p.dim() != 4:
            gi = gi.contiguous()
        if p.grad is not None:
            p.grad.add_(gi)
        else:
            if gi.stride() != p.stride():
                # same strides as the parameter, so that foreach optimisers keep their fused
                # path: a 1x1 filter is the same memory either way, anything else is copied
                if p.dim() == 4 and p.shape[2] == 1 and p.shape[3] == 1 and gi.is_contiguous(
                        memory_format=torch.channels_last) and p.is_contiguous(memory_format=torch.channels_last):
                    gi = gi.as_strided(p.shape, p.stride())
                else:
                    gi = torch.empty_like(p).copy_(gi)
            p.grad = gi
        if self.on_param_grad is not None:
            self.on_param_grad(name, p)

    def _release(self, node_id: int) -> None:
        """Called after the backward step of `node_id`: drop every value whose last backward
        reader was this step."""
        for t, last in self._need.items():
            if last == node_id and self._vals.get(t) is not None and t != self.out_id:
                self._vals[t] = None
        if self._vals.get(node_id) is not None and self._need.get(node_id, node_id) >= node_id:
            self._vals[node_id] = None


class GraphedStep:
    """One whole training step (forward, loss, backward, optimiser) captured as a CUDA graph.

    The executor above is a Python loop over a few hundred nodes; it enqueues a ResNet-50 step in
    about 12 ms whatever the batch size, which is hidden behind a large batch and dominant for a
    small one.  The reference has the same per-node host loop (schedule.py:145-311) with a
    synchronisation per operator on top.  A captured step replays all launches from one host
    call; the batch and the target live in fixed buffers that ``__call__`` overwrites.

    ``criterion`` has ``forward(output, target) -> loss`` and ``backward() -> grad_output``
    (e.g. ``lm_ops.softmax.SoftmaxCrossEntropy``).  Gradients, the loss and every activation
    are allocated in the graph's private pool during capture and keep their addresses.  The
    schedule (what is kept, dropped, recomputed) is the runner's and is frozen by the capture.
    """

    def __init__(self, run: Runner, criterion, optimizer, example_input: torch.Tensor,
                 example_target: torch.Tensor, warmup: int = 3):
        if not example_input.is_cuda:
            raise RuntimeError("GraphedStep needs CUDA tensors")
        self.run, self.criterion, self.optimizer = run, criterion, optimizer
        self.params = [p for g in optimizer.param_groups for p in g['params']]
        self.input = example_input.clone()
        self.target = example_target.clone()
        # warm-up on a side stream (first calls raise shared-memory limits, fill workspaces and
        # create the optimiser's state: none of that may happen during capture)
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for _ in range(max(warmup, 1)):
                self._eager()
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph):
            self.loss = self._eager()

    def _eager(self) -> torch.Tensor:
        for p in self.params:
            p.grad = None
        out = self.run.forward(self.input)
        loss = self.criterion.forward(out, self.target)
        self.run.backward(self.criterion.backward())
        self.optimizer.step()
        return loss

    def __call__(self, input_: torch.Tensor, target: torch.Tensor) -> torch.Tensor:
        """Runs one step on this batch; returns the loss tensor (overwritten by the next call)."""
        self.input.copy_(input_, non_blocking=True)
        self.target.copy_(target, non_blocking=True)
        self.graph.replay()
        return self.loss
