"""Runs MONeT's own host code (graph extractor, SolverInfo, profiler, Schedule, MONeTWrapper)
on top of this operator library, unmodified, under a current PyTorch.

MONeT's Python side programs against ``monet.lm_ops`` only through
``lm_ops.list_ops(mode, aten_name)[p]()`` and the three storage descriptors
(schedule.py:67-90,111-142,229-272; solver_info.py:119-136,204-212,370-371;
meminfo.py:38-56).  ``activate()`` therefore

1. puts a MONeT checkout's host modules on ``sys.path`` (``baseline/install_ref.py`` installs
   them under ``baseline/_ref``; any checkout works, ``$MONET_ROOT`` overrides);
2. registers this package's ``lm_ops`` as the module ``monet.lm_ops`` *before* MONeT's own is
   imported (that one JIT-compiles CUDA sources for PyTorch 1.5 / cuDNN 7 at import);
3. supplies what the 2020 code expects and a 2025 PyTorch no longer has:
   ``torch._C.Node.__getitem__`` (graph.py:139), a ``cvxpy`` module object when cvxpy is not
   installed (cvxpy_solver.py:1 is imported by schedule.py:7 for the ``Solution`` class only;
   solving goes through ``monet_b200.solver``), and a post-pass over ``Graph.create``'s result
   (``normalize_graph``) for three changes in what ``torch.jit`` traces today.

It returns the imported MONeT modules.  Nothing here touches a GPU.
"""
from __future__ import annotations

import importlib
import os
import sys
import types
from pathlib import Path
from typing import Optional

import torch

_REPO = Path(__file__).resolve().parent.parent
_DEFAULT_ROOT = _REPO / "baseline" / "_ref"
_HOST_MODULES = ("graph", "solver_info", "meminfo", "cvxpy_solver", "schedule", "monet_wrapper")
_active: Optional[types.SimpleNamespace] = None


def find_root(root=None) -> Path:
    """The directory that holds ``monet/schedule.py``: the argument, ``$MONET_ROOT`` or the
    in-tree install location."""
    for cand in (root, os.environ.get("MONET_ROOT"), _DEFAULT_ROOT):
        if cand and (Path(cand) / "monet" / "schedule.py").exists():
            return Path(cand)
    raise FileNotFoundError(
        "no MONeT host code found: run `python baseline/install_ref.py <MONeT checkout>` "
        "or set MONET_ROOT")


def _install_torch_shims() -> None:
    # graph.py:139 reads a constant node's payload as n['value']
    if not hasattr(torch._C.Node, "__getitem__"):
        def _getitem(self, key):
            return getattr(self, self.kindOf(key))(key)
        torch._C.Node.__getitem__ = _getitem
    # schedule.py:339 resets the allocator's peak with the pre-1.6 name
    if not hasattr(torch.cuda, "reset_max_memory_allocated"):
        torch.cuda.reset_max_memory_allocated = torch.cuda.reset_peak_memory_stats


def _install_cvxpy_placeholder() -> None:
    try:
        import cvxpy  # noqa: F401
        return
    except Exception:
        pass

    class _Missing(types.ModuleType):
        def __getattr__(self, name):
            if name.startswith("__"):
                raise AttributeError(name)
            raise ImportError("cvxpy is not installed: solve with monet_b200.solver.solve "
                              "(same ILP through scipy.optimize.milp / HiGHS)")
    sys.modules["cvxpy"] = _Missing("cvxpy")


def normalize_graph(graph):
    """Brings a graph traced by a current ``torch.jit`` to what MONeT's host code assumes
    (the shapes of the PyTorch-1.5 trace it was written for).  Returns a new graph.

    * every BatchNorm in training mode now contributes ``aten::add_(num_batches_tracked, 1)``,
      a node without backward.  ``SolverInfo.extract`` gives solver ids to ``has_backward``
      nodes only (solver_info.py:107-109) while ``Schedule.init_schedule`` looks up every
      compute node (schedule.py:70): such nodes are dropped (the counter is bookkeeping of the
      module, not part of the differentiated function) and the rest renumbered;
    * ``nn.Linear`` is traced as one ``aten::linear(x, W, b)`` instead of ``aten::t`` +
      ``aten::addmm(b, x, Wt, 1, 1)``.  The solver and executor special-case the *name*
      ``aten::addmm`` (two backward steps; schedule.py:123,220; solver_info.py:164,190,233),
      and graph.py:146-150 already hands addmm the un-transposed parameter, so the node is
      rewritten to ``aten::addmm`` with arguments ``(b, x, W, 1, 1)``;
    * the output of ``aten::_convolution`` reports ``requires_grad() == False`` in the trace;
      ``SolverInfo.extract`` asserts that an edge between compute nodes carries a gradient
      (solver_info.py:116): such edges get ``requires_grad = True`` when the producer has a
      backward.
    """
    g = importlib.import_module("monet.graph")
    ComputeNode = g.ComputeNode
    old = graph.nodes
    used = set()
    for n in old:
        if isinstance(n, ComputeNode) and n.has_backward:
            used.update(i for i, _ in n.dependencies)
    keep = []
    for k, n in enumerate(old):
        if isinstance(n, ComputeNode) and not n.has_backward and n.op != "aten::t" and k not in used:
            continue
        keep.append(k)
    new_id = {k: i for i, k in enumerate(keep)}

    out = g.Graph()
    for k in keep:
        n = old[k]
        if not isinstance(n, ComputeNode):
            out._add_node(n)
            continue
        args = []
        for a in n.args:
            if isinstance(a, ComputeNode.D):
                src = old[a.index]
                rg = bool(a.requires_grad)
                if isinstance(src, ComputeNode) and src.has_backward:
                    rg = True
                args.append(ComputeNode.D(new_id[a.index], rg))
            else:
                args.append(a)
        op = n.op
        if op == "aten::linear":
            if len(args) != 3 or not isinstance(args[2], ComputeNode.D):
                raise NotImplementedError("aten::linear without a bias parameter")
            op = "aten::addmm"
            args = [args[2], args[0], args[1], ComputeNode.V(1), ComputeNode.V(1)]
        out._add_node(ComputeNode(n.shape, new_id[k], op, args, n.has_backward, n.is_depthwise))
    for o in graph._outputs:
        out._add_output(new_id[o])
    return out


def activate(root=None) -> types.SimpleNamespace:
    """Import MONeT's host modules over this operator library (idempotent).

    Returns a namespace with ``root`` and the modules ``graph``, ``solver_info``, ``meminfo``,
    ``cvxpy_solver``, ``schedule``, ``monet_wrapper`` and ``lm_ops`` (this package's)."""
    global _active
    if _active is not None:
        return _active
    root = find_root(root)
    if str(root) not in sys.path:
        sys.path.insert(0, str(root))
    _install_torch_shims()
    _install_cvxpy_placeholder()

    from . import lm_ops as ours
    from .lm_ops import softmax as _softmax  # noqa: F401  (aten::softmax / log_softmax)
    import monet  # a namespace package: the checkout has no monet/__init__.py
    if (root / "monet" / "lm_ops").exists() and "monet.lm_ops" in sys.modules \
            and sys.modules["monet.lm_ops"] is not ours:
        raise RuntimeError("MONeT's own monet.lm_ops is already imported in this process")
    sys.modules["monet.lm_ops"] = ours
    for sub in ("base", "conv", "relu", "elementary", "pool", "linear", "bn", "cat", "hardtanh",
                "funcs", "softmax"):
        sys.modules["monet.lm_ops." + sub] = importlib.import_module(f"{ours.__name__}.{sub}")
    monet.lm_ops = ours

    mods = {name: importlib.import_module("monet." + name) for name in _HOST_MODULES}
    graph_mod = mods["graph"]
    if not getattr(graph_mod.Graph, "_monet_b200_normalized", False):
        original = graph_mod.Graph.create.__func__

        def create(cls, model, input_shape=(3, 224, 224)):
            return normalize_graph(original(cls, model, input_shape))

        graph_mod.Graph.create = classmethod(create)
        graph_mod.Graph._monet_b200_normalized = True
    _patch_inplace_info(mods["solver_info"])
    _active = types.SimpleNamespace(root=root, lm_ops=ours, **mods)
    return _active


def _patch_inplace_info(solver_info_mod) -> None:
    """``SolverInfo.get_inplace_info`` (solver_info.py:436-448) records, for an operator that can
    run in place, the LAST of its inputs nobody reads afterwards as the tensor it overwrites;
    the executor and every operator overwrite the FIRST input (schedule.py:175-179,
    funcs.py:47-50).  For ``aten::add_(a, b)`` with both inputs dying at the add the ILP then
    believes ``b`` is overwritten and may keep ``a`` stored for a backward while the add
    destroys it.  After the original runs, the table is rewritten to name the first input, and
    operators whose first input has a later reader are taken out of it."""
    cls = solver_info_mod.SolverInfo
    if getattr(cls, "_monet_b200_inplace_fixed", False):
        return
    original = cls.get_inplace_info

    def get_inplace_info(self):
        original(self)
        if not self.do_inplace:
            return
        for v in [v for v in list(self.inplace_list) if not isinstance(self.nodes[v], solver_info_mod.IntNode)]:
            inputs = self.nodes[v].args[0]
            first = inputs[0] if inputs else None
            ok = first is not None and self.nodes[first].last_used == v
            related = [v] + [i for (_, i) in getattr(self.nodes[v], "intermediates", [])]
            for k in related:
                if k in self.inplace_list:
                    if ok:
                        self.inplace_list[k] = first
                    else:
                        del self.inplace_list[k]

    cls.get_inplace_info = get_inplace_info
    cls._monet_b200_inplace_fixed = True


# ----------------------------------------------------------------------- solver info
class _in_dir:
    """MONeT reads and writes ``../data/*.pkl`` relative to the working directory
    (solver_info.py:152,347; cvxpy_solver.py:323): run it from ``<workdir>/monet``."""

    def __init__(self, workdir):
        self.workdir = Path(workdir)

    def __enter__(self):
        (self.workdir / "data").mkdir(parents=True, exist_ok=True)
        (self.workdir / "monet").mkdir(parents=True, exist_ok=True)
        self.prev = os.getcwd()
        os.chdir(self.workdir / "monet")
        return self

    def __exit__(self, *exc):
        os.chdir(self.prev)


def wrap_mobilenet(model):
    """The Sequential form MONeT traces MobileNetV2 in (monet_wrapper.py:27-31)."""
    if model._get_name() == "MobileNetV2":
        return torch.nn.Sequential(model.features, torch.nn.AdaptiveAvgPool2d((1, 1)),
                                   torch.nn.Flatten(start_dim=1), model.classifier[0],
                                   model.classifier[1])
    return model


def build_solver_info(model, batch: int, model_name: str, mode: str, input_shape=(3, 224, 224),
                      workdir=None, profile: bool = True, costs=None, profiler: str = "reference"):
    """(graph, solver_info) for ``model`` through MONeT's own ``Graph.create`` and
    ``SolverInfo.extract`` (solver_info.py:103-155).

    ``profile=True`` is MONeT's behaviour: every implementation of every operator is run on
    the current CUDA device by ``meminfo`` / ``computeinfo`` (meminfo.py) to fill the
    workspace-memory and run-time tables; ``model`` must then live on that device
    (``profiler="events"`` substitutes ``monet_b200.profiler``'s functions of the same
    signature: CUDA-event timing on channels_last activations).  With ``profile=False`` the tables are filled by ``costs(si, graph)`` instead (default:
    ``monet_b200.solver.estimate_costs``, a bytes-and-flops model), which needs no GPU.
    """
    ref = activate()
    import copy
    cpu_model = wrap_mobilenet(copy.deepcopy(model)).cpu()
    graph = ref.graph.Graph.create(cpu_model, input_shape)
    del cpu_model
    si = ref.solver_info.SolverInfo(batch, model_name, mode)
    workdir = (Path(workdir) if workdir is not None else ref.root).resolve()
    with _in_dir(workdir):
        cached = (workdir / "data" / f"cost_{si.data_path}.pkl").is_file()
        if profile and cached:
            # get_workspace_cost() reads the tables of an earlier profiling run from
            # ../data/cost_*.pkl (solver_info.py:347-360): no GPU needed
            si.extract(graph)
        elif profile:
            m = wrap_mobilenet(model)
            dev = next(m.parameters()).device
            if dev.type != "cuda":
                raise RuntimeError("profiling the cost tables needs the model on a CUDA device")
            x = torch.randn((batch,) + tuple(input_shape), device=dev)
            from . import profiler as own
            if profiler == "events":
                own.install(ref)
            elif profiler != "reference":
                raise ValueError(f"unknown profiler {profiler!r}")
            try:
                si.extract(graph, x, *list(m.state_dict(keep_vars=True).values()))
            finally:
                own.uninstall(ref)
        else:
            if costs is None:
                from .solver import estimate_costs as costs

            cls = type(si)
            original = cls.get_workspace_cost
            # patched on the class, not the instance: extract() pickles the instance at its end
            cls.get_workspace_cost = lambda self, graph_, *unused: costs(self, graph_)
            try:
                si.extract(graph)
            finally:
                cls.get_workspace_cost = original
    return graph, si


def save_solution(si, solution, path) -> Path:
    """Pickle ``[si, solution]`` the way cvxpy_solver.py:330-333 does, so that
    ``MONeTWrapper(model, path, input_shape)`` / ``create_schedule`` load it."""
    import pickle
    path = Path(path)
    path.parent.mkdir(parents=True, exist_ok=True)
    with open(path, "wb") as f:
        pickle.dump([si, solution], f)
    return path


def make_schedule(graph, si, solution):
    """``Schedule(graph, si)`` initialised with ``solution`` (schedule.py:326-346 without the
    file round trip)."""
    ref = activate()
    sched = ref.schedule.Schedule(graph, si)
    sched.init_schedule(solution, si.mode)
    return sched
