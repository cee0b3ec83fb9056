"""MONeT's joint checkpointing / operator-selection ILP through ``scipy.optimize.milp`` (HiGHS).

The reference states the ILP in cvxpy and hands it to Gurobi or CBC
(monet/cvxpy_solver.py:54-334, backend call :299-311); none of the three is needed here.
``solve(si, budget_gb)`` builds the same program directly as a sparse constraint matrix from a
``SolverInfo`` (monet/solver_info.py) and returns the reference's own ``Solution`` object
(cvxpy_solver.py:14-25), so ``Schedule.init_schedule`` / ``MONeTWrapper`` consume it unchanged
and ``reference_host.save_solution`` writes the pickle ``create_schedule`` loads.

Variables and constraints follow cvxpy_solver.py one for one (R recompute, S stored, P present,
M backward implementation, SM = S*M, RF convolution variant, IP in place; correctness rows
:139-163, variant rows :165-177, the three memory rows :179-258, objective :260-293).  Four
rewritings keep the optimum and make the program small enough for an open-source solver:

* *Dead columns.*  At time t >= 1 the backward of forward node f runs; forward tensors with
  an index above everything a remaining backward step reads can be neither useful nor free,
  so their R, S, P, IP are fixed to 0 (not created).
* *P only where it can differ from R.*  P[t,u] is a free variable only when u is the input an
  in-place operator may overwrite (:111-113); elsewhere P = R is optimal (P only relaxes rows).
* *One backward implementation.*  ``sum_p M[t,p] >= 1`` (:146) is written ``== 1``: a second
  selected implementation only adds cost and memory.  With that, the stored-tensor term of the
  backward memory row, ``sum_p sum_k SM[p][t,k] ram[k] [k not a dependency of p]`` (:249-253),
  equals ``sum_k S[t+1,k] ram[k] - sum_p sum_{k in deps_p} SM[p][t,k] ram[k]``, so SM is needed
  only for (p, t, k) with k a dependency of implementation p at time t.
* *Running sums.*  The forward rows (:190-231) hold, for every (t, j), the memory of all
  tensors stored while node j is recomputed: a sum over all V nodes.  Consecutive j differ by
  one term, so a continuous variable U[t,j] carries the sum
  (``U[t,j+1] = U[t,j] - ram[j] S[t,j] + ram[j] S[t+1,j]``): three non-zeros per row instead of V.

``check_solution`` re-evaluates the reference's rows literally (no rewriting) on a solution and
is what the tests hold ``solve`` and ``hand_solution`` to.

``estimate_costs`` fills the cost tables of a ``SolverInfo`` from a bytes-and-flops model so
that a schedule can be solved on a machine without a GPU; the measured tables come from
MONeT's profiler (``reference_host.build_solver_info(profile=True)``).
"""
from __future__ import annotations

import math
import time
from typing import Dict, List, Optional

import numpy as np

CPU_GCD_MULTIPLIER = 100      # cvxpy_solver.py:8-12
MEM_GCD_MULTIPLIER = 1
GB_TO_KB = 1024 * 1024
Y = 3                         # backward implementations per node the ILP has room for (:59)


# --------------------------------------------------------------------------- cost model
def _numel(shape, bs):
    n = 1
    for s in shape:
        n *= (bs if s == -1 else int(s))
    return float(abs(n))


def estimate_costs(si, graph, hbm_gbs: float = 6400.0, tensor_tflops: float = 400.0) -> None:
    """Fills ``workspace_mem`` (MB) / ``workspace_compute`` (ms) and their recompute / in-place
    twins for every solver node, in the layout ``SolverInfo.get_workspace_cost`` produces
    (solver_info.py:362-424): one entry per implementation (or per convolution variant in the
    ``conv`` modes).  Times are algorithmic HBM bytes over ``hbm_gbs`` plus flops over
    ``tensor_tflops``; workspaces are the scratch the operators allocate."""
    from . import lm_ops
    ref_si = __import__("monet.solver_info", fromlist=["BwdNode"])
    BwdNode, IntNode = ref_si.BwdNode, ref_si.IntNode
    bs = si.bs
    ms_per_byte = 1e3 / (hbm_gbs * 1e9)
    ms_per_flop = 1e3 / (tensor_tflops * 1e12)

    def conv_cost(n):
        e_out = _numel(n.shape, bs)
        w = graph.nodes[n.args[1].index].shape
        e_in = _numel(graph.nodes[n.args[0].index].shape, bs)
        byts = 4 * (e_in + e_out + float(np.prod(w)))
        flops = 2.0 * e_out * w[1] * w[2] * w[3]
        return max(byts * ms_per_byte, flops * ms_per_flop) + 0.004

    # bytes per output element: (forward, backward) per implementation
    fwd_b = {"aten::batch_norm": 12, "aten::relu": 8, "aten::relu_": 8, "aten::hardtanh": 8,
             "aten::hardtanh_": 8, "aten::add": 12, "aten::add_": 12, "aten::max_pool2d": 20,
             "aten::cat": 8, "aten::adaptive_avg_pool2d": 8, "aten::dropout": 12}
    bwd_b = {"aten::batch_norm": [20, 20], "aten::relu": [12, 12, 8.2], "aten::relu_": [12, 12, 8.2],
             "aten::hardtanh": [12, 12], "aten::hardtanh_": [12, 12], "aten::add": [0.1], "aten::add_": [0.1],
             "aten::max_pool2d": [40, 20], "aten::cat": [8], "aten::adaptive_avg_pool2d": [8],
             "aten::dropout": [12]}

    for i in si.nodes:
        for name in ("workspace_mem", "workspace_compute", "recompute_workspace_mem",
                     "recompute_workspace_compute", "inplace_workspace_mem", "inplace_workspace_compute"):
            setattr(si.nodes[i], name, [])

    for i in sorted(si.nodes.keys(), reverse=True):
        node = si.nodes[i]
        if isinstance(node, BwdNode):
            n = node.fwd_node
            f = si.bwd_to_fwd[i]
            fnode = si.nodes[f]
            impls = lm_ops.list_ops(si.mode, n.op)
            e_out = _numel(n.shape, bs)
            dense_conv = n.op == "aten::_convolution" and not n.is_depthwise
            if si.select_conv_algo and f in si.conv_list:
                t = conv_cost(n)
                count = impls[0].n_bwd_ip_algos() if node.bwd_op == "ip_grad" else impls[0].n_bwd_wt_algos()
                node.workspace_mem = [0.0] * count
                node.workspace_compute = [t * (1.0 + 0.05 * c) for c in range(count)]
                if node.bwd_op != "ip_grad":
                    cf = impls[0].n_fwd_algos()
                    fnode.workspace_mem = [0.0] * cf
                    fnode.workspace_compute = [t] * cf
                continue
            for p, _ in enumerate(impls):
                if dense_conv or n.op == "aten::addmm":
                    if n.op == "aten::addmm":
                        w = graph.nodes[n.args[2].index].shape
                        t = max(4 * float(np.prod(w)) * ms_per_byte,
                                2.0 * e_out * w[1] * ms_per_flop * 8) + 0.004
                    else:
                        t = conv_cost(n)
                    bt, ft = t, t
                else:
                    b = bwd_b.get(n.op, [8])
                    bt = b[min(p, len(b) - 1)] * e_out * ms_per_byte + 0.004
                    ft = fwd_b.get(n.op, 8) * e_out * ms_per_byte + 0.004
                    if n.op in ("aten::relu", "aten::relu_") and p == 2:
                        ft *= 1.02        # the mask is written beside the output
                    if n.op == "aten::_convolution":       # depthwise
                        ft = bt = 8 * e_out * ms_per_byte + 0.004
                        bt *= 2
                node.workspace_mem.append(0.0)
                node.workspace_compute.append(bt)
                split_ip = (dense_conv or n.op == "aten::addmm") and node.bwd_op == "ip_grad"
                if si.do_inplace and f in si.inplace_list:
                    fnode.workspace_mem.append(0.0)
                    fnode.workspace_compute.append(ft)
                    fnode.inplace_workspace_mem.append(-e_out * 4 / 2 ** 20)
                    fnode.inplace_workspace_compute.append(ft)
                elif not split_ip:
                    if n.op == "aten::batch_norm":
                        fnode.recompute_workspace_mem.append(0.0)
                        fnode.recompute_workspace_compute.append(8 * e_out * ms_per_byte + 0.004)
                    fnode.workspace_mem.append(0.0)
                    fnode.workspace_compute.append(ft)
        elif isinstance(node, IntNode):
            parent = si.nodes[node.solver_parent_id]
            p = node.op_idx
            node.workspace_mem = [parent.workspace_mem[p]]
            node.workspace_compute = [parent.workspace_compute[p] - parent.workspace_compute[0]]
            if si.do_inplace and node.solver_parent_id in si.inplace_list:
                node.inplace_workspace_mem = [parent.inplace_workspace_mem[p]]
                node.inplace_workspace_compute = [parent.inplace_workspace_compute[p]
                                                  - parent.inplace_workspace_compute[0]]
        elif "loss::" in node.op:
            node.workspace_mem, node.workspace_compute = [0], [0]
    for i in si.nodes:
        node = si.nodes[i]
        if not node.recompute_workspace_mem:
            node.recompute_workspace_mem = node.workspace_mem
            node.recompute_workspace_compute = node.workspace_compute
        if not node.inplace_workspace_mem:
            node.inplace_workspace_mem = node.workspace_mem
            node.inplace_workspace_compute = node.workspace_compute


# ------------------------------------------------------------------- shared quantities
class _Tables:
    """The integer tables cvxpy_solver.Model.__init__ derives from a SolverInfo (:33-52)."""

    def __init__(self, si):
        self.si = si
        nodes = si.nodes
        self.V = si.loss + 1
        self.T = len(nodes) - si.loss
        self.ram = np.array([math.ceil(nodes[i].mem * MEM_GCD_MULTIPLIER / 1024) for i in nodes], dtype=np.float64)
        up = lambda vals: [math.ceil(v * CPU_GCD_MULTIPLIER) for v in vals]      # noqa: E731
        self.cpu = {i: up(nodes[i].workspace_compute) for i in nodes}
        self.cpu_recompute = {i: up(nodes[i].recompute_workspace_compute) for i in nodes}
        self.cpu_inplace = {i: up(nodes[i].inplace_workspace_compute) for i in nodes}
        ref_si = __import__("monet.solver_info", fromlist=["IntNode"])
        self.is_int = [isinstance(nodes[i], ref_si.IntNode) for i in range(self.V)]

    def cmem(self, j, recompute=False, inplace=False):
        n = self.si.nodes[j]
        vals = n.inplace_workspace_mem if inplace else (n.recompute_workspace_mem if recompute else n.workspace_mem)
        return [math.ceil(v * MEM_GCD_MULTIPLIER * 1024) for v in vals]

    def local_memory(self, j):
        return math.ceil(self.si.nodes[j].local_memory * MEM_GCD_MULTIPLIER / 1024)

    def fixed_ram(self, j):
        return math.ceil(self.si.nodes[j].fixed_mem * MEM_GCD_MULTIPLIER / 1024)

    def bwd_node(self, t):
        return self.si.nodes[self.V + t - 1]

    def fwd_deps(self, t, p):
        """Forward solver nodes implementation p of the step at time t reads (args < V)."""
        node = self.bwd_node(t)
        if p >= len(node.args):
            return []
        return [j for j in node.args[p] if j < self.V]

    def horizon(self):
        """hi[t]: largest forward index any step at time >= t still reads (t >= 1)."""
        T, V = self.T, self.V
        hi = [V - 1] * (T + 1)
        run = -1
        for t in range(T - 1, 0, -1):
            node = self.bwd_node(t)
            for p in range(len(node.args)):
                for j in self.fwd_deps(t, p):
                    run = max(run, j)
            hi[t] = run
        hi[0] = V - 1
        hi[T] = -1
        return hi


def _solution_class():
    return __import__("monet.cvxpy_solver", fromlist=["Solution"]).Solution


# ----------------------------------------------------------------------------- the ILP
class _Program:
    """Sparse rows ``lo <= a.x <= up`` over named variables."""

    def __init__(self):
        self.nvar = 0
        self.integral: List[int] = []
        self.ub: List[float] = []
        self.rows_i: List[int] = []
        self.rows_j: List[int] = []
        self.rows_v: List[float] = []
        self.lo: List[float] = []
        self.up: List[float] = []
        self.cost: Dict[int, float] = {}

    def var(self, integral=True, ub=1.0) -> int:
        self.integral.append(1 if integral else 0)
        self.ub.append(ub)
        self.nvar += 1
        return self.nvar - 1

    def row(self, terms, lo=-np.inf, up=np.inf):
        """terms: iterable of (var index or None, coefficient); None entries are constants 0."""
        r = len(self.lo)
        acc: Dict[int, float] = {}
        for v, c in terms:
            if v is None or c == 0:
                continue
            acc[v] = acc.get(v, 0.0) + c
        for v, c in acc.items():
            if c != 0:
                self.rows_i.append(r); self.rows_j.append(v); self.rows_v.append(c)
        self.lo.append(lo); self.up.append(up)

    def add_cost(self, v, c):
        if v is not None and c:
            self.cost[v] = self.cost.get(v, 0.0) + c


def solve(si, budget_gb: float, time_limit: float = 3600.0, mip_rel_gap: float = 0.01,
          verbose: bool = False):
    """Solves MONeT's ILP for ``si`` under ``budget_gb`` and returns the reference's
    ``Solution`` (r, s, m, rf, ip, p as rounded numpy arrays, solve_time, fwd / bwd / total
    expected cost).  Raises ``ValueError("Model infeasible")`` like cvxpy_solver.py:327-328,
    and ``RuntimeError`` when HiGHS finds no feasible point inside ``time_limit``."""
    from scipy.optimize import Bounds, LinearConstraint, milp
    from scipy.sparse import csr_matrix

    tb = _Tables(si)
    V, T, ram = tb.V, tb.T, tb.ram
    budget = budget_gb * MEM_GCD_MULTIPLIER * GB_TO_KB
    hi = tb.horizon()
    inpl = si.do_inplace
    inplace_list = dict(si.inplace_list) if inpl else {}
    sources = set(inplace_list[v] for v in inplace_list if not tb.is_int[v]) if inpl else set()
    conv_list = dict(si.conv_list) if si.select_conv_algo else {}
    n_algos = si.num_conv_algos if si.select_conv_algo else 0

    pr = _Program()
    R = [[None] * V for _ in range(T)]
    S = [[None] * V for _ in range(T + 1)]
    P = [[None] * V for _ in range(T)]
    IP = [[None] * V for _ in range(T)]
    for t in range(T):
        for j in range(hi[t] + 1):
            R[t][j] = pr.var()
            if j in sources:
                P[t][j] = pr.var()
            if j in inplace_list:
                IP[t][j] = pr.var()
    for t in range(1, T + 1):                 # S[0] = 0 (:120).  S[t+1, j] is what the backward at
        for j in range(hi[t - 1] + 1):        # time t reads (:155), so it lives while j <= hi[t]
            S[t][j] = pr.var()
    Pv = lambda t, j: P[t][j] if j in sources else R[t][j]        # noqa: E731
    M = [[None] * Y for _ in range(T)]
    for t in range(T):
        paths = 1 if t == 0 else len(tb.bwd_node(t).args)
        for p in range(min(paths, Y)):
            M[t][p] = pr.var()
        pr.row([(M[t][p], 1.0) for p in range(Y)], 1.0, 1.0)     # :128-135,146 (as equality)
    SM: Dict[tuple, int] = {}
    for t in range(T):
        for p in range(Y):
            if M[t][p] is None:
                continue
            for k in tb.fwd_deps(t, p):
                if S[t + 1][k] is None:
                    continue
                v = SM[(p, t, k)] = pr.var()
                pr.row([(v, 1.0), (M[t][p], -1.0), (S[t + 1][k], -1.0)], -1.0, np.inf)   # :140-143
                pr.row([(v, 1.0), (M[t][p], -1.0)], -np.inf, 0.0)
                pr.row([(v, 1.0), (S[t + 1][k], -1.0)], -np.inf, 0.0)
    RF: Dict[tuple, int] = {}
    for i, ci in conv_list.items():
        valid = [c for c in range(n_algos) if c < len(tb.cpu[i]) and tb.cpu[i][c] >= 0]     # :137-141
        if i < si.loss:
            for t in range(T):
                if R[t][i] is None:
                    continue
                for c in valid:
                    RF[(c, t, ci)] = pr.var()
                pr.row([(RF[(c, t, ci)], 1.0) for c in valid] + [(R[t][i], -1.0)], 0.0, np.inf)   # :168
        else:
            t = i + 1 - V
            for c in valid:
                RF[(c, t, ci)] = pr.var()
            pr.row([(RF[(c, t, ci)], 1.0) for c in valid], 1.0, np.inf)                          # :171

    # ---- correctness
    for j in range(V):
        if not tb.is_int[j]:
            pr.row([(R[0][j], 1.0)], 1.0, 1.0)                                                   # :123-125
    if inpl:
        for t in range(T):
            for j in range(V):
                if P[t][j] is not None:
                    pr.row([(P[t][j], 1.0), (R[t][j], -1.0)], -np.inf, 0.0)                      # :104
                if IP[t][j] is not None:
                    pr.row([(IP[t][j], 1.0), (R[t][j], -1.0)], -np.inf, 0.0)                     # :105
        for v, u in inplace_list.items():
            if tb.is_int[v]:
                continue
            for t in range(T):
                if IP[t][v] is None:
                    continue
                pr.row([(P[t][u], 1.0), (R[t][u], -1.0), (IP[t][v], 2.0)], 0.0, np.inf)          # :115
                pr.row([(P[t][u], 1.0), (IP[t][v], 2.0)], -np.inf, 2.0)                          # :116
                if S[t + 1][u] is not None:
                    pr.row([(S[t + 1][u], 1.0), (IP[t][v], 2.0)], -np.inf, 2.0)                  # :117
    for t in range(T):
        for j in range(V):
            if S[t + 1][j] is not None:                                                          # :145
                pr.row([(S[t + 1][j], 1.0), (S[t][j], -1.0), (Pv(t, j), -1.0)], -np.inf, 0.0)
    for (u, v, p) in si.edge_list:                                                               # :150-156
        if u < V and v < V:
            for t in range(T):
                if R[t][v] is not None:
                    pr.row([(R[t][v], 1.0), (R[t][u], -1.0), (S[t][u], -1.0)], -np.inf, 0.0)
        elif u < V and v >= V:
            t = v + 1 - V
            if p < Y and M[t][p] is not None:
                pr.row([(M[t][p], 1.0), (Pv(t, u), -1.0), (S[t + 1][u], -1.0)], -np.inf, 0.0)
    for i in range(V):                                                                            # :158-164
        if si.nodes[i].has_intermediates:
            for (_, intid) in si.nodes[i].intermediates:
                for t in range(T):
                    if R[t][intid] is None:
                        continue
                    pr.row([(R[t][intid], 1.0), (R[t][i], -1.0)], -np.inf, 0.0)
                    if inpl and i in inplace_list and IP[t][intid] is not None:
                        pr.row([(IP[t][intid], 1.0), (IP[t][i], -1.0), (R[t][intid], -1.0)], -1.0, np.inf)
                        pr.row([(IP[t][intid], 1.0), (IP[t][i], -1.0)], -np.inf, 0.0)

    # ---- memory while (re)computing forward node j at time t (:179-231)
    keep_so_far = [[[] for _ in range(Y)] for _ in range(T)]       # deps of (t, p) with index < j
    gradm = [0.0] * T
    for t in range(T):
        bk = V + t - 1
        gradm[t] = (tb.local_memory(bk) if t != 0 else 0) + tb.fixed_ram(bk - 1)
    dep_at = [[set(tb.fwd_deps(t, p)) if M[t][p] is not None else set() for p in range(Y)] for t in range(T)]
    U = [None] * T
    for t in range(T):
        U[t] = pr.var(integral=False, ub=np.inf)
        pr.row([(U[t], 1.0)] + [(S[t][k], -ram[k]) for k in range(V)], 0.0, 0.0)   # U[t,0] = sum_k S[t,k] ram[k]
    for j in range(V):
        ws = tb.cmem(j)
        ws_re = tb.cmem(j, recompute=True)
        ws_ip = tb.cmem(j, inplace=True)
        local = tb.local_memory(j)
        local_set = list(si.nodes[j].local_tensors)
        for t in range(T):
            if R[t][j] is None and j != hi[t] + 1:
                continue          # rows for j > hi[t] + 1 repeat the row at hi[t] + 1
            keep = []
            for p in range(Y):
                for k in keep_so_far[t][p]:
                    keep.append((M[t][p], ram[k]))
                    keep.append((SM.get((p, t, k)), -ram[k]))
            # checkpoint row (:222-224)
            pr.row([(U[t], 1.0)] + keep, -np.inf, budget - gradm[t])
            if R[t][j] is None:
                continue
            # recomputation row (:226-228)
            w = ws if t == 0 else ws_re
            terms = [(U[t], 1.0), (S[t][j], -ram[j])] + keep
            for u in local_set:
                if u > j:
                    terms.append((S[t][u], -ram[u]))
                elif u < j:
                    terms.append((S[t + 1][u], -ram[u]))
            if conv_list and j in conv_list:
                for c in range(len(w)):
                    terms.append((RF.get((c, t, conv_list[j])), float(w[c])))
            elif inpl and j in inplace_list:
                terms.append((IP[t][j], float(ws_ip[0] - w[0])))
                terms.append((R[t][j], float(w[0])))
            else:
                terms.append((R[t][j], float(w[0])))
            terms.append((R[t][j], float(ram[j] + local)))
            pr.row(terms, -np.inf, budget - gradm[t])
        # advance the running sums to j + 1 and the kept dependencies past j
        for t in range(T):
            if S[t][j] is not None or S[t + 1][j] is not None:
                nu = pr.var(integral=False, ub=np.inf)
                pr.row([(nu, 1.0), (U[t], -1.0), (S[t][j], ram[j]), (S[t + 1][j], -ram[j])], 0.0, 0.0)
                U[t] = nu
            for p in range(Y):
                if j in dep_at[t][p]:
                    keep_so_far[t][p].append(j)
    # after the loop U[t] = sum_k S[t+1,k] ram[k]

    # ---- memory during the backward step at time t (:233-258)
    for t in range(1, T):
        bk = V + t - 1
        node = si.nodes[bk]
        const = tb.local_memory(bk) + tb.fixed_ram(bk) + ram[bk]
        terms = [(U[t], 1.0)]
        wmem = tb.cmem(bk)
        if conv_list and bk in conv_list:
            for c in range(len(wmem)):
                terms.append((RF.get((c, t, conv_list[bk])), float(wmem[c])))
        else:
            for p in range(min(len(node.args), Y)):
                if p < len(wmem):
                    terms.append((M[t][p], float(wmem[p])))
        for p in range(min(len(node.args), Y)):
            for k in dep_at[t][p]:
                terms.append((M[t][p], ram[k]))
                terms.append((SM.get((p, t, k)), -ram[k]))
        pr.row(terms, -np.inf, budget - const)

    # ---- objective (:260-293)
    for i in range(V):
        if conv_list and i in conv_list:
            for t in range(T):
                for c in range(len(tb.cpu[i])):
                    pr.add_cost(RF.get((c, t, conv_list[i])), tb.cpu[i][c])
            continue
        pr.add_cost(R[0][i], tb.cpu[i][0])
        for t in range(1, T):
            pr.add_cost(R[t][i], tb.cpu_recompute[i][0])
    if inpl:
        for i in inplace_list:
            for t in range(T):
                pr.add_cost(IP[t][i], tb.cpu_inplace[i][0] - tb.cpu[i][0])
    for t in range(T):
        bk = V + t - 1
        if conv_list and bk in conv_list:
            for c in range(len(tb.cpu[bk])):
                pr.add_cost(RF.get((c, t, conv_list[bk])), tb.cpu[bk][c])
        else:
            for p in range(Y):
                if p < len(tb.cpu[bk]):
                    pr.add_cost(M[t][p], tb.cpu[bk][p])

    c = np.zeros(pr.nvar)
    for v, w in pr.cost.items():
        c[v] = w
    A = csr_matrix((pr.rows_v, (pr.rows_i, pr.rows_j)), shape=(len(pr.lo), pr.nvar))
    t0 = time.time()
    res = milp(c, constraints=LinearConstraint(A, np.array(pr.lo), np.array(pr.up)),
               integrality=np.array(pr.integral), bounds=Bounds(np.zeros(pr.nvar), np.array(pr.ub)),
               options={"time_limit": float(time_limit), "disp": bool(verbose), "mip_rel_gap": float(mip_rel_gap)})
    solve_time = time.time() - t0
    if res.status == 2:
        raise ValueError("Model infeasible")
    if res.x is None:
        raise RuntimeError(f"no feasible schedule found within {time_limit:.0f} s: {res.message}")
    x = np.around(res.x)

    def val(v):
        return 0.0 if v is None else float(x[v])

    r = np.array([[val(R[t][j]) for j in range(V)] for t in range(T)])
    s = np.array([[val(S[t][j]) for j in range(V)] for t in range(T + 1)])
    pm = np.array([[val(Pv(t, j)) for j in range(V)] for t in range(T)])
    m = np.array([[val(M[t][p]) for p in range(Y)] for t in range(T)])
    ip = np.array([[val(IP[t][j]) for j in range(V)] for t in range(T)])
    rf = np.zeros((T, len(conv_list), si.num_conv_algos))
    for (cc, t, ci), v in RF.items():
        rf[t, ci, cc] = val(v)
    fwd_cost, bwd_cost = _expected_cost(tb, r, m, rf, ip)
    sol = _solution_class()(r, s, m, rf, ip, pm, solve_time, fwd_cost, bwd_cost, fwd_cost + bwd_cost)
    sol.mip_gap = getattr(res, "mip_gap", None)
    sol.status = int(res.status)
    sol.message = str(res.message)
    sol.size = (pr.nvar, len(pr.lo), len(pr.rows_v))
    return sol


def _expected_cost(tb: _Tables, r, m, rf, ip):
    """The objective of cvxpy_solver.py:260-293 evaluated on a solution."""
    si, V, T = tb.si, tb.V, tb.T
    conv_list = dict(si.conv_list) if si.select_conv_algo else {}
    fwd = bwd = 0.0
    for i in range(V):
        if i in conv_list:
            for t in range(T):
                for c in range(len(tb.cpu[i])):
                    fwd += rf[t, conv_list[i], c] * tb.cpu[i][c]
            continue
        fwd += r[0][i] * tb.cpu[i][0]
        for t in range(1, T):
            fwd += r[t][i] * tb.cpu_recompute[i][0]
    if si.do_inplace:
        for i in si.inplace_list:
            for t in range(T):
                fwd += ip[t][i] * (tb.cpu_inplace[i][0] - tb.cpu[i][0])
    for t in range(T):
        bk = V + t - 1
        if bk in conv_list:
            for c in range(len(tb.cpu[bk])):
                bwd += rf[t, conv_list[bk], c] * tb.cpu[bk][c]
        else:
            for p in range(Y):
                if p < len(tb.cpu[bk]):
                    bwd += m[t][p] * tb.cpu[bk][p]
    return fwd, bwd


# ------------------------------------------------------------------- literal re-check
def check_solution(si, sol, budget_gb: Optional[float] = None) -> dict:
    """Evaluates every row of cvxpy_solver.py:98-258 literally on a solution.

    Returns ``{"violations": [...], "peak_kb": max left-hand side of the memory rows,
    "cost": objective}``.  ``violations`` lists correctness rows that do not hold and, when
    ``budget_gb`` is given, memory rows above it."""
    tb = _Tables(si)
    V, T, ram = tb.V, tb.T, tb.ram
    # (stored schedules keep their 0/1 arrays as uint8: evaluate in floating point)
    R, S, M, IP, P, rf = (np.asarray(a, dtype=np.float64) for a in (sol.r, sol.s, sol.m, sol.ip, sol.p, sol.rf))
    bad: List[str] = []
    inpl = si.do_inplace
    conv_list = dict(si.conv_list) if si.select_conv_algo else {}
    n_algos = si.num_conv_algos

    def need(cond, msg):
        if not cond:
            bad.append(msg)

    need(np.all(S[0] == 0), "S[0] != 0")
    for i in range(V):
        if not tb.is_int[i]:
            need(R[0][i] == 1, f"R[0,{i}] != 1")
    need(M[0][0] == 1 and np.all(M[0][1:] == 0), "M[0] is not the first path")
    for t in range(1, T):
        paths = len(tb.bwd_node(t).args)
        need(np.all(M[t][paths:] == 0), f"M[{t}] selects a missing path")
        need(M[t].sum() >= 1, f"M[{t}] selects no path")
    if inpl:
        need(np.all(P <= R), "P > R")
        need(np.all(IP <= R), "IP > R")
        for v in range(V):
            if v not in si.inplace_list:
                need(np.all(IP[:, v] == 0), f"IP[:, {v}] set for a node that cannot run in place")
            elif not tb.is_int[v]:
                u = si.inplace_list[v]
                need(np.all(P[:, u] >= R[:, u] - 2 * IP[:, v]), f"P[{u}] < R - 2 IP[{v}]")
                need(np.all(P[:, u] <= 2 - 2 * IP[:, v]), f"P[{u}] present although overwritten by {v}")
                need(np.all(S[1:, u] <= 2 - 2 * IP[:, v]), f"S[{u}] stored although overwritten by {v}")
    else:
        need(np.all(P == R), "P != R")
    need(np.all(S[1:T + 1] <= S[:T] + P[:T]), "a tensor is stored that is not in memory")
    for (u, v, p) in si.edge_list:
        if u < V and v < V:
            need(np.all(R[:, v] <= R[:, u] + S[:T, u]), f"forward {v} runs without its input {u}")
        elif u < V and v >= V:
            t = v + 1 - V
            need(M[t, p] <= P[t, u] + S[t + 1, u], f"backward at t={t} path {p} misses tensor {u}")
    for i in range(V):
        if si.nodes[i].has_intermediates:
            for (_, intid) in si.nodes[i].intermediates:
                need(np.all(R[:, intid] <= R[:, i]), f"intermediate {intid} without its parent")
    for i, ci in conv_list.items():
        if i < si.loss:
            need(np.all(rf[:, ci, :].sum(axis=1) >= R[:, i]), f"convolution {i} runs without a variant")
        else:
            t = i + 1 - V
            need(rf[t, ci, :].sum() >= 1, f"backward convolution {i} has no variant")
        for c in range(n_algos):
            if c >= len(tb.cpu[i]) or tb.cpu[i][c] < 0:
                need(np.all(rf[:, ci, c] == 0), f"failed variant {c} chosen for {i}")

    # SM = S[1:] * M per path
    SMv = [S[1:] * M[:, p:p + 1] for p in range(Y)]
    peak = 0.0
    keep = [np.zeros((T, V)) for _ in range(Y)]
    gradm = np.zeros(T)
    for t in range(T):
        bk = V + t - 1
        gradm[t] = (tb.local_memory(bk) if t != 0 else 0) + tb.fixed_ram(bk - 1)
    ramV = ram[:V]
    for j in range(V):
        sm1 = S[:T, j:V] @ ramV[j:] + (S[1:, :j] @ ramV[:j] if j else 0)
        ws = np.repeat([tb.cmem(j, recompute=True)], T, axis=0).astype(float)
        ws[0] = tb.cmem(j)
        if conv_list and j in conv_list:
            wm = sum(rf[:, conv_list[j], c] * ws[:, c] for c in range(ws.shape[1]))
        elif inpl and j in si.inplace_list:
            ipw = float(tb.cmem(j, inplace=True)[0])
            wm = IP[:, j] * (ipw - ws[:, 0]) + R[:, j] * ws[:, 0]
        else:
            wm = R[:, j] * ws[:, 0]
        rm = R[:, j] * (ram[j] + tb.local_memory(j))
        sm2_ram = ramV.copy()
        lt = list(si.nodes[j].local_tensors)
        if lt:
            sm2_ram[[u for u in lt if u < V]] = 0
        sm2 = (S[:T, j + 1:V] @ sm2_ram[j + 1:] if j + 1 < V else 0) + (S[1:, :j] @ sm2_ram[:j] if j else 0)
        lm1 = sum(M[:, p] * keep[p].sum(axis=1) for p in range(Y))
        lm2 = sum((SMv[p] * -keep[p]).sum(axis=1) for p in range(Y))
        m1 = gradm + sm1 + lm1 + lm2
        m2 = gradm + wm + rm + sm2 + lm1 + lm2
        peak = max(peak, float(m1.max()), float(m2.max()))
        for t in range(T):
            node = tb.bwd_node(t)
            for p in range(min(len(node.args), Y)):
                if j in node.args[p]:
                    keep[p][t, j] += ram[j]
    for t in range(1, T):
        bk = V + t - 1
        node = si.nodes[bk]
        const = tb.local_memory(bk) + tb.fixed_ram(bk) + ram[bk]
        wmem = tb.cmem(bk)
        if conv_list and bk in conv_list:
            bwd_wm = sum(rf[t, conv_list[bk], c] * wmem[c] for c in range(len(wmem)))
        else:
            bwd_wm = sum(M[t, p] * wmem[p] for p in range(min(len(node.args), len(wmem))))
        lm3 = sum(M[t, p] * keep[p].sum(axis=1)[t] for p in range(min(len(node.args), Y)))
        lm4 = 0.0
        for p in range(min(len(node.args), Y)):
            r3 = ramV.copy()
            if len(node.dep_list_fwd[p]):
                r3[[u for u in node.dep_list_fwd[p] if u < V]] = 0
            lm4 += float((SMv[p][t] * r3).sum())
        peak = max(peak, float(bwd_wm + const + lm3 + lm4))
    if budget_gb is not None:
        need(peak <= budget_gb * GB_TO_KB + 1e-6, f"memory rows peak at {peak / GB_TO_KB:.3f} GB > {budget_gb} GB")
    fwd, bwd = _expected_cost(tb, R, M, rf, IP)
    return {"violations": bad, "peak_kb": peak, "peak_gb": peak / GB_TO_KB, "cost": fwd + bwd}


# --------------------------------------------------------------------- hand solutions
def hand_solution(si, kind: str = "store_all"):
    """A valid ``Solution`` without solving: what a trivial policy would choose.

    ``store_all``: implementation 0 of every operator, every forward output kept until its last
    backward reader, nothing recomputed, nothing in place (what stock autograd does).
    ``low_memory``: the last registered implementation of every multi-way operator (batch norm
    from its output, ReLU from a 1-bit mask or its output, max-pool from 4-bit indices), every
    forward output still kept (no recomputation), in place where the solver info allows it and
    the overwritten tensor has no backward reader."""
    if kind not in ("store_all", "low_memory"):
        raise ValueError(kind)
    tb = _Tables(si)
    V, T = tb.V, tb.T
    r = np.zeros((T, V)); s = np.zeros((T + 1, V)); m = np.zeros((T, Y)); ip = np.zeros((T, V))
    conv_list = dict(si.conv_list) if si.select_conv_algo else {}
    rf = np.zeros((T, len(conv_list), si.num_conv_algos))
    m[0, 0] = 1
    path = {}
    for t in range(1, T):
        paths = min(len(tb.bwd_node(t).args), Y)
        path[t] = paths - 1 if kind == "low_memory" else 0
        m[t, path[t]] = 1
    last_need = np.zeros(V, dtype=int)
    for t in range(1, T):
        for j in tb.fwd_deps(t, path[t]):
            last_need[j] = max(last_need[j], t)
    for j in range(V):
        if tb.is_int[j]:
            parent = si.nodes[j].solver_parent_id
            t_b = si.fwd_to_bwd[parent] - si.loss
            r[0, j] = 1 if (path.get(t_b, 0) == si.nodes[j].op_idx and last_need[j] > 0) else 0
        else:
            r[0, j] = 1
        if r[0, j] and last_need[j] > 0:
            s[1:last_need[j] + 2, j] = 1      # the backward at time t reads S[t+1] (:155)
    if kind == "low_memory" and si.do_inplace:
        for v, u in si.inplace_list.items():
            if tb.is_int[v]:
                continue
            if last_need[u] == 0 and r[0, v]:
                ip[0, v] = 1
        for v in list(si.inplace_list):
            if tb.is_int[v]:
                ip[0, v] = ip[0, si.nodes[v].solver_parent_id] * r[0, v]
    p = r.copy()
    if si.do_inplace:
        for v, u in si.inplace_list.items():
            if not tb.is_int[v] and ip[0, v]:
                p[0, u] = 0
    for i, ci in conv_list.items():
        valid = [c for c in range(si.num_conv_algos) if c < len(tb.cpu[i]) and tb.cpu[i][c] >= 0]
        c0 = valid[0] if valid else 0
        if i < si.loss:
            rf[0, ci, c0] = 1
        else:
            rf[i + 1 - V, ci, c0] = 1
    fwd, bwd = _expected_cost(tb, r, m, rf, ip)
    return _solution_class()(r, s, m, rf, ip, p, 0.0, fwd, bwd, fwd + bwd)


# ------------------------------------------------------------------------------- CLI
def main(argv=None):
    """``python -m monet_b200.solver MODEL BS BUDGET MODE [--time_limit S] [--costs ...]``: the
    command line of monet/cvxpy_solver.py:336-384 (positionals model, batch size, budget in GB,
    mode) with HiGHS as the only backend.  Writes ``solution_<model>_<bs>_<mode>_<budget>.pkl``
    (the reference's file name, cvxpy_solver.py:323) under ``--out`` and prints one JSON line."""
    import argparse
    import json
    from pathlib import Path

    import torch
    import torchvision

    from . import reference_host as rh

    ap = argparse.ArgumentParser(prog="python -m monet_b200.solver")
    ap.add_argument("model", help='e.g. "resnet50", or an expression like torchvision.models.vgg16_bn()')
    ap.add_argument("bs", type=int)
    ap.add_argument("budget", type=float, help="GB, in the ILP's accounting (activations + parameters + gradients)")
    ap.add_argument("mode", nargs="?", default="inplace_conv_multiway_newnode")
    ap.add_argument("--time_limit", type=float, default=3600.0)
    ap.add_argument("--gap", type=float, default=0.01)
    ap.add_argument("--costs", default="estimate", choices=["estimate", "reference", "events"],
                    help="cost tables: bytes-and-flops model (no GPU), MONeT's profiler, or the CUDA-event profiler")
    ap.add_argument("--cost_file", default=None, help="a cost_*.pkl written by an earlier profiling run")
    ap.add_argument("--height", type=int, default=224)
    ap.add_argument("--width", type=int, default=224)
    ap.add_argument("--out", default=None, help="directory for the solution pickle (default: <MONeT root>/data)")
    ap.add_argument("--verbose", action="store_true")
    ap.add_argument("--profile_only", action="store_true",
                    help="stop after the cost tables are written (cost_<model>_<bs>_<mode>.pkl under --out): "
                         "profile on the GPU machine, solve anywhere with --cost_file")
    args = ap.parse_args(argv)

    ref = rh.activate()
    if "(" in args.model:
        model = eval(args.model, {"torch": torch, "torchvision": torchvision})      # as cvxpy_solver.py:369
        name = args.model.split(".")[-1].split("(")[0]
    else:
        name = args.model
        model = getattr(torchvision.models, name)()
    shape = (3, args.height, args.width)
    out_dir = Path(args.out) if args.out else ref.root / "data"
    workdir = out_dir.parent if out_dir.name == "data" else out_dir
    if args.cost_file:
        import shutil
        (workdir / "data").mkdir(parents=True, exist_ok=True)
        si_probe = ref.solver_info.SolverInfo(args.bs, name, args.mode)
        shutil.copyfile(args.cost_file, workdir / "data" / f"cost_{si_probe.data_path}.pkl")
    profile = args.costs != "estimate" or bool(args.cost_file)
    if profile and not args.cost_file:
        model = model.cuda()
    graph, si = rh.build_solver_info(model, args.bs, name, args.mode, shape, workdir=workdir,
                                     profile=profile, profiler="events" if args.costs == "events" else "reference")
    if args.profile_only:
        print(json.dumps({"cost_file": str(workdir / "data" / f"cost_{si.data_path}.pkl"), "costs": args.costs}))
        return
    base = check_solution(si, hand_solution(si, "store_all"))
    sol = solve(si, args.budget, time_limit=args.time_limit, mip_rel_gap=args.gap, verbose=args.verbose)
    chk = check_solution(si, sol, args.budget)
    path = out_dir / ("solution_%s_%4.2f.pkl" % (si.data_path, args.budget))
    rh.save_solution(si, sol, path)
    print(json.dumps({"solution": str(path), "budget_gb": args.budget, "ilp_peak_gb": chk["peak_gb"],
                      "violations": chk["violations"], "expected_cost": sol.runtime_expected,
                      "store_all_cost": base["cost"], "store_all_ilp_peak_gb": base["peak_gb"],
                      "overhead_expected": sol.runtime_expected / base["cost"] - 1.0,
                      "recomputations": int(sol.r[1:].sum()), "in_place": int(sol.ip.sum()),
                      "solve_time_s": sol.solve_time, "mip_gap": sol.mip_gap, "size": sol.size,
                      "costs": args.cost_file or args.costs}))


if __name__ == "__main__":
    main()
