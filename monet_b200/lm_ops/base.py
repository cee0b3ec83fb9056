"""Operator protocol, storage descriptors and registry of the low-memory operator library.

Mirrors the contract of monet/lm_ops/base.py:2-53 in the reference, which is what
``Schedule`` (schedule.py:58-142), ``SolverInfo`` (solver_info.py:119-136) and the profiler
(meminfo.py) program against:

* an operator is a zero-argument-constructible class with ``forward(*aten_args)`` and
  ``backward(grad_output, stored, nodel=False)``;
* ``backward_storage`` says what the executor must keep alive for the backward:
  inputs by position, the output, or an operator-defined intermediate of a known size;
* ``@implements(names, modes)`` appends the class to ``registry[mode][aten_name]``; the
  list position is the implementation index stored in solutions, so registration order
  is part of the interface.
"""
from __future__ import annotations


class StorageInfo:
    """Base of the three descriptors of what a backward pass needs kept."""


class InputStorage(StorageInfo):
    """Keep the forward inputs at the given argument positions."""

    def __init__(self, *ids):
        self.ids = ids


class OutputStorage(StorageInfo):
    """Keep the forward output."""


class IntermediateStorage(StorageInfo):
    """Keep the second element of the forward's ``(output, intermediate)`` pair.

    ``size_fn(output_shape)`` gives its size in bytes for the solver's memory tables.
    """

    def __init__(self, size_fn):
        self.size = size_fn


class OP:
    names: list = []
    backward_storage = None

    def intermediate(self):
        return None

    def forward(self, *args, **kwargs):
        raise NotImplementedError

    def backward(self, *args, **kwargs):
        raise NotImplementedError


all_modes = ["none", "normal", "multiway", "newnode", "multiway_newnode",
             "conv_multiway_newnode", "conv_normal", "gist"]

# mode -> aten op name -> [implementation classes in registration order]
registry: dict = {}


def implements(names, modes):
    """Class decorator registering an implementation of `names` under every mode in `modes`."""
    for m in modes:
        if m not in all_modes:
            raise ValueError(f"unknown mode {m!r}")

    def decorate(cls):
        for m in modes:
            per_mode = registry.setdefault(m, {})
            for n in names:
                per_mode.setdefault(n, []).append(cls)
        cls.names = names
        return cls

    return decorate


def list_ops(mode, name):
    return registry[mode][name]


def install_into(reference_base) -> None:
    """Make the reference's registry serve these operators.

    `reference_base` is the imported ``monet.lm_ops.base`` module of a MONeT checkout whose
    own operator modules have NOT been imported (they JIT-compile CUDA sources written for
    PyTorch 1.5).  After the call ``reference_base.list_ops(mode, name)`` returns the
    classes of this package, in the reference's slot order.
    """
    reference_base.registry.clear()
    for mode, table in registry.items():
        reference_base.registry[mode] = {n: list(impls) for n, impls in table.items()}


# Modes every plain (single-implementation) operator registers under.
COMMON_MODES = ["normal", "multiway", "newnode", "multiway_newnode", "conv_multiway_newnode",
                "conv_normal"]
