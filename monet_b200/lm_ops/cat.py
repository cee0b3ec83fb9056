"""Concatenation (monet/lm_ops/cat.py:5-29)."""
from __future__ import annotations

import torch

from .base import COMMON_MODES, OP, implements


@implements(['aten::cat'], COMMON_MODES)
class Cat(OP):
    params = None

    def forward(self, *input_):
        tensors, dim = input_[:-1], input_[-1]
        self.params = dim, [int(t.shape[dim]) for t in tensors]
        with torch.no_grad():
            if len(tensors) == 1:
                return tensors[0]
            return torch.cat(tensors, dim=dim)

    def backward(self, *grad_output, nodel=False):
        dim, sizes = self.params
        with torch.no_grad():
            g = grad_output[0]
            if len(sizes) == 1:
                return g
            return [piece.contiguous() for piece in torch.split(g, sizes, dim=dim)]
