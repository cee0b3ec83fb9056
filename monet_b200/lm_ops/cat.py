"""Concatenation (monet/lm_ops/cat.py:5-29): forward and the split of the gradient each run as
one row-copy launch over all pieces."""
from __future__ import annotations

import torch

from .. import functional as F
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
            return F.cat([t.detach() for t in tensors], dim)

    def backward(self, grad_output, stored=None, nodel=False):
        # the executor calls backward(grad, stored) with an empty `stored` (no backward_storage)
        dim, sizes = self.params
        with torch.no_grad():
            if len(sizes) == 1:
                return grad_output
            return F.cat_bwd(grad_output, sizes, dim)
