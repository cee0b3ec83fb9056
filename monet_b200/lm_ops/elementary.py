"""Shape and small arithmetic operators that simply defer to autograd
(monet/lm_ops/elementary.py:5-95): the forward runs the torch op with grad enabled and
keeps its grad_fn, the backward calls it."""
from __future__ import annotations

import torch

from .base import COMMON_MODES, OP, implements


class NativeOP(OP):
    op = None
    grad_fn = None
    backward_storage = None

    def forward(self, input_, *args, **kwargs):
        with torch.enable_grad():
            r = self.op(input_.requires_grad_(True), *args, **kwargs)
        if r.grad_fn is None:
            if r is not input_:
                raise RuntimeError(f"{type(self).__name__}: result has no grad_fn")
            self.grad_fn = None        # the op returned its input unchanged (e.g. dropout with p = 0)
            return r.detach()
        self.grad_fn = r.grad_fn
        return r.detach()

    def backward(self, grad_output, stored, nodel=False):
        assert len(stored) == 0
        if self.grad_fn is None:
            return grad_output
        return self.grad_fn(grad_output)


def _native(name, fn):
    cls = type(name, (NativeOP,), {"op": staticmethod(fn), "__doc__": f"autograd-backed {name}"})
    return cls


def _avg_pool2d(*a):
    a = list(a)
    a[4] = bool(a[4])
    a[5] = bool(a[5])
    return torch._C._nn.avg_pool2d(*a)


Flatten = implements(['aten::flatten'], COMMON_MODES)(_native("Flatten", torch.flatten))
Permute = implements(['aten::permute'], COMMON_MODES)(_native("Permute", lambda x, d: x.permute(*d)))
Transpose = implements(['aten::transpose'], COMMON_MODES)(_native("Transpose", torch.transpose))
View = implements(['aten::view'], COMMON_MODES)(_native("View", lambda x, s: x.view(*s)))
Div = implements(['aten::div'], COMMON_MODES)(_native("Div", torch.div))
Contiguous = implements(['aten::contiguous'], COMMON_MODES)(
    _native("Contiguous", lambda x, *a: x.contiguous()))
Unsqueeze = implements(['aten::unsqueeze'], COMMON_MODES)(_native("Unsqueeze", torch.unsqueeze))
Mul = implements(['aten::mul'], COMMON_MODES)(_native("Mul", torch.mul))
T = implements(['aten::t'], COMMON_MODES)(_native("T", lambda x: x.t()))
AvgPool2D = implements(['aten::avg_pool2d'], COMMON_MODES)(_native("AvgPool2D", _avg_pool2d))
Dropout = implements(['aten::dropout'], COMMON_MODES)(
    _native("Dropout", lambda x, p, training=False: torch.nn.functional.dropout(x, p, bool(training))))
