"""Residual add and adaptive average pooling (monet/lm_ops/funcs.py:7-59)."""
from __future__ import annotations

import torch

from .. import functional as F
from .base import COMMON_MODES, OP, implements


@implements(['aten::adaptive_avg_pool2d'], COMMON_MODES)
class AdaptiveAvgPool2D(OP):
    """Global (1x1) pooling runs this library's kernels; other output sizes defer to torch
    on the GPU.  The backward needs only the input's shape."""
    params = None
    grad_fn = None

    def forward(self, x, os):
        with torch.no_grad():
            os = [int(v) for v in (os if isinstance(os, (list, tuple)) else [os, os])]
            self.params = tuple(x.shape), F.is_nhwc(x), os
            if os == [1, 1] and x.dim() == 4:
                return F.global_avgpool(x)
        with torch.enable_grad():
            r = torch._C._nn.adaptive_avg_pool2d(x.detach().requires_grad_(True), os)
        self.grad_fn = r.grad_fn
        return r.detach()

    def backward(self, grad_output, stored, nodel=False):
        assert len(stored) == 0
        with torch.no_grad():
            shape, nhwc, os = self.params
            if self.grad_fn is None:
                return F.global_avgpool_bwd(grad_output, shape, nhwc)
            return self.grad_fn(grad_output)


class _Add(OP):
    backward_storage = None
    params = None

    def forward(self, a, b, s):
        with torch.no_grad():
            self.params = s
            return F.add(a, b, s, inplace=bool(getattr(self, "inplace", False)))

    def backward(self, grad_output, stored, nodel=False):
        assert len(stored) == 0
        with torch.no_grad():
            s = self.params
            # the gradient is shared, not copied, when the scale is 1
            return grad_output, (grad_output if s == 1 else F.scale(grad_output, s))


@implements(['aten::add'], COMMON_MODES)
class Add(_Add):
    pass


@implements(['aten::add_'], COMMON_MODES)
class AddIP(_Add):
    # only the in-place spelling carries the attribute: SolverInfo.get_inplace_info offers the
    # solver an in-place choice exactly for operators that have it (solver_info.py:442)
    inplace = False
