"""Residual add and adaptive average pooling (monet/lm_ops/funcs.py:7-59)."""
from __future__ import annotations

import torch

from .. import functional as F
from .base import COMMON_MODES, OP, implements


@implements(['aten::adaptive_avg_pool2d'], COMMON_MODES)
class AdaptiveAvgPool2D(OP):
    """Global (1x1) pooling runs this library's kernels; other output sizes (the reference's
    UNet uses the operator to up-sample, models/unet/unet_parts.py:47) run ATen's kernel on
    the GPU, as the reference does (lrfuncs.cpp:11-14).  The backward needs only the input's
    shape, which travels in ``params`` (the executor hands ``params``, not the object, to the
    operator instance that runs the backward, schedule.py:247-251)."""
    params = None

    def forward(self, x, os):
        with torch.no_grad():
            os = [int(v) for v in (os if isinstance(os, (list, tuple)) else [os, os])]
            self.params = tuple(x.shape), F.is_nhwc(x), os
            if os == [1, 1] and x.dim() == 4:
                return F.global_avgpool(x)
            return torch._C._nn.adaptive_avg_pool2d(x.detach(), os)

    def backward(self, grad_output, stored, nodel=False):
        assert len(stored) == 0
        with torch.no_grad():
            shape, nhwc, os = self.params
            if os == [1, 1] and len(shape) == 4:
                return F.global_avgpool_bwd(grad_output, shape, nhwc)
            # ATen wants the forward input for its sizes only: a stride-0 view of one element
            like = grad_output.new_empty(1).expand(shape)
            return torch.ops.aten._adaptive_avg_pool2d_backward(grad_output.contiguous(), like)


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
