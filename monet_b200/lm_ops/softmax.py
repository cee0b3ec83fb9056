"""Softmax with the output kept for backward (monet/lm_ops/softmax.py:7-24), plus the
fused cross-entropy operator.  Like the reference's softmax module, this one registers
only when imported explicitly."""
from __future__ import annotations

import torch

from .. import functional as F
from .base import COMMON_MODES, OP, OutputStorage, implements


@implements(['aten::softmax'], COMMON_MODES)
class Softmax(OP):
    params = None
    backward_storage = OutputStorage()

    def forward(self, input_, dim, dtype=None):
        if dtype is not None:
            raise NotImplementedError("softmax with a dtype conversion")
        with torch.no_grad():
            self.params = input_.type(), dim
            return F.softmax(input_, dim)

    def backward(self, grad_output, stores, nodel=False):
        with torch.no_grad():
            output = stores[0]
            if not nodel:
                del stores[0]
            return F.softmax_bwd(grad_output, output, self.params[1])


@implements(['aten::log_softmax'], COMMON_MODES)
class LogSoftmax(OP):
    params = None
    backward_storage = OutputStorage()

    def forward(self, input_, dim, dtype=None):
        with torch.no_grad():
            self.params = input_.type(), dim
            return F.softmax(input_, dim, log=True)

    def backward(self, grad_output, stores, nodel=False):
        with torch.no_grad():
            output = stores[0]
            if not nodel:
                del stores[0]
            return F.softmax_bwd(grad_output, output, self.params[1], log=True)


class SoftmaxCrossEntropy(OP):
    """Mean cross-entropy whose forward also produces d(loss)/d(logits): one pass over the
    logits computes max, sum-exp, the per-sample loss and (softmax - onehot)/count.  The
    gradient is the operator's intermediate, so the backward is a scale by grad_output.
    Not registered under an aten name: the reference keeps the loss outside its graph
    (examples/imagenet.py:327)."""
    backward_storage = None
    params = None

    def forward(self, logits, target):
        with torch.no_grad():
            losses, dlogits = F.cross_entropy_fwd_bwd(logits, target, 1.0 / target.numel())
            self.params = dlogits
            return losses.mean()

    def backward(self, grad_output=None, stored=None, nodel=False):
        with torch.no_grad():
            d = self.params
            self.params = None
            if grad_output is None:
                return d
            g = float(grad_output)
            return d if g == 1.0 else F.scale(d, g)
