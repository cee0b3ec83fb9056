"""Batch-norm implementations in the reference's slot order (monet/lm_ops/bn.py:12-140).

Both cache the batch statistics of their first forward in ``op.params`` (the executor
copies ``params`` to the later instances of the node, schedule.py:159-173), so that a
recomputation reuses them instead of updating the running statistics twice.
"""
from __future__ import annotations

import torch

from .. import functional as F
from .base import OP, InputStorage, OutputStorage, implements


class _BatchNorm(OP):
    params = None
    running_mean = None
    running_var = None
    inplace = False
    input_sums = None      # F.ChannelSums left by the producer of the input, or None

    def forward(self, input_, weight, bias, running_mean, running_var,
                training=False, momentum=0.1, eps=1e-5, *args, **kwargs):
        with torch.no_grad():
            if self.running_mean is None:
                self.running_mean = running_mean.requires_grad_(False) if running_mean is not None else None
                self.running_var = running_var.requires_grad_(False) if running_var is not None else None
            if self.params is None:
                if training and self.input_sums is not None:
                    out, mean, invstd = F.bn_act_fwd_train_partials(
                        input_, self.input_sums, None, 0, weight, bias, self.running_mean,
                        self.running_var, momentum, eps, inplace=self.inplace)
                    self.input_sums = None
                elif training:
                    out, mean, invstd = F.bn_fwd_train(
                        input_, weight, bias, self.running_mean, self.running_var,
                        momentum, eps, inplace=self.inplace)
                else:
                    mean = self.running_mean
                    invstd = torch.rsqrt(self.running_var + eps)
                    out = F.bn_fwd_apply(input_, weight, bias, mean, invstd, eps, inplace=self.inplace)
                self.params = bool(training), eps, mean, invstd, None
            else:
                _, eps, mean, invstd, _ = self.params
                out = F.bn_fwd_apply(input_, weight, bias, mean, invstd, eps, inplace=self.inplace)
            return out


@implements(['aten::batch_norm'],
            ['normal', 'multiway', 'newnode', 'multiway_newnode', 'conv_multiway_newnode',
             'conv_normal'])
class InputActBatchNorm(_BatchNorm):
    """Backward from the stored input x."""
    backward_storage = InputStorage(0, 1, 2, 3, 4)

    def backward(self, grad_output, stored, nodel=False):
        with torch.no_grad():
            input_, weight, bias, running_mean, running_var = stored
            training, eps, save_mean, save_invstd, _ = self.params
            if not training:
                raise NotImplementedError("batch-norm backward in eval mode")
            dx, dw, db = F.bn_bwd_from_input(grad_output, input_, weight, save_mean, save_invstd)
            if not nodel:
                del stored[4], stored[3], stored[2], stored[1], stored[0]
            return dx, dw, db, None, None


@implements(['aten::batch_norm'], ['multiway', 'multiway_newnode', 'conv_multiway_newnode'])
class OutputActBatchNorm(_BatchNorm):
    """Backward from the stored OUTPUT y: xhat = (y - beta) / gamma, so the input never has
    to be kept and the forward can run in place."""
    backward_storage = [InputStorage(1, 2, 3, 4), OutputStorage()]

    def backward(self, grad_output, stored, nodel=False):
        with torch.no_grad():
            weight, bias, running_mean, running_var, output = stored
            training, eps, save_mean, save_invstd, _ = self.params
            if not training:
                raise NotImplementedError("batch-norm backward in eval mode")
            dx, dw, db = F.bn_bwd_from_output(grad_output, output, weight, bias, save_invstd)
            if not nodel:
                del stored[4], stored[3], stored[2], stored[1], stored[0]
            return dx, dw, db, None, None
