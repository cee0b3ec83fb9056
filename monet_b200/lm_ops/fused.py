"""Fused operators: batch norm + ReLU, batch norm + residual add + ReLU, add + ReLU.

The reference has no such operators: its graph runs ``aten::batch_norm``, ``aten::add`` and
``aten::relu`` as separate nodes (monet/lm_ops/bn.py, funcs.py, relu.py), each a full pass
over the activation.  On a B200 those passes are pure HBM traffic, so the element-wise tail
is folded into the batch-norm sweep.  They follow the same protocol (``backward_storage``,
``params`` carried to later instances of the node, ``inplace``) and register under node
names of their own, ``monet::batch_norm_relu`` (and ``_relu6``),
``monet::batch_norm_add_relu`` and ``monet::add_relu``, so the slot order of the reference's names is untouched; a graph
rewriter (``runner.fuse_graph``) produces those nodes from the unfused pattern.

Argument order = the batch-norm node's arguments, then the residual:
``(x, weight, bias, running_mean, running_var, training, momentum, eps, cudnn, residual)``.
"""
from __future__ import annotations

import torch

from .. import functional as F
from .base import COMMON_MODES, OP, InputStorage, OutputStorage, implements


class _FusedBatchNorm(OP):
    params = None
    running_mean = None
    running_var = None
    inplace = False
    relu = True
    input_sums = None      # F.ChannelSums left by the producer of the input, or None

    def _forward(self, input_, residual, weight, bias, running_mean, running_var, training,
                 momentum, eps):
        with torch.no_grad():
            if self.running_mean is None:
                self.running_mean = running_mean.requires_grad_(False) if running_mean is not None else None
                self.running_var = running_var.requires_grad_(False) if running_var is not None else None
            if self.params is None:
                if training and self.input_sums is not None:
                    out, mean, invstd = F.bn_act_fwd_train_partials(
                        input_, self.input_sums, residual, self.relu, weight, bias,
                        self.running_mean, self.running_var, momentum, eps, inplace=self.inplace)
                    self.input_sums = None
                elif training:
                    out, mean, invstd = F.bn_act_fwd_train(
                        input_, residual, self.relu, weight, bias, self.running_mean,
                        self.running_var, momentum, eps, inplace=self.inplace)
                else:
                    mean = self.running_mean
                    invstd = torch.rsqrt(self.running_var + eps)
                    out = F.bn_act_fwd_apply(input_, residual, self.relu, weight, bias, mean,
                                             invstd, inplace=self.inplace)
                self.params = bool(training), eps, mean, invstd, None
            else:
                _, eps, mean, invstd, _ = self.params
                out = F.bn_act_fwd_apply(input_, residual, self.relu, weight, bias, mean, invstd,
                                         inplace=self.inplace)
            return out


@implements(['monet::batch_norm_relu'], COMMON_MODES)
class InputActBatchNormReLU(_FusedBatchNorm):
    """y = relu(bn(x)); backward from the stored input x alone: the ReLU gate is re-evaluated
    from x, so neither y nor a mask is kept for this operator."""
    backward_storage = InputStorage(0, 1, 2, 3, 4)

    def forward(self, input_, weight, bias, running_mean, running_var,
                training=False, momentum=0.1, eps=1e-5, *args, **kwargs):
        return self._forward(input_, None, weight, bias, running_mean, running_var, training,
                             momentum, eps)

    def backward(self, grad_output, stored, nodel=False):
        with torch.no_grad():
            input_, weight, bias, running_mean, running_var = stored
            training, eps, save_mean, save_invstd, _ = self.params
            if not training:
                raise NotImplementedError("batch-norm backward in eval mode")
            dx, dw, db = F.bn_relu_bwd_from_input(grad_output, input_, weight, bias, save_mean,
                                                  save_invstd, inplace=True, act=int(self.relu))
            if not nodel:
                del stored[4], stored[3], stored[2], stored[1], stored[0]
            return dx, dw, db, None, None


@implements(['monet::batch_norm_relu6'], COMMON_MODES)
class InputActBatchNormReLU6(InputActBatchNormReLU):
    """y = clamp(bn(x), 0, 6) (MobileNetV2's batch norm + ReLU6); the gate 0 < z < 6 is
    re-evaluated from x in the backward."""
    relu = 2


@implements(['monet::batch_norm_add_relu'], COMMON_MODES)
class InputActBatchNormAddReLU(_FusedBatchNorm):
    """y = relu(bn(x) + residual).  Backward keeps x and y: the gated gradient
    d = dy * (y > 0) is what the residual branch receives, and batch norm backpropagates d
    from x; d is formed inside the batch-norm backward's first pass.  ``backward`` also accepts a pair ``(dy1, dy2)`` of gradients still to be summed
    (y read by two consumers) and folds the sum into the gate."""
    backward_storage = [InputStorage(0, 1, 2, 3, 4), OutputStorage()]
    accepts_grad_pair = True

    def forward(self, input_, weight, bias, running_mean, running_var,
                training=False, momentum=0.1, eps=1e-5, cudnn=True, residual=None, *args, **kwargs):
        if residual is None:
            raise RuntimeError("monet::batch_norm_add_relu needs the residual as its 10th argument")
        return self._forward(input_, residual, weight, bias, running_mean, running_var, training,
                             momentum, eps)

    def backward(self, grad_output, stored, nodel=False):
        with torch.no_grad():
            input_, weight, bias, running_mean, running_var, output = stored
            training, eps, save_mean, save_invstd, _ = self.params
            if not training:
                raise NotImplementedError("batch-norm backward in eval mode")
            if isinstance(grad_output, (tuple, list)):
                g1, g2 = grad_output
            else:
                g1, g2 = grad_output, None
            d, dx, dw, db = F.bn_add_relu_bwd(g1, g2, output, input_, weight, save_mean, save_invstd)
            if not nodel:
                del stored[5], stored[4], stored[3], stored[2], stored[1], stored[0]
            return dx, dw, db, None, None, d


@implements(['monet::add_relu'], COMMON_MODES)
class AddReLU(OP):
    """y = relu(a + alpha * b), keeping y for the gate; both inputs receive the gated gradient."""
    backward_storage = OutputStorage()
    accepts_grad_pair = True
    inplace = False
    params = None

    def forward(self, a, b, alpha=1):
        with torch.no_grad():
            self.params = float(alpha)
            return F.add_relu(a, b, float(alpha), inplace=self.inplace)

    def backward(self, grad_output, stored, nodel=False):
        with torch.no_grad():
            output = stored[0]
            if isinstance(grad_output, (tuple, list)):
                d = F.relu_bwd_act2(grad_output[0], grad_output[1], output)
            else:
                d = F.relu_bwd_act(grad_output, output, 0.0, inplace=True)
            if not nodel:
                del stored[0]
            alpha = self.params if self.params is not None else 1.0
            return d, (d if alpha == 1.0 else F.scale(d, alpha))
