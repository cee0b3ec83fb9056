"""Convolution implementations in the reference's slot order (monet/lm_ops/conv.py:11-341).

All three classes run the same tcgen05 implicit-GEMM kernels; they differ, as in the
reference, in who picks the variant ("algorithm"):

* ``PytorchConvolution``    mode 'none'  : always variant 0.
* ``GreedyAlgoConvolution`` 'normal',... : times every variant on its first call and keeps the
  fastest one whose peak memory stays under ``config.budget`` (conv.py:127-148).
* ``SpecificAlgoConvolution`` 'conv_*'   : the solver sets ``op.algorithm`` per pass
  (schedule.py:79-84, 123-139): forward variant = algorithm; backward
  ``convtype = algorithm // 10`` (0 weights, 1 input, 2 both), ``variant = algorithm % 10``.

A variant that cannot run raises ``RuntimeError``; like the reference (conv.py:279-283) the
operator then retries with the default variant.  Depthwise convolutions (groups == C) run the
bandwidth-bound depthwise kernels.  Transposed convolutions, which the reference refuses
(conv.py:269), run the same tensor-core kernels with the passes exchanged.  Outputs are
channels_last tensors.
"""
from __future__ import annotations

from time import time

import torch

from .. import functional as F
from .._lib import MB_CONV_DGRAD, MB_CONV_FPROP, MB_CONV_WGRAD
from .base import OP, InputStorage, implements

import sys


def _budget_gb() -> float:
    """``config.budget`` in GB: MONeT's global budget holder is an empty module named ``config``
    at the root of a checkout that the CLI fills in (schedule.py:379-380, read at
    conv.py:140); no such module, or no value in it, means no limit."""
    cfg = sys.modules.get("config")
    if cfg is None:
        try:
            import config as cfg
        except Exception:
            return float("inf")
    return float(getattr(cfg, "budget", float("inf")))


class _ConvBase(OP):
    backward_storage = InputStorage(0, 1)
    params = None
    algorithm = -1
    is_depthwise = False

    @staticmethod
    def n_fwd_algos():
        return F.conv_num_variants(MB_CONV_FPROP)

    @staticmethod
    def n_bwd_ip_algos():
        return F.conv_num_variants(MB_CONV_DGRAD)

    @staticmethod
    def n_bwd_wt_algos():
        return F.conv_num_variants(MB_CONV_WGRAD)

    # An executor that knows a batch norm is the only reader of this output sets
    # `emit_channel_sums` (and, optionally, a per-channel shift near the expected mean): the
    # forward then leaves the sums that batch norm needs in `channel_sums` (F.ChannelSums, or
    # None where the geometry has no such path) and the batch norm skips its statistics pass.
    emit_channel_sums = False
    channel_sums_shift = None
    channel_sums = None

    # -- the three passes, with the reference's "retry with the default" behaviour ----------
    def _fprop(self, x, w, bias, variant):
        stride, padding, dilation, groups = self.params[:4]
        if self.is_depthwise or groups != 1:
            return F.depthwise_fprop(x, w, bias, stride, padding, dilation, groups)
        if self.emit_channel_sums:
            y, self.channel_sums = F.conv2d_fprop(x, w, bias, stride, padding, dilation, groups,
                                                  max(variant, 0), stats_shift=self.channel_sums_shift,
                                                  want_stats=True)
            return y
        try:
            return F.conv2d_fprop(x, w, bias, stride, padding, dilation, groups, max(variant, 0))
        except RuntimeError:
            if variant <= 0:
                raise
            return F.conv2d_fprop(x, w, bias, stride, padding, dilation, groups, 0)

    def _dgrad(self, dy, w, variant):
        stride, padding, dilation, groups, x_shape = self.params[:5]
        try:
            return F.conv2d_dgrad(dy, w, x_shape, stride, padding, dilation, groups, max(variant, 0))
        except RuntimeError:
            if variant <= 0:
                raise
            return F.conv2d_dgrad(dy, w, x_shape, stride, padding, dilation, groups, 0)

    def _wgrad(self, x, dy, variant, need_bias):
        stride, padding, dilation, groups, _, w_shape = self.params[:6]
        try:
            return F.conv2d_wgrad(x, dy, w_shape, stride, padding, dilation, groups,
                                  max(variant, 0), need_bias)
        except RuntimeError:
            if variant <= 0:
                raise
            return F.conv2d_wgrad(x, dy, w_shape, stride, padding, dilation, groups, 0, need_bias)

    def _remember(self, input_, weight, bias, stride, padding, dilation, groups, transposed=False,
                  output_padding=(0, 0)):
        self.params = (stride, padding, dilation, groups, tuple(input_.shape), tuple(weight.shape),
                       [input_.requires_grad, weight.requires_grad,
                        bias is not None and bias.requires_grad], bool(transposed),
                       tuple(int(v) for v in output_padding))

    # -- transposed convolution -------------------------------------------------------------
    # Beyond the reference, whose operators assert `not transposed` (conv.py:269): a transposed
    # convolution with filter W[C_in][C_out][R][S] is, pass for pass, the ordinary convolution
    # C_out -> C_in with the same filter read as [K = C_in][C = C_out][R][S], run backwards:
    #   forward          y  = dgrad(dy := x, W)          (output extent (H-1)*s - 2p + d(R-1) + op + 1)
    #   backward-data    dx = fprop(x := dy, W)
    #   backward-filter  dW = wgrad(x := dy, dy := x)
    # so it runs on the same tcgen05 kernels (a 2x2 stride-2 up-convolution is four 1x1 phase
    # GEMMs).  The bias is added by the element-wise kernel, db is a plain reduction.
    def _transposed_out_shape(self, x, w):
        stride, padding, dilation, groups = self.params[:4]
        op = self.params[8]
        sh, sw = F._pair(stride); ph, pw = F._pair(padding); dh, dw = F._pair(dilation)
        N, _, H, W = (int(v) for v in x.shape)
        R, S = int(w.shape[2]), int(w.shape[3])
        return (N, int(w.shape[1]), (H - 1) * sh - 2 * ph + dh * (R - 1) + op[0] + 1,
                (W - 1) * sw - 2 * pw + dw * (S - 1) + op[1] + 1)

    def _forward_transposed(self, x, w, bias, variant):
        stride, padding, dilation, groups = self.params[:4]
        if groups != 1:
            raise NotImplementedError("grouped transposed convolution")
        y = F.conv2d_dgrad(x, w, self._transposed_out_shape(x, w), stride, padding, dilation, 1, 0)
        if bias is not None:
            y = F.add_channel_bias(y, bias.detach())
        return y

    def _backward_transposed(self, grad_output, stored, nodel, convtype):
        with torch.no_grad():
            input_, weight = stored
            stride, padding, dilation = self.params[:3]
            do_grad = self.params[6]
            if not nodel:
                del stored[1]
                del stored[0]
            di = dw = db = None
            if convtype in (0, 2) and input_ is not None:
                if do_grad[1]:
                    dw, _ = F.conv2d_wgrad(grad_output, input_.detach(), tuple(self.params[5]), stride,
                                           padding, dilation, 1, 0, False)
                if do_grad[2]:
                    db = grad_output.sum((0, 2, 3))
            del input_
            if convtype in (1, 2) and weight is not None and do_grad[0]:
                di = F.conv2d_fprop(grad_output, weight.detach(), None, stride, padding, dilation, 1, 0)
            if do_grad[2]:
                return di, dw, db
            return di, dw

    def _backward(self, grad_output, stored, nodel, convtype, wt_variant, ip_variant):
        if len(self.params) > 7 and self.params[7]:
            return self._backward_transposed(grad_output, stored, nodel, convtype)
        with torch.no_grad():
            input_, weight = stored
            groups, do_grad = self.params[3], self.params[6]
            if not nodel:
                del stored[1]
                del stored[0]
            di = dw = db = None
            if self.is_depthwise or groups != 1:
                di, dw, db = F.depthwise_bwd(grad_output, input_, weight, *self.params[:4],
                                             need=do_grad)
            else:
                if convtype in (0, 2) and input_ is not None and (do_grad[1] or do_grad[2]):
                    dw, db = self._wgrad(input_.detach(), grad_output, wt_variant, do_grad[2])
                    if not do_grad[1]:
                        dw = None
                del input_
                if convtype in (1, 2) and weight is not None and do_grad[0]:
                    di = self._dgrad(grad_output, weight.detach(), ip_variant)
            if do_grad[2]:
                return di, dw, db
            return di, dw


@implements(['aten::_convolution'], ['none'])
class PytorchConvolution(_ConvBase):
    """Default-variant convolution (the reference's cuDNN-benchmark op, conv.py:11-39)."""

    def forward(self, input_, weight, bias, stride, padding, dilation, transposed,
                output_padding, groups, *args, **kwargs):
        with torch.no_grad():
            self._remember(input_, weight, bias, stride, padding, dilation, groups, transposed, output_padding)
            if transposed:
                return self._forward_transposed(input_.detach(), weight.detach(), bias, 0)
            return self._fprop(input_.detach(), weight.detach(), bias, 0)

    def backward(self, grad_output, stored, nodel=False):
        return self._backward(grad_output, stored, nodel, 2, 0, 0)


@implements(['aten::_convolution'], ['normal', 'multiway_newnode', 'multiway', 'newnode'])
class GreedyAlgoConvolution(_ConvBase):
    """Autotunes each pass on first use: fastest variant that stays inside the memory budget."""
    fwd_algo = -1
    bwd_ip_algo = -1
    bwd_wt_algo = -1

    @staticmethod
    def _tune(count, run):
        best, best_t = -1, None
        limit = _budget_gb() * 1.01
        for alg in range(count):
            try:
                torch.cuda.reset_peak_memory_stats()
                torch.cuda.synchronize()
                t0 = time()
                for _ in range(10):
                    out = run(alg)
                    del out
                torch.cuda.synchronize()
                dt = time() - t0
                if torch.cuda.max_memory_allocated() / 2 ** 30 < limit and (best_t is None or dt < best_t):
                    best, best_t = alg, dt
            except RuntimeError:
                continue
        if best < 0:
            raise RuntimeError("no convolution variant fits the memory budget")
        return best

    def forward(self, input_, weight, bias, stride, padding, dilation, transposed,
                output_padding, groups, *args, **kwargs):
        with torch.no_grad():
            self._remember(input_, weight, bias, stride, padding, dilation, groups, transposed, output_padding)
            x, w = input_.detach(), weight.detach()
            if transposed:
                return self._forward_transposed(x, w, bias, 0)
            if self.is_depthwise or groups != 1:
                return self._fprop(x, w, bias, 0)
            if self.fwd_algo == -1:
                self.fwd_algo = self._tune(self.n_fwd_algos(), lambda a: self._fprop(x, w, bias, a))
            return self._fprop(x, w, bias, self.fwd_algo)

    def backward(self, grad_output, stored, nodel=False):
        convtype = self.algorithm // 10 if self.algorithm >= 0 else 2
        if not (self.is_depthwise or self.params[3] != 1 or self.params[7]):
            x, w = stored
            do_grad = self.params[6]
            with torch.no_grad():
                if convtype in (0, 2) and self.bwd_wt_algo == -1 and x is not None and do_grad[1]:
                    self.bwd_wt_algo = self._tune(
                        self.n_bwd_wt_algos(), lambda a: self._wgrad(x.detach(), grad_output, a, False))
                if convtype in (1, 2) and self.bwd_ip_algo == -1 and w is not None and do_grad[0]:
                    self.bwd_ip_algo = self._tune(
                        self.n_bwd_ip_algos(), lambda a: self._dgrad(grad_output, w.detach(), a))
            del x, w
        return self._backward(grad_output, stored, nodel, convtype,
                              max(self.bwd_wt_algo, 0), max(self.bwd_ip_algo, 0))


@implements(['aten::_convolution'], ['conv_multiway_newnode', 'conv_normal'])
class SpecificAlgoConvolution(_ConvBase):
    """The solver chooses the variant of every pass through ``op.algorithm``."""

    def forward(self, input_, weight, bias, stride, padding, dilation, transposed,
                output_padding, groups, *args, **kwargs):
        with torch.no_grad():
            self._remember(input_, weight, bias, stride, padding, dilation, groups, transposed, output_padding)
            if transposed:
                return self._forward_transposed(input_.detach(), weight.detach(), bias, self.algorithm)
            return self._fprop(input_.detach(), weight.detach(), bias, self.algorithm)

    def backward(self, grad_output, stored, nodel=False):
        algorithm = self.algorithm
        if algorithm < 0:
            convtype, algo = 2, 0
        else:
            convtype, algo = algorithm // 10, algorithm % 10
        return self._backward(grad_output, stored, nodel, convtype, algo, algo)
