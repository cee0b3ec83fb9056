"""Fully connected layer (monet/lm_ops/linear.py:25-61).  The reference calls the fp32 library
GEMM (``torch.addmm`` / ``mm``); here the three passes run on the tensor-core kernels of the
pointwise convolution (a linear layer is a 1x1 convolution over a 1x1 map), TF32 operands with
fp32 accumulation like every other contraction of the library.  The backward is split into the
weight/bias step and the input step by ``algorithm // 10`` exactly like the convolution."""
from __future__ import annotations

import torch

from .. import functional as F
from .base import COMMON_MODES, OP, InputStorage, implements


@implements(['aten::addmm'], COMMON_MODES)
class LowMemAddMM(OP):
    backward_storage = InputStorage(1, 2)
    params = None
    algorithm = -1

    def forward(self, bias, input_, weight, beta, alpha):
        if alpha != 1 or beta != 1:
            raise NotImplementedError("addmm with alpha/beta != 1")
        self.params = [input_.requires_grad, weight.requires_grad,
                       bias is not None and bias.requires_grad]
        with torch.no_grad():
            return F.linear_fwd(input_, weight, bias.detach() if bias is not None else None)

    def backward(self, output_grad, stores, nodel=False):
        with torch.no_grad():
            step = self.algorithm // 10 if self.algorithm >= 0 else 2
            input_, weight = stores[0], stores[1]
            if not nodel:
                del stores[1]
                del stores[0]
            di = dw = db = None
            if step in (0, 2) and input_ is not None and (self.params[1] or self.params[2]):
                dw, db = F.linear_wgrad(input_, output_grad, bool(self.params[2]))
                if not self.params[1]:
                    dw = None
            if step in (1, 2) and weight is not None and self.params[0]:
                di = F.linear_dgrad(output_grad, weight)
            return db, di, dw
