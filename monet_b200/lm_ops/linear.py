"""Fully connected layer (monet/lm_ops/linear.py:25-61).  A plain library GEMM (cuBLAS via
torch) as in the reference; the backward is split into the weight/bias step and the input
step by ``algorithm // 10`` exactly like the convolution."""
from __future__ import annotations

import torch

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
            return torch.addmm(bias, input_, weight.t())

    def backward(self, output_grad, stores, nodel=False):
        with torch.no_grad():
            step = self.algorithm // 10
            input_, weight = stores[0], stores[1]
            if not nodel:
                del stores[1]
                del stores[0]
            di = dw = db = None
            if step in (0, 2) and input_ is not None:
                if self.params[1]:
                    dw = output_grad.t().mm(input_)
                if self.params[2]:
                    db = output_grad.sum(0)
            if step in (1, 2) and weight is not None and self.params[0]:
                di = output_grad.mm(weight)
            return db, di, dw
