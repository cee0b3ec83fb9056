"""Max-pool implementations in the reference's slot order (monet/lm_ops/pool.py:8-69)."""
from __future__ import annotations

import numpy as np
import torch

from .. import functional as F
from .base import OP, InputStorage, IntermediateStorage, implements


@implements(['aten::max_pool2d'],
            ['normal', 'multiway', 'newnode', 'multiway_newnode', 'conv_multiway_newnode',
             'conv_normal'])
class SimpleMaxPool2D(OP):
    """Keeps the input; the backward recomputes the argmax nibbles from it and then gathers
    (the reference re-runs torch.max_pool2d under autograd, pool.py:26-36)."""
    backward_storage = InputStorage(0)
    params = None

    def forward(self, input_, kernel_size, stride, padding, dilation, ceil_mode):
        self.params = kernel_size, stride, padding, dilation, bool(ceil_mode)
        with torch.no_grad():
            y, _, _ = F.maxpool2d(input_, kernel_size, stride, padding, dilation, ceil_mode,
                                  with_indices=False)
            return y

    def backward(self, grad_output, stored, nodel=False):
        ip = stored[0]
        if not nodel:
            del stored[0]
        with torch.no_grad():
            y, nib, desc = F.maxpool2d(ip, *self.params, with_indices=True)
            del y, ip
            return F.maxpool2d_bwd(grad_output, nib, desc)


@implements(['aten::max_pool2d'], ['newnode', 'multiway_newnode', 'conv_multiway_newnode'])
class IndicesActMaxPool2D(OP):
    """Keeps ceil(E_out/2) bytes of window-local argmax nibbles (two outputs per byte)."""
    backward_storage = IntermediateStorage(lambda shape: (np.prod(shape) + 1) // 2)
    params = None

    def forward(self, input_, kernel_size, stride, padding, dilation, ceil_mode):
        with torch.no_grad():
            y, nib, desc = F.maxpool2d(input_, kernel_size, stride, padding, dilation, ceil_mode,
                                       with_indices=True)
            self.params = (desc,)
            return y, nib

    def backward(self, grad_output, stored, nodel=False):
        with torch.no_grad():
            nib = stored[0]
            if not nodel:
                del stored[0]
            return F.maxpool2d_bwd(grad_output, nib, self.params[0])
