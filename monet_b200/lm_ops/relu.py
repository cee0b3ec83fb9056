"""ReLU implementations, in the reference's slot order (monet/lm_ops/relu.py:9-118):
keep the input, keep the output, or keep a 1-bit mask."""
from __future__ import annotations

import numpy as np
import torch

from .. import functional as F
from .base import OP, InputStorage, IntermediateStorage, OutputStorage, implements


class _ActReLU(OP):
    """Backward gates the gradient by `saved > 0`, in place on the gradient like
    relu_backward in lrrelu.cpp:11-20."""
    params = None
    inplace = False

    def forward(self, x):
        with torch.no_grad():
            return F.relu(x, inplace=self.inplace)

    def backward(self, grad_output, stored, nodel=False):
        with torch.no_grad():
            saved = stored[0]
            if not nodel:
                del stored[0]
            return F.relu_bwd_act(grad_output, saved, 0.0, inplace=True)


@implements(['aten::relu', 'aten::relu_'],
            ['normal', 'multiway', 'newnode', 'multiway_newnode', 'conv_multiway_newnode'])
class InputActReLU(_ActReLU):
    backward_storage = InputStorage(0)


@implements(['aten::relu', 'aten::relu_'],
            ['multiway', 'multiway_newnode', 'conv_multiway_newnode', 'conv_normal'])
class OutputActReLU(_ActReLU):
    backward_storage = OutputStorage()


@implements(['aten::relu', 'aten::relu_'], ['newnode', 'multiway_newnode', 'conv_multiway_newnode'])
class BinaryActReLU(OP):
    """Keeps ceil(E/8) bytes: bit = (x > 0), packed in the physical element order of x.
    One fused kernel produces y and the mask (the reference runs clamp, compare and pack
    kernels with an E-byte bool temporary, relu.py:100-104)."""
    backward_storage = IntermediateStorage(lambda shape: (np.prod(shape) + 7) // 8)
    params = None
    inplace = False

    def forward(self, x):
        with torch.no_grad():
            y, mask = F.relu_mask(x, inplace=self.inplace)
            self.params = (F.is_nhwc(y),)
            return y, mask

    def intermediate(self, x):
        with torch.no_grad():
            return F.pack_bits((F.dense(x) > 0))

    def backward(self, grad_output, stored, nodel=False):
        with torch.no_grad():
            mask = stored[0]
            if not nodel:
                del stored[0]
            g = grad_output
            if g.dim() == 4 and self.params is not None:
                fmt = torch.channels_last if self.params[0] else torch.contiguous_format
                g = g.contiguous(memory_format=fmt)
            return F.relu_bwd_mask(g, mask, inplace=True)
