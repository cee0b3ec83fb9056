"""hardtanh / ReLU6 implementations in the reference's slot order
(monet/lm_ops/hardtanh.py:9-93)."""
from __future__ import annotations

import torch

from .. import functional as F
from .base import OP, InputStorage, OutputStorage, implements


class _HardTanh(OP):
    params = None
    inplace = False

    def forward(self, x, lower, upper):
        with torch.no_grad():
            self.params = lower, upper
            return F.hardtanh(x, lower, upper, inplace=self.inplace)

    def backward(self, grad_output, stored, nodel=False):
        with torch.no_grad():
            lower, upper = self.params
            saved = stored[0]
            if not nodel:
                del stored[0]
            return F.hardtanh_bwd(grad_output, saved, lower, upper)


@implements(['aten::hardtanh'],
            ['normal', 'multiway', 'newnode', 'multiway_newnode', 'conv_multiway_newnode',
             'conv_normal'])
class InputActHardTanh(_HardTanh):
    backward_storage = InputStorage(0)


@implements(['aten::hardtanh'], ['multiway', 'multiway_newnode', 'conv_multiway_newnode'])
class OutputActHardTanh(_HardTanh):
    backward_storage = OutputStorage()


@implements(['aten::hardtanh_'], ['multiway', 'newnode', 'multiway_newnode', 'conv_multiway_newnode'])
class InputActHardTanhIP(_HardTanh):
    backward_storage = InputStorage(0)


@implements(['aten::hardtanh_'],
            ['normal', 'multiway', 'multiway_newnode', 'conv_multiway_newnode', 'conv_normal'])
class OutputActHardTanhIP(_HardTanh):
    backward_storage = OutputStorage()
