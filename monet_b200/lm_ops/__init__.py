"""B200-native implementations of MONeT's low-memory operators.

Importing this package fills ``registry`` in the reference's module order
(monet/lm_ops/__init__.py:2): conv, relu, elementary, pool, linear, bn, cat, hardtanh, funcs.
``softmax`` registers only when imported explicitly, as in the reference.
"""
from .base import (COMMON_MODES, OP, InputStorage, IntermediateStorage, OutputStorage,
                   StorageInfo, all_modes, implements, install_into, list_ops, registry)
from . import conv, relu, elementary, pool, linear, bn, cat, hardtanh, funcs  # noqa: E402,F401
from .elementary import NativeOP  # noqa: F401
