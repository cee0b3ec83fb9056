"""monet_b200: sm_100a kernels behind MONeT's low-memory operator interface.

``monet_b200.lm_ops``      operator classes + registry (drop-in for monet/lm_ops)
``monet_b200.functional``  tensor-level wrappers of the C ABI
``monet_b200.build``       builds ``libmonet_b200.so`` in-tree with nvcc
"""
__version__ = "0.1.0"
