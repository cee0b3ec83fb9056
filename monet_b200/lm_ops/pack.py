"""Bit and nibble packers with the reference's names and byte formats
(monet/lm_ops/pack.py:9-55, pack.cu:3-50): MSB-first bits, high-nibble-first pairs."""
from __future__ import annotations

import torch

from .. import functional as F


def pack(v: torch.Tensor) -> torch.Tensor:
    """1-D bool tensor -> uint8 tensor of ceil(n/8) bytes, element 8j+k in bit 7-k of byte j."""
    return F.pack_bits(v)


def unpack(p: torch.Tensor, n: int = 0) -> torch.Tensor:
    """Inverse of `pack`; `n` defaults to 8 * len(p)."""
    return F.unpack_bits(p, n if n else p.numel() * 8)


def unpack_multiply(p: torch.Tensor, v: torch.Tensor) -> torch.Tensor:
    """v with the elements whose packed bit is 0 zeroed, without materialising the bools."""
    return F.unpack_multiply(p, v.contiguous()).view(v.shape)


def pack_two(v: torch.Tensor) -> torch.Tensor:
    """1-D uint8 tensor of values < 16 -> ceil(n/2) bytes, element 2j in the high nibble."""
    return F.pack_nibbles(v)


def unpack_two(p: torch.Tensor, n: int = 0) -> torch.Tensor:
    return F.unpack_nibbles(p, n if n else p.numel() * 2)
