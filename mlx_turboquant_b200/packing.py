"""Bit-packing of 1/2/3/4-bit indices into uint8 (reference: mlx_turboquant/packing.py).

Byte layouts are the reference's: 4-bit ``v0 | v1<<4``; 2-bit ``v0 | v1<<2 | v2<<4 | v3<<6``; 1-bit
bit i = v_i; 3-bit packs 8 codes into 3 bytes, little-endian.  The work runs in ``tq_pack`` / ``tq_unpack``.
"""

from __future__ import annotations

import torch

from . import _lib

_PER = {1: 8, 2: 4, 3: 8, 4: 2}


def _check_bits(bits: int) -> None:
    if bits not in _PER:
        raise ValueError(f"Unsupported bit-width: {bits}. Use 1, 2, 3, or 4.")


def pack_indices(indices: torch.Tensor, bits: int) -> torch.Tensor:
    """(..., d) uint8 -> (..., d*bits/8) uint8 (packing.py:211-222)."""
    _check_bits(bits)
    d = indices.shape[-1]
    assert d % _PER[bits] == 0, f"Last dimension {d} must be divisible by {_PER[bits]} for {bits}-bit packing"
    dev = _lib.require_cuda(indices)
    idx = indices.to(torch.uint8).contiguous()
    out = torch.empty(*indices.shape[:-1], d * bits // 8, dtype=torch.uint8, device=dev)
    n = idx.numel() // d if d else 0
    _lib.check(_lib.launch(dev, "tq_pack", idx.data_ptr(), out.data_ptr(), n, d, bits, _lib.stream_ptr(dev)))
    return out


def unpack_indices(packed: torch.Tensor, bits: int, d: int) -> torch.Tensor:
    """(..., d*bits/8) uint8 -> (..., d) uint8 (packing.py:225-236)."""
    _check_bits(bits)
    dev = _lib.require_cuda(packed)
    p = packed.to(torch.uint8).contiguous()
    w = d * bits // 8
    if p.shape[-1] != w:
        raise ValueError(f"packed last dimension {p.shape[-1]} does not match d={d} at {bits} bits ({w})")
    out = torch.empty(*packed.shape[:-1], d, dtype=torch.uint8, device=dev)
    n = p.numel() // w if w else 0
    _lib.check(_lib.launch(dev, "tq_unpack", p.data_ptr(), out.data_ptr(), n, d, bits, _lib.stream_ptr(dev)))
    return out


def pack_1bit(indices): return pack_indices(indices, 1)
def pack_2bit(indices): return pack_indices(indices, 2)
def pack_3bit(indices): return pack_indices(indices, 3)
def pack_4bit(indices): return pack_indices(indices, 4)
def unpack_1bit(packed, d): return unpack_indices(packed, 1, d)
def unpack_2bit(packed, d): return unpack_indices(packed, 2, d)
def unpack_3bit(packed, d): return unpack_indices(packed, 3, d)
def unpack_4bit(packed, d): return unpack_indices(packed, 4, d)
