"""TurboQuant quantizers on torch tensors (reference: mlx_turboquant/quantizer.py)."""

from __future__ import annotations

from dataclasses import dataclass

import torch

from . import kernels
from .codebook import get_codebook
from .qjl import get_projection_matrix, qjl_dequantize, qjl_quantize
from .rotation import get_rotation_matrix


@dataclass
class QuantizedTensor:
    """Compressed representation of a batch of vectors (quantizer.py:21-30)."""
    packed_indices: torch.Tensor   # bit-packed codes, uint8
    norms: torch.Tensor            # L2 norms, float32
    bits: int
    d: int
    qjl_signs: torch.Tensor | None = None   # TurboQuantProd only: (..., m) bool
    qjl_norms: torch.Tensor | None = None   # TurboQuantProd only: (...) float32


class TurboQuantMSE:
    """Algorithm 1: normalise, rotate, Lloyd-Max per coordinate, store codes + norm (quantizer.py:33-109)."""

    def __init__(self, d: int, bits: int = 4, seed: int = 42, device="cuda"):
        self.d, self.bits, self.seed = d, bits, seed
        self.rotation = get_rotation_matrix(d, seed, device)
        self.centroids, self.boundaries = get_codebook(d, bits, device)

    def quantize(self, x: torch.Tensor) -> QuantizedTensor:
        """(..., d) -> packed (..., d*bits/8) uint8 + norms (...) float32; a bare (d,) vector works too."""
        lead = x.shape[:-1]
        flat = x.reshape(-1, self.d)
        packed, _, norms = kernels.quantize_pack(flat, self.rotation, self.boundaries, self.bits)
        return QuantizedTensor(packed.reshape(*lead, -1), norms.reshape(lead), self.bits, self.d)

    def dequantize(self, qt: QuantizedTensor) -> torch.Tensor:
        lead = qt.norms.shape
        n = qt.norms.numel()
        out = kernels.dequantize(qt.packed_indices.reshape(n, -1), qt.norms.reshape(n), self.centroids,
                                 self.rotation, qt.bits, qt.d)
        return out.reshape(*lead, qt.d)


class TurboQuantProd:
    """Algorithm 2: (bits-1)-bit MSE stage + 1-bit QJL sketch of the residual (quantizer.py:112-195)."""

    def __init__(self, d: int, bits: int = 4, qjl_dim: int | None = None, seed: int = 42,
                 qjl_seed: int = 12345, device="cuda"):
        self.d, self.bits = d, bits
        self.qjl_dim = qjl_dim or d
        self.mse = TurboQuantMSE(d, bits=bits - 1, seed=seed, device=device)
        self.projection = get_projection_matrix(d, self.qjl_dim, qjl_seed, device)

    def quantize(self, x: torch.Tensor) -> QuantizedTensor:
        qt = self.mse.quantize(x)
        residual = x.to(torch.float32) - self.mse.dequantize(qt)
        signs, gamma = qjl_quantize(residual, self.projection)
        return QuantizedTensor(qt.packed_indices, qt.norms, self.bits, self.d, signs, gamma)

    def dequantize(self, qt: QuantizedTensor) -> torch.Tensor:
        x_hat = self.mse.dequantize(QuantizedTensor(qt.packed_indices, qt.norms, self.bits - 1, self.d))
        if qt.qjl_signs is not None and qt.qjl_norms is not None:
            return x_hat + qjl_dequantize(qt.qjl_signs, qt.qjl_norms, self.projection, self.d)
        return x_hat
