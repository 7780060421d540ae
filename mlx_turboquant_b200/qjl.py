"""1-bit quantized Johnson-Lindenstrauss sketch (reference: mlx_turboquant/qjl.py).

The projection matrix is built on the host with the reference's seed and generator (qjl.py:23-36).
These two stand-alone functions are small dense products and use torch's matmul on the GPU; the
sketch that the cache keeps per token is produced inside the fused quantize kernel instead.
"""

from __future__ import annotations

import math

import numpy as np
import torch

from . import _lib

DEFAULT_SEED = 12345

_host_cache: dict[tuple[int, int, int], np.ndarray] = {}
_device_cache: dict[tuple[int, int, int, str], torch.Tensor] = {}


def generate_projection_matrix_host(d: int, m: int, seed: int = DEFAULT_SEED) -> np.ndarray:
    key = (d, m, seed)
    if key not in _host_cache:
        _host_cache[key] = np.random.RandomState(seed).randn(m, d).astype(np.float32)
    return _host_cache[key]


def generate_projection_matrix(d: int, m: int, seed: int = DEFAULT_SEED, device="cuda") -> torch.Tensor:
    """(m, d) i.i.d. N(0, 1) float32 (qjl.py:23-36)."""
    return torch.from_numpy(generate_projection_matrix_host(d, m, seed).copy()).to(device)


def get_projection_matrix(d: int, m: int, seed: int = DEFAULT_SEED, device="cuda") -> torch.Tensor:
    device = torch.device(device)
    if device.type == "cuda" and device.index is None:
        device = torch.device("cuda", torch.cuda.current_device())
    key = (d, m, seed, str(device))
    if key not in _device_cache:
        _device_cache[key] = generate_projection_matrix(d, m, seed, device)
    return _device_cache[key]


def qjl_quantize(residual: torch.Tensor, projection: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """signs (..., m) bool = (r @ S.T >= 0); norms (...) = ||r|| (qjl.py:47-67)."""
    _lib.require_cuda(residual, projection)
    norms = torch.linalg.vector_norm(residual, dim=-1)
    return (residual @ projection.T) >= 0, norms


def qjl_dequantize(signs: torch.Tensor, norms: torch.Tensor, projection: torch.Tensor, d: int) -> torch.Tensor:
    """(sqrt(pi/2)/d) * gamma * (z @ S), z = +-1 (qjl.py:70-94)."""
    _lib.require_cuda(signs, norms, projection)
    z = torch.where(signs, 1.0, -1.0).to(projection.dtype)
    return (math.sqrt(math.pi / 2) / d) * norms[..., None] * (z @ projection)
