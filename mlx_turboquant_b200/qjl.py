"""1-bit quantized Johnson-Lindenstrauss sketch (reference: mlx_turboquant/qjl.py).

The projection matrix is built on the host with the reference's seed and generator (qjl.py:23-36).
The two stand-alone functions run as float32 CUDA kernels of the library (``tq_qjl_quantize`` /
``tq_qjl_dequantize``); the sketch that the cache keeps per token is produced inside the fused quantize
kernel instead.
"""

from __future__ import annotations

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
    dev = _lib.require_cuda(residual, projection)
    m, d = projection.shape
    if residual.shape[-1] != d:
        raise ValueError(f"residual has {residual.shape[-1]} coordinates, the projection {d}")
    lead = residual.shape[:-1]
    r = residual.reshape(-1, d).to(torch.float32).contiguous()
    s = projection.to(torch.float32).contiguous()
    signs = torch.empty(r.shape[0], m, dtype=torch.bool, device=dev)
    norms = torch.empty(r.shape[0], dtype=torch.float32, device=dev)
    _lib.check(_lib.launch(dev, "tq_qjl_quantize", r.data_ptr(), s.data_ptr(), signs.data_ptr(), norms.data_ptr(), r.shape[0], d, m,
                           _lib.stream_ptr(dev)))
    return signs.reshape(*lead, m), norms.reshape(lead)


def qjl_dequantize(signs: torch.Tensor, norms: torch.Tensor, projection: torch.Tensor, d: int) -> torch.Tensor:
    """(sqrt(pi/2)/d) * gamma * (z @ S), z = +-1 (qjl.py:70-94)."""
    dev = _lib.require_cuda(signs, norms, projection)
    m = projection.shape[0]
    if projection.shape[1] != d or signs.shape[-1] != m:
        raise ValueError(f"projection {tuple(projection.shape)} does not match d={d} / {signs.shape[-1]} signs")
    lead = signs.shape[:-1]
    z = signs.reshape(-1, m).to(torch.bool).contiguous()
    g = norms.reshape(-1).to(torch.float32).contiguous()
    s = projection.to(torch.float32).contiguous()
    out = torch.empty(z.shape[0], d, dtype=torch.float32, device=dev)
    _lib.check(_lib.launch(dev, "tq_qjl_dequantize", z.data_ptr(), g.data_ptr(), s.data_ptr(), out.data_ptr(), z.shape[0], d, m,
                           _lib.stream_ptr(dev)))
    return out.reshape(*lead, d)
