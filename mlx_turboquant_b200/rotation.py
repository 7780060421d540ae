"""Seed-fixed orthogonal rotation (reference: mlx_turboquant/rotation.py).

The matrix itself is built once on the host with NumPy, exactly as the reference does
(QR of a seeded Gaussian, rotation.py:17-36), so that the same bits feed the GPU kernels and
any CPU checker; applying it is a CUDA kernel (``tq_rotate``).
"""

from __future__ import annotations

import numpy as np
import torch

from . import _lib

DEFAULT_SEED = 42

_host_cache: dict[tuple[int, int], np.ndarray] = {}
_device_cache: dict[tuple[int, int, str], torch.Tensor] = {}


def generate_rotation_matrix_host(d: int, seed: int = DEFAULT_SEED) -> np.ndarray:
    """(d, d) float32 orthogonal matrix: sign-fixed Q of QR(randn(d, d)) (rotation.py:27-36)."""
    key = (d, seed)
    if key not in _host_cache:
        g = np.random.RandomState(seed).randn(d, d).astype(np.float32)
        q, r = np.linalg.qr(g)
        s = np.sign(np.diag(r))
        s[s == 0] = 1
        _host_cache[key] = np.ascontiguousarray((q * s[np.newaxis, :]).astype(np.float32))
    return _host_cache[key]


def generate_rotation_matrix(d: int, seed: int = DEFAULT_SEED, device="cuda") -> torch.Tensor:
    return torch.from_numpy(generate_rotation_matrix_host(d, seed).copy()).to(device)


def get_rotation_matrix(d: int, seed: int = DEFAULT_SEED, device="cuda") -> torch.Tensor:
    """Cached per (d, seed, device) (rotation.py:39-52)."""
    device = torch.device(device)
    if device.type == "cuda" and device.index is None:
        device = torch.device("cuda", torch.cuda.current_device())
    key = (d, seed, str(device))
    if key not in _device_cache:
        _device_cache[key] = generate_rotation_matrix(d, seed, device)
    return _device_cache[key]


def _apply(x: torch.Tensor, rotation: torch.Tensor, inverse: bool) -> torch.Tensor:
    dev = _lib.require_cuda(x, rotation)
    d = x.shape[-1]
    if rotation.shape != (d, d):
        raise ValueError(f"rotation must be ({d}, {d}), got {tuple(rotation.shape)}")
    rot = rotation.to(torch.float32).contiguous()
    xc = x.contiguous()
    if xc.dtype not in (torch.float16, torch.bfloat16, torch.float32):
        xc = xc.to(torch.float32)
    out = torch.empty(x.shape, dtype=torch.float32, device=dev)
    n = xc.numel() // d if d else 0
    _lib.check(_lib.launch(dev, "tq_rotate", xc.data_ptr(), _lib.dtype_code(xc.dtype), rot.data_ptr(), out.data_ptr(),
                           n, d, 1 if inverse else 0, _lib.stream_ptr(dev)))
    return out


def rotate(x: torch.Tensor, rotation: torch.Tensor) -> torch.Tensor:
    """x @ R.T over the last axis, float32 result (rotation.py:55-65)."""
    return _apply(x, rotation, False)


def inverse_rotate(y: torch.Tensor, rotation: torch.Tensor) -> torch.Tensor:
    """y @ R (rotation.py:68-78)."""
    return _apply(y, rotation, True)


def pre_rotate_query(query: torch.Tensor, rotation: torch.Tensor) -> torch.Tensor:
    """Q @ R.T, the transform that lets scores be taken against packed codes (rotation.py:81-110)."""
    return _apply(query, rotation, False)


def hadamard_matrix(d: int, device="cuda") -> torch.Tensor:
    """Normalised Walsh-Hadamard matrix, d a power of two (rotation.py:113-131)."""
    if d & (d - 1) != 0:
        raise ValueError(f"Dimension {d} must be a power of 2 for Hadamard transform")
    h = np.array([[1.0]], dtype=np.float32)
    while h.shape[0] < d:
        h = np.block([[h, h], [h, -h]])
    return torch.from_numpy((h / np.sqrt(d)).astype(np.float32)).to(device)


def randomized_hadamard(d: int, seed: int = DEFAULT_SEED, device="cuda") -> torch.Tensor:
    """diag(random signs) @ H (rotation.py:134-151)."""
    signs = np.random.RandomState(seed).choice([-1.0, 1.0], size=d).astype(np.float32)
    return torch.from_numpy(signs).to(device)[:, None] * hadamard_matrix(d, device)
