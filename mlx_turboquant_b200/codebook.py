"""Lloyd-Max codebooks and the scalar quantizer (reference: mlx_turboquant/codebook.py).

Codebook construction is one-off host work (NumPy, float64 like the reference); the sixteen tables the
reference ships (d in {64, 96, 128, 256} x bits in {1..4}) are stored bit-exactly in
``codebooks/shipped_codebooks.json`` and always preferred, because a boundary is the float32 cast of a
float64 midpoint and must be loaded, never recomputed from float32 centroids.  ``quantize_scalar`` and
``dequantize_scalar`` run on the GPU.
"""

from __future__ import annotations

import json
import math
import os
from pathlib import Path

import numpy as np
import torch

from . import _lib

CODEBOOK_DIR = Path(__file__).parent / "codebooks"

_host_cache: dict[tuple[int, int], tuple[np.ndarray, np.ndarray]] = {}
_device_cache: dict[tuple[int, int, str], tuple[torch.Tensor, torch.Tensor]] = {}
_shipped: dict | None = None


def _user_cache_dir() -> Path:
    """User-writable cache for codebooks computed at run time (codebook.py:19-28)."""
    base = os.environ.get("XDG_CACHE_HOME") or os.environ.get("MLX_TURBOQUANT_CACHE")
    if base:
        return Path(base) / "mlx_turboquant"
    return Path.home() / ".cache" / "mlx_turboquant"


def beta_pdf(x: np.ndarray, d: int) -> np.ndarray:
    """Density of one coordinate of a rotated unit vector in d dimensions (codebook.py:36-46)."""
    from scipy import special

    alpha = (d - 1) / 2.0
    log_norm = special.gammaln(2 * alpha) - 2 * special.gammaln(alpha) - (2 * alpha - 1) * math.log(2)
    return np.exp(log_norm + (alpha - 1) * np.log(np.maximum(1 - x * x, 1e-300)))


def gaussian_pdf(x: np.ndarray, d: int) -> np.ndarray:
    """N(0, 1/d) (codebook.py:49-52)."""
    var = 1.0 / d
    return np.exp(-0.5 * x * x / var) / math.sqrt(2 * math.pi * var)


def _grid(d: int, grid_size: int):
    sigma = 1.0 / math.sqrt(d)
    lo, hi = -6 * sigma, 6 * sigma
    grid = np.linspace(lo, hi, grid_size)
    dx = grid[1] - grid[0]
    pdf = gaussian_pdf(grid, d) if d >= 32 else beta_pdf(grid, d)
    return lo, hi, grid, dx, pdf / (np.sum(pdf) * dx)


def _cells(grid, edges, levels):
    for i in range(levels):
        upper = (grid <= edges[i + 1]) if i == levels - 1 else (grid < edges[i + 1])
        yield i, (grid >= edges[i]) & upper


def lloyd_max(d: int, bits: int, num_iter: int = 500, grid_size: int = 10000) -> tuple[np.ndarray, np.ndarray]:
    """Optimal scalar codebook for rotated unit-sphere coordinates (codebook.py:55-116)."""
    levels = 1 << bits
    lo, hi, grid, dx, pdf = _grid(d, grid_size)
    cdf = np.cumsum(pdf) * dx
    cdf = cdf / cdf[-1]
    cent = np.interp(np.linspace(0.5 / levels, 1 - 0.5 / levels, levels), cdf, grid)
    for _ in range(num_iter):
        edges = np.concatenate([[lo], (cent[:-1] + cent[1:]) / 2.0, [hi]])
        new = np.zeros(levels)
        for i, m in _cells(grid, edges, levels):
            w = pdf[m]
            new[i] = np.sum(grid[m] * w) / w.sum() if w.sum() > 0 else cent[i]
        if np.max(np.abs(new - cent)) < 1e-12:
            break
        cent = new
    return cent.astype(np.float32), ((cent[:-1] + cent[1:]) / 2.0).astype(np.float32)


def compute_theoretical_mse(d: int, bits: int, centroids: np.ndarray, boundaries: np.ndarray,
                            grid_size: int = 10000) -> float:
    """Expected squared error per coordinate of a codebook (codebook.py:119-143)."""
    lo, hi, grid, dx, pdf = _grid(d, grid_size)
    edges = np.concatenate([[lo], boundaries, [hi]])
    return float(sum(np.sum((grid[m] - centroids[i]) ** 2 * pdf[m]) * dx for i, m in _cells(grid, edges, len(centroids))))


def _shipped_table() -> dict:
    global _shipped
    if _shipped is None:
        path = CODEBOOK_DIR / "shipped_codebooks.json"
        _shipped = json.loads(path.read_text()) if path.exists() else {}
    return _shipped


def _hex_to_f32(words) -> np.ndarray:
    return np.array([int(h, 16) for h in words], dtype=np.uint32).view(np.float32)


def get_codebook_host(d: int, bits: int) -> tuple[np.ndarray, np.ndarray]:
    """(centroids, boundaries) as float32 NumPy arrays: shipped table, user cache, else computed."""
    key = (d, bits)
    if key not in _host_cache:
        name = f"d{d}_b{bits}"
        user_path = _user_cache_dir() / f"codebook_d{d}_b{bits}.npz"
        if name in _shipped_table():
            e = _shipped_table()[name]
            _host_cache[key] = (_hex_to_f32(e["centroids"]), _hex_to_f32(e["boundaries"]))
        elif user_path.exists():
            z = np.load(user_path)
            _host_cache[key] = (z["centroids"], z["boundaries"])
        else:
            c, b = lloyd_max(d, bits)
            _host_cache[key] = (c, b)
            try:
                user_path.parent.mkdir(parents=True, exist_ok=True)
                np.savez(user_path, centroids=c, boundaries=b)
            except OSError:
                pass
    return _host_cache[key]


def get_codebook(d: int, bits: int, device="cuda") -> tuple[torch.Tensor, torch.Tensor]:
    """Float32 (centroids, boundaries) tensors on ``device`` (codebook.py:146-174)."""
    device = torch.device(device)
    if device.type == "cuda" and device.index is None:
        device = torch.device("cuda", torch.cuda.current_device())
    key = (d, bits, str(device))
    if key not in _device_cache:
        c, b = get_codebook_host(d, bits)
        _device_cache[key] = (torch.from_numpy(np.array(c, dtype=np.float32)).to(device),
                              torch.from_numpy(np.array(b, dtype=np.float32)).to(device))
    return _device_cache[key]


def precompute_codebooks(dims=(64, 96, 128, 256), bits_range=(2, 3, 4), target_dir: Path | None = None) -> None:
    """Compute and save codebooks as .npz files (codebook.py:177-200)."""
    out_dir = target_dir if target_dir is not None else _user_cache_dir()
    out_dir.mkdir(parents=True, exist_ok=True)
    for d in dims:
        for b in bits_range:
            path = out_dir / f"codebook_d{d}_b{b}.npz"
            if not path.exists():
                c, bd = lloyd_max(d, b)
                np.savez(path, centroids=c, boundaries=bd)


def quantize_scalar(x: torch.Tensor, centroids: torch.Tensor, boundaries: torch.Tensor) -> torch.Tensor:
    """uint8 index = number of boundaries strictly exceeded (codebook.py:203-225)."""
    dev = _lib.require_cuda(x, boundaries)
    xf = x.to(torch.float32).contiguous()
    b = boundaries.to(torch.float32).contiguous()
    out = torch.empty(x.shape, dtype=torch.uint8, device=dev)
    _lib.check(_lib.launch(dev, "tq_quantize_scalar", xf.data_ptr(), b.data_ptr(), b.numel(), out.data_ptr(), xf.numel(),
                           _lib.stream_ptr(dev)))
    return out


def dequantize_scalar(indices: torch.Tensor, centroids: torch.Tensor) -> torch.Tensor:
    """centroids[indices] as float32 (codebook.py:228-238)."""
    dev = _lib.require_cuda(indices, centroids)
    idx = indices.to(torch.uint8).contiguous()
    c = centroids.to(torch.float32).contiguous()
    out = torch.empty(indices.shape, dtype=torch.float32, device=dev)
    _lib.check(_lib.launch(dev, "tq_dequantize_scalar", idx.data_ptr(), c.data_ptr(), c.numel(), out.data_ptr(), idx.numel(),
                           _lib.stream_ptr(dev)))
    return out
