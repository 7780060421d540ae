"""Python entry points of the fused CUDA kernels (reference: mlx_turboquant/kernels.py).

The reference's device code is Metal; here the same operations are sm_100a CUDA kernels behind
``libtq_b200.so``.  Kept by name from the reference: ``metal_dequantize`` / ``metal_quantize_4bit``
(aliases of :func:`dequantize` / :func:`quantize_4bit`) and ``fused_qk_scores_{2,3,4}bit``.  New here:
:func:`quantize_pack` (all bit widths, fractional split, optional QJL sketch) and
:func:`decode_attention`, attention over the packed cache that the reference only prototyped.
"""

from __future__ import annotations

import ctypes as C

import torch

from . import _lib
from .rotation import get_rotation_matrix  # noqa: F401  (re-exported for convenience)


def split_bits(bits: float) -> tuple[int, int]:
    """(bits_hi, bits_lo): 3.5 -> (4, 3); integer b -> (b, 0)  (cache.py:64-73)."""
    if bits != int(bits):
        return int(bits) + 1, int(bits)
    return int(bits), 0


def packed_widths(d: int, bits_hi: int, bits_lo: int) -> tuple[int, int]:
    half = d // 2 if bits_lo else d
    return half * bits_hi // 8, ((d - half) * bits_lo // 8 if bits_lo else 0)


def quantize_pack(x: torch.Tensor, rotation: torch.Tensor, boundaries_hi: torch.Tensor, bits_hi: int,
                  boundaries_lo: torch.Tensor | None = None, bits_lo: int = 0, *,
                  out_hi: torch.Tensor | None = None, out_lo: torch.Tensor | None = None,
                  out_norms: torch.Tensor | None = None, out_offset: int = 0,
                  qjl: dict | None = None, return_rotated: bool = False):
    """norm -> normalise -> rotate -> Lloyd-Max boundary count -> bit-pack, one kernel.

    ``x`` is (..., T, d); the last two axes are (rows, d) and everything before is flattened into
    lanes, so a (B, H, T, d) slice of a larger buffer works without a copy as long as the row stride
    is uniform.  Returns ``(packed_hi, packed_lo | None, norms)`` shaped (..., T, width) / (..., T).

    ``out_*`` + ``out_offset`` write rows at token offset ``out_offset`` of preallocated
    (lanes..., capacity, width) storage instead of allocating.  ``qjl`` = dict(proj_rot, cent_hi,
    cent_lo, bits, gamma) also emits the 1-bit sketch of the residual.
    """
    q_bufs = () if qjl is None else (qjl.get("proj_rot"), qjl.get("cent_hi"), qjl.get("cent_lo"), qjl.get("bits"), qjl.get("gamma"))
    dev = _lib.require_cuda(x, rotation, boundaries_hi, boundaries_lo, out_hi, out_lo, out_norms, *q_bufs)
    d = x.shape[-1]
    if x.dim() < 2:
        x = x.reshape(1, d)
    t = x.shape[-2]
    lead = x.shape[:-2]
    lanes = 1
    for s in lead:
        lanes *= s
    if x.dtype not in (torch.float16, torch.bfloat16, torch.float32):
        x = x.to(torch.float32)
    # lanes must be addressable with a single stride
    xv = x.reshape(lanes, t, d) if x.is_contiguous() else _uniform_lanes(x, lanes, t, d)
    w_hi, w_lo = packed_widths(d, bits_hi, bits_lo)
    if out_hi is None:
        out_hi = torch.empty(lanes, t, w_hi, dtype=torch.uint8, device=dev)
        out_lo = torch.empty(lanes, t, w_lo, dtype=torch.uint8, device=dev) if bits_lo else None
        out_norms = torch.empty(lanes, t, dtype=torch.float32, device=dev)
        cap, fresh = t, True
    else:
        cap, fresh = out_hi.shape[-2], False
        assert out_norms is not None and out_hi.is_contiguous() and out_norms.is_contiguous()
        assert out_offset + t <= cap
    a = _lib.QuantizeArgs()
    a.x, a.x_dtype, a.d = xv.data_ptr(), _lib.dtype_code(xv.dtype), d
    a.n_lanes, a.n_rows = lanes, t
    a.x_lane_stride, a.x_row_stride = (xv.stride(0) if lanes > 1 else 0), xv.stride(1) if t > 1 else d
    rot = rotation if rotation.dtype == torch.float32 and rotation.is_contiguous() else rotation.float().contiguous()
    a.rot = rot.data_ptr()
    a.bnd_hi, a.bits_hi = boundaries_hi.data_ptr(), bits_hi
    a.bnd_lo, a.bits_lo = (boundaries_lo.data_ptr() if bits_lo else None), bits_lo
    a.packed_hi = out_hi.data_ptr() + out_offset * w_hi
    a.packed_lo = (out_lo.data_ptr() + out_offset * w_lo) if bits_lo else None
    a.norms = out_norms.data_ptr() + out_offset * 4
    a.out_lane_stride = cap
    y = None
    if return_rotated:
        y = torch.empty(lanes, t, d, dtype=torch.float32, device=dev)
        a.y_out = y.data_ptr()
    if qjl is not None:
        a.qjl_proj_rot = qjl["proj_rot"].data_ptr()
        a.cent_hi = qjl["cent_hi"].data_ptr()
        a.cent_lo = qjl["cent_lo"].data_ptr() if bits_lo else None
        a.qjl_bits = qjl["bits"].data_ptr() + out_offset * 4
        a.qjl_gamma = qjl["gamma"].data_ptr() + out_offset * 4
    _lib.check(_lib.launch(dev, "tq_quantize_pack", C.byref(a), _lib.stream_ptr(dev)))
    if fresh:
        out_hi = out_hi.reshape(*lead, t, w_hi)
        out_lo = out_lo.reshape(*lead, t, w_lo) if bits_lo else None
        out_norms = out_norms.reshape(*lead, t)
    if return_rotated:
        return out_hi, out_lo, out_norms, y.reshape(*lead, t, d)
    return out_hi, out_lo, out_norms


def _uniform_lanes(x: torch.Tensor, lanes: int, t: int, d: int) -> torch.Tensor:
    """View x (..., t, d) as (lanes, t, d) with one lane stride, copying only if that is impossible."""
    if x.stride(-1) == 1:
        try:
            return x.view(lanes, t, d)
        except RuntimeError:
            pass
    return x.contiguous().reshape(lanes, t, d)


def dequantize_rows(packed_hi: torch.Tensor, packed_lo: torch.Tensor | None, norms: torch.Tensor,
                    rotation: torch.Tensor, centroids_hi: torch.Tensor, bits_hi: int,
                    centroids_lo: torch.Tensor | None, bits_lo: int, d: int, *, n_rows: int | None = None,
                    in_offset: int = 0, out: torch.Tensor | None = None, out_offset: int = 0, out_dtype=torch.float32,
                    qjl: dict | None = None) -> torch.Tensor:
    """unpack -> centroid -> inverse rotation -> scale.

    packed is (lanes..., cap, width); rows [in_offset, in_offset + n_rows) of every lane are expanded
    into ``out`` (lanes..., out_cap, d) starting at row ``out_offset`` (a fresh tensor if ``out`` is None).
    """
    q_bufs = () if qjl is None else (qjl.get("proj"), qjl.get("bits"), qjl.get("gamma"))
    dev = _lib.require_cuda(packed_hi, packed_lo, norms, rotation, centroids_hi, centroids_lo, out, *q_bufs)
    cap = packed_hi.shape[-2]
    t = cap - in_offset if n_rows is None else n_rows
    assert in_offset + t <= cap
    lead = packed_hi.shape[:-2]
    lanes = 1
    for s in lead:
        lanes *= s
    assert packed_hi.is_contiguous() and norms.is_contiguous()
    if out is None:
        out = torch.empty(*lead, t, d, dtype=out_dtype, device=dev)
        out_cap, out_offset = t, 0
    else:
        assert out.is_contiguous() and out.shape[-1] == d
        out_cap = out.shape[-2]
    a = _lib.DequantizeArgs()
    w_hi, w_lo = packed_widths(d, bits_hi, bits_lo)
    a.packed_hi = packed_hi.data_ptr() + in_offset * w_hi
    a.packed_lo = (packed_lo.data_ptr() + in_offset * w_lo) if bits_lo else None
    a.norms = norms.data_ptr() + in_offset * 4
    a.n_lanes, a.n_rows, a.in_lane_stride = lanes, t, cap
    a.d, a.bits_hi, a.bits_lo = d, bits_hi, bits_lo
    a.cent_hi, a.cent_lo = centroids_hi.data_ptr(), (centroids_lo.data_ptr() if bits_lo else None)
    rot = rotation if rotation.dtype == torch.float32 and rotation.is_contiguous() else rotation.float().contiguous()
    a.rot = rot.data_ptr()
    if qjl is not None:
        a.qjl_proj = qjl["proj"].data_ptr()
        a.qjl_bits, a.qjl_gamma = qjl["bits"].data_ptr() + in_offset * 4, qjl["gamma"].data_ptr() + in_offset * 4
    a.out = out.data_ptr() + out_offset * d * out.element_size()
    a.out_dtype = _lib.dtype_code(out.dtype)
    a.out_lane_stride, a.out_row_stride = out_cap * d, d
    _lib.check(_lib.launch(dev, "tq_dequantize", C.byref(a), _lib.stream_ptr(dev)))
    return out


def dequantize(packed: torch.Tensor, norms: torch.Tensor, centroids: torch.Tensor, rotation: torch.Tensor,
               bits: int, d: int) -> torch.Tensor:
    """Fused dequantize, (N, packed_dim) uint8 + (N,) norms -> (N, d) float32 (kernels.py:313-360)."""
    if bits not in (1, 2, 3, 4):
        raise ValueError(f"dequantize only supports 1, 2, 3, 4 bits, got {bits}")
    n = norms.shape[0]
    p = packed.reshape(n, -1).contiguous()
    nr = norms.reshape(n).to(torch.float32).contiguous()
    return dequantize_rows(p, None, nr, rotation, centroids.float().contiguous(), bits, None, 0, d)


def quantize_4bit(inp: torch.Tensor, rotation: torch.Tensor, boundaries: torch.Tensor):
    """Fused 4-bit quantize: (N, D) -> (packed (N, D/2) uint8, norms (N,) float32) (kernels.py:363-409)."""
    packed, _, norms = quantize_pack(inp, rotation, boundaries.float().contiguous(), 4)
    return packed, norms


metal_dequantize = dequantize
metal_quantize_4bit = quantize_4bit


def _fused_qk(q_rot, packed_k, norms_k, centroids, D, bits):
    dev = _lib.require_cuda(q_rot, packed_k, norms_k, centroids)
    t_q, t_kv = q_rot.shape[0], packed_k.shape[0]
    out = torch.zeros(t_q, t_kv, dtype=torch.float32, device=dev)
    if t_q == 0 or t_kv == 0:
        return out
    q = q_rot.to(torch.float32).contiguous()
    pk, nk, ce = packed_k.contiguous(), norms_k.to(torch.float32).contiguous(), centroids.to(torch.float32).contiguous()
    _lib.check(_lib.launch(dev, "tq_qk_scores", q.data_ptr(), pk.data_ptr(), nk.data_ptr(), ce.data_ptr(), bits, D, t_q, t_kv,
                           out.data_ptr(), _lib.stream_ptr(dev)))
    return out


def fused_qk_scores_4bit(q_rot, packed_k, norms_k, centroids, D):
    """Raw (T_q, T_kv) scores from 4-bit packed keys, no dequantized K materialised (kernels.py:593-613)."""
    return _fused_qk(q_rot, packed_k, norms_k, centroids, D, 4)


def fused_qk_scores_3bit(q_rot, packed_k, norms_k, centroids, D):
    return _fused_qk(q_rot, packed_k, norms_k, centroids, D, 3)


def fused_qk_scores_2bit(q_rot, packed_k, norms_k, centroids, D):
    return _fused_qk(q_rot, packed_k, norms_k, centroids, D, 2)


_workspaces: dict[tuple[int | None, int], torch.Tensor] = {}


def decode_workspace(device: torch.device, nbytes: int) -> torch.Tensor:
    """Scratch for the decode kernel, one zero-filled buffer per (device, stream), grown on demand.

    The kernel keeps arrival counters in it and leaves them at zero, so the buffer must start zeroed."""
    key = (device.index, _lib.stream_ptr(device))
    ws = _workspaces.get(key)
    if ws is None or ws.numel() < nbytes:
        ws = torch.zeros(max(nbytes, 1 << 20), dtype=torch.uint8, device=device)
        _workspaces[key] = ws
    return ws


_decode_tables: dict[tuple, torch.Tensor | None] = {}


def decode_tables(d: int, seed: int, rotation: torch.Tensor, k_cent: torch.Tensor, k_bits: int, v_cent: torch.Tensor, v_bits: int,
                  v_cent_scale: float) -> torch.Tensor | None:
    """Constants of the decode kernel for this (device, head_dim, rotation seed, bit widths), built once and shared by every
    cache that uses them: the image of the kernel's lookup tables and the rotation matrix split into fp16 halves in the
    order the tensor-core rotation consumes (``tq_decode_tables_build``).  ``None`` when no kernel uses prebuilt
    constants for the shape.  The first call for a key synchronises the stream; make it outside graph capture
    (a cache does, the first time it sees a tensor)."""
    dev = _lib.require_cuda(rotation, k_cent, v_cent)
    key = (dev.index, d, seed, k_bits, v_bits, float(v_cent_scale), rotation.data_ptr(), k_cent.data_ptr(), v_cent.data_ptr())
    if key not in _decode_tables:
        need = int(_lib.lib().tq_decode_tables_bytes(d, k_bits, v_bits))
        if need == 0:
            _decode_tables[key] = None
        else:
            buf = torch.empty(need, dtype=torch.uint8, device=dev)
            _lib.check(_lib.launch(dev, "tq_decode_tables_build", d, rotation.data_ptr(), k_cent.data_ptr(), k_bits, v_cent.data_ptr(),
                                   v_bits, float(v_cent_scale), buf.data_ptr(), need, _lib.stream_ptr(dev)))
            _decode_tables[key] = buf
    return _decode_tables[key]


def set_tuning(key: str, value: int) -> None:
    _lib.check(_lib.lib().tq_set_tuning(key.encode(), int(value)))
