"""ctypes binding of ``libtq_b200.so`` (declared in ``include/tq_abi.h``).

The library is the only compute path of this package: there is no CPU or PyTorch
fallback.  Importing this module never fails, but the first call that needs the
library raises ``RuntimeError`` when the shared object has not been built
(``python -c "import __graft_entry__ as g; g.build()"``).
"""

from __future__ import annotations

import ctypes as C
from pathlib import Path

import torch

LIB_PATH = Path(__file__).resolve().parent / "libtq_b200.so"

TQ_F16, TQ_BF16, TQ_F32 = 0, 1, 2
_DTYPES = {torch.float16: TQ_F16, torch.bfloat16: TQ_BF16, torch.float32: TQ_F32}

_vp, _i, _i64, _f, _sz = C.c_void_p, C.c_int, C.c_int64, C.c_float, C.c_size_t


class QuantizeArgs(C.Structure):
    _fields_ = [
        ("x", _vp), ("x_dtype", _i), ("d", _i), ("n_lanes", _i64), ("n_rows", _i64),
        ("x_lane_stride", _i64), ("x_row_stride", _i64), ("rot", _vp),
        ("bnd_hi", _vp), ("bits_hi", _i), ("bnd_lo", _vp), ("bits_lo", _i),
        ("packed_hi", _vp), ("packed_lo", _vp), ("norms", _vp), ("out_lane_stride", _i64),
        ("qjl_proj_rot", _vp), ("cent_hi", _vp), ("cent_lo", _vp), ("qjl_bits", _vp), ("qjl_gamma", _vp),
        ("y_out", _vp),
    ]


class DequantizeArgs(C.Structure):
    _fields_ = [
        ("packed_hi", _vp), ("packed_lo", _vp), ("norms", _vp),
        ("n_lanes", _i64), ("n_rows", _i64), ("in_lane_stride", _i64),
        ("d", _i), ("bits_hi", _i), ("bits_lo", _i),
        ("cent_hi", _vp), ("cent_lo", _vp), ("rot", _vp),
        ("qjl_proj", _vp), ("qjl_bits", _vp), ("qjl_gamma", _vp),
        ("out", _vp), ("out_dtype", _i), ("out_lane_stride", _i64), ("out_row_stride", _i64),
    ]


TQ_MAX_PEERS = 8


class PeerGather(C.Structure):
    """tq_peer_gather: every rank's landing buffer as addresses valid on this device, and this rank's epoch array."""
    _fields_ = [
        ("n_peers", _i), ("heads_total", _i), ("head_offset", _i),
        ("ll", _vp * TQ_MAX_PEERS), ("epochs", _vp),
    ]


class DecodeArgs(C.Structure):
    _fields_ = [
        ("batch", _i), ("n_q_heads", _i), ("n_kv_heads", _i), ("d", _i),
        ("q", _vp), ("q_dtype", _i), ("scale", _f), ("rot", _vp),
        ("c_len", _i64), ("c_lane_stride", _i64),
        ("k_bits_hi", _i), ("k_bits_lo", _i), ("v_bits_hi", _i), ("v_bits_lo", _i),
        ("k_hi", _vp), ("k_lo", _vp), ("v_hi", _vp), ("v_lo", _vp),
        ("k_norms", _vp), ("v_norms", _vp),
        ("k_cent_hi", _vp), ("k_cent_lo", _vp), ("v_cent_hi", _vp), ("v_cent_lo", _vp),
        ("v_cent_scale_hi", _f), ("v_cent_scale_lo", _f),
        ("qjl_proj", _vp), ("k_qjl_bits", _vp), ("v_qjl_bits", _vp), ("k_qjl_gamma", _vp), ("v_qjl_gamma", _vp),
        ("dense_dtype", _i),
        ("sink_k", _vp), ("sink_v", _vp), ("sink_len", _i64), ("sink_lane_stride", _i64),
        ("res_k", _vp), ("res_v", _vp), ("res_len", _i64), ("res_lane_stride", _i64),
        ("out", _vp), ("out_dtype", _i),
        ("workspace", _vp), ("workspace_bytes", _sz),
        ("gather", C.POINTER(PeerGather)),
        ("tables", _vp),
        ("await_ll", _vp), ("await_epochs", _vp), ("await_words", _i64), ("await_out", _vp),
    ]


# name -> (restype, argtypes); every symbol include/tq_abi.h declares
PROTOTYPES = {
    "tq_version": (_i, []),
    "tq_last_error": (C.c_char_p, []),
    "tq_pack": (_i, [_vp, _vp, _i64, _i, _i, _vp]),
    "tq_unpack": (_i, [_vp, _vp, _i64, _i, _i, _vp]),
    "tq_quantize_scalar": (_i, [_vp, _vp, _i, _vp, _i64, _vp]),
    "tq_dequantize_scalar": (_i, [_vp, _vp, _i, _vp, _i64, _vp]),
    "tq_quantize_from_rotated": (_i, [_vp, _i64, _i, _vp, _i, _vp, _i, _vp, _vp, _vp]),
    "tq_rotate": (_i, [_vp, _i, _vp, _vp, _i64, _i, _i, _vp]),
    "tq_quantize_pack": (_i, [C.POINTER(QuantizeArgs), _vp]),
    "tq_dequantize": (_i, [C.POINTER(DequantizeArgs), _vp]),
    "tq_qjl_quantize": (_i, [_vp, _vp, _vp, _vp, _i64, _i, _i, _vp]),
    "tq_qjl_dequantize": (_i, [_vp, _vp, _vp, _vp, _i64, _i, _i, _vp]),
    "tq_qk_scores": (_i, [_vp, _vp, _vp, _vp, _i, _i, _i64, _i64, _vp, _vp]),
    "tq_append_tokens": (_i, [_vp, _vp, _vp, _vp, _i64, _i64, _i64, _i64, _i64, _i64, _vp]),
    "tq_decode_workspace_bytes": (_sz, [_i, _i, _i, _i, _i64, _i64]),
    "tq_decode_tables_bytes": (_sz, [_i, _i, _i]),
    "tq_decode_tables_build": (_i, [_i, _vp, _vp, _i, _vp, _i, _f, _vp, _sz, _vp]),
    "tq_decode_attn": (_i, [C.POINTER(DecodeArgs), _vp]),
    "tq_decode_step": (_i, [C.POINTER(DecodeArgs), _vp, _vp, _vp]),
    "tq_prefill_attn": (_i, [C.POINTER(DecodeArgs), _i, _vp]),
    "tq_decode_attn_static": (_i, [C.POINTER(DecodeArgs), _vp]),
    "tq_set_tuning": (_i, [C.c_char_p, _i]),
    "tq_decode_kernel_choice": (_i, [C.POINTER(DecodeArgs)]),
    "tq_fp16_table_scale": (_f, [_vp, _i]),
    "tq_device_status": (_i, []),
    "tq_device_status_clear": (_i, []),
    "tq_gather_groups": (_i64, [_i, _i, _i]),
    "tq_gather_wait": (_i, [_vp, _vp, _i64, _vp, _vp]),
    "tq_peer_buffer_create": (_i, [_sz, C.POINTER(_vp), C.c_char_p]),
    "tq_peer_buffer_open": (_i, [C.c_char_p, _i, C.POINTER(_vp)]),
    "tq_peer_buffer_close": (_i, [_vp]),
    "tq_peer_buffer_destroy": (_i, [_vp]),
}

_lib = None


def lib():
    """The loaded library; raises RuntimeError if it has not been built."""
    global _lib
    if _lib is None:
        if not LIB_PATH.exists():
            raise RuntimeError(
                f"{LIB_PATH} is missing: build the CUDA library first "
                "(python -c 'import __graft_entry__ as g; g.build()'). There is no CPU fallback.")
        handle = C.CDLL(str(LIB_PATH))
        for name, (res, args) in PROTOTYPES.items():
            fn = getattr(handle, name)
            fn.restype, fn.argtypes = res, args
        _lib = handle
    return _lib


class TurboQuantError(RuntimeError):
    """A libtq_b200 call returned a negative status."""


def check(rc: int) -> None:
    if rc != 0:
        msg = lib().tq_last_error().decode("utf-8", "replace")
        if rc == -1:
            raise ValueError(msg)
        if rc == -2:
            raise NotImplementedError(msg)
        raise TurboQuantError(f"libtq_b200 error {rc}: {msg}")


def dtype_code(dt: torch.dtype) -> int:
    try:
        return _DTYPES[dt]
    except KeyError:
        raise TypeError(f"unsupported dtype {dt}; use float16, bfloat16 or float32") from None


def require_cuda(*tensors: torch.Tensor) -> torch.device:
    """All tensors must live on one CUDA device (this package has no CPU path)."""
    dev = None
    for t in tensors:
        if t is None:
            continue
        if not t.is_cuda:
            raise RuntimeError("mlx_turboquant_b200 runs on CUDA tensors only; got a tensor on " + str(t.device))
        if dev is None:
            dev = t.device
        elif t.device != dev:
            raise RuntimeError("tensors are on different devices")
    return dev


def launch(dev: torch.device, name: str, *args) -> int:
    """Call library function ``name`` with ``dev`` as the current CUDA device and return its status.

    The library launches on the device that is current when it is called, and its per-device tables (SM count,
    shared-memory plan, static scratch) are keyed on it; tensors on ``cuda:1`` handed over while ``cuda:0`` is current
    would be dereferenced on the wrong GPU.  ``stream`` arguments must already belong to ``dev`` (``stream_ptr(dev)``).
    """
    fn = getattr(lib(), name)
    idx = dev.index if dev.index is not None else torch.cuda.current_device()
    if idx == torch.cuda.current_device():
        return fn(*args)
    with torch.cuda.device(idx):
        return fn(*args)


def ptr(t: torch.Tensor | None) -> int | None:
    return None if t is None else t.data_ptr()


try:
    _raw_stream = torch._C._cuda_getCurrentRawStream      # the stream handle as an int, without building a Stream object
except AttributeError:                                    # pragma: no cover - older / newer torch
    _raw_stream = None


def stream_ptr(device: torch.device) -> int:
    if _raw_stream is not None:
        return _raw_stream(device.index if device.index is not None else torch.cuda.current_device())
    return torch.cuda.current_stream(device).cuda_stream
