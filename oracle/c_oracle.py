"""ctypes loader for the C restatement of the reference's kernel bodies (``tq_oracle.c``).

TEST INFRASTRUCTURE: used by tests, the smoke check and the benchmark's CPU-baseline leg only.
``load()`` compiles the library on first use when gcc is present.
"""

from __future__ import annotations

import ctypes as C
import subprocess
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
SRC, LIB = HERE / "tq_oracle.c", HERE / "libtq_oracle.so"
_f, _u8, _i, _i64 = C.POINTER(C.c_float), C.POINTER(C.c_uint8), C.c_int, C.c_int64
_lib = None


def load():
    global _lib
    if _lib is None:
        if not LIB.exists() or LIB.stat().st_mtime < SRC.stat().st_mtime:
            subprocess.run(["gcc", "-O3", "-march=native", "-fopenmp", "-shared", "-fPIC", "-o", str(LIB), str(SRC), "-lm"], check=True)
        h = C.CDLL(str(LIB))
        h.tqo_threads.restype = _i
        h.tqo_dequantize_rows.argtypes = [_u8, _f, _i64, _i, _i, _f, _f, _f]
        h.tqo_quantize_rows.argtypes = [_f, _i64, _i, _f, _f, _i, _u8, _f, _f]
        h.tqo_qk_scores.argtypes = [_f, _u8, _f, _f, _i, _i, _i64, _i64, _f]
        h.tqo_attention.argtypes = [_f, _f, _f, _i, _i, _i, _i64, _i, C.c_float, _f]
        _lib = h
    return _lib


def _fp(a):
    return a.ctypes.data_as(_f)


def _bp(a):
    return a.ctypes.data_as(_u8)


def quantize_rows(lib, x, rot, bnd, bits, want_y=False):
    x = np.ascontiguousarray(x, dtype=np.float32)
    d = x.shape[-1]
    n = x.size // d
    packed = np.empty(x.shape[:-1] + (d * bits // 8,), dtype=np.uint8)
    norms = np.empty(x.shape[:-1], dtype=np.float32)
    y = np.empty(x.shape, dtype=np.float32) if want_y else None
    lib.tqo_quantize_rows(_fp(x), n, d, _fp(np.ascontiguousarray(rot, np.float32)), _fp(np.ascontiguousarray(bnd, np.float32)),
                          bits, _bp(packed), _fp(norms), _fp(y) if want_y else None)
    return (packed, norms, y) if want_y else (packed, norms)


def dequantize_rows(lib, packed, norms, rot, cent, bits, d):
    packed = np.ascontiguousarray(packed)
    norms = np.ascontiguousarray(norms, dtype=np.float32)
    out = np.empty(norms.shape + (d,), dtype=np.float32)
    lib.tqo_dequantize_rows(_bp(packed), _fp(norms), norms.size, d, bits, _fp(np.ascontiguousarray(cent, np.float32)),
                            _fp(np.ascontiguousarray(rot, np.float32)), _fp(out))
    return out


def qk_scores(lib, q_rot, packed, norms, cent, bits, d):
    q_rot = np.ascontiguousarray(q_rot, np.float32)
    out = np.zeros((q_rot.shape[0], packed.shape[0]), dtype=np.float32)
    if out.size:
        lib.tqo_qk_scores(_fp(q_rot), _bp(np.ascontiguousarray(packed)), _fp(np.ascontiguousarray(norms, np.float32)),
                          _fp(np.ascontiguousarray(cent, np.float32)), bits, d, q_rot.shape[0], packed.shape[0], _fp(out))
    return out


def attention(lib, q, k, v, scale=None):
    """q (B, Hq, 1, D); k, v (B, Hkv, T, D) -> (B, Hq, 1, D) float32."""
    q = np.ascontiguousarray(q, np.float32)
    k = np.ascontiguousarray(k, np.float32)
    v = np.ascontiguousarray(v, np.float32)
    b, hq, _, d = q.shape
    out = np.empty((b, hq, 1, d), dtype=np.float32)
    lib.tqo_attention(_fp(q), _fp(k), _fp(v), b, hq, k.shape[1], k.shape[2], d, float(d ** -0.5 if scale is None else scale), _fp(out))
    return out


def use_c_kernels(cache, lib):
    """Make a ``KVCacheOracle`` with integer bit widths and no QJL run its per-chunk quantize / dequantize
    through the C loops (same algorithm, all host threads) instead of NumPy's comparison matrices."""
    if cache.proj is not None or cache.key_bits != int(cache.key_bits) or cache.value_bits != int(cache.value_bits):
        return cache

    def side(x, bits):
        b = int(bits)
        packed, norms = quantize_rows(lib, x, cache.rot, cache.tables[b][1], b)
        return packed, None, norms, dequantize_rows(lib, packed, norms, cache.rot, cache.tables[b][0], b, cache.d)

    cache._side = side
    return cache
