"""TurboQuant KV cache on torch CUDA tensors (reference: mlx_turboquant/cache.py).

Same protocol as the reference's ``TurboQuantKVCache`` - ``update_and_fetch``, ``offset``,
``make_mask``, ``state`` / ``meta_state``, ``empty``, ``is_trimmable``, ``size``, ``nbytes``,
``step`` - and the same compression schedule, sink routing and buffer-capacity rules, so a caller
written against the reference keeps working.  What differs is where the work happens:

* draining tokens out of the recent-token buffer is ONE fused CUDA kernel per side
  (norm, rotation, boundary search, bit-packing, optional QJL sketch) writing straight into
  preallocated packed storage that grows geometrically - no per-drain concatenation;
* ``update`` + ``attend`` compute a decode step directly on the packed storage (the path the
  reference only prototyped); ``update_and_fetch`` still returns the dense
  ``[sink | dequantized middle | recent]`` tensors for callers that run their own attention,
  building the dense middle lazily and incrementally;
* the QJL sketch (sign bits + residual norm per token) is kept, so the correction survives a
  state reload instead of being baked into a transient dense tensor.
"""

from __future__ import annotations

import ctypes as C

import numpy as np
from typing import Any

import torch

from . import _lib, kernels
from .codebook import get_codebook, get_codebook_host
from .qjl import generate_projection_matrix_host, get_projection_matrix
from .rotation import generate_rotation_matrix_host, get_rotation_matrix


def _round_up(n: int, m: int) -> int:
    return (n + m - 1) // m * m


_fp16_scales: dict[tuple[int, int], float] = {}


def _fp16_scale(d: int, bits: int) -> float:
    """Table-wide scale that makes the fp16 copies of a codebook's centroids (held by the decode kernel)
    accurate to ~1e-5 instead of 2^-11; see tq_fp16_table_scale."""
    key = (d, bits)
    if key not in _fp16_scales:
        import numpy as np
        c = np.ascontiguousarray(get_codebook_host(d, bits)[0], dtype=np.float32)
        _fp16_scales[key] = float(_lib.lib().tq_fp16_table_scale(c.ctypes.data, c.size))
    return _fp16_scales[key]


class _Side:
    """Packed storage of one side (keys or values): codes, norms and the optional QJL sketch."""

    def __init__(self, bits: float):
        self.bits = bits
        self.bits_hi, self.bits_lo = kernels.split_bits(bits)
        self.fractional = self.bits_lo != 0
        self.hi = self.lo = self.norms = self.qbits = self.qgamma = None
        self.cent_hi = self.cent_lo = self.bnd_hi = self.bnd_lo = None
        self.fp16_scale_hi = self.fp16_scale_lo = 0.0

    def load_tables(self, d: int, device) -> None:
        self.cent_hi, self.bnd_hi = get_codebook(d, self.bits_hi, device)
        self.fp16_scale_hi = _fp16_scale(d, self.bits_hi)
        if self.fractional:
            self.cent_lo, self.bnd_lo = get_codebook(d, self.bits_lo, device)
            self.fp16_scale_lo = _fp16_scale(d, self.bits_lo)

    def capacity(self) -> int:
        return 0 if self.hi is None else self.hi.shape[2]

    def reserve(self, b: int, h: int, d: int, need: int, used: int, device, with_qjl: bool) -> None:
        if self.capacity() >= need:
            return
        cap = _round_up(max(need, 2 * self.capacity(), 256), 16)
        w_hi, w_lo = kernels.packed_widths(d, self.bits_hi, self.bits_lo)

        def grow(old, shape, dtype):
            if old is None:   # e.g. a sketch that a reloaded state did not carry: zero = no correction
                return torch.zeros(shape, dtype=dtype, device=device)
            new = torch.empty(shape, dtype=dtype, device=device)
            if used > 0:
                new[:, :, :used] = old[:, :, :used]
            return new

        self.hi = grow(self.hi, (b, h, cap, w_hi), torch.uint8)
        if self.fractional:
            self.lo = grow(self.lo, (b, h, cap, w_lo), torch.uint8)
        self.norms = grow(self.norms, (b, h, cap), torch.float32)
        if with_qjl:
            self.qbits = grow(self.qbits, (b, h, cap), torch.int32)
            self.qgamma = grow(self.qgamma, (b, h, cap), torch.float32)


class TurboQuantKVCache:
    """TurboQuant-compressed KV cache: older tokens packed at ``key_bits`` / ``value_bits``, the most
    recent ``residual_window`` tokens and the first ``fp16_sink_size`` tokens kept uncompressed."""

    step = 256  # growth step of the recent-token buffer (cache.py:26)

    def __init__(self, head_dim: int = 128, num_kv_heads: int = 1, key_bits: float = 4, value_bits: float = 2,
                 residual_window: int = 128, rotation_seed: int = 42, fp16_sink_size: int = 0, chunk_size: int = 0,
                 qjl_correction: bool = False, qjl_n_proj: int = 32):
        self.head_dim = head_dim
        self.num_kv_heads = num_kv_heads
        self.key_bits = key_bits
        self.value_bits = value_bits
        self.residual_window = residual_window
        self.rotation_seed = rotation_seed
        self.fp16_sink_size = fp16_sink_size
        self.chunk_size = chunk_size
        self.qjl_correction = qjl_correction
        self.qjl_n_proj = qjl_n_proj
        if qjl_correction and qjl_n_proj != 32:
            raise NotImplementedError("the CUDA kernels keep the QJL sketch in one 32-bit word: qjl_n_proj must be 32")

        self._k = _Side(key_bits)
        self._v = _Side(value_bits)
        self._k_fractional, self._v_fractional = self._k.fractional, self._v.fractional
        self._device = None
        self._rotation = None
        self._qjl_proj = None       # S (m, d)
        self._qjl_proj_rot = None   # S @ R^T (m, d), used by the quantize kernel in rotated space

        self.sink_keys = self.sink_values = None   # (B, H, fp16_sink_size, D)
        self._sink_len = 0
        self.keys = self.values = None             # (B, H, capacity, D) recent tokens
        self._fp16_len = 0
        self._fp16_capacity = 0
        self._compressed_len = 0
        self._dense_k = self._dense_v = None       # lazily dequantized middle, float32
        self._dense_len = 0
        self._dargs = self._dargs_key = self._ws_key = None     # decode argument block kept between attend() calls
        self._ws_need = 0
        self._tables = None         # prebuilt constants of the decode kernel (shared between caches of the same shape)
        self.offset = 0

    # ---- constants -------------------------------------------------------------------------------
    def _bind(self, device) -> None:
        if self._device is not None:
            if device != self._device:
                raise RuntimeError(f"this cache lives on {self._device}; got tensors on {device}")
            return
        self._device = device
        d = self.head_dim
        self._rotation = get_rotation_matrix(d, self.rotation_seed, device)
        self._k.load_tables(d, device)
        self._v.load_tables(d, device)
        if not (self._k.fractional or self._v.fractional):      # (the streaming decode kernel takes sign sketches too)
            self._tables = kernels.decode_tables(d, self.rotation_seed, self._rotation, self._k.cent_hi, self._k.bits_hi,
                                                 self._v.cent_hi, self._v.bits_hi, self._v.fp16_scale_hi)
        if self.qjl_correction:
            self._qjl_proj = get_projection_matrix(d, self.qjl_n_proj, device=device)
            s = generate_projection_matrix_host(d, self.qjl_n_proj).astype("float64")
            r = generate_rotation_matrix_host(d, self.rotation_seed).astype("float64")
            self._qjl_proj_rot = torch.from_numpy((s @ r.T).astype("float32")).to(device)

    @property
    def rotation(self):
        if self._rotation is None:
            return get_rotation_matrix(self.head_dim, self.rotation_seed)
        return self._rotation

    @property
    def _qjl_projection(self):
        if not self.qjl_correction:
            return None
        return self._qjl_proj if self._qjl_proj is not None else get_projection_matrix(self.head_dim, self.qjl_n_proj)

    # Reference attribute names for the packed arrays (valid tokens only).
    def _view(self, t):
        return None if t is None or self._compressed_len == 0 else t[:, :, :self._compressed_len]

    _compressed_keys = property(lambda self: self._view(self._k.hi))
    _compressed_keys_lo = property(lambda self: self._view(self._k.lo))
    _compressed_key_norms = property(lambda self: self._view(self._k.norms))
    _compressed_values = property(lambda self: self._view(self._v.hi))
    _compressed_values_lo = property(lambda self: self._view(self._v.lo))
    _compressed_value_norms = property(lambda self: self._view(self._v.norms))

    # ---- checkpoint state (cache.py:118-200) --------------------------------------------------------
    @property
    def state(self):
        """10-tuple in the reference's order; with QJL on, four more: K bits, K gamma, V bits, V gamma."""
        base = (self.keys, self.values, self._compressed_keys, self._compressed_key_norms,
                self._compressed_values, self._compressed_value_norms, self.sink_keys, self.sink_values,
                self._compressed_keys_lo, self._compressed_values_lo)
        if self.qjl_correction:
            base = base + (self._view(self._k.qbits), self._view(self._k.qgamma),
                           self._view(self._v.qbits), self._view(self._v.qgamma))
        return base

    @state.setter
    def state(self, v):
        n = len(v)
        if n not in (6, 8, 10, 14):
            raise ValueError(f"state must have 6, 8, 10 or 14 elements, got {n}")
        # every kernel dereferences these arrays as device memory: a checkpoint loaded on the CPU (or spread over
        # several GPUs) is refused here rather than faulting at the next attend()
        dev = _lib.require_cuda(*v)
        if dev is not None and self._device is not None and dev != self._device:
            raise RuntimeError(f"state tensors are on {dev}, this cache is bound to {self._device}")
        v = tuple(v) + (None,) * (14 - n)
        self._dargs = self._dargs_key = self._ws_key = None     # the cached decode arguments pointed into the old arrays
        self.keys, self.values = v[0], v[1]
        def own(t):
            """Adopt a packed array as storage: contiguous, token capacity padded to a multiple of 16."""
            if t is None:
                return None
            cap = _round_up(max(t.shape[2], 16), 16)
            if cap == t.shape[2] and t.is_contiguous():
                return t
            new = torch.zeros(t.shape[:2] + (cap,) + t.shape[3:], dtype=t.dtype, device=t.device)
            new[:, :, :t.shape[2]] = t
            return new
        n_comp = None if v[2] is None else v[2].shape[2]
        self._k.hi, self._k.norms, self._v.hi, self._v.norms = own(v[2]), own(v[3]), own(v[4]), own(v[5])
        if n >= 8:
            self.sink_keys, self.sink_values = v[6], v[7]
        if n >= 10:
            self._k.lo, self._v.lo = own(v[8]), own(v[9])
        if n >= 14:
            self._k.qbits, self._k.qgamma, self._v.qbits, self._v.qgamma = own(v[10]), own(v[11]), own(v[12]), own(v[13])
        if n_comp is not None:
            self._compressed_len = n_comp
        self._dense_k = self._dense_v = None
        self._dense_len = 0
        if dev is not None:
            self._bind(dev)

    @property
    def meta_state(self):
        return {
            "offset": str(self.offset), "compressed_len": str(self._compressed_len),
            "head_dim": str(self.head_dim), "key_bits": str(self.key_bits), "value_bits": str(self.value_bits),
            "fp16_sink_size": str(self.fp16_sink_size), "sink_len": str(self._sink_len),
            "fp16_len": str(self._fp16_len), "fp16_capacity": str(self._fp16_capacity),
        }

    @meta_state.setter
    def meta_state(self, v):
        self.offset = int(v["offset"])
        self._compressed_len = int(v["compressed_len"])
        if "fp16_sink_size" in v:
            self.fp16_sink_size = int(v["fp16_sink_size"])
        if "sink_len" in v:
            self._sink_len = int(v["sink_len"])
        if "fp16_len" in v:
            self._fp16_len = int(v["fp16_len"])
        if "fp16_capacity" in v:
            self._fp16_capacity = int(v["fp16_capacity"])

    def empty(self) -> bool:
        return self._fp16_len == 0 and self._compressed_len == 0 and self._sink_len == 0

    def is_trimmable(self) -> bool:
        return False

    def size(self) -> int:
        return self.offset

    @property
    def nbytes(self) -> int:
        """Same accounting as the reference (cache.py:211-230): uncompressed regions at 4 B/element."""
        total, d = 0, self.head_dim
        if self.keys is not None and self._fp16_len > 0:
            b, h = self.keys.shape[0], self.keys.shape[1]
            total += 2 * b * h * self._fp16_len * d * 4
        if self.sink_keys is not None and self._sink_len > 0:
            b, h = self.sink_keys.shape[0], self.sink_keys.shape[1]
            total += 2 * b * h * self._sink_len * d * 4
        if self._k.hi is not None and self._compressed_len > 0:
            for side in (self._k, self._v):
                b, h = side.hi.shape[0], side.hi.shape[1]
                per_token = side.hi.shape[3] + 4 + (side.lo.shape[3] if side.lo is not None else 0)
                total += b * h * self._compressed_len * per_token
        return total

    # ---- compression ------------------------------------------------------------------------------
    def _qjl_args(self, side: _Side):
        if not self.qjl_correction:
            return None
        return dict(proj_rot=self._qjl_proj_rot, cent_hi=side.cent_hi, cent_lo=side.cent_lo,
                    bits=side.qbits, gamma=side.qgamma)

    def _drain_chunk(self, n: int) -> None:
        """Compress and evict the first n recent tokens (cache.py:535-575).

        The kernels read the buffer before the remaining tokens are shifted to the front (both
        are ordered on the current stream), so the chunk is never overwritten first.
        """
        b, h, _, d = self.keys.shape
        dev = self.keys.device
        for side, buf in ((self._k, self.keys), (self._v, self.values)):
            side.reserve(b, h, d, self._compressed_len + n, self._compressed_len, dev, self.qjl_correction)
            kernels.quantize_pack(buf[:, :, :n], self._rotation, side.bnd_hi, side.bits_hi, side.bnd_lo, side.bits_lo,
                                  out_hi=side.hi, out_lo=side.lo, out_norms=side.norms,
                                  out_offset=self._compressed_len, qjl=self._qjl_args(side))
        rem = self._fp16_len - n
        # A long prefill leaves buffers sized for the whole prompt; once most of it is packed they are swapped for
        # buffers of the size a fresh cache would get for what remains (batch 64 x 32K tokens: 17 GB per layer otherwise).
        small_cap = max(rem, self.residual_window * 2) + 256
        if self._fp16_capacity > 4 * small_cap:
            nk = torch.zeros((b, h, small_cap, d), dtype=self.keys.dtype, device=dev)
            nv = torch.zeros((b, h, small_cap, d), dtype=self.values.dtype, device=dev)
            if rem > 0:
                self._append(nk, nv, self.keys[:, :, n:self._fp16_len], self.values[:, :, n:self._fp16_len], 0)
            self.keys, self.values, self._fp16_capacity = nk, nv, small_cap
        elif rem > 0:
            for buf in (self.keys, self.values):
                tail = buf[:, :, n:self._fp16_len]
                buf[:, :, :rem] = tail.clone() if n < rem else tail
        self._fp16_len = rem
        self._compressed_len += n

    def _compress_old_tokens(self) -> None:
        """Drain schedule (cache.py:497-533)."""
        if self.keys is None:
            return
        if self.chunk_size <= 0:
            if self._fp16_len <= self.residual_window * 2:
                return
            self._drain_chunk(self._fp16_len - self.residual_window)
            return
        # The reference drains one chunk per loop iteration while fp16_len >= residual_window + chunk_size; tokens
        # are quantized independently, so all those chunks go to the GPU as one launch with the same result.
        threshold = self.residual_window + self.chunk_size
        if self._fp16_len >= threshold:
            n_chunks = (self._fp16_len - self.residual_window) // self.chunk_size
            self._drain_chunk(n_chunks * self.chunk_size)

    def _route_sink(self, keys, values):
        """Peel the tokens that belong to the permanent sink off the head of the batch (cache.py:577-618)."""
        if self.fp16_sink_size <= 0 or self.offset >= self.fp16_sink_size:
            return keys, values
        t_new = keys.shape[2]
        n_sink = min(self.fp16_sink_size - self.offset, t_new)
        if n_sink <= 0:
            return keys, values
        if self.sink_keys is None:
            b, h, _, d = keys.shape
            self.sink_keys = torch.zeros((b, h, self.fp16_sink_size, d), dtype=keys.dtype, device=keys.device)
            self.sink_values = torch.zeros((b, h, self.fp16_sink_size, d), dtype=values.dtype, device=values.device)
        if n_sink == t_new:
            self._append(self.sink_keys, self.sink_values, keys, values, self.offset)
        else:
            self.sink_keys[:, :, self.offset:self.offset + n_sink] = keys[:, :, :n_sink]
            self.sink_values[:, :, self.offset:self.offset + n_sink] = values[:, :, :n_sink]
        self._sink_len = self.offset + n_sink
        return keys[:, :, n_sink:], values[:, :, n_sink:]

    @staticmethod
    def _append(k_buf, v_buf, k_new, v_new, row0: int) -> None:
        """k_buf[:, :, row0:row0+T] = k_new (same for values): one library launch when the layout allows it."""
        t_new = k_new.shape[2]
        _lib.require_cuda(k_buf, v_buf, k_new, v_new)
        if (k_new.is_contiguous() and v_new.is_contiguous() and k_new.dtype == k_buf.dtype and v_new.dtype == v_buf.dtype
                and k_buf.dtype == v_buf.dtype and (k_buf.shape[3] * k_buf.element_size()) % 16 == 0):
            b, h, cap, d = k_buf.shape
            rc = _lib.launch(k_buf.device, "tq_append_tokens", k_new.data_ptr(), v_new.data_ptr(), k_buf.data_ptr(), v_buf.data_ptr(),
                             b * h, t_new, d * k_buf.element_size(), t_new, cap, row0, _lib.stream_ptr(k_buf.device))
            if rc == 0:
                return
            if rc != -2:                      # anything but "layout not supported" is an error
                _lib.check(rc)
        k_buf[:, :, row0:row0 + t_new] = k_new
        v_buf[:, :, row0:row0 + t_new] = v_new

    def update(self, keys: torch.Tensor, values: torch.Tensor) -> None:
        """Append new tokens (B, H, T, D) and compress what leaves the residual window.

        The state-changing half of ``update_and_fetch`` (cache.py:632-672) without building any dense
        output; pair it with :meth:`attend`.
        """
        dev = _lib.require_cuda(keys, values)
        self._bind(dev)
        t_total = keys.shape[2]
        keys_rest, values_rest = self._route_sink(keys, values)
        t_new = keys_rest.shape[2]
        if t_new > 0:
            if self.keys is None:
                b, h, _, d = keys_rest.shape
                cap = max(t_new, self.residual_window * 2) + 256
                self._fp16_capacity = cap
                self._fp16_len = 0
                self.keys = torch.zeros((b, h, cap, d), dtype=keys_rest.dtype, device=dev)
                self.values = torch.zeros((b, h, cap, d), dtype=values_rest.dtype, device=dev)
            new_len = self._fp16_len + t_new
            if new_len > self._fp16_capacity:
                b, h, _, d = self.keys.shape
                new_cap = new_len + 256
                nk = torch.zeros((b, h, new_cap, d), dtype=keys_rest.dtype, device=dev)
                nv = torch.zeros((b, h, new_cap, d), dtype=values_rest.dtype, device=dev)
                nk[:, :, :self._fp16_len] = self.keys[:, :, :self._fp16_len]
                nv[:, :, :self._fp16_len] = self.values[:, :, :self._fp16_len]
                self.keys, self.values, self._fp16_capacity = nk, nv, new_cap
            self._append(self.keys, self.values, keys_rest, values_rest, self._fp16_len)
            self._fp16_len = new_len
        self.offset += t_total
        self._compress_old_tokens()

    # ---- dense output ------------------------------------------------------------------------------
    def _ensure_dense(self) -> None:
        """Dequantize packed tokens [dense_len, compressed_len) into the dense middle (cache.py:276-394)."""
        n = self._compressed_len - self._dense_len
        if n <= 0:
            return
        k, v = self._k, self._v
        b, h = k.hi.shape[0], k.hi.shape[1]
        d, dev = self.head_dim, k.hi.device
        self._bind(dev)
        cap = 0 if self._dense_k is None else self._dense_k.shape[2]
        if cap < self._compressed_len:
            new_cap = _round_up(max(self._compressed_len, 2 * cap, 256), 16)
            for name in ("_dense_k", "_dense_v"):
                new = torch.empty((b, h, new_cap, d), dtype=torch.float32, device=dev)
                old = getattr(self, name)
                if old is not None and self._dense_len > 0:
                    new[:, :, :self._dense_len] = old[:, :, :self._dense_len]
                setattr(self, name, new)
        for side, out in ((k, self._dense_k), (v, self._dense_v)):
            qjl = None
            if self.qjl_correction and side.qbits is not None:
                qjl = dict(proj=self._qjl_proj, bits=side.qbits, gamma=side.qgamma)
            kernels.dequantize_rows(side.hi, side.lo, side.norms, self._rotation, side.cent_hi, side.bits_hi,
                                    side.cent_lo, side.bits_lo, d, n_rows=n, in_offset=self._dense_len,
                                    out=out, out_offset=self._dense_len, qjl=qjl)
        self._dense_len = self._compressed_len

    def update_and_fetch(self, keys: torch.Tensor, values: torch.Tensor):
        """Append, compress, and return the full dense (keys, values) for attention (cache.py:620-706).

        Result is ``[sink | dequantized middle (float32) | recent]`` along the token axis; its dtype is
        the input dtype until a compressed part exists and float32 afterwards.
        """
        self.update(keys, values)
        self._ensure_dense()
        pk, pv = [], []
        if self._sink_len > 0:
            pk.append(self.sink_keys[:, :, :self._sink_len])
            pv.append(self.sink_values[:, :, :self._sink_len])
        if self._compressed_len > 0:
            pk.append(self._dense_k[:, :, :self._compressed_len])
            pv.append(self._dense_v[:, :, :self._compressed_len])
        if self._fp16_len > 0:
            pk.append(self.keys[:, :, :self._fp16_len])
            pv.append(self.values[:, :, :self._fp16_len])
        if not pk:
            return keys[:, :, :0], values[:, :, :0]
        if len(pk) == 1:
            return pk[0], pv[0]
        return torch.cat(pk, dim=2), torch.cat(pv, dim=2)

    # ---- attention on the packed cache -----------------------------------------------------------
    def attend(self, queries: torch.Tensor, scale: float | None = None, out_dtype=None, gather=None,
               out: torch.Tensor | None = None, _new=None, after=None) -> torch.Tensor | None:
        """softmax(scale * q K^T) V straight from packed storage.

        ``queries`` is (B, n_q_heads, 1, D) or (B, n_q_heads, D) for a decode step, or (B, n_q_heads, T_q, D) for the last
        T_q tokens of the cache (causal; see ``_attend_many``); the result has the same shape and, unless
        ``out_dtype`` says otherwise, the same dtype.  Equals attention over what ``update_and_fetch``
        would return (to ~1e-3 with a float32 result; a float16 result adds its own rounding), without
        building it.  With ``gather`` (a slot of ``sharding.FusedGather``: this rank holds some of the heads) the
        kernel stores the result into every rank's gather buffer instead and nothing is returned.  ``out`` (contiguous,
        ``queries``' shape) receives the result in place of a fresh tensor.  ``after`` (``FusedGather.arrived(j)`` of an
        earlier call's slot) makes the kernel wait, before it reads the queries, until that gather is complete on this GPU.
        """
        dev = _lib.require_cuda(queries)
        self._bind(dev)
        d = self.head_dim
        squeeze = queries.dim() == 3
        if not squeeze and queries.shape[2] != 1:
            if gather is not None or _new is not None or after is not None:
                raise NotImplementedError("several query tokens per sequence: no fused gather, no fused append")
            return self._attend_many(queries, scale, out_dtype, out)
        b, hq = queries.shape[0], queries.shape[1]
        if self.empty() and _new is None:
            raise ValueError("attend on an empty cache")
        q = queries.reshape(b, hq, d)
        if q.dtype not in (torch.float16, torch.bfloat16, torch.float32):
            q = q.to(torch.float32)
        q = q.contiguous()
        given = out
        if gather is not None:
            out = None
        elif out is None:
            out = torch.empty((b, hq, d), dtype=out_dtype or q.dtype, device=dev)
        elif out.device != dev or out.numel() != b * hq * d or not out.is_contiguous() or out.dtype not in _lib._DTYPES:
            raise ValueError("out must be a contiguous float16 / bfloat16 / float32 tensor of the queries' shape on their device")
        out_dt = (out_dtype or q.dtype) if out is None else out.dtype
        if gather is not None and getattr(gather, "dtype", None) is not None:
            if out_dtype is not None and out_dtype != gather.dtype:
                raise ValueError(f"the gather buffers hold {gather.dtype}, not {out_dtype}")
            out_dt = gather.dtype                                   # element size of the peers' buffers
        if gather is not None and getattr(gather, "shape", None) is not None and gather.shape != (b, d):
            raise ValueError(f"the gather buffers are for batch {gather.shape[0]}, head_dim {gather.shape[1]}; got {b}, {d}")
        k, v = self._k, self._v
        # Everything but the query, the result and the three lengths only changes when a buffer is (re)allocated:
        # the filled-in argument block is kept and revalidated by the buffers' addresses.
        key = (b, hq, q.dtype, out_dt, scale, _lib.ptr(k.hi), _lib.ptr(v.hi), _lib.ptr(self.keys), _lib.ptr(self.sink_keys),
               _lib.ptr(k.qbits), k.capacity(), self._fp16_capacity)
        a = self._dargs
        if a is None or key != self._dargs_key:
            a = self._fill_decode_args(b, hq, q.dtype, out_dt, scale)
            self._dargs, self._dargs_key, self._ws_key = a, key, None
        a.q, a.out = q.data_ptr(), (None if out is None else out.data_ptr())
        a.gather = C.pointer(gather) if gather is not None else None
        a.await_ll, a.await_epochs, a.await_words, a.await_out = after if after is not None else (None, None, 0, None)
        a.c_len, a.sink_len, a.res_len = self._compressed_len, self._sink_len, self._fp16_len
        dense_len = self._sink_len + self._fp16_len + (0 if _new is None else 1)
        ws_key = (self._compressed_len, (dense_len + 15) >> 4)        # the split plan depends on whole 16-token tiles only
        if ws_key != self._ws_key:
            self._ws_need = _lib.lib().tq_decode_workspace_bytes(b, hq, a.n_kv_heads, d, self._compressed_len, ws_key[1] << 4)
            self._ws_key = ws_key
        ws = kernels.decode_workspace(dev, self._ws_need)
        a.workspace, a.workspace_bytes = ws.data_ptr(), ws.numel()
        if _new is None:
            _lib.check(_lib.launch(dev, "tq_decode_attn", C.byref(a), _lib.stream_ptr(dev)))
        else:      # append the token's rows and attend over them in the same launch
            _lib.check(_lib.launch(dev, "tq_decode_step", C.byref(a), _new[0].data_ptr(), _new[1].data_ptr(), _lib.stream_ptr(dev)))
        if out is None:
            return None
        if given is not None:
            return given
        return out if squeeze else out.reshape(b, hq, 1, d)

    def _attend_many(self, queries: torch.Tensor, scale, out_dtype, out) -> torch.Tensor:
        """Causal attention for queries (B, n_q_heads, T_q, D) that are the LAST T_q tokens of the cache (call ``update``
        with their keys and values first), straight from packed storage: query i sees every cached token up to and
        including itself.  Equals causal attention over what ``update_and_fetch`` returns, without building it."""
        dev = queries.device
        d = self.head_dim
        b, hq, tq = queries.shape[0], queries.shape[1], queries.shape[2]
        if self.qjl_correction:
            raise NotImplementedError("several query tokens over a cache with a QJL sketch: use update_and_fetch (dense route)")
        if tq > self._sink_len + self._compressed_len + self._fp16_len:
            raise ValueError("more query tokens than the cache holds: call update() with their keys and values first")
        q = queries
        if q.dtype not in (torch.float16, torch.bfloat16, torch.float32):
            q = q.to(torch.float32)
        q = q.contiguous()
        if out is None:
            out = torch.empty((b, hq, tq, d), dtype=out_dtype or q.dtype, device=dev)
        elif out.device != dev or tuple(out.shape) != (b, hq, tq, d) or not out.is_contiguous() or out.dtype not in _lib._DTYPES:
            raise ValueError("out must be a contiguous float16 / bfloat16 / float32 tensor of the queries' shape on their device")
        a = self._fill_decode_args(b, hq, q.dtype, out.dtype, scale)
        a.q, a.out = q.data_ptr(), out.data_ptr()
        a.c_len, a.sink_len, a.res_len = self._compressed_len, self._sink_len, self._fp16_len
        _lib.check(_lib.launch(dev, "tq_prefill_attn", C.byref(a), tq, _lib.stream_ptr(dev)))
        return out

    def decode_step(self, queries: torch.Tensor, keys: torch.Tensor, values: torch.Tensor, scale: float | None = None,
                    out: torch.Tensor | None = None) -> torch.Tensor:
        """One decode step: ``update(keys, values)`` followed by ``attend(queries)``, as ONE kernel launch when the new token
        simply joins the recent-token buffer (no growth, no compression due, not a sink token, same dtype as the buffer):
        the kernel stores the token's rows itself and attends over them.  Any other step takes the two calls."""
        t_new = keys.shape[2] if keys.dim() == 4 else 0
        fast = (t_new == 1 and self.keys is not None and self.offset >= self.fp16_sink_size
                and self._fp16_len + 1 <= self._fp16_capacity and keys.dtype == self.keys.dtype and values.dtype == self.values.dtype
                and keys.is_contiguous() and values.is_contiguous() and (queries.dim() == 3 or queries.shape[2] == 1))
        if fast:
            new_len = self._fp16_len + 1                     # would update() drain after this token?  (cache.py:497-533)
            if self.chunk_size <= 0:
                fast = new_len <= self.residual_window * 2
            else:
                fast = new_len < self.residual_window + self.chunk_size
        if not fast:
            self.update(keys, values)
            return self.attend(queries, scale=scale, out=out)
        if keys.device != self._device or values.device != self._device:
            raise RuntimeError(f"this cache lives on {self._device}; got tensors on {keys.device}")
        res = self.attend(queries, scale=scale, out=out, _new=(keys, values))
        self._fp16_len += 1
        self.offset += 1
        return res

    def _fill_decode_args(self, b: int, hq: int, q_dtype, out_dtype, scale) -> "_lib.DecodeArgs":
        d = self.head_dim
        ref = self.keys if self.keys is not None else self.sink_keys
        if ref is None:
            ref = self._k.hi
        hkv = ref.shape[1]
        a = _lib.DecodeArgs()
        a.batch, a.n_q_heads, a.n_kv_heads, a.d = b, hq, hkv, d
        a.q_dtype = _lib.dtype_code(q_dtype)
        a.scale = float(d ** -0.5 if scale is None else scale)
        a.rot = self._rotation.data_ptr()
        k, v = self._k, self._v
        if k.hi is not None:
            a.c_lane_stride = k.hi.shape[2]
            if v.hi.shape[2] != k.hi.shape[2]:
                raise RuntimeError("key and value packed storage have different capacities")
            a.k_bits_hi, a.k_bits_lo, a.v_bits_hi, a.v_bits_lo = k.bits_hi, k.bits_lo, v.bits_hi, v.bits_lo
            a.k_hi, a.k_lo, a.v_hi, a.v_lo = _lib.ptr(k.hi), _lib.ptr(k.lo), _lib.ptr(v.hi), _lib.ptr(v.lo)
            a.k_norms, a.v_norms = _lib.ptr(k.norms), _lib.ptr(v.norms)
            a.k_cent_hi, a.k_cent_lo = _lib.ptr(k.cent_hi), _lib.ptr(k.cent_lo)
            a.v_cent_hi, a.v_cent_lo = _lib.ptr(v.cent_hi), _lib.ptr(v.cent_lo)
            a.v_cent_scale_hi, a.v_cent_scale_lo = v.fp16_scale_hi, v.fp16_scale_lo
            a.tables = _lib.ptr(self._tables)
            if self.qjl_correction and k.qbits is not None:
                a.qjl_proj = _lib.ptr(self._qjl_proj)
                a.k_qjl_bits, a.v_qjl_bits = _lib.ptr(k.qbits), _lib.ptr(v.qbits)
                a.k_qjl_gamma, a.v_qjl_gamma = _lib.ptr(k.qgamma), _lib.ptr(v.qgamma)
        dense_dtype = None
        if self.sink_keys is not None:
            a.sink_k, a.sink_v = self.sink_keys.data_ptr(), self.sink_values.data_ptr()
            a.sink_lane_stride = self.sink_keys.shape[2]
            dense_dtype = self.sink_keys.dtype
        if self.keys is not None:
            a.res_k, a.res_v = self.keys.data_ptr(), self.values.data_ptr()
            a.res_lane_stride = self.keys.shape[2]
            if dense_dtype is not None and dense_dtype != self.keys.dtype:
                raise RuntimeError("sink and recent-token buffers have different dtypes")
            dense_dtype = self.keys.dtype
        a.dense_dtype = _lib.dtype_code(dense_dtype) if dense_dtype is not None else _lib.TQ_F16
        a.out_dtype = _lib.dtype_code(out_dtype)
        return a

    def make_mask(self, N: int, offset: int = 0, return_array: bool = False, window_size: int | None = None) -> Any | None:
        """``None`` for a single-token step, ``"causal"`` otherwise; sliding windows are rejected (cache.py:708-724)."""
        if window_size is not None:
            raise NotImplementedError(
                "TurboQuantKVCache does not support sliding-window attention "
                f"(window_size={window_size}). Use the model's default cache for sliding-window layers.")
        if N == 1 and not return_array:
            return None
        return "causal"
