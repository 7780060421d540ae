"""CPU oracle for the TurboQuant KV-compression / compressed-attention path.

TEST INFRASTRUCTURE, NOT PRODUCT CODE.  Only the test-suite, the smoke check and
the benchmark's CPU-baseline leg may import this module; the shipped package
never does (it fails loudly when its CUDA library is missing instead).

Every function restates, in float32-faithful NumPy, what the reference
(alex-rentel/mlx-turboquant v1.0.4) computes; the reference file:line each one
follows is given in its docstring.  Parity status: PINNED - the fixtures under
``tests/golden`` were produced by running the reference's own unmodified
modules (on a NumPy stand-in for ``mlx.core``) and every function here is
checked against them bit-for-bit by ``tests/test_oracle_golden.py``.

The decode-attention function has no counterpart on the reference's supported
path (the reference hands a dense K/V to a third-party attention call, mlx
``mx.fast.scaled_dot_product_attention``, mlx>=0.31.0); it is defined here as
plain float32 softmax attention over the reference cache's dense output.
"""

from __future__ import annotations

import math

import numpy as np

F32 = np.float32


# --------------------------------------------------------------------------- rotation
def rotation_matrix(d: int, seed: int = 42) -> np.ndarray:
    """Sign-fixed Q of the QR of a seeded Gaussian matrix (rotation.py:17-36)."""
    g = np.random.RandomState(seed).randn(d, d).astype(F32)
    q, r = np.linalg.qr(g)
    s = np.sign(np.diag(r))
    s[s == 0] = 1
    return (q * s[None, :]).astype(F32)


def rotate_fwd(x: np.ndarray, rot: np.ndarray) -> np.ndarray:
    """y = x @ R.T (rotation.py:55-65); the query pre-rotation is the same op (rotation.py:81-110)."""
    return x @ rot.T


def rotate_inv(y: np.ndarray, rot: np.ndarray) -> np.ndarray:
    """x = y @ R (rotation.py:68-78)."""
    return y @ rot


# --------------------------------------------------------------------------- codebook
def lloyd_max(d: int, bits: int, num_iter: int = 500, grid_size: int = 10000):
    """Lloyd-Max centroids/boundaries for N(0, 1/d) on a +-6 sigma grid (codebook.py:55-116).

    float64 throughout; centroids and boundaries are each cast to float32 at the
    end, so a float32 boundary is not the midpoint of the float32 centroids.
    Only d >= 32 (Gaussian density) is restated; the reference switches to a Beta
    density below that (codebook.py:36-46), which no shipped head size uses.
    """
    if d < 32:
        raise ValueError("oracle restates the Gaussian branch only (d >= 32)")
    levels = 1 << bits
    sigma = 1.0 / math.sqrt(d)
    lo, hi = -6 * sigma, 6 * sigma
    grid = np.linspace(lo, hi, grid_size)
    dx = grid[1] - grid[0]
    var = 1.0 / d
    pdf = np.exp(-0.5 * grid * grid / var) / math.sqrt(2 * math.pi * var)
    pdf = pdf / (np.sum(pdf) * dx)
    cdf = np.cumsum(pdf) * dx
    cdf = cdf / cdf[-1]
    cent = np.interp(np.linspace(0.5 / levels, 1 - 0.5 / levels, levels), cdf, grid)
    for _ in range(num_iter):
        bnd = (cent[:-1] + cent[1:]) / 2.0
        edges = np.concatenate([[lo], bnd, [hi]])
        new = np.zeros(levels)
        for i in range(levels):
            if i == levels - 1:
                m = (grid >= edges[i]) & (grid <= edges[i + 1])
            else:
                m = (grid >= edges[i]) & (grid < edges[i + 1])
            w = pdf[m]
            new[i] = np.sum(grid[m] * w) / w.sum() if w.sum() > 0 else cent[i]
        if np.max(np.abs(new - cent)) < 1e-12:
            break
        cent = new
    bnd = (cent[:-1] + cent[1:]) / 2.0
    return cent.astype(F32), bnd.astype(F32)


def quantize_scalar(y: np.ndarray, boundaries: np.ndarray) -> np.ndarray:
    """Index = number of boundaries strictly exceeded, uint8 (codebook.py:203-225)."""
    flat = np.asarray(y, dtype=F32).reshape(-1)
    out = np.empty(flat.shape, dtype=np.uint8)
    step = 1 << 20  # bound the (N, 2^b-1) comparison matrix
    b = np.asarray(boundaries, dtype=F32)[None, :]
    for s in range(0, flat.size, step):
        out[s:s + step] = np.sum(flat[s:s + step, None] > b, axis=-1).astype(np.uint8)
    return out.reshape(np.shape(y))


def dequantize_scalar(idx: np.ndarray, centroids: np.ndarray) -> np.ndarray:
    """Centroid gather (codebook.py:228-238)."""
    return np.asarray(centroids, dtype=F32)[np.asarray(idx).astype(np.int32)]


# --------------------------------------------------------------------------- packing
def packed_width(d: int, bits: int) -> int:
    """Bytes per vector: d/8, d/4, 3d/8, d/2 for 1..4 bits (packing.py:9-208)."""
    if bits not in (1, 2, 3, 4):
        raise ValueError(f"Unsupported bit-width: {bits}. Use 1, 2, 3, or 4.")
    return d * bits // 8


def pack(idx: np.ndarray, bits: int) -> np.ndarray:
    """Little-endian-in-byte packing (packing.py:9-34, 62-99, 134-156, 176-194, 211-222)."""
    idx = np.asarray(idx)
    d = idx.shape[-1]
    lead = idx.shape[:-1]
    if bits not in (1, 2, 3, 4):
        raise ValueError(f"Unsupported bit-width: {bits}. Use 1, 2, 3, or 4.")
    per = {1: 8, 2: 4, 3: 8, 4: 2}[bits]
    assert d % per == 0, f"Last dimension {d} must be divisible by {per} for {bits}-bit packing"
    g = idx.reshape(-1, d // per, per).astype(np.uint32)
    if bits == 3:
        b0 = g[..., 0] | (g[..., 1] << 3) | (g[..., 2] << 6)
        b1 = (g[..., 2] >> 2) | (g[..., 3] << 1) | (g[..., 4] << 4) | (g[..., 5] << 7)
        b2 = (g[..., 5] >> 1) | (g[..., 6] << 2) | (g[..., 7] << 5)
        out = np.stack([b0, b1, b2], axis=-1).astype(np.uint8)
        return out.reshape(*lead, d * 3 // 8)
    acc = np.zeros(g.shape[:-1], dtype=np.uint32)
    for k in range(per):
        acc |= g[..., k] << (bits * k)
    return acc.astype(np.uint8).reshape(*lead, d // per)


def unpack(packed: np.ndarray, bits: int, d: int) -> np.ndarray:
    """Inverse of :func:`pack` (packing.py:37-59, 102-131, 159-173, 197-208, 225-236)."""
    packed = np.asarray(packed)
    lead = packed.shape[:-1]
    if bits not in (1, 2, 3, 4):
        raise ValueError(f"Unsupported bit-width: {bits}. Use 1, 2, 3, or 4.")
    flat = packed.reshape(-1, packed.shape[-1]).astype(np.uint32)
    if bits == 3:
        g = flat.reshape(flat.shape[0], d // 8, 3)
        b0, b1, b2 = g[..., 0], g[..., 1], g[..., 2]
        v = [b0 & 7, (b0 >> 3) & 7, ((b0 >> 6) | (b1 << 2)) & 7, (b1 >> 1) & 7,
             (b1 >> 4) & 7, ((b1 >> 7) | (b2 << 1)) & 7, (b2 >> 2) & 7, (b2 >> 5) & 7]
        return np.stack(v, axis=-1).reshape(*lead, d).astype(np.uint8)
    per = 8 // bits
    mask = (1 << bits) - 1
    v = [(flat >> (bits * k)) & mask for k in range(per)]
    return np.stack(v, axis=-1).reshape(*lead, d).astype(np.uint8)


# --------------------------------------------------------------------------- MSE quantizer
def norms_f32(x: np.ndarray) -> np.ndarray:
    """float32 L2 norm over the last axis of the float32-cast input (cache.py:235-236)."""
    xf = np.asarray(x).astype(F32)
    return np.sqrt(np.sum(xf * xf, axis=-1, dtype=F32))


def normalise_rotate(x: np.ndarray, rot: np.ndarray):
    """cast -> norm -> divide by max(norm, 1e-10) -> @ R.T (cache.py:232-241, quantizer.py:64-73)."""
    xf = np.asarray(x).astype(F32)
    n = norms_f32(xf)
    safe = np.maximum(n, F32(1e-10))
    y = (xf / safe[..., None]).reshape(-1, xf.shape[-1]) @ rot.T
    return y.reshape(xf.shape), n


def mse_quantize(x, rot, boundaries, bits: int):
    """TurboQuantMSE.quantize (quantizer.py:54-85) -> (packed u8, norms f32, rotated y)."""
    y, n = normalise_rotate(x, rot)
    return pack(quantize_scalar(y, boundaries), bits), n, y


def mse_dequantize(packed, norms, rot, centroids, bits: int, d: int):
    """TurboQuantMSE.dequantize (quantizer.py:87-109; same math as cache.py:336-343)."""
    yh = dequantize_scalar(unpack(packed, bits, d), centroids)
    xh = yh.reshape(-1, d) @ rot
    return xh.reshape(yh.shape) * np.asarray(norms).astype(F32)[..., None]


def split_quantize(x, rot, bnd_hi, bits_hi: int, bnd_lo, bits_lo: int):
    """Fractional bits: first D/2 rotated coords at bits_hi, rest at bits_lo (cache.py:253-274)."""
    y, n = normalise_rotate(x, rot)
    h = y.shape[-1] // 2
    return (pack(quantize_scalar(y[..., :h], bnd_hi), bits_hi),
            pack(quantize_scalar(y[..., h:], bnd_lo), bits_lo), n, y)


def split_dequantize(p_hi, p_lo, norms, rot, cent_hi, bits_hi, cent_lo, bits_lo, d: int):
    """Fractional-bit dequantize (cache.py:276-300)."""
    h = d // 2
    yh = np.concatenate([dequantize_scalar(unpack(p_hi, bits_hi, h), cent_hi),
                         dequantize_scalar(unpack(p_lo, bits_lo, h), cent_lo)], axis=-1)
    xh = yh.reshape(-1, d) @ rot
    return xh.reshape(yh.shape) * np.asarray(norms).astype(F32)[..., None]


# --------------------------------------------------------------------------- QJL
def projection_matrix(d: int, m: int, seed: int = 12345) -> np.ndarray:
    """(m, d) i.i.d. N(0,1) float32 (qjl.py:23-36)."""
    return np.random.RandomState(seed).randn(m, d).astype(F32)


def qjl_quantize(residual, proj):
    """signs = (r @ S.T >= 0), gamma = ||r|| (qjl.py:47-67)."""
    r = np.asarray(residual)
    return (r @ proj.T) >= 0, np.sqrt(np.sum(r * r, axis=-1, dtype=r.dtype))


def qjl_dequantize(signs, gamma, proj, d: int):
    """(sqrt(pi/2)/d) * gamma * (z @ S), z = +-1 (qjl.py:70-94)."""
    z = np.where(signs, F32(1.0), F32(-1.0))
    return (math.sqrt(math.pi / 2) / d) * np.asarray(gamma)[..., None] * (z @ proj)


def qjl_correct(original, decompressed, proj):
    """Residual sketch applied at compression time (cache.py:396-427)."""
    r = np.asarray(original).astype(F32) - np.asarray(decompressed).astype(F32)
    d = r.shape[-1]
    flat = r.reshape(-1, d)
    s, g = qjl_quantize(flat, proj)
    return decompressed + qjl_dequantize(s, g, proj, d).reshape(r.shape)


def prod_quantize(x, rot, boundaries, centroids, bits: int, proj):
    """TurboQuantProd.quantize: (bits-1)-bit MSE + sketch of the residual (quantizer.py:142-168)."""
    d = np.shape(x)[-1]
    packed, n, _ = mse_quantize(x, rot, boundaries, bits - 1)
    r = x - mse_dequantize(packed, n, rot, centroids, bits - 1, d)
    s, g = qjl_quantize(r, proj)
    return packed, n, s, g


def prod_dequantize(packed, norms, signs, gamma, rot, centroids, bits: int, d: int, proj):
    """TurboQuantProd.dequantize (quantizer.py:170-195)."""
    return mse_dequantize(packed, norms, rot, centroids, bits - 1, d) + qjl_dequantize(signs, gamma, proj, d)


# --------------------------------------------------------------------------- scores / attention
def qk_scores(q_rot, packed, norms, centroids, bits: int, d: int):
    """score[q,k] = norm_k * sum_j q_rot[q,j] * c[idx(k,j)] (kernels.py:439-479, 488-506, 517-548)."""
    q_rot = np.asarray(q_rot, dtype=F32)
    if packed.shape[0] == 0 or q_rot.shape[0] == 0:
        return np.zeros((q_rot.shape[0], packed.shape[0]), dtype=F32)  # kernels.py:569-570
    yh = dequantize_scalar(unpack(packed, bits, d), centroids)
    return (q_rot @ yh.T) * np.asarray(norms, dtype=F32)[None, :]


def attention(q, k, v, scale: float | None = None):
    """float32 softmax(scale * q k^T) v with GQA head repeat; no mask (single-token step).

    q (B, Hq, Tq, D); k, v (B, Hkv, T, D).  Stands in for the third-party call the
    reference's consumer makes on the dense cache output (scale = D**-0.5).
    """
    q = np.asarray(q).astype(F32)
    k = np.asarray(k).astype(F32)
    v = np.asarray(v).astype(F32)
    b, hq, tq, d = q.shape
    rep = hq // k.shape[1]
    scale = d ** -0.5 if scale is None else scale
    out = np.empty((b, hq, tq, d), dtype=F32)
    for bi in range(b):
        for h in range(hq):
            s = (q[bi, h] @ k[bi, h // rep].T) * F32(scale)
            s = s - s.max(axis=-1, keepdims=True)
            p = np.exp(s)
            out[bi, h] = (p @ v[bi, h // rep]) / p.sum(axis=-1, keepdims=True)
    return out


# --------------------------------------------------------------------------- cache state machine
class KVCacheOracle:
    """Restatement of TurboQuantKVCache (cache.py:28-706) with value-semantic drains.

    ``tables`` maps bits -> (centroids, boundaries) for this head_dim.
    """

    def __init__(self, head_dim, tables, key_bits=4, value_bits=2, residual_window=128,
                 rotation_seed=42, fp16_sink_size=0, chunk_size=0, qjl_correction=False,
                 qjl_n_proj=32):
        self.d = head_dim
        self.tables = tables
        self.key_bits, self.value_bits = key_bits, value_bits
        self.rw, self.sink_size, self.chunk = residual_window, fp16_sink_size, chunk_size
        self.rot = rotation_matrix(head_dim, rotation_seed)
        self.proj = projection_matrix(head_dim, qjl_n_proj) if qjl_correction else None
        self.sketch = {}          # name -> (sign words uint32 (B,H,T_c), residual norms float32 (B,H,T_c)) when QJL is on
        self.sink_k = self.sink_v = None
        self.sink_len = 0
        self.k = self.v = None            # recent-token buffer, valid [:fp_len]
        self.fp_len = 0
        self.comp = {"k": None, "v": None}  # (packed_hi, packed_lo|None, norms)
        self.comp_len = 0
        self.dense_k = self.dense_v = None  # dequantized (and QJL-corrected) middle
        self.offset = 0

    def _side(self, x, bits):
        """Quantize then immediately dequantize one side of a chunk (cache.py:429-461)."""
        if bits != int(bits):
            bh, bl = int(bits) + 1, int(bits)
            ph, pl, n, _ = split_quantize(x, self.rot, self.tables[bh][1], bh, self.tables[bl][1], bl)
            dq = split_dequantize(ph, pl, n, self.rot, self.tables[bh][0], bh, self.tables[bl][0], bl, self.d)
        else:
            b = int(bits)
            ph, n, _ = mse_quantize(x, self.rot, self.tables[b][1], b)
            pl = None
            dq = mse_dequantize(ph, n, self.rot, self.tables[b][0], b, self.d)
        if self.proj is not None:
            # the reference applies the sketch and forgets it (cache.py:396-427); the signs and norms are kept here as
            # well, as 32-bit words and float32, so that tests can hand a kernel exactly the state the correction used
            r = np.asarray(x).astype(F32) - np.asarray(dq).astype(F32)
            sg, gm = qjl_quantize(r.reshape(-1, self.d), self.proj)
            words = (sg.astype(np.uint64) << np.arange(sg.shape[1], dtype=np.uint64)).sum(axis=1).astype(np.uint32)
            self._last_sketch = (words.reshape(r.shape[:-1]), gm.astype(F32).reshape(r.shape[:-1]))
            dq = qjl_correct(x, dq, self.proj)
        return ph, pl, n, dq

    def _drain(self, n):
        """Compress and evict the first n recent tokens (cache.py:535-575)."""
        old_k = self.k[:, :, :n].copy()
        old_v = self.v[:, :, :n].copy()
        rem = self.fp_len - n
        if rem > 0:
            self.k[:, :, :rem] = self.k[:, :, n:self.fp_len].copy()
            self.v[:, :, :rem] = self.v[:, :, n:self.fp_len].copy()
        self.fp_len = rem
        for name, x, bits in (("k", old_k, self.key_bits), ("v", old_v, self.value_bits)):
            ph, pl, nr, dq = self._side(x, bits)
            if self.proj is not None:
                w, g = self._last_sketch
                prev = self.sketch.get(name)
                self.sketch[name] = (w, g) if prev is None else (np.concatenate([prev[0], w], axis=2), np.concatenate([prev[1], g], axis=2))
            if self.comp[name] is None:
                self.comp[name] = [ph, pl, nr]
                dense = dq
            else:
                c = self.comp[name]
                c[0] = np.concatenate([c[0], ph], axis=2)
                if pl is not None:
                    c[1] = np.concatenate([c[1], pl], axis=2)
                c[2] = np.concatenate([c[2], nr], axis=2)
                prev = self.dense_k if name == "k" else self.dense_v
                dense = np.concatenate([prev, dq], axis=2)
            if name == "k":
                self.dense_k = dense
            else:
                self.dense_v = dense
        self.comp_len += n

    def update_and_fetch(self, keys, values):
        """cache.py:620-706 (sink routing :577-618, schedule :497-533)."""
        t_total = keys.shape[2]
        if self.sink_size > 0 and self.offset < self.sink_size:
            ns = min(self.sink_size - self.offset, t_total)
            if ns > 0:
                if self.sink_k is None:
                    b, h, _, d = keys.shape
                    self.sink_k = np.zeros((b, h, self.sink_size, d), dtype=keys.dtype)
                    self.sink_v = np.zeros((b, h, self.sink_size, d), dtype=values.dtype)
                self.sink_k[:, :, self.offset:self.offset + ns] = keys[:, :, :ns]
                self.sink_v[:, :, self.offset:self.offset + ns] = values[:, :, :ns]
                self.sink_len = self.offset + ns
                keys, values = keys[:, :, ns:], values[:, :, ns:]
        t_new = keys.shape[2]
        if t_new > 0:
            if self.k is None:
                b, h, _, d = keys.shape
                cap = max(t_new, self.rw * 2) + 256
                self.k = np.zeros((b, h, cap, d), dtype=keys.dtype)
                self.v = np.zeros((b, h, cap, d), dtype=values.dtype)
                self.fp_len = 0
            new_len = self.fp_len + t_new
            if new_len > self.k.shape[2]:
                b, h, _, d = self.k.shape
                nk = np.zeros((b, h, new_len + 256, d), dtype=keys.dtype)
                nv = np.zeros((b, h, new_len + 256, d), dtype=values.dtype)
                nk[:, :, :self.fp_len] = self.k[:, :, :self.fp_len]
                nv[:, :, :self.fp_len] = self.v[:, :, :self.fp_len]
                self.k, self.v = nk, nv
            self.k[:, :, self.fp_len:new_len] = keys
            self.v[:, :, self.fp_len:new_len] = values
            self.fp_len = new_len
        self.offset += t_total
        if self.k is not None:
            if self.chunk <= 0:
                if self.fp_len > 2 * self.rw:
                    self._drain(self.fp_len - self.rw)
            else:
                while self.fp_len >= self.rw + self.chunk:
                    self._drain(self.chunk)
        pk, pv = [], []
        if self.sink_len > 0:
            pk.append(self.sink_k[:, :, :self.sink_len])
            pv.append(self.sink_v[:, :, :self.sink_len])
        if self.comp_len > 0:
            pk.append(self.dense_k)
            pv.append(self.dense_v)
        if self.fp_len > 0:
            pk.append(self.k[:, :, :self.fp_len])
            pv.append(self.v[:, :, :self.fp_len])
        if not pk:
            return keys[:, :, :0], values[:, :, :0]
        if len(pk) == 1:
            return pk[0], pv[0]
        return np.concatenate(pk, axis=2), np.concatenate(pv, axis=2)
