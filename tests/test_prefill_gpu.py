"""Causal attention for several query tokens straight from packed storage against the oracle.

Oracle = reference cache (restated, pinned) -> dense K / V -> float32 causal softmax attention in which query i (one of
the last T_q tokens of the cache) sees tokens 0 .. its own position.  Same identical-state set-up and the same 1e-3
bound as the decode tests; the shapes follow the reference's fused-score tests (tests/test_fused_attention.py:150-288:
T_q in {1, 4, 32}, T_kv up to 4000, bits 2 / 3 / 4, head_dim 96 / 128 / 256) and go beyond them (T_q = 512, GQA, sink).
"""

import numpy as np
import pytest
import torch

from gpu_util import cu, host, host_tables, kv_like

pytestmark = pytest.mark.gpu


@pytest.fixture(params=["tcgen05", "mma.sync"], autouse=True)
def which_kernel(request):
    """Every case runs twice: with the tensor-core (tcgen05) kernel where it applies - head_dim 128, at least 64 query rows;
    byte-table unpack for 4-bit keys / 2-bit values, code by code for every other width - and with the mma.sync kernel everywhere."""
    from mlx_turboquant_b200 import kernels
    kernels.set_tuning("prefill_tc", 1 if request.param == "tcgen05" else 0)
    yield request.param
    kernels.set_tuning("prefill_tc", 1)
    from mlx_turboquant_b200 import _lib
    assert _lib.lib().tq_device_status() == 0


def causal_reference(q, k, v, scale=None):
    """q (B, Hq, Tq, D): the last Tq tokens; k, v (B, Hkv, T, D) float32.  float32 softmax, GQA head repeat."""
    q, k, v = (np.asarray(x).astype(np.float32) for x in (q, k, v))
    b, hq, tq, d = q.shape
    t = k.shape[2]
    rep = hq // k.shape[1]
    scale = np.float32(d ** -0.5 if scale is None else scale)
    out = np.zeros((b, hq, tq, d), dtype=np.float32)
    pos = (t - tq + np.arange(tq))[:, None]
    mask = np.arange(t)[None, :] <= pos
    for bi in range(b):
        for h in range(hq):
            s = (q[bi, h] @ k[bi, h // rep].T) * scale
            s = np.where(mask, s, -np.inf)
            s = s - s.max(axis=-1, keepdims=True)
            p = np.exp(s)
            p /= p.sum(axis=-1, keepdims=True)
            out[bi, h] = p @ v[bi, h // rep]
    return out


def _case(oracle, rs, b, hq, hkv, t, tq, d, kb, vb, rw, sink, chunk=0, dtype=np.float16, bf16=False):
    from mlx_turboquant_b200 import TurboQuantKVCache
    k, v = kv_like(rs, (b, hkv, t, d), dtype), kv_like(rs, (b, hkv, t, d), dtype)
    q = (rs.randn(b, hq, tq, d) / np.sqrt(d)).astype(dtype)
    if bf16:
        rnd = lambda a: torch.from_numpy(np.ascontiguousarray(a, dtype=np.float32)).to(torch.bfloat16).float().numpy()   # noqa: E731
        k, v, q = rnd(k), rnd(v), rnd(q)
    ref_c = oracle.KVCacheOracle(d, host_tables(d), kb, vb, rw, fp16_sink_size=sink, chunk_size=chunk)
    rk, rv = ref_c.update_and_fetch(k, v)
    c = TurboQuantKVCache(head_dim=d, num_kv_heads=hkv, key_bits=kb, value_bits=vb, residual_window=rw, fp16_sink_size=sink, chunk_size=chunk)
    g = lambda a: None if a is None else cu(a)   # noqa: E731
    gd = (lambda a: None if a is None else cu(a).to(torch.bfloat16)) if bf16 else g   # noqa: E731
    ck, cv = (ref_c.comp["k"] or [None] * 3), (ref_c.comp["v"] or [None] * 3)
    c.state = (gd(ref_c.k), gd(ref_c.v), g(ck[0]), g(ck[2]), g(cv[0]), g(cv[2]), gd(ref_c.sink_k), gd(ref_c.sink_v), g(ck[1]), g(cv[1]))
    c.meta_state = {"offset": str(ref_c.offset), "compressed_len": str(ref_c.comp_len), "sink_len": str(ref_c.sink_len),
                    "fp16_len": str(ref_c.fp_len), "fp16_capacity": str(0 if ref_c.k is None else ref_c.k.shape[2])}
    return c, (cu(q).to(torch.bfloat16) if bf16 else cu(q)), causal_reference(q, rk, rv)


def _check(out, ref, tol=1e-3):
    o = host(out.float())
    err = np.abs(o - ref).max() / np.abs(ref).max()
    assert np.isfinite(o).all() and err < tol, err


@pytest.mark.parametrize("tq", (4, 32, 512))
@pytest.mark.parametrize("t", (128, 4000))
@pytest.mark.parametrize("bits", (2, 3, 4))
def test_query_counts_context_lengths_and_bit_widths(oracle, tq, t, bits):
    """d = 128, GQA 4: queries inside the recent window only (T_q = 4), reaching back into the packed region (T_q = 512 of
    4000 with 16 recent tokens), or making up the whole cache (T_q = 512 > T_kv = 128 is skipped)."""
    if tq > t:
        pytest.skip("more query tokens than cached tokens")
    rs = np.random.RandomState(tq + t + bits)
    c, q, ref = _case(oracle, rs, 1, 8, 2, t, tq, 128, bits, bits, 16, 4)
    out = c.attend(q, out_dtype=torch.float32)
    assert tuple(out.shape) == (1, 8, tq, 128)
    _check(out, ref)


@pytest.mark.parametrize("d,hq,hkv", ((64, 4, 4), (96, 8, 8), (128, 8, 1), (128, 32, 2), (256, 4, 2), (128, 6, 2)))
def test_head_dims_and_groupings(oracle, d, hq, hkv):
    """MHA (one column per token), GQA 2 / 3 (padded to 4) / 8, 16 query heads per KV head in two head groups; batch 2."""
    rs = np.random.RandomState(d + hq)
    c, q, ref = _case(oracle, rs, 2, hq, hkv, 700, 70, d, 4, 2, 32, 8)
    _check(c.attend(q, out_dtype=torch.float32), ref)


@pytest.mark.parametrize("kw", (dict(kb=3.5, vb=3.5, rw=16, sink=0, chunk=64), dict(kb=4, vb=2, rw=0, sink=0), dict(kb=2, vb=3, rw=64, sink=16),
                                dict(kb=4, vb=2, rw=300, sink=40)))
def test_regions_and_fractional_widths(oracle, kw):
    """Fractional widths with chunked drains, no recent window, a cache that is still all uncompressed (window 300 > tokens),
    sink + window; the queries straddle whatever regions exist."""
    rs = np.random.RandomState(int(kw["kb"] * 10 + kw["rw"]))
    c, q, ref = _case(oracle, rs, 1, 8, 2, 290, 100, 128, kw["kb"], kw["vb"], kw["rw"], kw["sink"], chunk=kw.get("chunk", 0))
    _check(c.attend(q, out_dtype=torch.float32), ref)


@pytest.mark.parametrize("bf16", (False, True))
def test_float32_and_bfloat16_caches(oracle, bf16):
    rs = np.random.RandomState(99 + bf16)
    c, q, ref = _case(oracle, rs, 1, 8, 2, 500, 40, 128, 4, 2, 32, 8, dtype=np.float32, bf16=bf16)
    out = c.attend(q)
    assert out.dtype == (torch.bfloat16 if bf16 else torch.float32)
    _check(out, ref, tol=1e-3 + (2.0 ** -8 if bf16 else 0))


def test_single_query_token_agrees_with_the_decode_kernel(oracle):
    """T_q = 1 through the multi-token entry point equals the decode kernels' result (to rounding)."""
    import ctypes as C

    from mlx_turboquant_b200 import _lib
    rs = np.random.RandomState(3)
    c, q, ref = _case(oracle, rs, 1, 8, 2, 900, 1, 128, 4, 2, 32, 8)
    dec = c.attend(q, out_dtype=torch.float32)
    out = torch.empty_like(dec)
    a = c._fill_decode_args(1, 8, q.dtype, torch.float32, None)
    a.q, a.out = q.data_ptr(), out.data_ptr()
    a.c_len, a.sink_len, a.res_len = c._compressed_len, c._sink_len, c._fp16_len
    _lib.check(_lib.lib().tq_prefill_attn(C.byref(a), 1, torch.cuda.current_stream().cuda_stream))
    _check(out, ref)
    assert float((out - dec).abs().max()) <= 1e-3 * float(dec.abs().max())


def test_argument_errors(oracle):
    from mlx_turboquant_b200 import TurboQuantKVCache
    rs = np.random.RandomState(4)
    c, q, _ = _case(oracle, rs, 1, 8, 2, 100, 8, 128, 4, 2, 16, 0)
    with pytest.raises(ValueError):
        c.attend(torch.zeros(1, 8, 101, 128, device="cuda", dtype=torch.float16))          # more queries than cached tokens
    cq = TurboQuantKVCache(head_dim=128, num_kv_heads=2, qjl_correction=True)
    cq.update(cu(kv_like(rs, (1, 2, 300, 128))), cu(kv_like(rs, (1, 2, 300, 128))))
    with pytest.raises(NotImplementedError):
        cq.attend(q)


@pytest.mark.parametrize("b,hq,hkv,t,tq,rw,sink", ((1, 8, 2, 4000, 512, 16, 4), (2, 32, 8, 3000, 1000, 128, 128), (1, 4, 4, 2500, 2500, 64, 0),
                                                  (1, 16, 2, 1500, 130, 0, 32)))
def test_long_chunks_k4v2(oracle, b, hq, hkv, t, tq, rw, sink):
    """4-bit keys / 2-bit values at head_dim 128 (the tensor-core kernel's shape): chunks that span many 128-token tiles,
    a chunk that is the whole cache, row tiles that end inside a query token's head group, no recent window."""
    rs = np.random.RandomState(b * 1000 + tq)
    c, q, ref = _case(oracle, rs, b, hq, hkv, t, tq, 128, 4, 2, rw, sink)
    _check(c.attend(q, out_dtype=torch.float32), ref)
    out16 = c.attend(q)
    assert out16.dtype == torch.float16
    _check(out16, ref, tol=1e-3 + 2.0 ** -11)


@pytest.mark.parametrize("v_scale", (1e-4, 3e4))
def test_value_norm_range(oracle, v_scale):
    """Value norms far from 1 (the weights ride on fp16 operands under a power-of-two scale that follows the largest norm)."""
    from mlx_turboquant_b200 import TurboQuantKVCache
    rs = np.random.RandomState(77)
    b, hq, hkv, t, tq, d = 1, 8, 2, 1200, 256, 128
    k = kv_like(rs, (b, hkv, t, d), np.float32)
    v = (kv_like(rs, (b, hkv, t, d), np.float32) * v_scale * np.exp(rs.randn(b, hkv, t, 1))).astype(np.float32)
    q = (rs.randn(b, hq, tq, d) / np.sqrt(d)).astype(np.float32)
    ref_c = oracle.KVCacheOracle(d, host_tables(d), 4, 2, 64, fp16_sink_size=16, chunk_size=0)
    rk, rv = ref_c.update_and_fetch(k, v)
    c = TurboQuantKVCache(head_dim=d, num_kv_heads=hkv, key_bits=4, value_bits=2, residual_window=64, fp16_sink_size=16)
    g = lambda a: None if a is None else cu(a)   # noqa: E731
    ck, cv = ref_c.comp["k"], ref_c.comp["v"]
    c.state = (g(ref_c.k), g(ref_c.v), g(ck[0]), g(ck[2]), g(cv[0]), g(cv[2]), g(ref_c.sink_k), g(ref_c.sink_v), g(ck[1]), g(cv[1]))
    c.meta_state = {"offset": str(ref_c.offset), "compressed_len": str(ref_c.comp_len), "sink_len": str(ref_c.sink_len),
                    "fp16_len": str(ref_c.fp_len), "fp16_capacity": str(ref_c.k.shape[2])}
    _check(c.attend(cu(q)), causal_reference(q, rk, rv))
