"""Decode attention straight from the packed cache against the oracle.

Oracle = reference cache (restated, pinned) -> dense K/V -> float32 softmax attention.  Tolerance: 1e-3
of the output's largest magnitude (the task's bound for attention outputs at fp32 accumulation).
"""

import numpy as np
import pytest
import torch

from gpu_util import cu, host, host_tables, kv_like

pytestmark = pytest.mark.gpu


def _case(oracle, rs, b, hq, hkv, t, d, kb, vb, rw, sink, chunk=0, dtype=np.float16, qjl=False):
    """Build the cache with the oracle on the CPU and hand its exact state (packed codes, norms, sink and
    recent tokens) to a GPU cache, so the comparison isolates the attention arithmetic: packed codes are
    only bit-exact given identical rotated inputs, and one code that rounds the other way on a boundary
    would by itself move an output by more than 1e-3."""
    from mlx_turboquant_b200 import TurboQuantKVCache
    k, v = kv_like(rs, (b, hkv, t, d), dtype), kv_like(rs, (b, hkv, t, d), dtype)
    q = (rs.randn(b, hq, 1, d) / np.sqrt(d)).astype(dtype)
    ref_c = oracle.KVCacheOracle(d, host_tables(d), kb, vb, rw, fp16_sink_size=sink, chunk_size=chunk, qjl_correction=qjl)
    rk, rv = ref_c.update_and_fetch(k, v)
    c = TurboQuantKVCache(head_dim=d, num_kv_heads=hkv, key_bits=kb, value_bits=vb, residual_window=rw,
                          fp16_sink_size=sink, chunk_size=chunk, qjl_correction=qjl)
    g = lambda a: None if a is None else cu(a)   # noqa: E731
    ck, cv = (ref_c.comp["k"] or [None] * 3), (ref_c.comp["v"] or [None] * 3)
    state = (g(ref_c.k), g(ref_c.v), g(ck[0]), g(ck[2]), g(cv[0]), g(cv[2]), g(ref_c.sink_k), g(ref_c.sink_v),
             g(ck[1]), g(cv[1]))
    if qjl:
        sk, sv = ref_c.sketch.get("k", (None, None)), ref_c.sketch.get("v", (None, None))
        i32 = lambda a: None if a is None else cu(a.view(np.int32))   # noqa: E731  (sign words travel as int32)
        state = state + (i32(sk[0]), g(sk[1]), i32(sv[0]), g(sv[1]))
    c.state = state
    c.meta_state = {"offset": str(ref_c.offset), "compressed_len": str(ref_c.comp_len), "sink_len": str(ref_c.sink_len),
                    "fp16_len": str(ref_c.fp_len), "fp16_capacity": str(0 if ref_c.k is None else ref_c.k.shape[2])}
    return c, cu(q), oracle.attention(q, rk, rv)


def _check(out, ref, tol=1e-3):
    """1e-3 of the largest output magnitude for float32 results (fp32 accumulation); a float16 result is
    allowed one more half-ulp of its own rounding (2^-11)."""
    if out.dtype != torch.float32:
        tol = tol + 2.0 ** -11
    err = np.abs(host(out.float()) - ref).max() / np.abs(ref).max()
    assert np.isfinite(host(out.float())).all() and err < tol, err


@pytest.mark.parametrize("t", (1, 15, 16, 17, 129, 300, 1000, 2500))
def test_k4v2_direct_path_lengths(oracle, t):
    """d = 128, 4-bit keys / 2-bit values: the table-lookup kernel, ragged token counts, GQA 4."""
    rs = np.random.RandomState(t)
    c, q, ref = _case(oracle, rs, 1, 8, 2, t, 128, 4, 2, 32, 8)
    _check(c.attend(q, out_dtype=torch.float32), ref)


@pytest.mark.parametrize("d", (64, 96, 128, 256))
@pytest.mark.parametrize("kb,vb", ((4, 2), (3, 2), (2, 2), (3.5, 3.5), (4, 4), (2, 3)))
def test_general_path_bit_widths_and_head_dims(oracle, d, kb, vb):
    rs = np.random.RandomState(int(d + 10 * kb + vb))
    c, q, ref = _case(oracle, rs, 2, 4, 2, 333, d, kb, vb, 16, 4)
    _check(c.attend(q, out_dtype=torch.float32), ref)


@pytest.mark.parametrize("hq,hkv", ((4, 4), (8, 1), (16, 1), (12, 4), (32, 8)))
def test_head_grouping(oracle, hq, hkv):
    """MHA, GQA up to 8 query heads per KV head in one pass, 16 per KV head in two head groups."""
    rs = np.random.RandomState(hq * 100 + hkv)
    c, q, ref = _case(oracle, rs, 1, hq, hkv, 700, 128, 4, 2, 64, 16)
    _check(c.attend(q, out_dtype=torch.float32), ref)


def test_direct_and_general_paths_agree(oracle):
    from mlx_turboquant_b200.kernels import set_tuning
    rs = np.random.RandomState(9)
    c, q, ref = _case(oracle, rs, 2, 8, 2, 4000, 128, 4, 2, 128, 128)
    a = c.attend(q, out_dtype=torch.float32)
    set_tuning("decode_force_general", 1)
    try:
        g = c.attend(q, out_dtype=torch.float32)
    finally:
        set_tuning("decode_force_general", 0)
    _check(a, ref)
    _check(g, ref)
    assert np.abs(host(a.float()) - host(g.float())).max() <= 2e-3 * np.abs(ref).max()
    for splits in (1, 3, 64):                       # the result does not depend on the split count
        set_tuning("decode_splits", splits)
        try:
            _check(c.attend(q, out_dtype=torch.float32), ref)
        finally:
            set_tuning("decode_splits", 0)


def test_regions_present_or_absent(oracle):
    rs = np.random.RandomState(10)
    for (t, rw, sink) in ((40, 64, 0), (40, 64, 8), (500, 0, 0), (500, 16, 0), (8, 64, 16)):
        c, q, ref = _case(oracle, rs, 1, 4, 2, t, 128, 4, 2, rw, sink)
        _check(c.attend(q, out_dtype=torch.float32), ref)
    from mlx_turboquant_b200 import TurboQuantKVCache
    with pytest.raises(ValueError):
        TurboQuantKVCache(128, 2).attend(q)
    with pytest.raises(NotImplementedError):
        c.attend(torch.zeros(1, 4, 2, 128, device="cuda", dtype=torch.float16))


@pytest.mark.parametrize("dtype", (np.float32,))
def test_float32_cache_and_query(oracle, dtype):
    rs = np.random.RandomState(12)
    c, q, ref = _case(oracle, rs, 1, 8, 2, 600, 128, 4, 2, 32, 8, dtype=dtype)
    out = c.attend(q)
    assert out.dtype == torch.float32
    _check(out, ref)
    _check(c.attend(q.half()), ref)          # float16 query -> float16 result by default


def test_incremental_decode_steps_match_dense_attention(oracle):
    """Prefill then 40 single-token steps; every step's packed attention equals attention over the
    dense tensors the same cache returns (the reference's own consumer contract)."""
    from mlx_turboquant_b200 import TurboQuantKVCache
    rs = np.random.RandomState(13)
    d, hkv, hq = 128, 2, 8
    c = TurboQuantKVCache(head_dim=d, num_kv_heads=hkv, residual_window=16, fp16_sink_size=4)
    k, v = cu(kv_like(rs, (1, hkv, 340, d))), cu(kv_like(rs, (1, hkv, 340, d)))
    c.update(k[:, :, :300], v[:, :, :300])
    for i in range(300, 340):
        dk, dv = c.update_and_fetch(k[:, :, i:i + 1], v[:, :, i:i + 1])
        q = cu((rs.randn(1, hq, 1, d) / np.sqrt(d)).astype(np.float16))
        ref = oracle.attention(host(q), host(dk), host(dv))
        _check(c.attend(q, out_dtype=torch.float32), ref)


def test_benchmark_shape_against_gpu_dense_attention():
    """Llama-3.1-8B layer shape at the full 32768-token context (128 sink + 32512 packed + 128 recent):
    too large for the CPU oracle in a test, so the packed kernel is checked against float32 softmax
    attention over the dense tensors the same cache returns (torch, on the GPU)."""
    from mlx_turboquant_b200 import TurboQuantKVCache
    g = torch.Generator(device="cuda").manual_seed(1001)
    b, hq, hkv, t, d = 1, 32, 8, 32768, 128
    scale = torch.exp(0.5 * torch.randn(b, hkv, t, 1, device="cuda", generator=g))
    k = (torch.randn(b, hkv, t, d, device="cuda", generator=g) * scale).half()
    v = (torch.randn(b, hkv, t, d, device="cuda", generator=g) * scale).half()
    q = (torch.randn(b, hq, 1, d, device="cuda", generator=g) / d ** 0.5).half()
    c = TurboQuantKVCache(head_dim=d, num_kv_heads=hkv, residual_window=128, fp16_sink_size=128)
    dk, dv = c.update_and_fetch(k, v)
    assert (c._sink_len, c._compressed_len, c._fp16_len) == (128, 32512, 128)
    kk = dk.float().repeat_interleave(hq // hkv, dim=1)
    vv = dv.float().repeat_interleave(hq // hkv, dim=1)
    p = torch.softmax((q.float() @ kk.transpose(-1, -2)) * d ** -0.5, dim=-1)
    ref = (p @ vv).cpu().numpy()
    _check(c.attend(q, out_dtype=torch.float32), ref)


@pytest.mark.parametrize("d,hq,hkv", ((96, 4, 4), (128, 8, 2), (64, 4, 1)))
def test_qjl_sketch_in_packed_attention(oracle, d, hq, hkv):
    """QJL on: attention over packed codes plus sign sketches equals attention over the reference's corrected dense
    K / V (cache.py:396-427).  The sketch forces the general kernel also for 4-bit keys / 2-bit values at d = 128."""
    rs = np.random.RandomState(1000 + d)
    c, q, ref = _case(oracle, rs, 2, hq, hkv, 777, d, 4, 2, 32, 16, qjl=True)
    _check(c.attend(q, out_dtype=torch.float32), ref)
    c, q, ref = _case(oracle, rs, 1, hq, hkv, 300, d, 3.5, 3.5, 16, 0, chunk=64, qjl=True)
    _check(c.attend(q, out_dtype=torch.float32), ref)


def test_calls_of_different_shapes_share_a_workspace(oracle):
    """The scratch buffer is shared by every cache on a stream: a call with few (sequence, KV head) lanes followed by a
    call with many must not find the first call's partials where it expects zeroed arrival counters."""
    rs = np.random.RandomState(77)
    small = _case(oracle, rs, 1, 4, 1, 3000, 128, 4, 2, 32, 8)
    big = _case(oracle, rs, 6, 32, 32, 400, 64, 4, 2, 16, 4)
    for _ in range(2):
        for c, q, ref in (small, big, small):
            _check(c.attend(q, out_dtype=torch.float32), ref)


def test_attend_into_a_given_tensor(oracle):
    c, q, _ = _case(oracle, np.random.RandomState(77), 1, 8, 2, 700, 128, 4, 2, 32, 16)
    want = c.attend(q)
    out = torch.full_like(want, float("nan"))
    assert c.attend(q, out=out) is out and torch.equal(out, want)
    with pytest.raises(ValueError):
        c.attend(q, out=torch.empty(3, device="cuda", dtype=torch.float16))
