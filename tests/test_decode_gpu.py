"""Decode attention straight from the packed cache against the oracle.

Oracle = reference cache (restated, pinned) -> dense K/V -> float32 softmax attention.  Tolerance: 1e-3
of the output's largest magnitude (the task's bound for attention outputs at fp32 accumulation).
"""

import numpy as np
import pytest
import torch

from gpu_util import cu, host, host_tables, kv_like

pytestmark = pytest.mark.gpu


def _bf16_round(a):
    """float32 array rounded to the nearest bfloat16 value (still float32: bfloat16 is a subset)."""
    return torch.from_numpy(np.ascontiguousarray(a, dtype=np.float32)).to(torch.bfloat16).float().numpy()


def _case(oracle, rs, b, hq, hkv, t, d, kb, vb, rw, sink, chunk=0, dtype=np.float16, qjl=False, k_scale=1.0, v_scale=1.0,
          bf16=False):
    """Build the cache with the oracle on the CPU and hand its exact state (packed codes, norms, sink and
    recent tokens) to a GPU cache, so the comparison isolates the attention arithmetic: packed codes are
    only bit-exact given identical rotated inputs, and one code that rounds the other way on a boundary
    would by itself move an output by more than 1e-3.  `bf16`: the inputs are bfloat16 values (the oracle sees
    them as float32, the GPU cache keeps its uncompressed regions and the query in bfloat16)."""
    from mlx_turboquant_b200 import TurboQuantKVCache
    k, v = kv_like(rs, (b, hkv, t, d), dtype), kv_like(rs, (b, hkv, t, d), dtype)
    if k_scale != 1.0 or v_scale != 1.0:
        k, v = (k.astype(np.float32) * k_scale).astype(dtype), (v.astype(np.float32) * v_scale).astype(dtype)
    q = (rs.randn(b, hq, 1, d) / np.sqrt(d)).astype(dtype)
    if bf16:
        k, v, q = _bf16_round(k), _bf16_round(v), _bf16_round(q)
    ref_c = oracle.KVCacheOracle(d, host_tables(d), kb, vb, rw, fp16_sink_size=sink, chunk_size=chunk, qjl_correction=qjl)
    rk, rv = ref_c.update_and_fetch(k, v)
    c = TurboQuantKVCache(head_dim=d, num_kv_heads=hkv, key_bits=kb, value_bits=vb, residual_window=rw,
                          fp16_sink_size=sink, chunk_size=chunk, qjl_correction=qjl)
    g = lambda a: None if a is None else cu(a)   # noqa: E731
    gd = (lambda a: None if a is None else cu(a).to(torch.bfloat16)) if bf16 else g   # noqa: E731
    ck, cv = (ref_c.comp["k"] or [None] * 3), (ref_c.comp["v"] or [None] * 3)
    state = (gd(ref_c.k), gd(ref_c.v), g(ck[0]), g(ck[2]), g(cv[0]), g(cv[2]), gd(ref_c.sink_k), gd(ref_c.sink_v),
             g(ck[1]), g(cv[1]))
    if qjl:
        sk, sv = ref_c.sketch.get("k", (None, None)), ref_c.sketch.get("v", (None, None))
        i32 = lambda a: None if a is None else cu(a.view(np.int32))   # noqa: E731  (sign words travel as int32)
        state = state + (i32(sk[0]), g(sk[1]), i32(sv[0]), g(sv[1]))
    c.state = state
    c.meta_state = {"offset": str(ref_c.offset), "compressed_len": str(ref_c.comp_len), "sink_len": str(ref_c.sink_len),
                    "fp16_len": str(ref_c.fp_len), "fp16_capacity": str(0 if ref_c.k is None else ref_c.k.shape[2])}
    return c, (cu(q).to(torch.bfloat16) if bf16 else cu(q)), oracle.attention(q, rk, rv)


ELEMENTWISE = []      # (largest error / largest magnitude, median and largest element-wise relative error) of every check


def _check(out, ref, tol=1e-3):
    """"Within 1e-3 relative error" is read as: the largest absolute error is below 1e-3 of the tensor's largest
    magnitude (a float16 result is allowed one more half-ulp of its own rounding, 2^-11).  The element-wise reading
    |out - ref| / |ref| has no bound for elements that cancel to almost zero; it is recorded for every check and
    printed by test_zz_report_elementwise_error so that both readings are on record."""
    if out.dtype != torch.float32:
        tol = tol + 2.0 ** -11
    o = host(out.float())
    err = np.abs(o - ref).max() / np.abs(ref).max()
    big = np.abs(ref) > 0.05 * np.abs(ref).max()                 # elements that are not cancellation residue
    rel = np.abs(o - ref)[big] / np.abs(ref)[big]
    ELEMENTWISE.append((float(err), float(np.median(rel)), float(rel.max())))
    assert np.isfinite(o).all() and err < tol, err


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
    out2 = c.attend(torch.zeros(1, 4, 2, 128, device="cuda", dtype=torch.float16))     # several query tokens: the causal kernel
    assert out2.shape == (1, 4, 2, 128)


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


@pytest.mark.parametrize("v_scale", (1e5, 1e7, 1e-6))
@pytest.mark.parametrize("bf16", (False, True))
def test_value_norms_far_outside_the_fp16_range(oracle, v_scale, bf16):
    """Value norms of 1e5 and 1e7 (float32 and bfloat16 caches, un-normalised activations) and of 1e-6: the kernels carry
    the softmax weights times the value norm as fp16 operands under a power-of-two scale that follows the largest norm,
    so the result keeps the 1e-3 bound where the reference works in float32 throughout (cache.py:276-343; its own
    tests only ask for finite output, tests/test_edge_cases.py:131-151).  Direct kernel, general kernel, QJL sketch."""
    rs = np.random.RandomState(int(abs(np.log10(v_scale))) + (50 if bf16 else 0))
    for (d, kb, vb, qjl) in ((128, 4, 2, False), (128, 3, 2, False), (96, 4, 2, True)):
        c, q, ref = _case(oracle, rs, 1, 8, 2, 900, d, kb, vb, 32, 8, dtype=np.float32, qjl=qjl, v_scale=v_scale, bf16=bf16)
        assert np.abs(ref).max() > 1e-3 * v_scale
        _check(c.attend(q, out_dtype=torch.float32), ref)


def test_value_norms_growing_along_the_cache(oracle):
    """The value scale is picked from the first tile a warp sees and raised when a later norm needs it: norms that grow
    by twelve orders of magnitude along the sequence, and keys large enough for a one-hot softmax."""
    from mlx_turboquant_b200 import TurboQuantKVCache
    rs = np.random.RandomState(91)
    b, hq, hkv, t, d = 1, 8, 2, 1500, 128
    ramp = np.exp(np.linspace(np.log(1e-5), np.log(1e7), t)).astype(np.float32)[None, None, :, None]
    for k_scale in (1.0, 300.0):
        k = kv_like(rs, (b, hkv, t, d), np.float32) * k_scale
        v = kv_like(rs, (b, hkv, t, d), np.float32) * ramp
        q = (rs.randn(b, hq, 1, d) / np.sqrt(d)).astype(np.float32)
        ref_c = oracle.KVCacheOracle(d, host_tables(d), 4, 2, 32, fp16_sink_size=8)
        rk, rv = ref_c.update_and_fetch(k, v)
        c = TurboQuantKVCache(head_dim=d, num_kv_heads=hkv, residual_window=32, fp16_sink_size=8)
        ck, cv = ref_c.comp["k"], ref_c.comp["v"]
        c.state = (cu(ref_c.k), cu(ref_c.v), cu(ck[0]), cu(ck[2]), cu(cv[0]), cu(cv[2]), cu(ref_c.sink_k), cu(ref_c.sink_v), None, None)
        c.meta_state = {"offset": str(ref_c.offset), "compressed_len": str(ref_c.comp_len), "sink_len": str(ref_c.sink_len),
                        "fp16_len": str(ref_c.fp_len), "fp16_capacity": str(ref_c.k.shape[2])}
        _check(c.attend(cu(q), out_dtype=torch.float32), oracle.attention(q, rk, rv))


def test_zz_report_elementwise_error():
    """Not a bound: prints the element-wise relative error (elements above 5 % of the largest magnitude) of every
    comparison this module made, next to the max-norm figure the 1e-3 bound is applied to."""
    if not ELEMENTWISE:
        pytest.skip("no comparisons recorded")
    a = np.array(ELEMENTWISE)
    print(f"\ndecode parity over {len(a)} comparisons: max-norm error median {np.median(a[:, 0]):.2e} worst {a[:, 0].max():.2e}; "
          f"element-wise relative error median {np.median(a[:, 1]):.2e}, worst element {a[:, 2].max():.2e}")
    assert a[:, 0].max() < 1e-3 + 2.0 ** -11
