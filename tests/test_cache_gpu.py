"""TurboQuantKVCache on the GPU: the reference's state machine, replayed against its own vectors.

Dense outputs are compared at 1e-3 relative to the tensor's largest magnitude (the task's tolerance for
dequantized tensors); uncompressed regions must be bit-exact; packed bytes may differ from the
reference's only in the rare code whose rotated value sits on a boundary (see test_quantize_gpu.py).
"""

import numpy as np
import pytest
import torch

from gpu_util import cu, host, kv_like

pytestmark = pytest.mark.gpu


def _replay(name, golden, scenarios):
    from mlx_turboquant_b200 import TurboQuantKVCache
    sc = scenarios[name]
    c = TurboQuantKVCache(num_kv_heads=2, **sc["cfg"])
    k, v = cu(golden[name + "_k"]), cu(golden[name + "_v"])
    pos = 0
    for t in sc["steps"]:
        ok, ov = c.update_and_fetch(k[:, :, pos:pos + t], v[:, :, pos:pos + t])
        pos += t
    return c, ok, ov, sc


@pytest.mark.parametrize("name", ("c_k4v2", "c_chunk", "c_frac", "c_qjl", "c_w0"))
def test_update_and_fetch_matches_reference(golden, scenarios, name):
    c, ok, ov, sc = _replay(name, golden, scenarios)
    assert c.meta_state == sc["meta_state"]
    assert c.nbytes == sc["nbytes"]
    rk, rv = golden[name + "_out_k"], golden[name + "_out_v"]
    assert tuple(ok.shape) == rk.shape and str(ok.dtype).endswith(sc["out_dtype"])
    np.testing.assert_allclose(host(ok), rk, rtol=0, atol=1e-3 * np.abs(rk).max())
    np.testing.assert_allclose(host(ov), rv, rtol=0, atol=1e-3 * np.abs(rv).max())
    s, n = c._sink_len, c._fp16_len
    if s:
        assert np.array_equal(host(ok[:, :, :s]), rk[:, :, :s])            # sink is exact
    if n:
        assert np.array_equal(host(ok[:, :, -n:]), rk[:, :, -n:])          # recent tokens are exact
        assert np.array_equal(host(ov[:, :, -n:]), rv[:, :, -n:])
    if c._compressed_len:
        st = c.state
        for i in (2, 4, 8, 9):
            key = f"{name}_state{i}"
            if key in golden:
                assert tuple(st[i].shape) == golden[key].shape
                assert (host(st[i]) == golden[key]).mean() > 0.999
        np.testing.assert_allclose(host(st[3]), golden[name + "_state3"], rtol=2e-6)
        np.testing.assert_allclose(host(st[5]), golden[name + "_state5"], rtol=2e-6)


@pytest.mark.parametrize("name", ("c_k4v2", "c_chunk", "c_frac", "c_w0"))
def test_attend_matches_attention_over_reference_cache(golden, scenarios, name):
    """Packed decode over the REFERENCE's own packed state == float32 softmax attention over the reference's
    dense output, within 1e-3 (state injected so both sides see identical codes)."""
    from mlx_turboquant_b200 import TurboQuantKVCache
    sc = scenarios[name]
    ms = sc["meta_state"]
    s, n, m = int(ms["sink_len"]), int(ms["fp16_len"]), int(ms["compressed_len"])
    rk, rv = golden[name + "_out_k"], golden[name + "_out_v"]
    total = rk.shape[2]
    c = TurboQuantKVCache(num_kv_heads=2, **sc["cfg"])
    f16 = lambda a: cu(np.ascontiguousarray(a).astype(np.float16))   # noqa: E731 - sink / recent tokens were fp16 inputs
    g = lambda key: cu(golden[key]) if key in golden else None   # noqa: E731
    c.state = (f16(rk[:, :, total - n:]) if n else None, f16(rv[:, :, total - n:]) if n else None,
               g(name + "_state2"), g(name + "_state3"), g(name + "_state4"), g(name + "_state5"),
               f16(rk[:, :, :s]) if s else None, f16(rv[:, :, :s]) if s else None, g(name + "_state8"), g(name + "_state9"))
    c.meta_state = dict(ms, fp16_capacity=str(n))
    assert c._compressed_len == m
    q = cu(golden[name + "_q"])
    assert c.attend(q).dtype == q.dtype
    out = c.attend(q, out_dtype=torch.float32)
    ref = golden[name + "_attn"]
    assert tuple(out.shape) == ref.shape
    np.testing.assert_allclose(host(out), ref, rtol=0, atol=1e-3 * np.abs(ref).max())


def test_incremental_decode_and_lengths():
    """Reference tests/test_phase2.py:32-120."""
    from mlx_turboquant_b200 import TurboQuantKVCache
    rs = np.random.RandomState(0)
    c = TurboQuantKVCache(head_dim=128, num_kv_heads=4, residual_window=32)
    k = cu(rs.randn(1, 4, 200, 128).astype(np.float32))
    ok, ov = c.update_and_fetch(k[:, :, :10], k[:, :, :10])
    assert tuple(ok.shape) == (1, 4, 10, 128) and c.offset == 10 and ok.dtype == torch.float32
    for i in range(10, 100):
        ok, ov = c.update_and_fetch(k[:, :, i:i + 1], k[:, :, i:i + 1])
        assert ok.shape[2] == i + 1 and c.offset == i + 1
        assert c._fp16_len <= 2 * 32 and c._compressed_len + c._fp16_len == i + 1
    assert c._compressed_len > 0 and c._fp16_len >= 32
    n = c._fp16_len
    assert np.array_equal(host(ok[:, :, -n:]), host(k[:, :, 100 - n:100]))        # residual window is exact
    before = c.nbytes
    c.update_and_fetch(k[:, :, 100:101], k[:, :, 100:101])
    assert c.nbytes > before and not c.is_trimmable() and c.size() == 101 and not c.empty()
    dense = 2 * 4 * 101 * 128 * 4
    assert dense / c.nbytes > 1.0


def test_edge_cases_empty_short_and_window_zero():
    """Reference tests/test_edge_cases.py:195-287."""
    from mlx_turboquant_b200 import TurboQuantKVCache
    rs = np.random.RandomState(1)
    c = TurboQuantKVCache(head_dim=64, num_kv_heads=2, residual_window=16)
    z = torch.zeros(1, 2, 0, 64, device="cuda")
    ok, ov = c.update_and_fetch(z, z)
    assert tuple(ok.shape) == (1, 2, 0, 64) and c.offset == 0 and c.empty()
    x = cu(rs.randn(1, 2, 1, 64).astype(np.float32))
    ok, _ = c.update_and_fetch(x, x)
    assert tuple(ok.shape) == (1, 2, 1, 64) and np.array_equal(host(ok), host(x))
    c = TurboQuantKVCache(head_dim=64, num_kv_heads=2, residual_window=64)
    x = cu(rs.randn(1, 2, 20, 64).astype(np.float32))
    ok, _ = c.update_and_fetch(x, x)
    assert c._compressed_len == 0 and np.array_equal(host(ok), host(x))
    c = TurboQuantKVCache(head_dim=64, num_kv_heads=2, residual_window=0)        # compresses everything
    x = cu(rs.randn(1, 2, 10, 64).astype(np.float32))
    ok, _ = c.update_and_fetch(x, x)
    assert tuple(ok.shape) == (1, 2, 10, 64) and c._compressed_len == 10 and c._fp16_len == 0
    with pytest.raises(NotImplementedError):
        c.make_mask(4, window_size=128)
    for d in (64, 96, 128, 256):
        c = TurboQuantKVCache(head_dim=d, num_kv_heads=2, residual_window=8)
        x = cu(rs.randn(1, 2, 40, d).astype(np.float32))
        ok, ov = c.update_and_fetch(x, x)
        assert tuple(ok.shape) == (1, 2, 40, d) and torch.isfinite(ok).all()


def test_chunked_drains_and_sink_routing():
    """Reference tests/test_phase2.py:405-577."""
    from mlx_turboquant_b200 import TurboQuantKVCache
    rs = np.random.RandomState(2)
    x = cu(rs.randn(1, 2, 400, 128).astype(np.float32))
    c = TurboQuantKVCache(head_dim=128, num_kv_heads=2, residual_window=32, chunk_size=64)
    c.update_and_fetch(x[:, :, :95], x[:, :, :95])
    assert c._compressed_len == 0 and c._fp16_len == 95                   # below 32 + 64
    c.update_and_fetch(x[:, :, 95:96], x[:, :, 95:96])
    assert c._compressed_len == 64 and c._fp16_len == 32
    c = TurboQuantKVCache(head_dim=128, num_kv_heads=2, residual_window=32, chunk_size=64)
    c.update_and_fetch(x[:, :, :300], x[:, :, :300])                      # loops: 4 drains of 64
    assert c._compressed_len == 256 and c._fp16_len == 44
    c = TurboQuantKVCache(head_dim=128, num_kv_heads=2, residual_window=16, fp16_sink_size=8)
    ok, _ = c.update_and_fetch(x[:, :, :5], x[:, :, :5])                   # sink filled across calls
    assert c._sink_len == 5 and c._fp16_len == 0 and ok.shape[2] == 5
    ok, _ = c.update_and_fetch(x[:, :, 5:12], x[:, :, 5:12])               # straddles the sink boundary
    assert c._sink_len == 8 and c._fp16_len == 4 and ok.shape[2] == 12
    ok, _ = c.update_and_fetch(x[:, :, 12:200], x[:, :, 12:200])
    assert c._sink_len == 8 and c._compressed_len == 200 - 8 - 16 and c.offset == 200
    assert np.array_equal(host(ok[:, :, :8]), host(x[:, :, :8]))           # sink survives compression, at the head
    assert np.array_equal(host(ok[:, :, -16:]), host(x[:, :, 184:200]))


@pytest.mark.parametrize("kb,vb", ((4, 2), (3.5, 3.5), (3, 4)))
def test_state_roundtrip_and_reload(kb, vb):
    """Reference tests/test_phase2.py:169-325: 6/8/10-tuple states reload and keep decoding identically."""
    from mlx_turboquant_b200 import TurboQuantKVCache
    rs = np.random.RandomState(3)
    x = cu(kv_like(rs, (1, 2, 150, 128)))
    y = cu(kv_like(rs, (1, 2, 150, 128)))
    kw = dict(head_dim=128, num_kv_heads=2, key_bits=kb, value_bits=vb, residual_window=16, fp16_sink_size=4)
    a = TurboQuantKVCache(**kw)
    ak, av = a.update_and_fetch(x[:, :, :120], y[:, :, :120])
    st, meta = a.state, a.meta_state
    assert len(st) == 10 and all(isinstance(v, str) for v in meta.values())
    b = TurboQuantKVCache(**kw)
    b.state = tuple(None if t is None else t.clone() for t in st)
    b.meta_state = dict(meta)
    bk, bv = b.update_and_fetch(x[:, :, 120:121], y[:, :, 120:121])
    ak2, av2 = a.update_and_fetch(x[:, :, 120:121], y[:, :, 120:121])
    assert np.array_equal(host(ak2), host(bk)) and np.array_equal(host(av2), host(bv))
    q = cu((rs.randn(1, 4, 1, 128) / 11.3).astype(np.float16))
    assert np.array_equal(host(a.attend(q)), host(b.attend(q)))
    if kb == int(kb) and vb == int(vb):                                     # legacy tuples
        for n in (6, 8):
            kw2 = dict(kw, fp16_sink_size=0)
            s0 = TurboQuantKVCache(**kw2)
            s0.update_and_fetch(x[:, :, :120], y[:, :, :120])
            l = TurboQuantKVCache(**kw2)
            l.state = tuple(s0.state[:n])
            l.meta_state = s0.meta_state
            lk, _ = l.update_and_fetch(x[:, :, 120:121], y[:, :, 120:121])
            sk, _ = s0.update_and_fetch(x[:, :, 120:121], y[:, :, 120:121])
            assert np.array_equal(host(lk), host(sk))


def test_qjl_correction_reduces_error_and_leaves_fp16_regions_alone():
    """Reference tests/test_phase2.py:328-402."""
    from mlx_turboquant_b200 import TurboQuantKVCache
    rs = np.random.RandomState(4)
    x = cu(kv_like(rs, (1, 2, 200, 128), np.float32))
    outs = {}
    for on in (False, True):
        c = TurboQuantKVCache(head_dim=128, num_kv_heads=2, key_bits=3, value_bits=2, residual_window=16,
                              fp16_sink_size=8, qjl_correction=on)
        assert (c._qjl_projection is not None) == on
        outs[on], _ = c.update_and_fetch(x, x)
        if on:
            assert tuple(c._qjl_projection.shape) == (32, 128) and len(c.state) == 14
    mid = slice(8, 200 - 16)
    e_off = ((outs[False][:, :, mid] - x[:, :, mid]) ** 2).mean().item()
    e_on = ((outs[True][:, :, mid] - x[:, :, mid]) ** 2).mean().item()
    assert e_on < e_off
    assert torch.equal(outs[True][:, :, :8], x[:, :, :8]) and torch.equal(outs[True][:, :, -16:], x[:, :, -16:])


@pytest.mark.parametrize("kw", (dict(key_bits=4, value_bits=2, residual_window=8, fp16_sink_size=4),
                                dict(key_bits=3.5, value_bits=3, residual_window=8, chunk_size=16),
                                dict(key_bits=4, value_bits=2, residual_window=8, fp16_sink_size=4, qjl_correction=True)))
@pytest.mark.parametrize("dtype", (torch.float16, torch.float32))
def test_decode_step_equals_update_then_attend(kw, dtype):
    """`decode_step` (the token's append folded into the attention launch) against `update` + `attend` on a twin cache,
    token by token from an empty cache: through the sink, the first fills of the buffer, drains, and buffer growth.
    Same bits out, same state afterwards."""
    from mlx_turboquant_b200 import TurboQuantKVCache
    d, hkv, hq, b = 128, 2, 8, 2
    g = torch.Generator(device="cuda").manual_seed(5)
    a, c = TurboQuantKVCache(head_dim=d, num_kv_heads=hkv, **kw), TurboQuantKVCache(head_dim=d, num_kv_heads=hkv, **kw)
    pre = 300
    k0 = torch.randn(b, hkv, pre, d, device="cuda", generator=g).to(dtype)
    v0 = torch.randn(b, hkv, pre, d, device="cuda", generator=g).to(dtype)
    for cache in (a, c):
        cache.update(k0[:, :, :2], v0[:, :, :2])              # two tokens: still inside the sink
    fused = 0
    for i in range(2, 60):
        q = (torch.randn(b, hq, 1, d, device="cuda", generator=g) / d ** 0.5).to(dtype)
        k, v = k0[:, :, i:i + 1].contiguous(), v0[:, :, i:i + 1].contiguous()
        before = a._fp16_len
        out_a = a.decode_step(q, k, v)
        c.update(k, v)
        out_c = c.attend(q)
        fused += int(a._fp16_len == before + 1 and a._compressed_len == c._compressed_len)
        assert torch.equal(out_a, out_c), i
        assert (a.offset, a._fp16_len, a._compressed_len, a._sink_len) == (c.offset, c._fp16_len, c._compressed_len, c._sink_len)
    assert fused > 30                                          # most steps took the single launch
    for x, y in zip(a.state, c.state):
        assert (x is None) == (y is None)
        if x is not None:
            n = min(x.shape[2], y.shape[2])
            if x.dtype == torch.uint8 or x.shape[2] == y.shape[2]:
                assert torch.equal(x[:, :, :n], y[:, :, :n])
    assert torch.equal(a.keys[:, :, :a._fp16_len], c.keys[:, :, :c._fp16_len])
