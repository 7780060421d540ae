"""The benchmark configurations at their full sizes.

Where the CPU oracle would take minutes, the checks are size-independent properties of the path: agreement of two
independent kernels, invariance to how the work is partitioned (splits, chunks, batch), invariance of attention to
the order of the cached tokens, and the reconstruction-quality figures the reference's own tests pin.
"""

import numpy as np
import pytest
import torch

from gpu_util import cu, host, host_tables, kv_like

pytestmark = pytest.mark.gpu


def _cos_mse(x, y):
    x, y = x.reshape(-1, x.shape[-1]).astype(np.float64), y.reshape(-1, y.shape[-1]).astype(np.float64)
    cos = (x * y).sum(-1) / (np.linalg.norm(x, axis=-1) * np.linalg.norm(y, axis=-1))
    rel = ((x - y) ** 2).sum(-1) / (x ** 2).sum(-1)
    return float(cos.mean()), float(rel.mean())


def test_round_trip_quality_config0(oracle):
    """K4 / V2 quantize -> pack -> unpack -> dequantize of (1, 8, 4096, 128) fp16 with the benchmark's distribution:
    per-vector cosine / relative MSE at the values the codebooks give (4-bit 0.995 / 0.0093, 2-bit 0.941 / 0.116),
    and parity with the oracle on the same bytes."""
    from mlx_turboquant_b200 import kernels
    from mlx_turboquant_b200.codebook import get_codebook
    from mlx_turboquant_b200.rotation import get_rotation_matrix
    d = 128
    rs = np.random.RandomState(0)
    rot, orot = get_rotation_matrix(d), oracle.rotation_matrix(d)
    for bits, cos_lo, mse_hi in ((4, 0.994, 0.0105), (2, 0.935, 0.125)):
        xh = kv_like(rs, (1, 8, 4096, d))
        x = cu(xh)
        cent, bnd = get_codebook(d, bits)
        p, _, n = kernels.quantize_pack(x, rot, bnd, bits)
        assert tuple(p.shape) == (1, 8, 4096, d * bits // 8) and p.dtype == torch.uint8
        y = kernels.dequantize_rows(p, None, n, rot, cent, bits, None, 0, d)
        cos, mse = _cos_mse(xh.astype(np.float32), host(y.float()))
        assert cos > cos_lo and mse < mse_hi, (bits, cos, mse)
        tab = host_tables(d)
        rp, rn, _ = oracle.mse_quantize(xh, orot, tab[bits][1], bits)
        assert (host(p) != rp).mean() < 1e-4
        np.testing.assert_allclose(host(n), rn, rtol=2e-6)
        ry = oracle.mse_dequantize(host(p), host(n), orot, tab[bits][0], bits, d)      # same codes -> same tensor
        assert np.abs(host(y.float()) - ry).max() <= 1e-3 * np.abs(ry).max()


def _c1_cache(seed, hkv=8, ctx=32768, perm=None):
    from mlx_turboquant_b200 import TurboQuantKVCache
    g = torch.Generator(device="cuda").manual_seed(seed)
    k = (torch.randn(1, hkv, ctx, 128, device="cuda", generator=g) * torch.exp(0.5 * torch.randn(1, hkv, ctx, 1, device="cuda", generator=g))).half()
    v = (torch.randn(1, hkv, ctx, 128, device="cuda", generator=g) * torch.exp(0.5 * torch.randn(1, hkv, ctx, 1, device="cuda", generator=g))).half()
    if perm is not None:                                   # reorder the tokens that end up packed (same order for K and V)
        k[:, :, 128:ctx - 128] = k[:, :, 128:ctx - 128][:, :, perm]
        v[:, :, 128:ctx - 128] = v[:, :, 128:ctx - 128][:, :, perm]
    c = TurboQuantKVCache(head_dim=128, num_kv_heads=hkv, key_bits=4, value_bits=2, residual_window=128, fp16_sink_size=128)
    c.update(k, v)
    assert (c._sink_len, c._compressed_len, c._fp16_len) == (128, ctx - 256, 128)
    q = (torch.randn(1, 4 * hkv, 1, 128, device="cuda", generator=g) / 128 ** 0.5).half()
    return c, q, k, v


def test_decode_config1_full_size_properties():
    """32 query / 8 KV heads, 32768 tokens = 128 + 32512 packed + 128: the table-lookup kernel and the general kernel
    agree; the result does not depend on the split count nor on the order of the packed tokens."""
    from mlx_turboquant_b200 import _lib
    from mlx_turboquant_b200.kernels import set_tuning
    c, q, _, _ = _c1_cache(5)
    a = c.attend(q, out_dtype=torch.float32)
    assert _lib.lib().tq_device_status() == 0 and torch.isfinite(a).all()
    scale = float(a.abs().max())
    set_tuning("decode_force_general", 1)
    try:
        b = c.attend(q, out_dtype=torch.float32)
    finally:
        set_tuning("decode_force_general", 0)
    assert float((a - b).abs().max()) <= 2e-3 * scale
    for splits in (3, 40):
        set_tuning("decode_splits", splits)
        try:
            assert float((c.attend(q, out_dtype=torch.float32) - a).abs().max()) <= 1e-3 * scale
        finally:
            set_tuning("decode_splits", 0)
    perm = torch.randperm(32768 - 256, device="cuda", generator=torch.Generator(device="cuda").manual_seed(1))
    c2, q2, _, _ = _c1_cache(5, perm=perm)
    assert torch.equal(q, q2)
    assert float((c2.attend(q2, out_dtype=torch.float32) - a).abs().max()) <= 1e-3 * scale


def test_decode_config1_against_oracle_two_kv_heads(oracle):
    """Full 32768-token context against the CPU oracle (two KV heads keep the oracle within seconds), identical packed state."""
    from mlx_turboquant_b200 import TurboQuantKVCache
    rs = np.random.RandomState(21)
    hkv, ctx, d = 2, 32768, 128
    k, v = kv_like(rs, (1, hkv, ctx, d)), kv_like(rs, (1, hkv, ctx, d))
    q = (rs.randn(1, 4 * hkv, 1, d) / np.sqrt(d)).astype(np.float16)
    ref_c = oracle.KVCacheOracle(d, host_tables(d), 4, 2, 128, fp16_sink_size=128)
    try:
        from oracle import c_oracle
        c_oracle.use_c_kernels(ref_c, c_oracle.load())
    except Exception:
        pass
    rk, rv = ref_c.update_and_fetch(k, v)
    ref = oracle.attention(q, rk, rv)
    c = TurboQuantKVCache(head_dim=d, num_kv_heads=hkv, key_bits=4, value_bits=2, residual_window=128, fp16_sink_size=128)
    ck, cv = ref_c.comp["k"], ref_c.comp["v"]
    c.state = (cu(ref_c.k), cu(ref_c.v), cu(ck[0]), cu(ck[2]), cu(cv[0]), cu(cv[2]), cu(ref_c.sink_k), cu(ref_c.sink_v), None, None)
    c.meta_state = {"offset": str(ref_c.offset), "compressed_len": str(ref_c.comp_len), "sink_len": str(ref_c.sink_len),
                    "fp16_len": str(ref_c.fp_len), "fp16_capacity": str(ref_c.k.shape[2])}
    out = host(c.attend(cu(q), out_dtype=torch.float32))
    assert np.abs(out - ref).max() <= 1e-3 * np.abs(ref).max()


def test_decode_config3_against_oracle_two_heads(oracle):
    """Phi-3.5-mini shape at its full 8192-token context (128 sink + 7936 packed + 128 recent), d = 96, 4-bit keys /
    2-bit values with the QJL sketch, one sequence x two heads (MHA) so that the CPU oracle stays within seconds:
    identical packed state and sketches, attention against the reference's corrected dense K / V."""
    from mlx_turboquant_b200 import TurboQuantKVCache
    rs = np.random.RandomState(23)
    h, ctx, d = 2, 8192, 96
    k, v = kv_like(rs, (1, h, ctx, d)), kv_like(rs, (1, h, ctx, d))
    q = (rs.randn(1, h, 1, d) / np.sqrt(d)).astype(np.float16)
    ref_c = oracle.KVCacheOracle(d, host_tables(d), 4, 2, 128, fp16_sink_size=128, qjl_correction=True)
    rk, rv = ref_c.update_and_fetch(k, v)
    assert (ref_c.sink_len, ref_c.comp_len, ref_c.fp_len) == (128, ctx - 256, 128)
    ref = oracle.attention(q, rk, rv)
    c = TurboQuantKVCache(head_dim=d, num_kv_heads=h, key_bits=4, value_bits=2, residual_window=128, fp16_sink_size=128,
                          qjl_correction=True)
    ck, cv = ref_c.comp["k"], ref_c.comp["v"]
    sk, sv = ref_c.sketch["k"], ref_c.sketch["v"]
    i32 = lambda a: cu(a.view(np.int32))   # noqa: E731
    c.state = (cu(ref_c.k), cu(ref_c.v), cu(ck[0]), cu(ck[2]), cu(cv[0]), cu(cv[2]), cu(ref_c.sink_k), cu(ref_c.sink_v), None, None,
               i32(sk[0]), cu(sk[1]), i32(sv[0]), cu(sv[1]))
    c.meta_state = {"offset": str(ref_c.offset), "compressed_len": str(ref_c.comp_len), "sink_len": str(ref_c.sink_len),
                    "fp16_len": str(ref_c.fp_len), "fp16_capacity": str(ref_c.k.shape[2])}
    out = host(c.attend(cu(q), out_dtype=torch.float32))
    assert np.abs(out - ref).max() <= 1e-3 * np.abs(ref).max()


@pytest.mark.parametrize("kb", (3, 2, 3.5))
def test_compression_config2_chunking_invariance(kb):
    """126,976 tokens x 8 heads drained as 31 chunks of 4096 in ONE launch give byte-identical codes and norms to 31
    separate chunk launches, and to the CUDA-core kernel except on boundary ties."""
    from mlx_turboquant_b200 import kernels
    from mlx_turboquant_b200.codebook import get_codebook
    from mlx_turboquant_b200.rotation import get_rotation_matrix
    d, n_tok, chunk = 128, 126976, 4096
    g = torch.Generator(device="cuda").manual_seed(int(kb * 10))
    x = torch.randn(1, 8, n_tok, d, device="cuda", generator=g, dtype=torch.float16)
    x[..., [3, 40, 77, 101]] *= 20.0
    hi, lo = kernels.split_bits(kb)
    rot = get_rotation_matrix(d)
    bh = get_codebook(d, hi)[1]
    bl = get_codebook(d, lo)[1] if lo else None
    ph, pl, n = kernels.quantize_pack(x, rot, bh, hi, bl, lo)
    for c0 in (0, 5 * chunk, 30 * chunk):
        qh, ql, qn = kernels.quantize_pack(x[:, :, c0:c0 + chunk], rot, bh, hi, bl, lo)
        assert torch.equal(qh, ph[:, :, c0:c0 + chunk]) and torch.equal(qn, n[:, :, c0:c0 + chunk])
        if lo:
            assert torch.equal(ql, pl[:, :, c0:c0 + chunk])
    sl = slice(7 * chunk, 8 * chunk)
    gh, gl, gn = kernels.quantize_pack(x[:, :, sl].float(), rot, bh, hi, bl, lo)       # float32 input: the CUDA-core kernel
    assert (gh != ph[:, :, sl]).float().mean() < 1e-4
    torch.testing.assert_close(gn, n[:, :, sl], rtol=2e-6, atol=0)


def test_decode_config3_batch_independence():
    """Phi-3.5-shaped QJL decode (32 heads, d = 96, 8192 tokens): a sequence's output does not depend on what else is
    in the batch (its slice of the packed state attended alone gives the same numbers)."""
    from mlx_turboquant_b200 import TurboQuantKVCache
    b, h, d, ctx = 4, 32, 96, 8192
    g = torch.Generator(device="cuda").manual_seed(33)
    k = (torch.randn(b, h, ctx, d, device="cuda", generator=g) * torch.exp(0.5 * torch.randn(b, h, ctx, 1, device="cuda", generator=g))).half()
    v = (torch.randn(b, h, ctx, d, device="cuda", generator=g) * torch.exp(0.5 * torch.randn(b, h, ctx, 1, device="cuda", generator=g))).half()
    q = (torch.randn(b, h, 1, d, device="cuda", generator=g) / d ** 0.5).half()
    mk = lambda: TurboQuantKVCache(head_dim=d, num_kv_heads=h, key_bits=4, value_bits=2, residual_window=128, fp16_sink_size=128,   # noqa: E731
                                   qjl_correction=True)
    c = mk()
    c.update(k, v)
    full = c.attend(q, out_dtype=torch.float32)
    assert torch.isfinite(full).all()
    one = mk()
    st = tuple(None if t is None else t[2:3].contiguous() for t in c.state)
    one.state = st
    one.meta_state = c.meta_state
    alone = one.attend(q[2:3], out_dtype=torch.float32)
    # a batch of one gets a different split plan: same numbers up to the order of the fp32 / fp16 roundings
    assert float((alone - full[2:3]).abs().max()) <= 1e-3 * float(full.abs().max())
