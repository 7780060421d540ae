"""The C restatement of the reference's Metal kernel bodies agrees with the reference's Python path.

The reference itself checks its kernels against its Python path at cosine / 1e-3 level
(tests/test_phase2.py:641-672, tests/test_fused_attention.py:150-177); the C loops sum in a different
order than BLAS, so codes may differ where a rotated value sits on a boundary.
"""

import numpy as np
import pytest


@pytest.fixture(scope="module")
def clib():
    from oracle import c_oracle
    return c_oracle.load(), c_oracle


@pytest.mark.parametrize("d", (64, 96, 128, 256))
@pytest.mark.parametrize("bits", (2, 3, 4))
def test_quantize_and_dequantize_rows(clib, oracle, golden, tables, d, bits):
    lib, co = clib
    tag = f"mse_d{d}_b{bits}"
    rot = oracle.rotation_matrix(d)
    packed, norms, y = co.quantize_rows(lib, golden[tag + "_x"].astype(np.float32), rot, tables[(d, bits)][1], bits, want_y=True)
    np.testing.assert_allclose(norms, golden[tag + "_norms"], rtol=2e-6)
    np.testing.assert_allclose(y, golden[tag + "_y"], atol=3e-7)
    a, b = oracle.unpack(packed, bits, d).astype(int), oracle.unpack(golden[tag + "_packed"], bits, d).astype(int)
    assert (a != b).mean() < 1e-3 and np.abs(a - b).max() <= 1
    deq = co.dequantize_rows(lib, golden[tag + "_packed"], golden[tag + "_norms"], rot, tables[(d, bits)][0], bits, d)
    np.testing.assert_allclose(deq, golden[tag + "_deq"], atol=2e-6 * np.abs(golden[tag + "_deq"]).max())


@pytest.mark.parametrize("d,bits", ((128, 4), (96, 3), (256, 2)))
def test_fused_qk_body(clib, oracle, golden, tables, d, bits):
    lib, co = clib
    tag = f"qk_d{d}_b{bits}"
    qrot = oracle.rotate_fwd(golden[tag + "_q"], oracle.rotation_matrix(d))
    s = co.qk_scores(lib, qrot, golden[tag + "_packed"], golden[tag + "_norms"], tables[(d, bits)][0], bits, d)
    np.testing.assert_allclose(s, golden[tag + "_scores"], atol=1e-3, rtol=1e-3)


def test_attention_and_cache_hook(clib, oracle, golden, scenarios, tables):
    lib, co = clib
    name = "c_k4v2"
    att = co.attention(lib, golden[name + "_q"], golden[name + "_out_k"], golden[name + "_out_v"])
    np.testing.assert_allclose(att, golden[name + "_attn"], rtol=1e-5, atol=1e-6)
    sc = scenarios[name]
    cfg = dict(sc["cfg"])
    d = cfg.pop("head_dim")
    c = co.use_c_kernels(oracle.KVCacheOracle(d, {b: tables[(d, b)] for b in (1, 2, 3, 4)}, **cfg), lib)
    pos = 0
    for t in sc["steps"]:
        ok, ov = c.update_and_fetch(golden[name + "_k"][:, :, pos:pos + t], golden[name + "_v"][:, :, pos:pos + t])
        pos += t
    np.testing.assert_allclose(ok, golden[name + "_out_k"], atol=1e-3 * np.abs(golden[name + "_out_k"]).max())
    assert lib.tqo_threads() >= 1
