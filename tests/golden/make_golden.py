"""Regenerate the golden fixtures in this directory from the UNMODIFIED reference.

Run from the repository root, in a container that has the reference checked out:

    python tests/golden/make_golden.py /path/to/mlx-turboquant

The reference's pure-MLX modules are imported as they are and executed on the
NumPy stand-in for ``mlx.core`` that lives in ``_mlx_standin/`` (MLX itself is
Apple-only wheels and is not installable here).  Every array written below is an
output of the reference's own functions on seeded inputs, so the fixtures pin the
CPU oracle (``oracle/tq_oracle.py``) and, through it, the CUDA path.

Also writes ``shipped_codebooks.json`` (the sixteen codebooks the reference ships,
float32 bit patterns as hex) next to the fixtures and into the package's
``codebooks/`` folder.
"""

import json
import sys
import warnings
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
REPO = HERE.parent.parent


def main(ref_root: str) -> None:
    sys.path.insert(0, str(HERE / "_mlx_standin"))
    sys.path.insert(0, ref_root)
    warnings.simplefilter("ignore")
    import mlx.core as mx
    from mlx_turboquant import cache as rcache
    from mlx_turboquant import codebook, packing, qjl, quantizer, rotation

    A = np.asarray
    out = {}

    # ---- shipped codebooks (known answers of lloyd_max) ---------------------------------
    table = {}
    for d in (64, 96, 128, 256):
        for b in (1, 2, 3, 4):
            z = np.load(codebook.CODEBOOK_DIR / f"codebook_d{d}_b{b}.npz")
            table[f"d{d}_b{b}"] = {
                "centroids": [f"{v:08x}" for v in z["centroids"].astype(np.float32).view(np.uint32)],
                "boundaries": [f"{v:08x}" for v in z["boundaries"].astype(np.float32).view(np.uint32)],
            }
    text = json.dumps(table, indent=0, sort_keys=True)
    (HERE / "shipped_codebooks.json").write_text(text)
    (REPO / "mlx_turboquant_b200" / "codebooks" / "shipped_codebooks.json").write_text(text)

    # ---- rotation / projection ------------------------------------------------------------
    for d in (64, 96, 128, 256):
        out[f"rot_d{d}_head"] = A(rotation.get_rotation_matrix(d, 42))[:4, :16].copy()
        out[f"rot_d{d}_sum"] = np.array([np.abs(A(rotation.get_rotation_matrix(d, 42))).astype(np.float64).sum()])
    out["rot_d64_full"] = A(rotation.get_rotation_matrix(64, 42)).copy()
    out["rot_d64_seed7"] = A(rotation.get_rotation_matrix(64, 7)).copy()
    out["proj_m32_d96"] = A(qjl.get_projection_matrix(96, 32)).copy()

    # ---- packing --------------------------------------------------------------------------
    rs = np.random.RandomState(101)
    for bits in (1, 2, 3, 4):
        idx = rs.randint(0, 1 << bits, size=(3, 5, 128)).astype(np.uint8)
        out[f"pack_idx_b{bits}"] = idx
        p = packing.pack_indices(mx.array(idx), bits)
        out[f"pack_out_b{bits}"] = A(p).copy()
        assert np.array_equal(A(packing.unpack_indices(p, bits, 128)), idx)

    # ---- scalar quantizer incl. tie side and clipping -----------------------------------
    for d, bits in ((128, 4), (128, 3), (96, 2), (64, 1)):
        c, bnd = codebook.get_codebook(d, bits)
        bn = A(bnd)
        y = np.concatenate([
            rs.randn(512).astype(np.float32) / np.sqrt(d),
            bn, np.nextafter(bn, np.float32(1)), np.nextafter(bn, np.float32(-1)),
            bn + np.float32(1e-7), np.array([0.0, -0.0, 100.0, -100.0, 1e-30], dtype=np.float32),
        ]).astype(np.float32)
        out[f"qs_y_d{d}_b{bits}"] = y
        out[f"qs_idx_d{d}_b{bits}"] = A(codebook.quantize_scalar(mx.array(y), c, bnd)).copy()

    # ---- TurboQuantMSE --------------------------------------------------------------------
    for d in (64, 96, 128, 256):
        for bits in (2, 3, 4):
            x = (rs.randn(48, d) * np.exp(0.5 * rs.randn(48, 1))).astype(np.float16)
            x[5] = 0  # zero-vector guard
            q = quantizer.TurboQuantMSE(d, bits)
            qt = q.quantize(mx.array(x))
            xf = x.astype(np.float32)
            nrm = np.sqrt(np.sum(xf * xf, axis=-1, dtype=np.float32))
            y = (xf / np.maximum(nrm, np.float32(1e-10))[:, None]) @ A(q.rotation).T
            tag = f"mse_d{d}_b{bits}"
            out[tag + "_x"] = x
            out[tag + "_y"] = y.astype(np.float32)
            out[tag + "_packed"] = A(qt.packed_indices).copy()
            out[tag + "_norms"] = A(qt.norms).copy()
            out[tag + "_deq"] = A(q.dequantize(qt)).copy()

    # ---- TurboQuantProd / QJL -------------------------------------------------------------
    x = rs.randn(16, 128).astype(np.float32)
    pq = quantizer.TurboQuantProd(128, bits=3)
    qt = pq.quantize(mx.array(x))
    out["prod_x"] = x
    out["prod_packed"] = A(qt.packed_indices).copy()
    out["prod_norms"] = A(qt.norms).copy()
    out["prod_signs"] = A(qt.qjl_signs).copy()
    out["prod_gamma"] = A(qt.qjl_norms).copy()
    out["prod_deq"] = A(pq.dequantize(qt)).copy()
    r = (rs.randn(24, 96) * 0.05).astype(np.float32)
    S = qjl.get_projection_matrix(96, 32)
    s, g = qjl.qjl_quantize(mx.array(r), S)
    out["qjl_r"] = r
    out["qjl_signs"] = A(s).copy()
    out["qjl_gamma"] = A(g).copy()
    out["qjl_deq"] = A(qjl.qjl_dequantize(s, g, S, 96)).copy().astype(np.float32)

    # ---- fused QK scores: the reference's own parity statement, Q @ dequant(K).T ----------
    for d, bits, tq, tkv in ((128, 4, 4, 130), (96, 3, 1, 64), (256, 2, 2, 40)):
        qv = rs.randn(tq, d).astype(np.float32)
        kv = (rs.randn(tkv, d) * 2.0).astype(np.float32)
        q = quantizer.TurboQuantMSE(d, bits)
        qt = q.quantize(mx.array(kv))
        tag = f"qk_d{d}_b{bits}"
        out[tag + "_q"] = qv
        out[tag + "_packed"] = A(qt.packed_indices).copy()
        out[tag + "_norms"] = A(qt.norms).copy()
        out[tag + "_scores"] = (qv @ A(q.dequantize(qt)).T).astype(np.float32)

    # ---- cache scenarios --------------------------------------------------------------------
    scen = {
        "c_k4v2": dict(head_dim=128, key_bits=4, value_bits=2, residual_window=16, fp16_sink_size=4,
                       chunk_size=0, qjl_correction=False, steps=[60, 1, 1, 40, 1]),
        "c_chunk": dict(head_dim=128, key_bits=3, value_bits=2, residual_window=8, fp16_sink_size=0,
                        chunk_size=16, qjl_correction=False, steps=[70, 1, 9]),
        "c_frac": dict(head_dim=128, key_bits=3.5, value_bits=3.5, residual_window=8, fp16_sink_size=2,
                       chunk_size=0, qjl_correction=False, steps=[1, 40, 1, 30]),
        "c_qjl": dict(head_dim=96, key_bits=4, value_bits=2, residual_window=8, fp16_sink_size=8,
                      chunk_size=0, qjl_correction=True, steps=[50, 1, 1]),
        "c_w0": dict(head_dim=64, key_bits=4, value_bits=4, residual_window=0, fp16_sink_size=0,
                     chunk_size=0, qjl_correction=False, steps=[5, 0, 3]),
    }
    meta = {}
    for name, cfg in scen.items():
        steps = cfg.pop("steps")
        d = cfg["head_dim"]
        c = rcache.TurboQuantKVCache(num_kv_heads=2, **cfg)
        total = sum(steps)
        k_all = (rs.randn(1, 2, total, d) * np.exp(0.5 * rs.randn(1, 2, total, 1))).astype(np.float16)
        v_all = (rs.randn(1, 2, total, d) * np.exp(0.5 * rs.randn(1, 2, total, 1))).astype(np.float16)
        pos = 0
        for t in steps:
            ok, ov = c.update_and_fetch(mx.array(k_all[:, :, pos:pos + t]), mx.array(v_all[:, :, pos:pos + t]))
            pos += t
        out[name + "_k"] = k_all
        out[name + "_v"] = v_all
        out[name + "_out_k"] = A(ok).copy()
        out[name + "_out_v"] = A(ov).copy()
        st = c.state
        for i, s in enumerate(st):
            if s is not None and i >= 2:
                out[f"{name}_state{i}"] = A(s).copy()
        qv = (rs.randn(1, 4, 1, d) / np.sqrt(d)).astype(np.float16)
        out[name + "_q"] = qv
        # attention over the reference's dense output (plain float32 softmax, GQA repeat 2)
        kk, vv, qq = A(ok).astype(np.float32), A(ov).astype(np.float32), qv.astype(np.float32)
        att = np.empty((1, 4, 1, d), dtype=np.float32)
        for h in range(4):
            sc = (qq[0, h] @ kk[0, h // 2].T) * np.float32(d ** -0.5)
            sc = sc - sc.max(axis=-1, keepdims=True)
            p = np.exp(sc)
            att[0, h] = (p @ vv[0, h // 2]) / p.sum(axis=-1, keepdims=True)
        out[name + "_attn"] = att
        meta[name] = dict(cfg=cfg, steps=steps, meta_state=c.meta_state, nbytes=int(c.nbytes),
                          out_dtype=str(A(ok).dtype))
    (HERE / "cache_scenarios.json").write_text(json.dumps(meta, indent=1, sort_keys=True))
    np.savez_compressed(HERE / "reference_vectors.npz", **out)
    print("wrote", len(out), "arrays,", (HERE / "reference_vectors.npz").stat().st_size, "bytes")


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit("usage: make_golden.py <path to a checkout of alex-rentel/mlx-turboquant>")
    main(sys.argv[1])
