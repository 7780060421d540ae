"""Helpers shared by the GPU parity tests."""

import numpy as np
import torch

DEV = "cuda"


def cu(a):
    return torch.from_numpy(np.ascontiguousarray(a)).to(DEV)


def host(t):
    return t.detach().cpu().numpy()


def host_tables(d):
    from mlx_turboquant_b200.codebook import get_codebook_host
    return {b: get_codebook_host(d, b) for b in (1, 2, 3, 4)}


def kv_like(rs, shape, dtype=np.float16):
    """N(0,1) entries times a per-token LogNormal(0, 0.5) scale (the benchmark's K/V distribution)."""
    x = rs.randn(*shape) * np.exp(0.5 * rs.randn(*shape[:-1], 1))
    return x.astype(dtype)


def code_mismatch_report(got_packed, ref_packed, bits, d, y_ref, boundaries):
    """Unpack both, return (fraction of differing codes, max |code diff|, max distance of the
    reference's rotated value to the nearest boundary among differing codes)."""
    from oracle import tq_oracle as orc
    g = orc.unpack(got_packed, bits, d).astype(np.int32)
    r = orc.unpack(ref_packed, bits, d).astype(np.int32)
    diff = g != r
    if not diff.any():
        return 0.0, 0, 0.0
    yb = np.abs(np.asarray(y_ref)[diff][:, None] - np.asarray(boundaries)[None, :]).min(axis=1)
    return float(diff.mean()), int(np.abs(g - r)[diff].max()), float(yb.max())
