"""Dequantize (unpack -> centroid -> inverse rotation -> scale) against the oracle, under both kernels: the tensor-core
kernel (head_dim 64 / 96 / 128, no QJL correction) and the CUDA-core row kernel.  Bound: 2e-6 of the largest magnitude for
float32 results (the tensor-core kernel keeps three fp16 partial products in fp32 accumulators, the row kernel is plain
float32), plus the result type's own rounding for float16 / bfloat16."""

import numpy as np
import pytest
import torch

from gpu_util import cu, host

pytestmark = pytest.mark.gpu


@pytest.fixture(params=["tcgen05", "row kernel"], autouse=True)
def which_kernel(request):
    from mlx_turboquant_b200 import _lib, kernels
    kernels.set_tuning("dequantize_tc", 1 if request.param == "tcgen05" else 0)
    yield request.param
    kernels.set_tuning("dequantize_tc", 1)
    assert _lib.lib().tq_device_status() == 0


def _random_packed(rs, lead, t, d, bits):
    """Random codes in the reference's packed layout (through the oracle's packer) and positive norms."""
    from oracle import tq_oracle as oracle
    idx = rs.randint(0, 1 << bits, size=(*lead, t, d)).astype(np.uint8)
    packed = oracle.pack(idx, bits)
    norms = np.exp(rs.randn(*lead, t)).astype(np.float32)
    return packed, norms


@pytest.mark.parametrize("d", (64, 96, 128))
@pytest.mark.parametrize("bits", (1, 2, 3, 4))
def test_every_width_and_head_dim(oracle, tables, d, bits):
    from mlx_turboquant_b200 import kernels
    from mlx_turboquant_b200.codebook import get_codebook
    from mlx_turboquant_b200.rotation import get_rotation_matrix
    rs = np.random.RandomState(d * 10 + bits)
    packed, norms = _random_packed(rs, (3, 2), 211, d, bits)          # 1266 rows: tiles that straddle lanes, a ragged last tile
    c, _ = get_codebook(d, bits)
    got = host(kernels.dequantize_rows(cu(packed), None, cu(norms), get_rotation_matrix(d), c, bits, None, 0, d))
    ref = oracle.mse_dequantize(packed, norms, oracle.rotation_matrix(d), tables[(d, bits)][0], bits, d)
    np.testing.assert_allclose(got, ref, rtol=0, atol=2e-6 * np.abs(ref).max())


@pytest.mark.parametrize("d,hi,lo", ((128, 4, 3), (128, 3, 2), (96, 4, 3), (64, 2, 1)))
def test_fractional_widths(oracle, tables, d, hi, lo):
    from mlx_turboquant_b200 import kernels
    from mlx_turboquant_b200.codebook import get_codebook
    from mlx_turboquant_b200.rotation import get_rotation_matrix
    rs = np.random.RandomState(d + hi)
    from oracle import tq_oracle as orc
    t = 300
    ih = rs.randint(0, 1 << hi, size=(2, t, d // 2)).astype(np.uint8)
    il = rs.randint(0, 1 << lo, size=(2, t, d // 2)).astype(np.uint8)
    ph, pl = orc.pack(ih, hi), orc.pack(il, lo)
    norms = np.exp(rs.randn(2, t)).astype(np.float32)
    (ch, _), (cl, _) = get_codebook(d, hi), get_codebook(d, lo)
    got = host(kernels.dequantize_rows(cu(ph), cu(pl), cu(norms), get_rotation_matrix(d), ch, hi, cl, lo, d))
    ref = oracle.split_dequantize(ph, pl, norms, oracle.rotation_matrix(d), tables[(d, hi)][0], hi, tables[(d, lo)][0], lo, d)
    np.testing.assert_allclose(got, ref, rtol=0, atol=2e-6 * np.abs(ref).max())


@pytest.mark.parametrize("out_dtype,tol", ((torch.float16, 2.0 ** -11), (torch.bfloat16, 2.0 ** -8), (torch.float32, 0.0)))
def test_result_types_offsets_and_strides(oracle, tables, out_dtype, tol):
    """Rows [in_offset, in_offset + n) of every lane into rows [out_offset, ...) of a larger result buffer."""
    from mlx_turboquant_b200 import kernels
    from mlx_turboquant_b200.codebook import get_codebook
    from mlx_turboquant_b200.rotation import get_rotation_matrix
    d, bits = 128, 4
    rs = np.random.RandomState(5)
    packed, norms = _random_packed(rs, (2, 4), 400, d, bits)
    c, _ = get_codebook(d, bits)
    out = torch.full((2, 4, 700, d), 7.0, dtype=out_dtype, device="cuda")
    kernels.dequantize_rows(cu(packed), None, cu(norms), get_rotation_matrix(d), c, bits, None, 0, d, n_rows=333, in_offset=50, out=out,
                            out_offset=120)
    ref = oracle.mse_dequantize(packed[:, :, 50:383], norms[:, :, 50:383], oracle.rotation_matrix(d), tables[(d, bits)][0], bits, d)
    got = host(out.float())
    assert np.all(got[:, :, :120] == 7.0) and np.all(got[:, :, 453:] == 7.0)          # nothing outside the rows asked for
    np.testing.assert_allclose(got[:, :, 120:453], ref, rtol=tol, atol=(2e-6 + tol) * np.abs(ref).max())


def test_both_kernels_agree_on_a_large_batch(oracle, tables):
    """4-bit keys of a (1, 8, 8192) cache: 512 tiles over the persistent CTAs; the two kernels agree to float32 rounding."""
    from mlx_turboquant_b200 import kernels
    from mlx_turboquant_b200.codebook import get_codebook
    from mlx_turboquant_b200.rotation import get_rotation_matrix
    d, bits = 128, 4
    rs = np.random.RandomState(6)
    packed, norms = _random_packed(rs, (1, 8), 8192, d, bits)
    c, _ = get_codebook(d, bits)
    res = []
    for tc in (1, 0):
        kernels.set_tuning("dequantize_tc", tc)
        res.append(kernels.dequantize_rows(cu(packed), None, cu(norms), get_rotation_matrix(d), c, bits, None, 0, d))
    a, b = res
    assert float((a - b).abs().max()) <= 2e-6 * float(b.abs().max())
    assert torch.isfinite(a).all()
