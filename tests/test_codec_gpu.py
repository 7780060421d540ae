"""pack / unpack / scalar quantizer on the GPU: bit-exact against the oracle and the reference's vectors."""

import numpy as np
import pytest
import torch

from gpu_util import cu, host

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("bits", (1, 2, 3, 4))
def test_pack_unpack_match_reference_vectors(golden, bits):
    from mlx_turboquant_b200.packing import pack_indices, unpack_indices
    idx = golden[f"pack_idx_b{bits}"]
    packed = pack_indices(cu(idx), bits)
    assert packed.dtype == torch.uint8 and tuple(packed.shape) == golden[f"pack_out_b{bits}"].shape
    assert np.array_equal(host(packed), golden[f"pack_out_b{bits}"])
    assert np.array_equal(host(unpack_indices(packed, bits, 128)), idx)


@pytest.mark.parametrize("bits", (1, 2, 3, 4))
@pytest.mark.parametrize("shape", ((1, 8), (3, 24), (7, 40), (5, 96), (1000, 128), (2, 3, 5, 256), (0, 64), (4097, 64)))
def test_pack_unpack_ragged_sizes(oracle, bits, shape):
    from mlx_turboquant_b200.packing import pack_indices, unpack_indices
    rs = np.random.RandomState(bits * 100 + len(shape))
    idx = rs.randint(0, 1 << bits, size=shape).astype(np.uint8)
    packed = pack_indices(cu(idx), bits)
    assert np.array_equal(host(packed), oracle.pack(idx, bits))
    assert np.array_equal(host(unpack_indices(packed, bits, shape[-1])), idx)


@pytest.mark.parametrize("bits", (2, 3, 4))
def test_pack_unaligned_pointers_and_extremes(oracle, bits):
    from mlx_turboquant_b200 import _lib
    rs = np.random.RandomState(5)
    n, d = 33, 64
    idx = rs.randint(0, 1 << bits, size=(n, d)).astype(np.uint8)
    idx[0] = 0
    idx[1] = (1 << bits) - 1
    buf = torch.zeros(n * d + 3, dtype=torch.uint8, device="cuda")
    buf[3:] = cu(idx).reshape(-1)                       # source starts 3 bytes off alignment
    out = torch.zeros(n * d * bits // 8 + 1, dtype=torch.uint8, device="cuda")
    lib = _lib.lib()
    _lib.check(lib.tq_pack(buf.data_ptr() + 3, out.data_ptr() + 1, n, d, bits, None))
    torch.cuda.synchronize()
    assert np.array_equal(host(out[1:]).reshape(n, -1), oracle.pack(idx, bits))
    back = torch.zeros(n * d + 5, dtype=torch.uint8, device="cuda")
    _lib.check(lib.tq_unpack(out.data_ptr() + 1, back.data_ptr() + 5, n, d, bits, None))
    torch.cuda.synchronize()
    assert np.array_equal(host(back[5:]).reshape(n, d), idx)


@pytest.mark.parametrize("d,bits", ((128, 4), (128, 3), (96, 2), (64, 1)))
def test_quantize_scalar_ties_and_clipping(golden, tables, d, bits):
    from mlx_turboquant_b200.codebook import dequantize_scalar, get_codebook, quantize_scalar
    c, b = get_codebook(d, bits)
    assert np.array_equal(host(c), tables[(d, bits)][0]) and np.array_equal(host(b), tables[(d, bits)][1])
    y = golden[f"qs_y_d{d}_b{bits}"]
    ref = golden[f"qs_idx_d{d}_b{bits}"]
    yt = cu(y)
    for sl in (slice(None), slice(0, -3), slice(1, None)):     # vector path, ragged tail, unaligned start
        idx = quantize_scalar(yt[sl], c, b)
        assert idx.dtype == torch.uint8 and np.array_equal(host(idx), ref[sl])
    idx = quantize_scalar(cu(y), c, b)
    assert np.array_equal(host(dequantize_scalar(idx, c)), tables[(d, bits)][0][golden[f"qs_idx_d{d}_b{bits}"]])


def test_quantize_extreme_and_boundary_values(tables):
    """Reference tests/test_edge_cases.py:38-52: +-100 clip to the end codes; boundary + 1e-7 goes up."""
    from mlx_turboquant_b200.codebook import get_codebook, quantize_scalar
    c, b = get_codebook(128, 4)
    idx = host(quantize_scalar(cu(np.array([100.0, -100.0], np.float32)), c, b))
    assert idx[0] == 15 and idx[1] == 0
    bn = tables[(128, 4)][1]
    assert host(quantize_scalar(cu(np.array([bn[7] + 1e-7], np.float32)), c, b))[0] == 8
    assert host(quantize_scalar(cu(np.array([bn[7]], np.float32)), c, b))[0] == 7     # strict >


@pytest.mark.parametrize("d", (64, 96, 128, 256))
@pytest.mark.parametrize("bits", (2, 3, 4))
def test_quantize_from_rotated_is_bit_exact(golden, tables, d, bits):
    """Given the reference's own float32 rotated rows, packed codes are identical byte for byte."""
    from mlx_turboquant_b200 import _lib
    tag = f"mse_d{d}_b{bits}"
    y = cu(golden[tag + "_y"])
    bnd = cu(tables[(d, bits)][1])
    out = torch.zeros(golden[tag + "_packed"].shape, dtype=torch.uint8, device="cuda")
    _lib.check(_lib.lib().tq_quantize_from_rotated(y.data_ptr(), y.shape[0], d, bnd.data_ptr(), bits, None, 0,
                                                   out.data_ptr(), None, None))
    assert np.array_equal(host(out), golden[tag + "_packed"])


def test_quantize_from_rotated_fractional(oracle, tables):
    from mlx_turboquant_b200 import _lib
    rs = np.random.RandomState(3)
    d = 128
    y = (rs.randn(257, d) / np.sqrt(d)).astype(np.float32)
    bh, bl = cu(tables[(d, 4)][1]), cu(tables[(d, 3)][1])
    ph = torch.zeros(257, 32, dtype=torch.uint8, device="cuda")
    pl = torch.zeros(257, 24, dtype=torch.uint8, device="cuda")
    yc = cu(y)
    _lib.check(_lib.lib().tq_quantize_from_rotated(yc.data_ptr(), 257, d, bh.data_ptr(), 4, bl.data_ptr(), 3,
                                                   ph.data_ptr(), pl.data_ptr(), None))
    assert np.array_equal(host(ph), oracle.pack(oracle.quantize_scalar(y[:, :64], tables[(d, 4)][1]), 4))
    assert np.array_equal(host(pl), oracle.pack(oracle.quantize_scalar(y[:, 64:], tables[(d, 3)][1]), 3))
