"""The streaming decode kernel (persistent grid, 4-bit keys / 2-bit values at d = 96 / 128, sign sketches optional)
against the oracle and against the general kernel on the same cache state.

Oracle = reference cache (restated, pinned) -> dense K/V -> float32 softmax attention; tolerance 1e-3 of the output's
largest magnitude.  The kernel is chosen for calls with many tiles per warp; the tests lower that threshold to one so
that small caches (which the oracle finishes in seconds) take it, and check with tq_decode_kernel_choice that they did."""

import ctypes as C

import numpy as np
import pytest
import torch

from gpu_util import host
from test_decode_gpu import _case, _check

pytestmark = pytest.mark.gpu


@pytest.fixture()
def stream_forced():
    from mlx_turboquant_b200.kernels import set_tuning
    set_tuning("decode_stream_min_run", 1)
    set_tuning("decode_stream_max_parts", 64)
    yield
    set_tuning("decode_stream_min_run", 24)
    set_tuning("decode_stream_max_parts", 40)


def _choice(c):
    from mlx_turboquant_b200 import _lib
    return _lib.lib().tq_decode_kernel_choice(C.byref(c._dargs))


def _both(c, q, ref, want_stream=True):
    from mlx_turboquant_b200 import _lib
    from mlx_turboquant_b200.kernels import set_tuning
    s = c.attend(q, out_dtype=torch.float32)
    assert (_choice(c) == 2) == want_stream
    _check(s, ref)
    set_tuning("decode_stream", 0)
    try:
        g = c.attend(q, out_dtype=torch.float32)
        assert _choice(c) != 2
    finally:
        set_tuning("decode_stream", 1)
    _check(g, ref)
    assert np.abs(host(s) - host(g)).max() <= 2e-3 * np.abs(ref).max()
    assert _lib.lib().tq_device_status() == 0


@pytest.mark.parametrize("qjl", (False, True))
@pytest.mark.parametrize("d,b,hq,hkv,t", ((96, 6, 8, 8, 700), (96, 3, 32, 16, 523), (128, 5, 32, 8, 800), (128, 16, 32, 2, 700),
                                           (96, 12, 32, 2, 600)))
def test_stream_kernel_equals_oracle_and_general_kernel(oracle, stream_forced, d, b, hq, hkv, t, qjl):
    """MHA, GQA 2 / 4 and 16 query heads per KV head (two head groups); ragged lengths (the last tile is partial)."""
    rs = np.random.RandomState(d + b + t + int(qjl))
    c, q, ref = _case(oracle, rs, b, hq, hkv, t, d, 4, 2, 32, 16, qjl=qjl)
    _both(c, q, ref)


@pytest.mark.parametrize("qjl", (False, True))
def test_runs_that_span_several_lanes(oracle, stream_forced, qjl):
    """Many short lanes: a warp's run covers several (sequence, KV head) lanes and writes a partial for each."""
    rs = np.random.RandomState(5 + int(qjl))
    c, q, ref = _case(oracle, rs, 48, 64, 64, 100, 96, 4, 2, 16, 4, qjl=qjl)
    _both(c, q, ref)


def test_regions_and_dtypes(oracle, stream_forced):
    rs = np.random.RandomState(11)
    for (t, rw, sink) in ((600, 0, 0), (600, 16, 0), (600, 0, 8), (1100, 64, 64)):       # no uncompressed tokens / only one side
        c, q, ref = _case(oracle, rs, 8, 8, 8, t, 96, 4, 2, rw, sink, qjl=True)
        _both(c, q, ref)
    c, q, ref = _case(oracle, rs, 8, 8, 8, 640, 96, 4, 2, 32, 16, dtype=np.float32, qjl=True)   # float32 uncompressed tokens and query
    _both(c, q, ref)
    c, q, ref = _case(oracle, rs, 8, 16, 8, 640, 128, 4, 2, 32, 16, bf16=True)
    _both(c, q, ref)
    out = c.attend(q)                      # result in the query's dtype
    assert out.dtype == torch.bfloat16
    _check(out, ref, tol=1e-3 + 2.0 ** -9)            # (a bfloat16 result carries half an ulp of 2^-8)


def test_not_chosen_for_few_lanes_or_other_widths(oracle, stream_forced):
    rs = np.random.RandomState(12)
    c, q, ref = _case(oracle, rs, 1, 8, 2, 3000, 128, 4, 2, 32, 16)        # 188 tiles per lane and two lanes: too many partials per lane
    _both(c, q, ref, want_stream=False)
    c, q, ref = _case(oracle, rs, 8, 8, 8, 600, 96, 3, 2, 32, 16)          # 3-bit keys
    _both(c, q, ref, want_stream=False)
    c, q, ref = _case(oracle, rs, 8, 8, 8, 600, 64, 4, 2, 32, 16)          # d = 64
    _both(c, q, ref, want_stream=False)


def test_value_norms_far_outside_the_fp16_range(oracle, stream_forced):
    rs = np.random.RandomState(13)
    for v_scale in (1e5, 1e-6):
        c, q, ref = _case(oracle, rs, 8, 8, 8, 600, 96, 4, 2, 32, 16, dtype=np.float32, qjl=True, v_scale=v_scale)
        _both(c, q, ref)


def test_decode_steps_append_and_attend(oracle, stream_forced):
    """decode_step (append + attend in one call) through the streaming kernel equals update followed by attend."""
    from mlx_turboquant_b200 import TurboQuantKVCache
    torch.manual_seed(3)
    b, h, d, t = 8, 8, 96, 500
    k, v = torch.randn(b, h, t, d, device="cuda").half(), torch.randn(b, h, t, d, device="cuda").half()
    mk = lambda: TurboQuantKVCache(head_dim=d, num_kv_heads=h, key_bits=4, value_bits=2, residual_window=64, fp16_sink_size=16,  # noqa: E731
                                   qjl_correction=True)
    c1, c2 = mk(), mk()
    c1.update(k, v)
    c2.update(k, v)
    for i in range(5):
        kn, vn = torch.randn(b, h, 1, d, device="cuda").half(), torch.randn(b, h, 1, d, device="cuda").half()
        q = (torch.randn(b, h, 1, d, device="cuda") / d ** 0.5).half()
        o1 = c1.decode_step(q, kn, vn).float()
        assert _choice(c1) == 2
        c2.update(kn, vn)
        o2 = c2.attend(q).float()
        assert torch.allclose(o1, o2, rtol=0, atol=3e-3 * float(o2.abs().max()))
    assert torch.equal(c1.keys[:, :, :c1._fp16_len], c2.keys[:, :, :c2._fp16_len])
