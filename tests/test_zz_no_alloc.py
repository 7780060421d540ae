"""tq_decode_attn_static: decode attention on the scratch array built into the library.

Meant for hosts that cannot hand over a workspace and cannot allocate one when the call is made (all device
memory already given to their own pool, or no room for a driver allocation in the step's latency budget).
The entry point must give the same result as tq_decode_attn on the same inputs, call after call, although
every call finds the previous call's leftovers in the shared array; and it must refuse, not overrun, when
the sizes need more scratch than the array has.  Collected last on purpose (file name): a failure here
cannot hide another test's result in a run that stops at the first failure.
"""

import ctypes as C

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _args_for(cache, q, out, ws):
    """Fill tq_decode_args from a cache object (the same fields TurboQuantKVCache.attend passes)."""
    from mlx_turboquant_b200 import _lib
    a = _lib.DecodeArgs()
    b, hq, d = q.shape
    k, v = cache._k, cache._v
    a.batch, a.n_q_heads, a.n_kv_heads, a.d = b, hq, cache.keys.shape[1], d
    a.q, a.q_dtype, a.scale, a.rot = q.data_ptr(), _lib.dtype_code(q.dtype), float(d ** -0.5), cache._rotation.data_ptr()
    a.c_len, a.c_lane_stride = cache._compressed_len, k.hi.shape[2]
    a.k_bits_hi, a.k_bits_lo, a.v_bits_hi, a.v_bits_lo = k.bits_hi, k.bits_lo, v.bits_hi, v.bits_lo
    a.k_hi, a.k_lo, a.v_hi, a.v_lo = _lib.ptr(k.hi), _lib.ptr(k.lo), _lib.ptr(v.hi), _lib.ptr(v.lo)
    a.k_norms, a.v_norms = _lib.ptr(k.norms), _lib.ptr(v.norms)
    a.k_cent_hi, a.k_cent_lo, a.v_cent_hi, a.v_cent_lo = _lib.ptr(k.cent_hi), _lib.ptr(k.cent_lo), _lib.ptr(v.cent_hi), _lib.ptr(v.cent_lo)
    a.v_cent_scale_hi, a.v_cent_scale_lo = v.fp16_scale_hi, v.fp16_scale_lo
    a.dense_dtype = _lib.dtype_code(cache.keys.dtype)
    a.sink_k, a.sink_v = cache.sink_keys.data_ptr(), cache.sink_values.data_ptr()
    a.sink_len, a.sink_lane_stride = cache._sink_len, cache.sink_keys.shape[2]
    a.res_k, a.res_v = cache.keys.data_ptr(), cache.values.data_ptr()
    a.res_len, a.res_lane_stride = cache._fp16_len, cache.keys.shape[2]
    a.out, a.out_dtype = out.data_ptr(), _lib.dtype_code(out.dtype)
    a.tables = _lib.ptr(cache._tables)
    if ws is not None:
        a.workspace, a.workspace_bytes = ws.data_ptr(), ws.numel()
    return a


def _cache(rs, b, hq, hkv, t, d, kb, vb):
    from mlx_turboquant_b200 import TurboQuantKVCache
    k = (rs.randn(b, hkv, t, d) * np.exp(0.5 * rs.randn(b, hkv, t, 1))).astype(np.float16)
    v = (rs.randn(b, hkv, t, d) * np.exp(0.5 * rs.randn(b, hkv, t, 1))).astype(np.float16)
    c = TurboQuantKVCache(head_dim=d, num_kv_heads=hkv, key_bits=kb, value_bits=vb, residual_window=32, fp16_sink_size=16)
    c.update(torch.from_numpy(k).cuda(), torch.from_numpy(v).cuda())
    q = torch.from_numpy((rs.randn(b, hq, d) / np.sqrt(d)).astype(np.float16)).cuda()
    return c, q


def test_static_scratch_matches_workspace_entry_point_twice_in_a_row():
    from mlx_turboquant_b200 import _lib
    lib = _lib.lib()
    rs = np.random.RandomState(321)
    stream = torch.cuda.current_stream().cuda_stream
    # two different shapes back to back: the second call finds the first call's partials in the array
    for (b, hq, hkv, t, d, kb, vb) in ((1, 8, 2, 3000, 128, 4, 2), (2, 4, 4, 700, 96, 3, 2)):
        cache, q = _cache(rs, b, hq, hkv, t, d, kb, vb)
        need = lib.tq_decode_workspace_bytes(b, hq, hkv, d, cache._compressed_len, cache._sink_len + cache._fp16_len)
        ws = torch.zeros(need, dtype=torch.uint8, device="cuda")
        ref = torch.empty(b, hq, d, dtype=torch.float32, device="cuda")
        _lib.check(lib.tq_decode_attn(C.byref(_args_for(cache, q, ref, ws)), stream))
        for _ in range(2):
            out = torch.full((b, hq, d), float("nan"), dtype=torch.float32, device="cuda")
            _lib.check(lib.tq_decode_attn_static(C.byref(_args_for(cache, q, out, None)), stream))
            torch.cuda.synchronize()
            # same kernel, same split plan, and partials are merged in a fixed order whichever CTA arrives last:
            # the two entry points give the same bits
            assert torch.isfinite(out).all() and torch.equal(out, ref)
        # and it still agrees with attention over the dense tensors the cache would hand out
        dk, dv = cache.update_and_fetch(cache.keys[:, :, :0], cache.values[:, :, :0])
        rep = hq // hkv
        p = torch.softmax((q.float()[:, :, None] @ dk.float().repeat_interleave(rep, 1).transpose(-1, -2)) * d ** -0.5, dim=-1)
        dense = (p @ dv.float().repeat_interleave(rep, 1))[:, :, 0]
        assert (out - dense).abs().max().item() / dense.abs().max().item() < 2e-3


def test_static_scratch_refuses_sizes_beyond_its_array():
    from mlx_turboquant_b200 import _lib
    lib = _lib.lib()
    rs = np.random.RandomState(5)
    cache, q = _cache(rs, 1, 4, 2, 200, 128, 4, 2)
    out = torch.empty(1, 4, 128, dtype=torch.float32, device="cuda")
    a = _args_for(cache, q, out, None)
    a.batch = 4096            # scratch need grows with the batch: far past 8 MiB, rejected before anything is launched
    assert lib.tq_decode_attn_static(C.byref(a), None) == -2
    assert b"built-in array" in lib.tq_last_error()
    assert lib.tq_decode_attn_static(None, None) == -1


def test_static_scratch_keeps_its_shapes_where_the_streaming_kernel_would_need_more():
    """Many lanes of a short context: tq_decode_attn takes the persistent streaming kernel, whose partials (one per lane
    and warp that touches it) need more scratch than the built-in array has; the static entry point runs the
    table-lookup kernel on the same arguments instead of refusing them."""
    from mlx_turboquant_b200 import _lib
    lib = _lib.lib()
    rs = np.random.RandomState(99)
    b, hq, hkv, t, d = 64, 32, 8, 2000, 128
    cache, q = _cache(rs, b, hq, hkv, t, d, 4, 2)
    dense_len = cache._sink_len + cache._fp16_len
    need = lib.tq_decode_workspace_bytes(b, hq, hkv, d, cache._compressed_len, dense_len)
    assert need > 8 << 20
    ws = torch.zeros(need, dtype=torch.uint8, device="cuda")
    stream = torch.cuda.current_stream().cuda_stream
    ref = torch.empty(b, hq, d, dtype=torch.float32, device="cuda")
    a = _args_for(cache, q, ref, ws)
    assert lib.tq_decode_kernel_choice(C.byref(a)) == 2
    _lib.check(lib.tq_decode_attn(C.byref(a), stream))
    out = torch.full((b, hq, d), float("nan"), dtype=torch.float32, device="cuda")
    _lib.check(lib.tq_decode_attn_static(C.byref(_args_for(cache, q, out, None)), stream))
    torch.cuda.synchronize()
    assert torch.isfinite(out).all()
    assert (out - ref).abs().max().item() / ref.abs().max().item() < 2e-3        # two kernels, one answer
    assert lib.tq_device_status() == 0
