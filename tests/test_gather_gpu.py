"""Fused output gather of head-sharded decoding: the merge step stores each shard's heads into every rank's buffer and
bumps arrival counters.  On one GPU the ranks are emulated as consecutive launches whose "peer" buffers all live on the
same device (no launch waits for another: the wait kernels run after both decode launches on the same stream)."""

import ctypes as C

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _shard_caches(hkv, d, ctx, kb, vb, world, seed):
    from mlx_turboquant_b200 import TurboQuantKVCache
    from gpu_util import cu, kv_like
    rs = np.random.RandomState(seed)
    k, v = kv_like(rs, (1, hkv, ctx, d)), kv_like(rs, (1, hkv, ctx, d))
    per = hkv // world
    caches = []
    for r in range(world):
        c = TurboQuantKVCache(head_dim=d, num_kv_heads=per, key_bits=kb, value_bits=vb, residual_window=32, fp16_sink_size=16)
        c.update(cu(k[:, r * per:(r + 1) * per]), cu(v[:, r * per:(r + 1) * per]))
        caches.append(c)
    return caches


@pytest.mark.parametrize("d,kb,vb,ctx", [(128, 4, 2, 3000), (128, 3, 2, 700), (96, 4, 2, 500)])
def test_two_emulated_ranks_fill_both_buffers(d, kb, vb, ctx):
    from mlx_turboquant_b200 import _lib
    world, hq, hkv = 2, 8, 4
    caches = _shard_caches(hkv, d, ctx, kb, vb, world, seed=11)
    g = torch.Generator(device="cuda").manual_seed(12)
    q = (torch.randn(1, hq, 1, d, device="cuda", generator=g) / d ** 0.5).half()
    hq_loc = hq // world
    want = torch.cat([caches[r].attend(q[:, r * hq_loc:(r + 1) * hq_loc].contiguous()) for r in range(world)], dim=1)

    bufs = [torch.full((1, hq, d), float("nan"), dtype=torch.float16, device="cuda") for _ in range(world)]
    ctrs = torch.zeros(world, dtype=torch.int64, device="cuda")
    per_call = int(_lib.lib().tq_gather_arrivals_per_call(1, hq_loc, hkv // world))
    assert per_call == hkv // world
    for rep in (1, 2):                                     # counters only grow: the second round waits for twice as many
        for r in range(world):
            gs = _lib.PeerGather()
            gs.n_peers, gs.heads_total, gs.head_offset = world, hq, r * hq_loc
            for j in range(world):
                gs.out[j] = bufs[j].data_ptr()
                gs.arrivals[j] = ctrs.data_ptr() + 8 * j
            assert caches[r].attend(q[:, r * hq_loc:(r + 1) * hq_loc].contiguous(), gather=gs) is None
        for j in range(world):
            _lib.check(_lib.lib().tq_gather_wait(ctrs.data_ptr() + 8 * j, None, rep * world * per_call, _lib.stream_ptr(q.device)))
        torch.cuda.synchronize()
        assert ctrs.tolist() == [rep * world * per_call] * world
        for j in range(world):
            assert torch.equal(bufs[j].reshape(1, hq, 1, d), want)      # same kernel, same arithmetic: identical bits
        for b in bufs:
            b.fill_(float("nan"))
    assert _lib.lib().tq_device_status() == 0


def test_gather_argument_errors():
    from mlx_turboquant_b200 import _lib
    caches = _shard_caches(2, 128, 300, 4, 2, 1, seed=13)
    q = torch.zeros(1, 4, 1, 128, dtype=torch.float16, device="cuda")
    gs = _lib.PeerGather()
    gs.n_peers, gs.heads_total, gs.head_offset = 1, 4, 2    # heads 2..5 do not fit in 4
    buf = torch.zeros(1, 4, 128, dtype=torch.float16, device="cuda")
    ctr = torch.zeros(1, dtype=torch.int64, device="cuda")
    gs.out[0], gs.arrivals[0] = buf.data_ptr(), ctr.data_ptr()
    with pytest.raises(ValueError):
        caches[0].attend(q, gather=gs)
    gs.head_offset = 0
    gs.arrivals[0] = None
    with pytest.raises(ValueError):
        caches[0].attend(q, gather=gs)
    with pytest.raises(ValueError):
        _lib.check(_lib.lib().tq_gather_wait(None, None, 1, _lib.stream_ptr(q.device)))


def test_fused_gather_object_single_rank():
    """The IPC-backed helper with a world of one: allocation, views, call counting, wait, close."""
    import torch.distributed as dist
    from mlx_turboquant_b200 import sharding
    own_group = not dist.is_initialized()
    if own_group:
        dist.init_process_group("gloo", init_method="tcp://127.0.0.1:29533", rank=0, world_size=1)
    try:
        caches = _shard_caches(2, 128, 1000, 4, 2, 1, seed=14)
        q = (torch.randn(1, 8, 1, 128, device="cuda") / 128 ** 0.5).half()
        want = caches[0].attend(q)
        fg = sharding.FusedGather(1, 8, 128, torch.float16, n_buffers=2, head_offset=0, n_local_heads=8, n_local_kv_heads=2,
                                  device=q.device)
        for i in (0, 1, 0):
            caches[0].attend(q, gather=fg.slot(i))
            fg.wait(i)
            torch.cuda.synchronize()
            assert torch.equal(fg.result(i).reshape(1, 8, 1, 128), want)
            fg.result(i).zero_()
        # the pair of launches takes the same arguments every time: capture once, replay
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            caches[0].attend(q, gather=fg.slot(1))
            fg.wait(1)
        for _ in range(3):
            fg.result(1).zero_()
            graph.replay()
            torch.cuda.synchronize()
            assert torch.equal(fg.result(1).reshape(1, 8, 1, 128), want)
        from mlx_turboquant_b200 import _lib
        assert _lib.lib().tq_device_status() == 0
        fg.close()
    finally:
        if own_group:
            dist.destroy_process_group()


def test_wait_that_nothing_satisfies_gives_up_and_reports():
    """A counter nobody increments: the wait ends by itself after its poll limit, leaves status 201, and the stream,
    the context and later waits keep working."""
    from mlx_turboquant_b200 import _lib, kernels
    lib = _lib.lib()
    assert lib.tq_device_status() == 0
    ctr = torch.zeros(2, dtype=torch.int64, device="cuda")             # [arrivals, consumed]
    kernels.set_tuning("gather_wait_polls", 20000)                      # some 25 ms
    try:
        _lib.check(lib.tq_gather_wait(ctr.data_ptr(), ctr.data_ptr() + 8, 3, _lib.stream_ptr(ctr.device)))
        torch.cuda.synchronize()
        assert lib.tq_device_status() == 201
        assert ctr.tolist() == [0, 3]                                   # the consumed counter moved on all the same
        assert lib.tq_device_status_clear() == 0 and lib.tq_device_status() == 0
        ctr[0] = 5
        _lib.check(lib.tq_gather_wait(ctr.data_ptr(), ctr.data_ptr() + 8, 2, _lib.stream_ptr(ctr.device)))   # 5 >= 3 + 2
        torch.cuda.synchronize()
        assert lib.tq_device_status() == 0 and ctr.tolist() == [5, 5]
    finally:
        kernels.set_tuning("gather_wait_polls", 2000000)
        lib.tq_device_status_clear()
