"""Fused output gather of head-sharded decoding: the merge step sends each shard's heads into every rank's landing buffer
as {payload, epoch} words.  On one GPU the ranks are emulated as consecutive launches whose "peer" buffers all live on the
same device (no launch waits for another: the waits run after both decode launches on the same stream)."""

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

    words = hq * d // 2
    lls = [torch.zeros(words, dtype=torch.int64, device="cuda") for _ in range(world)]        # rank j's landing buffer
    outs = [torch.full((1, hq, d), float("nan"), dtype=torch.float16, device="cuda") for _ in range(world)]
    groups = int(_lib.lib().tq_gather_groups(1, hq_loc, hkv // world))
    assert groups == hkv // world
    epochs = [torch.zeros(groups, dtype=torch.int32, device="cuda") for _ in range(world)]
    stream = _lib.stream_ptr(q.device)
    for rep in (1, 2, 3):
        for r in range(world):
            gs = _lib.PeerGather()
            gs.n_peers, gs.heads_total, gs.head_offset = world, hq, r * hq_loc
            for j in range(world):
                gs.ll[j] = lls[j].data_ptr()
            gs.epochs = epochs[r].data_ptr()
            assert caches[r].attend(q[:, r * hq_loc:(r + 1) * hq_loc].contiguous(), gather=gs) is None
        if rep < 3:
            for j in range(world):
                _lib.check(_lib.lib().tq_gather_wait(lls[j].data_ptr(), epochs[j].data_ptr(), words, outs[j].data_ptr(), stream))
        else:       # the wait inside a following decode call (both producers are earlier on the stream: nothing waits for a later launch)
            for j in range(world):
                caches[j].attend(q[:, j * hq_loc:(j + 1) * hq_loc].contiguous(),
                                 after=(lls[j].data_ptr(), epochs[j].data_ptr(), words, outs[j].data_ptr()))
        torch.cuda.synchronize()
        for j in range(world):
            assert epochs[j].tolist() == [rep] * groups
            assert (lls[j] >> 32).tolist() == [rep] * words
            assert torch.equal(outs[j].reshape(1, hq, 1, d), want)      # same kernel, same arithmetic: identical bits
        for b in outs:
            b.fill_(float("nan"))
    assert _lib.lib().tq_device_status() == 0


def test_gather_argument_errors():
    from mlx_turboquant_b200 import _lib
    caches = _shard_caches(2, 128, 300, 4, 2, 1, seed=13)
    q = torch.zeros(1, 4, 1, 128, dtype=torch.float16, device="cuda")
    gs = _lib.PeerGather()
    gs.n_peers, gs.heads_total, gs.head_offset = 1, 4, 2    # heads 2..5 do not fit in 4
    ll = torch.zeros(4 * 128 // 2, dtype=torch.int64, device="cuda")
    ep = torch.zeros(2, dtype=torch.int32, device="cuda")
    gs.ll[0], gs.epochs = ll.data_ptr(), ep.data_ptr()
    with pytest.raises(ValueError):
        caches[0].attend(q, gather=gs)
    gs.head_offset = 0
    gs.epochs = None
    with pytest.raises(ValueError):
        caches[0].attend(q, gather=gs)
    with pytest.raises(ValueError):
        _lib.check(_lib.lib().tq_gather_wait(None, None, 1, None, _lib.stream_ptr(q.device)))
    with pytest.raises(ValueError):
        caches[0].attend(q, after=(ll.data_ptr(), None, 256, None))


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
        # the launches take the same arguments every time: capture once, replay; the second call waits for the first
        # one's gather in its prologue, the last one's gather gets a wait launch
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            caches[0].attend(q, gather=fg.slot(1))
            caches[0].attend(q, gather=fg.slot(0), after=fg.arrived(1))
            fg.wait(0)
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
    ll = torch.zeros(256, dtype=torch.int64, device="cuda")            # no word carries epoch 3
    ep = torch.tensor([3], dtype=torch.int32, device="cuda")
    out = torch.zeros(256, dtype=torch.int32, device="cuda")
    kernels.set_tuning("gather_wait_polls", 20000)                      # some 10 ms
    try:
        _lib.check(lib.tq_gather_wait(ll.data_ptr(), ep.data_ptr(), 256, out.data_ptr(), _lib.stream_ptr(ll.device)))
        torch.cuda.synchronize()
        assert lib.tq_device_status() == 201
        assert lib.tq_device_status_clear() == 0 and lib.tq_device_status() == 0
        # the same wait inside a decode call: the kernel gives up, reports and still computes its result
        caches = _shard_caches(2, 128, 300, 4, 2, 1, seed=15)
        q = (torch.randn(1, 8, 1, 128, device="cuda") / 128 ** 0.5).half()
        want = caches[0].attend(q)
        after = (ll.data_ptr(), ep.data_ptr(), 256, out.data_ptr())
        got = caches[0].attend(q, after=after)
        torch.cuda.synchronize()
        assert lib.tq_device_status() == 201 and torch.equal(got, want)
        assert lib.tq_device_status_clear() == 0
        ll.copy_((torch.arange(256, device="cuda") + 7) | (3 << 32))   # the words arrive
        _lib.check(lib.tq_gather_wait(ll.data_ptr(), ep.data_ptr(), 256, out.data_ptr(), _lib.stream_ptr(ll.device)))
        torch.cuda.synchronize()
        assert lib.tq_device_status() == 0 and out.tolist() == list(range(7, 263))
        out.zero_()
        got = caches[0].attend(q, after=after)
        torch.cuda.synchronize()
        assert lib.tq_device_status() == 0 and out.tolist() == list(range(7, 263)) and torch.equal(got, want)
    finally:
        kernels.set_tuning("gather_wait_polls", 2000000)
        lib.tq_device_status_clear()
