"""The Llama-shaped caller (reference: mlx-lm's Attention.__call__, docs/attention_source_dump.txt:70-98) driving the cache.

CPU: the caller's own logic (RoPE offsets, causal mask, incremental decoding) with uncompressed caches.
GPU: prefill + decode through TurboQuant caches - the packed route (update + attend) against the dense route the
reference takes (update_and_fetch + softmax attention), and one layer's cache traffic replayed through the oracle.
"""

import numpy as np
import pytest
import torch

from mlx_turboquant_b200.consumer import LlamaShaped, ModelArgs, generate, rope

TINY = dict(hidden_size=256, num_hidden_layers=2, num_attention_heads=8, num_key_value_heads=4, head_dim=128,
            intermediate_size=512, vocab_size=512)


def test_rope_is_a_rotation_and_relative():
    g = torch.Generator().manual_seed(0)
    q, k = torch.randn(1, 1, 1, 64, generator=g), torch.randn(1, 1, 1, 64, generator=g)
    assert torch.allclose(rope(q, 7, 1e4).norm(), q.norm(), rtol=1e-5)
    a = (rope(q, 10, 1e4) * rope(k, 3, 1e4)).sum()
    b = (rope(q, 107, 1e4) * rope(k, 100, 1e4)).sum()
    assert torch.allclose(a, b, atol=1e-4)                     # scores depend on the distance only


def test_incremental_decoding_matches_full_forward_cpu():
    m = LlamaShaped(ModelArgs(**TINY), dtype=torch.float32, device="cpu", seed=1, std=0.05)
    tok = torch.randint(0, 512, (2, 12), generator=torch.Generator().manual_seed(2))
    full = m(tok)                                              # no cache: causal attention over the whole sequence
    for packed in (False, True):
        cache = m.make_cache()
        got = [m(tok[:, :5], cache=cache, packed=packed)]
        got += [m(tok[:, i:i + 1], cache=cache, packed=packed) for i in range(5, 9)]
        got.append(m(tok[:, 9:], cache=cache, packed=packed))  # a multi-token call on a non-empty cache
        assert torch.allclose(torch.cat(got, dim=1), full, atol=2e-4), packed
        assert cache[0].offset == 12


def test_generate_is_greedy_cpu():
    m = LlamaShaped(ModelArgs(**TINY), dtype=torch.float32, device="cpu", seed=3, std=0.05)
    prompt = torch.randint(0, 512, (1, 6), generator=torch.Generator().manual_seed(4))
    out = generate(m, prompt, 4)
    seq = prompt
    for i in range(4):
        nxt = m(seq)[:, -1].argmax(-1, keepdim=True)
        assert int(nxt) == int(out[0, i])
        seq = torch.cat([seq, nxt], dim=1)
    assert torch.equal(generate(m, prompt, 4, prefill_chunk=4), out)


class _Recorder:
    """Wraps one layer's cache and keeps what the caller fed it and got back."""

    def __init__(self, inner):
        self.inner, self.fed, self.calls = inner, [], []

    def __getattr__(self, name):
        return getattr(self.inner, name)

    def update(self, k, v):
        self.fed.append((k.clone(), v.clone()))
        self.inner.update(k, v)

    def update_and_fetch(self, k, v):
        self.fed.append((k.clone(), v.clone()))
        return self.inner.update_and_fetch(k, v)

    def attend(self, q, scale=None):
        out = self.inner.attend(q, scale)
        self.calls.append((len(self.fed) - 1, q.clone(), out.clone()))
        return out

    def decode_step(self, q, k, v, scale=None):
        self.fed.append((k.clone(), v.clone()))
        out = self.inner.decode_step(q, k, v, scale)
        self.calls.append((len(self.fed) - 1, q.clone(), out.clone()))
        return out


@pytest.mark.gpu
@pytest.mark.parametrize("kb,vb,qjl", [(4, 2, False), (3.5, 3, False), (4, 2, True)])
def test_packed_route_matches_dense_route_and_oracle(kb, vb, qjl):
    from mlx_turboquant_b200 import apply_turboquant
    from oracle import tq_oracle as oracle
    from gpu_util import host, host_tables

    m = LlamaShaped(ModelArgs(**TINY), dtype=torch.float32, device="cuda", seed=5, std=0.05)
    apply_turboquant(m, key_bits=kb, value_bits=vb, residual_window=32, fp16_sink_size=16, chunk_size=0,
                     qjl_correction=qjl, auto_detect_outliers=False)
    g = torch.Generator().manual_seed(6)
    prompt = torch.randint(0, 512, (2, 150), generator=g).cuda()
    steps = torch.randint(0, 512, (2, 40), generator=g).cuda()     # forced tokens: both routes see the same inputs

    logits = {}
    rec = None
    for packed in (False, True):
        cache = m.make_cache()
        if packed:
            rec = cache[0] = _Recorder(cache[0])
        lg = [m(prompt, cache=cache, packed=packed, last_only=True)]
        for i in range(steps.shape[1]):                             # crosses a drain of the recent-token buffer
            lg.append(m(steps[:, i:i + 1], cache=cache, packed=packed))
        logits[packed] = torch.cat(lg, dim=1)
        assert cache[1].offset == 190
    err = (logits[True] - logits[False]).abs().max() / logits[False].abs().max()
    assert err < 2e-3, float(err)

    # layer 0's traffic through the oracle's cache: same inputs, attention in float32 over its dense output
    d = 128
    ref_c = oracle.KVCacheOracle(d, host_tables(d), kb, vb, 32, fp16_sink_size=16, chunk_size=0, qjl_correction=qjl)
    dense = [ref_c.update_and_fetch(host(k), host(v)) for (k, v) in rec.fed]
    assert len(rec.calls) == (40 if qjl else 41)                     # with a sketch the prefill call goes the dense way
    for (i, q, got) in rec.calls:
        rk, rv = dense[i]
        tq, tkv = q.shape[2], rk.shape[2]
        ref = np.concatenate([oracle.attention(host(q)[:, :, j:j + 1], rk[:, :, :tkv - tq + j + 1], rv[:, :, :tkv - tq + j + 1])
                              for j in range(tq)], axis=2)           # causal: query j sees the keys up to its own
        assert np.abs(host(got) - ref).max() / np.abs(ref).max() < 1e-3
    assert ref_c.offset == 190 and ref_c.comp_len > 0


@pytest.mark.gpu
def test_generate_through_compressed_caches_bf16():
    from mlx_turboquant_b200 import apply_turboquant, TurboQuantKVCache
    m = LlamaShaped(ModelArgs(**TINY), dtype=torch.bfloat16, device="cuda", seed=7, std=0.05)
    apply_turboquant(m, key_bits=4, value_bits=2, residual_window=128, fp16_sink_size=128, auto_detect_outliers=False)
    prompt = torch.randint(0, 512, (3, 700), generator=torch.Generator().manual_seed(8)).cuda()
    cache = m.make_cache()
    out = generate(m, prompt, 8, cache=cache, prefill_chunk=256)
    assert out.shape == (3, 8) and int(out.min()) >= 0 and int(out.max()) < 512
    c = cache[0]
    assert isinstance(c, TurboQuantKVCache) and c.offset == 707 and c._compressed_len > 0 and c._sink_len == 128


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_graphed_decoder_equals_eager_steps(dtype):
    """The decode step with its library part replayed from CUDA graphs produces the tokens of the eager step, across a
    drain of the recent-token buffer (steps that compress are ordinary cache calls between two graph launches)."""
    from mlx_turboquant_b200 import apply_turboquant
    from mlx_turboquant_b200.consumer import GraphedDecoder
    m = LlamaShaped(ModelArgs(**TINY), dtype=dtype, device="cuda", seed=9, std=0.05)
    apply_turboquant(m, key_bits=4, value_bits=2, residual_window=32, fp16_sink_size=16, auto_detect_outliers=False)
    g = torch.Generator().manual_seed(10)
    prompt = torch.randint(0, 512, (3, 100), generator=g).cuda()
    runs = []
    for graphed in (False, True):
        cache = m.make_cache()
        tok = m(prompt, cache=cache, packed=True, last_only=True)[:, -1].argmax(-1, keepdim=True)
        toks = []
        if graphed:
            dec = GraphedDecoder(m, cache, tok)
            for _ in range(80):
                toks.append(dec.step().clone())
        else:
            for _ in range(80):
                tok = m(tok, cache=cache, packed=True)[:, -1].argmax(-1, keepdim=True)
                toks.append(tok)
        assert cache[0].offset == 180 and cache[0]._compressed_len > 0
        runs.append(torch.cat(toks, dim=1))
    assert torch.equal(runs[0], runs[1])
