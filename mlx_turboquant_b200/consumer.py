"""A minimal Llama-shaped consumer of the cache protocol: the caller on the far side of the hot path.

The reference never runs attention itself; mlx-lm's Llama ``Attention.__call__`` does
(docs/attention_source_dump.txt:70-98): project, RoPE at ``cache.offset``, ``cache.update_and_fetch``,
softmax attention, output projection.  This module restates that caller on torch so the cache can be
exercised end to end: RMSNorm, rotary embedding (non-traditional layout, base ``rope_theta``), grouped-query
attention, SwiGLU, tied to nothing but ``torch`` library calls (GEMMs and the dense prefill attention are
library work, not part of the compressed path).  Two ways through the cache:

* dense (the reference's only way): ``keys, values = cache.update_and_fetch(k, v)`` then softmax attention;
* packed: attention straight from packed storage - ``cache.decode_step(q, k, v)`` for one new token per sequence
  (append and attention in one launch), ``cache.update(k, v)`` then the causal ``cache.attend(q)`` for a prefill
  chunk.  Caches with a QJL sketch take the dense way for multi-token calls.

``GraphedDecoder`` replays the library part of a decode step (everything between two cache calls) as CUDA graphs.

``generate`` is the greedy loop of the reference's command line (cli.py:81-104) without its tokenizer.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.nn.functional as F


@dataclass
class ModelArgs:
    """Field names follow the Hugging Face / mlx-lm config the reference reads (patch.py:13-86)."""

    hidden_size: int = 4096
    num_hidden_layers: int = 32
    num_attention_heads: int = 32
    num_key_value_heads: int = 8
    head_dim: int = 128
    intermediate_size: int = 14336
    rope_theta: float = 500000.0
    vocab_size: int = 128256
    rms_norm_eps: float = 1e-5


def _rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    return F.rms_norm(x, (x.shape[-1],), weight, eps)


def rope_tables(offset: int, length: int, dim: int, theta: float, device) -> tuple[torch.Tensor, torch.Tensor]:
    """(cos | cos) and (-sin | sin) rows, float32 (length, dim), for positions ``offset ... offset+length-1``."""
    half = dim // 2
    inv = theta ** (-torch.arange(0, half, device=device, dtype=torch.float32) / half)
    ang = torch.arange(offset, offset + length, device=device, dtype=torch.float32)[:, None] * inv[None, :]
    cos, sin = ang.cos(), ang.sin()
    return torch.cat([cos, cos], dim=-1), torch.cat([-sin, sin], dim=-1)


def apply_rope(x: torch.Tensor, tables) -> torch.Tensor:
    """Half-split rotary embedding (``traditional=False``): (a, b) -> (a cos - b sin, b cos + a sin), in float32."""
    cos2, sin2 = tables
    xf = x.float()
    return torch.addcmul(xf * cos2, torch.roll(xf, x.shape[-1] // 2, dims=-1), sin2).to(x.dtype)


def rope(x: torch.Tensor, offset: int, theta: float) -> torch.Tensor:
    """Rotary embedding of ``x`` (B, H, L, D) at positions ``offset ... offset+L-1``."""
    return apply_rope(x, rope_tables(offset, x.shape[2], x.shape[3], theta, x.device))


class Attention(torch.nn.Module):
    def __init__(self, args: ModelArgs, dtype, device):
        super().__init__()
        self.n_heads, self.n_kv_heads, self.head_dim = args.num_attention_heads, args.num_key_value_heads, args.head_dim
        self.scale = self.head_dim ** -0.5
        self.rope_theta = args.rope_theta
        kw = dict(bias=False, dtype=dtype, device=device)
        # one fused projection for q, k and v (same arithmetic as three separate matrices)
        self.qkv_proj = torch.nn.Linear(args.hidden_size, (self.n_heads + 2 * self.n_kv_heads) * self.head_dim, **kw)
        self.o_proj = torch.nn.Linear(self.n_heads * self.head_dim, args.hidden_size, **kw)

    def forward(self, x: torch.Tensor, cache=None, packed: bool = True, rope_memo: dict | None = None) -> torch.Tensor:
        B, L, _ = x.shape
        hq, hkv, d = self.n_heads, self.n_kv_heads, self.head_dim
        qkv = self.qkv_proj(x).view(B, L, hq + 2 * hkv, d).transpose(1, 2)            # (B, heads, L, d)
        offset = cache.offset if cache is not None else 0                               # read before the update
        # queries and keys sit at the same positions: one pass over both; the tables are shared by layers at one offset
        tables = rope_memo.get((offset, L)) if rope_memo is not None else None
        if tables is None:
            tables = rope_tables(offset, L, d, self.rope_theta, x.device)
            if rope_memo is not None:
                rope_memo[(offset, L)] = tables
        qk = apply_rope(qkv[:, :hq + hkv], tables)
        queries, keys, values = qk[:, :hq], qk[:, hq:], qkv[:, hq + hkv:]
        if cache is not None and packed and hasattr(cache, "attend") and (L == 1 or not getattr(cache, "qjl_correction", False)):
            # attention straight from packed storage: one launch for a decode step (the token's append included), the
            # causal multi-token kernel for prefill chunks (caches with a QJL sketch take the dense route there)
            if L == 1:
                out = cache.decode_step(queries.contiguous(), keys.contiguous(), values.contiguous(), self.scale)     # (B, hq, 1, d)
            else:
                cache.update(keys.contiguous(), values.contiguous())
                out = cache.attend(queries.contiguous(), self.scale)                   # (B, hq, L, d)
        else:
            if cache is not None:
                keys, values = cache.update_and_fetch(keys.contiguous(), values.contiguous())
            q = queries.float() if keys.dtype == torch.float32 else queries
            T = keys.shape[2]
            if L == 1:
                mask = None
            else:                                                                       # causal, aligned to the end
                pos = torch.arange(T - L, T, device=x.device)
                mask = torch.arange(T, device=x.device)[None, :] <= pos[:, None]
            out = F.scaled_dot_product_attention(q, keys.to(q.dtype), values.to(q.dtype), attn_mask=mask, scale=self.scale,
                                                 enable_gqa=hq != hkv).to(x.dtype)
        return self.o_proj(out.transpose(1, 2).reshape(B, L, hq * d))


class Block(torch.nn.Module):
    def __init__(self, args: ModelArgs, dtype, device):
        super().__init__()
        kw = dict(bias=False, dtype=dtype, device=device)
        self.eps = args.rms_norm_eps
        self.self_attn = Attention(args, dtype, device)
        self.gate_up_proj = torch.nn.Linear(args.hidden_size, 2 * args.intermediate_size, **kw)
        self.down_proj = torch.nn.Linear(args.intermediate_size, args.hidden_size, **kw)
        self.input_layernorm = torch.nn.Parameter(torch.ones(args.hidden_size, dtype=dtype, device=device))
        self.post_attention_layernorm = torch.nn.Parameter(torch.ones(args.hidden_size, dtype=dtype, device=device))

    def forward(self, x, cache=None, packed=True, rope_memo=None):
        h = x + self.self_attn(_rms_norm(x, self.input_layernorm, self.eps), cache, packed, rope_memo)
        gate, up = self.gate_up_proj(_rms_norm(h, self.post_attention_layernorm, self.eps)).chunk(2, dim=-1)
        return h + self.down_proj(F.silu(gate) * up)


class LlamaShaped(torch.nn.Module):
    """Random-init decoder with Llama-3.1 structure; ``model(tokens, cache=[...])`` like an mlx-lm model."""

    def __init__(self, args: ModelArgs | None = None, dtype=torch.bfloat16, device="cuda", seed: int = 0, std: float = 0.02):
        super().__init__()
        self.args = args or ModelArgs()
        a = self.args
        self.embed_tokens = torch.nn.Embedding(a.vocab_size, a.hidden_size, dtype=dtype, device=device)
        self.layers = torch.nn.ModuleList(Block(a, dtype, device) for _ in range(a.num_hidden_layers))
        self.norm = torch.nn.Parameter(torch.ones(a.hidden_size, dtype=dtype, device=device))
        self.lm_head = torch.nn.Linear(a.hidden_size, a.vocab_size, bias=False, dtype=dtype, device=device)
        g = torch.Generator(device=device).manual_seed(seed)
        with torch.no_grad():
            for p in self.parameters():
                if p.dim() > 1:
                    p.normal_(0.0, std, generator=g)

    def make_cache(self):
        """Default (uncompressed) caches; ``apply_turboquant`` replaces this on the instance."""
        from .patch import KVCache
        return [KVCache() for _ in self.layers]

    @torch.no_grad()
    def forward(self, tokens: torch.Tensor, cache=None, packed: bool = True, last_only: bool = False) -> torch.Tensor:
        h = self.embed_tokens(tokens)
        rope_memo = {}
        for i, layer in enumerate(self.layers):
            h = layer(h, cache[i] if cache is not None else None, packed, rope_memo)
        if last_only:
            h = h[:, -1:]
        return self.lm_head(_rms_norm(h, self.norm, self.args.rms_norm_eps))


@torch.no_grad()
def generate(model: LlamaShaped, prompt: torch.Tensor, max_new_tokens: int, cache=None, packed: bool = True,
             prefill_chunk: int = 0) -> torch.Tensor:
    """Greedy decoding: prefill ``prompt`` (B, T), then one token per step; returns (B, max_new_tokens).

    ``prefill_chunk`` > 0 feeds the prompt in pieces of that many tokens (bounded activation memory).
    """
    cache = cache if cache is not None else model.make_cache()
    T = prompt.shape[1]
    step = prefill_chunk if prefill_chunk > 0 else T
    logits = None
    for s in range(0, T, step):
        logits = model(prompt[:, s:s + step], cache=cache, packed=packed, last_only=True)
    out = []
    tok = logits[:, -1].argmax(-1, keepdim=True)
    for i in range(max_new_tokens):
        out.append(tok)
        if i + 1 < max_new_tokens:
            tok = model(tok, cache=cache, packed=packed, last_only=True)[:, -1].argmax(-1, keepdim=True)
    return torch.cat(out, dim=1)


class GraphedDecoder:
    """Greedy one-token-per-sequence decoding with the torch part of the step replayed from CUDA graphs.

    A decode step is 32 cache calls with library work in between.  The cache calls stay eager: their launch parameters
    (lengths, split plan, which buffer a token joins, whether a chunk is due for compression) are host-side state that
    changes from step to step.  Everything between two of them - output projection, SwiGLU, the next layer's norm,
    projections and RoPE; embedding before the first, logits and arg-max after the last - has fixed shapes and reads its
    position from a device tensor, so each such piece is captured once and replayed: per step ``layers + 1`` graph
    launches and ``layers`` cache calls instead of some twenty eager launches per layer.  Same arithmetic, same order, as
    ``model(tok, cache=caches, packed=True)``.
    """

    def __init__(self, model: LlamaShaped, caches: list, first_tokens: torch.Tensor):
        a = model.args
        self.model, self.caches = model, caches
        dev, dt = first_tokens.device, model.lm_head.weight.dtype
        B = first_tokens.shape[0]
        hq, hkv, d = a.num_attention_heads, a.num_key_value_heads, a.head_dim
        self.tok = first_tokens.clone().reshape(B, 1)
        self.pos = torch.full((1,), float(caches[0].offset), dtype=torch.float32, device=dev)
        self.h = torch.empty(B, 1, a.hidden_size, dtype=dt, device=dev)
        self.q = torch.empty(B, hq, 1, d, dtype=dt, device=dev)
        self.k = torch.empty(B, hkv, 1, d, dtype=dt, device=dev)
        self.v = torch.empty(B, hkv, 1, d, dtype=dt, device=dev)
        self.attn = torch.zeros(B, hq, 1, d, dtype=dt, device=dev)
        half = d // 2
        self._inv = a.rope_theta ** (-torch.arange(0, half, device=dev, dtype=torch.float32) / half)
        n = len(model.layers)
        pieces = [self._piece(i) for i in range(n + 1)]
        # warm up on a side stream (library handles, autotuning), then capture each piece
        side = torch.cuda.Stream(device=dev)
        side.wait_stream(torch.cuda.current_stream(dev))
        saved = (self.tok.clone(), self.pos.clone())
        with torch.cuda.stream(side):
            for _ in range(2):
                for f in pieces:
                    f()
        torch.cuda.current_stream(dev).wait_stream(side)
        self.graphs = []
        pool = None
        for f in pieces:
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, pool=pool):
                f()
            pool = pool or g.pool()
            self.graphs.append(g)
        self.tok.copy_(saved[0])
        self.pos.copy_(saved[1])

    def _pre_attention(self, i: int, h: torch.Tensor) -> None:
        m, a = self.model, self.model.args
        att = m.layers[i].self_attn
        hq, hkv, d = att.n_heads, att.n_kv_heads, att.head_dim
        B = h.shape[0]
        qkv = att.qkv_proj(_rms_norm(h, m.layers[i].input_layernorm, a.rms_norm_eps)).view(B, 1, hq + 2 * hkv, d).transpose(1, 2)
        ang = self.pos[:, None] * self._inv[None, :]                                  # (1, d/2): this step's position
        cos, sin = ang.cos(), ang.sin()
        qk = apply_rope(qkv[:, :hq + hkv], (torch.cat([cos, cos], dim=-1), torch.cat([-sin, sin], dim=-1)))
        self.q.copy_(qk[:, :hq])
        self.k.copy_(qk[:, hq:])
        self.v.copy_(qkv[:, hq + hkv:])

    def _post_attention(self, i: int) -> torch.Tensor:
        m, a = self.model, self.model.args
        layer = m.layers[i]
        B = self.attn.shape[0]
        h = self.h + layer.self_attn.o_proj(self.attn.transpose(1, 2).reshape(B, 1, -1))
        gate, up = layer.gate_up_proj(_rms_norm(h, layer.post_attention_layernorm, a.rms_norm_eps)).chunk(2, dim=-1)
        return h + layer.down_proj(F.silu(gate) * up)

    def _piece(self, i: int):
        m, n = self.model, len(self.model.layers)

        def first():
            h = m.embed_tokens(self.tok)
            self.h.copy_(h)
            self._pre_attention(0, h)

        def middle():
            h = self._post_attention(i - 1)
            self.h.copy_(h)
            self._pre_attention(i, h)

        def last():
            h = self._post_attention(n - 1)
            logits = m.lm_head(_rms_norm(h, m.norm, m.args.rms_norm_eps))
            self.tok.copy_(logits[:, -1].argmax(-1, keepdim=True))
            self.pos.add_(1.0)

        return first if i == 0 else last if i == n else middle

    @torch.no_grad()
    def step(self) -> torch.Tensor:
        """Feeds ``self.tok`` (B, 1) through the model and the caches and leaves the next greedy token there (returned too;
        the same tensor every step - clone it to keep it)."""
        scale = self.model.layers[0].self_attn.scale
        for i, c in enumerate(self.caches):
            self.graphs[i].replay()
            c.decode_step(self.q, self.k, self.v, scale, out=self.attn)
        self.graphs[-1].replay()
        return self.tok
