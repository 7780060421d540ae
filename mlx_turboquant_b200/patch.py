"""Model patching: give every attention layer of a model a TurboQuant cache (reference: mlx_turboquant/patch.py).

The reference walks mlx-lm modules; this version applies the same rules to any Python model object
that exposes its configuration the usual way (``model.args`` / ``model.config`` / nested
``language_model``) and whose attention layers call ``cache.update_and_fetch`` (dense) or
``cache.update`` + ``cache.attend`` (packed).  ``model.make_cache()`` then returns one cache per layer.
"""

from __future__ import annotations

import warnings

import torch

from .cache import TurboQuantKVCache


class KVCache:
    """Plain uncompressed cache for layers that are skipped (stands in for mlx-lm's ``KVCache``)."""

    step = 256

    def __init__(self):
        self.keys = self.values = None
        self.offset = 0

    def update_and_fetch(self, keys, values):
        if self.keys is None:
            self.keys, self.values = keys, values
        else:
            self.keys = torch.cat([self.keys, keys], dim=2)
            self.values = torch.cat([self.values, values], dim=2)
        self.offset = self.keys.shape[2]
        return self.keys, self.values

    def update(self, keys, values):
        self.update_and_fetch(keys, values)

    def attend(self, queries, scale=None):
        """Causal attention of the last ``T_q`` positions over everything stored (float32 arithmetic)."""
        d, tq = queries.shape[-1], queries.shape[2] if queries.dim() == 4 else 1
        q = queries.reshape(queries.shape[0], queries.shape[1], tq, d).float()
        rep = q.shape[1] // self.keys.shape[1]
        k = self.keys.float().repeat_interleave(rep, dim=1)
        v = self.values.float().repeat_interleave(rep, dim=1)
        s = (q @ k.transpose(-1, -2)) * (d ** -0.5 if scale is None else scale)
        if tq > 1:
            t = k.shape[2]
            pos = torch.arange(t - tq, t, device=s.device)
            s = s.masked_fill(torch.arange(t, device=s.device)[None, :] > pos[:, None], float("-inf"))
        return (torch.softmax(s, dim=-1) @ v).to(queries.dtype).reshape(queries.shape)

    def decode_step(self, queries, keys, values, scale=None):
        self.update(keys, values)
        return self.attend(queries, scale)

    def make_mask(self, N, offset=0, return_array=False, window_size=None):
        return None if N == 1 and not return_array else "causal"

    def size(self):
        return self.offset

    def empty(self):
        return self.keys is None

    def is_trimmable(self):
        return True


def _candidates(model):
    lm = getattr(model, "language_model", None)
    return [getattr(model, "model", model), model, lm, getattr(lm, "model", None)]


def _get_model_config(model) -> dict:
    """head_dim / num_kv_heads / num_layers from the model's config object (patch.py:13-86)."""
    args = None
    for path in _candidates(model):
        if path is None:
            continue
        for name in ("args", "config"):
            cand = getattr(path, name, None)
            if cand is not None and getattr(cand, "hidden_size", None) is not None:
                args = cand
                break
        if args is not None:
            break
    if args is not None:
        head_dim = getattr(args, "head_dim", None)
        num_kv_heads = getattr(args, "num_key_value_heads", None)
        num_heads = getattr(args, "num_attention_heads", None)
        hidden_size = getattr(args, "hidden_size", None)
        num_layers = getattr(args, "num_hidden_layers", None)
        if head_dim is None and hidden_size is not None and num_heads is not None:
            head_dim = hidden_size // num_heads
        if num_kv_heads is None:
            num_kv_heads = getattr(args, "num_kv_heads", num_heads)
        if num_layers is None:
            for cand in _candidates(model):
                layers = getattr(cand, "layers", None) if cand is not None else None
                if layers is not None and len(layers) > 0:
                    num_layers = len(layers)
                    break
        return {"head_dim": head_dim or 128, "num_kv_heads": num_kv_heads or 1, "num_layers": num_layers or 1}
    inner = getattr(model, "model", model)
    layers = getattr(inner, "layers", None)
    if layers is not None and len(layers) > 0:
        attn = getattr(layers[0], "self_attn", getattr(layers[0], "attention", None))
        k_proj = getattr(attn, "k_proj", None) if attn is not None else None
        if k_proj is not None:
            nkv = getattr(attn, "n_kv_heads", getattr(attn, "num_kv_heads", 1))
            return {"head_dim": k_proj.weight.shape[0] // nkv, "num_kv_heads": nkv, "num_layers": len(layers)}
    raise ValueError("Could not determine model configuration. Please specify head_dim and num_kv_heads manually.")


def detect_outlier_layers(model, threshold: float = 3.0) -> list[int]:
    """Layers whose largest key norm exceeds ``threshold`` x the median stay uncompressed (patch.py:89-133).

    Runs a five-token forward pass ``model(tokens, cache=[KVCache()...])`` like the reference does.
    """
    inner = getattr(model, "model", model)
    layers = getattr(inner, "layers", [])
    cache = [KVCache() for _ in range(len(layers))]
    try:
        dev = next(model.parameters()).device
    except (AttributeError, StopIteration, TypeError):
        dev = "cpu"
    model(torch.tensor([[0, 1, 2, 3, 4]], device=dev), cache=cache)
    max_norms = []
    for c in cache:
        max_norms.append(float(torch.linalg.vector_norm(c.keys.float(), dim=-1).max()) if c.keys is not None else 0.0)
    positive = sorted(n for n in max_norms if n > 0)
    if not positive:
        return []
    mid = len(positive) // 2
    median = positive[mid] if len(positive) % 2 else 0.5 * (positive[mid - 1] + positive[mid])
    return [i for i, n in enumerate(max_norms) if n > threshold * median]


def _is_sliding_window_cache(c) -> bool:
    return "Rotating" in type(c).__name__ or getattr(c, "is_sliding_window", False)


def apply_turboquant(model, key_bits: float = 4, value_bits: float = 2, residual_window: int = 128,
                     head_dim: int | None = None, num_kv_heads: int | None = None, num_layers: int | None = None,
                     rotation_seed: int = 42, skip_layers: list[int] | None = None, auto_detect_outliers: bool = True,
                     fp16_sink_size: int = 0, chunk_size: int = 0, qjl_correction: bool = False, qjl_n_proj: int = 32):
    """Make ``model.make_cache()`` return TurboQuant caches (patch.py:136-371); returns the same model.

    Arguments and defaults are the reference's.  Layers listed in ``skip_layers`` (or auto-detected as
    outliers), linear-attention layers and sliding-window layers keep an uncompressed / model-default cache.
    """
    config = _get_model_config(model)
    hd = head_dim or config["head_dim"]
    nkv = num_kv_heads or config["num_kv_heads"]
    nl = num_layers or config["num_layers"]

    if nkv <= 2 and key_bits < 4:   # few KV heads are more sensitive (patch.py:198-217)
        old, key_bits = key_bits, 4
        warnings.warn(f"Model has only {nkv} KV heads — upgrading key_bits {old} → {key_bits} for stability. "
                      f"Effective config: key_bits={key_bits}, value_bits={value_bits}.", UserWarning, stacklevel=2)
    if nkv <= 2 and value_bits < 3:
        old, value_bits = value_bits, 3
        warnings.warn(f"Model has only {nkv} KV heads — upgrading value_bits {old} → {value_bits} for stability. "
                      f"Effective config: key_bits={key_bits}, value_bits={value_bits}.", UserWarning, stacklevel=2)

    layers_to_skip = set(skip_layers or [])
    if auto_detect_outliers and not skip_layers:
        try:
            layers_to_skip = set(detect_outlier_layers(model))
        except Exception:
            pass   # detection is best-effort: compress every layer

    inner = getattr(model, "model", model)
    raw_layers = getattr(inner, "layers", None)
    if raw_layers is None:
        raw_layers = getattr(model, "layers", []) or []
    linear_attn_layers = set()
    for i, layer in enumerate(raw_layers):
        if hasattr(layer, "linear_attn") or hasattr(layer, "linear_attention"):
            if not (hasattr(layer, "self_attn") or hasattr(layer, "attention")):
                linear_attn_layers.add(i)
    if linear_attn_layers:
        warnings.warn(f"Detected {len(linear_attn_layers)} linear-attention layers in model (hybrid architecture). "
                      "These layers will use the model's default cache type instead of TurboQuantKVCache.",
                      UserWarning, stacklevel=2)

    class_level_make_cache = getattr(type(model), "make_cache", None)

    def _build_default_caches():
        if class_level_make_cache is not None:
            return class_level_make_cache(model)
        return [KVCache() for _ in range(nl)]

    swa_layers: set[int] = set()
    try:
        for i, c in enumerate(_build_default_caches()):
            if i not in linear_attn_layers and _is_sliding_window_cache(c):
                swa_layers.add(i)
    except Exception:
        pass
    if swa_layers:
        warnings.warn(f"Detected {len(swa_layers)} sliding-window-attention layers in model. These layers will use "
                      "the model's default cache type instead of TurboQuantKVCache.", UserWarning, stacklevel=2)

    default_cache_layers = linear_attn_layers | swa_layers

    def make_cache():
        defaults = _build_default_caches() if default_cache_layers else None
        caches = []
        for i in range(nl):
            if i in default_cache_layers:
                caches.append(defaults[i])
            elif i in layers_to_skip:
                caches.append(KVCache())
            else:
                caches.append(TurboQuantKVCache(
                    head_dim=hd, num_kv_heads=nkv, key_bits=key_bits, value_bits=value_bits,
                    residual_window=residual_window, rotation_seed=rotation_seed, fp16_sink_size=fp16_sink_size,
                    chunk_size=chunk_size, qjl_correction=qjl_correction, qjl_n_proj=qjl_n_proj))
        return caches

    model.make_cache = make_cache
    model._turboquant_config = {
        "head_dim": hd, "num_kv_heads": nkv, "num_layers": nl, "key_bits": key_bits, "value_bits": value_bits,
        "residual_window": residual_window, "fp16_sink_size": fp16_sink_size, "chunk_size": chunk_size,
        "qjl_correction": qjl_correction, "qjl_n_proj": qjl_n_proj,
    }
    return model


def enable_turboquant(model, bits: int = 4, **kwargs):
    """Same bit width for keys and values (patch.py:374-385)."""
    return apply_turboquant(model, key_bits=bits, value_bits=bits, **kwargs)
