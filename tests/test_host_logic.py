"""Host-side behaviour that needs no GPU: cache protocol surface, codebook host code, model patching."""

import types
import warnings

import numpy as np
import pytest


def test_public_surface():
    """Reference tests/test_smoke.py:43-71."""
    import mlx_turboquant_b200 as m
    assert set(m.__all__) == {"__version__", "apply_turboquant", "enable_turboquant", "TurboQuantKVCache",
                              "TurboQuantMSE", "TurboQuantProd"}
    for name in ("update_and_fetch", "make_mask", "state", "meta_state", "empty", "is_trimmable", "size", "nbytes",
                 "step", "update", "attend"):
        assert hasattr(m.TurboQuantKVCache, name)
    from mlx_turboquant_b200 import kernels, rotation
    for name in ("fused_qk_scores_2bit", "fused_qk_scores_3bit", "fused_qk_scores_4bit", "metal_dequantize",
                 "metal_quantize_4bit"):
        assert callable(getattr(kernels, name))
    assert callable(rotation.pre_rotate_query)


def test_cache_constructor_and_protocol_without_gpu():
    from mlx_turboquant_b200 import TurboQuantKVCache
    c = TurboQuantKVCache(head_dim=128, num_kv_heads=8, key_bits=3.5, value_bits=2, fp16_sink_size=128, chunk_size=4096)
    assert c.step == 256 and c.offset == 0 and c.empty() and not c.is_trimmable() and c.size() == 0 and c.nbytes == 0
    assert c._k_fractional and not c._v_fractional and (c._k.bits_hi, c._k.bits_lo) == (4, 3)
    assert c.make_mask(1) is None and c.make_mask(5) == "causal" and c.make_mask(1, return_array=True) == "causal"
    with pytest.raises(NotImplementedError):
        c.make_mask(4, window_size=16)
    m = c.meta_state
    assert m["key_bits"] == "3.5" and m["fp16_sink_size"] == "128" and all(isinstance(v, str) for v in m.values())
    c.meta_state = dict(m, offset="77", compressed_len="10", sink_len="3", fp16_len="5", fp16_capacity="300")
    assert (c.offset, c._compressed_len, c._sink_len, c._fp16_len, c._fp16_capacity) == (77, 10, 3, 5, 300)
    assert len(c.state) == 10
    with pytest.raises(ValueError):
        c.state = (None,) * 7
    assert TurboQuantKVCache(qjl_correction=False)._qjl_projection is None
    with pytest.raises(NotImplementedError):
        TurboQuantKVCache(qjl_correction=True, qjl_n_proj=64)


def test_host_codebooks_match_shipped_tables(tables):
    from mlx_turboquant_b200.codebook import compute_theoretical_mse, get_codebook_host, lloyd_max
    for (d, b), (c, bd) in tables.items():
        hc, hb = get_codebook_host(d, b)
        assert np.array_equal(hc, c) and np.array_equal(hb, bd)
        assert hc.shape == (1 << b,) and hb.shape == ((1 << b) - 1,) and np.all(np.diff(hc) > 0)
        np.testing.assert_allclose(hc, -hc[::-1], atol=1e-3)                    # symmetric
    c, bd = lloyd_max(128, 3)                                                   # recomputed == shipped centroids
    assert np.array_equal(c, tables[(128, 3)][0])
    for b in (2, 3, 4):                                                         # within 3x of 4^-b per unit vector
        c, bd = tables[(128, b)]
        assert compute_theoretical_mse(128, b, c, bd) * 128 < 3.0 * 4.0 ** -b
    c, bd = lloyd_max(16, 2)                                                    # Beta branch for small d
    assert c.shape == (4,) and np.all(np.diff(c) > 0)


def test_codebook_cache_location(tmp_path, monkeypatch):
    """Reference tests/test_edge_cases.py:293-322."""
    from mlx_turboquant_b200 import codebook
    monkeypatch.setenv("XDG_CACHE_HOME", str(tmp_path))
    codebook._host_cache.pop((48, 2), None)
    c, b = codebook.get_codebook_host(48, 2)
    assert (tmp_path / "mlx_turboquant" / "codebook_d48_b2.npz").exists() and c.shape == (4,)
    codebook.precompute_codebooks(dims=(40,), bits_range=(2,), target_dir=tmp_path / "x")
    assert (tmp_path / "x" / "codebook_d40_b2.npz").exists()


def test_host_rotation_and_projection(golden):
    from mlx_turboquant_b200.qjl import generate_projection_matrix_host
    from mlx_turboquant_b200.rotation import generate_rotation_matrix_host
    assert np.array_equal(generate_rotation_matrix_host(64, 42), golden["rot_d64_full"])
    assert np.array_equal(generate_rotation_matrix_host(64, 7), golden["rot_d64_seed7"])
    assert np.array_equal(generate_projection_matrix_host(96, 32), golden["proj_m32_d96"])
    from mlx_turboquant_b200.kernels import packed_widths, split_bits
    assert split_bits(3.5) == (4, 3) and split_bits(4) == (4, 0) and split_bits(2.5) == (3, 2)
    assert packed_widths(128, 4, 3) == (32, 24) and packed_widths(96, 3, 0) == (36, 0) and packed_widths(128, 2, 0) == (32, 0)


# ---- model patching (reference tests/test_edge_cases.py:328-643) ---------------------------------------
class _Args:
    def __init__(self, **kw):
        self.__dict__.update(kw)


def _fake_model(n_layers=4, **args):
    inner = types.SimpleNamespace(layers=[types.SimpleNamespace(self_attn=object()) for _ in range(n_layers)],
                                  args=_Args(**args))
    class M:   # noqa: D401 - plain container
        pass
    m = M()
    m.model = inner
    return m


def test_apply_turboquant_builds_per_layer_caches():
    from mlx_turboquant_b200 import TurboQuantKVCache, apply_turboquant, enable_turboquant
    from mlx_turboquant_b200.patch import KVCache
    m = _fake_model(hidden_size=4096, num_attention_heads=32, num_key_value_heads=8, num_hidden_layers=4)
    out = apply_turboquant(m, key_bits=4, value_bits=2, skip_layers=[1], fp16_sink_size=128, chunk_size=4096,
                           qjl_correction=False, residual_window=64)
    assert out is m
    caches = m.make_cache()
    assert len(caches) == 4 and isinstance(caches[1], KVCache)
    for i in (0, 2, 3):
        c = caches[i]
        assert isinstance(c, TurboQuantKVCache) and (c.head_dim, c.num_kv_heads) == (128, 8)
        assert (c.key_bits, c.value_bits, c.residual_window, c.fp16_sink_size, c.chunk_size) == (4, 2, 64, 128, 4096)
    assert m._turboquant_config == {"head_dim": 128, "num_kv_heads": 8, "num_layers": 4, "key_bits": 4, "value_bits": 2,
                                    "residual_window": 64, "fp16_sink_size": 128, "chunk_size": 4096,
                                    "qjl_correction": False, "qjl_n_proj": 32}
    enable_turboquant(m, bits=3, auto_detect_outliers=False)
    assert all(c.key_bits == 3 and c.value_bits == 3 for c in m.make_cache())


def test_apply_turboquant_low_kv_head_upgrade_warns():
    from mlx_turboquant_b200 import apply_turboquant
    m = _fake_model(hidden_size=2048, num_attention_heads=16, num_key_value_heads=2, num_hidden_layers=2)
    with warnings.catch_warnings(record=True) as w:
        warnings.simplefilter("always")
        apply_turboquant(m, key_bits=3, value_bits=2, auto_detect_outliers=False)
    assert len([x for x in w if issubclass(x.category, UserWarning)]) == 2
    assert m._turboquant_config["key_bits"] == 4 and m._turboquant_config["value_bits"] == 3


def test_model_config_fallbacks():
    from mlx_turboquant_b200.patch import _get_model_config
    m = _fake_model(hidden_size=1024, num_attention_heads=8, num_hidden_layers=None, num_key_value_heads=None)
    assert _get_model_config(m) == {"head_dim": 128, "num_kv_heads": 8, "num_layers": 4}
    m = _fake_model(hidden_size=1024, num_attention_heads=8, num_hidden_layers=3, num_key_value_heads=2, head_dim=64)
    assert _get_model_config(m) == {"head_dim": 64, "num_kv_heads": 2, "num_layers": 3}
    with pytest.raises(ValueError):
        _get_model_config(types.SimpleNamespace())


def test_hybrid_and_sliding_window_layers_keep_model_default_cache():
    from mlx_turboquant_b200 import TurboQuantKVCache, apply_turboquant

    class RotatingKVCache:
        pass

    class LinearState:
        pass

    class Model:
        def __init__(self):
            layers = [types.SimpleNamespace(self_attn=object()), types.SimpleNamespace(linear_attn=object()),
                      types.SimpleNamespace(self_attn=object()), types.SimpleNamespace(self_attn=object())]
            self.model = types.SimpleNamespace(layers=layers, args=_Args(hidden_size=512, num_attention_heads=8,
                                                                         num_key_value_heads=4, num_hidden_layers=4))

        def make_cache(self):
            return [object(), LinearState(), RotatingKVCache(), object()]

    m = Model()
    with warnings.catch_warnings(record=True) as w:
        warnings.simplefilter("always")
        apply_turboquant(m, auto_detect_outliers=False)
    assert len(w) == 2
    caches = m.make_cache()
    assert isinstance(caches[0], TurboQuantKVCache) and isinstance(caches[1], LinearState)
    assert isinstance(caches[2], RotatingKVCache) and isinstance(caches[3], TurboQuantKVCache)


def test_detect_outlier_layers_on_cpu_model():
    import torch
    from mlx_turboquant_b200.patch import detect_outlier_layers

    class Tiny:
        def __init__(self, scales):
            self.model = types.SimpleNamespace(layers=[None] * len(scales))
            self.scales = scales

        def __call__(self, tokens, cache):
            for c, s in zip(cache, self.scales):
                k = torch.ones(1, 2, tokens.shape[1], 8) * s
                c.update_and_fetch(k, k)

    assert detect_outlier_layers(Tiny([1.0, 1.0, 10.0, 1.0])) == [2]
    assert detect_outlier_layers(Tiny([0.0, 0.0])) == []


def test_library_calls_run_with_the_tensors_device_current(monkeypatch):
    """A cache on cuda:1 used while cuda:0 is current: the launch helper makes cuda:1 current around the call (the
    library launches on the current device).  Faked: no GPU is touched."""
    import contextlib

    import torch

    from mlx_turboquant_b200 import _lib
    state = {"current": 0, "seen": []}

    class FakeLib:
        def tq_pack(self, *args):
            state["seen"].append((state["current"], args))
            return 0

    @contextlib.contextmanager
    def fake_device(idx):
        prev, state["current"] = state["current"], idx
        try:
            yield
        finally:
            state["current"] = prev

    monkeypatch.setattr(_lib, "lib", lambda: FakeLib())
    monkeypatch.setattr(torch.cuda, "current_device", lambda: state["current"])
    monkeypatch.setattr(torch.cuda, "device", fake_device)
    assert _lib.launch(torch.device("cuda", 1), "tq_pack", 1, 2) == 0
    assert _lib.launch(torch.device("cuda", 0), "tq_pack", 3) == 0
    assert _lib.launch(torch.device("cuda"), "tq_pack", 4) == 0            # no index: the current device
    assert [s[0] for s in state["seen"]] == [1, 0, 0] and state["current"] == 0


def test_cpu_tensors_are_refused_before_any_launch():
    """`cache.state = <checkpoint loaded on the CPU>` and CPU inputs raise instead of reaching a kernel."""
    import torch

    from mlx_turboquant_b200 import TurboQuantKVCache, _lib, kernels
    c = TurboQuantKVCache(head_dim=128, num_kv_heads=2)
    cpu_state = (torch.zeros(1, 2, 8, 128, dtype=torch.float16), torch.zeros(1, 2, 8, 128, dtype=torch.float16),
                 torch.zeros(1, 2, 16, 64, dtype=torch.uint8), torch.zeros(1, 2, 16), torch.zeros(1, 2, 16, 32, dtype=torch.uint8),
                 torch.zeros(1, 2, 16))
    c._dargs, c._dargs_key, c._ws_key = object(), ("stale",), ("stale",)
    with pytest.raises(RuntimeError, match="CUDA tensors only"):
        c.state = cpu_state
    assert c._k.hi is None and c.keys is None                                # nothing was adopted
    c.state = (None,) * 6                                                     # an empty state is fine and drops the cached arguments
    assert c._dargs is None and c._dargs_key is None and c._ws_key is None
    with pytest.raises(RuntimeError, match="CUDA tensors only"):
        c.update(torch.zeros(1, 2, 1, 128), torch.zeros(1, 2, 1, 128))
    with pytest.raises(RuntimeError, match="CUDA tensors only"):
        c.attend(torch.zeros(1, 8, 1, 128))
    with pytest.raises(RuntimeError, match="CUDA tensors only"):
        kernels.quantize_pack(torch.zeros(4, 128), torch.eye(128), torch.zeros(15), 4)
    with pytest.raises(RuntimeError, match="CUDA tensors only"):
        TurboQuantKVCache._append(torch.zeros(1, 2, 8, 128), torch.zeros(1, 2, 8, 128), torch.zeros(1, 2, 1, 128), torch.zeros(1, 2, 1, 128), 0)
    assert _lib.require_cuda(None, None) is None


def test_gather_slot_ledger():
    from mlx_turboquant_b200.sharding import SlotLedger
    with pytest.raises(ValueError):
        SlotLedger(2, 1)
    with pytest.raises(ValueError):
        SlotLedger(1, 0)
    one = SlotLedger(1, 1)                    # a single rank has no peer to race with
    one.use(0); one.use(0)
    led = SlotLedger(4, 3)
    led.use(0); led.use(1); led.use(0); led.use(2)
    with pytest.raises(RuntimeError, match="alternate"):
        led.use(2)
    with pytest.raises(IndexError):
        led.use(3)
