"""The C-ABI shared library loads and exports every symbol include/tq_abi.h declares (no GPU needed)."""

import ctypes
import re
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent


@pytest.fixture(scope="module")
def built():
    import __graft_entry__ as g
    g.build()
    from mlx_turboquant_b200 import _lib
    return _lib


def test_header_symbols_are_exported(built):
    header = (ROOT / "include" / "tq_abi.h").read_text()
    declared = set(re.findall(r"^\s*(?:const\s+)?[\w\*]+\s+\*?(tq_\w+)\s*\(", header, flags=re.M))
    assert {"tq_version", "tq_pack", "tq_unpack", "tq_quantize_pack", "tq_dequantize", "tq_decode_attn",
            "tq_qk_scores", "tq_rotate", "tq_quantize_from_rotated", "tq_decode_workspace_bytes"} <= declared
    handle = ctypes.CDLL(str(built.LIB_PATH))
    for name in declared:
        assert hasattr(handle, name), f"{name} declared in tq_abi.h but not exported"
    assert declared == set(built.PROTOTYPES), "ctypes prototypes and header disagree"


def test_version_and_argument_errors_without_gpu(built):
    lib = built.lib()
    assert lib.tq_version() == 2
    # argument validation happens on the host before any CUDA call
    assert lib.tq_pack(None, None, 4, 128, 5, None) == -1
    assert b"Unsupported bit-width: 5" in lib.tq_last_error()
    assert lib.tq_pack(None, None, 4, 6, 3, None) == -1
    assert lib.tq_unpack(None, None, 4, 128, 0, None) == -1
    assert lib.tq_rotate(None, 0, None, None, 4, 100, 0, None) == -2
    assert lib.tq_qk_scores(None, None, None, None, 5, 128, 1, 1, None, None) == -1
    assert lib.tq_pack(None, None, 0, 128, 4, None) == 0          # empty input is a no-op
    assert lib.tq_decode_attn(None, None) == -1
    assert lib.tq_set_tuning(b"nope", 1) == -1
    with pytest.raises(ValueError):
        built.check(-1)
    with pytest.raises(NotImplementedError):
        built.check(-2)


def test_decode_workspace_sizes_without_gpu(built):
    """Pure host arithmetic (the split plans and the streaming kernel's layout for 148 SMs when no device answers): the
    scratch for a call the streaming kernel can take holds its prepared queries and partials on top of the other kernels'
    need; sizes it cannot take (other head dims, no packed tokens) are unaffected; the knobs are accepted."""
    lib = built.lib()
    assert lib.tq_decode_kernel_choice(None) == -1
    c3 = lib.tq_decode_workspace_bytes(16, 32, 32, 96, 7936, 256)        # batch 16, MHA, d = 96
    d64 = lib.tq_decode_workspace_bytes(16, 32, 32, 64, 7936, 256)
    assert c3 > d64 > 0
    # queries: 512 heads x (2 x 96 + 32) halves; partials: 512 lanes x (6 + 4) slots x (96 + 36) floats
    assert c3 >= 65536 + 512 * 224 * 2 + 512 * 10 * 132 * 4
    assert 0 < lib.tq_decode_workspace_bytes(16, 32, 32, 96, 0, 256) < c3                 # only uncompressed tokens: no streaming layout
    assert lib.tq_decode_workspace_bytes(0, 32, 32, 96, 7936, 256) == 0
    for key, good, bad in ((b"decode_stream", 0, 2), (b"decode_stream_min_run", 8, 0), (b"decode_stream_max_parts", 64, 65)):
        assert lib.tq_set_tuning(key, bad) == -1
        assert lib.tq_set_tuning(key, good) == 0
    assert lib.tq_decode_workspace_bytes(16, 32, 32, 96, 7936, 256) == c3    # (the knobs steer the choice, not the size)
    assert lib.tq_set_tuning(b"decode_stream", 1) == 0 and lib.tq_set_tuning(b"decode_stream_min_run", 24) == 0
    assert lib.tq_set_tuning(b"decode_stream_max_parts", 40) == 0


def test_missing_library_fails_loudly(monkeypatch, built):
    monkeypatch.setattr(built, "_lib", None)
    monkeypatch.setattr(built, "LIB_PATH", ROOT / "does_not_exist.so")
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        built.lib()


def test_cpu_tensors_are_rejected(built):
    import torch
    from mlx_turboquant_b200.packing import pack_indices
    with pytest.raises(ValueError):
        pack_indices(torch.zeros(1, 8, dtype=torch.uint8), 5)
    with pytest.raises(AssertionError):
        pack_indices(torch.zeros(1, 6, dtype=torch.uint8), 3)
    with pytest.raises(RuntimeError, match="CUDA tensors only"):
        pack_indices(torch.zeros(1, 8, dtype=torch.uint8), 4)
