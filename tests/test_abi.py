"""The C-ABI library loads on a machine without a GPU and exports every symbol the header declares."""
import ctypes
import re
from pathlib import Path

ROOT = Path(__file__).resolve().parents[1]


def _declared_symbols():
    text = (ROOT / "include" / "rfa_b200.h").read_text() + (ROOT / "include" / "rfa_b200_debug.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(rfa_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    from opt_ring_flash_attn_b200 import _native, build

    build.build()
    lib = ctypes.CDLL(str(_native.library_path()))
    names = _declared_symbols()
    assert len(names) >= 12
    for n in names:
        assert hasattr(lib, n), f"{n} is declared in include/*.h but not exported"
    # the ctypes binding covers the same set
    assert set(_native.SIGNATURES) == set(names)


def test_pure_host_entry_points():
    from opt_ring_flash_attn_b200 import _native

    lib = _native.load()
    assert lib.rfa_version() >= 100
    assert lib.rfa_seq_tile() == 128
    assert lib.rfa_fwd_acc_elems(1, 200, 4, 96) == 1 * 4 * 256 * 128
    assert lib.rfa_dq_acc_elems(2, 128, 2, 256) == 2 * 2 * 128 * 256
    assert lib.rfa_fwd_acc_elems(1, 128, 2, 100) == 0  # head dim not a multiple of 8
    assert lib.rfa_noalloc_scratch_bytes() == 32 * 1024 * 1024


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    from opt_ring_flash_attn_b200 import _native
    import pytest

    monkeypatch.setattr(_native, "_lib", None)
    monkeypatch.setattr(_native, "_LIB_PATH", tmp_path / "nope.so")
    with pytest.raises(RuntimeError, match="no non-CUDA fallback"):
        _native.load()


def test_cpu_tensors_are_refused():
    import pytest
    import torch
    from opt_ring_flash_attn_b200 import ring_flash_attn

    q = torch.zeros(1, 128, 2, 64, dtype=torch.bfloat16)
    with pytest.raises(RuntimeError, match="CUDA tensors only"):
        ring_flash_attn(q, q, q)
