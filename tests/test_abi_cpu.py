"""CPU-side checks of the C-ABI boundary: the library loads and exports every symbol that
include/stbpe.h declares (no compute calls: there is no GPU here)."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_symbols():
    text = open(os.path.join(ROOT, "include", "stbpe.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(stbpe_[a-z0-9_]+)\s*\(", text)))


def test_header_declares_symbols():
    syms = _declared_symbols()
    assert "stbpe_train" in syms and "stbpe_count_initial" in syms and len(syms) >= 20


def test_library_exports_every_declared_symbol():
    from supertoken_b200 import _lib
    lib = _lib.load()
    for name in _declared_symbols():
        assert hasattr(lib, name), f"{name} declared in stbpe.h but not exported"
        assert name in _lib.SIGNATURES, f"{name} has no ctypes signature"
    assert set(_lib.SIGNATURES) == set(_declared_symbols())
    assert lib.stbpe_version().startswith(b"stbpe")


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    from supertoken_b200 import _lib
    monkeypatch.setattr(_lib, "_lib", None)
    monkeypatch.setattr(_lib, "LIB_PATH", str(tmp_path / "nope.so"))
    with pytest.raises(ImportError, match="no CPU fallback"):
        _lib.load()


def test_trainer_refuses_cpu_device():
    from supertoken_b200 import GPUBPETrainer
    with pytest.raises(RuntimeError, match="CUDA devices only"):
        GPUBPETrainer(device="cpu")


def test_create_rejects_bad_config_without_gpu_work():
    from supertoken_b200 import _lib
    lib = _lib.load()
    h = ctypes.c_void_p()
    cfg = _lib.Config(0, 256, -5, 0, 10, 1, 0, 0)
    assert lib.stbpe_create(ctypes.byref(h), ctypes.byref(cfg)) == _lib.E_BADARG
    cfg = _lib.Config(0, 0x7FFFFFF0, 10, 0, 100, 1, 0, 0)
    assert lib.stbpe_create(ctypes.byref(h), ctypes.byref(cfg)) == _lib.E_ID_OVERFLOW
    assert b"overflow" in lib.stbpe_last_error(None)
