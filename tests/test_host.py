"""CPU-only checks: the C-ABI library loads and exports every declared symbol; argument
validation that needs no GPU; the engine's flag handling."""

import ctypes
import os
import re

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared():
    text = open(os.path.join(ROOT, "include", "tybok_b200.h"), encoding="utf-8").read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(tybok_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    from tybok_b200 import _lib, build

    build.build()
    lib = ctypes.CDLL(_lib.LIB_PATH)
    names = _declared()
    assert len(names) >= 10
    for name in names:
        assert hasattr(lib, name), f"{name} declared in include/tybok_b200.h but not exported"
    assert set(_lib.SIGNATURES) == set(names), "ctypes table and header disagree"
    assert _lib.load().tybok_version() >= 100


def test_argument_validation_without_gpu():
    from tybok_b200 import _lib

    lib = _lib.load()
    assert lib.tybok_w8a16_workspace_bytes(50, 2048, 1024, 0) == 3 * 50 * 1024
    # null pointers / bad K are refused before any CUDA call
    assert lib.tybok_split3(None, 8, None, 4, 64, 4, None) == 1
    assert b"null" in lib.tybok_last_error()
    rc = lib.tybok_w8x3_linear(ctypes.c_void_p(16), 4, ctypes.c_void_p(16), ctypes.c_void_p(16), None,
                               ctypes.c_void_p(16), 64, None, 0, 4, 64, 72, 0, None, 0, None, 0, 1, 0, 0, 0, None, None)
    assert rc == 1 and b"multiple of 16" in lib.tybok_last_error()


def test_ops_have_no_cpu_implementation():
    from tybok_b200 import ops

    with pytest.raises(NotImplementedError):
        ops.split3(torch.zeros(4, 64, dtype=torch.bfloat16))
    with pytest.raises(NotImplementedError):
        ops.rmsnorm(torch.zeros(4, 64, dtype=torch.bfloat16), weight=torch.zeros(64))


def test_engine_refuses_cpu_and_foreign_flags():
    from tybok_b200.engine import PI05B200Engine

    with pytest.raises(RuntimeError, match="no CPU fallback"):
        PI05B200Engine("synthetic:pi05_tiny", device="cpu")
    with pytest.raises(NotImplementedError, match="tl-fp8-expert-mlp"):
        PI05B200Engine("synthetic:pi05_tiny", device="cpu", tl_fp8_expert_mlp=True)
    with pytest.raises(NotImplementedError, match="compile"):
        PI05B200Engine("synthetic:pi05_tiny", device="cpu", compile_model=True)


def test_registered_under_its_own_key():
    from tybok_b200 import base, engine

    if base.HAVE_REFERENCE:
        from tybok.registry import _REGISTRY
    else:
        _REGISTRY = base._REGISTRY
    assert _REGISTRY["pi05_b200"] is engine.PI05B200Engine
    with pytest.raises(ValueError):
        base.register("pi05_b200")(engine.PI05B200Engine)
