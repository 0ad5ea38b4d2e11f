"""ctypes binding of ``libtybok_b200.so`` (the C ABI declared in ``include/tybok_b200.h``).

There is no fallback: if the library is missing or does not export a declared symbol, import
of the ops fails with an error that says how to build it.
"""

from __future__ import annotations

import ctypes
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libtybok_b200.so")

c_void_p, c_int, c_i64, c_size_t = ctypes.c_void_p, ctypes.c_int, ctypes.c_int64, ctypes.c_size_t

#: name -> (restype, argtypes); must list every function ``include/tybok_b200.h`` declares.
SIGNATURES = {
    "tybok_version": (c_int, []),
    "tybok_last_error": (ctypes.c_char_p, []),
    "tybok_launch_count": (ctypes.c_longlong, []),
    "tybok_set_pdl": (None, [c_int]),
    "tybok_debug_set_trace": (None, [c_void_p]),
    "tybok_debug_set_counters": (None, [c_void_p]),
    "tybok_debug_set_epilogue_wait_limit": (None, [ctypes.c_longlong]),
    "tybok_split3": (c_int, [c_void_p, c_i64, c_void_p, c_int, c_int, c_int, c_void_p]),
    "tybok_w8x3_linear": (
        c_int,
        [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_i64, c_void_p, c_int, c_int, c_int, c_int, c_int,
         c_void_p, c_i64, c_void_p, c_i64, c_int, c_int, c_int, c_int, c_void_p, c_void_p],
    ),
    "tybok_w8x3_geglu": (
        c_int,
        [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_i64, c_void_p, c_int, c_int, c_int,
         c_int, c_int, c_int, c_void_p, c_void_p],
    ),
    "tybok_rmsnorm": (c_int, [c_void_p, c_i64, c_void_p, c_void_p, c_i64, c_int, c_int, c_int, ctypes.c_float,
                              c_void_p, c_i64, c_void_p, c_int, c_void_p]),
    "tybok_layernorm_modulate": (c_int, [c_void_p, c_i64, c_void_p, c_void_p, c_int, c_int, ctypes.c_float, c_void_p,
                                         c_i64, c_void_p, c_int, c_void_p]),
    "tybok_action_tail": (c_int, [c_void_p, c_i64, c_void_p, c_i64, c_int, ctypes.c_float, c_void_p, c_void_p, c_void_p,
                                  ctypes.c_float, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p]),
    "tybok_rope_store": (c_int, [c_void_p, c_i64, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int,
                                 c_int, c_int, c_int, c_int, c_int, c_int, c_void_p]),
    "tybok_attention": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
                                c_int, c_int, c_int, c_int, ctypes.c_float, c_void_p, c_size_t, c_void_p, c_void_p]),
    "tybok_attention_workspace_bytes": (c_size_t, [c_int, c_int, c_int, c_int]),
    "tybok_w8x3_geglu_packed": (
        c_int,
        [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_i64, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int,
         c_void_p, c_void_p],
    ),
    "tybok_w8x3_qkv_rope": (
        c_int,
        [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int,
         c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p],
    ),
    "tybok_add_layernorm": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, ctypes.c_float, c_void_p,
                                    c_void_p, c_void_p]),
    "tybok_add_layernorm_mixed": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, ctypes.c_float, c_void_p,
                                          c_void_p, c_void_p]),
    "tybok_add_layernorm_mixed_f16": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, ctypes.c_float, c_void_p,
                                          c_void_p, c_void_p]),
    "tybok_add_layernorm_f32": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, ctypes.c_float, c_void_p,
                                        c_void_p, c_void_p]),
    "tybok_layernorm_affine": (c_int, [c_void_p, c_i64, c_void_p, c_void_p, c_int, c_int, ctypes.c_float, c_void_p,
                                       c_i64, c_void_p, c_int, c_void_p]),
    "tybok_qknorm_rope_store": (c_int, [c_void_p, c_i64, c_int, c_int, c_int, c_void_p, c_void_p, ctypes.c_float,
                                        c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
                                        c_int, c_int, c_void_p]),
    "tybok_norm_planes2": (c_int, [c_void_p, c_i64, c_int, c_void_p, c_void_p, c_i64, c_int, c_int, c_int, ctypes.c_float,
                                   c_void_p, c_void_p, c_void_p]),
    "tybok_w8x2_gemm": (
        c_int,
        [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_i64, c_void_p, c_int, c_int, c_int, c_int, c_int,
         c_void_p, c_i64, c_void_p, c_i64, c_int, c_int, c_int, c_int, c_void_p, c_void_p],
    ),
    "tybok_w8x2_qkv_rope": (
        c_int,
        [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int,
         c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p],
    ),
    "tybok_w8x3_residual_next_adarms": (
        c_int,
        [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_i64, c_void_p, c_i64, c_void_p, c_void_p, c_void_p, c_int,
         c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p],
    ),
    "tybok_w8x3_geglu_packed_adarms": (
        c_int,
        [c_void_p, c_int, c_void_p, c_int, ctypes.c_float, c_void_p, c_void_p, c_void_p, c_void_p, c_i64, c_void_p, c_int, c_int,
         c_int, c_int, c_int, c_int, c_void_p, c_void_p],
    ),
    "tybok_w8x3_qkv_rope_adarms": (
        c_int,
        [c_void_p, c_int, c_void_p, c_int, ctypes.c_float, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
         c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p],
    ),
    "tybok_w8a16_workspace_bytes": (c_size_t, [c_int, c_int, c_int, c_int]),
    "tybok_w8a16_linear": (
        c_int,
        [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_i64, c_i64, c_int, c_void_p, c_i64,
         c_void_p, c_i64, c_int, c_int, c_int, c_int, c_void_p, c_size_t, c_void_p, c_void_p],
    ),
    "tybok_w8a16_linear_noalloc": (
        c_int,
        [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_i64, c_i64, c_int, c_void_p, c_i64,
         c_void_p, c_i64, c_int, c_int, c_void_p, c_void_p],
    ),
    "tybok_w8a16_geglu": (
        c_int,
        [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_i64, c_i64, c_int, c_int,
         c_void_p, c_size_t, c_void_p, c_void_p],
    ),
}

_lib = None


class TybokError(RuntimeError):
    """A C-ABI call returned a non-zero status."""


def load() -> ctypes.CDLL:
    """Load the shared library once and type every entry point."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python -m tybok_b200.build` (needs nvcc). "
            "tybok_b200 has no CPU or library fallback."
        )
    lib = ctypes.CDLL(LIB_PATH)
    for name, (restype, argtypes) in SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError here = stale library
        fn.restype = restype
        fn.argtypes = argtypes
    _lib = lib
    return lib


def check(rc: int, what: str) -> None:
    if rc != 0:
        msg = load().tybok_last_error().decode("utf-8", "replace")
        raise TybokError(f"{what} failed with status {rc}: {msg}")
