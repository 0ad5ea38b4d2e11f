"""torch custom ops over the C ABI (``torch.ops.tybok_b200.*``), CUDA only.

Each op validates tensors, allocates its output with torch (so CUDA-graph capture sees an
ordinary allocation), and launches on the current torch stream.  The split-K scratch is one
per-device buffer owned by this module; it is allocated on first use, before any capture.
"""

from __future__ import annotations

import torch

from . import _lib

EPI_NONE, EPI_GELU, EPI_RESIDUAL = 0, 1, 2

_L = torch.library.Library("tybok_b200", "DEF")
_L.define(
    "w8a16_linear(Tensor x, Tensor w8, Tensor scale, Tensor? bias, int epilogue, Tensor? residual, Tensor? gate, "
    "int rows_per_gate, int token_tile, int splits) -> Tensor"
)
_L.define("w8a16_geglu(Tensor x, Tensor w8_gate, Tensor scale_gate, Tensor w8_up, Tensor scale_up, int token_tile, "
          "int splits) -> Tensor")

_workspaces: dict[int, torch.Tensor] = {}
_status: dict[int, torch.Tensor] = {}
WORKSPACE_BYTES = 96 << 20


def workspace(device: torch.device) -> torch.Tensor:
    """The per-device scratch (arrival counters + split-K partials), zeroed once."""
    idx = device.index if device.index is not None else torch.cuda.current_device()
    ws = _workspaces.get(idx)
    if ws is None:
        ws = torch.zeros(WORKSPACE_BYTES, dtype=torch.uint8, device=torch.device("cuda", idx))
        _workspaces[idx] = ws
        _status[idx] = torch.zeros(1, dtype=torch.int32, device=torch.device("cuda", idx))
    return ws


def status_word(device: torch.device) -> torch.Tensor:
    workspace(device)
    idx = device.index if device.index is not None else torch.cuda.current_device()
    return _status[idx]


def check_status(device: torch.device | None = None) -> None:
    """Synchronise and raise if any kernel reported a timed-out device wait."""
    device = device or torch.device("cuda", torch.cuda.current_device())
    word = status_word(device)
    torch.cuda.synchronize(device)
    code = int(word.item())
    if code != 0:
        word.zero_()
        raise _lib.TybokError(f"device status {code}: a bounded wait inside a tybok_b200 kernel ran out")


def _ptr(t: torch.Tensor | None) -> int | None:
    return None if t is None else t.data_ptr()


def _rows(x: torch.Tensor) -> tuple[torch.Tensor, int]:
    k = x.shape[-1]
    x2 = x.reshape(-1, k)
    if x2.stride(-1) != 1:
        x2 = x2.contiguous()
    return x2, x2.shape[0]


def _w8a16_linear_cuda(x, w8, scale, bias, epilogue, residual, gate, rows_per_gate, token_tile, splits):
    lib = _lib.load()
    if x.dtype != torch.bfloat16:
        raise TypeError(f"w8a16_linear: x must be bf16, got {x.dtype}")
    if w8.dtype not in (torch.float8_e4m3fn, torch.uint8) or not w8.is_contiguous():
        raise TypeError("w8a16_linear: w8 must be a contiguous e4m3 (or raw uint8) [N, K] tensor")
    if scale.dtype != torch.float32:
        raise TypeError("w8a16_linear: scale must be fp32")
    n, k = w8.shape
    x2, m = _rows(x)
    if x2.shape[1] != k:
        raise ValueError(f"w8a16_linear: x has K={x2.shape[1]}, weight has K={k}")
    y = torch.empty((m, n), dtype=torch.bfloat16, device=x.device)
    res2 = None
    if residual is not None:
        res2, mr = _rows(residual)
        if mr != m or res2.shape[1] != n or res2.dtype != torch.bfloat16:
            raise ValueError("w8a16_linear: residual must be bf16 [M, N]")
    gate_bf16 = 0
    ldgate = 0
    if gate is not None:
        if gate.dtype not in (torch.float32, torch.bfloat16) or gate.stride(-1) != 1:
            raise TypeError("w8a16_linear: gate must be fp32 or bf16 with unit inner stride")
        gate_bf16 = int(gate.dtype == torch.bfloat16)
        gate = gate.reshape(-1, n) if gate.is_contiguous() else gate
        ldgate = gate.stride(0) if gate.dim() > 1 else n
    ws = workspace(x.device)
    rc = lib.tybok_w8a16_linear(
        x2.data_ptr(), w8.data_ptr(), scale.data_ptr(), _ptr(bias), y.data_ptr(), m, n, k, x2.stride(0), y.stride(0),
        int(epilogue), _ptr(res2), res2.stride(0) if res2 is not None else 0, _ptr(gate), ldgate,
        int(rows_per_gate), gate_bf16, int(token_tile), int(splits), ws.data_ptr(), ws.numel(),
        status_word(x.device).data_ptr(), torch.cuda.current_stream(x.device).cuda_stream,
    )
    _lib.check(rc, "tybok_w8a16_linear")
    return y.reshape(*x.shape[:-1], n)


def _w8a16_geglu_cuda(x, w8_gate, scale_gate, w8_up, scale_up, token_tile, splits):
    lib = _lib.load()
    if x.dtype != torch.bfloat16:
        raise TypeError(f"w8a16_geglu: x must be bf16, got {x.dtype}")
    for w in (w8_gate, w8_up):
        if w.dtype not in (torch.float8_e4m3fn, torch.uint8) or not w.is_contiguous():
            raise TypeError("w8a16_geglu: weights must be contiguous e4m3 [I, K] tensors")
    if w8_gate.shape != w8_up.shape:
        raise ValueError("w8a16_geglu: gate and up weights differ in shape")
    i, k = w8_gate.shape
    x2, m = _rows(x)
    h = torch.empty((m, i), dtype=torch.bfloat16, device=x.device)
    ws = workspace(x.device)
    rc = lib.tybok_w8a16_geglu(
        x2.data_ptr(), w8_gate.data_ptr(), scale_gate.data_ptr(), w8_up.data_ptr(), scale_up.data_ptr(), h.data_ptr(),
        m, i, k, x2.stride(0), h.stride(0), int(token_tile), int(splits), ws.data_ptr(), ws.numel(),
        status_word(x.device).data_ptr(), torch.cuda.current_stream(x.device).cuda_stream,
    )
    _lib.check(rc, "tybok_w8a16_geglu")
    return h.reshape(*x.shape[:-1], i)


_L.impl("w8a16_linear", _w8a16_linear_cuda, "CUDA")
_L.impl("w8a16_geglu", _w8a16_geglu_cuda, "CUDA")


def w8a16_linear(x, w8, scale, bias=None, *, epilogue=EPI_NONE, residual=None, gate=None, rows_per_gate=1,
                 token_tile=0, splits=0) -> torch.Tensor:
    """``epilogue(x @ (w8*scale).T + bias)`` in bf16; see ``tybok_w8a16_linear`` in the C header."""
    return torch.ops.tybok_b200.w8a16_linear(x, w8, scale, bias, epilogue, residual, gate, rows_per_gate, token_tile,
                                             splits)


def w8a16_geglu(x, w8_gate, scale_gate, w8_up, scale_up, *, token_tile=0, splits=0) -> torch.Tensor:
    """``gelu_tanh(x@Wg.T) * (x@Wu.T)`` in one launch; see ``tybok_w8a16_geglu``."""
    return torch.ops.tybok_b200.w8a16_geglu(x, w8_gate, scale_gate, w8_up, scale_up, token_tile, splits)


def launch_count() -> int:
    return int(_lib.load().tybok_launch_count())
