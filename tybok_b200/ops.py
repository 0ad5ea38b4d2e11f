"""torch custom ops over the C ABI (``torch.ops.tybok_b200.*``), CUDA only.

Each op validates tensors, allocates its outputs with torch (so CUDA-graph capture sees
ordinary allocations) and launches on the current torch stream.  There is no CPU
implementation: calling an op with CPU tensors raises ``NotImplementedError``.

Activation planes: the GEMMs take activations as a ``uint8 [3, M, K]`` tensor of e5m2 bytes
whose three planes sum to ``x * 2**shift`` (exactly, for bf16 ``x`` in the window documented in
``include/tybok_b200.h``).  ``split3`` makes them from bf16; the fused producers write them
directly.
"""

from __future__ import annotations

import torch

from . import _lib

EPI_NONE, EPI_GELU, EPI_RESIDUAL = 0, 1, 2
DEFAULT_SHIFT = 4

_L = torch.library.Library("tybok_b200", "DEF")
_L.define("split3(Tensor x, int shift) -> Tensor")
_L.define(
    "w8x3_linear(Tensor planes, int shift, Tensor w8, Tensor scale, Tensor? bias, int epilogue, Tensor? residual, "
    "Tensor? gate, int rows_per_gate, bool out_bf16, bool out_planes, int out_shift, int token_tile, int splits) "
    "-> (Tensor, Tensor)"
)
_L.define(
    "w8x3_geglu(Tensor planes, int shift, Tensor w8_gate, Tensor scale_gate, Tensor w8_up, Tensor scale_up, "
    "bool out_bf16, bool out_planes, int out_shift, int token_tile, int splits) -> (Tensor, Tensor)"
)

_L.define("rmsnorm(Tensor x, Tensor? weight, Tensor? mod, int rows_per_group, float eps, bool out_bf16, "
          "bool out_planes, int out_shift) -> (Tensor, Tensor)")

_L.define("rope_store(Tensor qkv, Tensor pos, Tensor cos, Tensor sin, Tensor(a!) k_cache, Tensor(b!) v_cache, int heads, "
          "int key_off) -> Tensor")
_L.define("attention(Tensor q, Tensor k_cache, Tensor v_cache, Tensor? key_valid, int tokens, int keys, float scale, "
          "bool out_bf16, bool out_planes, int out_shift) -> (Tensor, Tensor)")

_L.define("layernorm_modulate(Tensor x, Tensor shift, Tensor scale, float eps, bool out_bf16, bool out_planes, "
          "int out_shift) -> (Tensor, Tensor)")

_L.define("action_tail(Tensor? x, Tensor? mod, int rows_per_group, float eps, Tensor? w_out, Tensor? b_out, "
          "Tensor(a!) x_t, float dt, Tensor? w_in, Tensor? b_in, bool embed) -> Tensor")

_L.define("w8x3_geglu_packed(Tensor planes, int shift, Tensor w8_packed, Tensor scale_packed, bool out_bf16, "
          "bool out_planes, int out_shift, int token_tile, int splits) -> (Tensor, Tensor)")

_L.define("w8x3_qkv_rope(Tensor planes, int shift, Tensor w8_paired, Tensor scale_paired, Tensor pos, Tensor cos, "
          "Tensor sin, Tensor(a!) k_cache, Tensor(b!) v_cache, int heads, int key_off, int token_tile, int splits) "
          "-> Tensor")

_L.define("add_layernorm(Tensor x, Tensor? y, Tensor weight, Tensor bias, float eps) -> (Tensor, Tensor)")

_L.define("layernorm_affine(Tensor x, Tensor weight, Tensor bias, float eps, bool out_bf16, bool out_planes, "
          "int out_shift) -> (Tensor, Tensor)")
_L.define("qknorm_rope_store(Tensor src, int q_off, int k_off, int v_off, Tensor? norm_q, Tensor? norm_k, float eps, "
          "Tensor? cos, Tensor? sin, Tensor(a!)? k_cache, Tensor(b!)? v_cache, int batch, int heads, int head_dim, "
          "int key_off) -> Tensor")

_L.define("norm_planes2(Tensor x, int mode, Tensor a, Tensor? b, int rows_per_group, float eps) -> (Tensor, Tensor)")
_L.define("w8x2_gemm(Tensor planes2, Tensor row_scale, Tensor w8, Tensor scale, Tensor? bias, int epilogue, "
          "Tensor? residual, Tensor? gate, int rows_per_gate, bool out_bf16, bool out_planes, int out_shift, "
          "int token_tile, int splits) -> (Tensor, Tensor)")
_L.define("w8x2_qkv_rope(Tensor planes2, Tensor row_scale, Tensor w8_paired, Tensor scale_paired, Tensor pos, Tensor cos, "
          "Tensor sin, Tensor(a!) k_cache, Tensor(b!) v_cache, int heads, int key_off, int token_tile, int splits) -> Tensor")

_L.define("w8x3_residual_next_adarms(Tensor planes, int shift, Tensor w8, Tensor scale, Tensor residual, Tensor gate, "
          "Tensor next_scale, int out_shift, int token_tile, int splits) -> (Tensor, Tensor, Tensor)")
_L.define("w8x3_geglu_packed_adarms(Tensor u_planes, int shift, Tensor ss_part, float eps, Tensor bias_rows, "
          "Tensor w8_packed, Tensor scale_packed, bool out_bf16, bool out_planes, int out_shift, int token_tile, "
          "int splits) -> (Tensor, Tensor)")
_L.define("w8x3_qkv_rope_adarms(Tensor u_planes, int shift, Tensor ss_part, float eps, Tensor bias_rows, Tensor w8_paired, "
          "Tensor scale_paired, Tensor pos, Tensor cos, Tensor sin, Tensor(a!) k_cache, Tensor(b!) v_cache, int heads, "
          "int key_off, int token_tile, int splits) -> Tensor")

NORM_RMS, NORM_ADARMS, NORM_LN_MODULATE, NORM_LN_AFFINE = 0, 1, 2, 3
EPI_GEGLU_PACKED = 4

_status: dict[int, torch.Tensor] = {}


def _dev_index(device: torch.device) -> int:
    return device.index if device.index is not None else torch.cuda.current_device()


def status_word(device: torch.device) -> torch.Tensor:
    """Per-device int32 that kernels set when one of their bounded waits runs out."""
    idx = _dev_index(device)
    word = _status.get(idx)
    if word is None:
        word = torch.zeros(1, dtype=torch.int32, device=torch.device("cuda", idx))
        _status[idx] = word
    return word


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


def _stream(t: torch.Tensor) -> int:
    return torch.cuda.current_stream(t.device).cuda_stream


def _rows(x: torch.Tensor) -> torch.Tensor:
    x2 = x.reshape(-1, x.shape[-1])
    return x2 if x2.stride(-1) == 1 else x2.contiguous()


def _check_w8(w8: torch.Tensor, what: str) -> None:
    if w8.dtype not in (torch.float8_e4m3fn, torch.uint8) or not w8.is_contiguous() or w8.dim() != 2:
        raise TypeError(f"{what}: weight must be a contiguous e4m3 (or raw uint8) [N, K] tensor")


def _check_scale(scale: torch.Tensor, rows: int, what: str) -> None:
    if scale.dtype != torch.float32 or scale.numel() != rows or not scale.is_contiguous():
        raise TypeError(f"{what}: scale must be contiguous fp32 [{rows}] (one per weight row)")


def _split3_cuda(x: torch.Tensor, shift: int) -> torch.Tensor:
    lib = _lib.load()
    if x.dtype != torch.bfloat16:
        raise TypeError(f"split3: x must be bf16, got {x.dtype}")
    x2 = _rows(x)
    m, k = x2.shape
    planes = torch.empty((3, m, k), dtype=torch.uint8, device=x.device)
    rc = lib.tybok_split3(x2.data_ptr(), x2.stride(0), planes.data_ptr(), m, k, int(shift), _stream(x))
    _lib.check(rc, "tybok_split3")
    return planes


def _outputs(m, n, device, out_bf16, out_planes):
    if not (out_bf16 or out_planes):
        raise ValueError("at least one of out_bf16 / out_planes must be set")
    y = torch.empty((m, n) if out_bf16 else (0,), dtype=torch.bfloat16, device=device)
    yp = torch.empty((3, m, n) if out_planes else (0,), dtype=torch.uint8, device=device)
    return y, yp


def _w8x3_linear_cuda(planes, shift, w8, scale, bias, epilogue, residual, gate, rows_per_gate, out_bf16, out_planes,
                      out_shift, token_tile, splits):
    lib = _lib.load()
    _check_w8(w8, "w8x3_linear")
    if planes.dtype != torch.uint8 or planes.dim() != 3 or planes.shape[0] != 3 or not planes.is_contiguous():
        raise TypeError("w8x3_linear: planes must be a contiguous uint8 [3, M, K] tensor")
    n, k = w8.shape
    _check_scale(scale, n, "w8x3_linear")
    m = planes.shape[1]
    if planes.shape[2] != k:
        raise ValueError(f"w8x3_linear: planes have K={planes.shape[2]}, weight has K={k}")
    y, yp = _outputs(m, n, planes.device, out_bf16, out_planes)
    res2 = None
    if residual is not None:
        res2 = _rows(residual)
        if res2.shape != (m, n) or res2.dtype != torch.bfloat16:
            raise ValueError("w8x3_linear: residual must be bf16 [M, N]")
    gate_bf16 = ldgate = 0
    if gate is not None:
        if gate.dtype not in (torch.float32, torch.bfloat16) or gate.stride(-1) != 1 or gate.shape[-1] != n:
            raise TypeError("w8x3_linear: gate must be fp32 or bf16 [groups, N] with unit inner stride")
        gate_bf16 = int(gate.dtype == torch.bfloat16)
        ldgate = gate.stride(-2) if gate.dim() > 1 else n
    rc = lib.tybok_w8x3_linear(
        planes.data_ptr(), int(shift), w8.data_ptr(), scale.data_ptr(), _ptr(bias), y.data_ptr() if out_bf16 else None,
        n, yp.data_ptr() if out_planes else None, int(out_shift), m, n, k, int(epilogue), _ptr(res2),
        res2.stride(0) if res2 is not None else 0, _ptr(gate), ldgate, int(rows_per_gate), gate_bf16, int(token_tile),
        int(splits), status_word(planes.device).data_ptr(), _stream(planes),
    )
    _lib.check(rc, "tybok_w8x3_linear")
    return y, yp


def _w8x3_geglu_cuda(planes, shift, w8_gate, scale_gate, w8_up, scale_up, out_bf16, out_planes, out_shift, token_tile,
                     splits):
    lib = _lib.load()
    _check_w8(w8_gate, "w8x3_geglu")
    _check_w8(w8_up, "w8x3_geglu")
    if w8_gate.shape != w8_up.shape:
        raise ValueError("w8x3_geglu: gate and up weights differ in shape")
    if planes.dtype != torch.uint8 or planes.dim() != 3 or planes.shape[0] != 3 or not planes.is_contiguous():
        raise TypeError("w8x3_geglu: planes must be a contiguous uint8 [3, M, K] tensor")
    i, k = w8_gate.shape
    m = planes.shape[1]
    if planes.shape[2] != k:
        raise ValueError(f"w8x3_geglu: planes have K={planes.shape[2]}, weights have K={k}")
    h, hp = _outputs(m, i, planes.device, out_bf16, out_planes)
    rc = lib.tybok_w8x3_geglu(
        planes.data_ptr(), int(shift), w8_gate.data_ptr(), scale_gate.data_ptr(), w8_up.data_ptr(),
        scale_up.data_ptr(), h.data_ptr() if out_bf16 else None, i, hp.data_ptr() if out_planes else None,
        int(out_shift), m, i, k, int(token_tile), int(splits), status_word(planes.device).data_ptr(), _stream(planes),
    )
    _lib.check(rc, "tybok_w8x3_geglu")
    return h, hp


def _rmsnorm_cuda(x, weight, mod, rows_per_group, eps, out_bf16, out_planes, out_shift):
    lib = _lib.load()
    if x.dtype != torch.bfloat16:
        raise TypeError(f"rmsnorm: x must be bf16, got {x.dtype}")
    x2 = _rows(x)
    m, w = x2.shape
    if weight is not None and (weight.dtype != torch.float32 or weight.numel() != w or not weight.is_contiguous()):
        raise TypeError("rmsnorm: weight must be contiguous fp32 [W]")
    ldmod = 0
    if mod is not None:
        if mod.dtype != torch.float32 or mod.stride(-1) != 1 or mod.shape[-1] < 2 * w:
            raise TypeError("rmsnorm: mod must be fp32 [groups, >= 2*W] with unit inner stride")
        ldmod = mod.stride(-2) if mod.dim() > 1 else mod.shape[-1]
    y, yp = _outputs(m, w, x.device, out_bf16, out_planes)
    rc = lib.tybok_rmsnorm(x2.data_ptr(), x2.stride(0), _ptr(weight), _ptr(mod), ldmod, int(rows_per_group), m, w,
                           float(eps), y.data_ptr() if out_bf16 else None, w, yp.data_ptr() if out_planes else None,
                           int(out_shift), _stream(x))
    _lib.check(rc, "tybok_rmsnorm")
    return y, yp


def _rope_store_cuda(qkv, pos, cos, sin, k_cache, v_cache, heads, key_off):
    lib = _lib.load()
    b, g, lcap, d = k_cache.shape
    if qkv.dtype != torch.bfloat16 or qkv.dim() != 2 or qkv.stride(1) != 1 or qkv.shape[1] != (heads + 2 * g) * d:
        raise TypeError("rope_store: qkv must be bf16 [B*L, (H+2G)*D]")
    if pos.dtype != torch.int32 or pos.numel() != qkv.shape[0] or not pos.is_contiguous():
        raise TypeError("rope_store: pos must be contiguous int32 [B*L]")
    for t in (k_cache, v_cache, cos, sin):
        if t.dtype != torch.bfloat16 or not t.is_contiguous():
            raise TypeError("rope_store: caches and cos/sin tables must be contiguous bf16")
    if v_cache.shape != k_cache.shape or cos.shape[-1] != d:
        raise ValueError("rope_store: cache / table shapes disagree")
    l = qkv.shape[0] // b
    q = torch.empty((qkv.shape[0], heads * d), dtype=torch.bfloat16, device=qkv.device)
    rc = lib.tybok_rope_store(qkv.data_ptr(), qkv.stride(0), pos.data_ptr(), cos.data_ptr(), sin.data_ptr(),
                              q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), b, l, heads, g, d, lcap,
                              int(key_off), _stream(qkv))
    _lib.check(rc, "tybok_rope_store")
    return q


def _attention_cuda(q, k_cache, v_cache, key_valid, tokens, keys, scale, out_bf16, out_planes, out_shift):
    lib = _lib.load()
    b, g, lcap, d = k_cache.shape
    if q.dtype != torch.bfloat16 or q.dim() != 2 or not q.is_contiguous() or q.shape[0] != b * tokens:
        raise TypeError("attention: q must be contiguous bf16 [B*L, H*D]")
    h = q.shape[1] // d
    if key_valid is not None and (key_valid.dtype != torch.uint8 or key_valid.shape != (b, keys)
                                  or not key_valid.is_contiguous()):
        raise TypeError("attention: key_valid must be contiguous uint8 [B, Lk]")
    y, yp = _outputs(b * tokens, h * d, q.device, out_bf16, out_planes)
    # head_dim 128 always takes the key-loop kernel, which exchanges nothing
    need = 0 if d == 128 else int(lib.tybok_attention_workspace_bytes(b, int(tokens), h, int(keys)))
    ws = torch.empty(need, dtype=torch.uint8, device=q.device) if need else None
    rc = lib.tybok_attention(q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), _ptr(key_valid),
                             y.data_ptr() if out_bf16 else None, yp.data_ptr() if out_planes else None, int(out_shift),
                             b, int(tokens), h, g, d, int(keys), lcap, float(scale), _ptr(ws), need,
                             status_word(q.device).data_ptr(), _stream(q))
    _lib.check(rc, "tybok_attention")
    return y, yp


def _layernorm_modulate_cuda(x, shift, scale, eps, out_bf16, out_planes, out_shift):
    lib = _lib.load()
    if x.dtype != torch.bfloat16:
        raise TypeError(f"layernorm_modulate: x must be bf16, got {x.dtype}")
    x2 = _rows(x)
    m, w = x2.shape
    for t in (shift, scale):
        if t.dtype != torch.bfloat16 or t.numel() != w or not t.is_contiguous():
            raise TypeError("layernorm_modulate: shift/scale must be contiguous bf16 with W elements")
    y, yp = _outputs(m, w, x.device, out_bf16, out_planes)
    rc = lib.tybok_layernorm_modulate(x2.data_ptr(), x2.stride(0), shift.data_ptr(), scale.data_ptr(), m, w, float(eps),
                                      y.data_ptr() if out_bf16 else None, w, yp.data_ptr() if out_planes else None,
                                      int(out_shift), _stream(x))
    _lib.check(rc, "tybok_layernorm_modulate")
    return y, yp


_L.impl("layernorm_modulate", _layernorm_modulate_cuda, "CUDA")
def _action_tail_cuda(x, mod, rows_per_group, eps, w_out, b_out, x_t, dt, w_in, b_in, embed):
    lib = _lib.load()
    if x_t.dtype != torch.float32 or not x_t.is_contiguous():
        raise TypeError("action_tail: x_t must be contiguous fp32 [M, A]")
    a = x_t.shape[-1]
    m = x_t.numel() // a
    for t in (mod, w_out, b_out, w_in, b_in):
        if t is not None and (t.dtype != torch.float32 or not t.is_contiguous()):
            raise TypeError("action_tail: modulation and projection tensors must be contiguous fp32")
    if x is not None:
        x = _rows(x)
        if x.dtype != torch.bfloat16 or x.shape[0] != m:
            raise TypeError("action_tail: x must be bf16 [M, W]")
        w = x.shape[1]
    else:
        w = w_in.shape[0]
    h = torch.empty((m, w) if embed else (0,), dtype=torch.bfloat16, device=x_t.device)
    rc = lib.tybok_action_tail(_ptr(x), x.stride(0) if x is not None else 0, _ptr(mod),
                               mod.shape[-1] if mod is not None else 0, int(rows_per_group), float(eps), _ptr(w_out),
                               _ptr(b_out), x_t.data_ptr(), float(dt), _ptr(w_in) if embed else None,
                               _ptr(b_in) if embed else None, h.data_ptr() if embed else None, m, w, a, _stream(x_t))
    _lib.check(rc, "tybok_action_tail")
    return h


_L.impl("action_tail", _action_tail_cuda, "CUDA")
def _w8x3_qkv_rope_cuda(planes, shift, w8_paired, scale_paired, pos, cos, sin, k_cache, v_cache, heads, key_off,
                        token_tile, splits):
    lib = _lib.load()
    _check_w8(w8_paired, "w8x3_qkv_rope")
    b, g, lcap, d = k_cache.shape
    if planes.dtype != torch.uint8 or planes.dim() != 3 or planes.shape[0] != 3 or not planes.is_contiguous():
        raise TypeError("w8x3_qkv_rope: planes must be a contiguous uint8 [3, M, K] tensor")
    m, k = planes.shape[1], planes.shape[2]
    if w8_paired.shape != ((heads + 2 * g) * d, k) or scale_paired.numel() != w8_paired.shape[0] or d % 128 != 0:
        raise ValueError("w8x3_qkv_rope: weight must be [(H+2G)*D, K] with head_dim % 128 == 0")
    if pos.dtype != torch.int32 or pos.numel() != m or not pos.is_contiguous() or m % b != 0:
        raise TypeError("w8x3_qkv_rope: pos must be contiguous int32 [B*L]")
    for t in (k_cache, v_cache, cos, sin):
        if t.dtype != torch.bfloat16 or not t.is_contiguous():
            raise TypeError("w8x3_qkv_rope: caches and cos/sin tables must be contiguous bf16")
    if v_cache.shape != k_cache.shape or cos.shape[-1] != d or sin.shape != cos.shape:
        raise ValueError("w8x3_qkv_rope: cache / table shapes disagree")
    q = torch.empty((m, heads * d), dtype=torch.bfloat16, device=planes.device)
    rc = lib.tybok_w8x3_qkv_rope(planes.data_ptr(), int(shift), w8_paired.data_ptr(), scale_paired.data_ptr(),
                                 pos.data_ptr(), cos.data_ptr(), sin.data_ptr(), q.data_ptr(), k_cache.data_ptr(),
                                 v_cache.data_ptr(), b, m // b, heads, g, d, lcap, int(key_off), k, int(token_tile),
                                 int(splits), status_word(planes.device).data_ptr(), _stream(planes))
    _lib.check(rc, "tybok_w8x3_qkv_rope")
    return q


_L.impl("w8x3_qkv_rope", _w8x3_qkv_rope_cuda, "CUDA")
_L.impl("rope_store", _rope_store_cuda, "CUDA")
_L.impl("attention", _attention_cuda, "CUDA")
_L.impl("rmsnorm", _rmsnorm_cuda, "CUDA")
def _w8x3_geglu_packed_cuda(planes, shift, w8_packed, scale_packed, out_bf16, out_planes, out_shift, token_tile, splits):
    lib = _lib.load()
    _check_w8(w8_packed, "w8x3_geglu_packed")
    if planes.dtype != torch.uint8 or planes.dim() != 3 or planes.shape[0] != 3 or not planes.is_contiguous():
        raise TypeError("w8x3_geglu_packed: planes must be a contiguous uint8 [3, M, K] tensor")
    n2, k = w8_packed.shape
    if n2 % 128 != 0 or planes.shape[2] != k or scale_packed.numel() != n2:
        raise ValueError("w8x3_geglu_packed: packed weight must be [2*I, K] with I % 64 == 0 and a [2*I] scale")
    i, m = n2 // 2, planes.shape[1]
    h, hp = _outputs(m, i, planes.device, out_bf16, out_planes)
    rc = lib.tybok_w8x3_geglu_packed(planes.data_ptr(), int(shift), w8_packed.data_ptr(), scale_packed.data_ptr(),
                                     h.data_ptr() if out_bf16 else None, i, hp.data_ptr() if out_planes else None,
                                     int(out_shift), m, i, k, int(token_tile), int(splits),
                                     status_word(planes.device).data_ptr(), _stream(planes))
    _lib.check(rc, "tybok_w8x3_geglu_packed")
    return h, hp


_L.impl("w8x3_geglu_packed", _w8x3_geglu_packed_cuda, "CUDA")
def _add_layernorm_cuda(x, y, weight, bias, eps):
    lib = _lib.load()
    w = x.shape[-1]
    for t in (x, y, weight, bias):
        if t is not None and (t.dtype != torch.bfloat16 or not t.is_contiguous()):
            raise TypeError("add_layernorm: tensors must be contiguous bf16")
    if (y is not None and y.shape != x.shape) or weight.numel() != w or bias.numel() != w:
        raise ValueError("add_layernorm: shapes disagree")
    m = x.numel() // w
    x_out = torch.empty_like(x) if y is not None else x.new_empty(0)  # an op output must not alias an input
    h = torch.empty_like(x)
    rc = lib.tybok_add_layernorm(x.data_ptr(), _ptr(y), weight.data_ptr(), bias.data_ptr(), m, w, float(eps),
                                 x_out.data_ptr() if y is not None else None, h.data_ptr(), _stream(x))
    _lib.check(rc, "tybok_add_layernorm")
    return x_out, h


def _add_layernorm_any(x, y, weight, bias, eps):
    """All bf16, all fp32, or the mixed form (fp32 ``x`` with bf16 or fp16 ``y`` / ``weight`` / ``bias``)."""
    if x.dtype != torch.float32:
        return _add_layernorm_cuda(x, y, weight, bias, eps)
    lib = _lib.load()
    w = x.shape[-1]
    if weight.dtype in (torch.bfloat16, torch.float16):
        t16 = weight.dtype
        for t in (x, y, weight, bias):
            if t is not None and not t.is_contiguous():
                raise TypeError("add_layernorm: tensors must be contiguous")
        if (y is not None and (y.shape != x.shape or y.dtype != t16)) or bias.dtype != t16 \
                or weight.numel() != w or bias.numel() != w:
            raise ValueError("add_layernorm (fp32 stream): y / weight / bias must share one 16-bit dtype and match in shape")
        m = x.numel() // w
        x_out = torch.empty_like(x) if y is not None else x.new_empty(0)
        h = torch.empty(x.shape, dtype=t16, device=x.device)
        fn = lib.tybok_add_layernorm_mixed if t16 == torch.bfloat16 else lib.tybok_add_layernorm_mixed_f16
        rc = fn(x.data_ptr(), _ptr(y), weight.data_ptr(), bias.data_ptr(), m, w, float(eps),
                x_out.data_ptr() if y is not None else None, h.data_ptr(), _stream(x))
        _lib.check(rc, "tybok_add_layernorm_mixed")
        return x_out, h
    for t in (x, y, weight, bias):
        if t is not None and (t.dtype != torch.float32 or not t.is_contiguous()):
            raise TypeError("add_layernorm: tensors must be contiguous and of one dtype (bf16 or fp32)")
    if (y is not None and y.shape != x.shape) or weight.numel() != w or bias.numel() != w:
        raise ValueError("add_layernorm: shapes disagree")
    m = x.numel() // w
    x_out = torch.empty_like(x) if y is not None else x.new_empty(0)
    h = torch.empty_like(x)
    rc = lib.tybok_add_layernorm_f32(x.data_ptr(), _ptr(y), weight.data_ptr(), bias.data_ptr(), m, w, float(eps),
                                     x_out.data_ptr() if y is not None else None, h.data_ptr(), _stream(x))
    _lib.check(rc, "tybok_add_layernorm_f32")
    return x_out, h


def _layernorm_affine_cuda(x, weight, bias, eps, out_bf16, out_planes, out_shift):
    lib = _lib.load()
    if x.dtype != torch.bfloat16:
        raise TypeError(f"layernorm_affine: x must be bf16, got {x.dtype}")
    x2 = _rows(x)
    m, w = x2.shape
    for t in (weight, bias):
        if t.dtype != torch.bfloat16 or t.numel() != w or not t.is_contiguous():
            raise TypeError("layernorm_affine: weight/bias must be contiguous bf16 with W elements")
    y, yp = _outputs(m, w, x.device, out_bf16, out_planes)
    rc = lib.tybok_layernorm_affine(x2.data_ptr(), x2.stride(0), weight.data_ptr(), bias.data_ptr(), m, w, float(eps),
                                    y.data_ptr() if out_bf16 else None, w, yp.data_ptr() if out_planes else None,
                                    int(out_shift), _stream(x))
    _lib.check(rc, "tybok_layernorm_affine")
    return y, yp


def _qknorm_rope_store_cuda(src, q_off, k_off, v_off, norm_q, norm_k, eps, cos, sin, k_cache, v_cache, batch, heads,
                            head_dim, key_off):
    lib = _lib.load()
    if src.dtype != torch.bfloat16 or src.dim() != 2 or src.stride(1) != 1:
        raise TypeError("qknorm_rope_store: src must be bf16 [B*L, C] with unit inner stride")
    m, a = src.shape[0], heads * head_dim
    if m % batch != 0:
        raise ValueError("qknorm_rope_store: rows must be a multiple of the batch size")
    l = m // batch
    for t in (norm_q, norm_k):
        if t is not None and (t.dtype != torch.bfloat16 or t.numel() != a or not t.is_contiguous()):
            raise TypeError("qknorm_rope_store: norm weights must be contiguous bf16 [H*D]")
    for t in (cos, sin):
        if t is not None and (t.dtype != torch.float32 or tuple(t.shape) != (l, head_dim // 2) or not t.is_contiguous()):
            raise TypeError("qknorm_rope_store: cos/sin must be contiguous fp32 [L, D/2]")
    lcap = 0
    for t in (k_cache, v_cache):
        if t is not None:
            if t.dtype != torch.bfloat16 or not t.is_contiguous() or t.dim() != 4 or t.shape[0] != batch \
                    or t.shape[1] != heads or t.shape[3] != head_dim:
                raise TypeError("qknorm_rope_store: caches must be contiguous bf16 [B, H, Lcap, D]")
            lcap = t.shape[2]
    q = torch.empty((m, a) if q_off >= 0 else (0,), dtype=torch.bfloat16, device=src.device)
    rc = lib.tybok_qknorm_rope_store(src.data_ptr(), src.stride(0), int(q_off), int(k_off), int(v_off), _ptr(norm_q),
                                     _ptr(norm_k), float(eps), _ptr(cos), _ptr(sin), q.data_ptr() if q_off >= 0 else None,
                                     _ptr(k_cache), _ptr(v_cache), batch, l, heads, head_dim, lcap, int(key_off),
                                     _stream(src))
    _lib.check(rc, "tybok_qknorm_rope_store")
    return q


_L.impl("layernorm_affine", _layernorm_affine_cuda, "CUDA")
_L.impl("qknorm_rope_store", _qknorm_rope_store_cuda, "CUDA")
_L.impl("add_layernorm", _add_layernorm_any, "CUDA")
_L.impl("split3", _split3_cuda, "CUDA")
_L.impl("w8x3_linear", _w8x3_linear_cuda, "CUDA")
_L.impl("w8x3_geglu", _w8x3_geglu_cuda, "CUDA")


def split3(x: torch.Tensor, shift: int = DEFAULT_SHIFT) -> torch.Tensor:
    """bf16 ``[..., K]`` -> uint8 ``[3, M, K]`` e5m2 planes of ``x * 2**shift``."""
    return torch.ops.tybok_b200.split3(x, shift)


def w8x3_linear(planes, shift, w8, scale, bias=None, *, epilogue=EPI_NONE, residual=None, gate=None, rows_per_gate=1,
                out_bf16=True, out_planes=False, out_shift=DEFAULT_SHIFT, token_tile=0, splits=0):
    """W8 linear on activation planes; returns ``(y_bf16 [M,N], y_planes [3,M,N])`` (an output
    that was not requested is an empty tensor).  See ``tybok_w8x3_linear`` in the C header."""
    return torch.ops.tybok_b200.w8x3_linear(planes, shift, w8, scale, bias, epilogue, residual, gate, rows_per_gate,
                                            out_bf16, out_planes, out_shift, token_tile, splits)


def w8x3_geglu(planes, shift, w8_gate, scale_gate, w8_up, scale_up, *, out_bf16=True, out_planes=False,
               out_shift=DEFAULT_SHIFT, token_tile=0, splits=0):
    """``gelu_tanh(x@Wg.T) * (x@Wu.T)`` on activation planes; see ``tybok_w8x3_geglu``."""
    return torch.ops.tybok_b200.w8x3_geglu(planes, shift, w8_gate, scale_gate, w8_up, scale_up, out_bf16, out_planes,
                                           out_shift, token_tile, splits)


def pack_gate_up(w8_gate, scale_gate, w8_up, scale_up):
    """Interleave gate and up rows in blocks of 64 -> ``([2I, K] e4m3, [2I] fp32)`` for
    ``w8x3_geglu_packed`` (rows 128j..128j+63 = gate channels 64j.., rows +64.. = their up rows)."""
    i, k = w8_gate.shape
    if i % 64 != 0:
        raise ValueError("pack_gate_up: the FFN width must be a multiple of 64")
    g = w8_gate.view(torch.uint8).view(i // 64, 64, k)
    u = w8_up.view(torch.uint8).view(i // 64, 64, k)
    w = torch.stack((g, u), dim=1).reshape(2 * i, k).contiguous().view(torch.float8_e4m3fn)
    s = torch.stack((scale_gate.view(i // 64, 64), scale_up.view(i // 64, 64)), dim=1).reshape(2 * i).contiguous()
    return w, s


def pair_qkv_rows(w8_qkv, scale_qkv, head_dim):
    """Reorder the rows of a packed q/k/v weight for ``w8x3_qkv_rope``: inside every head slot,
    blocks of 64 dimensions alternate with the block of their rotate-half partners."""
    n, k = w8_qkv.shape
    if head_dim % 128 != 0 or n % head_dim != 0:
        raise ValueError("pair_qkv_rows: head_dim must be a multiple of 128")
    half = head_dim // 2
    d = torch.arange(half, device=w8_qkv.device).view(half // 64, 1, 64)
    within = torch.cat((d, d + half), dim=1).reshape(-1)  # [D]: 64 dims, 64 partners, next 64 dims, ...
    idx = (torch.arange(n // head_dim, device=w8_qkv.device)[:, None] * head_dim + within[None]).reshape(-1)
    w = w8_qkv.view(torch.uint8)[idx].contiguous().view(torch.float8_e4m3fn)
    return w, scale_qkv[idx].contiguous()


def w8x3_qkv_rope(planes, shift, w8_paired, scale_paired, pos, cos, sin, k_cache, v_cache, *, heads, key_off,
                  token_tile=0, splits=0):
    """q/k/v projection + RoPE + KV store in one kernel; returns rotated q ``[B*L, H*D]``; see
    ``tybok_w8x3_qkv_rope``."""
    return torch.ops.tybok_b200.w8x3_qkv_rope(planes, shift, w8_paired, scale_paired, pos, cos, sin, k_cache, v_cache,
                                              heads, key_off, token_tile, splits)


def w8x3_geglu_packed(planes, shift, w8_packed, scale_packed, *, out_bf16=True, out_planes=False,
                      out_shift=DEFAULT_SHIFT, token_tile=0, splits=0):
    """Gated FFN front half on a ``pack_gate_up`` weight; see ``tybok_w8x3_geglu_packed``."""
    return torch.ops.tybok_b200.w8x3_geglu_packed(planes, shift, w8_packed, scale_packed, out_bf16, out_planes,
                                                  out_shift, token_tile, splits)


def w8a16_linear(x, w8, scale, bias=None, *, epilogue=EPI_NONE, residual=None, gate=None, rows_per_gate=1,
                 token_tile=0, splits=0, shift=DEFAULT_SHIFT) -> torch.Tensor:
    """``epilogue(x @ (w8*scale).T + bias)`` for bf16 ``x``: ``split3`` then ``w8x3_linear``."""
    y, _ = w8x3_linear(split3(x, shift), shift, w8, scale, bias, epilogue=epilogue, residual=residual, gate=gate,
                       rows_per_gate=rows_per_gate, token_tile=token_tile, splits=splits)
    return y.reshape(*x.shape[:-1], w8.shape[0])


def w8a16_geglu(x, w8_gate, scale_gate, w8_up, scale_up, *, token_tile=0, splits=0, shift=DEFAULT_SHIFT):
    """``gelu_tanh(x@Wg.T) * (x@Wu.T)`` for bf16 ``x``."""
    h, _ = w8x3_geglu(split3(x, shift), shift, w8_gate, scale_gate, w8_up, scale_up, token_tile=token_tile,
                      splits=splits)
    return h.reshape(*x.shape[:-1], w8_gate.shape[0])


def rmsnorm(x, weight=None, mod=None, *, rows_per_group=1, eps=1e-6, out_bf16=False, out_planes=True,
            out_shift=DEFAULT_SHIFT):
    """Gemma RMSNorm (``weight``) or AdaRMS norm (``mod`` = precomputed ``dense(cond)``); returns
    ``(y_bf16, y_planes)``; see ``tybok_rmsnorm``."""
    return torch.ops.tybok_b200.rmsnorm(x, weight, mod, rows_per_group, eps, out_bf16, out_planes, out_shift)


def rope_store(qkv, pos, cos, sin, k_cache, v_cache, *, heads, key_off):
    """RoPE on the packed projection rows; rotated q is returned ``[B*L, H*D]``, rotated k and v are
    written into the caches ``[B, G, Lcap, D]`` at ``key_off``; see ``tybok_rope_store``."""
    return torch.ops.tybok_b200.rope_store(qkv, pos, cos, sin, k_cache, v_cache, heads, key_off)


def attention(q, k_cache, v_cache, key_valid=None, *, tokens, keys, scale, out_bf16=True, out_planes=False,
              out_shift=DEFAULT_SHIFT):
    """GQA attention over the first ``keys`` cache rows; returns ``(out_bf16, out_planes)``; see
    ``tybok_attention``."""
    return torch.ops.tybok_b200.attention(q, k_cache, v_cache, key_valid, tokens, keys, scale, out_bf16, out_planes,
                                          out_shift)


def layernorm_modulate(x, shift, scale, *, eps=1e-6, out_bf16=False, out_planes=True, out_shift=DEFAULT_SHIFT):
    """``modulate(LayerNorm(x), shift, scale)`` of a DiT block; returns ``(y_bf16, y_planes)``; see
    ``tybok_layernorm_modulate``."""
    return torch.ops.tybok_b200.layernorm_modulate(x, shift, scale, eps, out_bf16, out_planes, out_shift)


def action_tail(x, mod, w_out, b_out, x_t, dt, w_in, b_in, *, rows_per_group=1, eps=1e-6, embed=True):
    """Final norm + fp32 out-projection + Euler update of ``x_t`` (in place) + next suffix
    embedding (returned, bf16); ``x=None`` computes only the embedding; see ``tybok_action_tail``."""
    return torch.ops.tybok_b200.action_tail(x, mod, rows_per_group, eps, w_out, b_out, x_t, dt, w_in, b_in, embed)


def add_layernorm(x, y, weight, bias, *, eps=1e-6):
    """``x_new = x + y`` (``y=None``: ``x``) and ``LayerNorm(x_new) * weight + bias``, one kernel, all
    tensors bf16 or all fp32; returns ``(x_new, h)``; see ``tybok_add_layernorm`` / ``_f32``."""
    x_new, h = torch.ops.tybok_b200.add_layernorm(x, y, weight, bias, eps)
    return (x if y is None else x_new), h


def layernorm_affine(x, weight, bias, *, eps=1e-6, out_bf16=False, out_planes=True, out_shift=DEFAULT_SHIFT):
    """``LayerNorm(x) * weight + bias`` (fp32 statistics and affine, one bf16 rounding); returns
    ``(y_bf16, y_planes)``; see ``tybok_layernorm_affine``."""
    return torch.ops.tybok_b200.layernorm_affine(x, weight, bias, eps, out_bf16, out_planes, out_shift)


def qknorm_rope_store(src, *, q_off=-1, k_off=-1, v_off=-1, norm_q=None, norm_k=None, eps=1e-6, cos=None, sin=None,
                      k_cache=None, v_cache=None, batch=1, heads, head_dim, key_off=0):
    """Full-row RMS qk-norm + pair-wise rotary embedding + KV store of a DiT attention; returns the
    finished q ``[B*L, H*D]`` (empty when ``q_off < 0``); see ``tybok_qknorm_rope_store``."""
    return torch.ops.tybok_b200.qknorm_rope_store(src, q_off, k_off, v_off, norm_q, norm_k, eps, cos, sin, k_cache,
                                                  v_cache, batch, heads, head_dim, key_off)


def _norm_planes2_cuda(x, mode, a, b, rows_per_group, eps):
    lib = _lib.load()
    if x.dtype != torch.bfloat16:
        raise TypeError(f"norm_planes2: x must be bf16, got {x.dtype}")
    x2 = _rows(x)
    m, w = x2.shape
    ldmod = 0
    if mode in (NORM_RMS, NORM_ADARMS):
        if a.dtype != torch.float32 or a.stride(-1) != 1:
            raise TypeError("norm_planes2: the RMS weight / AdaRMS modulation must be fp32 with unit inner stride")
        if mode == NORM_RMS and (a.numel() != w or not a.is_contiguous()):
            raise TypeError("norm_planes2: weight must be contiguous fp32 [W]")
        if mode == NORM_ADARMS:
            if a.shape[-1] < 2 * w:
                raise TypeError("norm_planes2: mod must be fp32 [groups, >= 2*W]")
            ldmod = a.stride(-2) if a.dim() > 1 else a.shape[-1]
    else:
        for t in (a, b):
            if t is None or t.dtype != torch.bfloat16 or t.numel() != w or not t.is_contiguous():
                raise TypeError("norm_planes2: the LayerNorm forms take two contiguous bf16 [W] vectors")
    planes = torch.empty((2, m, w), dtype=torch.uint8, device=x.device)
    row_scale = torch.empty(m, dtype=torch.float32, device=x.device)
    rc = lib.tybok_norm_planes2(x2.data_ptr(), x2.stride(0), int(mode), a.data_ptr(), _ptr(b), ldmod, int(rows_per_group),
                                m, w, float(eps), planes.data_ptr(), row_scale.data_ptr(), _stream(x))
    _lib.check(rc, "tybok_norm_planes2")
    return planes, row_scale


def _check_planes2(planes, row_scale, k, what):
    if planes.dtype != torch.uint8 or planes.dim() != 3 or planes.shape[0] != 2 or not planes.is_contiguous():
        raise TypeError(f"{what}: planes must be a contiguous uint8 [2, M, K] tensor")
    if planes.shape[2] != k:
        raise ValueError(f"{what}: planes have K={planes.shape[2]}, weight has K={k}")
    if row_scale.dtype != torch.float32 or row_scale.numel() != planes.shape[1] or not row_scale.is_contiguous():
        raise TypeError(f"{what}: row_scale must be contiguous fp32 [M]")


def _w8x2_gemm_cuda(planes, row_scale, w8, scale, bias, epilogue, residual, gate, rows_per_gate, out_bf16, out_planes,
                    out_shift, token_tile, splits):
    lib = _lib.load()
    _check_w8(w8, "w8x2_gemm")
    n, k = w8.shape
    _check_scale(scale, n, "w8x2_gemm")
    _check_planes2(planes, row_scale, k, "w8x2_gemm")
    m = planes.shape[1]
    n_out = n // 2 if epilogue == EPI_GEGLU_PACKED else n
    y, yp = _outputs(m, n_out, planes.device, out_bf16, out_planes)
    res2 = None
    if residual is not None:
        res2 = _rows(residual)
        if res2.shape != (m, n) or res2.dtype != torch.bfloat16:
            raise ValueError("w8x2_gemm: residual must be bf16 [M, N]")
    gate_bf16 = ldgate = 0
    if gate is not None:
        if gate.dtype not in (torch.float32, torch.bfloat16) or gate.stride(-1) != 1 or gate.shape[-1] != n:
            raise TypeError("w8x2_gemm: gate must be fp32 or bf16 [groups, N] with unit inner stride")
        gate_bf16 = int(gate.dtype == torch.bfloat16)
        ldgate = gate.stride(-2) if gate.dim() > 1 else n
    rc = lib.tybok_w8x2_gemm(planes.data_ptr(), row_scale.data_ptr(), w8.data_ptr(), scale.data_ptr(), _ptr(bias),
                             y.data_ptr() if out_bf16 else None, n_out, yp.data_ptr() if out_planes else None,
                             int(out_shift), m, n, k, int(epilogue), _ptr(res2), res2.stride(0) if res2 is not None else 0,
                             _ptr(gate), ldgate, int(rows_per_gate), gate_bf16, int(token_tile), int(splits),
                             status_word(planes.device).data_ptr(), _stream(planes))
    _lib.check(rc, "tybok_w8x2_gemm")
    return y, yp


def _w8x2_qkv_rope_cuda(planes, row_scale, w8_paired, scale_paired, pos, cos, sin, k_cache, v_cache, heads, key_off,
                        token_tile, splits):
    lib = _lib.load()
    _check_w8(w8_paired, "w8x2_qkv_rope")
    b, g, lcap, d = k_cache.shape
    m, k = planes.shape[1], planes.shape[2]
    _check_planes2(planes, row_scale, w8_paired.shape[1], "w8x2_qkv_rope")
    _check_scale(scale_paired, w8_paired.shape[0], "w8x2_qkv_rope")
    if w8_paired.shape != ((heads + 2 * g) * d, k) or scale_paired.numel() != w8_paired.shape[0] or d % 128 != 0:
        raise ValueError("w8x2_qkv_rope: weight must be [(H+2G)*D, K] with head_dim % 128 == 0")
    if pos.dtype != torch.int32 or pos.numel() != m or not pos.is_contiguous() or m % b != 0:
        raise TypeError("w8x2_qkv_rope: pos must be contiguous int32 [B*L]")
    for t in (k_cache, v_cache, cos, sin):
        if t.dtype != torch.bfloat16 or not t.is_contiguous():
            raise TypeError("w8x2_qkv_rope: caches and cos/sin tables must be contiguous bf16")
    if v_cache.shape != k_cache.shape or cos.shape[-1] != d or sin.shape != cos.shape:
        raise ValueError("w8x2_qkv_rope: cache / table shapes disagree")
    q = torch.empty((m, heads * d), dtype=torch.bfloat16, device=planes.device)
    rc = lib.tybok_w8x2_qkv_rope(planes.data_ptr(), row_scale.data_ptr(), w8_paired.data_ptr(), scale_paired.data_ptr(),
                                 pos.data_ptr(), cos.data_ptr(), sin.data_ptr(), q.data_ptr(), k_cache.data_ptr(),
                                 v_cache.data_ptr(), b, m // b, heads, g, d, lcap, int(key_off), k, int(token_tile),
                                 int(splits), status_word(planes.device).data_ptr(), _stream(planes))
    _lib.check(rc, "tybok_w8x2_qkv_rope")
    return q


_L.impl("norm_planes2", _norm_planes2_cuda, "CUDA")
_L.impl("w8x2_gemm", _w8x2_gemm_cuda, "CUDA")
_L.impl("w8x2_qkv_rope", _w8x2_qkv_rope_cuda, "CUDA")


def norm_planes2(x, mode, a, b=None, *, rows_per_group=1, eps=1e-6):
    """A norm of this package with its output as two e4m3 planes of ``y * 2**k(row)`` plus
    ``row_scale = 2**-k(row)``: ``(planes [2, M, W] uint8, row_scale [M] fp32)``; ``mode`` is one of
    ``NORM_RMS`` (``a`` = fp32 weight), ``NORM_ADARMS`` (``a`` = fp32 modulation rows),
    ``NORM_LN_MODULATE`` (``a`` = shift, ``b`` = scale, bf16), ``NORM_LN_AFFINE`` (``a`` = weight,
    ``b`` = bias, bf16); see ``tybok_norm_planes2``."""
    return torch.ops.tybok_b200.norm_planes2(x, mode, a, b, rows_per_group, eps)


def w8x2_gemm(planes2, row_scale, w8, scale, bias=None, *, epilogue=EPI_NONE, residual=None, gate=None, rows_per_gate=1,
              out_bf16=True, out_planes=False, out_shift=DEFAULT_SHIFT, token_tile=0, splits=0):
    """W8 linear (or, with ``EPI_GEGLU_PACKED``, the gated FFN front half on a ``pack_gate_up`` weight)
    on two-plane activations; returns ``(y_bf16, y_planes)`` like ``w8x3_linear``; see ``tybok_w8x2_gemm``."""
    return torch.ops.tybok_b200.w8x2_gemm(planes2, row_scale, w8, scale, bias, epilogue, residual, gate, rows_per_gate,
                                          out_bf16, out_planes, out_shift, token_tile, splits)


def w8x2_qkv_rope(planes2, row_scale, w8_paired, scale_paired, pos, cos, sin, k_cache, v_cache, *, heads, key_off,
                  token_tile=0, splits=0):
    """``w8x3_qkv_rope`` on two-plane activations; see ``tybok_w8x2_qkv_rope``."""
    return torch.ops.tybok_b200.w8x2_qkv_rope(planes2, row_scale, w8_paired, scale_paired, pos, cos, sin, k_cache,
                                              v_cache, heads, key_off, token_tile, splits)


def _check_fold_in(u_planes, ss_part, bias_rows, rows, what):
    if u_planes.dtype != torch.uint8 or u_planes.dim() != 3 or u_planes.shape[0] != 3 or not u_planes.is_contiguous():
        raise TypeError(f"{what}: u_planes must be a contiguous uint8 [3, M, K] tensor")
    m = u_planes.shape[1]
    if ss_part.dtype != torch.float32 or ss_part.dim() != 2 or ss_part.shape[1] != m or not ss_part.is_contiguous():
        raise TypeError(f"{what}: ss_part must be contiguous fp32 [tiles, M]")
    if bias_rows.dtype != torch.float32 or bias_rows.numel() != rows or not bias_rows.is_contiguous():
        raise TypeError(f"{what}: bias_rows must be contiguous fp32 [weight rows]")


def _w8x3_residual_next_adarms_cuda(planes, shift, w8, scale, residual, gate, next_scale, out_shift, token_tile, splits):
    lib = _lib.load()
    _check_w8(w8, "w8x3_residual_next_adarms")
    n, k = w8.shape
    _check_scale(scale, n, "w8x3_residual_next_adarms")
    if planes.dtype != torch.uint8 or planes.dim() != 3 or planes.shape[0] != 3 or planes.shape[2] != k \
            or not planes.is_contiguous():
        raise TypeError("w8x3_residual_next_adarms: planes must be contiguous uint8 [3, M, K]")
    m = planes.shape[1]
    res2 = _rows(residual)
    if res2.shape != (m, n) or res2.dtype != torch.bfloat16 or n % 128 != 0:
        raise ValueError("w8x3_residual_next_adarms: residual must be bf16 [M, N], N % 128 == 0")
    for t, name in ((gate, "gate"), (next_scale, "next_scale")):
        if t.dtype != torch.float32 or t.numel() != n or t.stride(-1) != 1:
            raise TypeError(f"w8x3_residual_next_adarms: {name} must be fp32 [N] with unit stride")
    y = torch.empty((m, n), dtype=torch.bfloat16, device=planes.device)
    up = torch.empty((3, m, n), dtype=torch.uint8, device=planes.device)
    part = torch.empty((n // 128, m), dtype=torch.float32, device=planes.device)
    rc = lib.tybok_w8x3_residual_next_adarms(planes.data_ptr(), int(shift), w8.data_ptr(), scale.data_ptr(), y.data_ptr(), n,
                                             res2.data_ptr(), res2.stride(0), gate.data_ptr(), next_scale.data_ptr(),
                                             up.data_ptr(), int(out_shift), part.data_ptr(), m, n, k, int(token_tile),
                                             int(splits), status_word(planes.device).data_ptr(), _stream(planes))
    _lib.check(rc, "tybok_w8x3_residual_next_adarms")
    return y, up, part


def _w8x3_geglu_packed_adarms_cuda(u_planes, shift, ss_part, eps, bias_rows, w8_packed, scale_packed, out_bf16, out_planes,
                                   out_shift, token_tile, splits):
    lib = _lib.load()
    _check_w8(w8_packed, "w8x3_geglu_packed_adarms")
    n2, k = w8_packed.shape
    _check_scale(scale_packed, n2, "w8x3_geglu_packed_adarms")
    _check_fold_in(u_planes, ss_part, bias_rows, n2, "w8x3_geglu_packed_adarms")
    if u_planes.shape[2] != k:
        raise ValueError("w8x3_geglu_packed_adarms: planes and weight disagree on K")
    m = u_planes.shape[1]
    h, hp = _outputs(m, n2 // 2, u_planes.device, out_bf16, out_planes)
    rc = lib.tybok_w8x3_geglu_packed_adarms(u_planes.data_ptr(), int(shift), ss_part.data_ptr(), ss_part.shape[0], float(eps),
                                            bias_rows.data_ptr(), w8_packed.data_ptr(), scale_packed.data_ptr(),
                                            h.data_ptr() if out_bf16 else None, n2 // 2, hp.data_ptr() if out_planes else None,
                                            int(out_shift), m, n2 // 2, k, int(token_tile), int(splits),
                                            status_word(u_planes.device).data_ptr(), _stream(u_planes))
    _lib.check(rc, "tybok_w8x3_geglu_packed_adarms")
    return h, hp


def _w8x3_qkv_rope_adarms_cuda(u_planes, shift, ss_part, eps, bias_rows, w8_paired, scale_paired, pos, cos, sin, k_cache,
                               v_cache, heads, key_off, token_tile, splits):
    lib = _lib.load()
    _check_w8(w8_paired, "w8x3_qkv_rope_adarms")
    b, g, lcap, d = k_cache.shape
    _check_fold_in(u_planes, ss_part, bias_rows, w8_paired.shape[0], "w8x3_qkv_rope_adarms")
    _check_scale(scale_paired, w8_paired.shape[0], "w8x3_qkv_rope_adarms")
    m, k = u_planes.shape[1], u_planes.shape[2]
    if w8_paired.shape != ((heads + 2 * g) * d, k) or scale_paired.numel() != w8_paired.shape[0] or d % 128 != 0:
        raise ValueError("w8x3_qkv_rope_adarms: weight must be [(H+2G)*D, K] with head_dim % 128 == 0")
    if pos.dtype != torch.int32 or pos.numel() != m or not pos.is_contiguous() or m % b != 0:
        raise TypeError("w8x3_qkv_rope_adarms: pos must be contiguous int32 [B*L]")
    for t in (k_cache, v_cache, cos, sin):
        if t.dtype != torch.bfloat16 or not t.is_contiguous():
            raise TypeError("w8x3_qkv_rope_adarms: caches and cos/sin tables must be contiguous bf16")
    if v_cache.shape != k_cache.shape or cos.shape[-1] != d or sin.shape != cos.shape:
        raise ValueError("w8x3_qkv_rope_adarms: cache / table shapes disagree")
    q = torch.empty((m, heads * d), dtype=torch.bfloat16, device=u_planes.device)
    rc = lib.tybok_w8x3_qkv_rope_adarms(u_planes.data_ptr(), int(shift), ss_part.data_ptr(), ss_part.shape[0], float(eps),
                                        bias_rows.data_ptr(), w8_paired.data_ptr(), scale_paired.data_ptr(), pos.data_ptr(),
                                        cos.data_ptr(), sin.data_ptr(), q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(),
                                        b, m // b, heads, g, d, lcap, int(key_off), k, int(token_tile), int(splits),
                                        status_word(u_planes.device).data_ptr(), _stream(u_planes))
    _lib.check(rc, "tybok_w8x3_qkv_rope_adarms")
    return q


_L.impl("w8x3_residual_next_adarms", _w8x3_residual_next_adarms_cuda, "CUDA")
_L.impl("w8x3_geglu_packed_adarms", _w8x3_geglu_packed_adarms_cuda, "CUDA")
_L.impl("w8x3_qkv_rope_adarms", _w8x3_qkv_rope_adarms_cuda, "CUDA")


def w8x3_residual_next_adarms(planes, shift, w8, scale, residual, gate, next_scale, *, out_shift=0, token_tile=0, splits=0):
    """``x_new = residual + gate * (W8 a)`` with the next AdaRMS norm's input prepared in the epilogue:
    returns ``(x_new bf16 [M, N], u_planes [3, M, N] of bf16(x_new * (1 + next_scale)) * 2**out_shift,
    ss_part [N / 128, M])``; see ``tybok_w8x3_residual_next_adarms``."""
    return torch.ops.tybok_b200.w8x3_residual_next_adarms(planes, shift, w8, scale, residual, gate, next_scale, out_shift,
                                                          token_tile, splits)


def w8x3_geglu_packed_adarms(u_planes, shift, ss_part, bias_rows, w8_packed, scale_packed, *, eps=1e-6, out_bf16=True,
                             out_planes=False, out_shift=DEFAULT_SHIFT, token_tile=0, splits=0):
    """``w8x3_geglu_packed`` on the output of ``w8x3_residual_next_adarms`` (the norm's rstd and ``W shift``
    applied in the epilogue); see ``tybok_w8x3_geglu_packed_adarms``."""
    return torch.ops.tybok_b200.w8x3_geglu_packed_adarms(u_planes, shift, ss_part, eps, bias_rows, w8_packed, scale_packed,
                                                         out_bf16, out_planes, out_shift, token_tile, splits)


def w8x3_qkv_rope_adarms(u_planes, shift, ss_part, bias_rows, w8_paired, scale_paired, pos, cos, sin, k_cache, v_cache, *,
                         heads, key_off, eps=1e-6, token_tile=0, splits=0):
    """``w8x3_qkv_rope`` on the output of ``w8x3_residual_next_adarms``; see ``tybok_w8x3_qkv_rope_adarms``."""
    return torch.ops.tybok_b200.w8x3_qkv_rope_adarms(u_planes, shift, ss_part, eps, bias_rows, w8_paired, scale_paired, pos,
                                                     cos, sin, k_cache, v_cache, heads, key_off, token_tile, splits)


def shift_bias_rows(w8_rows: torch.Tensor, scale_rows: torch.Tensor, shift_row: torch.Tensor) -> torch.Tensor:
    """``W shift`` for the folded AdaRMS form: dequantised weight rows (in the order the kernel streams
    them) times the norm's shift row, fp32 ``[rows]``."""
    w = w8_rows.view(torch.float8_e4m3fn).float() if w8_rows.dtype == torch.uint8 else w8_rows.float()
    return ((w @ shift_row.reshape(-1).float()) * scale_rows.reshape(-1).float()).contiguous()


def launch_count() -> int:
    return int(_lib.load().tybok_launch_count())
