"""Callables with the reference's per-module hook signatures, backed by the fp8 kernels.

The reference swaps tiers in by assigning callables onto its own model objects:
``layer.mlp.forward = fn(x[B,L,W])`` (tybok/policies/pi05/engine.py:296-298) and
``blk._fused_ffn_tail = fn(x, shift_mlp, scale_mlp, gate_mlp)``
(tybok/policies/fastwam/models/dit_block.py:205-210,392-394).  The two factories here build such
callables from a module of the reference (or anything with the same attributes), so a reference
model object can run its FFNs on this package without any other change:

    for layer in vlm.layers:
        layer.mlp.forward = make_mlp_forward(layer.mlp)
    for blk in dit.blocks:
        blk._fused_ffn_tail = make_fused_ffn_tail(blk)

Weights are read once, at construction: an ``nn.Linear``-like ``.weight`` (any float dtype, quantised
here with the reference recipe) or an ``FP8Linear``-like pair ``.weight`` (e4m3) + ``.weight_scale``.
The callables take CUDA tensors and raise for anything else; there is no CPU path.
"""

from __future__ import annotations

import torch

from . import ops
from .dit import SHIFT_HIDDEN, SHIFT_IN
from .weights import quantize_w8

SHIFT_X = 4
SHIFT_H = 4


def _w8(linear, device) -> tuple[torch.Tensor, torch.Tensor]:
    w = linear.weight.detach()
    if w.dtype == torch.float8_e4m3fn:
        scale = getattr(linear, "weight_scale", None)
        if scale is None:
            raise TypeError("an e4m3 weight needs its per-output-channel `weight_scale`")
        return w.to(device).contiguous(), scale.detach().to(device).float().reshape(-1).contiguous()
    return quantize_w8(w.to(device))


def _bias(linear, device):
    b = getattr(linear, "bias", None)
    return None if b is None else b.detach().to(device, torch.bfloat16).contiguous()


def _rows(x: torch.Tensor) -> torch.Tensor:
    if not x.is_cuda:
        raise RuntimeError("tybok_b200 hooks run on CUDA tensors only: there is no CPU path")
    x2 = x.reshape(-1, x.shape[-1])
    return (x2 if x2.dtype == torch.bfloat16 else x2.to(torch.bfloat16)).contiguous()


def make_mlp_forward(mlp, device: str | torch.device = "cuda"):
    """``fn(x [B, L, W]) -> [B, L, W]`` computing ``down(gelu_tanh(gate(x)) * up(x))`` of a
    ``GemmaMLP`` (tybok/policies/pi05/models/layers.py:87-95): bf16 -> planes, one gate/up GEMM
    whose epilogue writes the planes of the intermediate, the down projection."""
    gate, up, down = _w8(mlp.gate_proj, device), _w8(mlp.up_proj, device), _w8(mlp.down_proj, device)
    packed = ops.pack_gate_up(*gate, *up) if gate[0].shape[0] % 64 == 0 else None

    def forward(x: torch.Tensor) -> torch.Tensor:
        xp = ops.split3(_rows(x), SHIFT_X)
        if packed is not None:
            _, hp = ops.w8x3_geglu_packed(xp, SHIFT_X, *packed, out_bf16=False, out_planes=True, out_shift=SHIFT_H)
        else:
            _, hp = ops.w8x3_geglu(xp, SHIFT_X, *gate, *up, out_bf16=False, out_planes=True, out_shift=SHIFT_H)
        y, _ = ops.w8x3_linear(hp, SHIFT_H, *down)
        return y.view(*x.shape[:-1], y.shape[-1]).to(x.dtype)

    return forward


def make_fused_ffn_tail(blk, device: str | torch.device = "cuda"):
    """``fn(x [B, S, H], shift_mlp, scale_mlp, gate_mlp) -> [B, S, H]`` computing
    ``x + gate_mlp * ffn(modulate(norm2(x), shift_mlp, scale_mlp))`` of a ``FastWAMAttentionBlock``
    (tybok/policies/fastwam/models/dit_block.py:392-397).  The three modulation tensors hold one row
    of ``H`` values per batch element (``[B, 1, H]``, ``[1, 1, H]`` or ``[H]``; strided views of the
    ``[B, 6, H]`` table are fine); each batch element is one launch chain."""
    up = (*_w8(blk.ffn[0], device), _bias(blk.ffn[0], device))
    down = (*_w8(blk.ffn[2], device), _bias(blk.ffn[2], device))
    eps = float(getattr(blk, "eps", 1e-6))

    def mod_row(t: torch.Tensor, b: int, h: int) -> torch.Tensor:
        t = t.reshape(-1, h)
        return t[b if t.shape[0] > 1 else 0].to(torch.bfloat16).contiguous()

    def tail(x: torch.Tensor, shift_mlp: torch.Tensor, scale_mlp: torch.Tensor, gate_mlp: torch.Tensor) -> torch.Tensor:
        if not x.is_cuda:
            raise RuntimeError("tybok_b200 hooks run on CUDA tensors only: there is no CPU path")
        x3 = x if x.dim() == 3 else x[None]
        h = x3.shape[-1]
        outs = []
        for b in range(x3.shape[0]):
            xb = _rows(x3[b])
            _, xp = ops.layernorm_modulate(xb, mod_row(shift_mlp, b, h), mod_row(scale_mlp, b, h), eps=eps,
                                           out_shift=SHIFT_IN)
            _, hp = ops.w8x3_linear(xp, SHIFT_IN, *up, epilogue=ops.EPI_GELU, out_bf16=False, out_planes=True,
                                    out_shift=SHIFT_HIDDEN)
            y, _ = ops.w8x3_linear(hp, SHIFT_HIDDEN, *down, epilogue=ops.EPI_RESIDUAL, residual=xb,
                                   gate=mod_row(gate_mlp, b, h).reshape(1, -1), rows_per_gate=xb.shape[0])
            outs.append(y)
        out = torch.stack(outs) if x.dim() == 3 else outs[0]
        return out.to(x.dtype)

    return tail
