"""TEST INFRASTRUCTURE -- CPU restatement of the reference's fastWAM DiT block and denoise loop.

Functional torch code over a flat ``{name: tensor}`` dict whose keys are the parameter paths of
``FastWAMAttentionBlock`` (``self_attn.q.weight`` ... ``ffn.2.bias``, ``modulation``).  The six
projections and the two FFN matrices may be stored as e4m3 weight + ``scale_weight``; they are
dequantised to bf16 as the reference's loader does (tybok/policies/fastwam/models/policy.py:48-58)
and run through the unmodified eager math, every bf16 rounding point included.  Only tests,
``smoke()`` and the CPU-baseline legs of ``bench.py`` import this file.

Pinned against ``FastWAMAttentionBlock.forward`` itself by ``tests/golden/make_golden.py`` (fixture
``dit_block`` / ``dit_block_video_kv``).
"""

from __future__ import annotations

import numpy as np
import torch
import torch.nn.functional as F  # noqa: N812

from . import w8_ref as R


def _weight(p: dict, name: str) -> torch.Tensor:
    w = p[f"{name}.weight"]
    if w.dtype == torch.float8_e4m3fn:
        return R.dequant_w8(w, p[f"{name}.scale_weight"])
    return w


def _linear(p: dict, name: str, x: torch.Tensor) -> torch.Tensor:
    w = _weight(p, name)
    return F.linear(x.to(w.dtype), w, p.get(f"{name}.bias"))  # _linear_input: cast to the bf16 weight dtype


def wan_rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """``WanRMSNorm.forward`` (tybok/policies/fastwam/models/wan_base.py:114-128): RMS over the whole
    last dimension in fp32, cast back, times the weight."""
    xf = x.float()
    return (xf * torch.rsqrt(xf.pow(2).mean(dim=-1, keepdim=True) + eps)).type_as(x) * weight


def wan_layer_norm(x: torch.Tensor, eps: float, weight=None, bias=None) -> torch.Tensor:
    """``_wan_layer_norm`` (wan_base.py:131-148): fp32 statistics (and fp32 affine), cast back."""
    w = None if weight is None else weight.float()
    b = None if bias is None else bias.float()
    return F.layer_norm(x.float(), (x.shape[-1],), w, b, eps).to(x.dtype)


def apply_dense_rope(x: torch.Tensor, freqs: torch.Tensor, num_heads: int) -> torch.Tensor:
    """wan_base.py:97-108: adjacent pairs rotated by the complex table ``freqs [S, 1, d/2]`` in fp32."""
    b, s, _ = x.shape
    xh = x.view(b, s, num_heads, -1)
    xc = torch.view_as_complex(xh.to(torch.float32).reshape(b, s, num_heads, -1, 2))
    out = torch.view_as_real(xc * freqs.to(torch.complex64)).flatten(2)
    return out.to(x.dtype)


def masked_attention(q, k, v, num_heads: int, mask=None) -> torch.Tensor:
    """``fastwam_masked_attention`` with the default fp32 upcast (dit_block.py:72-98); fp32 out."""
    b = q.shape[0]
    q, k, v = (t.view(b, t.shape[1], num_heads, -1).permute(0, 2, 1, 3).float() for t in (q, k, v))
    x = F.scaled_dot_product_attention(q, k, v, attn_mask=mask)
    return x.permute(0, 2, 1, 3).reshape(b, x.shape[2], -1)


def cross_kv(p: dict, context: torch.Tensor, eps: float = 1e-6):
    """Keys (qk-normed) and values of the cross attention for a context ``[B, C, H]``
    (dit_block.py:255-266, the part ``precompute_action_context`` caches across steps)."""
    k = wan_rms_norm(_linear(p, "cross_attn.k", context), p["cross_attn.norm_k.weight"], eps)
    return k, _linear(p, "cross_attn.v", context)


def block_forward(p: dict, num_heads: int, x, context, t_mod, freqs, context_mask=None, video_kv=None,
                  eps: float = 1e-6, return_kv: bool = False):
    """``FastWAMAttentionBlock.forward`` (dit_block.py:328-400) on ``x [B, S, H]`` bf16:
    modulated self-attention with gated residual, cross-attention over ``context [B, C, H]``
    (``context_mask`` bool ``[B, C]`` or broadcastable), modulated FFN with gated residual.
    ``t_mod [B, 6, H]``; ``freqs`` complex ``[S, 1, d/2]``; ``video_kv`` = ``(k, v)`` ``[B, Lv, n*d]``
    prepended to this block's keys."""
    shift_msa, scale_msa, gate_msa, shift_mlp, scale_mlp, gate_mlp = (p["modulation"].to(t_mod.dtype) + t_mod).chunk(6, dim=1)
    h = wan_layer_norm(x, eps) * (1 + scale_msa) + shift_msa
    q = wan_rms_norm(_linear(p, "self_attn.q", h), p["self_attn.norm_q.weight"], eps)
    k = wan_rms_norm(_linear(p, "self_attn.k", h), p["self_attn.norm_k.weight"], eps)
    v = _linear(p, "self_attn.v", h)
    q, k = apply_dense_rope(q, freqs, num_heads), apply_dense_rope(k, freqs, num_heads)
    k_att, v_att = k, v
    if video_kv is not None:
        k_att, v_att = torch.cat([video_kv[0], k], dim=1), torch.cat([video_kv[1], v], dim=1)
    y = masked_attention(q, k_att, v_att, num_heads)
    x = x + gate_msa * _linear(p, "self_attn.o", y)
    if context is not None:
        hc = wan_layer_norm(x, eps, p["norm3.weight"], p["norm3.bias"])
        qc = wan_rms_norm(_linear(p, "cross_attn.q", hc), p["cross_attn.norm_q.weight"], eps)
        kc, vc = cross_kv(p, context, eps)
        mask = None
        if context_mask is not None:
            mask = context_mask.reshape(context_mask.shape[0], 1, 1, -1) if context_mask.dim() == 2 else context_mask
        x = x + _linear(p, "cross_attn.o", masked_attention(qc, kc, vc, num_heads, mask))
    m = wan_layer_norm(x, eps) * (1 + scale_mlp) + shift_mlp
    out = x + gate_mlp * _linear(p, "ffn.2", R.gelu_tanh(_linear(p, "ffn.0", m)))
    return (out, (k, v)) if return_kv else out


def sampling_deltas(steps: int, shift: float = 5.0) -> list[float]:
    """Step sizes ``sigma_{i+1} - sigma_i`` of the shifted flow schedule
    (tybok/policies/fastwam/models/fastwam.py:35-66)."""
    sigma = np.linspace(1, 0, steps + 1)[:steps]
    sigma = shift * sigma / (1 + (shift - 1) * sigma)
    sig = torch.as_tensor(sigma, dtype=torch.float32)
    nxt = torch.cat([sig[1:], sig.new_zeros(1)])
    return [float(d) for d in (nxt - sig)]


@torch.no_grad()
def denoise(blocks: list[dict], num_heads: int, x, context, t_mods, freqs, context_mask, deltas):
    """The denoise loop over token space: per step all blocks in order, then the scheduler's update
    ``x + model_output * delta`` in the activation dtype (fastwam.py:68-73)."""
    for t_mod, delta in zip(t_mods, deltas):
        y = x
        for p in blocks:
            y = block_forward(p, num_heads, y, context, t_mod, freqs, context_mask)
        x = x + y * torch.tensor(delta, dtype=x.dtype)
    return x
