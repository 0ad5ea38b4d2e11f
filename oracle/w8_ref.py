"""TEST INFRASTRUCTURE -- CPU restatement of the reference's W8 linear / FFN / attention math.

This file is the parity oracle for the CUDA kernels.  Only ``tests/``,
``__graft_entry__.smoke()`` and the ``cpu_baseline`` / ``--impl reference`` legs of
``bench.py`` may import it; the product package never does.

Every function restates one reference function in plain torch and cites it.  The
restatement is pinned in two ways (``tests/test_oracle.py``): against fixtures under
``tests/golden/`` that were produced by importing the reference itself
(``tests/golden/make_golden.py``), and against the closed-form identities the
reference documents for its quantiser (docs/fastWAM_weight_quantization.md:26-30,141-158).
"""

from __future__ import annotations

import math

import torch
import torch.nn.functional as F  # noqa: N812

FP8_MAX = 448.0
MASK_VALUE = -2.3819763e38  # tybok/policies/pi05/models/flow_matching.py:24


def quantize_w8(w: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """Per-output-channel e4m3 quantisation.

    Follows ``FP8Linear.from_linear`` (tybok/policies/fastwam/models/fp8_linear.py:299-310):
    fp32 row absmax / 448 clamped at 1e-12, then a round-to-nearest-even cast."""
    w = w.float()
    scale = (w.abs().amax(dim=1) / FP8_MAX).clamp_min(1e-12)
    return (w / scale[:, None]).to(torch.float8_e4m3fn).contiguous(), scale


def dequant_w8(w8: torch.Tensor, scale: torch.Tensor) -> torch.Tensor:
    """e4m3 + per-row fp32 scale -> bf16 weight.

    Follows ``_dequant_fp8_weight`` (tybok/policies/fastwam/models/policy.py:48-58):
    the product is formed in fp32 and rounded to bf16 once, per weight."""
    if w8.dtype != torch.float8_e4m3fn:
        raise TypeError(f"expected float8_e4m3fn weight, got {w8.dtype}")
    return (w8.float() * scale.float().unsqueeze(1)).to(torch.bfloat16)


def w8_linear(x: torch.Tensor, w8: torch.Tensor, scale: torch.Tensor, bias: torch.Tensor | None = None) -> torch.Tensor:
    """The W8A16 linear oracle: ``F.linear`` on the dequantised bf16 weight
    (the loader path of tybok/policies/fastwam/models/policy.py:127-129)."""
    return F.linear(x, dequant_w8(w8, scale), bias)


def gelu_tanh(x: torch.Tensor) -> torch.Tensor:
    """tybok/policies/pi05/models/layers.py:22-24."""
    return F.gelu(x, approximate="tanh")


def gemma_mlp(x, gate, up, down) -> torch.Tensor:
    """Gated FFN ``down(gelu_tanh(gate(x)) * up(x))`` (tybok/policies/pi05/models/layers.py:87-95).
    ``gate``/``up``/``down`` are ``(w8, scale)`` pairs; every op rounds to bf16 like the
    reference's bf16 modules do."""
    g = w8_linear(x, *gate)
    u = w8_linear(x, *up)
    return w8_linear(gelu_tanh(g) * u, *down)


def dit_ffn(x, up, down) -> torch.Tensor:
    """Ungated FFN with bias ``down(gelu_tanh(up(x)))``
    (tybok/policies/fastwam/models/dit_block.py:197-201). ``up``/``down`` are
    ``(w8, scale, bias)`` triples."""
    return w8_linear(gelu_tanh(w8_linear(x, *up)), *down)


def dit_ffn_tail(x, shift, scale, gate, up, down, eps: float = 1e-6) -> torch.Tensor:
    """FFN tail of a DiT block: ``x + gate * ffn(modulate(LN(x), shift, scale))``
    (tybok/policies/fastwam/models/dit_block.py:67-69,392-397; wan_base.py:131-148): LayerNorm
    without affine in fp32 cast back to bf16, every modulation op in bf16.  ``up``/``down`` are
    ``(w8, scale, bias)`` triples; ``shift``/``scale``/``gate`` broadcast over tokens."""
    n = F.layer_norm(x.float(), (x.shape[-1],), None, None, eps).type_as(x)
    h = n * (1 + scale) + shift
    return x + gate * dit_ffn(h, up, down)


def rms_norm(x: torch.Tensor, eps: float = 1e-6) -> torch.Tensor:
    """``x * rsqrt(mean(x^2) + eps)`` with fp32 statistics
    (tybok/policies/pi05/models/layers.py:51-53). The product promotes to fp32."""
    var = torch.mean(torch.square(x.float()), dim=-1, keepdim=True)
    return x * torch.rsqrt(var + eps)


def gemma_norm(x: torch.Tensor, weight: torch.Tensor, eps: float = 1e-6) -> torch.Tensor:
    """Plain Gemma RMSNorm (tybok/policies/pi05/models/layers.py:68-71)."""
    return (rms_norm(x, eps) * (1.0 + weight.float())).type_as(x)


def adarms_norm(x: torch.Tensor, modulation: torch.Tensor, eps: float = 1e-6):
    """AdaRMS norm with a precomputed ``dense(cond)`` (layers.py:72-84): returns
    ``(normed, gate)``; a ``2*dim`` modulation has no gate."""
    dim = x.shape[-1]
    normed = rms_norm(x, eps)
    if x.dim() == 3:
        modulation = modulation.unsqueeze(1)
    if modulation.shape[-1] == 2 * dim:
        scale, shift = modulation.chunk(2, dim=-1)
        return (normed * (1 + scale.float()) + shift.float()).to(x.dtype), None
    scale, shift, gate = modulation.chunk(3, dim=-1)
    return (normed * (1 + scale.float()) + shift.float()).to(x.dtype), gate.to(x.dtype)


def rope_cos_sin(position_ids: torch.Tensor, head_dim: int, dtype, theta: float = 10000.0):
    """Gemma RoPE tables (tybok/policies/pi05/models/rope.py:19-46): bf16-rounded inverse
    frequencies, fp32 angles, cos/sin cast to the activation dtype."""
    inv_freq = 1.0 / (theta ** (torch.arange(0, head_dim, 2, dtype=torch.int64).float() / head_dim))
    inv_freq = inv_freq.to(torch.bfloat16).float()
    freqs = position_ids[:, :, None].float() * inv_freq[None, None, :]
    emb = torch.cat((freqs, freqs), dim=-1)
    return emb.cos().to(dtype), emb.sin().to(dtype)


def rotate_half(x: torch.Tensor) -> torch.Tensor:
    """rope.py:49-52."""
    h = x.shape[-1] // 2
    return torch.cat((-x[..., h:], x[..., :h]), dim=-1)


def apply_rope(q, k, cos, sin):
    """rope.py:67-75; q/k ``[B,H,L,D]``, cos/sin ``[B,L,D]``."""
    cos, sin = cos.unsqueeze(1), sin.unsqueeze(1)
    return q * cos + rotate_half(q) * sin, k * cos + rotate_half(k) * sin


def gqa_attention(q, k, v, mask, scaling: float) -> torch.Tensor:
    """Eager GQA attention core (tybok/policies/pi05/models/layers.py:166-189):
    q ``[B,H,Lq,D]``, k/v ``[B,Hkv,Lk,D]`` (already ``[prefix ; suffix]``), additive fp32
    ``mask`` ``[B,1,Lq,Lk]``; logits in the activation dtype, softmax in fp32, output
    ``[B,Lq,H*D]``."""
    b, h, lq, d = q.shape
    rep = h // k.shape[1]
    if rep > 1:
        k = k[:, :, None].expand(b, k.shape[1], rep, k.shape[2], d).reshape(b, h, -1, d)
        v = v[:, :, None].expand(b, v.shape[1], rep, v.shape[2], d).reshape(b, h, -1, d)
    w = torch.matmul(q, k.transpose(2, 3)) * scaling
    if mask is not None:
        w = w + mask
    w = F.softmax(w, dim=-1, dtype=torch.float32).to(q.dtype)
    out = torch.matmul(w, v)
    return out.transpose(1, 2).contiguous().reshape(b, lq, h * d)


def gated_residual(x, y, gate):
    """layers.py:27-31."""
    return x + y if gate is None else x + y * gate


def sinusoidal_embedding(time: torch.Tensor, dim: int, min_period: float, max_period: float) -> torch.Tensor:
    """fp64 sine/cosine time embedding (flow_matching.py:153-168), returned in fp64."""
    fraction = torch.linspace(0.0, 1.0, dim // 2, dtype=torch.float64)
    period = min_period * (max_period / min_period) ** fraction
    scaling = 1.0 / period * 2 * math.pi
    s = scaling[None, :] * time[:, None]
    return torch.cat([torch.sin(s), torch.cos(s)], dim=1)


def rel_l2(a: torch.Tensor, b: torch.Tensor) -> float:
    """``||a-b||_2 / ||b||_2`` in fp64 -- the metric of every GEMM/FFN tolerance."""
    a, b = a.double().flatten(), b.double().flatten()
    return float((a - b).norm() / b.norm().clamp_min(1e-30))
