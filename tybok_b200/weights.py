"""Weight containers: seeded random init, e4m3 per-output-channel quantisation.

Parameter names are the reference's module paths relative to ``PI05FlowMatching``
(tybok/policies/pi05/models/paligemma_with_expert.py, flow_matching.py:260-270), so a
state dict produced here loads into the reference's modules by name and a real
checkpoint loads into this package unchanged.

The quantisation recipe is the reference's ``FP8Linear.from_linear``
(tybok/policies/fastwam/models/fp8_linear.py:299-310):
``scale[n] = clamp_min(max_k |W[n,k]| / 448, 1e-12)`` in fp32 and
``W8 = RNE(W / scale[:, None])`` to e4m3fn.
"""

from __future__ import annotations

import torch

from .shapes import DiTShape, GemmaSpec, PI05Shape

FP8_MAX = 448.0
VLM = "paligemma_with_expert.paligemma.model.language_model"
EXPERT = "paligemma_with_expert.gemma_expert.model"
VISION = "paligemma_with_expert.paligemma.model.vision_tower.vision_model"
PROJECTOR = "paligemma_with_expert.paligemma.model.multi_modal_projector.linear"

#: Linear sub-modules of one Gemma decoder layer that run as W8 GEMMs.
HOT_LINEARS = (
    "self_attn.q_proj",
    "self_attn.k_proj",
    "self_attn.v_proj",
    "self_attn.o_proj",
    "mlp.gate_proj",
    "mlp.up_proj",
    "mlp.down_proj",
)


def quantize_w8(w: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """``W[N,K]`` (any float dtype) -> (``W8[N,K]`` float8_e4m3fn, ``scale[N]`` fp32)."""
    w = w.float()
    scale = (w.abs().amax(dim=1) / FP8_MAX).clamp_min(1e-12)
    w8 = (w / scale[:, None]).to(torch.float8_e4m3fn).contiguous()
    return w8, scale


def hot_linear_names(shape: PI05Shape) -> list[str]:
    """Every linear of the pi0.5-shaped policy that is stored as e4m3 (weight key names)."""
    names = []
    for root, spec in ((VLM, shape.vlm), (EXPERT, shape.expert)):
        for i in range(spec.depth):
            names += [f"{root}.layers.{i}.{lin}.weight" for lin in HOT_LINEARS]
    return names


def _normal(gen: torch.Generator, shape, dtype, device, std=0.02) -> torch.Tensor:
    # Generated in fp32 and cast, so the values do not depend on the target dtype.
    t = torch.empty(shape, dtype=torch.float32, device=device)
    t.normal_(0.0, std, generator=gen)
    return t.to(dtype)


def _gemma_params(p, gen, root: str, spec: GemmaSpec, adarms: bool, device):
    bf16, f32 = torch.bfloat16, torch.float32
    qd, kvd = spec.num_heads * spec.head_dim, spec.num_kv_heads * spec.head_dim
    for i in range(spec.depth):
        base = f"{root}.layers.{i}"
        p[f"{base}.self_attn.q_proj.weight"] = _normal(gen, (qd, spec.width), bf16, device)
        p[f"{base}.self_attn.k_proj.weight"] = _normal(gen, (kvd, spec.width), bf16, device)
        p[f"{base}.self_attn.v_proj.weight"] = _normal(gen, (kvd, spec.width), bf16, device)
        p[f"{base}.self_attn.o_proj.weight"] = _normal(gen, (spec.width, qd), bf16, device)
        p[f"{base}.mlp.gate_proj.weight"] = _normal(gen, (spec.mlp_dim, spec.width), bf16, device)
        p[f"{base}.mlp.up_proj.weight"] = _normal(gen, (spec.mlp_dim, spec.width), bf16, device)
        p[f"{base}.mlp.down_proj.weight"] = _normal(gen, (spec.width, spec.mlp_dim), bf16, device)
        for norm in ("input_layernorm", "post_attention_layernorm"):
            if adarms:
                p[f"{base}.{norm}.dense.weight"] = _normal(gen, (3 * spec.width, spec.width), f32, device)
                p[f"{base}.{norm}.dense.bias"] = _normal(gen, (3 * spec.width,), f32, device)
            else:
                p[f"{base}.{norm}.weight"] = _normal(gen, (spec.width,), f32, device)
    if adarms:
        p[f"{root}.norm.dense.weight"] = _normal(gen, (3 * spec.width, spec.width), f32, device)
        p[f"{root}.norm.dense.bias"] = _normal(gen, (3 * spec.width,), f32, device)
    else:
        p[f"{root}.norm.weight"] = _normal(gen, (spec.width,), f32, device)


def random_pi05_params(shape: PI05Shape, seed: int = 0, device: str = "cpu") -> dict[str, torch.Tensor]:
    """Seeded N(0, 0.02) parameters of a pi0.5-shaped policy, in the dtypes the reference
    engine builds them in (decoders bf16; vision, norms, AdaRMS and action/time
    projections fp32 -- tybok/policies/pi05/engine.py:184-189)."""
    gen = torch.Generator(device=device).manual_seed(seed)
    f32, bf16 = torch.float32, torch.bfloat16
    p: dict[str, torch.Tensor] = {}
    v = shape.vision
    p[f"{VISION}.embeddings.patch_embedding.weight"] = _normal(gen, (v.hidden, 3, v.patch, v.patch), f32, device)
    p[f"{VISION}.embeddings.patch_embedding.bias"] = _normal(gen, (v.hidden,), f32, device)
    p[f"{VISION}.embeddings.position_embedding.weight"] = _normal(gen, (v.tokens, v.hidden), f32, device)
    for i in range(v.layers):
        base = f"{VISION}.encoder.layers.{i}"
        for ln in ("layer_norm1", "layer_norm2"):
            p[f"{base}.{ln}.weight"] = 1.0 + _normal(gen, (v.hidden,), f32, device)
            p[f"{base}.{ln}.bias"] = _normal(gen, (v.hidden,), f32, device)
        for lin in ("q_proj", "k_proj", "v_proj", "out_proj"):
            p[f"{base}.self_attn.{lin}.weight"] = _normal(gen, (v.hidden, v.hidden), f32, device)
            p[f"{base}.self_attn.{lin}.bias"] = _normal(gen, (v.hidden,), f32, device)
        p[f"{base}.mlp.fc1.weight"] = _normal(gen, (v.mlp_dim, v.hidden), f32, device)
        p[f"{base}.mlp.fc1.bias"] = _normal(gen, (v.mlp_dim,), f32, device)
        p[f"{base}.mlp.fc2.weight"] = _normal(gen, (v.hidden, v.mlp_dim), f32, device)
        p[f"{base}.mlp.fc2.bias"] = _normal(gen, (v.hidden,), f32, device)
    p[f"{VISION}.post_layernorm.weight"] = 1.0 + _normal(gen, (v.hidden,), f32, device)
    p[f"{VISION}.post_layernorm.bias"] = _normal(gen, (v.hidden,), f32, device)
    p[f"{PROJECTOR}.weight"] = _normal(gen, (shape.vlm.width, v.hidden), f32, device)
    p[f"{PROJECTOR}.bias"] = _normal(gen, (shape.vlm.width,), f32, device)
    p[f"{VLM}.embed_tokens.weight"] = _normal(gen, (shape.vocab, shape.vlm.width), bf16, device)
    _gemma_params(p, gen, VLM, shape.vlm, False, device)
    _gemma_params(p, gen, EXPERT, shape.expert, True, device)
    ew = shape.expert.width
    p["action_in_proj.weight"] = _normal(gen, (ew, shape.max_action_dim), f32, device)
    p["action_in_proj.bias"] = _normal(gen, (ew,), f32, device)
    p["action_out_proj.weight"] = _normal(gen, (shape.max_action_dim, ew), f32, device)
    p["action_out_proj.bias"] = _normal(gen, (shape.max_action_dim,), f32, device)
    for name in ("time_mlp_in", "time_mlp_out"):
        p[f"{name}.weight"] = _normal(gen, (ew, ew), f32, device)
        p[f"{name}.bias"] = _normal(gen, (ew,), f32, device)
    return p


def quantize_hot_linears(params: dict[str, torch.Tensor], shape: PI05Shape) -> dict[str, torch.Tensor]:
    """Replace every hot-path ``<lin>.weight`` by ``<lin>.weight`` (e4m3) + ``<lin>.scale_weight``
    (fp32), the on-disk form of the reference's fp8 checkpoints
    (docs/fastWAM_weight_quantization.md:14-24).  Weights that are already e4m3 are kept."""
    out = dict(params)
    for name in hot_linear_names(shape):
        w = out[name]
        if w.dtype == torch.float8_e4m3fn:
            continue
        w8, scale = quantize_w8(w)
        out[name] = w8
        out[name[: -len("weight")] + "scale_weight"] = scale
    return out


def random_dit_block_params(shape: DiTShape, seed: int = 0, device: str = "cpu") -> dict[str, torch.Tensor]:
    """Seeded N(0, 0.02) parameters of one ``FastWAMAttentionBlock``
    (tybok/policies/fastwam/models/dit_block.py:283-326)."""
    gen = torch.Generator(device=device).manual_seed(seed)
    bf16 = torch.bfloat16
    h, f = shape.hidden, shape.ffn
    p: dict[str, torch.Tensor] = {}
    for attn in ("self_attn", "cross_attn"):
        for lin in ("q", "k", "v", "o"):
            p[f"{attn}.{lin}.weight"] = _normal(gen, (h, h), bf16, device)
            p[f"{attn}.{lin}.bias"] = _normal(gen, (h,), bf16, device)
        p[f"{attn}.norm_q.weight"] = 1.0 + _normal(gen, (h,), bf16, device)
        p[f"{attn}.norm_k.weight"] = 1.0 + _normal(gen, (h,), bf16, device)
    p["norm3.weight"] = 1.0 + _normal(gen, (h,), bf16, device)
    p["norm3.bias"] = _normal(gen, (h,), bf16, device)
    p["ffn.0.weight"] = _normal(gen, (f, h), bf16, device)
    p["ffn.0.bias"] = _normal(gen, (f,), bf16, device)
    p["ffn.2.weight"] = _normal(gen, (h, f), bf16, device)
    p["ffn.2.bias"] = _normal(gen, (h,), bf16, device)
    p["modulation"] = _normal(gen, (1, 6, h), bf16, device, std=1.0 / h**0.5)
    return p


#: Linear sub-modules of one DiT block that run as W8 GEMMs.
DIT_HOT_LINEARS = ("self_attn.q", "self_attn.k", "self_attn.v", "self_attn.o", "cross_attn.q", "cross_attn.k",
                   "cross_attn.v", "cross_attn.o", "ffn.0", "ffn.2")


def quantize_dit_block(params: dict[str, torch.Tensor]) -> dict[str, torch.Tensor]:
    """The on-disk fp8 form of one DiT block: every projection and FFN matrix as e4m3 ``<lin>.weight``
    + fp32 ``<lin>.scale_weight`` (docs/fastWAM_weight_quantization.md:14-24); biases, norm weights and
    the modulation table stay bf16.  Weights that are already e4m3 are kept."""
    out = dict(params)
    for lin in DIT_HOT_LINEARS:
        w = out[f"{lin}.weight"]
        if w.dtype == torch.float8_e4m3fn:
            continue
        out[f"{lin}.weight"], out[f"{lin}.scale_weight"] = quantize_w8(w)
    return out
