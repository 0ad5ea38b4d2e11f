"""TEST INFRASTRUCTURE -- CPU restatement of the reference's pi0.5 eager inference path.

Functional torch code over a flat ``{name: tensor}`` dict whose keys are the reference's
parameter paths relative to ``PI05FlowMatching``.  Hot-path linears may be stored as
e4m3 weight + ``scale_weight``; they are dequantised to bf16 exactly as the reference's
loader does (tybok/policies/fastwam/models/policy.py:48-58,127-129) and then run through
the unmodified eager math.  Only tests, ``smoke()`` and the CPU-baseline legs of
``bench.py`` import this file.

Pinned against the reference's own modules at a small shape by
``tests/golden/make_golden.py`` (run where the reference is importable) and the fixture
it commits.
"""

from __future__ import annotations

import torch
import torch.nn.functional as F  # noqa: N812

from . import w8_ref as R

VLM = "paligemma_with_expert.paligemma.model.language_model"
EXPERT = "paligemma_with_expert.gemma_expert.model"
VISION = "paligemma_with_expert.paligemma.model.vision_tower.vision_model"
PROJECTOR = "paligemma_with_expert.paligemma.model.multi_modal_projector.linear"


def _weight(p: dict, name: str) -> torch.Tensor:
    """bf16/fp32 weight as stored, or the bf16 dequantisation of an e4m3 weight."""
    w = p[f"{name}.weight"]
    if w.dtype == torch.float8_e4m3fn:
        return R.dequant_w8(w, p[f"{name}.scale_weight"])
    return w


def _linear(p: dict, name: str, x: torch.Tensor) -> torch.Tensor:
    return F.linear(x, _weight(p, name), p.get(f"{name}.bias"))


# --------------------------------------------------------------------------- vision
def siglip_tower(p: dict, pixel_values: torch.Tensor, heads: int, patch: int, eps: float = 1e-6) -> torch.Tensor:
    """fp32 SigLIP tower incl. post_layernorm (tybok/policies/pi05/models/vision.py:22-36,
    39-68,71-95,117-181,200-289)."""
    x = F.conv2d(pixel_values.float(), p[f"{VISION}.embeddings.patch_embedding.weight"],
                 p[f"{VISION}.embeddings.patch_embedding.bias"], stride=patch)
    x = x.flatten(2).transpose(1, 2) + p[f"{VISION}.embeddings.position_embedding.weight"][None]
    hidden = x.shape[-1]
    hd = hidden // heads
    i = 0
    while f"{VISION}.encoder.layers.{i}.layer_norm1.weight" in p:
        base = f"{VISION}.encoder.layers.{i}"
        h = F.layer_norm(x, (hidden,), p[f"{base}.layer_norm1.weight"], p[f"{base}.layer_norm1.bias"], eps)
        b, l, _ = h.shape
        q = _linear(p, f"{base}.self_attn.q_proj", h).view(b, l, heads, hd).transpose(1, 2)
        k = _linear(p, f"{base}.self_attn.k_proj", h).view(b, l, heads, hd).transpose(1, 2)
        v = _linear(p, f"{base}.self_attn.v_proj", h).view(b, l, heads, hd).transpose(1, 2)
        a = F.scaled_dot_product_attention(q, k, v, scale=hd**-0.5)
        a = a.transpose(1, 2).contiguous().reshape(b, l, hidden)
        x = x + _linear(p, f"{base}.self_attn.out_proj", a)
        h = F.layer_norm(x, (hidden,), p[f"{base}.layer_norm2.weight"], p[f"{base}.layer_norm2.bias"], eps)
        h = _linear(p, f"{base}.mlp.fc2", R.gelu_tanh(_linear(p, f"{base}.mlp.fc1", h)))
        x = x + h
        i += 1
    return F.layer_norm(x, (hidden,), p[f"{VISION}.post_layernorm.weight"], p[f"{VISION}.post_layernorm.bias"], eps)


def embed_image(p: dict, image: torch.Tensor, heads: int, patch: int) -> torch.Tensor:
    """paligemma_with_expert.py:76-88,134-143: tower + fp32 projector."""
    return _linear(p, PROJECTOR, siglip_tower(p, image, heads, patch))


def embed_language(p: dict, tokens: torch.Tensor, width: int) -> torch.Tensor:
    """paligemma_with_expert.py:145-161: table lookup times ``bf16(sqrt(width))``."""
    emb = F.embedding(tokens, p[f"{VLM}.embed_tokens.weight"])
    return emb * torch.tensor(width**0.5, dtype=emb.dtype)


# --------------------------------------------------------------------------- decoder
def decoder_layer(p, base, spec, x, mask, cos, sin, prefix_kv, mods):
    """One ``GemmaDecoderLayer.forward`` (tybok/policies/pi05/models/layers.py:268-308).
    ``mods`` is ``None`` (plain Gemma norms) or ``(mod_in, mod_post)`` AdaRMS modulations."""
    h, hkv, d = spec.num_heads, spec.num_kv_heads, spec.head_dim
    res = x
    if mods is None:
        y, gate = R.gemma_norm(x, p[f"{base}.input_layernorm.weight"]), None
    else:
        y, gate = R.adarms_norm(x, mods[0])
    b, l, _ = y.shape
    q = _linear(p, f"{base}.self_attn.q_proj", y).view(b, l, h, d).transpose(1, 2)
    k = _linear(p, f"{base}.self_attn.k_proj", y).view(b, l, hkv, d).transpose(1, 2)
    v = _linear(p, f"{base}.self_attn.v_proj", y).view(b, l, hkv, d).transpose(1, 2)
    q, k = R.apply_rope(q, k, cos, sin)
    if prefix_kv is not None:
        k = torch.cat([prefix_kv[0], k], dim=2)
        v = torch.cat([prefix_kv[1], v], dim=2)
    a = R.gqa_attention(q, k, v, mask, d**-0.5)
    x = R.gated_residual(res, _linear(p, f"{base}.self_attn.o_proj", a), gate)
    res = x
    if mods is None:
        y, gate = R.gemma_norm(x, p[f"{base}.post_attention_layernorm.weight"]), None
    else:
        y, gate = R.adarms_norm(x, mods[1])
    g = _linear(p, f"{base}.mlp.gate_proj", y)
    u = _linear(p, f"{base}.mlp.up_proj", y)
    y = _linear(p, f"{base}.mlp.down_proj", R.gelu_tanh(g) * u)
    return R.gated_residual(res, y, gate), k, v


def make_att_2d_masks(pad_masks, att_masks):
    """flow_matching.py:171-176."""
    cumsum = torch.cumsum(att_masks, dim=1)
    att = cumsum[:, None, :] <= cumsum[:, :, None]
    pad = pad_masks[:, None, :] * pad_masks[:, :, None]
    return att & pad


def masks_4d(att_2d):
    """flow_matching.py:179-182."""
    return torch.where(att_2d[:, None], 0.0, R.MASK_VALUE)


def prefix_prefill(p, shape, prefix_embs, prefix_pad_masks):
    """VLM prefill with KV collection (gemma.py:61-125 with ``use_cache``; the final norm's
    output is unused by the policy and skipped). Returns per-layer post-RoPE ``(K, V)``."""
    spec = shape.vlm
    att = torch.zeros_like(prefix_pad_masks, dtype=torch.bool)
    mask = masks_4d(make_att_2d_masks(prefix_pad_masks, att))
    pos = torch.cumsum(prefix_pad_masks, dim=1) - 1
    x = prefix_embs.to(torch.bfloat16) if _weight(p, f"{VLM}.layers.0.self_attn.q_proj").dtype == torch.bfloat16 \
        else prefix_embs
    cos, sin = R.rope_cos_sin(pos, spec.head_dim, x.dtype)
    kv = []
    for i in range(spec.depth):
        x, k, v = decoder_layer(p, f"{VLM}.layers.{i}", spec, x, mask, cos, sin, None, None)
        kv.append((k, v))
    return kv


def adarms_cond(p, time_emb):
    """flow_matching.py:376-381."""
    c = F.silu(F.linear(time_emb, p["time_mlp_in.weight"], p["time_mlp_in.bias"]))
    return F.silu(F.linear(c, p["time_mlp_out.weight"], p["time_mlp_out.bias"]))


def denoise_step(p, shape, prefix_pad_masks, kv, x_t, timestep):
    """flow_matching.py:505-556 (eager branch): one expert pass -> velocity ``[B,chunk,A]`` fp32."""
    spec = shape.expert
    b = x_t.shape[0]
    temb = R.sinusoidal_embedding(timestep, spec.width, shape.min_period, shape.max_period).to(timestep.dtype)
    cond = adarms_cond(p, temb)
    x = F.linear(x_t, p["action_in_proj.weight"], p["action_in_proj.bias"])
    s = x.shape[1]
    suffix_pad = torch.ones(b, s, dtype=torch.bool)
    suffix_att = torch.tensor([1.0] + [0.0] * (s - 1))[None].expand(b, s)
    pre2d = prefix_pad_masks[:, None, :].expand(b, s, prefix_pad_masks.shape[1])
    mask = masks_4d(torch.cat([pre2d, make_att_2d_masks(suffix_pad, suffix_att)], dim=2))
    pos = torch.sum(prefix_pad_masks, dim=-1)[:, None] + torch.cumsum(suffix_pad, dim=1) - 1
    if _weight(p, f"{EXPERT}.layers.0.self_attn.q_proj").dtype == torch.bfloat16:
        x = x.to(torch.bfloat16)
    cos, sin = R.rope_cos_sin(pos, spec.head_dim, x.dtype)
    for i in range(spec.depth):
        base = f"{EXPERT}.layers.{i}"
        mods = tuple(
            F.linear(cond, p[f"{base}.{n}.dense.weight"], p[f"{base}.{n}.dense.bias"])
            for n in ("input_layernorm", "post_attention_layernorm")
        )
        x, _, _ = decoder_layer(p, base, spec, x, mask, cos, sin, kv[i], mods)
    final = F.linear(cond, p[f"{EXPERT}.norm.dense.weight"], p[f"{EXPERT}.norm.dense.bias"])
    x, _ = R.adarms_norm(x, final)
    x = x[:, -shape.chunk:].float()
    return F.linear(x, p["action_out_proj.weight"], p["action_out_proj.bias"])


@torch.no_grad()
def sample_actions(p, shape, images, img_masks, tokens, masks, noise, return_intermediates=False):
    """``PI05FlowMatching.sample_actions`` sequential branch (flow_matching.py:761-838):
    ``images`` list of ``[B,3,H,W]`` fp32 in [-1,1], ``img_masks`` list of ``[B]`` bool,
    ``tokens``/``masks`` ``[B,L]``, ``noise`` ``[B,chunk,A]`` fp32.  Returns ``[B,chunk,A]`` fp32."""
    embs, pads = [], []
    for img, m in zip(images, img_masks):
        e = embed_image(p, img, shape.vision.heads, shape.vision.patch)
        embs.append(e)
        pads.append(m[:, None].expand(e.shape[0], e.shape[1]))
    embs.append(embed_language(p, tokens, shape.vlm.width))
    pads.append(masks.bool())
    prefix_embs = torch.cat(embs, dim=1)  # fp32 by type promotion
    prefix_pad = torch.cat(pads, dim=1)
    kv = prefix_prefill(p, shape, prefix_embs, prefix_pad)
    dt = -1.0 / shape.steps
    x_t = noise
    vs = []
    for step in range(shape.steps):
        t = torch.tensor(1.0 + step * dt, dtype=torch.float32).expand(x_t.shape[0])
        v_t = denoise_step(p, shape, prefix_pad, kv, x_t, t)
        vs.append(v_t)
        x_t = x_t + dt * v_t
    if return_intermediates:
        return x_t, {"prefix_embs": prefix_embs, "kv": kv, "velocities": vs}
    return x_t
