"""Generate the golden fixtures in this directory by running the REFERENCE's own modules.

Run where the reference checkout is importable, with ``TYBOK_REFERENCE`` naming its root:

    TYBOK_REFERENCE=<reference checkout> PYTHONDONTWRITEBYTECODE=1 python tests/golden/make_golden.py

Inputs and weights are seeded (``tybok_b200.weights`` + the generators below), so the
fixtures hold only outputs plus an fp64 checksum of the inputs they belong to.  The
fixtures pin ``oracle/`` (tests/test_oracle.py) and, through it, the CUDA kernels.

Reference entry points exercised:
  * ``FP8Linear.from_linear``        tybok/policies/fastwam/models/fp8_linear.py:299-310
  * ``_dequant_fp8_weight``          tybok/policies/fastwam/models/policy.py:48-58
  * ``GemmaMLP`` / ``GemmaAttention`` / ``GemmaDecoderLayer``  tybok/policies/pi05/models/layers.py
  * ``PI05FlowMatching.sample_actions``  tybok/policies/pi05/models/flow_matching.py:761-838
"""

from __future__ import annotations

import os
import sys

import torch
from torch import nn

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
if "TYBOK_REFERENCE" in os.environ:  # only needed by main(); the seeded input generators import without it
    sys.path.insert(0, os.environ["TYBOK_REFERENCE"])
sys.dont_write_bytecode = True

from tybok_b200.shapes import PI05_TINY  # noqa: E402
from tybok_b200.weights import quantize_hot_linears, random_pi05_params  # noqa: E402


def checksum(*tensors) -> float:
    return float(sum(t.double().abs().sum() for t in tensors))


def tiny_inputs(shape, seed=0, batch=1):
    """Seeded synthetic request: images in [-1,1], token ids, all-ones masks, zero noise."""
    g = torch.Generator().manual_seed(seed)
    images = [torch.rand(batch, 3, shape.vision.image, shape.vision.image, generator=g) * 2 - 1
              for _ in range(shape.n_cams)]
    img_masks = [torch.ones(batch, dtype=torch.bool) for _ in range(shape.n_cams)]
    tokens = torch.randint(0, shape.vocab, (batch, shape.lang_len), generator=g)
    masks = torch.ones(batch, shape.lang_len, dtype=torch.bool)
    masks[:, shape.lang_len - 3:] = False  # a padded tail, so the pad mask is exercised
    noise = torch.zeros(batch, shape.chunk, shape.max_action_dim)
    return images, img_masks, tokens, masks, noise


def linear_case(seed, m, n, k):
    g = torch.Generator().manual_seed(seed)
    w = torch.empty(n, k).normal_(0, 0.02, generator=g)
    x = torch.empty(m, k).normal_(0, 1, generator=g).to(torch.bfloat16)
    return w, x


def dit_case(seed=4, m=70, h=256, f=512):
    """Seeded inputs of the DiT FFN-tail fixture: x [1,m,h] bf16, (shift, scale, gate) [1,1,h] bf16,
    and fp32 master weights/bf16 biases of the two FFN linears."""
    g = torch.Generator().manual_seed(seed)
    x = torch.empty(1, m, h).normal_(0, 1, generator=g).to(torch.bfloat16)
    mods = tuple(torch.empty(1, 1, h).normal_(0, 0.5, generator=g).to(torch.bfloat16) for _ in range(3))
    ws = [(torch.empty(f, h).normal_(0, 0.02, generator=g), torch.empty(f).normal_(0, 0.1, generator=g).to(torch.bfloat16)),
          (torch.empty(h, f).normal_(0, 0.02, generator=g), torch.empty(h).normal_(0, 0.1, generator=g).to(torch.bfloat16))]
    return x, mods, ws


def dit_block_case(shape, seed=8, video_prefix=0):
    """Seeded inputs of the whole-DiT-block fixtures: tokens, context with a padded tail, the
    per-step modulation table, the dense rotary table (complex, ``[S, 1, d/2]``) and, optionally,
    keys / values of ``video_prefix`` earlier tokens."""
    g = torch.Generator().manual_seed(seed)
    s, h, c = shape.seq, shape.hidden, shape.context_len
    x = torch.empty(1, s, h).normal_(0, 1, generator=g).to(torch.bfloat16)
    context = torch.empty(1, c, h).normal_(0, 1, generator=g).to(torch.bfloat16)
    context_mask = torch.ones(1, c, dtype=torch.bool)
    context_mask[:, c - 4:] = False
    t_mod = torch.empty(1, 6, h).normal_(0, 0.5, generator=g).to(torch.bfloat16)
    pos = torch.arange(video_prefix, video_prefix + s, dtype=torch.float64)
    inv = 1.0 / torch.pow(10000, torch.arange(0, shape.head_dim, 2, dtype=torch.float64) / shape.head_dim)
    ang = torch.outer(pos, inv)
    freqs = torch.polar(torch.ones_like(ang), ang)[:, None, :]
    video_kv = None
    if video_prefix:
        video_kv = tuple(torch.empty(1, video_prefix, shape.heads * shape.head_dim).normal_(0, 1, generator=g).to(torch.bfloat16)
                         for _ in range(2))
    return x, context, context_mask, t_mod, freqs, video_kv


def request_case(seed=6):
    """Seeded inputs of the request-path fixture: a state vector with its statistics, an action
    chunk with its statistics, and two non-square camera frames."""
    g = torch.Generator().manual_seed(seed)
    state = torch.empty(8).normal_(0, 1.5, generator=g)
    stats = {"observation.state.mean": torch.empty(8).normal_(0, 0.5, generator=g),
             "observation.state.std": torch.empty(8).uniform_(0.5, 2.0, generator=g),
             "action.mean": torch.empty(7).normal_(0, 0.5, generator=g),
             "action.std": torch.empty(7).uniform_(0.5, 2.0, generator=g)}
    actions = torch.empty(1, 10, 7).normal_(0, 1, generator=g)
    frames = [torch.rand(3, 96, 160, generator=g), torch.rand(3, 150, 75, generator=g)]
    return state, stats, actions, frames


def main() -> None:
    from tybok.policies.fastwam.models.fp8_linear import FP8Linear
    from tybok.policies.fastwam.models.policy import _dequant_fp8_weight
    from tybok.policies.pi05 import config as ref_config
    from tybok.policies.pi05.models.flow_matching import PI05FlowMatching
    from tybok.policies.pi05.models.layers import GemmaMLP
    from tybok.policies.pi05.models.paligemma_with_expert import PaliGemmaMultiModalProjector
    from tybok.policies.pi05.models.vision import SiglipVisionTransformer

    out: dict[str, object] = {}

    # ---- a1/a2: quantiser + dequant linear ------------------------------------------
    for tag, (m, n, k) in {"lin_small": (50, 256, 512), "lin_ragged": (7, 192, 320)}.items():
        w, x = linear_case(1, m, n, k)
        lin = nn.Linear(k, n, bias=False)
        lin.weight.data.copy_(w)
        q = FP8Linear.from_linear(lin)
        w8, scale = q.weight.data, q.weight_scale.data
        y = torch.nn.functional.linear(x, _dequant_fp8_weight(w8, scale))
        out[tag] = {"in_sum": checksum(w, x), "w8": w8.view(torch.uint8).clone(), "scale": scale.clone(), "y": y}

    # ---- a4: gated MLP on dequantised weights ----------------------------------------
    g = torch.Generator().manual_seed(2)
    mlp = GemmaMLP(256, 512)
    x = torch.empty(1, 50, 256).normal_(0, 1, generator=g).to(torch.bfloat16)
    ws = {}
    for name in ("gate_proj", "up_proj", "down_proj"):
        lin = getattr(mlp, name)
        w = torch.empty(lin.weight.shape).normal_(0, 0.02, generator=g)
        src = nn.Linear(w.shape[1], w.shape[0], bias=False)
        src.weight.data.copy_(w)
        q = FP8Linear.from_linear(src)
        lin.weight.data.copy_(_dequant_fp8_weight(q.weight.data, q.weight_scale.data))
        ws[name] = w
    with torch.no_grad():
        out["mlp"] = {"in_sum": checksum(x, *ws.values()), "y": mlp(x)}

    # ---- a6: DiT FFN tail on dequantised weights ---------------------------------------
    from tybok.policies.fastwam.models.dit_block import FastWAMAttentionBlock, modulate

    x, mods, ws = dit_case()
    torch.set_default_dtype(torch.bfloat16)
    try:
        blk = FastWAMAttentionBlock(256, 128, 2, 512)
    finally:
        torch.set_default_dtype(torch.float32)
    for idx, (w, b) in zip((0, 2), ws):
        src = nn.Linear(w.shape[1], w.shape[0], bias=False)
        src.weight.data.copy_(w)
        q = FP8Linear.from_linear(src)
        blk.ffn[idx].weight.data.copy_(_dequant_fp8_weight(q.weight.data, q.weight_scale.data))
        blk.ffn[idx].bias.data.copy_(b)
    shift, scale, gate = mods
    with torch.no_grad():
        y = x + gate * blk.ffn(modulate(blk.apply_norm2(x), shift, scale))
    out["dit_ffn"] = {"in_sum": checksum(x, *mods, *[t for pair in ws for t in pair]), "y": y}

    # ---- a9 / a12: a whole DiT block on dequantised weights -------------------------------
    from tybok_b200.shapes import DIT_TINY
    from tybok_b200.weights import DIT_HOT_LINEARS, quantize_dit_block, random_dit_block_params

    bp = quantize_dit_block(random_dit_block_params(DIT_TINY, seed=0))
    torch.set_default_dtype(torch.bfloat16)
    try:
        blk = FastWAMAttentionBlock(DIT_TINY.hidden, DIT_TINY.head_dim, DIT_TINY.heads, DIT_TINY.ffn)
    finally:
        torch.set_default_dtype(torch.float32)
    sd = {k: v for k, v in bp.items() if not k.endswith(".scale_weight")}
    for lin in DIT_HOT_LINEARS:
        sd[f"{lin}.weight"] = _dequant_fp8_weight(bp[f"{lin}.weight"], bp[f"{lin}.scale_weight"])
    missing, unexpected = blk.load_state_dict(sd, strict=False)
    assert not unexpected and not missing, (missing, unexpected)
    blk.eval()
    for tag, prefix in (("dit_block", 0), ("dit_block_video_kv", 40)):
        x, context, context_mask, t_mod, freqs, video_kv = dit_block_case(DIT_TINY, video_prefix=prefix)
        with torch.no_grad():
            y, (k, v) = blk(x, context, t_mod, freqs, context_mask=context_mask, video_kv=video_kv, return_kv=True)
        out[tag] = {"in_sum": checksum(x, context, t_mod, torch.view_as_real(freqs), *[t for t in bp.values()]),
                    "y": y.clone(), "k": k.clone(), "v": v.clone()}

    # ---- request path: normaliser, prompt text, centred-padding resize -------------------
    from tybok.policies.pi05.models.flow_matching import resize_with_pad_torch
    from tybok.policies.pi05.preprocess import Normalizer, build_prompt

    state, stats, actions, frames = request_case()
    norm = Normalizer.from_state_dict({"VISUAL": "IDENTITY", "STATE": "MEAN_STD", "ACTION": "MEAN_STD"}, stats)
    nstate = norm.normalize(state[None], "observation.state", "STATE")
    out["request"] = {
        "in_sum": checksum(state, actions, *frames, *stats.values()),
        "state": nstate.clone(),
        "prompt": build_prompt("pick_up the\nred block ", nstate[0]),
        "actions": norm.unnormalize(actions, "action", "ACTION").clone(),
        "resized": [resize_with_pad_torch(f[None], 56, 56)[0].clone() for f in frames],
    }

    # ---- whole tiny policy -------------------------------------------------------------
    shape = PI05_TINY
    ref_config.GEMMA_VARIANTS["tiny_vlm"] = dict(vars(shape.vlm))
    ref_config.GEMMA_VARIANTS["tiny_expert"] = dict(vars(shape.expert))
    cfg = ref_config.PI05Config(
        chunk_size=shape.chunk, n_action_steps=shape.chunk, max_action_dim=shape.max_action_dim,
        paligemma_variant="tiny_vlm", action_expert_variant="tiny_expert",
        image_resolution=(shape.vision.image, shape.vision.image),
        tokenizer_max_length=shape.lang_len, num_steps=shape.steps,
        min_period=shape.min_period, max_period=shape.max_period,
    )
    cfg._image_features = [f"observation.images.cam{i}" for i in range(shape.n_cams)]
    torch.set_default_dtype(torch.bfloat16)  # as tybok/policies/pi05/engine.py:184-189
    try:
        model = PI05FlowMatching(cfg)
        pg = model.paligemma_with_expert.paligemma.model
        v = shape.vision
        # The reference hard-codes the So400m tower and the PaliGemma vocabulary; swap in
        # smaller instances of the same reference classes so the fixture stays small.
        pg.vision_tower.vision_model = SiglipVisionTransformer(
            hidden_size=v.hidden, num_heads=v.heads, num_layers=v.layers,
            intermediate_size=v.mlp_dim, image_size=v.image, patch_size=v.patch)
        pg.multi_modal_projector = PaliGemmaMultiModalProjector(v.hidden, shape.vlm.width)
        pg.language_model.embed_tokens = nn.Embedding(shape.vocab, shape.vlm.width, dtype=torch.bfloat16)
    finally:
        torch.set_default_dtype(torch.float32)
    model.eval()

    params = quantize_hot_linears(random_pi05_params(shape, seed=0), shape)
    sd = {}
    for name, t in params.items():
        if name.endswith(".scale_weight"):
            continue
        if t.dtype == torch.float8_e4m3fn:  # the loader's dequant path, policy.py:127-129
            t = _dequant_fp8_weight(t, params[name[: -len("weight")] + "scale_weight"])
        sd[name] = t
    missing, unexpected = model.load_state_dict(sd, strict=False)
    assert not unexpected, unexpected
    assert all("position_ids" in m or "inv_freq" in m for m in missing), missing

    images, img_masks, tokens, masks, noise = tiny_inputs(shape)
    with torch.no_grad():
        actions = model.sample_actions(images, img_masks, tokens, masks, noise=noise)
        # intermediates for finer-grained pins
        embs, pad, att = model.embed_prefix(images, img_masks, tokens, masks)
    out["pi05_tiny"] = {
        "in_sum": checksum(*images, tokens, *[t for t in params.values()]),
        "actions": actions.clone(),
        "prefix_embs": embs[:, ::37].clone(),
    }
    # batch-2 determinism of the eager path (the same oracle serves batched throughput)
    images2, img_masks2, tokens2, masks2, noise2 = tiny_inputs(shape, seed=3, batch=2)
    with torch.no_grad():
        out["pi05_tiny_b2"] = {"actions": model.sample_actions(images2, img_masks2, tokens2, masks2, noise=noise2).clone()}

    path = os.path.join(HERE, "pi05_golden.pt")
    torch.save(out, path)
    print("wrote", path, os.path.getsize(path), "bytes")


if __name__ == "__main__":
    main()
