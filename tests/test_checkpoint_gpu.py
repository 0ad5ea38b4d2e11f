"""The engine on a checkpoint DIRECTORY in the reference's on-disk format: ``config.json``, fp8
``*.safetensors`` with ``.scale_weight`` companions, normaliser / un-normaliser statistics files,
``policy_preprocessor.json`` + ``tokenizer.json``
(tybok/policies/pi05/config.py:134-174, preprocess.py:88-110, docs/fastWAM_weight_quantization.md:14-24).

What is checked: loading by directory gives bit for bit what the same weights give when handed
over in memory; the state is normalised before it enters the prompt and the returned actions are
un-normalised; the checkpoint's tokenizer is used; ``camera_alias`` maps client keys onto slots;
missing cameras follow the present ones; ``validate`` reports the reference harness's components.
"""

import json
import os

import pytest
import torch

from oracle import pi05_ref, w8_ref
from tybok_b200 import request as rq
from tybok_b200.shapes import GEMMA_VARIANTS, PI05_TINY
from tybok_b200.weights import quantize_hot_linears, random_pi05_params

pytestmark = pytest.mark.gpu
ACTION_DIM = 7
WORDS = ("Task: pick up the red block cube , State: ; Action: " + " ".join(str(i) for i in range(256))).split()


def write_tokenizer(path: str) -> str:
    """A word-level ``tokenizer.json`` with ``<pad>`` = 0 and a post-processor that prepends
    ``<bos>`` = 2, as the PaliGemma file does."""
    from tokenizers import Tokenizer, models, pre_tokenizers, processors

    os.makedirs(path, exist_ok=True)
    vocab = {"<pad>": 0, "<eos>": 1, "<bos>": 2, "<unk>": 3}
    for w in WORDS:
        vocab.setdefault(w, len(vocab))
    tok = Tokenizer(models.WordLevel(vocab, unk_token="<unk>"))
    tok.pre_tokenizer = pre_tokenizers.WhitespaceSplit()
    tok.post_processor = processors.TemplateProcessing(single="<bos> $A", special_tokens=[("<bos>", 2)])
    tok.save(os.path.join(path, "tokenizer.json"))
    return path


def write_checkpoint(path: str, seed: int = 0):
    """Tiny fp8 checkpoint directory; returns ``(params, stats)`` as written."""
    from safetensors.torch import save_file

    shape = PI05_TINY
    GEMMA_VARIANTS["tiny_vlm"], GEMMA_VARIANTS["tiny_expert"] = shape.vlm, shape.expert
    os.makedirs(path, exist_ok=True)
    params = quantize_hot_linears(random_pi05_params(shape, seed=seed), shape)
    save_file({f"model.{k}": v.contiguous() for k, v in params.items()}, os.path.join(path, "model.fp8.safetensors"))
    g = torch.Generator().manual_seed(seed + 1)
    stats = {"observation.state.mean": torch.empty(8).normal_(0, 0.3, generator=g),
             "observation.state.std": torch.empty(8).uniform_(0.5, 1.5, generator=g),
             "action.mean": torch.empty(ACTION_DIM).normal_(0, 0.3, generator=g),
             "action.std": torch.empty(ACTION_DIM).uniform_(0.5, 1.5, generator=g)}
    save_file({k: v for k, v in stats.items() if k.startswith("observation")},
              os.path.join(path, "policy_preprocessor_step_2_normalizer_processor.safetensors"))
    save_file({k: v for k, v in stats.items() if k.startswith("action")},
              os.path.join(path, "policy_postprocessor_step_0_unnormalizer_processor.safetensors"))
    res = shape.vision.image
    cfg = {
        "type": "pi05_b200",
        "input_features": {"observation.images.image": {"type": "VISUAL", "shape": [3, res, res]},
                           "observation.images.image2": {"type": "VISUAL", "shape": [3, res, res]},
                           "observation.state": {"type": "STATE", "shape": [8]}},
        "output_features": {"action": {"type": "ACTION", "shape": [ACTION_DIM]}},
        "image_resolution": [res, res], "paligemma_variant": "tiny_vlm", "action_expert_variant": "tiny_expert",
        "tokenizer_max_length": shape.lang_len, "chunk_size": shape.chunk, "n_action_steps": shape.chunk,
        "num_inference_steps": shape.steps, "max_action_dim": shape.max_action_dim, "vision_heads": shape.vision.heads,
        "normalization_mapping": {"VISUAL": "IDENTITY", "STATE": "MEAN_STD", "ACTION": "MEAN_STD"},
    }
    with open(os.path.join(path, "config.json"), "w", encoding="utf-8") as f:
        json.dump(cfg, f)
    write_tokenizer(os.path.join(path, "tokenizer"))
    with open(os.path.join(path, "policy_preprocessor.json"), "w", encoding="utf-8") as f:
        json.dump({"steps": [{"registry_name": "tokenizer_processor", "config": {"tokenizer_name": "tokenizer"}}]}, f)
    return params, stats


def _frame(seed, res, names=("image", "image2")):
    g = torch.Generator().manual_seed(seed)
    frame = {f"observation.images.{n}": torch.rand(3, res, res, generator=g) for n in names}
    frame["observation.state"] = torch.empty(8).normal_(0, 1, generator=g)
    frame["task"] = "pick up the red block"
    return frame


@pytest.fixture(scope="module")
def ckpt(tmp_path_factory):
    path = str(tmp_path_factory.mktemp("pi05_tiny_fp8"))
    params, stats = write_checkpoint(path)
    return path, params, stats


def _expected_inputs(frame, stats, path, names=("image", "image2")):
    st = rq.FeatureStats(None, stats)
    nstate = st.normalize(frame["observation.state"], rq.STATE_KEY, "STATE")
    tokens, mask = rq.PromptTokenizer(os.path.join(path, "tokenizer"), PI05_TINY.lang_len).encode(
        rq.prompt_text(frame["task"], nstate))
    images = [frame[f"observation.images.{n}"][None] * 2.0 - 1.0 for n in names]
    return st, images, tokens[None], mask[None]


def test_engine_on_a_checkpoint_directory(ckpt):
    from tybok_b200 import ops
    from tybok_b200.engine import PI05B200Engine
    from tybok_b200.pi05 import PI05Model

    path, params, stats = ckpt
    eng = PI05B200Engine(path, device="cuda", graph=True, seed=0)
    spec = eng.describe()
    assert spec["cameras"] == ["image", "image2"] and spec["action_dim"] == ACTION_DIM and spec["pad_mode"] == "center"
    assert eng.tokenizer is not None and eng.config.shape.vision == PI05_TINY.vision
    frame = _frame(3, PI05_TINY.vision.image)
    noise = torch.zeros(1, PI05_TINY.chunk, ACTION_DIM)
    got = torch.from_numpy(eng.predict_action_chunk(frame, noise=noise))
    ops.check_status()
    assert got.shape == (PI05_TINY.chunk, ACTION_DIM)

    # the same weights handed over in memory, inputs prepared by hand
    st, images, tokens, mask = _expected_inputs(frame, stats, path)
    assert int(tokens[0, 0]) == 2 and int(tokens.max()) < 300  # <bos> first, word-level ids: the checkpoint's tokenizer ran
    model = PI05Model(params, PI05_TINY, device="cuda", vision_dtype=torch.float16)  # the engine's default tower
    ones = [torch.ones(1, dtype=torch.bool, device="cuda") for _ in images]
    full_noise = torch.zeros(1, PI05_TINY.chunk, PI05_TINY.max_action_dim, device="cuda")
    raw = model.sample_actions([i.cuda() for i in images], ones, tokens.cuda(), mask.cuda(), full_noise)
    want = st.unnormalize(raw[0, :, :ACTION_DIM].float().cpu(), rq.ACTION_KEY, "ACTION")
    assert torch.equal(got, want)
    # ... and against the oracle (fp32 tower there, bf16 here), on the normalised chunk
    ref = pi05_ref.sample_actions(params, PI05_TINY, images, [torch.ones(1, dtype=torch.bool)] * 2, tokens, mask,
                                  full_noise.cpu())
    assert float((raw.cpu() - ref).abs().max()) <= 2e-2
    # the statistics matter: the un-normalised chunk is not the raw one
    assert not torch.allclose(got, raw[0, :, :ACTION_DIM].float().cpu())


def test_camera_alias_and_missing_cameras(ckpt):
    from tybok_b200.engine import PI05B200Engine

    path, _, _ = ckpt
    res = PI05_TINY.vision.image
    noise = torch.zeros(1, PI05_TINY.chunk, ACTION_DIM)
    direct = PI05B200Engine(path, device="cuda", graph=True, seed=0)
    aliased = PI05B200Engine(path, device="cuda", graph=True, seed=0, camera_alias={"left_wrist_image": "image2"})
    frame = _frame(4, res)
    client = dict(frame)
    client["observation.images.left_wrist_image"] = client.pop("observation.images.image2")
    a = direct.predict_action_chunk(frame, noise=noise)
    b = aliased.predict_action_chunk(client, noise=noise)
    assert (a == b).all()
    with pytest.raises(ValueError, match="not an expected image feature"):
        PI05B200Engine(path, device="cuda", graph=False, warmup=False, camera_alias={"cam": "image7"})
    # a frame that needs the centred-padding resize, and one whose first camera is missing: the present
    # camera takes the first slot, the empty slot follows with mask 0
    wide = _frame(5, res)
    wide["observation.images.image"] = torch.rand(3, res, 2 * res)
    assert torch.isfinite(torch.from_numpy(direct.predict_action_chunk(wide, noise=noise))).all()
    only2 = {k: v for k, v in frame.items() if k != "observation.images.image"}
    images, masks, _, _ = direct._preprocess([only2])
    assert masks[0].tolist() == [True] and masks[1].tolist() == [False]
    assert torch.equal(images[0][0].cpu(), frame["observation.images.image2"] * 2 - 1) and bool((images[1] == -1).all())
    none = {k: v for k, v in frame.items() if not k.startswith("observation.images.")}
    with pytest.raises(ValueError, match="All image features are missing"):
        direct.predict_action_chunk(none, noise=noise)
    # a real checkpoint without a tokenizer refuses to invent token ids
    direct.tokenizer = None
    with pytest.raises(ValueError, match="no tokenizer"):
        direct.predict_action_chunk(frame, noise=noise)


def test_validate_reports_the_reference_components(ckpt, tmp_path):
    """Dumps in the reference harness's format, produced here by the CPU oracle, and the engine's
    per-component errors against them (tybok/policies/pi05/engine.py:740-857)."""
    from tybok_b200.engine import PI05B200Engine

    path, params, stats = ckpt
    shape = PI05_TINY
    frame = _frame(9, shape.vision.image)
    st, images, tokens, mask = _expected_inputs(frame, stats, path)
    ones = [torch.ones(1, dtype=torch.bool)] * 2
    zero = torch.zeros(1, shape.chunk, shape.max_action_dim)
    chunk, inter = pi05_ref.sample_actions(params, shape, images, ones, tokens, mask, zero, return_intermediates=True)
    pad = torch.cat([torch.ones(1, 2 * shape.vision.tokens, dtype=torch.bool), mask], dim=1)
    v_t = pi05_ref.denoise_step(params, shape, pad, inter["kv"], zero, torch.tensor([0.5]))
    d = str(tmp_path)
    torch.save(frame, os.path.join(d, "frame.pt"))
    batch = {k: v[None] for k, v in frame.items() if isinstance(v, torch.Tensor)}
    batch[rq.STATE_KEY] = st.normalize(frame[rq.STATE_KEY], rq.STATE_KEY, "STATE")[None]
    batch[rq.TOKENS_KEY], batch[rq.TOKEN_MASK_KEY] = tokens, mask
    torch.save(batch, os.path.join(d, "batch.pt"))
    torch.save({"embs": inter["prefix_embs"], "pad_masks": pad, "att_masks": torch.zeros_like(pad)}, os.path.join(d, "prefix.pt"))
    torch.save({f"layer{i}": {"keys": k, "values": v} for i, (k, v) in enumerate(inter["kv"])}, os.path.join(d, "prefix_kv.pt"))
    torch.save({"v_t": v_t}, os.path.join(d, "denoise.pt"))
    torch.save({"chunk": chunk[:, :, :ACTION_DIM],
                "chunk_post": st.unnormalize(chunk[:, :, :ACTION_DIM], rq.ACTION_KEY, "ACTION")}, os.path.join(d, "chunk.pt"))

    eng = PI05B200Engine(path, device="cuda", graph=True, seed=0)
    errors = eng.validate(d)
    for name in ("batch.observation.state", "batch.observation.language.tokens", "prefix.embs", "prefix.pad_masks",
                 "prefix_kv.layer0.keys", "prefix_kv.layer1.values", "denoise.v_t", "chunk", "chunk_post"):
        assert name + ".max" in errors and name + ".mean" in errors, name
    assert errors["batch.observation.state.max"] == 0.0 and errors["batch.observation.language.tokens.max"] == 0.0
    assert errors["prefix.pad_masks.max"] == 0.0 and errors["prefix.att_masks.max"] == 0.0
    assert errors["denoise.v_t.max"] <= 2e-2 and errors["chunk.max"] <= 2e-2
    with pytest.raises(FileNotFoundError):
        eng.validate(os.path.join(d, "missing"))
