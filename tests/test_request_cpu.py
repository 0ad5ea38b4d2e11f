"""Host-side request path (``tybok_b200/request.py``) against outputs of the reference's own
processor functions (fixture made by ``tests/golden/make_golden.py``), and the route a running
tybok installation takes to this backend: ``tybok.registry.create_engine``."""

import os
import subprocess
import sys

import pytest
import torch

sys.path.insert(0, os.path.join(os.path.dirname(__file__), "golden"))
from make_golden import checksum, request_case  # noqa: E402

from tybok_b200 import request as rq  # noqa: E402

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_normaliser_prompt_and_resize_match_reference(golden):
    state, stats, actions, frames = request_case()
    g = golden["request"]
    assert checksum(state, actions, *frames, *stats.values()) == g["in_sum"]
    st = rq.FeatureStats(None, stats)
    nstate = st.normalize(state[None], rq.STATE_KEY, "STATE")
    assert torch.equal(nstate, g["state"])
    assert rq.prompt_text("pick_up the\nred block ", nstate[0]) == g["prompt"]
    assert torch.equal(st.unnormalize(actions, rq.ACTION_KEY, "ACTION"), g["actions"])
    for f, want in zip(frames, g["resized"]):
        assert torch.equal(rq.resize_with_pad(f, 56, 56), want)
    # identity when a feature has no statistics or its mode is IDENTITY
    assert torch.equal(rq.FeatureStats().normalize(state, rq.STATE_KEY, "STATE"), state)
    assert torch.equal(rq.FeatureStats({"STATE": "IDENTITY"}, stats).normalize(state, rq.STATE_KEY, "STATE"), state)
    with pytest.raises(ValueError, match="Unsupported normalization mode"):
        rq.FeatureStats({"STATE": "MIN_MAX"}, stats).normalize(state, rq.STATE_KEY, "STATE")


def test_camera_alias_moves_client_keys_onto_checkpoint_slots():
    feats = ["observation.images.image", "observation.images.image2"]
    alias = rq.normalise_alias({"left_wrist_image": "image2"}, feats)
    assert alias == {"observation.images.left_wrist_image": "observation.images.image2"}
    frame = {"observation.images.image": 1, "observation.images.left_wrist_image": 2, "task": "t"}
    out = rq.alias_frame(frame, alias)
    assert out["observation.images.image2"] == 2 and "observation.images.left_wrist_image" not in out
    assert "observation.images.left_wrist_image" in frame  # the caller's frame is not modified
    # the slot wins when the client sends both
    both = dict(frame, **{"observation.images.image2": 3})
    assert rq.alias_frame(both, alias)["observation.images.image2"] == 3
    with pytest.raises(ValueError, match="not an expected image feature"):
        rq.normalise_alias({"cam": "image9"}, feats)
    with pytest.raises(ValueError, match="already an expected image feature"):
        rq.normalise_alias({"image": "image2"}, feats)


def test_tokenizer_from_checkpoint_files(tmp_path):
    from test_checkpoint_gpu import write_tokenizer  # the tiny tokenizer the checkpoint test ships

    tok_dir = write_tokenizer(str(tmp_path / "tok"))
    with open(tmp_path / "policy_preprocessor.json", "w", encoding="utf-8") as f:
        f.write('{"steps": [{"registry_name": "tokenizer_processor", "config": {"tokenizer_name": "tok"}}]}')
    assert rq.resolve_tokenizer_dir(str(tmp_path)) == tok_dir
    tok = rq.PromptTokenizer(tok_dir, 24)
    ids, mask = tok.encode("Task: pick up the cube, State: 3 200;\nAction: ")
    assert ids.shape == (24,) and mask.dtype == torch.bool and int(ids[0]) == tok.tok.token_to_id("<bos>")
    assert int(mask.sum()) < 24 and bool((ids[~mask] == tok.pad_id).all())
    long_ids, long_mask = tok.encode("cube " * 100)
    assert long_ids.shape == (24,) and bool(long_mask.all())  # truncated
    assert rq.resolve_tokenizer_dir(str(tmp_path / "tok")) == tok_dir  # tokenizer.json beside the checkpoint
    assert rq.resolve_tokenizer_dir(str(tmp_path / "nothing")) is None


def _reference_root():
    root = os.environ.get("TYBOK_REFERENCE") or os.path.join(os.path.dirname(ROOT), "reference")
    return root if os.path.isdir(os.path.join(root, "tybok")) else None


@pytest.mark.skipif(_reference_root() is None, reason="needs a tybok checkout (TYBOK_REFERENCE)")
def test_reference_registry_reaches_this_backend():
    """With the reference importable, ``import tybok_b200.engine`` registers ``pi05_b200`` in the
    reference's own registry and ``create_engine`` with the kwarg set the worker always builds
    (tybok/worker.py:811-858) reaches this backend's constructor: on a machine without a GPU that
    constructor answers that there is no CPU path; another tier's flag is refused before it."""
    code = r'''
import sys
import tybok_b200.engine  # registers the backend
from tybok_b200 import base
from tybok import registry
assert base.HAVE_REFERENCE and registry._REGISTRY["pi05_b200"] is tybok_b200.engine.PI05B200Engine
assert issubclass(tybok_b200.engine.PI05B200Engine, __import__("tybok.base").base.PolicyEngine)
worker_kwargs = dict(
    compile_model=False, graph=True, graph_cameras=None, num_steps=None, seed=None, sampler="euler",
    cache_expert_prefix_kv=True, cache_prompt=True, profile=False, overlap=True, tl_fused_vit=False,
    tl_llm_flash_attn=False, tl_llm_fused_attn=False, tl_vit_oproj=False, tl_fused_expert=False, tl_fp8_llm_mlp=False,
    tl_fp8_expert_mlp=False, vit_mlp_dtype=None, skip_empty_images=False, pad_free=False, pack_qkv=False,
    video_fp8=False, action_fp8=False, text_fp8=False, action_fused=True, action_fused_split=True,
    action_pre_fused=False, video_pre_fused=False, video_fused=True, video_fused_split=True, action_context_cache=True,
    text_fused=False, text_fused_split=False, require_fused=True, camera_alias=None, shm_ipc=False, tokenizer_dir=None,
    text_encoder_dir=None, vae_dir=None, text_encoder_device=None, text_emb_cpu=False, rtc_config=None)
try:
    registry.create_engine("synthetic:pi05_tiny", model_type="pi05_b200", device="cpu", **worker_kwargs)
except RuntimeError as e:
    assert "no CPU fallback" in str(e), e
else:
    raise SystemExit("constructor did not run")
try:
    registry.create_engine("synthetic:pi05_tiny", model_type="pi05_b200", device="cpu",
                           **dict(worker_kwargs, tl_fused_expert=True))
except NotImplementedError as e:
    assert "tl-fused-expert" in str(e), e
else:
    raise SystemExit("foreign flag accepted")
print("REGISTRY_OK")
'''
    env = dict(os.environ, TYBOK_REFERENCE=_reference_root(), PYTHONDONTWRITEBYTECODE="1", PYTHONPATH=ROOT)
    proc = subprocess.run([sys.executable, "-c", code], env=env, capture_output=True, text=True, timeout=300)
    assert proc.returncode == 0 and "REGISTRY_OK" in proc.stdout, proc.stdout + proc.stderr
