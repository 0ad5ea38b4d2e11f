"""``pi05_b200``: a PolicyEngine backend running the pi0.5-shaped policy on the B200 kernels.

Drop-in surface (tybok/base.py:84-108, tybok/policies/pi05/engine.py:74-160,668-737):
``describe`` / ``predict_action_chunk`` / ``select_action`` / ``validate``, constructor
``(checkpoint_dir, device="auto", **kwargs)``, the ``--cu-fused-*`` flags as kwargs
(``action_fused`` / ``video_fused`` / ``require_fused`` and the worker's ``*_fused_split``
companions, tybok/worker.py:840-849) and the ``_UNSUPPORTED_FLAGS`` rejection table.

There is one tier: every decoder layer runs on the fused fp8 kernels.  ``action_fused`` /
``video_fused`` are accepted in either value when ``require_fused`` is off; with
``require_fused`` they must be on -- there is nothing to degrade to, and no CPU path.
"""

from __future__ import annotations

import hashlib
import json
import logging
import os
from collections import deque
from dataclasses import dataclass, field
from typing import Any

import numpy as np
import torch
import torch.nn.functional as F  # noqa: N812

from . import request as rq
from .base import PolicyEngine, register, reject_unsupported_flags
from .pi05 import PI05Model
from .shapes import GEMMA_VARIANTS, PI05_FULL, PI05_SMALL, PI05_TINY, PI05Shape, SiglipSpec
from .weights import VISION, random_pi05_params

log = logging.getLogger("tybok.pi05_b200")

SYNTHETIC = {"pi05_full": PI05_FULL, "pi05_tiny": PI05_TINY, "pi05_small": PI05_SMALL}


@dataclass
class EngineConfig:
    """What the model-agnostic layers read from ``engine.config`` (tybok/base.py:58-64)."""

    shape: PI05Shape
    cameras: list[str]
    num_steps: int
    chunk_size: int
    n_action_steps: int
    action_dim: int
    max_state_dim: int = 32
    proprio_dim: int = 8
    sampler: str = "euler"
    extra: dict[str, Any] = field(default_factory=dict)


def _vision_spec(cfg: dict, params: dict[str, torch.Tensor], image: int) -> SiglipSpec:
    """Tower geometry from the checkpoint's own tensors (the reference hard-codes So400m,
    paligemma_with_expert.py:48-58; a ``vision_heads`` entry of config.json overrides the head count)."""
    pe = params[f"{VISION}.embeddings.patch_embedding.weight"]
    layers = 0
    while f"{VISION}.encoder.layers.{layers}.layer_norm1.weight" in params:
        layers += 1
    return SiglipSpec(hidden=int(pe.shape[0]), heads=int(cfg.get("vision_heads", 16)), layers=layers,
                      mlp_dim=int(params[f"{VISION}.encoder.layers.0.mlp.fc1.weight"].shape[0]), image=image,
                      patch=int(pe.shape[-1]))


def _load_checkpoint(checkpoint_dir: str):
    """A reference-format checkpoint directory: ``config.json`` + ``*.safetensors`` whose keys are
    the reference's parameter paths (tybok/policies/pi05/models/policy.py:47-76); fp8 files carry
    ``<module>.scale_weight`` companions (docs/fastWAM_weight_quantization.md:14-24).  Returns
    ``(shape, params, image feature keys, action_dim, config dict)``."""
    from glob import glob

    from safetensors import safe_open

    with open(os.path.join(checkpoint_dir, "config.json"), encoding="utf-8") as f:
        cfg = json.load(f)
    image_features = [k for k, v in cfg.get("input_features", {}).items() if v.get("type") == "VISUAL"]
    res = cfg.get("image_resolution", [224, 224])
    params: dict[str, torch.Tensor] = {}
    for file in sorted(glob(os.path.join(checkpoint_dir, "*.safetensors"))):
        if "processor" in os.path.basename(file):  # normaliser statistics: request.load_*_stats
            continue
        with safe_open(file, "pt", "cpu") as f:
            for name in f.keys():
                key = name[len("model."):] if name.startswith("model.") else name
                key = key.replace("paligemma_with_expert.paligemma.lm_head.weight",
                                  "paligemma_with_expert.paligemma.model.language_model.embed_tokens.weight")
                params[key] = f.get_tensor(name)
    for variant in (cfg.get("paligemma_variant", "gemma_2b"), cfg.get("action_expert_variant", "gemma_300m")):
        if variant not in GEMMA_VARIANTS:
            raise ValueError(f"unknown Gemma variant {variant!r}; known: {sorted(GEMMA_VARIANTS)}")
    embed = params["paligemma_with_expert.paligemma.model.language_model.embed_tokens.weight"]
    action_dim = int(cfg.get("output_features", {}).get("action", {}).get("shape", [cfg.get("max_action_dim", 32)])[0])
    shape = PI05Shape(
        vlm=GEMMA_VARIANTS[cfg.get("paligemma_variant", "gemma_2b")],
        expert=GEMMA_VARIANTS[cfg.get("action_expert_variant", "gemma_300m")],
        vision=_vision_spec(cfg, params, int(res[0])),
        n_cams=len(image_features),
        lang_len=cfg.get("tokenizer_max_length", 200),
        vocab=int(embed.shape[0]),
        chunk=cfg.get("chunk_size", 50),
        steps=cfg.get("num_inference_steps", 10),
        max_action_dim=cfg.get("max_action_dim", 32),
        action_dim=action_dim,
        min_period=cfg.get("min_period", 4e-3),
        max_period=cfg.get("max_period", 4.0),
    )
    return shape, params, image_features, action_dim, cfg


@register("pi05_b200")
class PI05B200Engine(PolicyEngine):
    # Flags owned by other backends / tiers: their inert defaults; any other value is refused
    # (same table mechanism as tybok/policies/pi05/engine.py:77-102).
    _UNSUPPORTED_FLAGS = {
        "tl_llm_fused_attn": False, "tl_vit_oproj": False, "tl_fused_vit": False, "tl_llm_flash_attn": False,
        "tl_fused_expert": False, "tl_fp8_llm_mlp": False, "tl_fp8_expert_mlp": False, "vit_mlp_dtype": None,
        "pack_qkv": False, "text_fused": False, "text_fused_split": False, "action_pre_fused": False,
        "video_pre_fused": False, "text_encoder_dir": None, "vae_dir": None, "pad_free": False,
        "skip_empty_images": False, "rtc_config": None, "graph_cameras": None,
    }

    def __init__(self, checkpoint_dir: str, device: str = "auto", compile_model: bool = False, warmup: bool = True,
                 graph: bool = True, num_steps: int | None = None, seed: int | None = None, sampler: str = "euler",
                 profile: bool = False, overlap: bool = False, action_fused: bool = True, video_fused: bool = True,
                 action_fused_split: bool = True, video_fused_split: bool = True, require_fused: bool = False,
                 camera_alias: dict[str, str] | None = None, tokenizer_dir: str | None = None, batch_size: int = 1,
                 vision_precision: str = "fp16", **kwargs: Any):
        super().__init__(checkpoint_dir, device=device)
        reject_unsupported_flags(type(self), "pi05_b200", kwargs)
        if compile_model:
            raise NotImplementedError("--compile cannot be combined with the fused CUDA tiers "
                                      "(as tybok/policies/fastwam/engine.py:117-133)")
        if sampler != "euler":
            raise ValueError(f"sampler {sampler!r} not supported (only 'euler')")
        if require_fused and not (action_fused and video_fused):
            raise RuntimeError("--require-fused: this backend only has the fused fp8 tier; "
                               "--cu-fused-adit and --cu-fused-vdit must both be on")
        if not str(self.device).startswith("cuda"):
            raise RuntimeError("pi05_b200 needs a CUDA sm_100 device: there is no CPU fallback")
        # *_fused_split (cooperative vs split launches in the reference) has no meaning here.
        del action_fused_split, video_fused_split
        self.compile_model = False
        self.batch_size = int(batch_size)

        self.synthetic = checkpoint_dir.startswith("synthetic:")
        self.tokenizer = None
        if self.synthetic:
            name, _, seed_s = checkpoint_dir[len("synthetic:"):].partition("@")
            shape = SYNTHETIC[name]
            params = random_pi05_params(shape, seed=int(seed_s or 0), device=str(self.device))
            image_features = [f"{rq.IMAGE_PREFIX}camera{i + 1}" for i in range(shape.n_cams)]
            action_dim, n_action_steps = shape.action_dim, shape.chunk
            self.state_stats = self.action_stats = rq.FeatureStats()  # no statistics: identity
        else:
            shape, params, image_features, action_dim, cfg = _load_checkpoint(checkpoint_dir)
            n_action_steps = int(cfg.get("n_action_steps", shape.chunk))
            norm_map = cfg.get("normalization_mapping") or None
            self.state_stats = rq.load_state_stats(checkpoint_dir, norm_map)
            self.action_stats = rq.load_action_stats(checkpoint_dir, norm_map)
            tok_dir = rq.resolve_tokenizer_dir(checkpoint_dir, tokenizer_dir)
            if tok_dir is not None:
                self.tokenizer = rq.PromptTokenizer(tok_dir, shape.lang_len)
        if num_steps is not None:
            shape = shape.with_(steps=int(num_steps))
        self.image_features = image_features
        # {client key: checkpoint slot}, full observation.images.* keys (worker.py:41-60)
        self.camera_alias = rq.normalise_alias(camera_alias, image_features)
        self.config = EngineConfig(shape=shape, cameras=[k[len(rq.IMAGE_PREFIX):] for k in image_features],
                                   num_steps=shape.steps, chunk_size=shape.chunk, n_action_steps=n_action_steps,
                                   action_dim=action_dim)
        # overlap: the first denoise step runs layer by layer behind the prefix (the reference's
        # --overlap, tybok/policies/pi05/models/flow_matching.py:609-720)
        # SigLIP tower (not an fp8 module in the reference): "fp16" = fp16 GEMM / attention operands with an
        # fp32 residual stream (11 significant bits like TF32 at the speed of bf16; sublayer outputs must
        # stay below 65504), "tf32" = fp32 activations with TF32 tensor-core GEMMs (0.9 ms slower per
        # chunk, no range limit), "bf16" = bf16 operands (ten times the embedding error), "fp32" = plain fp32.
        if vision_precision not in ("tf32", "fp16", "bf16", "fp32"):
            raise ValueError(f"vision_precision {vision_precision!r}: expected 'tf32', 'fp16', 'bf16' or 'fp32'")
        self.model = PI05Model(params, shape, device=str(self.device), overlap=overlap,
                               vision_dtype={"bf16": torch.bfloat16, "fp16": torch.float16}.get(vision_precision, torch.float32),
                               vision_tf32=vision_precision == "tf32")
        del params
        self._gen = torch.Generator(device=self.device)
        if seed is not None:
            self._gen.manual_seed(int(seed))
        self._queue: deque = deque(maxlen=shape.chunk)
        self._graph = None
        self._static: dict[str, torch.Tensor] = {}
        self._static_masks_true = False  # the graph's camera-presence inputs are known to be all True
        self._pin_out = None
        self.graph_enabled = False
        if warmup:
            self._warm()
        if graph:
            self._capture()
        if profile and hasattr(self, "profile"):
            self.profile()

    # ------------------------------------------------------------------ interface
    def describe(self) -> dict[str, Any]:
        v = self.config.shape.vision
        return {"model_type": "pi05_b200", "cameras": list(self.config.cameras), "resize": [v.image, v.image],
                "action_dim": self.config.action_dim, "chunk_size": self.config.chunk_size, "pad_mode": "center"}

    def select_action(self, frame: dict[str, Any], noise: torch.Tensor | None = None) -> np.ndarray:
        """FIFO semantics of tybok/policies/pi05/models/policy.py:159-172."""
        if not self._queue:
            self._queue.extend(self.predict_action_chunk(frame, noise=noise)[: self.config.n_action_steps])
        return self._queue.popleft()

    def predict_action_chunk(self, frame: dict[str, Any], noise: torch.Tensor | None = None) -> np.ndarray:
        """``(chunk_size, action_dim)`` numpy, un-normalised (tybok/policies/pi05/engine.py:668-720)."""
        frame = rq.alias_frame(frame, self.camera_alias)
        fast = self._predict_chunk_static(frame, noise)
        if fast is not None:
            return fast
        images, img_masks, tokens, masks = self._preprocess([frame])
        s = self.config.shape
        if noise is None:
            noise = torch.randn(1, s.chunk, s.max_action_dim, device=self.device, generator=self._gen)
        else:
            noise = self._pad_noise(noise)
        out = self._run(images, img_masks, tokens, masks, noise)
        return self._postprocess(out[0, :, : self.config.action_dim].float().cpu()).numpy()

    def predict_action_chunks(self, frames: list[dict[str, Any]], noise: torch.Tensor | None = None) -> np.ndarray:
        """Batched requests ``[B, chunk, action_dim]`` (the batched-throughput configuration; the
        reference's eager path is batch-generic, its engines are batch-1)."""
        frames = [rq.alias_frame(fr, self.camera_alias) for fr in frames]
        images, img_masks, tokens, masks = self._preprocess(frames)
        s = self.config.shape
        b = len(frames)
        if noise is None:
            noise = torch.randn(b, s.chunk, s.max_action_dim, device=self.device, generator=self._gen)
        out = self._run(images, img_masks, tokens, masks, noise.to(self.device))
        return self._postprocess(out[:, :, : self.config.action_dim].float().cpu()).numpy()

    def validate(self, reference_dir: str) -> dict[str, float]:
        """Compare this engine with the reference's dumps ``frame.pt`` / ``batch.pt`` / ``prefix.pt`` /
        ``prefix_kv.pt`` / ``denoise.pt`` / ``chunk.pt`` component by component and return
        ``{"<component>.max": ..., "<component>.mean": ...}`` absolute errors, with the component
        names of the reference's own harness (tybok/policies/pi05/engine.py:740-857): preprocessed
        batch, prefix embeddings and masks, per-layer prefix keys / values, one denoise step at
        t = 0.5 from zero actions, the zero-noise chunk before and after un-normalisation."""

        def load(name: str):
            path = os.path.join(reference_dir, name)
            if not os.path.exists(path):
                raise FileNotFoundError(f"reference dump {path} missing")
            return torch.load(path, weights_only=False)

        frame, ref_batch, ref_prefix = load("frame.pt"), load("batch.pt"), load("prefix.pt")
        ref_kv, ref_denoise, ref_chunk = load("prefix_kv.pt"), load("denoise.pt"), load("chunk.pt")
        errors: dict[str, float] = {}

        def max_err(name: str, a: torch.Tensor, b: torch.Tensor) -> None:
            a, b = a.detach().float().cpu(), b.detach().float().cpu()
            if a.shape != b.shape:
                raise AssertionError(f"{name}: shape mismatch {tuple(a.shape)} vs {tuple(b.shape)}")
            diff = (a - b).abs()
            errors[name + ".max"], errors[name + ".mean"] = float(diff.max()), float(diff.mean())

        with torch.no_grad():
            frame = rq.alias_frame(frame, self.camera_alias)
            batch = self._batch_from_frame(frame)
            for key in [rq.STATE_KEY, rq.TOKENS_KEY, rq.TOKEN_MASK_KEY] + [k for k in ref_batch if k.startswith(rq.IMAGE_PREFIX)]:
                if key in batch and key in ref_batch:
                    max_err(f"batch.{key}", batch[key], ref_batch[key])
            images, img_masks, tokens, masks = self._preprocess([frame])
            embs, pad = self.model.embed_prefix(images, img_masks, tokens, masks)
            max_err("prefix.embs", embs, ref_prefix["embs"])
            max_err("prefix.pad_masks", pad, ref_prefix["pad_masks"])
            max_err("prefix.att_masks", torch.zeros_like(pad), ref_prefix["att_masks"])
            kv = self.model.prefill(embs, pad)
            for i, (k, v) in enumerate(kv):
                max_err(f"prefix_kv.layer{i}.keys", k, ref_kv[f"layer{i}"]["keys"])
                max_err(f"prefix_kv.layer{i}.values", v, ref_kv[f"layer{i}"]["values"])
            s = self.config.shape
            x_t = torch.zeros(1, s.chunk, s.max_action_dim, device=self.device)
            max_err("denoise.v_t", self.model.velocity_at(0.5, x_t, pad), ref_denoise["v_t"])
            chunk = self._run(images, img_masks, tokens, masks, torch.zeros_like(x_t))
            chunk = chunk[:, :, : self.config.action_dim]
            max_err("chunk", chunk, ref_chunk["chunk"])
            max_err("chunk_post", self._postprocess(chunk.float().cpu()), ref_chunk["chunk_post"])
        return errors

    # ------------------------------------------------------------------ internals
    def _postprocess(self, actions: torch.Tensor) -> torch.Tensor:
        """Un-normalise actions with the checkpoint's statistics (preprocess.py:192-200)."""
        return self.action_stats.unnormalize(actions, rq.ACTION_KEY, "ACTION")

    def _batch_from_frame(self, frame: dict[str, Any]) -> dict[str, torch.Tensor]:
        """The reference's preprocessed batch (preprocess.py:158-189): batched observation tensors,
        normalised state, prompt tokens and mask."""
        batch: dict[str, torch.Tensor] = {}
        for key, value in frame.items():
            if key.startswith("observation.") and isinstance(value, torch.Tensor):
                batch[key] = value[None] if value.ndim in (1, 3) else value
        if rq.STATE_KEY in batch:
            batch[rq.STATE_KEY] = self.state_stats.normalize(batch[rq.STATE_KEY].float(), rq.STATE_KEY, "STATE")
        t, m = self._tokens(frame)
        batch[rq.TOKENS_KEY], batch[rq.TOKEN_MASK_KEY] = t[None], m[None]
        return batch

    def _predict_chunk_static(self, frame: dict[str, Any], noise) -> np.ndarray | None:
        """Batch-1 request whose camera frames already have the model's resolution, with a captured
        graph: the frames are copied from host memory straight into the graph's input buffers and
        rescaled there (the same two fp32 operations as ``_preprocess``), the chunk comes back
        through a pinned buffer.  Anything else returns None and takes the general path."""
        if self._graph is None or self._static["noise"].shape[0] != 1:
            return None
        s, st = self.config.shape, self._static
        res = s.vision.image
        imgs = []
        for key in self.image_features:
            img = frame.get(key)
            if not (isinstance(img, torch.Tensor) and img.dtype == torch.float32 and img.device.type == "cpu"
                    and tuple(img.shape) == (3, res, res)):
                return None
            imgs.append(img)
        t, m = self._tokens(frame)
        for dst, img in zip(st["images"], imgs):
            dst[0].copy_(img, non_blocking=True)
            dst.mul_(2.0).sub_(1.0)
        if not self._static_masks_true:
            for msk in st["img_masks"]:
                msk.fill_(True)
            self._static_masks_true = True
        st["tokens"][0].copy_(t, non_blocking=True)
        st["masks"][0].copy_(m, non_blocking=True)
        if noise is None:
            st["noise"].copy_(torch.randn(1, s.chunk, s.max_action_dim, device=self.device, generator=self._gen))
        else:
            st["noise"].copy_(self._pad_noise(noise))
        self._graph.replay()
        if self._pin_out is None:
            self._pin_out = torch.empty(st["out"].shape, dtype=st["out"].dtype).pin_memory()
        self._pin_out.copy_(st["out"], non_blocking=True)
        torch.cuda.current_stream(self.device).synchronize()
        return self._postprocess(self._pin_out[0, :, : self.config.action_dim].float().clone()).numpy()

    def _pad_noise(self, noise: torch.Tensor) -> torch.Tensor:
        s = self.config.shape
        noise = torch.as_tensor(noise, dtype=torch.float32)
        if noise.dim() == 2:
            noise = noise[None]
        if noise.shape[-1] < s.max_action_dim:  # zero-pad (tybok/policies/pi05/engine.py:486-493)
            noise = F.pad(noise, (0, s.max_action_dim - noise.shape[-1]))
        return noise.to(self.device)

    def _tokens(self, frame: dict[str, Any]) -> tuple[torch.Tensor, torch.Tensor]:
        """Prompt ids and mask ``[lang_len]``: taken from the frame when the client tokenised, else
        built from the task and the normalised state with the checkpoint's tokenizer."""
        s = self.config.shape
        if rq.TOKENS_KEY in frame:
            t = torch.as_tensor(frame[rq.TOKENS_KEY]).long().reshape(-1)[: s.lang_len]
            m = torch.as_tensor(frame.get(rq.TOKEN_MASK_KEY, torch.ones_like(t))).bool().reshape(-1)
        else:
            if rq.STATE_KEY not in frame:
                raise ValueError("state is required for PI05")
            task = frame.get("task", "")
            if not isinstance(task, str):
                raise ValueError(f"task must be a string, got {type(task).__name__}")
            state = torch.as_tensor(frame[rq.STATE_KEY]).float().flatten()
            text = rq.prompt_text(task, self.state_stats.normalize(state, rq.STATE_KEY, "STATE"))
            if self.tokenizer is not None:
                return self.tokenizer.encode(text)
            if not self.synthetic:
                raise ValueError("this checkpoint has no tokenizer (policy_preprocessor.json names none and no "
                                 "tokenizer.json lies beside it): pass tokenizer_dir, or send "
                                 f"{rq.TOKENS_KEY!r} with the frame")
            # Synthetic weights ship no tokenizer files: a deterministic stand-in maps the words of
            # the prompt to ids.  Never used with a real checkpoint.
            ids = [int.from_bytes(hashlib.blake2b(f"{i}:{w}".encode(), digest_size=4).digest(), "little") % s.vocab
                   for i, w in enumerate(text.split())][: s.lang_len]
            t = torch.tensor(ids, dtype=torch.long)
            m = torch.ones(len(ids), dtype=torch.bool)
        pad = s.lang_len - t.numel()
        return F.pad(t, (0, pad)), F.pad(m[: s.lang_len], (0, pad))

    def _preprocess(self, frames: list[dict[str, Any]]):
        """Frames (already aliased) -> per-slot images in [-1, 1], presence masks, tokens, masks.
        Per request the cameras that are present fill the leading slots in checkpoint order and the
        missing ones follow as all(-1) images with mask 0; a request without any camera is an
        error (tybok/policies/pi05/models/policy.py:176-232)."""
        s = self.config.shape
        res = s.vision.image
        n = len(self.image_features)
        per_slot: list[list[torch.Tensor]] = [[] for _ in range(n)]
        per_mask: list[list[bool]] = [[] for _ in range(n)]
        for fr in frames:
            present = [k for k in self.image_features if fr.get(k) is not None]
            if not present:
                raise ValueError(f"All image features are missing from the frame. At least one expected. "
                                 f"(frame: {sorted(fr)}) (image_features: {self.image_features})")
            for slot in range(n):
                if slot < len(present):
                    # upload the frame as it is (one asynchronous copy when it is pinned); resize and
                    # rescale on the device
                    img = torch.as_tensor(fr[present[slot]]).to(self.device, non_blocking=True).float()
                    if img.ndim == 3 and img.shape[0] not in (1, 3) and img.shape[-1] in (1, 3):
                        img = img.permute(2, 0, 1)  # channels-last client frame
                    if tuple(img.shape[-2:]) != (res, res):
                        img = rq.resize_with_pad(img, res, res)
                    per_slot[slot].append(img * 2.0 - 1.0)
                    per_mask[slot].append(True)
                else:
                    per_slot[slot].append(torch.full((3, res, res), -1.0, device=self.device))
                    per_mask[slot].append(False)
        images = [torch.stack(p) for p in per_slot]
        img_masks = [torch.tensor(m, dtype=torch.bool, device=self.device) for m in per_mask]
        toks = [self._tokens(fr) for fr in frames]
        tokens = torch.stack([t for t, _ in toks]).to(self.device)
        masks = torch.stack([m for _, m in toks]).to(self.device)
        return images, img_masks, tokens, masks

    def _run(self, images, img_masks, tokens, masks, noise) -> torch.Tensor:
        if self._graph is not None and noise.shape[0] == self._static["noise"].shape[0]:
            st = self._static
            for dst, src in zip(st["images"], images):
                dst.copy_(src, non_blocking=True)
            for dst, src in zip(st["img_masks"], img_masks):
                dst.copy_(src, non_blocking=True)
            self._static_masks_true = False
            st["tokens"].copy_(tokens, non_blocking=True)
            st["masks"].copy_(masks, non_blocking=True)
            st["noise"].copy_(noise, non_blocking=True)
            self._graph.replay()
            return st["out"].clone()
        return self.model.sample_actions(images, img_masks, tokens, masks, noise)

    def _dummy_inputs(self, b: int):
        s = self.config.shape
        res = s.vision.image
        images = [torch.zeros(b, 3, res, res, device=self.device) for _ in range(s.n_cams)]
        img_masks = [torch.ones(b, dtype=torch.bool, device=self.device) for _ in range(s.n_cams)]
        tokens = torch.zeros(b, s.lang_len, dtype=torch.long, device=self.device)
        masks = torch.ones(b, s.lang_len, dtype=torch.bool, device=self.device)
        noise = torch.zeros(b, s.chunk, s.max_action_dim, device=self.device)
        return images, img_masks, tokens, masks, noise

    def _warm(self) -> None:
        """One chunk on dummy inputs before serving.  Also the place where a checkpoint whose vision tower
        does not fit the fp16 range shows: sublayer outputs beyond 65504 turn the image features, and with
        them the chunk, into inf / NaN; the TF32 and bf16 towers have no such limit."""
        out = self.model.sample_actions(*self._dummy_inputs(self.batch_size))
        torch.cuda.synchronize(self.device)
        if self.model.vision_dtype == torch.float16 and not bool(torch.isfinite(out).all()):
            raise RuntimeError("pi05_b200: the warm-up chunk is not finite with the fp16 vision tower; "
                               "construct the engine with vision_precision='tf32'")

    def _capture(self) -> None:
        """Whole ``sample_actions`` (prefix + every denoise step) as one CUDA graph with static
        inputs/outputs (tybok/graph.py:86-251; tybok/policies/pi05/engine.py:542-662)."""
        from . import ops

        images, img_masks, tokens, masks, noise = self._dummy_inputs(self.batch_size)
        self._static = {"images": images, "img_masks": img_masks, "tokens": tokens, "masks": masks, "noise": noise}
        side = torch.cuda.Stream(device=self.device)
        side.wait_stream(torch.cuda.current_stream(self.device))
        with torch.cuda.stream(side):  # warm every kernel / lazy init outside the capture
            for _ in range(2):
                self.model.sample_actions(images, img_masks, tokens, masks, noise)
        torch.cuda.current_stream(self.device).wait_stream(side)
        ops.check_status(torch.device(self.device))
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            self._static["out"] = self.model.sample_actions(images, img_masks, tokens, masks, noise)
        self._graph = graph
        self.graph_enabled = True
