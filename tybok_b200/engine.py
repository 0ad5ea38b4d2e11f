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

from .base import PolicyEngine, register, reject_unsupported_flags
from .pi05 import PI05Model
from .shapes import GEMMA_2B, GEMMA_300M, PI05_FULL, PI05_SMALL, PI05_TINY, GemmaSpec, PI05Shape, SiglipSpec
from .weights import random_pi05_params

log = logging.getLogger("tybok.pi05_b200")

SYNTHETIC = {"pi05_full": PI05_FULL, "pi05_tiny": PI05_TINY, "pi05_small": PI05_SMALL}
_VARIANTS = {"gemma_2b": GEMMA_2B, "gemma_300m": GEMMA_300M}


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


def _load_checkpoint(checkpoint_dir: str) -> tuple[PI05Shape, dict[str, torch.Tensor], list[str], int]:
    """A reference-format checkpoint directory: ``config.json`` + ``*.safetensors`` whose keys are
    the reference's parameter paths (tybok/policies/pi05/models/policy.py:47-76); fp8 files carry
    ``<module>.scale_weight`` companions (docs/fastWAM_weight_quantization.md:14-24)."""
    from glob import glob

    from safetensors import safe_open

    with open(os.path.join(checkpoint_dir, "config.json"), encoding="utf-8") as f:
        cfg = json.load(f)
    cams = [k for k, v in cfg.get("input_features", {}).items() if v.get("type") == "VISUAL"]
    res = cfg.get("image_resolution", [224, 224])
    shape = PI05Shape(
        vlm=_VARIANTS[cfg.get("paligemma_variant", "gemma_2b")],
        expert=_VARIANTS[cfg.get("action_expert_variant", "gemma_300m")],
        vision=SiglipSpec(image=int(res[0])),
        n_cams=len(cams),
        lang_len=cfg.get("tokenizer_max_length", 200),
        chunk=cfg.get("chunk_size", 50),
        steps=cfg.get("num_inference_steps", 10),
        max_action_dim=cfg.get("max_action_dim", 32),
        min_period=cfg.get("min_period", 4e-3),
        max_period=cfg.get("max_period", 4.0),
    )
    params: dict[str, torch.Tensor] = {}
    for file in sorted(glob(os.path.join(checkpoint_dir, "*.safetensors"))):
        if "processor" in os.path.basename(file):
            continue
        with safe_open(file, "pt", "cpu") as f:
            for name in f.keys():
                key = name[len("model."):] if name.startswith("model.") else name
                key = key.replace("paligemma_with_expert.paligemma.lm_head.weight",
                                  "paligemma_with_expert.paligemma.model.language_model.embed_tokens.weight")
                params[key] = f.get_tensor(name)
    action_dim = int(cfg.get("output_features", {}).get("action", {}).get("shape", [shape.max_action_dim])[0])
    return shape, params, cams, action_dim


@register("pi05_b200")
class PI05B200Engine(PolicyEngine):
    # Flags owned by other backends / tiers: their inert defaults; any other value is refused
    # (same table mechanism as tybok/policies/pi05/engine.py:77-102).
    _UNSUPPORTED_FLAGS = {
        "tl_llm_fused_attn": False, "tl_vit_oproj": False, "tl_fused_vit": False, "tl_llm_flash_attn": False,
        "tl_fused_expert": False, "tl_fp8_llm_mlp": False, "tl_fp8_expert_mlp": False, "vit_mlp_dtype": None,
        "pack_qkv": False, "text_fused": False, "text_fused_split": False, "action_pre_fused": False,
        "video_pre_fused": False, "text_encoder_dir": None, "vae_dir": None, "pad_free": False,
        "skip_empty_images": False, "rtc_config": None,
    }

    def __init__(self, checkpoint_dir: str, device: str = "auto", compile_model: bool = False, warmup: bool = True,
                 graph: bool = True, num_steps: int | None = None, seed: int | None = None, sampler: str = "euler",
                 profile: bool = False, overlap: bool = False, action_fused: bool = True, video_fused: bool = True,
                 action_fused_split: bool = True, video_fused_split: bool = True, require_fused: bool = False,
                 camera_alias: dict[str, str] | None = None, batch_size: int = 1, **kwargs: Any):
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
        self.camera_alias = dict(camera_alias or {})
        self.batch_size = int(batch_size)

        if checkpoint_dir.startswith("synthetic:"):
            name, _, seed_s = checkpoint_dir[len("synthetic:"):].partition("@")
            shape = SYNTHETIC[name]
            params = random_pi05_params(shape, seed=int(seed_s or 0), device=str(self.device))
            cams = [f"camera{i + 1}" for i in range(shape.n_cams)]
            action_dim = shape.action_dim
        else:
            shape, params, cams, action_dim = _load_checkpoint(checkpoint_dir)
        if num_steps is not None:
            shape = shape.with_(steps=int(num_steps))
        self.config = EngineConfig(shape=shape, cameras=cams, num_steps=shape.steps, chunk_size=shape.chunk,
                                   n_action_steps=shape.chunk, action_dim=action_dim)
        # overlap: the first denoise step runs layer by layer behind the prefix (the reference's
        # --overlap, tybok/policies/pi05/models/flow_matching.py:609-720)
        self.model = PI05Model(params, shape, device=str(self.device), overlap=overlap)
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

    def validate(self, reference_dir: str) -> dict[str, float]:
        raise NotImplementedError("pi05_b200 is validated against the torch dequant oracle by its test-suite "
                                  "(tests/test_pi05_gpu.py); reference dumps are not consumed")

    def select_action(self, frame: dict[str, Any], noise: torch.Tensor | None = None) -> np.ndarray:
        """FIFO semantics of tybok/policies/pi05/models/policy.py:159-172."""
        if not self._queue:
            self._queue.extend(self.predict_action_chunk(frame, noise=noise)[: self.config.n_action_steps])
        return self._queue.popleft()

    def predict_action_chunk(self, frame: dict[str, Any], noise: torch.Tensor | None = None) -> np.ndarray:
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
        return out[0, :, : self.config.action_dim].float().cpu().numpy()

    def predict_action_chunks(self, frames: list[dict[str, Any]], noise: torch.Tensor | None = None) -> np.ndarray:
        """Batched requests ``[B, chunk, action_dim]`` (the batched-throughput configuration; the
        reference's eager path is batch-generic, its engines are batch-1)."""
        images, img_masks, tokens, masks = self._preprocess(frames)
        s = self.config.shape
        b = len(frames)
        if noise is None:
            noise = torch.randn(b, s.chunk, s.max_action_dim, device=self.device, generator=self._gen)
        out = self._run(images, img_masks, tokens, masks, noise.to(self.device))
        return out[:, :, : self.config.action_dim].float().cpu().numpy()

    # ------------------------------------------------------------------ internals
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
        for cam in self.config.cameras:
            key = self.camera_alias.get(cam, cam)
            key = key if key.startswith("observation.images.") else f"observation.images.{key}"
            img = frame.get(key)
            if not (isinstance(img, torch.Tensor) and img.dtype == torch.float32 and img.device.type == "cpu"
                    and tuple(img.shape) == (3, res, res)):
                return None
            imgs.append(img)
        for dst, img in zip(st["images"], imgs):
            dst[0].copy_(img, non_blocking=True)
            dst.mul_(2.0).sub_(1.0)
        if not self._static_masks_true:
            for m in st["img_masks"]:
                m.fill_(True)
            self._static_masks_true = True
        t, m = self._tokens(frame)
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
        return self._pin_out[0, :, : self.config.action_dim].float().numpy().copy()

    def _pad_noise(self, noise: torch.Tensor) -> torch.Tensor:
        s = self.config.shape
        noise = torch.as_tensor(noise, dtype=torch.float32)
        if noise.dim() == 2:
            noise = noise[None]
        if noise.shape[-1] < s.max_action_dim:  # zero-pad (tybok/policies/pi05/engine.py:486-493)
            noise = F.pad(noise, (0, s.max_action_dim - noise.shape[-1]))
        return noise.to(self.device)

    def _tokens(self, frame: dict[str, Any]) -> tuple[torch.Tensor, torch.Tensor]:
        s = self.config.shape
        if "observation.language.tokens" in frame:
            t = torch.as_tensor(frame["observation.language.tokens"]).long().reshape(-1)[: s.lang_len]
            m = torch.as_tensor(frame.get("observation.language.attention_mask", torch.ones_like(t))).bool().reshape(-1)
        else:
            # No tokenizer files ship with a synthetic checkpoint: a deterministic stand-in maps the
            # prompt (task + discretised state, as preprocess.py:112-123 builds it) to ids.
            state = torch.as_tensor(frame.get("observation.state", torch.zeros(1))).float().flatten()
            disc = np.digitize(state.clamp(-1, 1).numpy(), np.linspace(-1, 1, 257)[:-1]) - 1
            text = f"Task: {frame.get('task', '')}, State: {' '.join(map(str, disc))};\nAction: "
            ids = [int.from_bytes(hashlib.blake2b(f"{i}:{w}".encode(), digest_size=4).digest(), "little") % s.vocab
                   for i, w in enumerate(text.split())][: s.lang_len]
            t = torch.tensor(ids, dtype=torch.long)
            m = torch.ones(len(ids), dtype=torch.bool)
        pad = s.lang_len - t.numel()
        return F.pad(t, (0, pad)), F.pad(m[: s.lang_len], (0, pad))

    def _preprocess(self, frames: list[dict[str, Any]]):
        s = self.config.shape
        res = s.vision.image
        images, img_masks = [], []
        for cam in self.config.cameras:
            key = self.camera_alias.get(cam, cam)
            key = key if key.startswith("observation.images.") else f"observation.images.{key}"
            per = []
            present = []
            for fr in frames:
                img = fr.get(key)
                present.append(img is not None)
                if img is None:  # missing camera: all(-1) image, mask 0 (policy.py:222-228)
                    per.append(torch.full((3, res, res), -1.0, device=self.device))
                    continue
                # upload the frame as it is (one copy, asynchronous from pinned memory); resize and
                # rescale on the device
                img = torch.as_tensor(img).to(self.device, non_blocking=True).float()
                if img.shape[-2:] != (res, res):
                    img = F.interpolate(img[None], size=(res, res), mode="bilinear", align_corners=False)[0].clamp(0, 1)
                per.append(img * 2.0 - 1.0)
            images.append(torch.stack(per) if len(per) > 1 else per[0][None])
            img_masks.append(torch.tensor(present, dtype=torch.bool, device=self.device))
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
        self.model.sample_actions(*self._dummy_inputs(self.batch_size))
        torch.cuda.synchronize(self.device)

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
