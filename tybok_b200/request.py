"""Host-side request path of the ``pi05_b200`` engine: what turns a client frame into model inputs
and a model chunk into the returned actions.

Mirrors the reference's processor pipeline (tybok/policies/pi05/preprocess.py:39-200,
tokenizer.py:16-48, models/flow_matching.py:842-874, models/policy.py:176-232):

* MEAN_STD normalisation of ``observation.state`` with the statistics stored beside the checkpoint
  (``policy_preprocessor_step_*_normalizer_processor.safetensors``) and the inverse on the
  returned actions (``policy_postprocessor_step_*_unnormalizer_processor.safetensors``);
* the PaliGemma prompt ``"Task: <task>, State: <256-bin discretised state>;\\nAction: "`` tokenised
  with the checkpoint's ``tokenizer.json`` (truncation and right padding to the prompt length);
* camera aliasing (client key -> checkpoint slot) and the centred-padding resize.

Everything here is plain torch / numpy on the host; none of it is on the fp8 hot path.
"""

from __future__ import annotations

import glob
import json
import os
from typing import Any

import numpy as np
import torch
import torch.nn.functional as F  # noqa: N812

IMAGE_PREFIX = "observation.images."
STATE_KEY = "observation.state"
ACTION_KEY = "action"
TOKENS_KEY = "observation.language.tokens"
TOKEN_MASK_KEY = "observation.language.attention_mask"
DEFAULT_NORM_MAP = {"VISUAL": "IDENTITY", "STATE": "MEAN_STD", "ACTION": "MEAN_STD"}


class FeatureStats:
    """Per-feature ``mean`` / ``std`` tables and the feature-type -> mode map of a checkpoint.

    ``(x - mean) / (std + eps)`` forwards, ``x * std + mean`` backwards, eps 1e-8; a feature
    without statistics or with mode IDENTITY passes through (preprocess.py:61-85)."""

    def __init__(self, norm_map: dict[str, str] | None = None, tensors: dict[str, torch.Tensor] | None = None,
                 eps: float = 1e-8):
        self.norm_map = dict(DEFAULT_NORM_MAP if norm_map is None else norm_map)
        self.eps = eps
        self.stats: dict[str, dict[str, torch.Tensor]] = {}
        for flat, t in (tensors or {}).items():
            feature, stat = flat.rsplit(".", 1)
            self.stats.setdefault(feature, {})[stat] = t.to(torch.float32)

    @classmethod
    def from_files(cls, checkpoint_dir: str, pattern: str, norm_map: dict[str, str] | None) -> "FeatureStats":
        from safetensors import safe_open

        tensors: dict[str, torch.Tensor] = {}
        for path in sorted(glob.glob(os.path.join(checkpoint_dir, pattern))):
            with safe_open(path, "pt", "cpu") as f:
                for key in f.keys():
                    tensors[key] = f.get_tensor(key)
        return cls(norm_map, tensors)

    def _mode(self, feature: str, feature_type: str) -> str:
        mode = self.norm_map.get(feature_type, "IDENTITY")
        if mode == "IDENTITY" or feature not in self.stats:
            return "IDENTITY"
        if mode != "MEAN_STD":
            raise ValueError(f"Unsupported normalization mode: {mode}")
        if "mean" not in self.stats[feature] or "std" not in self.stats[feature]:
            raise ValueError("MEAN_STD normalization mode requires mean and std stats")
        return mode

    def normalize(self, x: torch.Tensor, feature: str, feature_type: str) -> torch.Tensor:
        if self._mode(feature, feature_type) == "IDENTITY":
            return x
        st = self.stats[feature]
        return (x - st["mean"].to(x.device, x.dtype)) / (st["std"].to(x.device, x.dtype) + self.eps)

    def unnormalize(self, x: torch.Tensor, feature: str, feature_type: str) -> torch.Tensor:
        if self._mode(feature, feature_type) == "IDENTITY":
            return x
        st = self.stats[feature]
        return x * st["std"].to(x.device, x.dtype) + st["mean"].to(x.device, x.dtype)


def load_state_stats(checkpoint_dir: str, norm_map) -> FeatureStats:
    return FeatureStats.from_files(checkpoint_dir, "policy_preprocessor_step_*_normalizer_processor.safetensors", norm_map)


def load_action_stats(checkpoint_dir: str, norm_map) -> FeatureStats:
    return FeatureStats.from_files(checkpoint_dir, "policy_postprocessor_step_*_unnormalizer_processor.safetensors", norm_map)


def prompt_text(task: str, normalized_state: torch.Tensor) -> str:
    """The pi0.5 prompt: the normalised state goes into the text, 256 bins over [-1, 1)
    (preprocess.py:112-123)."""
    edges = np.linspace(-1, 1, 257)[:-1]
    bins = np.digitize(normalized_state.detach().cpu().numpy(), bins=edges) - 1
    clean = task.strip().replace("_", " ").replace("\n", " ")
    return f"Task: {clean}, State: {' '.join(str(int(v)) for v in bins.reshape(-1))};\nAction: "


class PromptTokenizer:
    """``tokenizer.json`` of the checkpoint through the ``tokenizers`` package: truncation and
    right padding to ``max_length``; the file's own post-processor prepends ``<bos>``
    (tokenizer.py:16-48)."""

    def __init__(self, tokenizer_dir: str, max_length: int):
        from tokenizers import Tokenizer

        path = os.path.join(tokenizer_dir, "tokenizer.json")
        if not os.path.isfile(path):
            raise FileNotFoundError(f"{path} not found")
        self.tok = Tokenizer.from_file(path)
        self.max_length = int(max_length)
        self.tok.enable_truncation(max_length=self.max_length)
        pad = self.tok.token_to_id("<pad>")
        self.pad_id = 0 if pad is None else pad
        self.tok.enable_padding(pad_id=self.pad_id, pad_token="<pad>", length=self.max_length, direction="right")

    def encode(self, prompt: str) -> tuple[torch.Tensor, torch.Tensor]:
        """-> ``(ids [max_length] int64, mask [max_length] bool)``."""
        enc = self.tok.encode(prompt)
        return torch.tensor(enc.ids, dtype=torch.long), torch.tensor(enc.attention_mask, dtype=torch.bool)


def resolve_tokenizer_dir(checkpoint_dir: str, override: str | None = None) -> str | None:
    """Tokenizer directory: an explicit override, else ``tokenizer_processor.tokenizer_name`` of
    ``policy_preprocessor.json`` (absolute, or relative to the checkpoint), else a
    ``tokenizer.json`` lying in the checkpoint directory itself; ``None`` when there is none
    (config.py:177-210 raises there; this engine raises when a prompt has to be tokenised)."""
    if override:
        return os.path.abspath(override)
    name = ""
    pre = os.path.join(checkpoint_dir, "policy_preprocessor.json")
    if os.path.isfile(pre):
        with open(pre, encoding="utf-8") as f:
            for step in json.load(f).get("steps", []):
                if step.get("registry_name") == "tokenizer_processor":
                    name = step.get("config", {}).get("tokenizer_name", "")
                    break
    if name:
        for cand in (name, os.path.join(checkpoint_dir, name)):
            if os.path.isdir(cand):
                return cand
        raise ValueError(f"tokenizer dir {name!r} from policy_preprocessor.json does not exist "
                         f"(also not relative to {checkpoint_dir}); pass tokenizer_dir")
    if os.path.isfile(os.path.join(checkpoint_dir, "tokenizer.json")):
        return checkpoint_dir
    return None


def image_key(name: str) -> str:
    return name if name.startswith(IMAGE_PREFIX) else IMAGE_PREFIX + name


def normalise_alias(alias: dict[str, str] | None, image_features: list[str]) -> dict[str, str]:
    """``{client camera: checkpoint slot}`` with full ``observation.images.*`` keys on both sides
    and the reference's consistency checks (tybok/policies/pi05/engine.py:311-337)."""
    full: dict[str, str] = {}
    for src, dst in (alias or {}).items():
        s, d = image_key(src), image_key(dst)
        if d not in image_features:
            raise ValueError(f"camera_alias target {dst!r} is not an expected image feature "
                             f"(available: {[k[len(IMAGE_PREFIX):] for k in image_features]})")
        if s in image_features:
            raise ValueError(f"camera_alias source {src!r} is already an expected image feature")
        if s in full and full[s] != d:
            raise ValueError(f"camera_alias maps {src!r} twice to different targets")
        full[s] = d
    return full


def alias_frame(frame: dict[str, Any], alias: dict[str, str]) -> dict[str, Any]:
    """Rename aliased camera keys in a copy of the frame; a source is moved onto its slot only when
    the slot is not already there (preprocess.py:149-156)."""
    if not alias:
        return frame
    out = dict(frame)
    for src, dst in alias.items():
        if src in out and dst not in out:
            out[dst] = out.pop(src)
    return out


def resize_with_pad(img: torch.Tensor, height: int, width: int) -> torch.Tensor:
    """``[..., C, H, W]`` in [0, 1] -> ``[..., C, height, width]``: bilinear resize that keeps the
    aspect ratio, clamp, then zero padding centred with the odd pixel at the bottom / right
    (flow_matching.py:842-874)."""
    lead = img.shape[:-3]
    x = img.reshape(-1, *img.shape[-3:]).float()
    h, w = x.shape[-2:]
    ratio = max(w / width, h / height)
    nh, nw = int(h / ratio), int(w / ratio)
    x = F.interpolate(x, size=(nh, nw), mode="bilinear", align_corners=False).clamp(0.0, 1.0)
    top, rh = divmod(height - nh, 2)
    left, rw = divmod(width - nw, 2)
    x = F.pad(x, (left, left + rw, top, top + rh), value=0.0)
    return x.reshape(*lead, *x.shape[-3:])
