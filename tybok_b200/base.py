"""The engine interface this package plugs into.

When the reference package is importable, ``PolicyEngine`` / ``register`` are the reference's
own (tybok/base.py:50-108, tybok/registry.py:33-42), so an engine defined here is a genuine
backend of a running tybok installation.  Otherwise a structural twin with the same method set
is used, so the engine and its tests do not depend on the reference being installed.
"""

from __future__ import annotations

import os
import sys
from abc import ABC, abstractmethod
from typing import Any

import numpy as np
import torch


def _import_reference():
    root = os.environ.get("TYBOK_REFERENCE")
    if root and os.path.isdir(root) and root not in sys.path:
        sys.path.insert(0, root)
    try:
        from tybok.base import PolicyEngine as RefEngine  # type: ignore
        from tybok.registry import register as ref_register  # type: ignore
        from tybok.registry import reject_unsupported_flags as ref_reject  # type: ignore

        return RefEngine, ref_register, ref_reject
    except Exception:  # the reference is optional
        return None


_ref = _import_reference()
HAVE_REFERENCE = _ref is not None

if HAVE_REFERENCE:
    PolicyEngine, register, reject_unsupported_flags = _ref
else:
    _REGISTRY: dict[str, type] = {}

    def register(name: str):
        """Class decorator with the reference's semantics (tybok/registry.py:33-42)."""

        def deco(cls):
            if name in _REGISTRY:
                raise ValueError(f"engine '{name}' already registered")
            _REGISTRY[name] = cls
            return cls

        return deco

    def reject_unsupported_flags(cls, model_type: str, kwargs: dict[str, Any]) -> None:
        """tybok/registry.py:97-119: a flag whose value differs from its inert default was
        requested; a backend that does not implement it must fail loudly."""
        for flag, inert in (getattr(cls, "_UNSUPPORTED_FLAGS", None) or {}).items():
            if flag in kwargs and kwargs[flag] != inert:
                raise NotImplementedError(f"--{flag.replace('_', '-')} is not supported by the {model_type} backend")

    class PolicyEngine(ABC):
        """Structural twin of tybok/base.py:50-156 (interface + ``make_frame``)."""

        config: Any
        compile_model: bool
        graph_enabled: bool

        def __init__(self, checkpoint_dir: str, device: str = "auto", **kwargs):
            self.checkpoint_dir = checkpoint_dir
            if device == "auto":
                device = "cuda" if torch.cuda.is_available() else "cpu"
            self.device = device
            self.compiled_regions: list[str] = []
            if isinstance(device, str) and device.startswith("cuda"):
                dev = torch.device(device)
                if dev.index is not None:
                    torch.cuda.set_device(dev)

        @abstractmethod
        def describe(self) -> dict[str, Any]: ...

        @abstractmethod
        def select_action(self, frame, noise=None) -> np.ndarray: ...

        @abstractmethod
        def predict_action_chunk(self, frame, noise=None) -> np.ndarray: ...

        @abstractmethod
        def validate(self, reference_dir: str) -> dict[str, float]: ...

        def supports_rtc(self) -> bool:
            return False

        def make_frame(self, images, state, task: str) -> dict[str, Any]:
            frame: dict[str, Any] = {}
            for key, img in images.items():
                if isinstance(img, np.ndarray):
                    img = torch.from_numpy(img)
                if not torch.is_tensor(img):
                    raise TypeError(f"image {key} must be a tensor or ndarray")
                if img.ndim == 3 and img.shape[0] not in (1, 3, 4):
                    img = img.permute(2, 0, 1)
                frame[f"observation.images.{key}"] = img.float().contiguous()
            if isinstance(state, (list, tuple)):
                state = np.asarray(state, dtype=np.float32)
            if isinstance(state, np.ndarray):
                state = torch.from_numpy(state.astype(np.float32))
            frame["observation.state"] = state.float().contiguous()
            frame["task"] = task
            return frame
