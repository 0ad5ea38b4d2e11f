"""Shape descriptions of the policies this package accelerates.

The hot path is shape-generic; these dataclasses only name the configurations
the parity tests and the benchmark run.  Field names follow the reference's
``GEMMA_VARIANTS`` table and ``PI05Config`` (tybok/policies/pi05/config.py:15-32,54-90)
so a checkpoint ``config.json`` maps onto them one to one.
"""

from __future__ import annotations

from dataclasses import dataclass, field, replace


@dataclass(frozen=True)
class GemmaSpec:
    """One Gemma decoder stack (tybok/policies/pi05/config.py:35-50)."""

    width: int
    depth: int
    mlp_dim: int
    num_heads: int
    num_kv_heads: int
    head_dim: int


@dataclass(frozen=True)
class SiglipSpec:
    """SigLIP tower geometry (tybok/policies/pi05/models/paligemma_with_expert.py:48-58)."""

    hidden: int = 1152
    heads: int = 16
    layers: int = 27
    mlp_dim: int = 4304
    image: int = 224
    patch: int = 14

    @property
    def tokens(self) -> int:
        return (self.image // self.patch) ** 2


@dataclass(frozen=True)
class PI05Shape:
    """A pi0.5-shaped policy: SigLIP -> projector -> VLM prefix -> AdaRMS expert."""

    vlm: GemmaSpec
    expert: GemmaSpec
    vision: SiglipSpec = field(default_factory=SiglipSpec)
    n_cams: int = 2
    lang_len: int = 32
    vocab: int = 257152
    chunk: int = 50
    steps: int = 10
    max_action_dim: int = 32
    action_dim: int = 32
    min_period: float = 4e-3
    max_period: float = 4.0

    @property
    def prefix_len(self) -> int:
        return self.n_cams * self.vision.tokens + self.lang_len

    def with_(self, **kw) -> "PI05Shape":
        return replace(self, **kw)


GEMMA_2B = GemmaSpec(2048, 18, 16384, 8, 1, 256)
GEMMA_300M = GemmaSpec(1024, 18, 4096, 8, 1, 256)

#: Variant names a checkpoint's ``config.json`` may carry (``paligemma_variant`` /
#: ``action_expert_variant``).  A plain module dict, as the reference's ``GEMMA_VARIANTS``
#: (tybok/policies/pi05/config.py:15-32): tests register small variants at run time.
GEMMA_VARIANTS: dict[str, GemmaSpec] = {"gemma_2b": GEMMA_2B, "gemma_300m": GEMMA_300M}

#: The pi0.5-shaped policy the headline latency is quoted on: SigLIP-So400m on two 224x224
#: cameras, a Gemma-2B-shaped prefix over 544 tokens, a Gemma-300M-shaped expert, chunk 50, 10 steps.
PI05_FULL = PI05Shape(vlm=GEMMA_2B, expert=GEMMA_300M)

#: A tiny policy with the same structure (MQA like pi0.5) and head_dim 128, the smaller of the
#: two head sizes the attention kernels serve; used by the CPU oracle fixtures and GPU parity tests.
PI05_TINY = PI05Shape(
    vlm=GemmaSpec(256, 2, 512, 2, 1, 128),
    expert=GemmaSpec(128, 2, 256, 2, 1, 128),
    vision=SiglipSpec(hidden=128, heads=4, layers=2, mlp_dim=256, image=56, patch=14),
    n_cams=2,
    lang_len=16,
    vocab=512,
    chunk=10,
    steps=3,
)

#: A small policy with the real head geometry (MQA, head_dim 256), so GPU parity tests run the
#: attention kernel inside the model; 130-token prefix = two key blocks.
PI05_SMALL = PI05Shape(
    vlm=GemmaSpec(256, 2, 512, 2, 1, 256),
    expert=GemmaSpec(128, 2, 256, 2, 1, 256),
    vision=SiglipSpec(hidden=128, heads=4, layers=2, mlp_dim=256, image=70, patch=14),
    n_cams=2,
    lang_len=80,
    vocab=512,
    chunk=10,
    steps=3,
)

#: The W8 linear sweep: the Gemma-2B and Gemma-300M-expert projection shapes (N, K) and token counts M.
W8_SWEEP_NK = ((16384, 2048), (2048, 16384), (2560, 2048), (4096, 1024), (1024, 4096))
W8_SWEEP_M = (1, 50, 256, 800)


@dataclass(frozen=True)
class DiTShape:
    """fastWAM-class DiT denoiser: 30 blocks of hidden 3072, 24 heads x 128, FFN 14336 over 4096
    latent-video + 50 action tokens (tybok/policies/fastwam/models/dit_block.py:328-400)."""

    hidden: int = 3072
    heads: int = 24
    head_dim: int = 128
    ffn: int = 14336
    blocks: int = 30
    video_tokens: int = 4096
    action_tokens: int = 50
    steps: int = 4
    state_dim: int = 14
    context_len: int = 129
    text_dim: int = 4096

    @property
    def seq(self) -> int:
        return self.video_tokens + self.action_tokens


DIT_FULL = DiTShape()
DIT_TINY = DiTShape(hidden=256, heads=2, head_dim=128, ffn=512, blocks=2, video_tokens=96,
                    action_tokens=10, steps=2, context_len=17, text_dim=64)
