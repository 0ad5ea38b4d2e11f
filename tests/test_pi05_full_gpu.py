"""The benchmarked configuration itself against the CPU oracle.

The pi0.5-shaped policy at full size (SigLIP-So400m on two 224x224 cameras, 18-layer Gemma-2B-shaped
prefix over 544 tokens, 18-layer Gemma-300M-shaped expert, chunk 50, 10 flow steps), built exactly
as ``bench.py`` builds it -- vision tower in fp32 with TF32 GEMMs, first denoise step overlapped with the prefix, whole
chunk replayed from one CUDA graph, request through ``predict_action_chunk`` -- compared with
``oracle/pi05_ref.sample_actions`` (fp32 vision tower, bf16 dequantised decoders; the reference's
eager path, tybok/policies/pi05/models/flow_matching.py:761-838) on the same seeded weights and
inputs.  Tolerance: final action chunk with zero noise max-abs <= 2e-2; rel-L2 is printed.
"""

import pytest
import torch

from oracle import pi05_ref, w8_ref
from tybok_b200.shapes import PI05_FULL
from tybok_b200.weights import quantize_hot_linears, random_pi05_params

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def full_oracle_params():
    """Seed-0 weights of the full configuration, quantised and dequantised once for the oracle."""
    params = quantize_hot_linears(random_pi05_params(PI05_FULL, seed=0, device="cuda"), PI05_FULL)
    params = {k: v.cpu() for k, v in params.items()}
    torch.cuda.empty_cache()
    deq = {}
    for k, v in params.items():
        if k.endswith(".scale_weight"):
            continue
        deq[k] = w8_ref.dequant_w8(v, params[k[: -len("weight")] + "scale_weight"]) if v.dtype == torch.float8_e4m3fn else v
    return deq


def _frames(engine, batch, seed):
    s = engine.config.shape
    g = torch.Generator().manual_seed(seed)
    frames = []
    for _ in range(batch):
        images = {c: torch.rand(3, s.vision.image, s.vision.image, generator=g) for c in engine.describe()["cameras"]}
        fr = engine.make_frame(images, torch.randn(8, generator=g), "pick up the red block")
        fr["observation.language.tokens"] = torch.randint(0, s.vocab, (s.lang_len,), generator=g)
        mask = torch.ones(s.lang_len, dtype=torch.bool)
        mask[s.lang_len - 4:] = False  # a padded prompt tail: the pad mask and positions are exercised
        fr["observation.language.attention_mask"] = mask
        frames.append(fr)
    return frames


def _oracle_chunk(deq, frames, cams, noise):
    images = [torch.stack([fr[f"observation.images.{c}"] for fr in frames]) * 2.0 - 1.0 for c in cams]
    img_masks = [torch.ones(len(frames), dtype=torch.bool) for _ in cams]
    tokens = torch.stack([fr["observation.language.tokens"] for fr in frames])
    masks = torch.stack([fr["observation.language.attention_mask"] for fr in frames])
    return pi05_ref.sample_actions(deq, PI05_FULL, images, img_masks, tokens, masks, noise)


def test_benchmarked_configuration_matches_oracle(full_oracle_params):
    from tybok_b200 import ops
    from tybok_b200.engine import PI05B200Engine

    torch.set_num_threads(max(1, len(__import__("os").sched_getaffinity(0))))
    eng = PI05B200Engine("synthetic:pi05_full@0", device="cuda", graph=True, overlap=True, seed=0)
    assert eng.graph_enabled and eng.model.overlap and eng.model.vision_dtype == torch.float16  # the default tower
    frames = _frames(eng, 1, seed=100)
    noise = torch.zeros(1, PI05_FULL.chunk, PI05_FULL.max_action_dim)
    assert eng._predict_chunk_static(frames[0], noise) is not None  # the path bench.py's e2e leg times
    out = torch.from_numpy(eng.predict_action_chunk(frames[0], noise=noise))
    ops.check_status()
    ref = _oracle_chunk(full_oracle_params, frames, eng.describe()["cameras"], noise)[0]
    err, rel = float((out - ref).abs().max()), w8_ref.rel_l2(out, ref)
    print(f"pi05_full batch 1: max-abs {err:.3e}, rel-L2 {rel:.3e}, |ref|max {float(ref.abs().max()):.3f}")
    assert torch.isfinite(out).all()
    assert err <= 2e-2
    del eng
    torch.cuda.empty_cache()


def test_benchmarked_configuration_batch8_matches_oracle(full_oracle_params):
    """The batched-throughput form (8 requests per replica, one graph) against the batch-generic oracle."""
    from tybok_b200 import ops
    from tybok_b200.engine import PI05B200Engine

    b = 8
    eng = PI05B200Engine("synthetic:pi05_full@0", device="cuda", graph=True, overlap=True, seed=0, batch_size=b)
    frames = _frames(eng, b, seed=200)
    noise = torch.zeros(b, PI05_FULL.chunk, PI05_FULL.max_action_dim)
    out = torch.from_numpy(eng.predict_action_chunks(frames, noise=noise))
    ops.check_status()
    ref = _oracle_chunk(full_oracle_params, frames, eng.describe()["cameras"], noise)
    err, rel = float((out - ref).abs().max()), w8_ref.rel_l2(out, ref)
    print(f"pi05_full batch {b}: max-abs {err:.3e}, rel-L2 {rel:.3e}")
    assert err <= 2e-2
    del eng
    torch.cuda.empty_cache()
