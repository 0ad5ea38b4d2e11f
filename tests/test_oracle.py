"""The CPU oracle against fixtures produced by the reference's own modules
(tests/golden/make_golden.py) and against the quantiser's documented identities."""

import os
import sys

import pytest
import torch

sys.path.insert(0, os.path.join(os.path.dirname(__file__), "golden"))

from make_golden import checksum, dit_case, linear_case, tiny_inputs  # noqa: E402

from oracle import pi05_ref, w8_ref  # noqa: E402
from tybok_b200.shapes import PI05_TINY  # noqa: E402
from tybok_b200.weights import quantize_hot_linears, quantize_w8, random_pi05_params  # noqa: E402


@pytest.mark.parametrize("tag,mnk", [("lin_small", (50, 256, 512)), ("lin_ragged", (7, 192, 320))])
def test_w8_linear_matches_reference(golden, tag, mnk):
    w, x = linear_case(1, *mnk)
    g = golden[tag]
    assert checksum(w, x) == g["in_sum"], "seeded inputs differ from the ones the fixture was made with"
    w8, scale = w8_ref.quantize_w8(w)
    assert torch.equal(w8.view(torch.uint8), g["w8"])  # bit-exact quantiser
    assert torch.equal(scale, g["scale"])
    assert torch.equal(w8_ref.w8_linear(x, w8, scale), g["y"])
    # the product package's quantiser is the same recipe
    w8p, scalep = quantize_w8(w)
    assert torch.equal(w8p.view(torch.uint8), g["w8"]) and torch.equal(scalep, g["scale"])


def test_quantiser_identities():
    """docs/fastWAM_weight_quantization.md:26-30,141-158: worst-case error 16/448 of the row
    maximum, and re-quantising with the stored scale is byte-exact."""
    g = torch.Generator().manual_seed(5)
    w = torch.empty(64, 4096).normal_(0, 0.02, generator=g)
    w8, scale = w8_ref.quantize_w8(w)
    deq = w8.float() * scale[:, None]
    err = ((deq - w).abs().amax(dim=1) / w.abs().amax(dim=1)).max()
    assert err <= 16.0 / 448.0 + 1e-6
    again = (deq / scale[:, None]).to(torch.float8_e4m3fn)
    assert torch.equal(again.view(torch.uint8), w8.view(torch.uint8))
    assert float(w8.float().abs().max()) == 448.0
    # all-zero row -> clamp, not NaN
    w8z, sz = w8_ref.quantize_w8(torch.zeros(2, 16))
    assert float(sz[0]) == pytest.approx(1e-12) and not torch.isnan(w8z.float()).any()


def test_gated_mlp_matches_reference(golden):
    g = torch.Generator().manual_seed(2)
    x = torch.empty(1, 50, 256).normal_(0, 1, generator=g).to(torch.bfloat16)
    ws = [torch.empty(s).normal_(0, 0.02, generator=g) for s in ((512, 256), (512, 256), (256, 512))]
    assert checksum(x, *ws) == golden["mlp"]["in_sum"]
    gate, up, down = (w8_ref.quantize_w8(w) for w in ws)
    assert torch.equal(w8_ref.gemma_mlp(x, gate, up, down), golden["mlp"]["y"])


def test_dit_ffn_tail_matches_reference(golden):
    x, mods, ws = dit_case()
    assert checksum(x, *mods, *[t for pair in ws for t in pair]) == golden["dit_ffn"]["in_sum"]
    up, down = ((*w8_ref.quantize_w8(w), b) for w, b in ws)
    assert torch.equal(w8_ref.dit_ffn_tail(x, *mods, up, down), golden["dit_ffn"]["y"])


def _tiny_params():
    return quantize_hot_linears(random_pi05_params(PI05_TINY, seed=0), PI05_TINY)


def test_pi05_tiny_chunk_matches_reference(golden):
    params = _tiny_params()
    images, img_masks, tokens, masks, noise = tiny_inputs(PI05_TINY)
    g = golden["pi05_tiny"]
    assert checksum(*images, tokens, *params.values()) == g["in_sum"]
    actions, inter = pi05_ref.sample_actions(params, PI05_TINY, images, img_masks, tokens, masks, noise,
                                             return_intermediates=True)
    assert torch.equal(inter["prefix_embs"][:, ::37], g["prefix_embs"])
    assert torch.equal(actions, g["actions"])


def test_pi05_tiny_batch2_matches_reference(golden):
    params = _tiny_params()
    images, img_masks, tokens, masks, noise = tiny_inputs(PI05_TINY, seed=3, batch=2)
    actions = pi05_ref.sample_actions(params, PI05_TINY, images, img_masks, tokens, masks, noise)
    assert torch.equal(actions, golden["pi05_tiny_b2"]["actions"])


@pytest.mark.parametrize("tag,prefix", [("dit_block", 0), ("dit_block_video_kv", 40)])
def test_dit_block_matches_reference(golden, tag, prefix):
    """``FastWAMAttentionBlock.forward`` (self-attention with qk-norm and dense RoPE, masked
    cross-attention, modulated FFN), without and with keys / values of earlier tokens."""
    from make_golden import dit_block_case

    from oracle import dit_ref
    from tybok_b200.shapes import DIT_TINY
    from tybok_b200.weights import quantize_dit_block, random_dit_block_params

    bp = quantize_dit_block(random_dit_block_params(DIT_TINY, seed=0))
    x, context, context_mask, t_mod, freqs, video_kv = dit_block_case(DIT_TINY, video_prefix=prefix)
    g = golden[tag]
    assert checksum(x, context, t_mod, torch.view_as_real(freqs), *bp.values()) == g["in_sum"]
    y, (k, v) = dit_ref.block_forward(bp, DIT_TINY.heads, x, context, t_mod, freqs, context_mask, video_kv, return_kv=True)
    assert torch.equal(k, g["k"]) and torch.equal(v, g["v"])
    assert torch.equal(y, g["y"])
