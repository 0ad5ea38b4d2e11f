"""The DiT block on the GPU kernels -- qk-norm + rotary + KV-store kernel, affine LayerNorm, head_dim
128 attention (self over ``[earlier ; own]`` keys, masked cross), FFN tail -- against the oracle's
restatement of ``FastWAMAttentionBlock.forward`` (tybok/policies/fastwam/models/dit_block.py:328-400)
and against the fixture that the reference's own block produced.  Tolerance rel-L2 <= 1e-2 per block."""

import os
import sys

import pytest
import torch

sys.path.insert(0, os.path.join(os.path.dirname(__file__), "golden"))
from make_golden import dit_block_case  # noqa: E402

from oracle import dit_ref, w8_ref  # noqa: E402
from tybok_b200.shapes import DIT_TINY, DiTShape  # noqa: E402
from tybok_b200.weights import quantize_dit_block, random_dit_block_params  # noqa: E402

pytestmark = pytest.mark.gpu


def _ulp_close(a, b, ulps=2):
    """bf16 tensors equal up to a couple of units in the last place of the larger magnitude."""
    a, b = a.float(), b.float()
    tol = ulps * 2.0**-8 * torch.maximum(a.abs(), b.abs()).clamp_min(1e-30)
    return bool(((a - b).abs() <= tol).all())


@pytest.mark.parametrize("b,l,h,d,key_off", [(1, 70, 2, 128, 0), (2, 33, 24, 128, 5), (1, 9, 3, 256, 0)])
def test_qknorm_rope_store(b, l, h, d, key_off):
    from tybok_b200 import ops

    g = torch.Generator().manual_seed(b * 100 + l)
    a = h * d
    qkv = torch.empty(b * l, 3 * a).normal_(0, 1.5, generator=g).to(torch.bfloat16)
    wq, wk = ((1 + torch.empty(a).normal_(0, 0.2, generator=g)).to(torch.bfloat16) for _ in range(2))
    ang = torch.outer(torch.arange(l, dtype=torch.float64), 1.0 / torch.pow(10000, torch.arange(0, d, 2, dtype=torch.float64) / d))
    freqs = torch.polar(torch.ones_like(ang), ang)[:, None, :]
    q3, k3, v3 = (t.reshape(b, l, a) for t in qkv.chunk(3, dim=-1))
    rq = dit_ref.apply_dense_rope(dit_ref.wan_rms_norm(q3, wq, 1e-6), freqs, h)
    rk = dit_ref.apply_dense_rope(dit_ref.wan_rms_norm(k3, wk, 1e-6), freqs, h)
    lcap = key_off + l + 2
    kc = torch.zeros(b, h, lcap, d, dtype=torch.bfloat16, device="cuda")
    vc = torch.zeros_like(kc)
    f = freqs.reshape(l, -1).to(torch.complex64)
    q = ops.qknorm_rope_store(qkv.cuda(), q_off=0, k_off=a, v_off=2 * a, norm_q=wq.cuda(), norm_k=wk.cuda(),
                              cos=f.real.float().contiguous().cuda(), sin=f.imag.float().contiguous().cuda(), k_cache=kc,
                              v_cache=vc, batch=b, heads=h, head_dim=d, key_off=key_off)
    torch.cuda.synchronize()
    assert _ulp_close(q.cpu().view(b, l, a), rq) and w8_ref.rel_l2(q.cpu().view(b, l, a), rq) <= 2e-3
    got_k = kc[:, :, key_off : key_off + l].cpu().transpose(1, 2).reshape(b, l, a)
    assert _ulp_close(got_k, rk) and w8_ref.rel_l2(got_k, rk) <= 2e-3
    assert torch.equal(vc[:, :, key_off : key_off + l].cpu().transpose(1, 2).reshape(b, l, a), v3)
    assert not kc[:, :, :key_off].any() and not kc[:, :, key_off + l :].any()  # nothing outside the key range
    # q only, no rotation (the cross-attention query)
    q2 = ops.qknorm_rope_store(qkv.cuda(), q_off=0, norm_q=wq.cuda(), batch=b, heads=h, head_dim=d)
    assert _ulp_close(q2.cpu().view(b, l, a), dit_ref.wan_rms_norm(q3, wq, 1e-6))


@pytest.mark.parametrize("m,w", [(70, 256), (33, 3072), (5, 1024)])
def test_layernorm_affine(m, w):
    from tybok_b200 import ops

    g = torch.Generator().manual_seed(m + w)
    x = torch.empty(m, w).normal_(0.3, 2, generator=g).to(torch.bfloat16)
    wt = (1 + torch.empty(w).normal_(0, 0.3, generator=g)).to(torch.bfloat16)
    bs = torch.empty(w).normal_(0, 0.3, generator=g).to(torch.bfloat16)
    ref = dit_ref.wan_layer_norm(x, 1e-6, wt, bs)
    y, yp = ops.layernorm_affine(x.cuda(), wt.cuda(), bs.cuda(), out_bf16=True, out_planes=True, out_shift=4)
    assert _ulp_close(y.cpu(), ref) and w8_ref.rel_l2(y.cpu(), ref) <= 2e-3
    got, want = yp.cpu().view(torch.float8_e5m2).float().sum(0), y.cpu().float() * 16.0
    inside = want.abs() >= 2.0**-7
    assert torch.equal(got[inside], want[inside])


def _run_block(bp, shape, x, context, context_mask, t_mod, freqs, video_kv=None):
    from tybok_b200 import ops
    from tybok_b200.dit import DiTBlock, rotary_parts

    blk = DiTBlock(bp, shape, device="cuda")
    s = x.shape[1]
    lv = 0 if video_kv is None else video_kv[0].shape[1]
    cos, sin = rotary_parts(freqs, "cuda")
    if video_kv is None:
        mk = lambda: torch.zeros(1, shape.heads, s + 3, shape.head_dim, dtype=torch.bfloat16, device="cuda")  # noqa: E731
        cache = (mk(), mk())
    else:
        kc, vc = blk.store_context_kv(video_kv[0].cuda(), video_kv[1].cuda())
        pad = torch.zeros(1, shape.heads, s, shape.head_dim, dtype=torch.bfloat16, device="cuda")
        cache = (torch.cat([kc, pad], 2).contiguous(), torch.cat([vc, pad], 2).contiguous())
    cross = blk.context_cache(context[0].cuda())
    valid = context_mask.to(torch.uint8).cuda().contiguous()
    y = blk.forward(x[0].cuda(), blk.modulations(t_mod[0].cuda()), cos, sin, cache, lv, cross, valid)
    ops.check_status()
    return y.cpu()[None], cache, lv


@pytest.mark.parametrize("tag,prefix", [("dit_block", 0), ("dit_block_video_kv", 40)])
def test_block_matches_reference_fixture(golden, tag, prefix):
    bp = quantize_dit_block(random_dit_block_params(DIT_TINY, seed=0))
    x, context, context_mask, t_mod, freqs, video_kv = dit_block_case(DIT_TINY, video_prefix=prefix)
    y, cache, lv = _run_block(bp, DIT_TINY, x, context, context_mask, t_mod, freqs, video_kv)
    g = golden[tag]
    s, a = x.shape[1], DIT_TINY.heads * DIT_TINY.head_dim
    k = cache[0][:, :, lv : lv + s].cpu().transpose(1, 2).reshape(1, s, a)
    assert w8_ref.rel_l2(k, g["k"]) <= 1e-2
    err, added = w8_ref.rel_l2(y, g["y"]), w8_ref.rel_l2(y.float() - x.float(), g["y"].float() - x.float())
    print(f"{tag}: rel-L2 of the block output {err:.3e}, of what the block adds to x {added:.3e}")
    assert err <= 1e-2  # the stated per-block tolerance
    assert added <= 3e-2  # six GEMMs and two attentions deep, measured against the part the block computes


def test_block_at_the_full_widths():
    """Hidden 3072, 24 heads x 128, FFN 14336 (one block of the fastWAM-class denoiser) on 300 tokens
    over a 129-token context with a padded tail, against the oracle."""
    shape = DiTShape(video_tokens=250, action_tokens=50)
    bp = quantize_dit_block(random_dit_block_params(shape, seed=1, device="cuda"))
    bp_cpu = {k: v.cpu() for k, v in bp.items()}
    x, context, context_mask, t_mod, freqs, _ = dit_block_case(shape, seed=12)
    ref = dit_ref.block_forward(bp_cpu, shape.heads, x, context, t_mod, freqs, context_mask)
    y, _, _ = _run_block(bp, shape, x, context, context_mask, t_mod, freqs)
    assert torch.isfinite(y.float()).all()
    err, added = w8_ref.rel_l2(y, ref), w8_ref.rel_l2(y.float() - x.float(), ref.float() - x.float())
    print(f"full-width block: rel-L2 of the output {err:.3e}, of what the block adds to x {added:.3e}")
    assert err <= 1e-2 and added <= 3e-2


def test_denoiser_loop_and_runner_contract():
    """Two blocks, two steps over token space against ``dit_ref.denoise``; and the fused-runner
    contract (``run_action_layers``: per-layer video keys / values and finished cross keys / values
    handed in by the caller, tybok/policies/fastwam/models/fused_action.py:318-357) against the
    oracle's per-layer loop."""
    from tybok_b200 import ops
    from tybok_b200.dit import DiTDenoiser, rotary_parts

    shape = DIT_TINY
    bps = [quantize_dit_block(random_dit_block_params(shape, seed=20 + i)) for i in range(2)]
    x, context, context_mask, t_mod, freqs, _ = dit_block_case(shape, seed=30)
    g = torch.Generator().manual_seed(31)
    t_mods = torch.empty(2, 1, 6, shape.hidden).normal_(0, 0.5, generator=g).to(torch.bfloat16)
    deltas = dit_ref.sampling_deltas(2)
    ref = dit_ref.denoise(bps, shape.heads, x, context, list(t_mods), freqs, context_mask, deltas)
    den = DiTDenoiser(bps, shape, device="cuda")
    den.prepare_context(context[0].cuda(), context_mask[0])
    cos, sin = rotary_parts(freqs, "cuda")
    out = den.denoise(x[0].cuda(), t_mods[:, 0].cuda(), cos, sin, deltas)
    ops.check_status()
    assert w8_ref.rel_l2(out.cpu()[None], ref) <= 1e-2

    # runner contract: the action tokens attend to 40 video keys per layer; cross k/v arrive finished
    xa, context, context_mask, t_mod, freqs, _ = dit_block_case(shape, seed=32, video_prefix=40)
    a = shape.heads * shape.head_dim
    video = [{"k": torch.empty(1, 40, a).normal_(0, 1, generator=g).to(torch.bfloat16),
              "v": torch.empty(1, 40, a).normal_(0, 1, generator=g).to(torch.bfloat16)} for _ in bps]
    cross = [dit_ref.cross_kv(p, context) for p in bps]
    want = xa
    for p, vkv in zip(bps, video):
        want = dit_ref.block_forward(p, shape.heads, want, context, t_mod, freqs, context_mask, (vkv["k"], vkv["v"]))
    got = den.run_action_layers(xa.cuda(), t_mod.cuda(), freqs, [{k: v.cuda() for k, v in d.items()} for d in video],
                                [(k.cuda(), v.cuda()) for k, v in cross], context_mask[0].cuda())
    ops.check_status()
    assert got.shape == xa.shape and w8_ref.rel_l2(got.cpu(), want) <= 1e-2
    with pytest.raises(ValueError, match="layer counts"):
        den.run_action_layers(xa.cuda(), t_mod.cuda(), freqs, video[:1], cross, context_mask[0].cuda())
