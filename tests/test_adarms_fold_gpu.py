"""The AdaRMS norm folded into the GEMMs around it (action expert below the two-plane threshold):
the residual GEMM writes planes of ``bf16(x (1 + scale))`` and per-tile row sums of squares, the next
GEMM applies ``rsqrt(mean + eps)`` and ``W shift`` in its epilogue.  Checked against the norm kernel
followed by the plain GEMM (same math, another bf16 rounding point) and against the oracle's
W8A16 linear on a torch restatement of the norm (layers.py:34-84), rel-L2 <= 1e-2."""

import os
import sys

import pytest
import torch

sys.path.insert(0, os.path.join(os.path.dirname(__file__), "golden"))

from oracle import w8_ref  # noqa: E402

pytestmark = pytest.mark.gpu
TOL = 1e-2
EPS = 1e-6


def adarms_ref(x: torch.Tensor, scale: torch.Tensor, shift: torch.Tensor) -> torch.Tensor:
    xf = x.float()
    r = torch.rsqrt(xf.pow(2).mean(dim=-1, keepdim=True) + EPS)
    return (xf * r * (1.0 + scale) + shift).to(torch.bfloat16)


def _setup(m, w, k_in, seed, stream_scale=1.0):
    g = torch.Generator().manual_seed(seed)
    a = torch.empty(m, k_in).normal_(0, 0.5, generator=g).to(torch.bfloat16)                  # input of the residual GEMM
    res = (torch.empty(m, w).normal_(0, stream_scale, generator=g) *
           torch.exp(torch.empty(1, w).normal_(0, 1, generator=g))).to(torch.bfloat16)      # residual stream with wide channels
    wo = w8_ref.quantize_w8(torch.empty(w, k_in).normal_(0, 0.03, generator=g))
    mod = torch.empty(1, 3 * w).normal_(0, 0.3, generator=g)                                   # scale | shift | gate of the next norm
    gate = torch.empty(w).normal_(0, 1, generator=g)
    return g, a, res, wo, mod, gate


@pytest.mark.parametrize("m,w,k_in,inter,stream_scale", [(50, 1024, 2048, 4096, 1.0), (50, 1024, 4096, 1024, 30.0),
                                                         (10, 256, 256, 512, 0.05), (100, 384, 128, 192, 1.0)])
def test_residual_then_gated_ffn_with_the_norm_folded_in(m, w, k_in, inter, stream_scale):
    from tybok_b200 import ops

    g, a, res, wo, mod, gate = _setup(m, w, k_in, 11 + m, stream_scale)
    wg = w8_ref.quantize_w8(torch.empty(inter, w).normal_(0, 0.03, generator=g))
    wu = w8_ref.quantize_w8(torch.empty(inter, w).normal_(0, 0.03, generator=g))
    dev = torch.device("cuda")
    ap = ops.split3(a.to(dev), 6)
    wod = (wo[0].to(dev), wo[1].to(dev))
    modd, gated, resd = mod.to(dev), gate.to(dev), res.to(dev)
    packed = ops.pack_gate_up(wg[0].to(dev), wg[1].to(dev), wu[0].to(dev), wu[1].to(dev))
    # the norm kernel between the two GEMMs
    x1, _ = ops.w8x3_linear(ap, 6, *wod, epilogue=ops.EPI_RESIDUAL, residual=resd, gate=gated[None], rows_per_gate=m)
    xp = ops.rmsnorm(x1, mod=modd, rows_per_group=m, out_shift=4)[1]
    h_plain, _ = ops.w8x3_geglu_packed(xp, 4, *packed)
    # the folded form
    x2, up, part = ops.w8x3_residual_next_adarms(ap, 6, *wod, resd, gated, modd[0, :w], out_shift=0)
    bias = ops.shift_bias_rows(packed[0], packed[1], modd[0, w : 2 * w])
    h_fold, hp = ops.w8x3_geglu_packed_adarms(up, 0, part, bias, *packed, out_bf16=True, out_planes=True, out_shift=4)
    ops.check_status()
    assert torch.equal(x1, x2)
    ss = x1.double().pow(2).sum(dim=1).cpu()
    assert part.shape == (w // 128, m)
    assert torch.allclose(part.double().sum(dim=0).cpu(), ss, rtol=1e-5)
    u_ref = (x1.float().cpu() * (1.0 + mod[0, :w])).to(torch.bfloat16).float()
    u_got = up.cpu().view(torch.float8_e5m2).float().sum(0)
    inside = u_ref.abs() >= 2.0**-7
    assert torch.equal(u_got[inside], u_ref[inside])
    assert float((u_got - u_ref).abs().max()) <= 2.0**-16
    # against the oracle on the norm restated in torch, and against the unfolded kernels
    y = adarms_ref(x1.cpu(), mod[0, :w], mod[0, w : 2 * w])
    ref = w8_ref.gelu_tanh(w8_ref.w8_linear(y, *wg)) * w8_ref.w8_linear(y, *wu)
    assert w8_ref.rel_l2(h_plain.cpu(), ref) <= TOL
    assert w8_ref.rel_l2(h_fold.cpu(), ref) <= TOL
    assert w8_ref.rel_l2(h_fold.cpu(), h_plain.cpu()) <= 8e-3  # two bf16 rounding points apart
    got, want = hp.cpu().view(torch.float8_e5m2).float().sum(0), h_fold.cpu().float() * 16.0
    inside = want.abs() >= 2.0**-7
    assert torch.equal(got[inside], want[inside])
    # bit-reproducible
    x3, up3, part3 = ops.w8x3_residual_next_adarms(ap, 6, *wod, resd, gated, modd[0, :w], out_shift=0)
    assert torch.equal(up, up3) and torch.equal(part, part3)


@pytest.mark.parametrize("b,l,h,gk,w,k_in,key_off,d", [(1, 50, 8, 1, 1024, 4096, 544, 256), (2, 10, 2, 1, 256, 128, 38, 128)])
def test_residual_then_qkv_rope_with_the_norm_folded_in(b, l, h, gk, w, k_in, key_off, d):
    from tybok_b200 import ops

    m = b * l
    g, a, res, wo, mod, gate = _setup(m, w, k_in, 5 + l)
    wq = w8_ref.quantize_w8(torch.empty((h + 2 * gk) * d, w).normal_(0, 0.03, generator=g))
    dev = torch.device("cuda")
    ap = ops.split3(a.to(dev), 4)
    wod = (wo[0].to(dev), wo[1].to(dev))
    modd, gated, resd = mod.to(dev), gate.to(dev), res.to(dev)
    pos = (torch.arange(l, dtype=torch.int32)[None] + torch.tensor([[3], [11]], dtype=torch.int32)[:b]).reshape(-1).to(dev)
    cos, sin = w8_ref.rope_cos_sin(torch.arange(1024)[None], d, torch.bfloat16)
    cos, sin = cos[0].contiguous().to(dev), sin[0].contiguous().to(dev)
    lcap = key_off + l + 3
    caches = [torch.zeros(b, gk, lcap, d, dtype=torch.bfloat16, device=dev) for _ in range(4)]
    wp, sp = ops.pair_qkv_rows(wq[0].to(dev), wq[1].to(dev), d)
    x1, _ = ops.w8x3_linear(ap, 4, *wod, epilogue=ops.EPI_RESIDUAL, residual=resd, gate=gated[None], rows_per_gate=m)
    xp = ops.rmsnorm(x1, mod=modd, rows_per_group=m, out_shift=4)[1]
    q_plain = ops.w8x3_qkv_rope(xp, 4, wp, sp, pos, cos, sin, caches[0], caches[1], heads=h, key_off=key_off)
    x2, up, part = ops.w8x3_residual_next_adarms(ap, 4, *wod, resd, gated, modd[0, :w], out_shift=0)
    bias = ops.shift_bias_rows(wp, sp, modd[0, w : 2 * w])
    q_fold = ops.w8x3_qkv_rope_adarms(up, 0, part, bias, wp, sp, pos, cos, sin, caches[2], caches[3], heads=h, key_off=key_off)
    ops.check_status()
    assert torch.equal(x1, x2)
    assert w8_ref.rel_l2(q_fold.float().cpu(), q_plain.float().cpu()) <= 8e-3  # two bf16 rounding points apart
    assert w8_ref.rel_l2(caches[2].float().cpu(), caches[0].float().cpu()) <= 8e-3
    assert w8_ref.rel_l2(caches[3].float().cpu(), caches[1].float().cpu()) <= 8e-3
    # the unrotated value rows against the oracle
    y = adarms_ref(x1.cpu(), mod[0, :w], mod[0, w : 2 * w])
    v_ref = w8_ref.w8_linear(y, *wq)[:, (h + gk) * d :].reshape(b, l, gk, d).permute(0, 2, 1, 3)
    assert w8_ref.rel_l2(caches[3][:, :, key_off : key_off + l].float().cpu(), v_ref.float()) <= TOL


def test_expert_pass_with_and_without_the_fold():
    """A whole sample of the tiny policy (expert width 128, three steps), folded against the norm-kernel
    form: the action chunks agree to the rounding-point difference, far inside the chunk tolerance."""
    from make_golden import tiny_inputs
    from tybok_b200 import ops
    from tybok_b200.pi05 import PI05Model
    from tybok_b200.shapes import PI05_TINY
    from tybok_b200.weights import quantize_hot_linears, random_pi05_params

    params = quantize_hot_linears(random_pi05_params(PI05_TINY, seed=0), PI05_TINY)
    model = PI05Model(params, PI05_TINY, device="cuda", vision_dtype=torch.float32)
    assert model.fold is not None
    images, img_masks, tokens, masks, noise = tiny_inputs(PI05_TINY, seed=5)
    noise = torch.randn(noise.shape, generator=torch.Generator().manual_seed(4))
    args = ([t.cuda() for t in images], [t.cuda() for t in img_masks], tokens.cuda(), masks.cuda(), noise.cuda())
    n0 = ops.launch_count()
    a_fold = model.sample_actions(*args).clone()
    n1 = ops.launch_count()
    fold, model.fold = model.fold, None
    a_plain = model.sample_actions(*args).clone()
    n2 = ops.launch_count()
    model.fold = fold
    ops.check_status()
    layers, steps = PI05_TINY.expert.depth, PI05_TINY.steps
    assert (n2 - n1) - (n1 - n0) == steps * (2 * layers - 1)  # every norm launch of a pass but its first
    assert torch.isfinite(a_fold).all()
    assert float((a_fold - a_plain).abs().max()) <= 1e-2
    assert w8_ref.rel_l2(a_fold.cpu(), a_plain.cpu()) <= 5e-3
