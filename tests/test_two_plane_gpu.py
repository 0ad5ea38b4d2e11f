"""The two-plane activation form: a norm kernel writes two e4m3 planes of ``y * 2**k(row)`` plus
``row_scale = 2**-k(row)`` and the W8 GEMM consumes them.  Checked here: the planes reproduce the
bf16 norm output exactly (within the documented window), the exponent puts the row maximum into
(224, 448], and the GEMMs on that form match the oracle's W8A16 linear / gated FFN / q-k-v
projection with RoPE within rel-L2 <= 1e-2, on planes built independently in torch."""

import pytest
import torch

from oracle import w8_ref
from tybok_b200.shapes import W8_SWEEP_NK

pytestmark = pytest.mark.gpu
TOL = 1e-2


def torch_planes2(x: torch.Tensor):
    """The decomposition restated in torch: per-row exponent, ``hi = rn_e4m3(x')``, ``lo = rn_e4m3(x' - hi)``."""
    xf = x.float()
    amax = xf.abs().amax(dim=1, keepdim=True)
    e = torch.floor(torch.log2(amax.clamp_min(1e-30)))
    f = amax / torch.exp2(e)
    k = torch.where(amax > 0, 8 - e - (f > 1.75).float(), torch.zeros_like(e))
    xs = xf * torch.exp2(k)
    hi = xs.to(torch.float8_e4m3fn)
    lo = (xs - hi.float()).to(torch.float8_e4m3fn)
    planes = torch.stack([hi.view(torch.uint8), lo.view(torch.uint8)]).contiguous()
    return planes, torch.exp2(-k).reshape(-1).contiguous()


@pytest.mark.parametrize("mode", ["rms", "adarms", "ln_modulate", "ln_affine"])
@pytest.mark.parametrize("m,w", [(544, 2048), (130, 1024), (200, 3072), (9, 264)])
def test_norm_planes2_reproduce_the_bf16_norm(mode, m, w):
    from tybok_b200 import ops

    g = torch.Generator().manual_seed(m + w)
    x = (torch.empty(m, w).normal_(0, 2, generator=g) * torch.exp(torch.empty(m, 1).normal_(0, 2, generator=g))).to(torch.bfloat16)
    x[3 % m, 5] = 300.0  # an outlier row
    xd = x.cuda()
    if mode == "rms":
        wt = torch.empty(w).normal_(0, 0.3, generator=g).cuda()
        y, _ = ops.rmsnorm(xd, weight=wt, out_bf16=True, out_planes=False)
        planes, rs = ops.norm_planes2(xd, ops.NORM_RMS, wt)
    elif mode == "adarms":
        mod = torch.empty(1, 3 * w).normal_(0, 0.3, generator=g).cuda()
        y, _ = ops.rmsnorm(xd, mod=mod, rows_per_group=m, out_bf16=True, out_planes=False)
        planes, rs = ops.norm_planes2(xd, ops.NORM_ADARMS, mod, rows_per_group=m)
    elif mode == "ln_modulate":
        sh, sc = (torch.empty(w).normal_(0, 0.5, generator=g).to(torch.bfloat16).cuda() for _ in range(2))
        y, _ = ops.layernorm_modulate(xd, sh, sc, out_bf16=True, out_planes=False)
        planes, rs = ops.norm_planes2(xd, ops.NORM_LN_MODULATE, sh, sc)
    else:
        wt, b = (torch.empty(w).normal_(1, 0.3, generator=g).to(torch.bfloat16).cuda() for _ in range(2))
        y, _ = ops.layernorm_affine(xd, wt, b, out_bf16=True, out_planes=False)
        planes, rs = ops.norm_planes2(xd, ops.NORM_LN_AFFINE, wt, b)
    torch.cuda.synchronize()
    y, planes, rs = y.cpu().float(), planes.cpu(), rs.cpu()
    assert planes.shape == (2, m, w) and rs.shape == (m,)
    scaled = planes.view(torch.float8_e4m3fn).float().sum(0)
    amax = y.abs().amax(dim=1)
    top = amax / rs  # the row maximum in scaled units
    assert bool(((top > 224) & (top <= 448) | (amax == 0)).all())
    assert bool((torch.log2(rs) == torch.log2(rs).round()).all())  # exact powers of two
    got = scaled * rs[:, None]
    inside = (y.abs() / rs[:, None]) >= 0.25
    assert torch.equal(got[inside], y[inside])
    assert float(((got - y).abs() / amax.clamp_min(1e-30)[:, None]).max()) <= 2.0**-10 / 224
    # the same planes as the torch restatement of the decomposition
    ref_planes, ref_rs = torch_planes2(y.to(torch.bfloat16))
    assert torch.equal(ref_rs, rs) and torch.equal(ref_planes, planes)


def _case(seed, m, n, k, bias=False):
    g = torch.Generator().manual_seed(seed)
    w8, scale = w8_ref.quantize_w8(torch.empty(n, k).normal_(0, 0.02, generator=g))
    x = (torch.empty(m, k).normal_(0, 1, generator=g) * torch.exp(torch.empty(m, 1).normal_(0, 1, generator=g))).to(torch.bfloat16)
    b = torch.empty(n).normal_(0, 0.5, generator=g).to(torch.bfloat16) if bias else None
    return x, w8, scale, b


@pytest.mark.parametrize("n,k", W8_SWEEP_NK)
@pytest.mark.parametrize("m", [1, 50, 256, 800])
def test_w8x2_linear_sweep_matches_oracle(m, n, k):
    from tybok_b200 import ops

    x, w8, scale, _ = _case(m + n, m, n, k)
    planes, rs = torch_planes2(x)
    y, _ = ops.w8x2_gemm(planes.cuda(), rs.cuda(), w8.cuda(), scale.cuda())
    ops.check_status()
    assert w8_ref.rel_l2(y.cpu(), w8_ref.w8_linear(x, w8, scale)) <= TOL
    y2, _ = ops.w8x2_gemm(planes.cuda(), rs.cuda(), w8.cuda(), scale.cuda())
    assert torch.equal(y, y2)  # bit-reproducible


@pytest.mark.parametrize("m,n,k,tile", [(544, 2560, 2048, 0), (130, 384, 320, 0), (300, 1024, 1024, 64), (4146, 512, 256, 0),
                                        (200, 256, 512, 256)])
def test_w8x2_epilogues(m, n, k, tile):
    """Bias, GELU, gated residual and three-plane output on the two-plane form, incl. a multi-wave
    grid (CTA pairs) and a forced token tile beyond the merged-UMMA limit."""
    from tybok_b200 import ops

    x, w8, scale, bias = _case(7 + m, m, n, k, bias=True)
    g = torch.Generator().manual_seed(m)
    res = torch.empty(m, n).normal_(0, 1, generator=g).to(torch.bfloat16)
    gate = torch.empty(1, n).normal_(0, 1, generator=g).to(torch.bfloat16)
    planes, rs = torch_planes2(x)
    pd, rd, wd, sd, bd = planes.cuda(), rs.cuda(), w8.cuda(), scale.cuda(), bias.cuda()
    lin = w8_ref.w8_linear(x, w8, scale, bias)
    y0, _ = ops.w8x2_gemm(pd, rd, wd, sd, bd, token_tile=tile)
    y1, yp = ops.w8x2_gemm(pd, rd, wd, sd, bd, epilogue=ops.EPI_GELU, out_bf16=True, out_planes=True, out_shift=4,
                           token_tile=tile)
    y2, _ = ops.w8x2_gemm(pd, rd, wd, sd, bd, epilogue=ops.EPI_RESIDUAL, residual=res.cuda(), gate=gate.cuda(),
                          rows_per_gate=m, token_tile=tile)
    ops.check_status()
    assert w8_ref.rel_l2(y0.cpu(), lin) <= TOL
    assert w8_ref.rel_l2(y1.cpu(), w8_ref.gelu_tanh(lin)) <= TOL
    assert w8_ref.rel_l2(y2.cpu(), res + lin * gate) <= TOL
    got, want = yp.cpu().view(torch.float8_e5m2).float().sum(0), y1.cpu().float() * 16.0
    inside = want.abs() >= 2.0**-7
    assert torch.equal(got[inside], want[inside])
    # against the three-plane kernel on the same activations: fp32 summation order only
    y3, _ = ops.w8x3_linear(ops.split3(x.cuda(), 4), 4, wd, sd, bd)
    assert w8_ref.rel_l2(y0.cpu(), y3.cpu()) <= 2e-3


@pytest.mark.parametrize("m,i,k", [(544, 1024, 512), (200, 192, 320), (4146, 256, 256)])
def test_w8x2_geglu_packed(m, i, k):
    from tybok_b200 import ops

    g = torch.Generator().manual_seed(i + k)
    gate = w8_ref.quantize_w8(torch.empty(i, k).normal_(0, 0.02, generator=g))
    up = w8_ref.quantize_w8(torch.empty(i, k).normal_(0, 0.02, generator=g))
    x = torch.empty(m, k).normal_(0, 1, generator=g).to(torch.bfloat16)
    ref = w8_ref.gelu_tanh(w8_ref.w8_linear(x, *gate)) * w8_ref.w8_linear(x, *up)
    packed = ops.pack_gate_up(gate[0].cuda(), gate[1].cuda(), up[0].cuda(), up[1].cuda())
    planes, rs = torch_planes2(x)
    h, hp = ops.w8x2_gemm(planes.cuda(), rs.cuda(), *packed, epilogue=ops.EPI_GEGLU_PACKED, out_bf16=True,
                          out_planes=True, out_shift=4)
    ops.check_status()
    assert h.shape == (m, i) and hp.shape == (3, m, i)
    assert w8_ref.rel_l2(h.cpu(), ref) <= 6e-3


@pytest.mark.parametrize("b,l,h,g,k,key_off,d", [(1, 544, 8, 1, 512, 0, 256), (2, 130, 2, 1, 256, 38, 128)])
def test_w8x2_qkv_rope_matches_the_three_plane_form(b, l, h, g, k, key_off, d):
    from tybok_b200 import ops

    dev = torch.device("cuda")
    gen = torch.Generator().manual_seed(5)
    w8, sc = w8_ref.quantize_w8(torch.empty((h + 2 * g) * d, k).normal_(0, 0.02, generator=gen))
    x = torch.empty(b * l, k).normal_(0, 1, generator=gen).to(torch.bfloat16)
    pos = (torch.arange(l, dtype=torch.int32)[None] + torch.tensor([[3], [11]], dtype=torch.int32)[:b]).reshape(-1).to(dev)
    cos, sin = w8_ref.rope_cos_sin(torch.arange(1024)[None], d, torch.bfloat16)
    cos, sin = cos[0].contiguous().to(dev), sin[0].contiguous().to(dev)
    lcap = key_off + l + 3
    caches = [torch.zeros(b, g, lcap, d, dtype=torch.bfloat16, device=dev) for _ in range(4)]
    wp, sp = ops.pair_qkv_rows(w8.to(dev), sc.to(dev), d)
    q3 = ops.w8x3_qkv_rope(ops.split3(x.to(dev), 4), 4, wp, sp, pos, cos, sin, caches[0], caches[1], heads=h, key_off=key_off)
    planes, rs = torch_planes2(x)
    q2 = ops.w8x2_qkv_rope(planes.to(dev), rs.to(dev), wp, sp, pos, cos, sin, caches[2], caches[3], heads=h, key_off=key_off)
    ops.check_status()
    assert w8_ref.rel_l2(q2.float().cpu(), q3.float().cpu()) <= 2e-3
    assert w8_ref.rel_l2(caches[2].float().cpu(), caches[0].float().cpu()) <= 2e-3
    assert w8_ref.rel_l2(caches[3].float().cpu(), caches[1].float().cpu()) <= 2e-3
