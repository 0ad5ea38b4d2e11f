"""The two numerical identities the GPU path rests on, restated in torch on the CPU (no kernel runs here):

* the activation decompositions -- three e5m2 terms with a fixed exponent shift, two e4m3 terms with a
  per-row power-of-two scale -- reproduce bf16 values exactly inside the windows the header documents,
  and bound the error outside them;
* the AdaRMS norm folded into the GEMMs around it, ``W (x r (1 + s) + sh) = r W (x (1 + s)) + W sh``,
  stays within the linear tolerance of the oracle when ``x (1 + s)`` is what gets rounded to bf16."""

import torch

from oracle import w8_ref


def split3_e5m2(x: torch.Tensor, shift: int):
    xs = x.float() * 2.0**shift
    h1 = xs.to(torch.float8_e5m2).float()
    h2 = (xs - h1).to(torch.float8_e5m2).float()
    h3 = (xs - h1 - h2).to(torch.float8_e5m2).float()
    return (h1 + h2 + h3) * 2.0**-shift


def split2_e4m3(x: torch.Tensor):
    xf = x.float()
    amax = xf.abs().amax(dim=1, keepdim=True)
    e = torch.floor(torch.log2(amax))
    k = 8 - e - (amax / torch.exp2(e) > 1.75).float()
    xs = xf * torch.exp2(k)
    g1 = xs.to(torch.float8_e4m3fn).float()
    g2 = (xs - g1).to(torch.float8_e4m3fn).float()
    return (g1 + g2) * torch.exp2(-k), xs, k


def _bf16_rows(rows, width, seed, spread=3.0):
    g = torch.Generator().manual_seed(seed)
    x = torch.empty(rows, width).normal_(0, 1, generator=g) * torch.exp(torch.empty(rows, width).normal_(0, spread, generator=g))
    return x.to(torch.bfloat16)


def test_three_e5m2_terms_are_exact_inside_the_window():
    x = _bf16_rows(64, 512, 0)
    for shift in (0, 4, 6):
        got = split3_e5m2(x, shift)
        mag = x.float().abs() * 2.0**shift
        inside = (mag >= 2.0**-7) & (mag <= 57344.0)
        assert torch.equal(got[inside], x.float()[inside])
        below = mag < 2.0**-7
        assert float(((got - x.float()).abs() * 2.0**shift)[below].max()) <= 2.0**-17 + 2.0**-25


def test_two_e4m3_terms_with_a_row_scale():
    x = _bf16_rows(64, 512, 1)
    got, xs, k = split2_e4m3(x)
    top = xs.abs().amax(dim=1)
    assert bool(((top > 224) & (top <= 448)).all())  # the row maximum sits just under the e4m3 limit
    inside = xs.abs() >= 0.25
    assert torch.equal(got[inside], x.float()[inside])  # eight significant bits from two four-bit terms
    err_scaled = ((got - x.float()) * torch.exp2(k)).abs()
    assert float(err_scaled.max()) <= 2.0**-10  # below the window: absolute, 4e-6 of the row maximum
    assert float((err_scaled / top[:, None]).max()) <= 2.0**-10 / 224


def test_a_linear_on_either_decomposition_matches_the_oracle():
    g = torch.Generator().manual_seed(2)
    x = _bf16_rows(40, 256, 3, spread=1.0)
    w8, scale = w8_ref.quantize_w8(torch.empty(96, 256).normal_(0, 0.03, generator=g))
    ref = w8_ref.w8_linear(x, w8, scale)
    wq = w8.view(torch.float8_e4m3fn).float() if w8.dtype == torch.uint8 else w8.float()
    for planes in (split3_e5m2(x, 4), split2_e4m3(x)[0]):
        y = ((planes.double() @ wq.double().t()) * scale.double()).float().to(torch.bfloat16)
        assert w8_ref.rel_l2(y, ref) <= 1e-2


def test_adarms_norm_folded_into_the_gemms_around_it():
    g = torch.Generator().manual_seed(4)
    m, w, n, eps = 50, 256, 192, 1e-6
    x = (torch.empty(m, w).normal_(0, 1, generator=g) * torch.exp(torch.empty(1, w).normal_(0, 1, generator=g))).to(torch.bfloat16)
    s, sh = torch.empty(w).normal_(0, 0.3, generator=g), torch.empty(w).normal_(0, 0.3, generator=g)
    w8, scale = w8_ref.quantize_w8(torch.empty(n, w).normal_(0, 0.03, generator=g))
    wq = (w8.view(torch.float8_e4m3fn).float() if w8.dtype == torch.uint8 else w8.float())
    r = torch.rsqrt(x.float().pow(2).mean(dim=1, keepdim=True) + eps)
    # the reference order: normalise, modulate, round to bf16, then the W8A16 linear
    y = (x.float() * r * (1.0 + s) + sh).to(torch.bfloat16)
    ref = w8_ref.w8_linear(y, w8, scale)
    # the folded order: round x (1 + s) to bf16, multiply, then the row's rstd and W sh in fp32
    u = (x.float() * (1.0 + s)).to(torch.bfloat16).float()
    bias = (wq @ sh) * scale
    folded = ((u @ wq.t()) * r * scale + bias).to(torch.bfloat16)
    assert w8_ref.rel_l2(folded, ref) <= 1e-2
    assert w8_ref.rel_l2(folded, ref) <= 6e-3  # one bf16 rounding point apart, not a looser computation
