"""W8A16 linear / gated FFN front half on the GPU against the CPU oracle.

Tolerance: rel-L2 <= 1e-2 on bf16 outputs.  The kernel multiplies the
exact e4m3 weights with the exact bf16 activations and applies the per-channel scale to the
fp32 accumulator; the oracle rounds ``w8*scale`` to bf16 per weight before the GEMM.  That
difference measures ~2.6e-3 rel-L2.
"""

import pytest
import torch

from oracle import w8_ref
from tybok_b200.shapes import W8_SWEEP_M, W8_SWEEP_NK

pytestmark = pytest.mark.gpu
TOL = 1e-2


def _ops():
    from tybok_b200 import ops

    return ops


def _case(seed, m, n, k, bias=False):
    g = torch.Generator().manual_seed(seed)
    w = torch.empty(n, k).normal_(0, 0.02, generator=g)
    x = torch.empty(m, k).normal_(0, 1, generator=g).to(torch.bfloat16)
    b = torch.empty(n).normal_(0, 0.5, generator=g).to(torch.bfloat16) if bias else None
    w8, scale = w8_ref.quantize_w8(w)
    return x, w8, scale, b


def _run(x, w8, scale, b=None, **kw):
    ops = _ops()
    y = ops.w8a16_linear(x.cuda(), w8.cuda(), scale.cuda(), None if b is None else b.cuda(), **kw)
    ops.check_status()
    return y.cpu()


@pytest.mark.parametrize("m,n,k", [(1, 128, 128), (16, 128, 256), (7, 192, 320), (50, 256, 512), (64, 384, 1024),
                                   (130, 256, 384), (300, 128, 2048)])
@pytest.mark.parametrize("splits", [1, 2, 3])
def test_small_shapes(m, n, k, splits):
    x, w8, scale, _ = _case(m * 7 + n, m, n, k)
    ref = w8_ref.w8_linear(x, w8, scale)
    y = _run(x, w8, scale, splits=splits)
    assert w8_ref.rel_l2(y, ref) <= TOL


@pytest.mark.parametrize("bt", [16, 32, 64, 128, 256])
def test_token_tiles(bt):
    x, w8, scale, b = _case(11, 200, 256, 640, bias=True)
    ref = w8_ref.w8_linear(x, w8, scale, b)
    y = _run(x, w8, scale, b, token_tile=bt)
    assert w8_ref.rel_l2(y, ref) <= TOL


def test_exact_on_representable_inputs():
    """Small-integer activations and power-of-two scales make every product and partial sum
    exact in fp32, so the kernel must reproduce the oracle bit for bit: this pins the e4m3
    expansion (all 254 finite codes), the swizzled addressing and the K ordering."""
    n, k, m = 256, 512, 48
    codes = torch.arange(256, dtype=torch.uint8)
    codes = codes[(codes & 0x7F) != 0x7F]  # drop the two NaN encodings
    g = torch.Generator().manual_seed(3)
    w8 = codes[torch.randint(0, len(codes), (n, k), generator=g)].view(torch.float8_e4m3fn)
    scale = torch.full((n,), 2.0**-10)
    x = torch.randint(-2, 3, (m, k), generator=g).to(torch.bfloat16)
    ref = w8_ref.w8_linear(x, w8, scale)
    y = _run(x, w8, scale, splits=2)
    assert torch.equal(y, ref)


@pytest.mark.parametrize("n,k", W8_SWEEP_NK)
@pytest.mark.parametrize("m", W8_SWEEP_M)
def test_baseline_sweep(m, n, k):
    x, w8, scale, _ = _case(0, m, n, k)
    ref = w8_ref.w8_linear(x, w8, scale)
    y = _run(x, w8, scale)
    assert w8_ref.rel_l2(y, ref) <= TOL
    # split-K sums in a fixed order: a second launch is bit-identical
    assert torch.equal(y, _run(x, w8, scale))


def test_gelu_and_bias_epilogue():
    ops = _ops()
    x, w8, scale, b = _case(5, 50, 512, 256, bias=True)
    ref = w8_ref.gelu_tanh(w8_ref.w8_linear(x, w8, scale, b))
    y = _run(x, w8, scale, b, epilogue=ops.EPI_GELU)
    assert w8_ref.rel_l2(y, ref) <= TOL


@pytest.mark.parametrize("gated", [False, True])
@pytest.mark.parametrize("splits", [1, 4])
def test_residual_epilogue(gated, splits):
    ops = _ops()
    batch, rows = 2, 50
    x, w8, scale, _ = _case(6, batch * rows, 256, 1024)
    g = torch.Generator().manual_seed(8)
    res = torch.empty(batch * rows, 256).normal_(0, 1, generator=g).to(torch.bfloat16)
    gate = torch.empty(batch, 256).normal_(0, 1, generator=g) if gated else None
    lin = w8_ref.w8_linear(x, w8, scale)
    if gated:
        gb = gate.to(torch.bfloat16).repeat_interleave(rows, dim=0)
        ref = res + lin * gb
    else:
        ref = res + lin
    y = ops.w8a16_linear(x.cuda(), w8.cuda(), scale.cuda(), epilogue=ops.EPI_RESIDUAL, residual=res.cuda(),
                         gate=None if gate is None else gate.cuda(), rows_per_gate=rows, splits=splits)
    ops.check_status()
    assert w8_ref.rel_l2(y.cpu(), ref) <= TOL


@pytest.mark.parametrize("m,i,k,splits", [(50, 256, 512, 1), (50, 4096, 1024, 0), (544, 1024, 256, 1), (10, 384, 128, 1),
                                          (50, 256, 1024, 4), (50, 256, 2048, 8)])
def test_geglu(m, i, k, splits):
    ops = _ops()
    g = torch.Generator().manual_seed(9)
    x = torch.empty(m, k).normal_(0, 1, generator=g).to(torch.bfloat16)
    gate = w8_ref.quantize_w8(torch.empty(i, k).normal_(0, 0.02, generator=g))
    up = w8_ref.quantize_w8(torch.empty(i, k).normal_(0, 0.02, generator=g))
    ref = w8_ref.gelu_tanh(w8_ref.w8_linear(x, *gate)) * w8_ref.w8_linear(x, *up)
    h = ops.w8a16_geglu(x.cuda(), gate[0].cuda(), gate[1].cuda(), up[0].cuda(), up[1].cuda(), splits=splits)
    ops.check_status()
    assert w8_ref.rel_l2(h.cpu(), ref) <= TOL


def test_split3_planes_are_exact():
    """The three e5m2 planes sum to x * 2**shift exactly inside the documented window."""
    ops = _ops()
    g = torch.Generator().manual_seed(4)
    x = (torch.empty(37, 256).normal_(0, 1, generator=g) * torch.exp(torch.empty(37, 256).normal_(0, 2, generator=g)))
    x = x.clamp(-3000, 3000).to(torch.bfloat16)
    planes = ops.split3(x.cuda(), 4).cpu()
    total = planes.view(torch.float8_e5m2).float().sum(0)
    want = x.float() * 16.0
    inside = want.abs() >= 2.0**-7
    assert torch.equal(total[inside], want[inside])
    assert float((total - want).abs().max()) <= 2.0**-17 + 2.0**-24


def test_planes_in_planes_out_chain():
    """geglu -> planes -> down projection, never materialising the bf16 intermediate:
    the gated FFN of tybok/policies/pi05/models/layers.py:87-95."""
    ops = _ops()
    g = torch.Generator().manual_seed(12)
    m, k, i = 50, 256, 512
    x = torch.empty(m, k).normal_(0, 1, generator=g).to(torch.bfloat16)
    gate, up, down = (w8_ref.quantize_w8(torch.empty(s).normal_(0, 0.02, generator=g)) for s in ((i, k), (i, k), (k, i)))
    ref = w8_ref.gemma_mlp(x, gate, up, down)
    cu = lambda t: tuple(a.cuda() for a in t)  # noqa: E731
    xp = ops.split3(x.cuda(), 4)
    h, hp = ops.w8x3_geglu(xp, 4, *cu(gate), *cu(up), out_bf16=True, out_planes=True, out_shift=6)
    y, _ = ops.w8x3_linear(hp, 6, *cu(down))
    ops.check_status()
    assert w8_ref.rel_l2(y.cpu(), ref) <= TOL
    # the planes hold exactly the bf16 intermediate
    got, want = hp.cpu().view(torch.float8_e5m2).float().sum(0), h.cpu().float() * 64.0
    inside = want.abs() >= 2.0**-7
    assert torch.equal(got[inside], want[inside]) and float((got - want).abs().max()) <= 2.0**-17 + 2.0**-24


@pytest.mark.parametrize("m,k,i", [(50, 1024, 4096), (544, 2048, 16384)])
def test_ffn_chain_at_the_model_shapes(m, k, i):
    """The gated FFN exactly as a decoder layer of the full policy runs it -- packed gate/up GEMM
    writing planes, down projection with the residual epilogue -- at the action-expert shape
    (50 tokens, 1024 -> 4096 -> 1024) and the prefix shape (544 tokens, 2048 -> 16384 -> 2048),
    against ``x + GemmaMLP(x)`` of the oracle (tybok/policies/pi05/models/layers.py:87-95,295-308)."""
    ops = _ops()
    g = torch.Generator().manual_seed(31)
    x = torch.empty(m, k).normal_(0, 1, generator=g).to(torch.bfloat16)
    res = torch.empty(m, k).normal_(0, 1, generator=g).to(torch.bfloat16)
    gate, up, down = (w8_ref.quantize_w8(torch.empty(s).normal_(0, 0.02, generator=g)) for s in ((i, k), (i, k), (k, i)))
    mlp = w8_ref.gemma_mlp(x, gate, up, down)
    ref = res + mlp
    cu = lambda t: tuple(a.cuda() for a in t)  # noqa: E731
    packed = ops.pack_gate_up(*cu(gate), *cu(up))
    xp = ops.split3(x.cuda(), 4)
    _, hp = ops.w8x3_geglu_packed(xp, 4, *packed, out_bf16=False, out_planes=True, out_shift=4)
    y, _ = ops.w8x3_linear(hp, 4, *cu(down), epilogue=ops.EPI_RESIDUAL, residual=res.cuda())
    ops.check_status()
    # the tolerance applies to the FFN output; the residual only changes the last rounding
    assert w8_ref.rel_l2(y.cpu().float() - res.float(), mlp.float()) <= TOL
    assert w8_ref.rel_l2(y.cpu(), ref) <= TOL


def test_c_abi_bf16_entry_point_with_workspace():
    """``tybok_w8a16_linear`` as a C caller sees it: bf16 in, caller-owned workspace."""
    ops = _ops()
    lib = ops._lib.load()
    x, w8, scale, _ = _case(21, 50, 256, 512)
    xd, wd, sd = x.cuda(), w8.cuda(), scale.cuda()
    y = torch.empty(50, 256, dtype=torch.bfloat16, device="cuda")
    need = lib.tybok_w8a16_workspace_bytes(50, 256, 512, 0)
    ws = torch.empty(need, dtype=torch.uint8, device="cuda")
    stream = torch.cuda.current_stream().cuda_stream
    rc = lib.tybok_w8a16_linear(xd.data_ptr(), wd.data_ptr(), sd.data_ptr(), None, y.data_ptr(), 50, 256, 512, 512, 256,
                                0, None, 0, None, 0, 1, 0, 0, 0, ws.data_ptr(), need, None, stream)
    assert rc == 0, lib.tybok_last_error()
    torch.cuda.synchronize()
    assert w8_ref.rel_l2(y.cpu(), w8_ref.w8_linear(x, w8, scale)) <= TOL
    rc = lib.tybok_w8a16_linear(xd.data_ptr(), wd.data_ptr(), sd.data_ptr(), None, y.data_ptr(), 50, 256, 512, 512, 256,
                                0, None, 0, None, 0, 1, 0, 0, 0, ws.data_ptr(), need - 1, None, stream)
    assert rc == 3 and b"workspace" in lib.tybok_last_error()


def test_bad_arguments_raise():
    ops = _ops()
    x, w8, scale, _ = _case(1, 4, 128, 128)
    with pytest.raises(Exception):
        ops.w8a16_linear(x.cuda().float(), w8.cuda(), scale.cuda())
    with pytest.raises(Exception):  # K not a multiple of 16
        ops.w8a16_linear(x.cuda()[:, :120].contiguous(), w8.cuda()[:, :120].contiguous(), scale.cuda())
    with pytest.raises(Exception):  # bad token tile
        ops.w8a16_linear(x.cuda(), w8.cuda(), scale.cuda(), token_tile=24)
    with pytest.raises(NotImplementedError):  # no CPU path
        ops.w8a16_linear(x, w8, scale)


@pytest.mark.gpu
@pytest.mark.parametrize("m,i,k", [(50, 256, 512), (130, 512, 256), (7, 192, 320), (200, 1024, 1024)])
def test_geglu_packed_matches_two_matrix_form(m, i, k):
    """The interleaved gate/up matrix gives the two-matrix kernel's result (same split count ->
    bit-equal; otherwise within the GEMM tolerance) and the oracle's within rel-L2 6e-3."""
    gen = torch.Generator().manual_seed(11)
    wg = torch.empty(i, k).normal_(0, 0.02, generator=gen)
    wu = torch.empty(i, k).normal_(0, 0.02, generator=gen)
    x = torch.empty(m, k).normal_(0, 1, generator=gen).to(torch.bfloat16)
    (g8, gs), (u8, us) = w8_ref.quantize_w8(wg), w8_ref.quantize_w8(wu)
    ref = w8_ref.gelu_tanh(w8_ref.w8_linear(x, g8, gs)) * w8_ref.w8_linear(x, u8, us)
    ops = _ops()
    dev = torch.device("cuda")
    g8, gs, u8, us = (t.to(dev) for t in (g8, gs, u8, us))
    p8, ps = ops.pack_gate_up(g8, gs, u8, us)
    xp = ops.split3(x.to(dev), 4)
    h0, hp0 = ops.w8x3_geglu(xp, 4, g8, gs, u8, us, out_bf16=True, out_planes=True, splits=1)
    h1, hp1 = ops.w8x3_geglu_packed(xp, 4, p8, ps, out_bf16=True, out_planes=True, splits=1)
    h2, _ = ops.w8x3_geglu_packed(xp, 4, p8, ps, out_bf16=True, out_planes=False)
    torch.cuda.synchronize()
    ops.check_status()
    assert torch.equal(h0, h1) and torch.equal(hp0, hp1)
    assert w8_ref.rel_l2(h1.cpu(), ref) < 6e-3
    assert w8_ref.rel_l2(h2.cpu(), ref) < 6e-3


@pytest.mark.gpu
def test_geglu_packed_rejects_ragged_width():
    ops = _ops()
    dev = torch.device("cuda")
    w = torch.zeros(192, 64, dtype=torch.uint8, device=dev).view(torch.float8_e4m3fn)  # 2*I = 192: I = 96
    xp = torch.zeros(3, 4, 64, dtype=torch.uint8, device=dev)
    with pytest.raises(ValueError):
        ops.w8x3_geglu_packed(xp, 4, w, torch.ones(192, device=dev))


@pytest.mark.gpu
@pytest.mark.parametrize("m,n,k", [(544, 8192, 512), (300, 12800, 320), (1200, 2560, 256)])
def test_multi_wave_launches_run_as_cta_pairs(m, n, k):
    """Enough full-K tiles for two waves: the launch takes the CTA-pair form (one UMMA of 256
    weight rows per two CTAs, each loading half of the activation planes).  Same tolerance as the
    single-CTA form, bit-reproducible, and equal to a forced split-K launch up to summation order."""
    ops = _ops()
    x, w8, scale, _ = _case(41, m, n, k)
    ref = w8_ref.w8_linear(x, w8, scale)
    xp = ops.split3(x.cuda(), 4)
    y0, _ = ops.w8x3_linear(xp, 4, w8.cuda(), scale.cuda())
    y1, _ = ops.w8x3_linear(xp, 4, w8.cuda(), scale.cuda())
    y2, _ = ops.w8x3_linear(xp, 4, w8.cuda(), scale.cuda(), splits=2)
    torch.cuda.synchronize()
    ops.check_status()
    assert torch.equal(y0, y1)
    assert w8_ref.rel_l2(y0.cpu(), ref) <= TOL
    assert w8_ref.rel_l2(y0.cpu(), y2.cpu()) <= 2e-3


@pytest.mark.gpu
def test_cta_pair_form_with_paired_and_residual_epilogues():
    """The CTA-pair launch under the packed gate/up epilogue (bit-equal to the two-matrix form,
    which never pairs) and under the gated residual epilogue (against the oracle)."""
    ops = _ops()
    dev = torch.device("cuda")
    gen = torch.Generator().manual_seed(43)
    m, i, k = 544, 4096, 256
    wg, wu = (torch.empty(i, k).normal_(0, 0.02, generator=gen) for _ in range(2))
    x = torch.empty(m, k).normal_(0, 1, generator=gen).to(torch.bfloat16)
    (g8, gs), (u8, us) = w8_ref.quantize_w8(wg), w8_ref.quantize_w8(wu)
    g8, gs, u8, us = (t.to(dev) for t in (g8, gs, u8, us))
    p8, ps = ops.pack_gate_up(g8, gs, u8, us)
    xp = ops.split3(x.to(dev), 4)
    h0, hp0 = ops.w8x3_geglu(xp, 4, g8, gs, u8, us, out_bf16=True, out_planes=True)
    h1, hp1 = ops.w8x3_geglu_packed(xp, 4, p8, ps, out_bf16=True, out_planes=True)
    assert torch.equal(h0, h1) and torch.equal(hp0, hp1)
    # down-projection-like launch with residual and fp32 gate: 544 x 8192 x 256
    w8, sc = w8_ref.quantize_w8(torch.empty(8192, k).normal_(0, 0.02, generator=gen))
    res = torch.empty(m, 8192).normal_(0, 1, generator=gen).to(torch.bfloat16)
    gate = torch.empty(1, 8192).normal_(0, 0.5, generator=gen)
    ref = res + w8_ref.w8_linear(x, w8, sc) * gate.to(torch.bfloat16)
    y, _ = ops.w8x3_linear(xp, 4, w8.to(dev), sc.to(dev), epilogue=ops.EPI_RESIDUAL, residual=res.to(dev),
                           gate=gate.to(dev), rows_per_gate=m)
    torch.cuda.synchronize()
    ops.check_status()
    assert w8_ref.rel_l2(y.cpu(), ref) <= TOL


def test_epilogue_wait_time_out_is_reported_and_the_device_stays_usable():
    """A bounded device wait that runs out ends in an error status, not in a hang or a fault: with
    the epilogue's wait for its accumulator cut to a few hundred SM clocks, a single-CTA launch
    over a long K (its products take far longer than that) gives up, skips its stores and records
    ``TYBOK_DEV_TIMEOUT_EPILOGUE``; the producer drains its copies, the MMA warp sees its products
    retire before the tensor memory is freed, the kernel returns, ``check_status`` raises, and the
    next launch on the device is correct.  (The reference's rule for its cooperative kernels:
    an error, never an exit -- tybok/policies/fastwam/kernels/coop_grid.h:20-27.)"""
    ops = _ops()
    lib = ops._lib.load()
    x, w8, scale, _ = _case(41, 64, 128, 32768)
    xp = ops.split3(x.cuda(), 4)
    w8d, sd = w8.cuda(), scale.cuda()
    ref = w8_ref.w8_linear(x, w8, scale)
    good, _ = ops.w8x3_linear(xp, 4, w8d, sd, token_tile=64, splits=1)
    ops.check_status()
    assert w8_ref.rel_l2(good.cpu(), ref) <= TOL
    torch.cuda.synchronize()
    lib.tybok_debug_set_epilogue_wait_limit(300)
    try:
        ops.w8x3_linear(xp, 4, w8d, sd, token_tile=64, splits=1)
        torch.cuda.synchronize()  # the kernel came back
    finally:
        lib.tybok_debug_set_epilogue_wait_limit(0)
    assert int(ops.status_word(xp.device).item()) == 104  # TYBOK_DEV_TIMEOUT_EPILOGUE
    with pytest.raises(ops._lib.TybokError, match="bounded wait"):
        ops.check_status()
    again, _ = ops.w8x3_linear(xp, 4, w8d, sd, token_tile=64, splits=1)
    ops.check_status()  # the status word was cleared by the raise; this launch reports nothing
    assert torch.equal(again, good)
