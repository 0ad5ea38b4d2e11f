"""DiT FFN tail (fastWAM-class geometry: hidden 3072, ffn 14336) against the oracle, single
rank and tensor-parallel (ranks emulated on one GPU: each shard's partial is computed in turn and
the partials are summed as the all-reduce would).  Tolerance rel-L2 <= 1e-2."""

import os
import sys

import pytest
import torch

sys.path.insert(0, os.path.join(os.path.dirname(__file__), "golden"))
from make_golden import dit_case  # noqa: E402

from oracle import w8_ref  # noqa: E402

pytestmark = pytest.mark.gpu


def _case(m, h, f, seed=0):
    g = torch.Generator().manual_seed(seed)
    x = torch.empty(m, h).normal_(0, 1, generator=g).to(torch.bfloat16)
    mods = tuple(torch.empty(h).normal_(0, 0.5, generator=g).to(torch.bfloat16) for _ in range(3))
    up = (torch.empty(f, h).normal_(0, 0.02, generator=g), torch.empty(f).normal_(0, 0.1, generator=g).to(torch.bfloat16))
    down = (torch.empty(h, f).normal_(0, 0.02, generator=g), torch.empty(h).normal_(0, 0.1, generator=g).to(torch.bfloat16))
    return x, mods, up, down


def _oracle(x, mods, up, down):
    return w8_ref.dit_ffn_tail(x, *mods, (*w8_ref.quantize_w8(up[0]), up[1]), (*w8_ref.quantize_w8(down[0]), down[1]))


def test_layernorm_modulate_matches_oracle():
    from tybok_b200 import ops

    x, (shift, scale, _), _, _ = _case(37, 3072, 128)
    n = torch.nn.functional.layer_norm(x.float(), (3072,), None, None, 1e-6).type_as(x)
    ref = n * (1 + scale) + shift
    y, yp = ops.layernorm_modulate(x.cuda(), shift.cuda(), scale.cuda(), out_bf16=True, out_planes=True)
    assert w8_ref.rel_l2(y.cpu(), ref) <= 2e-3
    got, want = yp.cpu().view(torch.float8_e5m2).float().sum(0), y.cpu().float() * 16.0
    inside = want.abs() >= 2.0**-7
    assert torch.equal(got[inside], want[inside])


@pytest.mark.parametrize("m,h,f", [(70, 256, 512), (200, 3072, 14336)])
def test_dit_ffn_tail_single_rank(m, h, f):
    from tybok_b200 import ops
    from tybok_b200.dit import DiTFFN

    x, mods, up, down = _case(m, h, f)
    ref = _oracle(x, mods, up, down)
    ffn = DiTFFN(up[0], up[1], down[0], down[1])
    y = ffn(x.cuda(), *(t.cuda() for t in mods))
    ops.check_status()
    assert w8_ref.rel_l2(y.cpu(), ref) <= 1e-2


def test_golden_fixture_case(golden):
    from tybok_b200.dit import DiTFFN

    x, mods, ws = dit_case()
    ffn = DiTFFN(ws[0][0], ws[0][1], ws[1][0], ws[1][1])
    y = ffn(x[0].cuda(), *(t.reshape(-1).cuda() for t in mods))
    assert w8_ref.rel_l2(y.cpu(), golden["dit_ffn"]["y"][0]) <= 1e-2


@pytest.mark.parametrize("world", [2, 4, 8])
def test_dit_ffn_tensor_parallel_emulated(world):
    from tybok_b200.dit import DiTFFN, finish_after_reduce

    m, h, f = 150, 3072, 14336
    x, mods, up, down = _case(m, h, f, seed=world)
    ref = _oracle(x, mods, up, down)
    xd, (shift, scale, gate) = x.cuda(), tuple(t.cuda() for t in mods)
    total = None
    for rank in range(world):
        ffn = DiTFFN(up[0], up[1], down[0], down[1], rank=rank, world=world)
        part = ffn.partial(xd, shift, scale)
        total = part if total is None else total + part  # bf16 sum, as a bf16 all-reduce does
        del ffn
    y = finish_after_reduce(xd, total, down[1].cuda(), gate)
    assert w8_ref.rel_l2(y.cpu(), ref) <= 1e-2
