"""The hook-shaped callables (``tybok_b200/hooks.py``) installed on torch modules that have the
attribute layout of the reference's ``GemmaMLP`` and ``FastWAMAttentionBlock``, against the oracle.
Tolerance rel-L2 <= 1e-2."""

import pytest
import torch
from torch import nn

from oracle import w8_ref

pytestmark = pytest.mark.gpu


class _MLP(nn.Module):
    """Attribute layout of tybok/policies/pi05/models/layers.py:87-95."""

    def __init__(self, width, inter):
        super().__init__()
        self.gate_proj, self.up_proj = nn.Linear(width, inter, bias=False), nn.Linear(width, inter, bias=False)
        self.down_proj = nn.Linear(inter, width, bias=False)

    def forward(self, x):
        return self.down_proj(nn.functional.gelu(self.gate_proj(x), approximate="tanh") * self.up_proj(x))


@pytest.mark.parametrize("b,l,w,i", [(2, 25, 256, 512), (1, 130, 1024, 4096)])
def test_mlp_forward_hook(b, l, w, i):
    from tybok_b200.hooks import make_mlp_forward

    torch.manual_seed(3)
    mlp = _MLP(w, i)
    for p in mlp.parameters():
        nn.init.normal_(p, 0, 0.02)
    x = torch.randn(b, l, w).to(torch.bfloat16)
    ref = w8_ref.gemma_mlp(x, *(w8_ref.quantize_w8(m.weight.data) for m in (mlp.gate_proj, mlp.up_proj, mlp.down_proj)))
    mlp.forward = make_mlp_forward(mlp)  # the assignment the reference's engine makes
    y = mlp.forward(x.cuda())
    assert y.shape == x.shape and y.dtype == x.dtype
    assert w8_ref.rel_l2(y.cpu(), ref) <= 1e-2
    with pytest.raises(RuntimeError, match="no CPU path"):
        mlp.forward(x)


def test_mlp_forward_hook_takes_fp8_linears():
    """``FP8Linear``-like modules (e4m3 ``weight`` + ``weight_scale``) are used as stored."""
    from tybok_b200.hooks import make_mlp_forward

    torch.manual_seed(4)
    w, i = 256, 512

    class FP8:
        def __init__(self, n, k):
            self.weight, self.weight_scale = w8_ref.quantize_w8(torch.randn(n, k) * 0.02)

    class M:
        gate_proj, up_proj, down_proj = FP8(i, w), FP8(i, w), FP8(w, i)

    x = torch.randn(1, 50, w).to(torch.bfloat16)
    ref = w8_ref.gemma_mlp(x, *((m.weight, m.weight_scale) for m in (M.gate_proj, M.up_proj, M.down_proj)))
    y = make_mlp_forward(M)(x.cuda())
    assert w8_ref.rel_l2(y.cpu(), ref) <= 1e-2


def test_fused_ffn_tail_hook():
    from tybok_b200.hooks import make_fused_ffn_tail

    torch.manual_seed(5)
    h, f, b, s = 256, 512, 2, 70

    class Blk(nn.Module):
        """Attribute layout of tybok/policies/fastwam/models/dit_block.py:283-326 (FFN part)."""

        def __init__(self):
            super().__init__()
            self.eps = 1e-6
            self.ffn = nn.Sequential(nn.Linear(h, f), nn.GELU(approximate="tanh"), nn.Linear(f, h))
            self._fused_ffn_tail = None

    blk = Blk().to(torch.bfloat16)
    for p in blk.parameters():
        nn.init.normal_(p, 0, 0.05)
    x = torch.randn(b, s, h).to(torch.bfloat16)
    t_mod = (torch.randn(b, 6, h) * 0.5).to(torch.bfloat16)  # strided views of one table, as the reference passes them
    shift, scale, gate = t_mod[:, 3:4], t_mod[:, 4:5], t_mod[:, 5:6]
    up = (*w8_ref.quantize_w8(blk.ffn[0].weight.data), blk.ffn[0].bias.data)
    down = (*w8_ref.quantize_w8(blk.ffn[2].weight.data), blk.ffn[2].bias.data)
    ref = w8_ref.dit_ffn_tail(x, shift, scale, gate, up, down)
    blk._fused_ffn_tail = make_fused_ffn_tail(blk)
    y = blk._fused_ffn_tail(x.cuda(), shift.cuda(), scale.cuda(), gate.cuda())
    assert y.shape == x.shape
    assert w8_ref.rel_l2(y.cpu().float() - x.float(), ref.float() - x.float()) <= 1e-2
    assert w8_ref.rel_l2(y.cpu(), ref) <= 1e-2
