"""RoPE/KV-store + prefix-cache attention on the GPU against the oracle's eager GQA attention
(tybok/policies/pi05/models/layers.py:145-191, rope.py:19-75).  Tolerance: rel-L2 <= 1e-2."""

import pytest
import torch

from oracle import w8_ref

pytestmark = pytest.mark.gpu
D = 256


def _tables(max_pos, D=D):
    pos = torch.arange(max_pos)[None]
    cos, sin = w8_ref.rope_cos_sin(pos, D, torch.bfloat16)
    return cos[0].contiguous(), sin[0].contiguous()


def _reference(qkv, b, l, h, g, pos, prefix_k, prefix_v, key_valid, D=D):
    """Oracle path: split, RoPE, concat with the prefix cache, eager attention with additive mask."""
    q = qkv[:, : h * D].view(b, l, h, D).transpose(1, 2)
    k = qkv[:, h * D : (h + g) * D].view(b, l, g, D).transpose(1, 2)
    v = qkv[:, (h + g) * D :].view(b, l, g, D).transpose(1, 2)
    cos, sin = w8_ref.rope_cos_sin(pos, D, torch.bfloat16)
    q, k = w8_ref.apply_rope(q, k, cos, sin)
    kk = k if prefix_k is None else torch.cat([prefix_k, k], dim=2)
    vv = v if prefix_v is None else torch.cat([prefix_v, v], dim=2)
    mask = torch.where(key_valid[:, None, None, :].bool(), 0.0, w8_ref.MASK_VALUE).expand(b, 1, l, kk.shape[2])
    return w8_ref.gqa_attention(q, kk, vv, mask, D**-0.5), k, v


_CASES = [(1, 50, 544, 8, 1), (2, 50, 300, 8, 1), (1, 544, 0, 8, 1), (2, 130, 0, 4, 2), (1, 10, 968, 8, 1),
          (1, 7, 5, 2, 2),
          # grids beyond one wave: each CTA works through several key blocks
          (2, 544, 0, 8, 1), (2, 300, 400, 8, 1), (4, 130, 300, 8, 1), (1, 544, 480, 8, 1)]


@pytest.mark.parametrize("b,l,lp,h,g,D", [c + (256,) for c in _CASES] + [
    # head_dim 128 (always the key-loop kernel): short suffixes over a prefix, prefill, MHA, many heads
    (1, 50, 544, 8, 1, 128), (2, 10, 130, 2, 1, 128), (1, 7, 5, 2, 2, 128), (2, 130, 0, 4, 4, 128),
    (1, 544, 480, 8, 1, 128), (1, 300, 0, 24, 24, 128), (3, 70, 129, 6, 6, 128)])
def test_attention_matches_oracle(b, l, lp, h, g, D):
    from tybok_b200 import ops

    gen = torch.Generator().manual_seed(b * 1000 + l + lp)
    qkv = torch.empty(b * l, (h + 2 * g) * D).normal_(0, 1, generator=gen).to(torch.bfloat16)
    lk = lp + l
    key_valid = torch.ones(b, lk, dtype=torch.uint8)
    if lp > 8:
        key_valid[:, lp - 5 : lp] = 0  # padded prefix tail
    elif lp == 0 and l > 20:
        key_valid[:, l - 9 :] = 0  # padded prompt tail during prefill
    pos = (torch.arange(l)[None] + lp).expand(b, l).contiguous()
    prefix_k = prefix_v = None
    if lp:
        prefix_k = torch.empty(b, g, lp, D).normal_(0, 1, generator=gen).to(torch.bfloat16)
        prefix_v = torch.empty(b, g, lp, D).normal_(0, 1, generator=gen).to(torch.bfloat16)
    ref, rk, rv = _reference(qkv, b, l, h, g, pos, prefix_k, prefix_v, key_valid, D)

    lcap = lk + 3
    kc = torch.zeros(b, g, lcap, D, dtype=torch.bfloat16, device="cuda")
    vc = torch.zeros_like(kc)
    if lp:
        kc[:, :, :lp] = prefix_k.cuda()
        vc[:, :, :lp] = prefix_v.cuda()
    cos, sin = _tables(lk + 8, D)
    q = ops.rope_store(qkv.cuda(), pos.reshape(-1).int().cuda(), cos.cuda(), sin.cuda(), kc, vc, heads=h, key_off=lp)
    # RoPE uses the same bf16 operations as torch: the stored keys are bit-identical
    assert torch.equal(kc[:, :, lp:lk].cpu(), rk) and torch.equal(vc[:, :, lp:lk].cpu(), rv)
    out, planes = ops.attention(q, kc, vc, key_valid.cuda(), tokens=l, keys=lk, scale=D**-0.5, out_bf16=True,
                                out_planes=True, out_shift=6)
    ops.check_status()
    out = out.cpu().view(b, l, h * D)
    valid_q = torch.ones(b, l, dtype=torch.bool) if lp else key_valid.bool()
    assert w8_ref.rel_l2(out[valid_q], ref[valid_q]) <= 1e-2
    got, want = planes.cpu().view(torch.float8_e5m2).float().sum(0), out.reshape(b * l, h * D).float() * 64.0
    inside = want.abs() >= 2.0**-7
    assert torch.equal(got[inside], want[inside])
    # bit-reproducible
    out2, _ = ops.attention(q, kc, vc, key_valid.cuda(), tokens=l, keys=lk, scale=D**-0.5)
    assert torch.equal(out2.cpu().view(b, l, h * D), out)


@pytest.mark.parametrize("D", [256, 128])
@pytest.mark.parametrize("pattern", ["rising", "one_late_spike", "masked_first_blocks"])
def test_prefill_attention_rescales_when_the_row_maximum_grows(pattern, D):
    """Long query sequences keep O in tensor memory and move a row's reference maximum only when a
    key block exceeds it by more than 2^8: keys whose scores grow block by block, a single late
    outlier, and leading key blocks without a valid key all take that rescale (against the oracle's
    eager attention evaluated in fp32 on the same bf16 caches, no RoPE; rel-L2 <= 1e-2)."""
    from tybok_b200 import ops

    b, l, h, g, lk = 1, 200, 4, 1, 200
    gen = torch.Generator().manual_seed(11)
    q = torch.empty(b * l, h * D).normal_(0, 1, generator=gen).to(torch.bfloat16)
    k = torch.empty(b, g, lk, D).normal_(0, 1, generator=gen).to(torch.bfloat16)
    v = torch.empty(b, g, lk, D).normal_(0, 1, generator=gen).to(torch.bfloat16)
    key_valid = torch.ones(b, lk, dtype=torch.uint8)
    if pattern == "rising":
        k = (k.float() * (1.0 + 3.0 * (torch.arange(lk) // 64))[None, None, :, None]).to(torch.bfloat16)
    elif pattern == "one_late_spike":
        k[:, :, 170] = (k[:, :, 170].float() * 12.0).to(torch.bfloat16)
    else:
        key_valid[:, :130] = 0
    qh = q.view(b, l, h, D).transpose(1, 2)
    mask = torch.where(key_valid[:, None, None, :].bool(), 0.0, w8_ref.MASK_VALUE).expand(b, 1, l, lk)
    # fp32 logits here: at these magnitudes the oracle's bf16 logits are themselves 1e-1 apart
    ref = w8_ref.gqa_attention(qh.float(), k.float(), v.float(), mask, D**-0.5)
    out, _ = ops.attention(q.cuda(), k.cuda().contiguous(), v.cuda().contiguous(), key_valid.cuda(), tokens=l, keys=lk,
                           scale=D**-0.5)
    ops.check_status()
    out = out.cpu().view(b, l, h * D)
    assert torch.isfinite(out.float()).all()
    assert w8_ref.rel_l2(out.float(), ref) <= 1e-2


@pytest.mark.gpu
@pytest.mark.parametrize("b,l,h,g,k,key_off,d", [(1, 50, 8, 1, 1024, 544, 256), (2, 10, 2, 1, 128, 130, 256),
                                                  (1, 130, 2, 2, 256, 0, 256), (2, 10, 2, 1, 128, 38, 128),
                                                  (1, 130, 3, 3, 256, 0, 128)])
def test_qkv_rope_epilogue_matches_projection_then_rope_store(b, l, h, g, k, key_off, d):
    """The projection with RoPE + KV store as its epilogue writes bit-for-bit what the plain
    projection followed by the rope_store kernel writes (same split count)."""
    from tybok_b200 import ops

    dev = torch.device("cuda")
    gen = torch.Generator().manual_seed(5)
    w = torch.empty((h + 2 * g) * d, k).normal_(0, 0.02, generator=gen)
    w8, sc = w8_ref.quantize_w8(w)
    w8, sc = w8.to(dev), sc.to(dev)
    x = torch.empty(b * l, k).normal_(0, 1, generator=gen).to(torch.bfloat16).to(dev)
    pos = (torch.arange(l, dtype=torch.int32)[None] + torch.tensor([[3], [11]], dtype=torch.int32)[:b]).reshape(-1).to(dev)
    cos, sin = w8_ref.rope_cos_sin(torch.arange(1024)[None], d, torch.bfloat16)
    cos, sin = cos[0].contiguous().to(dev), sin[0].contiguous().to(dev)
    lcap = key_off + l + 3
    caches = [torch.zeros(b, g, lcap, d, dtype=torch.bfloat16, device=dev) for _ in range(4)]
    xp = ops.split3(x, 4)
    qkv, _ = ops.w8x3_linear(xp, 4, w8, sc, splits=1)
    q0 = ops.rope_store(qkv, pos, cos, sin, caches[0], caches[1], heads=h, key_off=key_off)
    wp, sp = ops.pair_qkv_rows(w8, sc, d)
    q1 = ops.w8x3_qkv_rope(xp, 4, wp, sp, pos, cos, sin, caches[2], caches[3], heads=h, key_off=key_off, splits=1)
    q2 = ops.w8x3_qkv_rope(xp, 4, wp, sp, pos, cos, sin, caches[2].clone(), caches[3].clone(), heads=h, key_off=key_off)
    torch.cuda.synchronize()
    ops.check_status()
    assert torch.equal(q0, q1)
    assert torch.equal(caches[0], caches[2]) and torch.equal(caches[1], caches[3])
    assert w8_ref.rel_l2(q2.float().cpu(), q0.float().cpu()) < 2e-3  # other split count: fp32 summation order only


def test_long_self_attention_at_head_dim_128():
    """The DiT self-attention geometry at reduced head count: 4146 queries over 4146 keys (65 key
    blocks per CTA, 33 query tiles), MHA, no mask, fp32-SDPA oracle as the reference's DiT block
    uses it (tybok/policies/fastwam/models/dit_block.py:72-98); rel-L2 <= 1e-2."""
    from tybok_b200 import ops

    b, l, h, d = 1, 4146, 3, 128
    gen = torch.Generator().manual_seed(23)
    q = torch.empty(b * l, h * d).normal_(0, 1, generator=gen).to(torch.bfloat16)
    k = torch.empty(b, h, l, d).normal_(0, 1, generator=gen).to(torch.bfloat16)
    v = torch.empty(b, h, l, d).normal_(0, 1, generator=gen).to(torch.bfloat16)
    ref = torch.nn.functional.scaled_dot_product_attention(q.view(b, l, h, d).transpose(1, 2).float(), k.float(), v.float())
    ref = ref.transpose(1, 2).reshape(b, l, h * d)
    out, _ = ops.attention(q.cuda(), k.cuda(), v.cuda(), None, tokens=l, keys=l, scale=d**-0.5)
    ops.check_status()
    out = out.cpu().view(b, l, h * d)
    assert torch.isfinite(out.float()).all()
    assert w8_ref.rel_l2(out.float(), ref) <= 1e-2


def test_attention_refuses_other_head_sizes():
    from tybok_b200 import _lib, ops

    q = torch.zeros(4, 2 * 64, dtype=torch.bfloat16, device="cuda")
    kc = torch.zeros(1, 2, 8, 64, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(_lib.TybokError, match="head_dim must be 128 or 256"):
        ops.attention(q, kc, kc.clone(), None, tokens=4, keys=4, scale=0.125)
