"""Host logic of the tensor-parallel DiT FFN on two gloo ranks (no GPU): weight sharding, the
all-reduce of the partials and the post-reduce epilogue.  The per-rank partial product is the CPU
oracle's linear here (the product's GEMM needs a GPU); what is under test is that shards + sum +
``finish_after_reduce`` reproduce the unsharded oracle."""

import os
import sys

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def _case():
    g = torch.Generator().manual_seed(0)
    m, h, f = 20, 128, 512
    x = torch.empty(m, h).normal_(0, 1, generator=g).to(torch.bfloat16)
    mods = tuple(torch.empty(h).normal_(0, 0.5, generator=g).to(torch.bfloat16) for _ in range(3))
    up = (torch.empty(f, h).normal_(0, 0.02, generator=g), torch.empty(f).normal_(0, 0.1, generator=g).to(torch.bfloat16))
    down = (torch.empty(h, f).normal_(0, 0.02, generator=g), torch.empty(h).normal_(0, 0.1, generator=g).to(torch.bfloat16))
    return x, mods, up, down


def _worker(rank, world, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from oracle import w8_ref
    from tybok_b200.dit import finish_after_reduce, shard_ffn

    x, (shift, scale, gate), up, down = _case()
    (up8, up_s, up_b), (down8, down_s, down_b) = shard_ffn(up[0], up[1], down[0], down[1], rank, world)
    n = torch.nn.functional.layer_norm(x.float(), (x.shape[-1],), None, None, 1e-6).type_as(x)
    hid = w8_ref.gelu_tanh(w8_ref.w8_linear(n * (1 + scale) + shift, up8, up_s, up_b))
    part = w8_ref.w8_linear(hid, down8, down_s).float()  # gloo has no bf16 sum everywhere: reduce in fp32
    dist.all_reduce(part)
    y = finish_after_reduce(x, part.to(torch.bfloat16), down_b, gate)
    if rank == 0:
        torch.save(y, out)
    dist.destroy_process_group()


def test_two_rank_sharding_reproduces_unsharded_oracle(tmp_path):
    from oracle import w8_ref

    out = str(tmp_path / "y.pt")
    mp.spawn(_worker, args=(2, 29533, out), nprocs=2, join=True)
    x, mods, up, down = _case()
    ref = w8_ref.dit_ffn_tail(x, *mods, (*w8_ref.quantize_w8(up[0]), up[1]), (*w8_ref.quantize_w8(down[0]), down[1]))
    y = torch.load(out)
    assert w8_ref.rel_l2(y, ref) <= 5e-3


def test_shard_keeps_full_row_scales():
    from tybok_b200.dit import shard_ffn
    from tybok_b200.weights import quantize_w8

    _, _, up, down = _case()
    full8, full_s = quantize_w8(down[0])
    cols = []
    for r in range(4):
        _, (d8, ds, _) = shard_ffn(up[0], up[1], down[0], down[1], r, 4)
        assert torch.equal(ds, full_s)
        cols.append(d8.view(torch.uint8))
    assert torch.equal(torch.cat(cols, dim=1), full8.view(torch.uint8))
