"""FFN tail of a fastWAM-class DiT block on the fp8 kernels, optionally tensor-parallel.

``out = x + gate * down(gelu_tanh(up(modulate(LayerNorm(x), shift, scale))))`` with biases
(tybok/policies/fastwam/models/dit_block.py:67-69,197-201,392-397).  Three launches:
LayerNorm+modulate -> planes, up GEMM with bias+GELU epilogue -> planes of the hidden
activation (no bf16 round trip), down GEMM with bias + gate + residual epilogue.

Tensor parallel form (the only collective in this package): ``up`` is split by output rows,
``down`` by input columns; every rank produces a partial ``[M, H]`` bf16, one NCCL all-reduce
sums them, and bias / gate / residual are applied after the reduce on every rank.
"""

from __future__ import annotations

import torch

from . import ops
from .weights import quantize_w8

SHIFT_IN = 4
SHIFT_HIDDEN = 4


def shard_ffn(up_w, up_b, down_w, down_b, rank: int = 0, world: int = 1):
    """Quantise the two FFN matrices with the reference recipe and cut this rank's shard.

    ``down`` is quantised as a whole first: its per-output-channel scale is the absmax over the
    full input dimension, so a column shard keeps exactly the e4m3 codes and scales of the
    single-GPU weight (the sum over ranks then equals the unsharded product)."""
    f = up_w.shape[0]
    if f % (world * 128) != 0:
        raise ValueError(f"ffn dim {f} must be a multiple of 128 * world ({world})")
    lo, hi = rank * f // world, (rank + 1) * f // world
    up8, up_s = quantize_w8(up_w[lo:hi])
    down8, down_s = quantize_w8(down_w)
    down8 = down8.view(torch.uint8)[:, lo:hi].contiguous().view(torch.float8_e4m3fn)
    return (up8, up_s, up_b[lo:hi].to(torch.bfloat16).contiguous()), (down8, down_s, down_b.to(torch.bfloat16).contiguous())


def finish_after_reduce(x: torch.Tensor, summed: torch.Tensor, down_bias: torch.Tensor, gate: torch.Tensor) -> torch.Tensor:
    """bias, gate and residual after the all-reduce, with the reference's bf16 rounding points."""
    return x + gate * (summed + down_bias)


class DiTFFN:
    """One block's FFN tail on this rank's weight shard."""

    def __init__(self, up_w, up_b, down_w, down_b, device="cuda", rank: int = 0, world: int = 1, group=None,
                 eps: float = 1e-6):
        if not str(device).startswith("cuda"):
            raise RuntimeError("tybok_b200 has no CPU path: DiTFFN needs a CUDA (sm_100) device")
        up, down = shard_ffn(up_w.to(device), up_b.to(device), down_w.to(device), down_b.to(device), rank, world)
        self.up, self.down = up, down
        self.world, self.group, self.eps = world, group, eps

    def partial(self, x: torch.Tensor, shift: torch.Tensor, scale: torch.Tensor) -> torch.Tensor:
        """This rank's un-biased contribution ``[M, H]`` bf16 to ``down(gelu(up(...)))``."""
        _, xp = ops.layernorm_modulate(x, shift, scale, eps=self.eps, out_shift=SHIFT_IN)
        _, hp = ops.w8x3_linear(xp, SHIFT_IN, *self.up, epilogue=ops.EPI_GELU, out_bf16=False, out_planes=True,
                                out_shift=SHIFT_HIDDEN)
        y, _ = ops.w8x3_linear(hp, SHIFT_HIDDEN, self.down[0], self.down[1])
        return y

    def __call__(self, x: torch.Tensor, shift: torch.Tensor, scale: torch.Tensor, gate: torch.Tensor) -> torch.Tensor:
        """``x [M, H]`` bf16; ``shift``/``scale``/``gate`` bf16 ``[H]``."""
        m = x.shape[0]
        if self.world == 1:
            _, xp = ops.layernorm_modulate(x, shift, scale, eps=self.eps, out_shift=SHIFT_IN)
            _, hp = ops.w8x3_linear(xp, SHIFT_IN, *self.up, epilogue=ops.EPI_GELU, out_bf16=False, out_planes=True,
                                    out_shift=SHIFT_HIDDEN)
            y, _ = ops.w8x3_linear(hp, SHIFT_HIDDEN, *self.down, epilogue=ops.EPI_RESIDUAL, residual=x,
                                   gate=gate.reshape(1, -1), rows_per_gate=m)
            return y
        import torch.distributed as dist

        part = self.partial(x, shift, scale)
        dist.all_reduce(part, group=self.group)
        return finish_after_reduce(x, part, self.down[2], gate)
