"""A fastWAM-class DiT block and denoiser on the fp8 kernels; the FFN optionally tensor-parallel.

``DiTBlock`` is ``FastWAMAttentionBlock.forward`` (tybok/policies/fastwam/models/dit_block.py:328-400):
modulated self-attention (packed q/k/v projection, full-row RMS qk-norm, pair-wise rotary
embedding, attention over ``[earlier keys ; own]``, gated residual), masked cross-attention over a
cached context (affine LayerNorm, q projection + qk-norm, attention, residual) and the FFN tail.
``DiTDenoiser`` stacks the blocks, runs the denoise loop over token space and offers the runner
contract of the reference's fused action tier (``run_action_layers``,
tybok/policies/fastwam/models/fused_action.py:318-357).

FFN tail: ``out = x + gate * down(gelu_tanh(up(modulate(LayerNorm(x), shift, scale))))`` with biases
(dit_block.py:67-69,197-201,392-397).  Three launches: LayerNorm+modulate -> planes, up GEMM with
bias+GELU epilogue -> planes of the hidden activation (no bf16 round trip), down GEMM with bias +
gate + residual epilogue.

Tensor parallel form (the only collective in this package): ``up`` is split by output rows,
``down`` by input columns; every rank produces a partial ``[M, H]`` bf16, one NCCL all-reduce
sums them, and bias / gate / residual are applied after the reduce on every rank.
"""

from __future__ import annotations

import torch

from . import ops
from .shapes import DiTShape
from .weights import quantize_w8

SHIFT_IN = 4
SHIFT_HIDDEN = 4
SHIFT_ATTN = 6  # attention outputs are convex combinations of value rows
#: From this many token rows the GEMMs fed by a norm take two e4m3 planes with a per-row scale.
TWO_PLANE_MIN_TOKENS = 128


def _ln_planes(x, shift, scale, eps):
    """modulate(LayerNorm(x)) as GEMM input: ``(planes, row_scale)`` (two-plane form) or
    ``(planes, None)`` (three planes at SHIFT_IN)."""
    if x.shape[0] >= TWO_PLANE_MIN_TOKENS:
        return ops.norm_planes2(x, ops.NORM_LN_MODULATE, shift, scale, eps=eps)
    return ops.layernorm_modulate(x, shift, scale, eps=eps, out_shift=SHIFT_IN)[1], None


def _gemm(xp, rs, w8, sc, bias=None, **kw):
    """The W8 linear on either activation form."""
    if rs is not None:
        return ops.w8x2_gemm(xp, rs, w8, sc, bias, **kw)
    return ops.w8x3_linear(xp, SHIFT_IN, w8, sc, bias, **kw)


def _as_w8(w: torch.Tensor, scale: torch.Tensor | None):
    """(e4m3 weight, fp32 scale) as stored, or quantised with the reference recipe."""
    if w.dtype == torch.float8_e4m3fn:
        if scale is None:
            raise TypeError("an e4m3 weight needs its per-output-channel scale")
        return w.contiguous(), scale.float().contiguous()
    return quantize_w8(w)


def shard_ffn(up_w, up_b, down_w, down_b, rank: int = 0, world: int = 1, up_scale=None, down_scale=None):
    """Quantise the two FFN matrices with the reference recipe (or take them as stored when they are
    e4m3 with ``up_scale`` / ``down_scale``) and cut this rank's shard.

    ``down`` is quantised as a whole first: its per-output-channel scale is the absmax over the
    full input dimension, so a column shard keeps exactly the e4m3 codes and scales of the
    single-GPU weight (the sum over ranks then equals the unsharded product).  ``up`` is sharded by
    output rows, whose codes and scales do not depend on the other rows."""
    f = up_w.shape[0]
    if f % (world * 128) != 0:
        raise ValueError(f"ffn dim {f} must be a multiple of 128 * world ({world})")
    lo, hi = rank * f // world, (rank + 1) * f // world
    up8, up_s = _as_w8(up_w[lo:hi], None if up_scale is None else up_scale[lo:hi])
    down8, down_s = _as_w8(down_w, down_scale)
    down8 = down8.view(torch.uint8)[:, lo:hi].contiguous().view(torch.float8_e4m3fn)
    return (up8, up_s, up_b[lo:hi].to(torch.bfloat16).contiguous()), (down8, down_s, down_b.to(torch.bfloat16).contiguous())


def finish_after_reduce(x: torch.Tensor, summed: torch.Tensor, down_bias: torch.Tensor, gate: torch.Tensor) -> torch.Tensor:
    """bias, gate and residual after the all-reduce, with the reference's bf16 rounding points."""
    return x + gate * (summed + down_bias)


class DiTFFN:
    """One block's FFN tail on this rank's weight shard."""

    def __init__(self, up_w, up_b, down_w, down_b, device="cuda", rank: int = 0, world: int = 1, group=None,
                 eps: float = 1e-6, up_scale=None, down_scale=None):
        if not str(device).startswith("cuda"):
            raise RuntimeError("tybok_b200 has no CPU path: DiTFFN needs a CUDA (sm_100) device")
        dv = lambda t: None if t is None else t.to(device)  # noqa: E731
        up, down = shard_ffn(up_w.to(device), up_b.to(device), down_w.to(device), down_b.to(device), rank, world,
                             dv(up_scale), dv(down_scale))
        self.up, self.down = up, down
        self.world, self.group, self.eps = world, group, eps

    def partial(self, x: torch.Tensor, shift: torch.Tensor, scale: torch.Tensor) -> torch.Tensor:
        """This rank's un-biased contribution ``[M, H]`` bf16 to ``down(gelu(up(...)))``."""
        xp, rs = _ln_planes(x, shift, scale, self.eps)
        _, hp = _gemm(xp, rs, *self.up, epilogue=ops.EPI_GELU, out_bf16=False, out_planes=True, out_shift=SHIFT_HIDDEN)
        y, _ = ops.w8x3_linear(hp, SHIFT_HIDDEN, self.down[0], self.down[1])
        return y

    def __call__(self, x: torch.Tensor, shift: torch.Tensor, scale: torch.Tensor, gate: torch.Tensor) -> torch.Tensor:
        """``x [M, H]`` bf16; ``shift``/``scale``/``gate`` bf16 ``[H]``."""
        m = x.shape[0]
        if self.world == 1:
            xp, rs = _ln_planes(x, shift, scale, self.eps)
            _, hp = _gemm(xp, rs, *self.up, epilogue=ops.EPI_GELU, out_bf16=False, out_planes=True, out_shift=SHIFT_HIDDEN)
            y, _ = ops.w8x3_linear(hp, SHIFT_HIDDEN, *self.down, epilogue=ops.EPI_RESIDUAL, residual=x,
                                   gate=gate.reshape(1, -1), rows_per_gate=m)
            return y
        import torch.distributed as dist

        part = self.partial(x, shift, scale)
        dist.all_reduce(part, group=self.group)
        return finish_after_reduce(x, part, self.down[2], gate)


class DiTBlock:
    """One ``FastWAMAttentionBlock`` (dit_block.py:178-400) on this rank: attention replicated, FFN on
    this rank's shard.  ``params`` uses the reference's parameter paths (``self_attn.q.weight`` ...
    ``ffn.2.bias``, ``modulation``); the ten matrices may be bf16 (quantised here) or e4m3 with
    ``<lin>.scale_weight`` companions (taken as stored)."""

    def __init__(self, params: dict, shape: DiTShape, device="cuda", rank: int = 0, world: int = 1, group=None,
                 eps: float = 1e-6):
        if not str(device).startswith("cuda"):
            raise RuntimeError("tybok_b200 has no CPU path: DiTBlock needs a CUDA (sm_100) device")
        if shape.head_dim not in (128, 256):
            raise ValueError(f"DiTBlock: head_dim must be 128 or 256, got {shape.head_dim}")
        self.shape, self.eps, self.device = shape, eps, torch.device(device)
        self.heads, self.hd = shape.heads, shape.head_dim
        self.attn_dim = shape.heads * shape.head_dim
        dev = self.device
        g = lambda n: params[n].to(dev)  # noqa: E731

        def lin(name):
            sc = params.get(f"{name}.scale_weight")
            w8, sc = _as_w8(g(f"{name}.weight"), None if sc is None else sc.to(dev))
            return w8, sc, g(f"{name}.bias").to(torch.bfloat16).contiguous()

        def packed(names):
            parts = [lin(n) for n in names]
            return (torch.cat([p[0].view(torch.uint8) for p in parts]).contiguous().view(torch.float8_e4m3fn),
                    torch.cat([p[1] for p in parts]).contiguous(), torch.cat([p[2] for p in parts]).contiguous())

        bf = lambda n: g(n).to(torch.bfloat16).contiguous()  # noqa: E731
        self.qkv = packed(["self_attn.q", "self_attn.k", "self_attn.v"])  # one [3A, H] projection
        self.o = lin("self_attn.o")
        self.cross_q = lin("cross_attn.q")
        self.cross_kv = packed(["cross_attn.k", "cross_attn.v"])
        self.cross_o = lin("cross_attn.o")
        self.norm_q, self.norm_k = bf("self_attn.norm_q.weight"), bf("self_attn.norm_k.weight")
        self.cross_norm_q, self.cross_norm_k = bf("cross_attn.norm_q.weight"), bf("cross_attn.norm_k.weight")
        self.norm3 = (bf("norm3.weight"), bf("norm3.bias"))
        self.modulation = bf("modulation").reshape(6, shape.hidden)
        self.ffn = DiTFFN(g("ffn.0.weight"), g("ffn.0.bias"), g("ffn.2.weight"), g("ffn.2.bias"), device=device, rank=rank,
                          world=world, group=group, eps=eps, up_scale=params.get("ffn.0.scale_weight"),
                          down_scale=params.get("ffn.2.scale_weight"))

    def modulations(self, t_mod: torch.Tensor) -> torch.Tensor:
        """``modulation + t_mod`` -> six contiguous bf16 rows ``[6, H]``: shift / scale / gate of the
        attention half, then of the FFN half (``split_modulation``, dit_block.py:216-231)."""
        return (self.modulation + t_mod.reshape(6, -1).to(torch.bfloat16)).contiguous()

    def context_cache(self, context: torch.Tensor, lcap: int | None = None):
        """Cross-attention keys (qk-normed) and values of a context ``[C, H]`` bf16 as head-major
        caches ``[1, heads, Lcap, D]``: constant across denoise steps, so computed once
        (``precompute_action_context``; dit_block.py:255-266)."""
        c = context.shape[0]
        cp = ops.split3(context.to(torch.bfloat16).contiguous(), SHIFT_IN)
        kv, _ = ops.w8x3_linear(cp, SHIFT_IN, *self.cross_kv)
        mk = lambda: torch.zeros(1, self.heads, lcap or c, self.hd, dtype=torch.bfloat16, device=self.device)  # noqa: E731
        kc, vc = mk(), mk()
        ops.qknorm_rope_store(kv, k_off=0, v_off=self.attn_dim, norm_k=self.cross_norm_k, eps=self.eps, k_cache=kc,
                              v_cache=vc, heads=self.heads, head_dim=self.hd)
        return kc, vc

    def store_context_kv(self, k: torch.Tensor, v: torch.Tensor):
        """Head-major caches from finished cross keys / values ``[1, C, heads*D]`` (qk-norm applied),
        the form the reference's runner is handed (fused_action.py:325-326)."""
        c = k.shape[-2]
        tr = lambda t: t.reshape(c, self.heads, self.hd).transpose(0, 1).to(torch.bfloat16).contiguous()[None]  # noqa: E731
        return tr(k), tr(v)

    def forward(self, x: torch.Tensor, mods: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, self_cache, key_off: int = 0,
                cross_cache=None, ctx_valid: torch.Tensor | None = None) -> torch.Tensor:
        """``x [S, H]`` bf16 (one sequence) -> ``[S, H]``.  ``mods [6, H]`` from ``modulations``;
        ``cos`` / ``sin`` fp32 ``[S, D/2]`` (the complex rotary table's parts); ``self_cache`` =
        ``(K, V)`` ``[1, heads, Lcap, D]`` whose first ``key_off`` rows hold earlier keys / values
        (this block's own are appended there); ``cross_cache`` from ``context_cache`` with
        ``ctx_valid`` uint8 ``[1, C]`` (``None`` skips the cross-attention, dit_block.py:385-390)."""
        s = x.shape[0]
        a, hd = self.attn_dim, self.hd
        hp, rs = _ln_planes(x, mods[0], mods[1], self.eps)
        qkv, _ = _gemm(hp, rs, *self.qkv)
        q = ops.qknorm_rope_store(qkv, q_off=0, k_off=a, v_off=2 * a, norm_q=self.norm_q, norm_k=self.norm_k, eps=self.eps,
                                  cos=cos, sin=sin, k_cache=self_cache[0], v_cache=self_cache[1], heads=self.heads,
                                  head_dim=hd, key_off=key_off)
        _, ap = ops.attention(q, self_cache[0], self_cache[1], None, tokens=s, keys=key_off + s, scale=hd**-0.5,
                              out_bf16=False, out_planes=True, out_shift=SHIFT_ATTN)
        x, _ = ops.w8x3_linear(ap, SHIFT_ATTN, *self.o, epilogue=ops.EPI_RESIDUAL, residual=x, gate=mods[2:3],
                               rows_per_gate=s)
        if cross_cache is not None:
            if s >= TWO_PLANE_MIN_TOKENS:
                cp, rs = ops.norm_planes2(x, ops.NORM_LN_AFFINE, *self.norm3, eps=self.eps)
            else:
                cp, rs = ops.layernorm_affine(x, *self.norm3, eps=self.eps, out_shift=SHIFT_IN)[1], None
            qc, _ = _gemm(cp, rs, *self.cross_q)
            qc = ops.qknorm_rope_store(qc, q_off=0, norm_q=self.cross_norm_q, eps=self.eps, heads=self.heads, head_dim=hd)
            lc = ctx_valid.shape[1] if ctx_valid is not None else cross_cache[0].shape[2]
            _, cap = ops.attention(qc, cross_cache[0], cross_cache[1], ctx_valid, tokens=s, keys=lc, scale=hd**-0.5,
                                   out_bf16=False, out_planes=True, out_shift=SHIFT_ATTN)
            x, _ = ops.w8x3_linear(cap, SHIFT_ATTN, *self.cross_o, epilogue=ops.EPI_RESIDUAL, residual=x)
        return self.ffn(x, mods[3], mods[4], mods[5])


def rotary_parts(freqs: torch.Tensor, device) -> tuple[torch.Tensor, torch.Tensor]:
    """Complex rotary table ``[S, 1, d/2]`` (or ``[S, d/2]``) -> fp32 ``(cos, sin)`` ``[S, d/2]``."""
    f = freqs.reshape(freqs.shape[0], -1).to(torch.complex64)
    return f.real.float().contiguous().to(device), f.imag.float().contiguous().to(device)


class DiTDenoiser:
    """A stack of ``DiTBlock`` s with the denoise loop and the fused-runner contract."""

    def __init__(self, block_params: list[dict], shape: DiTShape, device="cuda", rank: int = 0, world: int = 1, group=None):
        self.shape, self.device = shape, torch.device(device)
        self.blocks = [DiTBlock(p, shape, device=device, rank=rank, world=world, group=group) for p in block_params]
        self._self_cache = None
        self._cross = None
        self._ctx_valid = None

    def _cache(self, rows: int):
        c = self._self_cache
        if c is None or c[0].shape[2] < rows:
            mk = lambda: torch.zeros(1, self.shape.heads, rows, self.shape.head_dim, dtype=torch.bfloat16,  # noqa: E731
                                     device=self.device)
            self._self_cache = c = (mk(), mk())
        return c

    def prepare_context(self, context: torch.Tensor, context_mask: torch.Tensor | None) -> None:
        """Per-block cross-attention caches of ``context [C, H]`` and the key mask ``[C]`` (bool)."""
        self._cross = [b.context_cache(context) for b in self.blocks]
        self._ctx_valid = None if context_mask is None else context_mask.reshape(1, -1).to(self.device, torch.uint8).contiguous()

    @torch.no_grad()
    def step(self, x: torch.Tensor, t_mod: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
        """All blocks on ``x [S, H]`` for one modulation table ``t_mod [6, H]``.  Every block's own
        keys / values are consumed inside the block, so one cache pair serves the whole stack."""
        cache = self._cache(x.shape[0])
        for i, blk in enumerate(self.blocks):
            x = blk.forward(x, blk.modulations(t_mod), cos, sin, cache, 0, None if self._cross is None else self._cross[i],
                            self._ctx_valid)
        return x

    @torch.no_grad()
    def denoise(self, x: torch.Tensor, t_mods: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, deltas) -> torch.Tensor:
        """``len(deltas)`` denoise steps over token space: ``x <- x + stack(x, t_mods[s]) * delta_s``
        in bf16 (the scheduler's update, tybok/policies/fastwam/models/fastwam.py:68-73)."""
        for s, delta in enumerate(deltas):
            x = x + self.step(x, t_mods[s], cos, sin) * torch.tensor(float(delta), dtype=x.dtype, device=x.device)
        return x

    @torch.no_grad()
    def run_action_layers(self, tokens: torch.Tensor, t_mod: torch.Tensor, freqs: torch.Tensor, video_kv: list[dict],
                          cross_kv: list[tuple], context_mask: torch.Tensor) -> torch.Tensor:
        """The reference runner's contract (fused_action.py:318-357): ``tokens [1, M, H]`` bf16,
        ``t_mod [1, 6, H]``, ``freqs`` complex ``[M, 1, d/2]``, per layer ``video_kv[i] = {"k", "v"}``
        ``[1, L_video, heads*D]`` (keys / values every action token also attends to) and
        ``cross_kv[i] = (k, v)`` ``[1, C, heads*D]`` with qk-norm applied, ``context_mask`` bool ``[C]``
        -> ``[1, M, H]``.  The caller's tensors are copied once per call into head-major caches."""
        n = len(self.blocks)
        if len(video_kv) != n or len(cross_kv) != n:
            raise ValueError(f"video/cross KV layer counts {len(video_kv)}/{len(cross_kv)} != {n}")
        if tokens.dtype != torch.bfloat16 or not tokens.is_cuda or tokens.dim() != 3 or tokens.shape[0] != 1:
            raise ValueError("tokens must be bf16 CUDA [1, M, H]")
        if context_mask.numel() != cross_kv[0][0].shape[-2]:
            raise ValueError("context mask length != context KV row count")
        x = tokens[0].contiguous()
        m = x.shape[0]
        cos, sin = rotary_parts(freqs, self.device)
        valid = context_mask.reshape(1, -1).to(self.device, torch.uint8).contiguous()
        for i, blk in enumerate(self.blocks):
            lv = video_kv[i]["k"].shape[-2]
            kc, vc = blk.store_context_kv(video_kv[i]["k"], video_kv[i]["v"])  # [1, heads, Lv, D]
            pad = torch.zeros(1, blk.heads, m, blk.hd, dtype=torch.bfloat16, device=self.device)
            cache = (torch.cat([kc, pad], dim=2).contiguous(), torch.cat([vc, pad], dim=2).contiguous())
            cross = blk.store_context_kv(*cross_kv[i])
            x = blk.forward(x, blk.modulations(t_mod), cos, sin, cache, lv, cross, valid)
        return x[None]
