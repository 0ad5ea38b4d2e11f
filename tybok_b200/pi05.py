"""pi0.5-shaped policy on the B200 kernels: VLM prefix prefill + action-expert Euler loop.

Structure follows the reference's eager path (tybok/policies/pi05/models/flow_matching.py:761-838,
505-556; gemma.py:61-125; layers.py:268-308) with these substitutions on the hot path:

* every decoder linear is an e4m3 weight with per-channel fp32 scale run by the W8 GEMM of
  this package (q/k/v are packed into one weight, as the reference's ``--tl-llm-flash-attn``
  tier does, layers.py:207-214);
* the RMS / AdaRMS norms write the GEMM's activation planes directly; gate/up/GELU/multiply is
  one kernel that writes the planes of the FFN intermediate, so the down projection reads it
  without a bf16 round trip; residual adds (and AdaRMS gates) are GEMM epilogues;
* per-step constants (time embedding -> AdaRMS conditioning -> per-layer modulations) are
  precomputed once, exactly as the reference's graph path does (flow_matching.py:321-407).

The SigLIP tower, the projector, the embedding lookup and the fp32 action/time projections
are not part of the fp8 path; they run as torch ops.
"""

from __future__ import annotations

import math

import torch
import torch.nn.functional as F  # noqa: N812

from . import ops
from .shapes import GemmaSpec, PI05Shape
from .weights import EXPERT, PROJECTOR, VISION, VLM, quantize_w8

#: Exponent shifts of the activation planes per producer (planes hold value * 2**shift and are
#: exact for |value * 2**shift| in [2**-7, 57344]).
SHIFT_NORMED = 4  # RMS-normalised activations, O(1)
SHIFT_ATTN = 6  # attention outputs (convex combinations of V rows)
SHIFT_FFN = 4  # gelu(gate) * up
SHIFT_FOLD = 0  # residual stream times (1 + scale), not normalised: exact from 2^-7 to 57344
#: From this many token rows a GEMM fed by a norm takes its activations as two e4m3 planes with a
#: per-row power-of-two scale (a third less tensor work, token tiles to 128); below it the GEMMs are
#: bound by launch latency and keep the three-plane form.
TWO_PLANE_MIN_TOKENS = 128


class _Layer:
    """Packed weights of one Gemma decoder layer."""

    __slots__ = ("qkv_paired", "o", "gate", "up", "gate_up", "down", "norm_in", "norm_post")


def _q(params: dict, name: str, device) -> tuple[torch.Tensor, torch.Tensor]:
    """(e4m3 weight, fp32 scale) of ``name``: taken as stored when the checkpoint is fp8
    (``<name>.scale_weight`` present), quantised with the reference recipe otherwise."""
    w = params[f"{name}.weight"]
    if w.dtype == torch.float8_e4m3fn:
        return w.to(device).contiguous(), params[f"{name}.scale_weight"].to(device).float().contiguous()
    w8, s = quantize_w8(w.to(device))
    return w8, s


def _pack_decoder(params: dict, root: str, spec: GemmaSpec, adarms: bool, device) -> list[_Layer]:
    layers = []
    for i in range(spec.depth):
        base = f"{root}.layers.{i}"
        lay = _Layer()
        q, k, v = (_q(params, f"{base}.self_attn.{n}_proj", device) for n in ("q", "k", "v"))
        qkv8 = torch.cat([q[0].view(torch.uint8), k[0].view(torch.uint8), v[0].view(torch.uint8)]).contiguous()
        # RoPE runs in the projection's epilogue, on rows paired with their rotate-half partners
        lay.qkv_paired = ops.pair_qkv_rows(qkv8.view(torch.float8_e4m3fn), torch.cat([q[1], k[1], v[1]]).contiguous(),
                                           spec.head_dim)
        lay.o = _q(params, f"{base}.self_attn.o_proj", device)
        gate = _q(params, f"{base}.mlp.gate_proj", device)
        up = _q(params, f"{base}.mlp.up_proj", device)
        if gate[0].shape[0] % 64 == 0:  # one interleaved matrix: a single weight tile per K block
            lay.gate_up, lay.gate, lay.up = ops.pack_gate_up(*gate, *up), None, None
        else:
            lay.gate_up, lay.gate, lay.up = None, gate, up
        lay.down = _q(params, f"{base}.mlp.down_proj", device)
        if adarms:
            lay.norm_in = (params[f"{base}.input_layernorm.dense.weight"].to(device).float(),
                           params[f"{base}.input_layernorm.dense.bias"].to(device).float())
            lay.norm_post = (params[f"{base}.post_attention_layernorm.dense.weight"].to(device).float(),
                             params[f"{base}.post_attention_layernorm.dense.bias"].to(device).float())
        else:
            lay.norm_in = params[f"{base}.input_layernorm.weight"].to(device).float().contiguous()
            lay.norm_post = params[f"{base}.post_attention_layernorm.weight"].to(device).float().contiguous()
        layers.append(lay)
    return layers


def _rope_table(head_dim: int, max_pos: int, device) -> tuple[torch.Tensor, torch.Tensor]:
    """cos/sin ``[max_pos, D]`` in bf16 from bf16-rounded inverse frequencies
    (tybok/policies/pi05/models/rope.py:24-46,55-64)."""
    inv = 1.0 / (10000.0 ** (torch.arange(0, head_dim, 2, dtype=torch.int64).float() / head_dim))
    inv = inv.to(torch.bfloat16).float().to(device)
    freqs = torch.arange(max_pos, dtype=torch.float32, device=device)[:, None] * inv[None, :]
    emb = torch.cat((freqs, freqs), dim=-1)
    return emb.cos().to(torch.bfloat16), emb.sin().to(torch.bfloat16)


class PI05Model:
    """Weights + forward of a pi0.5-shaped policy on one GPU (inference only)."""

    def __init__(self, params: dict[str, torch.Tensor], shape: PI05Shape, device: str = "cuda",
                 vision_dtype: torch.dtype = torch.bfloat16, overlap: bool = False, vision_tf32: bool = False):
        if not str(device).startswith("cuda"):
            raise RuntimeError("tybok_b200 has no CPU path: PI05Model needs a CUDA (sm_100) device")
        hd = shape.vlm.head_dim
        if hd not in (128, 256) or shape.expert.head_dim != hd:
            raise ValueError(f"PI05Model: both decoder stacks need the same head_dim, 128 or 256 (the sizes the "
                             f"attention kernels are built for); got {hd} and {shape.expert.head_dim}")
        if shape.vlm.num_kv_heads != shape.expert.num_kv_heads:
            raise ValueError("PI05Model: prefix and expert must have the same number of KV heads (shared caches)")
        self.shape = shape
        #: run the first denoise step layer by layer behind the prefix, on a second stream
        #: (flow_matching.py:609-720: expert layer l only needs the prefix keys of layer l)
        self.overlap = bool(overlap)
        self._side = None
        self.device = torch.device(device)
        dev = self.device
        self.vision_dtype = vision_dtype
        #: fp32 tower with TF32 tensor-core GEMMs (10-bit mantissa operands, fp32 accumulation): the
        #: prefix embeddings then agree with an fp32 tower to ~2e-3 rel-L2 where a bf16 tower is at 1.4e-2
        self.vision_tf32 = bool(vision_tf32) and vision_dtype == torch.float32
        self.vision = {k: v.to(dev, vision_dtype) for k, v in params.items() if k.startswith(VISION)}
        # the 7-kernel-per-layer form: bf16 or fp16 operands, or fp32 with TF32 GEMMs; plain fp32 keeps the
        # unfused torch chain.  fp16 carries 11 significant bits like TF32 (the tower's weights need them, see
        # vision_tf32) at the speed of bf16, with the residual stream in fp32 either way; its exponent range
        # (65504) is the price, so a checkpoint with larger sublayer outputs should run the TF32 form.
        self.vis_layers = self._pack_vision() if (vision_dtype in (torch.bfloat16, torch.float16) or self.vision_tf32) else None
        self.pos_embed_f32 = params[f"{VISION}.embeddings.position_embedding.weight"].to(dev).float()
        self.proj_w = params[f"{PROJECTOR}.weight"].to(dev, vision_dtype)
        self.proj_b = params[f"{PROJECTOR}.bias"].to(dev, vision_dtype)
        self.embed = params[f"{VLM}.embed_tokens.weight"].to(dev)
        self.embed_scale = torch.tensor(shape.vlm.width**0.5, dtype=self.embed.dtype, device=dev)
        self.vlm_layers = _pack_decoder(params, VLM, shape.vlm, False, dev)
        self.exp_layers = _pack_decoder(params, EXPERT, shape.expert, True, dev)
        self.final_norm = (params[f"{EXPERT}.norm.dense.weight"].to(dev).float(),
                           params[f"{EXPERT}.norm.dense.bias"].to(dev).float())
        f32 = lambda n: params[n].to(dev).float()  # noqa: E731
        self.action_in = (f32("action_in_proj.weight"), f32("action_in_proj.bias"))
        self.action_out = (f32("action_out_proj.weight"), f32("action_out_proj.bias"))
        self.time_in = (f32("time_mlp_in.weight"), f32("time_mlp_in.bias"))
        self.time_out = (f32("time_mlp_out.weight"), f32("time_mlp_out.bias"))
        self.cos, self.sin = _rope_table(shape.vlm.head_dim, shape.prefix_len + shape.chunk + 8, dev)
        self._cache_by_batch: dict[int, list] = {}
        self._precompute_step_constants()

    # ------------------------------------------------------------------ constants
    def _adarms_cond(self, times: torch.Tensor) -> torch.Tensor:
        """AdaRMS conditioning ``silu(time_mlp_out(silu(time_mlp_in(temb(t)))))`` ``[n, W]`` fp32 for
        flow times ``[n]`` (fp64 sinusoid cast to fp32; flow_matching.py:153-168,376-381)."""
        s = self.shape
        w = s.expert.width
        frac = torch.linspace(0.0, 1.0, w // 2, dtype=torch.float64)
        period = s.min_period * (s.max_period / s.min_period) ** frac
        ang = (1.0 / period * 2 * math.pi)[None, :] * times.to(torch.float32)[:, None]
        temb = torch.cat([torch.sin(ang), torch.cos(ang)], dim=1).float().to(self.device)
        return F.silu(F.linear(F.silu(F.linear(temb, *self.time_in)), *self.time_out))

    def _layer_mods(self, cond_row: torch.Tensor):
        """Per-layer ``(in [1,3W], post [1,3W])`` modulations and the final norm's ``[1,3W]`` for one
        conditioning row ``[1, W]``."""
        mods = [(F.linear(cond_row, *lay.norm_in).contiguous(), F.linear(cond_row, *lay.norm_post).contiguous())
                for lay in self.exp_layers]
        return mods, F.linear(cond_row, *self.final_norm).contiguous()

    def _precompute_step_constants(self) -> None:
        """Per-step AdaRMS modulations ``dense(cond)`` for every expert norm:
        ``mods[step][layer] = (in [1,3W], post [1,3W])`` and the final norm's ``[1,3W]``
        (tybok/policies/pi05/models/flow_matching.py:321-407)."""
        s = self.shape
        dt = -1.0 / s.steps
        cond = self._adarms_cond(torch.tensor([1.0 + i * dt for i in range(s.steps)], dtype=torch.float32))
        self.mods, self.final_mods = [], []
        for i in range(s.steps):
            mods, final = self._layer_mods(cond[i : i + 1])
            self.mods.append(mods)
            self.final_mods.append(final)
        # W * shift of both norms of every layer and step, for the form that folds the AdaRMS norm
        # into the GEMMs around it: fold[step][layer] = (bias of the paired qkv rows, bias of the packed gate/up rows).
        self.fold = None
        w = s.expert.width
        if w % 128 == 0 and all(lay.gate_up is not None for lay in self.exp_layers):
            per_layer = []
            for li, lay in enumerate(self.exp_layers):
                sh_in = torch.stack([self.mods[i][li][0][0, w : 2 * w] for i in range(s.steps)])    # [steps, W]
                sh_post = torch.stack([self.mods[i][li][1][0, w : 2 * w] for i in range(s.steps)])
                per_layer.append((self._shift_bias(lay.qkv_paired, sh_in), self._shift_bias(lay.gate_up, sh_post)))
            self.fold = [[(bq[i].contiguous(), bg[i].contiguous()) for bq, bg in per_layer] for i in range(s.steps)]

    @staticmethod
    def _shift_bias(w8_scale, shifts: torch.Tensor) -> torch.Tensor:
        """``[steps, rows]`` fp32: dequantised weight rows times each step's shift row."""
        w8, scale = w8_scale
        return (shifts.float() @ w8.view(torch.float8_e4m3fn).float().t()) * scale.reshape(1, -1).float()

    # ------------------------------------------------------------------ non-fp8 front end
    def _pack_vision(self):
        """Per-layer tensors of the bf16 tower in the form ``_embed_image_fused`` uses: q/k/v as one
        projection, fc1 transposed for the bias+GELU GEMM epilogue."""
        p, layers = self.vision, []
        for i in range(self.shape.vision.layers):
            base = f"{VISION}.encoder.layers.{i}"
            g = lambda n: p[f"{base}.{n}"]  # noqa: E731
            layers.append({
                "ln1": (g("layer_norm1.weight").contiguous(), g("layer_norm1.bias").contiguous()),
                "qkv_w": torch.cat([g(f"self_attn.{n}_proj.weight") for n in "qkv"]).contiguous(),
                "qkv_b": torch.cat([g(f"self_attn.{n}_proj.bias") for n in "qkv"]).contiguous(),
                "o": (g("self_attn.out_proj.weight"), g("self_attn.out_proj.bias")),
                "ln2": (g("layer_norm2.weight").contiguous(), g("layer_norm2.bias").contiguous()),
                "fc1_wt": g("mlp.fc1.weight").t(), "fc1_b": g("mlp.fc1.bias"),
                "fc2": (g("mlp.fc2.weight"), g("mlp.fc2.bias")),
            })
        return layers

    def _embed_image_fused(self, image: torch.Tensor) -> torch.Tensor:
        """The tower with 7 kernels per encoder layer instead of 14: each residual add runs inside
        the LayerNorm kernel that follows it, q/k/v are one GEMM, GELU is the epilogue of fc1 (same
        layer math as ``embed_image``; vision.py:200-289).  bf16 or fp16 operands, or fp32 activations
        with TF32 GEMMs; the residual stream is fp32 in every form."""
        v, p, dt = self.shape.vision, self.vision, self.vision_dtype
        # Patch embedding as a GEMM over flattened patches (the stride == kernel convolution of
        # vision.py; cuDNN runs it as an fp32 direct convolution that takes longer than 20 layers' GEMMs).
        b, side = image.shape[0], v.image // v.patch
        patches = image.to(dt).view(b, 3, side, v.patch, side, v.patch).permute(0, 2, 4, 1, 3, 5)
        patches = patches.reshape(b, side * side, 3 * v.patch * v.patch)
        wp = p[f"{VISION}.embeddings.patch_embedding.weight"]
        x = F.linear(patches, wp.view(wp.shape[0], -1), p[f"{VISION}.embeddings.patch_embedding.bias"])
        # The residual stream is fp32 whatever the GEMM precision (the LayerNorm kernel adds the bf16
        # sublayer output to it): a stream rounded to bf16 after each of the 54 adds is where a bf16
        # tower loses most of its accuracy, and the fp32 stream costs a few bytes per element.
        x = x.float() + self.pos_embed_f32[None]
        b, l, hid = x.shape
        hd = hid // v.heads
        y = None
        for lay in self.vis_layers:
            x, h = ops.add_layernorm(x, y, *lay["ln1"])
            # attention itself always runs on bf16 operands (the flash kernel; an fp32 tower would take
            # a three times slower one): what it rounds is per-token noise that the 256-token averages
            # after it wash out, unlike a rounded weight, which errs the same way for every token
            qkv = F.linear(h, lay["qkv_w"], lay["qkv_b"])
            if qkv.dtype == torch.float32:
                qkv = qkv.to(torch.bfloat16)
            qkv = qkv.view(b, l, 3, v.heads, hd)
            q, k, val = (qkv[:, :, j].transpose(1, 2) for j in range(3))
            a = F.scaled_dot_product_attention(q, k, val, scale=hd**-0.5).transpose(1, 2).reshape(b, l, hid)
            y = F.linear(a.to(dt), *lay["o"])
            x, h = ops.add_layernorm(x, y, *lay["ln2"])
            h = torch._addmm_activation(lay["fc1_b"], h.view(b * l, hid), lay["fc1_wt"], use_gelu=True)  # tanh GELU
            y = F.linear(h, *lay["fc2"]).view(b, l, hid)
        _, h = ops.add_layernorm(x, y, p[f"{VISION}.post_layernorm.weight"].contiguous(),
                                 p[f"{VISION}.post_layernorm.bias"].contiguous())
        return F.linear(h, self.proj_w, self.proj_b)

    def embed_image(self, image: torch.Tensor) -> torch.Tensor:
        """SigLIP tower + projector (tybok/policies/pi05/models/vision.py:200-289); plain torch ops
        unless the tower is bf16."""
        if self.vis_layers is not None:
            if not self.vision_tf32:
                return self._embed_image_fused(image)
            prev = torch.backends.cuda.matmul.allow_tf32
            torch.backends.cuda.matmul.allow_tf32 = True
            try:
                return self._embed_image_fused(image)
            finally:
                torch.backends.cuda.matmul.allow_tf32 = prev
        v, p, dt = self.shape.vision, self.vision, self.vision_dtype
        x = F.conv2d(image.to(dt), p[f"{VISION}.embeddings.patch_embedding.weight"],
                     p[f"{VISION}.embeddings.patch_embedding.bias"], stride=v.patch)
        x = x.flatten(2).transpose(1, 2) + p[f"{VISION}.embeddings.position_embedding.weight"][None]
        b, l, hid = x.shape
        hd = hid // v.heads
        for i in range(v.layers):
            base = f"{VISION}.encoder.layers.{i}"
            h = F.layer_norm(x, (hid,), p[f"{base}.layer_norm1.weight"], p[f"{base}.layer_norm1.bias"], 1e-6)
            q = F.linear(h, p[f"{base}.self_attn.q_proj.weight"], p[f"{base}.self_attn.q_proj.bias"])
            k = F.linear(h, p[f"{base}.self_attn.k_proj.weight"], p[f"{base}.self_attn.k_proj.bias"])
            val = F.linear(h, p[f"{base}.self_attn.v_proj.weight"], p[f"{base}.self_attn.v_proj.bias"])
            q, k, val = (t.view(b, l, v.heads, hd).transpose(1, 2) for t in (q, k, val))
            a = F.scaled_dot_product_attention(q, k, val, scale=hd**-0.5).transpose(1, 2).reshape(b, l, hid)
            x = x + F.linear(a, p[f"{base}.self_attn.out_proj.weight"], p[f"{base}.self_attn.out_proj.bias"])
            h = F.layer_norm(x, (hid,), p[f"{base}.layer_norm2.weight"], p[f"{base}.layer_norm2.bias"], 1e-6)
            h = F.gelu(F.linear(h, p[f"{base}.mlp.fc1.weight"], p[f"{base}.mlp.fc1.bias"]), approximate="tanh")
            x = x + F.linear(h, p[f"{base}.mlp.fc2.weight"], p[f"{base}.mlp.fc2.bias"])
        x = F.layer_norm(x, (hid,), p[f"{VISION}.post_layernorm.weight"], p[f"{VISION}.post_layernorm.bias"], 1e-6)
        return F.linear(x, self.proj_w, self.proj_b)

    def embed_prefix(self, images, img_masks, tokens, masks) -> tuple[torch.Tensor, torch.Tensor]:
        """Prefix embeddings ``[B, L, W]`` bf16 and pad mask ``[B, L]`` bool
        (flow_matching.py:410-461; paligemma_with_expert.py:134-161)."""
        embs, pads = [], []
        # all cameras in one tower pass: [n_cams*B, 3, H, W]
        feats = self.embed_image(torch.cat(list(images), dim=0)).to(torch.bfloat16)
        b = tokens.shape[0]
        for i, m in enumerate(img_masks):
            e = feats[i * b : (i + 1) * b]
            embs.append(e)
            pads.append(m[:, None].expand(b, e.shape[1]))
        embs.append(F.embedding(tokens, self.embed) * self.embed_scale)
        pads.append(masks.bool())
        return torch.cat(embs, dim=1), torch.cat(pads, dim=1)

    # ------------------------------------------------------------------ decoder pieces
    def _caches(self, b: int):
        """Per-layer K/V caches ``[B, G, prefix_len + chunk, D]`` (zero-initialised once per batch
        size): the prefill writes keys [0, Lp), every expert layer-step rewrites [Lp, Lp + L)."""
        c = self._cache_by_batch.get(b)
        if c is None:
            s = self.shape
            lcap = s.prefix_len + s.chunk
            mk = lambda: torch.zeros(b, s.vlm.num_kv_heads, lcap, s.vlm.head_dim, dtype=torch.bfloat16,  # noqa: E731
                                     device=self.device)
            c = [(mk(), mk()) for _ in range(s.vlm.depth)]
            self._cache_by_batch[b] = c
        return c

    def _layer(self, spec, lay: _Layer, x, b, l, pos, cache, key_off, key_valid, mods):
        """One decoder layer on ``x [B*L, W]`` bf16 (layers.py:268-308). ``mods`` is None for the
        VLM (plain norms) or ``(mod_in, mod_post)`` ``[1, 3W]`` AdaRMS modulations.  ``cache`` is
        this layer's ``(K, V)`` cache; the layer appends its keys at ``key_off``."""
        w = spec.width
        m = x.shape[0]
        two = m >= TWO_PLANE_MIN_TOKENS and lay.gate_up is not None
        gate_in = gate_post = None
        if mods is not None:
            gate_in, gate_post = mods[0][:, 2 * w :], mods[1][:, 2 * w :]

        def norm(which):
            """This layer's input (0) or post-attention (1) norm -> the activation form the next GEMM takes."""
            if two:
                if mods is None:
                    return ops.norm_planes2(x, ops.NORM_RMS, lay.norm_in if which == 0 else lay.norm_post)
                return ops.norm_planes2(x, ops.NORM_ADARMS, mods[which], rows_per_group=m)
            if mods is None:
                return ops.rmsnorm(x, weight=lay.norm_in if which == 0 else lay.norm_post, out_shift=SHIFT_NORMED)[1], None
            return ops.rmsnorm(x, mod=mods[which], rows_per_group=m, out_shift=SHIFT_NORMED)[1], None

        xp, rs = norm(0)
        if two:
            q = ops.w8x2_qkv_rope(xp, rs, *lay.qkv_paired, pos, self.cos, self.sin, cache[0], cache[1],
                                  heads=spec.num_heads, key_off=key_off)
        else:
            q = ops.w8x3_qkv_rope(xp, SHIFT_NORMED, *lay.qkv_paired, pos, self.cos, self.sin, cache[0], cache[1],
                                  heads=spec.num_heads, key_off=key_off)
        _, ap = ops.attention(q, cache[0], cache[1], key_valid, tokens=l, keys=key_off + l,
                              scale=spec.head_dim**-0.5, out_bf16=False, out_planes=True, out_shift=SHIFT_ATTN)
        x, _ = ops.w8x3_linear(ap, SHIFT_ATTN, *lay.o, epilogue=ops.EPI_RESIDUAL, residual=x, gate=gate_in,
                               rows_per_gate=m)
        xp, rs = norm(1)
        if two:
            _, hp = ops.w8x2_gemm(xp, rs, *lay.gate_up, epilogue=ops.EPI_GEGLU_PACKED, out_bf16=False, out_planes=True,
                                  out_shift=SHIFT_FFN)
        elif lay.gate_up is not None:
            _, hp = ops.w8x3_geglu_packed(xp, SHIFT_NORMED, *lay.gate_up, out_bf16=False, out_planes=True,
                                          out_shift=SHIFT_FFN)
        else:
            _, hp = ops.w8x3_geglu(xp, SHIFT_NORMED, *lay.gate, *lay.up, out_bf16=False, out_planes=True,
                                   out_shift=SHIFT_FFN)
        x, _ = ops.w8x3_linear(hp, SHIFT_FFN, *lay.down, epilogue=ops.EPI_RESIDUAL, residual=x, gate=gate_post,
                               rows_per_gate=m)
        return x

    def _expert_pass(self, mods, fold, x, b, l, pos, caches, key_off, key_valid, wait=None):
        """All expert layers of one denoise step on the suffix embedding ``x [B*L, W]``; ``wait(i)`` runs
        before layer ``i``.  Below the two-plane threshold, and with the step's ``W shift`` constants at
        hand (``fold``), only the first norm of the pass is a kernel: every later AdaRMS norm is folded
        into the GEMM that writes its input (sums of squares, planes of ``x (1 + scale)``) and the GEMM
        that reads its output (rstd and ``W shift`` in the epilogue)."""
        spec = self.shape.expert
        m, w = x.shape[0], spec.width
        if fold is None or m >= TWO_PLANE_MIN_TOKENS:
            for i, lay in enumerate(self.exp_layers):
                if wait is not None:
                    wait(i)
                x = self._layer(spec, lay, x, b, l, pos, caches[i], key_off, key_valid, mods[i])
            return x
        carry = None  # (u_planes, ss_part) of the residual stream, written by the previous layer's down projection
        last = len(self.exp_layers) - 1
        for i, lay in enumerate(self.exp_layers):
            if wait is not None:
                wait(i)
            mod_in, mod_post = mods[i]
            cache = caches[i]
            if carry is None:
                xp = ops.rmsnorm(x, mod=mod_in, rows_per_group=m, out_shift=SHIFT_NORMED)[1]
                q = ops.w8x3_qkv_rope(xp, SHIFT_NORMED, *lay.qkv_paired, pos, self.cos, self.sin, cache[0], cache[1],
                                      heads=spec.num_heads, key_off=key_off)
            else:
                q = ops.w8x3_qkv_rope_adarms(carry[0], SHIFT_FOLD, carry[1], fold[i][0], *lay.qkv_paired, pos, self.cos,
                                             self.sin, cache[0], cache[1], heads=spec.num_heads, key_off=key_off)
            _, ap = ops.attention(q, cache[0], cache[1], key_valid, tokens=l, keys=key_off + l,
                                  scale=spec.head_dim**-0.5, out_bf16=False, out_planes=True, out_shift=SHIFT_ATTN)
            x, up, part = ops.w8x3_residual_next_adarms(ap, SHIFT_ATTN, *lay.o, x, mod_in[0, 2 * w :], mod_post[0, :w],
                                                        out_shift=SHIFT_FOLD)
            _, hp = ops.w8x3_geglu_packed_adarms(up, SHIFT_FOLD, part, fold[i][1], *lay.gate_up, out_bf16=False,
                                                 out_planes=True, out_shift=SHIFT_FFN)
            if i == last:
                x, _ = ops.w8x3_linear(hp, SHIFT_FFN, *lay.down, epilogue=ops.EPI_RESIDUAL, residual=x,
                                       gate=mod_post[:, 2 * w :], rows_per_gate=m)
            else:
                x, up, part = ops.w8x3_residual_next_adarms(hp, SHIFT_FFN, *lay.down, x, mod_post[0, 2 * w :],
                                                            mods[i + 1][0][0, :w], out_shift=SHIFT_FOLD)
                carry = (up, part)
        return x

    # ------------------------------------------------------------------ prefix + denoise
    def prefill(self, prefix_embs: torch.Tensor, pad: torch.Tensor, layer_done=None):
        """VLM prefix pass filling the per-layer post-RoPE (K, V) caches (gemma.py:61-125,
        use_cache); returns views ``[B, G, Lp, D]`` of the prefix part of every layer's cache."""
        spec = self.shape.vlm
        b, l, w = prefix_embs.shape
        caches = self._caches(b)
        pos = (torch.cumsum(pad, dim=1) - 1).clamp_min(0).to(torch.int32).reshape(-1)
        key_valid = pad.to(torch.uint8).contiguous()
        x = prefix_embs.reshape(b * l, w)
        for lay, cache in zip(self.vlm_layers, caches):
            x = self._layer(spec, lay, x, b, l, pos, cache, 0, key_valid, None)
            if layer_done is not None:
                layer_done()
        return [(kc[:, :, :l], vc[:, :, :l]) for kc, vc in caches]

    @torch.no_grad()
    def velocity_at(self, t: float, x_t: torch.Tensor, pad: torch.Tensor) -> torch.Tensor:
        """One expert pass at an arbitrary flow time ``t`` over the caches the last ``prefill`` wrote
        (the single-step check of the reference's ``validate``, tybok/policies/pi05/engine.py:796-826)."""
        mods, final = self._layer_mods(self._adarms_cond(torch.tensor([float(t)])))
        return self.denoise_step(0, x_t, pad, mods=(mods, final))

    def denoise_step(self, step: int, x_t: torch.Tensor, pad: torch.Tensor, mods=None) -> torch.Tensor:
        """One expert pass over the prefix caches -> velocity ``[B, chunk, A]`` fp32
        (flow_matching.py:505-556).  ``mods`` overrides the precomputed modulations of ``step``."""
        layer_mods, final_mod = mods if mods is not None else (self.mods[step], self.final_mods[step])
        s = self.shape
        spec = s.expert
        b, l = x_t.shape[0], x_t.shape[1]
        lp = pad.shape[1]
        caches = self._caches(b)
        x = F.linear(x_t, *self.action_in).to(torch.bfloat16).reshape(b * l, spec.width)
        allowed = torch.cat([pad, torch.ones(b, l, dtype=torch.bool, device=x.device)], dim=1)  # [B, Lp+L]
        key_valid = allowed.to(torch.uint8).contiguous()
        pos = (pad.sum(dim=-1, keepdim=True) + torch.arange(l, device=x.device)[None, :]).to(torch.int32).reshape(-1)
        fold = self.fold[step] if mods is None and self.fold is not None else None
        x = self._expert_pass(layer_mods, fold, x, b, l, pos, caches, lp, key_valid)
        y, _ = ops.rmsnorm(x, mod=final_mod, rows_per_group=b * l, out_bf16=True, out_planes=False)
        y = y.view(b, l, spec.width)[:, -s.chunk :].float()
        return F.linear(y, *self.action_out)

    def _expert_layers(self, step: int, h: torch.Tensor, b: int, l: int, pad: torch.Tensor, key_valid, pos):
        """All expert layers of one denoise step on the suffix embedding ``h [B*L, W]``."""
        fold = self.fold[step] if self.fold is not None else None
        return self._expert_pass(self.mods[step], fold, h, b, l, pos, self._caches(b), pad.shape[1], key_valid)

    @torch.no_grad()
    def sample_actions(self, images, img_masks, tokens, masks, noise: torch.Tensor) -> torch.Tensor:
        """Prefix prefill + ``steps`` forward-Euler updates from ``noise`` (flow_matching.py:761-838)."""
        s = self.shape
        embs, pad = self.embed_prefix(images, img_masks, tokens, masks)
        dt = -1.0 / s.steps
        b, l = noise.shape[0], noise.shape[1]
        fused_tail = s.max_action_dim == 32 and l == s.chunk and s.expert.width in (128, 256, 512, 1024, 2048)
        if fused_tail and self.overlap:
            return self._sample_actions_overlapped(embs, pad, noise, dt)
        self.prefill(embs, pad)
        if not fused_tail:
            x_t = noise
            for step in range(s.steps):
                x_t = x_t + dt * self.denoise_step(step, x_t, pad)
            return x_t
        # Fused tail: one launch per step does final norm + out-projection + Euler update + the
        # next step's suffix embedding; masks and positions are built once per chunk.
        key_valid, pos = self._suffix_constants(pad, b, l)
        x_t = noise.float().contiguous().clone()
        h = ops.action_tail(None, None, None, None, x_t, dt, *self.action_in)
        for step in range(s.steps):
            x = self._expert_layers(step, h, b, l, pad, key_valid, pos)
            h = ops.action_tail(x, self.final_mods[step], *self.action_out, x_t, dt, *self.action_in,
                                rows_per_group=b * l, embed=step + 1 < s.steps)
        return x_t

    def _suffix_constants(self, pad: torch.Tensor, b: int, l: int):
        lp = pad.shape[1]
        allowed = torch.cat([pad, torch.ones(b, l, dtype=torch.bool, device=pad.device)], dim=1)
        key_valid = allowed.to(torch.uint8).contiguous()
        pos = (pad.sum(dim=-1, keepdim=True) + torch.arange(l, device=pad.device)[None, :]).to(torch.int32).reshape(-1)
        return key_valid, pos

    def _sample_actions_overlapped(self, embs, pad, noise, dt):
        """``sample_actions`` with the first denoise step pipelined behind the prefix: expert layer
        l of step 0 starts as soon as prefix layer l has written its keys and values, on a second
        stream (captured into the same CUDA graph as a fork / join).  Same kernels, same
        arithmetic; the first of the ten expert passes hides inside the prefix window."""
        s = self.shape
        b, l = noise.shape[0], noise.shape[1]
        lp = pad.shape[1]
        main = torch.cuda.current_stream(self.device)
        if self._side is None:
            self._side = torch.cuda.Stream(device=self.device)
        side = self._side
        key_valid, pos = self._suffix_constants(pad, b, l)
        x_t = noise.float().contiguous().clone()
        caches = self._caches(b)
        fork = torch.cuda.Event()
        fork.record(main)
        with torch.cuda.stream(side):
            side.wait_event(fork)
            h = ops.action_tail(None, None, None, None, x_t, dt, *self.action_in)
        done = []

        def layer_done():
            ev = torch.cuda.Event()
            ev.record(main)
            done.append(ev)

        self.prefill(embs, pad, layer_done)
        with torch.cuda.stream(side):
            x = self._expert_pass(self.mods[0], self.fold[0] if self.fold is not None else None, h, b, l, pos, caches,
                                  lp, key_valid, wait=lambda i: side.wait_event(done[i]))
            h = ops.action_tail(x, self.final_mods[0], *self.action_out, x_t, dt, *self.action_in,
                                rows_per_group=b * l, embed=s.steps > 1)
            join = torch.cuda.Event()
            join.record(side)
        main.wait_event(join)
        for t in (h, x_t, key_valid, pos):  # used on both streams: keep the allocator from recycling them early
            t.record_stream(main)
            t.record_stream(side)
        for step in range(1, s.steps):
            x = self._expert_layers(step, h, b, l, pad, key_valid, pos)
            h = ops.action_tail(x, self.final_mods[step], *self.action_out, x_t, dt, *self.action_in,
                                rows_per_group=b * l, embed=step + 1 < s.steps)
        return x_t
