"""The pi0.5-shaped policy on the GPU kernels against the CPU oracle (torch dequant path).

Tolerances: final action chunk with zero noise max-abs <= 2e-2; per-kernel outputs rel-L2 <= 1e-2.
Every model here runs the attention kernels of this package (head_dim 128 in the tiny shape,
256 in the small and full ones); no other attention implementation exists on the decoder path.
"""

import os
import sys

import pytest
import torch

sys.path.insert(0, os.path.join(os.path.dirname(__file__), "golden"))
from make_golden import tiny_inputs  # noqa: E402

from oracle import pi05_ref, w8_ref  # noqa: E402
from tybok_b200.shapes import PI05_SMALL, PI05_TINY  # noqa: E402
from tybok_b200.weights import quantize_hot_linears, random_pi05_params  # noqa: E402

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("m,w,ada", [(50, 1024, True), (544, 2048, False), (7, 128, True), (3, 4096, False),
                                     (9, 520, True), (33, 2056, False), (5, 264, True)])  # ragged row widths
def test_rmsnorm_planes_and_bf16(m, w, ada):
    """tybok/policies/pi05/models/layers.py:51-84 on the GPU: bf16 output bit-exact up to one
    bf16 ulp of rounding-order difference, planes exactly equal to the bf16 output."""
    from tybok_b200 import ops

    g = torch.Generator().manual_seed(m + w)
    x = torch.empty(m, w).normal_(0, 2, generator=g).to(torch.bfloat16)
    if ada:
        rows = 25 if m % 25 == 0 else m
        mod = torch.empty(m // rows, 3 * w).normal_(0, 0.3, generator=g)
        ref, _ = w8_ref.adarms_norm(x.view(m // rows, rows, w), mod)
        ref = ref.reshape(m, w)
        y, yp = ops.rmsnorm(x.cuda(), mod=mod.cuda(), rows_per_group=rows, out_bf16=True, out_planes=True, out_shift=4)
    else:
        weight = torch.empty(w).normal_(0, 0.3, generator=g)
        ref = w8_ref.gemma_norm(x, weight)
        y, yp = ops.rmsnorm(x.cuda(), weight=weight.cuda(), out_bf16=True, out_planes=True, out_shift=4)
    y, yp = y.cpu(), yp.cpu()
    assert w8_ref.rel_l2(y, ref) <= 2e-3
    assert float((y.float() - ref.float()).abs().max()) <= 2 * float(ref.float().abs().max()) * 2.0**-8
    got, want = yp.view(torch.float8_e5m2).float().sum(0), y.float() * 16.0
    inside = want.abs() >= 2.0**-7
    assert torch.equal(got[inside], want[inside])


def _tiny_model(shape=PI05_TINY):
    from tybok_b200.pi05 import PI05Model

    params = quantize_hot_linears(random_pi05_params(shape, seed=0), shape)
    return params, PI05Model(params, shape, device="cuda", vision_dtype=torch.float32)


@pytest.mark.parametrize("batch", [1, 3])
def test_small_policy_with_attention_kernel_matches_oracle(batch):
    """head_dim 256 / MQA with a 130-token prefix: the split-key suffix attention and the key-loop
    prefill attention run inside the model."""
    from tybok_b200 import ops

    params, model = _tiny_model(PI05_SMALL)
    images, img_masks, tokens, masks, noise = tiny_inputs(PI05_SMALL, seed=7, batch=batch)
    noise = torch.randn(noise.shape, generator=torch.Generator().manual_seed(1))
    ref = pi05_ref.sample_actions(params, PI05_SMALL, images, img_masks, tokens, masks, noise)
    out = model.sample_actions([t.cuda() for t in images], [t.cuda() for t in img_masks], tokens.cuda(), masks.cuda(),
                               noise.cuda())
    ops.check_status()
    assert float((out.cpu() - ref).abs().max()) <= 2e-2
    assert w8_ref.rel_l2(out.cpu(), ref) <= 1e-2


def test_chunk_does_not_depend_on_programmatic_dependent_launch():
    """Every kernel is launched with programmatic stream serialisation and waits for its
    predecessor itself; with that switched off (plain stream order) the chunk is bit for bit
    the same."""
    from tybok_b200 import _lib, ops

    params, model = _tiny_model(PI05_SMALL)
    images, img_masks, tokens, masks, noise = tiny_inputs(PI05_SMALL, seed=8, batch=2)
    noise = torch.randn(noise.shape, generator=torch.Generator().manual_seed(2))
    args = ([t.cuda() for t in images], [t.cuda() for t in img_masks], tokens.cuda(), masks.cuda(), noise.cuda())
    with_pdl = model.sample_actions(*args).clone()
    lib = _lib.load()
    lib.tybok_set_pdl(0)
    try:
        without = model.sample_actions(*args).clone()
    finally:
        lib.tybok_set_pdl(1)
    ops.check_status()
    assert torch.equal(with_pdl, without)


def test_tiny_policy_chunk_matches_oracle():
    from tybok_b200 import ops

    params, model = _tiny_model()
    images, img_masks, tokens, masks, noise = tiny_inputs(PI05_TINY)
    ref, inter = pi05_ref.sample_actions(params, PI05_TINY, images, img_masks, tokens, masks, noise,
                                         return_intermediates=True)
    cu = lambda ts: [t.cuda() for t in ts]  # noqa: E731
    embs, pad = model.embed_prefix(cu(images), cu(img_masks), tokens.cuda(), masks.cuda())
    assert w8_ref.rel_l2(embs.cpu(), inter["prefix_embs"].to(torch.bfloat16)) <= 1e-2
    kv = model.prefill(embs, pad)
    valid = pad[0].cpu()
    for (k, v), (rk, rv) in zip(kv, inter["kv"]):
        assert w8_ref.rel_l2(k.cpu()[0, :, valid], rk[0, :, valid]) <= 2e-2
        assert w8_ref.rel_l2(v.cpu()[0, :, valid], rv[0, :, valid]) <= 2e-2
    out = model.sample_actions(cu(images), cu(img_masks), tokens.cuda(), masks.cuda(), noise.cuda())
    ops.check_status()
    assert float((out.cpu() - ref).abs().max()) <= 2e-2
    assert w8_ref.rel_l2(out.cpu(), ref) <= 2e-2


def test_tiny_policy_batch2_and_graph_replay():
    """Batched requests equal the oracle; a captured graph replays bit-identically and follows
    new inputs (the reference's graph contract, tests/fastwam/graph_replay.py:200-330)."""
    params, model = _tiny_model()
    images, img_masks, tokens, masks, noise = tiny_inputs(PI05_TINY, seed=3, batch=2)
    ref = pi05_ref.sample_actions(params, PI05_TINY, images, img_masks, tokens, masks, noise)
    st = [[t.cuda() for t in images], [t.cuda() for t in img_masks], tokens.cuda(), masks.cuda(), noise.cuda()]
    eager = model.sample_actions(*st)
    assert float((eager.cpu() - ref).abs().max()) <= 2e-2
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        model.sample_actions(*st)
    torch.cuda.current_stream().wait_stream(side)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        out = model.sample_actions(*st)
    graph.replay()
    torch.cuda.synchronize()
    first = out.clone()
    assert torch.equal(first, eager)
    graph.replay()
    torch.cuda.synchronize()
    assert torch.equal(out, first)
    st[4].copy_(torch.randn_like(st[4]))  # new noise through the static buffer
    graph.replay()
    torch.cuda.synchronize()
    assert torch.equal(out, model.sample_actions(*st))
    assert not torch.equal(out, first) and torch.isfinite(out).all()


def test_engine_interface_on_synthetic_checkpoint():
    from tybok_b200.engine import PI05B200Engine

    eng = PI05B200Engine("synthetic:pi05_tiny", device="cuda", graph=True, seed=0)
    spec = eng.describe()
    assert spec["model_type"] == "pi05_b200" and spec["chunk_size"] == PI05_TINY.chunk and eng.graph_enabled
    g = torch.Generator().manual_seed(1)
    frame = eng.make_frame({c: torch.rand(3, 56, 56, generator=g) for c in spec["cameras"]},
                           torch.rand(8, generator=g), "pick up the cube")
    noise = torch.zeros(1, PI05_TINY.chunk, PI05_TINY.max_action_dim)
    a = eng.predict_action_chunk(frame, noise=noise)
    b = eng.predict_action_chunk(frame, noise=noise)
    assert a.shape == (PI05_TINY.chunk, spec["action_dim"]) and (a == b).all() and abs(a).max() > 0
    one = eng.select_action(frame, noise=noise)
    assert (one == a[0]).all() and len(eng._queue) == PI05_TINY.chunk - 1
    with pytest.raises(NotImplementedError):
        PI05B200Engine("synthetic:pi05_tiny", device="cuda", tl_fused_expert=True)
    with pytest.raises(NotImplementedError):
        PI05B200Engine("synthetic:pi05_tiny", device="cuda", compile_model=True)
    with pytest.raises(RuntimeError):
        PI05B200Engine("synthetic:pi05_tiny", device="cuda", require_fused=True, action_fused=False)


def test_static_buffer_request_path_equals_the_general_path():
    """A batch-1 request whose frames have the model's resolution is copied straight into the
    graph's input buffers; it returns bit for bit what the general preprocessing path returns
    (eager engine, same seed), also when requests of the other kind (a frame that needs resizing,
    a missing camera) come in between."""
    from tybok_b200.engine import PI05B200Engine

    fast = PI05B200Engine("synthetic:pi05_tiny", device="cuda", graph=True, seed=0)
    gen = PI05B200Engine("synthetic:pi05_tiny", device="cuda", graph=False, seed=0)
    spec = fast.describe()
    res = spec["resize"][0]
    g = torch.Generator().manual_seed(5)
    noise = torch.randn(1, PI05_TINY.chunk, PI05_TINY.max_action_dim, generator=g)
    cams = spec["cameras"]
    for kind in ("at_res", "resize", "at_res", "missing", "at_res"):
        side = res if kind != "resize" else res + 14
        images = {c: torch.rand(3, side, side, generator=g) for c in cams}
        frame = fast.make_frame(images, torch.rand(8, generator=g), f"task {kind}")
        if kind == "missing":
            key = [k for k in frame if k.startswith("observation.images.")][-1]
            frame[key] = None
        took_static = fast._predict_chunk_static(frame, noise) is not None
        assert took_static == (kind == "at_res")
        a = fast.predict_action_chunk(frame, noise=noise)
        b = gen.predict_action_chunk(frame, noise=noise)
        assert a.shape == b.shape and (a == b).all()


def test_fused_bf16_vision_tower_matches_the_torch_layer_chain():
    """bf16 tower: residual adds inside the LayerNorm kernel, one q/k/v GEMM and the GELU GEMM
    epilogue against the plain torch chain of the same weights."""
    from tybok_b200.pi05 import PI05Model

    params = quantize_hot_linears(random_pi05_params(PI05_TINY, seed=0), PI05_TINY)
    model = PI05Model(params, PI05_TINY, device="cuda", vision_dtype=torch.bfloat16)
    assert model.vis_layers is not None
    images, *_ = tiny_inputs(PI05_TINY, seed=5, batch=2)
    img = torch.cat([t.cuda() for t in images], dim=0)
    fused = model.embed_image(img)
    packed, model.vis_layers = model.vis_layers, None
    plain = model.embed_image(img)
    model.vis_layers = packed
    assert fused.dtype == plain.dtype == torch.bfloat16
    assert w8_ref.rel_l2(fused.float().cpu(), plain.float().cpu()) < 2e-2


def test_add_layernorm_kernel():
    from tybok_b200 import ops

    g = torch.Generator().manual_seed(9)
    for m, w in ((37, 1152), (5, 128), (64, 2048), (512, 1152), (200, 1160), (70, 72)):
        x, y = (torch.empty(m, w).normal_(0, 1, generator=g).to(torch.bfloat16) for _ in range(2))
        wt, b = (torch.empty(w).normal_(0, 1, generator=g).to(torch.bfloat16) for _ in range(2))
        xs = x + y
        ref = torch.nn.functional.layer_norm(xs.float(), (w,), wt.float(), b.float(), 1e-6).to(torch.bfloat16)
        x_new, h = ops.add_layernorm(x.cuda(), y.cuda(), wt.cuda(), b.cuda())
        assert torch.equal(x_new.cpu(), xs)
        assert float((h.cpu().float() - ref.float()).abs().max()) <= 2.0**-6 * float(ref.float().abs().max())
        _, h0 = ops.add_layernorm(xs.cuda(), None, wt.cuda(), b.cuda())
        assert torch.equal(h0, h)


@pytest.mark.parametrize("m,w", [(512, 1152), (37, 128), (5, 2048)])
def test_add_layernorm_with_an_fp32_stream(m, w):
    """The forms that keep the residual stream in fp32: bf16 or fp16 sublayer output / weights (a bf16
    or fp16 tower) and all-fp32 (a TF32 tower), against torch in fp32."""
    from tybok_b200 import ops

    g = torch.Generator().manual_seed(m + w)
    x = torch.empty(m, w).normal_(0, 3, generator=g)
    y = torch.empty(m, w).normal_(0, 1, generator=g)
    wt, b = (1 + torch.empty(w).normal_(0, 0.3, generator=g)), torch.empty(w).normal_(0, 0.3, generator=g)
    for dt in (torch.bfloat16, torch.float16, torch.float32):
        yd, wd, bd = y.to(dt), wt.to(dt), b.to(dt)
        xs = x + yd.float()
        ref = torch.nn.functional.layer_norm(xs, (w,), wd.float(), bd.float(), 1e-6)
        x_new, h = ops.add_layernorm(x.cuda(), yd.cuda(), wd.cuda(), bd.cuda())
        assert x_new.dtype == torch.float32 and h.dtype == dt
        assert torch.equal(x_new.cpu(), xs)
        tol = {torch.bfloat16: 2.0**-7, torch.float16: 2.0**-10}.get(dt, 1e-5)
        assert float((h.cpu().float() - ref).abs().max()) <= tol * max(1.0, float(ref.abs().max()))
        _, h0 = ops.add_layernorm(xs.cuda(), None, wd.cuda(), bd.cuda())
        assert torch.equal(h0, h)


@pytest.mark.parametrize("m,w", [(50, 1024), (50, 2048), (7, 256), (10, 128), (130, 512)])
def test_action_tail_matches_torch(m, w):
    """Final AdaRMS norm + fp32 out-projection + Euler update + next embedding
    (flow_matching.py:193-254,464-556) against the same steps in torch fp32."""
    from tybok_b200 import ops

    g = torch.Generator().manual_seed(17)
    rnd = lambda *s, std=1.0: torch.empty(*s).normal_(0, std, generator=g)  # noqa: E731
    x = rnd(m, w).to(torch.bfloat16)
    mod = rnd(1, 3 * w, std=0.3)
    w_out, b_out, w_in, b_in = rnd(32, w, std=0.05), rnd(32, std=0.1), rnd(w, 32, std=0.2), rnd(w, std=0.1)
    x_t = rnd(m, 32)
    dt = -0.1
    y = w8_ref.adarms_norm(x, mod[:, : 2 * w])[0].float()
    xt_ref = x_t + dt * (y @ w_out.T + b_out)
    h_ref = (xt_ref @ w_in.T + b_in).to(torch.bfloat16)
    xt = x_t.cuda().clone()
    h = ops.action_tail(x.cuda(), mod.cuda(), w_out.cuda(), b_out.cuda(), xt, dt, w_in.cuda(), b_in.cuda(),
                        rows_per_group=m)
    torch.cuda.synchronize()
    assert float((xt.cpu() - xt_ref).abs().max()) <= 2e-4 * max(1.0, float(xt_ref.abs().max()))
    assert w8_ref.rel_l2(h.float().cpu(), h_ref.float()) <= 4e-3
    # embedding only (the first step), and update only (the last step)
    h0 = ops.action_tail(None, None, None, None, xt, dt, w_in.cuda(), b_in.cuda())
    assert torch.equal(h0, h)
    xt2 = x_t.cuda().clone()
    none = ops.action_tail(x.cuda(), mod.cuda(), w_out.cuda(), b_out.cuda(), xt2, dt, w_in.cuda(), b_in.cuda(),
                           rows_per_group=m, embed=False)
    assert none.numel() == 0 and torch.equal(xt2, xt)


@pytest.mark.parametrize("graph", [False, True])
def test_first_step_overlapped_with_prefix_gives_the_same_chunk(graph):
    """The first denoise step pipelined behind the prefix on a second stream (eager, and captured
    into one CUDA graph) returns bit for bit what the sequential order returns."""
    from tybok_b200.engine import PI05B200Engine

    seq = PI05B200Engine("synthetic:pi05_small", device="cuda", graph=graph, seed=0, overlap=False)
    ovl = PI05B200Engine("synthetic:pi05_small", device="cuda", graph=graph, seed=0, overlap=True)
    assert ovl.model.overlap and not seq.model.overlap
    g = torch.Generator().manual_seed(3)
    for i in range(3):
        frame = {f"observation.images.camera{c + 1}": torch.rand(3, 70, 70, generator=g) for c in range(2)}
        frame["observation.state"] = torch.randn(8, generator=g)
        frame["task"] = f"pick up the cube {i}"
        noise = torch.randn(1, 10, 32, generator=g)
        a = seq.predict_action_chunk(frame, noise=noise)
        b = ovl.predict_action_chunk(frame, noise=noise)
        assert (a == b).all()
