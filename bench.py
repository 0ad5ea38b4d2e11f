"""Benchmark of the fp8 hot path on B200: pi0.5-shaped action-chunk latency, and the W8 GEMM
against its roofline.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--batch B]
    torchrun --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...

Default workload (``pi05_chunk``): one "step" = one action chunk (SigLIP-So400m on two 224x224
cameras, 18-layer Gemma-2B-shaped prefix over 544 tokens, 18-layer Gemma-300M-shaped expert, chunk
50, 10 flow steps) of the random-init fp8 policy on synthetic inputs.  ``value`` is the p50 of K
CUDA-event-timed graph replays with inputs resident in HBM; ``e2e`` is the same chunk through
``engine.predict_action_chunk`` from pinned host frames (H2D of images / tokens / noise and D2H of the
chunk inside the timed region).  With N > 1 every rank runs an independent replica (no data-path
collective); the time is the max over ranks.  The line also carries

* ``parity``: the chunk the timed engine returns for a zero-noise request against the CPU oracle on
  the same weights and inputs;
* ``roofline``: the dominant kernel (``w8_gemm_kernel``) timed live, per call signature of the model
  and over the whole W8 linear sweep (5 projection shapes x M in {1, 50, 256, 800});
* ``cpu_baseline``: the oracle (the reference's eager torch path on dequantised weights) on the host cores;
* ``extra.batch_sweep`` (N = 1): chunks/s at 8 / 32 / 64 requests per replica;
  ``extra.dit_ffn_tp`` (N > 1): the tensor-parallel DiT FFN over the N ranks with its all-reduce timed.

``--impl reference`` times the CPU oracle alone (rank 0 only under torchrun).  Other workloads:
``dit`` (the fastWAM-class DiT denoiser, 30 blocks x 4 steps over 4146 tokens, its FFN tensor-parallel
over the N ranks), ``dit_ffn`` (one block's FFN tail), ``gemm`` / ``attention`` (small fixed cases
for profiler captures).  One JSON line on rank 0.
"""

from __future__ import annotations

import argparse
import hashlib
import json
import os
import statistics
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

METRIC = "pi05_fp8_action_chunk_p50_ms"
WORKLOAD = "pi05_full: SigLIP-So400m 2x224^2 + Gemma-2B prefix (544 tok) + Gemma-300M expert, chunk 50, 10 steps"
DTYPE = "e4m3 weights x bf16 activations, fp32 accumulate"
TRAFFIC_FILE = os.path.join(ROOT, "profiles", "w8_gemm_m50_n1024_k4096.json")
TRAFFIC_SOURCES = ("tybok_b200/csrc/w8_gemm.cu", "tybok_b200/csrc/ptx.cuh")


def _config(batch: int, replicas: int) -> dict:
    """The workload description both arms print (identical keys and values)."""
    return {"workload": WORKLOAD, "batch_per_gpu": batch, "replicas": replicas,
            "l2": "weights streamed per chunk (3.4 GB) exceed the 126 MB L2"}


def _peaks() -> tuple[dict, str]:
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        return json.load(open(path)), "measured"
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}, "fallback"


def _all_host_threads() -> int:
    """Every host thread this process may use (a torchrun launch sets OMP_NUM_THREADS=1 for its ranks)."""
    try:
        n = max(1, len(os.sched_getaffinity(0)))
    except (AttributeError, OSError):
        n = max(1, os.cpu_count() or 1)
    # A container may see more logical CPUs than its CPU-time quota lets run at once; a thread pool sized
    # past the quota spends its time throttled (seen: 45 s instead of 1 s per oracle chunk with 24 threads).
    try:
        quota, period = open("/sys/fs/cgroup/cpu.max").read().split()[:2]
        if quota != "max":
            n = max(1, min(n, int(int(quota) / int(period) + 0.5)))
    except (OSError, ValueError):
        pass
    torch.set_num_threads(n)
    return n


class ClockSampler:
    """SM clock and throttle reasons of one GPU while the timed region runs, sampled by an
    ``nvidia-smi`` child process (every 50 ms), not through NVML inside this process: an in-process
    NVML poll running beside NCCL collectives stalled both ranks of the tensor-parallel workload.
    ``start()`` spawns the child (early, it needs a moment to come up), ``mark()`` opens the window
    whose samples count, ``stop()`` closes it and returns the summary."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
    NAMES = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")

    def __init__(self, index: int):
        self.index, self.rows, self.t0, self.proc, self.note = index, [], None, None, None

    def start(self):
        import shutil
        import subprocess

        if os.environ.get("TYBOK_BENCH_NO_CLOCKS") or not shutil.which("nvidia-smi"):
            self.note = "sampling_disabled" if os.environ.get("TYBOK_BENCH_NO_CLOCKS") else "nvidia-smi_unavailable"
            return
        visible = os.environ.get("CUDA_VISIBLE_DEVICES")
        gpu = visible.split(",")[self.index] if visible else str(self.index)
        self.proc = subprocess.Popen(["nvidia-smi", "-i", gpu, f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                                      "-lms", "50"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)

        def pump():
            for line in self.proc.stdout:
                self.rows.append((time.time(), line))

        threading.Thread(target=pump, daemon=True).start()

    def mark(self):
        self.t0 = time.time()

    def stop(self) -> dict:
        t1 = time.time()
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [self.note]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except Exception:
            self.proc.kill()
        t0 = self.t0 if self.t0 is not None else 0.0
        inside = [ln for t, ln in self.rows if t0 <= t <= t1 + 0.06] or [ln for _, ln in self.rows[-3:]]
        mhz, reasons, mx = [], set(), None
        for ln in inside:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 6 or not f[0].isdigit():
                continue
            mhz.append(int(f[0]))
            mx = int(f[1]) if f[1].isdigit() else mx
            reasons |= {n for n, v in zip(self.NAMES, f[2:6]) if v.lower().startswith("active")}
        return {"sm_mhz": statistics.median(mhz) if mhz else None, "sm_max_mhz": mx, "reasons": sorted(reasons),
                "samples": len(mhz)}


# ------------------------------------------------------------------------------------ inputs
def _synthetic_frame(shape, cameras, seed: int, pin: bool = True) -> dict:
    """One seeded request: camera frames in [0, 1] at the model's resolution, a state vector, prompt
    token ids (no tokenizer files exist for a random-init policy) with an all-ones mask."""
    g = torch.Generator().manual_seed(seed)
    res = shape.vision.image
    frame = {}
    for c in cameras:
        img = torch.rand(3, res, res, generator=g)
        frame[f"observation.images.{c}"] = img.pin_memory() if pin else img
    frame["observation.state"] = torch.randn(8, generator=g)
    frame["task"] = "pick up the red block"
    frame["observation.language.tokens"] = torch.randint(0, shape.vocab, (shape.lang_len,), generator=g)
    frame["observation.language.attention_mask"] = torch.ones(shape.lang_len, dtype=torch.bool)
    return frame


def _oracle_inputs(frames, cameras):
    images = [torch.stack([fr[f"observation.images.{c}"] for fr in frames]).float() * 2.0 - 1.0 for c in cameras]
    img_masks = [torch.ones(len(frames), dtype=torch.bool) for _ in cameras]
    tokens = torch.stack([fr["observation.language.tokens"] for fr in frames])
    masks = torch.stack([fr["observation.language.attention_mask"] for fr in frames])
    return images, img_masks, tokens, masks


def _oracle_weights(seed: int, device: str):
    """Seeded weights of the full configuration in the oracle's form: quantised with the reference
    recipe, dequantised to bf16 once (what the reference's loader does), on the CPU."""
    from oracle import w8_ref
    from tybok_b200.shapes import PI05_FULL
    from tybok_b200.weights import quantize_hot_linears, random_pi05_params

    params = quantize_hot_linears(random_pi05_params(PI05_FULL, seed=seed, device=device), PI05_FULL)
    params = {k: v.cpu() for k, v in params.items()}
    if device != "cpu":
        torch.cuda.empty_cache()
    deq = {}
    for k, v in params.items():
        if k.endswith(".scale_weight"):
            continue
        deq[k] = w8_ref.dequant_w8(v, params[k[: -len("weight")] + "scale_weight"]) if v.dtype == torch.float8_e4m3fn else v
    return deq


def _cpu_chunks(deq, frames_list, cameras, noise, warmup: int, reps: int, budget_s: float | None = None):
    """Warm-up and timed oracle chunks; returns (times in ms, last output).  With ``budget_s`` the leg
    stays bounded on a slow host: warm-ups beyond the first are dropped once a quarter of the budget is
    gone, and the timed chunks stop (after at least one) when the budget is spent."""
    from oracle import pi05_ref
    from tybok_b200.shapes import PI05_FULL

    times, out = [], None
    start = time.perf_counter()
    i = warm = 0
    while len(times) < reps:
        inputs = _oracle_inputs(frames_list[i % len(frames_list)], cameras)
        t0 = time.perf_counter()
        out = pi05_ref.sample_actions(deq, PI05_FULL, *inputs, noise)
        now = time.perf_counter()
        i += 1
        if warm < warmup and not (budget_s is not None and warm >= 1 and now - start > budget_s / 4):
            warm += 1
            if warm < warmup and budget_s is not None and now - start > budget_s / 4:
                warm = warmup  # the first warm-up was slow enough: the next chunk is timed
            continue
        times.append((now - t0) * 1e3)
        if budget_s is not None and now - start > budget_s:
            break
    return times, out


# ------------------------------------------------------------------------------------ GEMM timing
def _time_graph(call, iters: int) -> float:
    """Microseconds per call of ``call(i)``, ``iters`` calls captured back to back in one CUDA graph,
    best of three replays timed with CUDA events on the launching stream."""
    for i in range(3):
        call(i)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        for i in range(iters):
            call(i)
    graph.replay()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    best = float("inf")
    for _ in range(3):
        e0.record()
        graph.replay()
        e1.record()
        torch.cuda.synchronize()
        best = min(best, e0.elapsed_time(e1) / iters * 1e3)
    del graph
    return best


def _rotating_weights(n: int, k: int, dev, budget: float = 400e6):
    """Weight copies whose total exceeds 3x L2, so that every launch streams its weights from HBM
    as it does inside a chunk."""
    nbuf = min(48, max(4, int(budget // (n * k)) + 1))
    return [torch.randint(0, 120, (n, k), dtype=torch.uint8, device=dev).view(torch.float8_e4m3fn) for _ in range(nbuf)]


def _traffic() -> tuple[int | None, str]:
    """DRAM bytes of one captured launch of the expert down projection, from the machine-readable
    record beside the ncu summary; ``None`` (with the reason) when the kernel sources have changed
    since the capture."""
    if not os.path.exists(TRAFFIC_FILE):
        return None, "no ncu record (profiles/w8_gemm_m50_n1024_k4096.json missing)"
    rec = json.load(open(TRAFFIC_FILE))
    for rel in TRAFFIC_SOURCES:
        digest = hashlib.sha256(open(os.path.join(ROOT, rel), "rb").read()).hexdigest()
        if rec.get("source_sha256", {}).get(rel) != digest:
            return None, f"stale: {rel} changed after the ncu capture ({rec.get('captured', '?')})"
    return int(rec["dram_bytes_per_launch"]), (f"M=50 N=1024 K=4096: {rec['dram_bytes_per_launch']} B measured (ncu, "
                                               f"{rec.get('captured', '?')}) vs {rec['algorithmic_bytes']} B algorithmic per launch")


def _gemm_roofline(shape, batch: int, dev, peaks, peaks_kind, sweep: bool) -> dict:
    """Roofline of the dominant kernel (``w8_gemm_kernel``), measured live: every GEMM call
    signature of one chunk is replayed as a CUDA graph of back-to-back launches over rotating
    weight copies and timed with CUDA events.  Algorithmic bytes per launch =
    nw*(N*K + 4N) + 2*M*K + 2*M*N (nw = 2 for the gated form), flops = 2*nw*M*N*K.
    ``achieved`` aggregates the action-expert launches (M = 50*batch, HBM-bound, 720 of the 792
    launches of a chunk); the prefix launches (M = 544*batch, tensor-bound) are reported beside."""
    from tybok_b200 import ops
    from tybok_b200.pi05 import TWO_PLANE_MIN_TOKENS

    s = shape

    def shapes(spec, m, layers, reps):
        hd, kvd = spec.num_heads * spec.head_dim, spec.num_kv_heads * spec.head_dim
        return [("qkv", m, hd + 2 * kvd, spec.width, 1, layers * reps), ("o", m, spec.width, hd, 1, layers * reps),
                ("geglu", m, spec.mlp_dim, spec.width, 2, layers * reps),
                ("down", m, spec.width, spec.mlp_dim, 1, layers * reps)]

    groups = {"expert": shapes(s.expert, batch * s.chunk, s.expert.depth, s.steps),
              "prefix": shapes(s.vlm, batch * s.prefix_len, s.vlm.depth, 1)}
    out = {}
    for gname, lst in groups.items():
        rows = []
        for name, m, n, k, nw, count in lst:
            ws = _rotating_weights(nw * n, k, dev)  # the gated form streams gate and up as one interleaved [2N, K] matrix
            nbuf = len(ws)
            sc = torch.rand(nw * n, device=dev)
            x = torch.randn(m, k, device=dev).to(torch.bfloat16)
            xp = ops.split3(x, 4)
            res = torch.randn(m, n, device=dev).to(torch.bfloat16)
            # the GEMMs fed by a norm take two e4m3 planes from the model's two-plane threshold on
            two = m >= TWO_PLANE_MIN_TOKENS and name in ("qkv", "geglu")
            if two:
                x2, rs = ops.norm_planes2(x, ops.NORM_RMS, torch.zeros(k, device=dev))

            def call(i):
                w = ws[i % nbuf]
                if two:
                    return ops.w8x2_gemm(x2, rs, w, sc, epilogue=ops.EPI_GEGLU_PACKED if nw == 2 else ops.EPI_NONE,
                                         out_bf16=nw == 1, out_planes=nw == 2)
                if nw == 2:
                    return ops.w8x3_geglu_packed(xp, 4, w, sc, out_bf16=False, out_planes=True)
                if name == "qkv":
                    return ops.w8x3_linear(xp, 4, w, sc)
                return ops.w8x3_linear(xp, 4, w, sc, epilogue=ops.EPI_RESIDUAL, residual=res)

            us = _time_graph(call, 2 * nbuf)
            byts = nw * (n * k + 4 * n) + 2 * m * k + 2 * m * n
            rows.append({"gemm": name, "M": m, "N": n, "K": k, "nw": nw, "planes": 2 if two else 3, "us": round(us, 2), "count": count,
                         "GBps": round(byts / us / 1e3, 1), "TFps": round(2.0 * nw * m * n * k / us / 1e6, 1),
                         "bytes": byts, "flops": 2.0 * nw * m * n * k})
            del ws
        out[gname] = rows
    torch.cuda.empty_cache()

    def agg(rows, key):
        return sum(r["count"] * r[key] for r in rows) / sum(r["count"] * r["us"] for r in rows)

    hbm = agg(out["expert"], "bytes") / 1e3  # bytes/us -> GB/s
    tc = agg(out["prefix"], "flops") / 1e6  # flops/us -> TFLOP/s
    strip = lambda rows: [{k: v for k, v in r.items() if k not in ("bytes", "flops")} for r in rows]  # noqa: E731
    traffic, traffic_note = _traffic()
    if (batch * s.chunk, s.expert.width, s.expert.mlp_dim) != (50, 1024, 4096):
        traffic, traffic_note = None, "the ncu record covers M=50 N=1024 K=4096 only"
    roof = {
        "bound": "hbm", "kernel": "w8_gemm_kernel (action-expert launches, M=%d)" % (batch * s.chunk),
        "achieved": round(hbm, 1), "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": round(hbm / peaks["hbm_gbs"], 4),
        "traffic": traffic, "traffic_case": traffic_note, "peak_source": peaks_kind, "per_shape": strip(out["expert"]),
        "prefix": {"bound": "tensor", "achieved": round(tc, 1), "peak": peaks["bf16_tflops"], "unit": "TFLOP/s",
                   "frac": round(tc / peaks["bf16_tflops"], 4), "per_shape": strip(out["prefix"])},
    }
    if sweep:
        roof["sweep"] = _w8_sweep(dev, peaks)
    return roof


def _w8_sweep(dev, peaks) -> list[dict]:
    """The W8 linear sweep: the Gemma-2B and Gemma-300M-expert projection shapes at M in {1, 50, 256, 800}
    (bf16 activations ~N(0,1), e4m3 weights, fp32 accumulation).  ``us`` times the GEMM kernel on
    activation planes (the form the fused producers feed); ``us_bf16_in`` the two-launch bf16 entry
    point (plane split + GEMM).  Each case is held against both rooflines -- HBM (measured copy
    bandwidth) and tensor (measured dense bf16) -- and ``binds`` names the slower of the two floors."""
    from tybok_b200 import ops
    from tybok_b200.shapes import W8_SWEEP_M, W8_SWEEP_NK

    rows = []
    for n, k in W8_SWEEP_NK:
        ws = _rotating_weights(n, k, dev)
        nbuf = len(ws)
        sc = torch.rand(n, device=dev)
        for m in W8_SWEEP_M:
            x = torch.randn(m, k, device=dev).to(torch.bfloat16)
            xp = ops.split3(x, 4)
            us = _time_graph(lambda i: ops.w8x3_linear(xp, 4, ws[i % nbuf], sc), 2 * nbuf)
            us2 = _time_graph(lambda i: ops.w8a16_linear(x, ws[i % nbuf], sc), 2 * nbuf)
            us_two = None
            if m >= 128 and k <= 4096:  # the two-plane form a norm kernel (rows of up to 4096 channels) can feed
                x2, rs = ops.norm_planes2(x, ops.NORM_RMS, torch.zeros(k, device=dev))
                us_two = _time_graph(lambda i: ops.w8x2_gemm(x2, rs, ws[i % nbuf], sc), 2 * nbuf)
            byts = n * k + 4 * n + 2 * m * k + 2 * m * n
            flops = 2.0 * m * n * k
            t_hbm, t_tc = byts / peaks["hbm_gbs"] / 1e3, flops / peaks["bf16_tflops"] / 1e6  # us
            rows.append({"N": n, "K": k, "M": m, "us": round(us, 2), "us_bf16_in": round(us2, 2),
                         "us_two_plane": None if us_two is None else round(us_two, 2),
                         "frac_tensor_two_plane": None if us_two is None else round(t_tc / us_two, 4),
                         "GBps": round(byts / us / 1e3, 1), "TFps": round(flops / us / 1e6, 1),
                         "frac_hbm": round(t_hbm / us, 4), "frac_tensor": round(t_tc / us, 4),
                         "binds": "hbm" if t_hbm >= t_tc else "tensor", "frac_of_binding": round(max(t_hbm, t_tc) / us, 4)})
        del ws
    torch.cuda.empty_cache()
    return rows


# ------------------------------------------------------------------------------------ arms
def run_reference(args, rank: int) -> None:
    """The reference arm: the CPU oracle on the host cores, rank 0 only, nothing on a GPU."""
    if rank != 0:
        return
    from tybok_b200.shapes import PI05_FULL as S

    cores = _all_host_threads()
    deq = _oracle_weights(seed=0, device="cpu")
    cams = [f"camera{i + 1}" for i in range(S.n_cams)]
    frames = [[_synthetic_frame(S, cams, 100 + i, pin=False) for _ in range(args.batch)] for i in range(4)]
    noise = torch.randn(args.batch, S.chunk, S.max_action_dim, generator=torch.Generator().manual_seed(1))
    times, _ = _cpu_chunks(deq, frames, cams, noise, max(1, args.warmup), max(1, args.steps), budget_s=240.0)
    p50 = statistics.median(times)
    line = {
        "impl": "reference", "metric": METRIC, "value": round(p50, 2), "unit": "ms", "n_gpus": args.gpus,
        "steps": len(times), "requested_steps": max(1, args.steps), "warmup": max(1, args.warmup),
        "ms_per_step": round(sum(times) / len(times), 2),
        "higher_is_better": False, "scaling": "weak", "vs_baseline": None,
        "dtype": DTYPE + " (weights dequantised to bf16, the reference's loader path)", "data": "synthetic",
        "config": _config(args.batch, args.gpus),
        "cpu_baseline": {"value": round(p50, 2), "unit": "ms", "cores": cores, "kind": "port",
                         "min": round(min(times), 2), "max": round(max(times), 2),
                         "sample": f"{len(times)} full chunks of the config (240 s budget) after up to {max(1, args.warmup)} warm-up "
                                   f"(oracle/pi05_ref.py, torch {torch.__version__}, {os.cpu_count()} logical CPUs)"},
        "e2e": {"value": round(p50, 2), "unit": "ms", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def _phases(engine) -> dict:
    """Where a chunk's time goes: the three phases of ``sample_actions`` (vision tower + projector,
    prefix pass, the denoise passes) each captured as its own CUDA graph on the engine's static
    inputs and timed with CUDA events (median of 10 replays); the expert passes also with every AdaRMS
    norm as its own kernel, for the effect of folding them into the GEMMs."""
    from tybok_b200 import ops

    m = engine.model
    s = m.shape
    st = engine._static

    def timed(fn):
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            fn()
        torch.cuda.current_stream().wait_stream(side)
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            out = fn()
        g.replay()
        ts = []
        for _ in range(10):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            g.replay()
            e1.record()
            torch.cuda.synchronize()
            ts.append(e0.elapsed_time(e1))
        return round(statistics.median(ts), 4), out

    with torch.no_grad():
        out = {}
        out["tower_projector_ms"], (embs, pad) = timed(lambda: m.embed_prefix(st["images"], st["img_masks"], st["tokens"], st["masks"]))
        out["prefix_ms"], _ = timed(lambda: m.prefill(embs, pad))
        b, l = st["noise"].shape[0], st["noise"].shape[1]
        key_valid, pos = m._suffix_constants(pad, b, l)
        x_t = st["noise"].float().contiguous().clone()
        dt = -1.0 / s.steps

        def expert():
            h = ops.action_tail(None, None, None, None, x_t, dt, *m.action_in)
            for step in range(s.steps):
                x = m._expert_layers(step, h, b, l, pad, key_valid, pos)
                h = ops.action_tail(x, m.final_mods[step], *m.action_out, x_t, dt, *m.action_in, rows_per_group=b * l,
                                    embed=step + 1 < s.steps)
            return x_t

        out["expert_passes_ms"], _ = timed(expert)
        out["expert_us_per_layer_step"] = round(out["expert_passes_ms"] * 1e3 / (s.steps * s.expert.depth), 2)
        if m.fold is not None:
            fold, m.fold = m.fold, None
            try:
                out["expert_passes_norm_kernels_ms"], _ = timed(expert)
            finally:
                m.fold = fold
    return out


def _batch_sweep(rank: int, local: int, overlap: bool, vision: str, batches=(8, 32, 64)) -> list[dict]:
    """Batched throughput of one replica: ``b`` requests per graph replay (the data-parallel serving
    configuration at batch {8, 32, 64} per GPU); chunks/s from 5 event-timed replays."""
    from tybok_b200.engine import PI05B200Engine

    rows = []
    for b in batches:
        eng = PI05B200Engine(f"synthetic:pi05_full@{rank}", device=f"cuda:{local}", graph=True, warmup=True, seed=rank,
                             batch_size=b, overlap=overlap, vision_precision=vision)
        for _ in range(2):
            eng._graph.replay()
        torch.cuda.synchronize()
        evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(5)]
        for e0, e1 in evs:
            e0.record()
            eng._graph.replay()
            e1.record()
        torch.cuda.synchronize()
        ms = statistics.median(a.elapsed_time(c) for a, c in evs)
        rows.append({"batch": b, "ms_per_batch": round(ms, 3), "chunks_per_s": round(b / ms * 1e3, 1),
                     "ms_per_chunk": round(ms / b, 3)})
        if b == 32:  # where a batched chunk's time goes (tower / prefix / expert passes as separate graphs)
            rows[-1]["phases"] = {k: v for k, v in _phases(eng).items() if k.endswith("_ms")}
        del eng
        torch.cuda.empty_cache()
    return rows


def _dit_ffn_tp(rank: int, world: int, local: int, peaks, steps: int = 10) -> dict:
    """The tensor-parallel DiT FFN tail (hidden 3072, ffn 14336, 4146 tokens) over the ranks of this
    run: ms per block, the all-reduce's own share from CUDA events around it, and the result
    against the single-GPU form computed on rank 0 (rel-L2 <= 1e-2)."""
    import torch.distributed as dist

    from oracle import w8_ref
    from tybok_b200.dit import DiTFFN, finish_after_reduce
    from tybok_b200.shapes import DIT_FULL as S

    g = torch.Generator(device="cuda").manual_seed(0)  # same weights and inputs on every rank
    rn = lambda *sh, std=1.0: torch.empty(*sh, device="cuda").normal_(0, std, generator=g)  # noqa: E731
    raw = [(rn(S.ffn, S.hidden, std=0.02), rn(S.ffn, std=0.1), rn(S.hidden, S.ffn, std=0.02), rn(S.hidden, std=0.1))
           for _ in range(3)]  # 3 x 88 MB of e4m3 weights (per-rank shards still exceed L2 together with activations)
    blocks = [DiTFFN(*w, device=f"cuda:{local}", rank=rank, world=world) for w in raw]
    x = rn(S.seq, S.hidden).to(torch.bfloat16)
    shift, scale, gate = (rn(S.hidden, std=0.5).to(torch.bfloat16) for _ in range(3))
    for i in range(3):
        y = blocks[i % 3](x, shift, scale, gate)
    torch.cuda.synchronize()
    dist.barrier()
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(3 * steps + 1)]
    ev[0].record()
    for i in range(steps):
        blk = blocks[i % 3]
        part = blk.partial(x, shift, scale)
        ev[3 * i + 1].record()
        dist.all_reduce(part, group=blk.group)
        ev[3 * i + 2].record()
        y = finish_after_reduce(x, part, blk.down[2], gate)
        ev[3 * i + 3].record()
    torch.cuda.synchronize()
    total = ev[0].elapsed_time(ev[-1]) / steps
    reduce_ms = statistics.median(ev[3 * i + 1].elapsed_time(ev[3 * i + 2]) for i in range(steps))
    t = torch.tensor([total, reduce_ms], device="cuda", dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    out = {"ranks": world, "ms_per_block": round(float(t[0]), 4), "allreduce_ms": round(float(t[1]), 4),
           "allreduce_bytes": S.seq * S.hidden * 2,
           "TFps": round(4.0 * S.seq * S.hidden * S.ffn / float(t[0]) / 1e9, 1),
           "frac_of_bf16_peak_x_ranks": round(4.0 * S.seq * S.hidden * S.ffn / float(t[0]) / 1e9 / (peaks["bf16_tflops"] * world), 4)}
    if rank == 0:
        last = (steps - 1) % 3
        single = DiTFFN(*raw[last], device=f"cuda:{local}", rank=0, world=1)(x, shift, scale, gate)
        out["rel_l2_vs_single_gpu"] = round(w8_ref.rel_l2(y.float().cpu(), single.float().cpu()), 6)
        out["parity_ok"] = out["rel_l2_vs_single_gpu"] <= 1e-2
    return out


def run_ours(args, rank: int, world: int) -> None:
    import torch.distributed as dist

    from tybok_b200 import ops
    from tybok_b200.engine import PI05B200Engine

    local = int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    peaks, peaks_kind = _peaks()

    engine = PI05B200Engine(f"synthetic:pi05_full@{rank}", device=f"cuda:{local}", graph=False, warmup=True,
                            seed=rank, batch_size=args.batch, overlap=not args.no_overlap,
                            vision_precision=args.vision_precision)
    if args.no_fold:  # comparison run: every AdaRMS norm as its own kernel
        engine.model.fold = None
    adarms_folded = engine.model.fold is not None
    l1 = ops.launch_count()
    engine._capture()
    launches_per_chunk = (ops.launch_count() - l1) // 3  # two warm-up passes + the captured pass

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    graph = engine._graph
    sampler = ClockSampler(local)
    sampler.start()
    for _ in range(max(3, args.warmup)):
        graph.replay()
    barrier()
    sampler.mark()
    evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(args.steps)]
    t_all0, t_all1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t_all0.record()
    for e0, e1 in evs:
        e0.record()
        graph.replay()
        e1.record()
    t_all1.record()
    barrier()
    per = sorted(a.elapsed_time(b) for a, b in evs)
    p50 = statistics.median(per)
    total_ms = t_all0.elapsed_time(t_all1)
    if world > 1:
        t = torch.tensor([p50, total_ms], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        p50, total_ms = float(t[0]), float(t[1])

    # end to end through the public call: host frames -> numpy chunk(s)
    s = engine.config.shape
    cams = engine.describe()["cameras"]
    frames = [[_synthetic_frame(s, cams, 100 + 10 * i + j) for j in range(args.batch)] for i in range(4)]
    call = (lambda fr: engine.predict_action_chunk(fr[0])) if args.batch == 1 else engine.predict_action_chunks
    for i in range(3):
        call(frames[i % 4])
    barrier()
    e2e = []
    for i in range(args.steps):
        t0 = time.perf_counter()
        call(frames[i % 4])
        e2e.append((time.perf_counter() - t0) * 1e3)
    clocks = sampler.stop()  # the window covers the device-timed replays and the end-to-end calls after them
    e2e_p50 = statistics.median(e2e)
    if world > 1:
        t = torch.tensor([e2e_p50], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_p50 = float(t[0])
    res = s.vision.image
    h2d = args.batch * (s.n_cams * 3 * res * res * 4 + s.n_cams + s.lang_len * 9 + s.chunk * s.max_action_dim * 4)
    d2h = args.batch * s.chunk * engine.config.action_dim * 4

    extra: dict = {}
    if world > 1 and not args.no_extras:
        extra["dit_ffn_tp"] = _dit_ffn_tp(rank, world, local, peaks)
    line = None
    if rank == 0:
        # parity of the timed engine: a zero-noise request against the CPU oracle (computed below)
        zero = torch.zeros(args.batch, s.chunk, s.max_action_dim)
        gpu_chunk = None
        if not args.no_cpu_baseline and world == 1:  # the CPU leg (and with it the parity field) runs at N = 1 only
            got = engine.predict_action_chunk(frames[0][0], noise=zero) if args.batch == 1 else \
                engine.predict_action_chunks(frames[0], noise=zero)
            gpu_chunk = torch.from_numpy(got).reshape(args.batch, s.chunk, -1)
        roof = _gemm_roofline(s, args.batch, torch.device("cuda", local), peaks, peaks_kind,
                              sweep=world == 1 and not args.no_extras)
        if world == 1 and args.batch == 1 and not args.no_extras:
            extra["phases"] = _phases(engine)
        ops.check_status()
        del engine, graph
        torch.cuda.empty_cache()
        if world == 1 and args.batch == 1 and not args.no_extras:
            extra["batch_sweep"] = _batch_sweep(rank, local, not args.no_overlap, args.vision_precision)
        cpu = parity = None
        if not args.no_cpu_baseline and world == 1:  # the CPU leg (and with it the parity field) runs at N = 1 only
            cores = _all_host_threads()
            deq = _oracle_weights(seed=rank, device="cuda")
            unpinned = [[{k: (v.clone() if isinstance(v, torch.Tensor) else v) for k, v in fr.items()} for fr in fl]
                        for fl in frames[:1]]
            reps = 5 if world == 1 else 1
            times, ref = _cpu_chunks(deq, unpinned, cams, zero, 1, reps)
            cpu = {"value": round(statistics.median(times), 1), "unit": "ms", "cores": cores, "kind": "port",
                   "min": round(min(times), 1), "max": round(max(times), 1),
                   "sample": f"{reps} full chunks of the same config (batch {args.batch}) after 1 warm-up "
                             f"(oracle/pi05_ref.py, {os.cpu_count()} logical CPUs)"}
            from oracle import w8_ref
            ref = ref[:, :, : gpu_chunk.shape[-1]]
            parity = {"max_abs": round(float((gpu_chunk - ref).abs().max()), 6), "rel_l2": round(w8_ref.rel_l2(gpu_chunk, ref), 6),
                      "tolerance_max_abs": 2e-2, "config": "pi05_full", "batch": args.batch,
                      "what": f"engine.predict_action_chunk (graph replay, {args.vision_precision} tower, step-0 overlap) vs "
                              "oracle/pi05_ref.sample_actions on the same seeded weights and request, zero noise"}
        line = {
            "metric": METRIC, "value": round(p50, 4), "unit": "ms", "n_gpus": world, "steps": args.steps,
            "warmup": max(3, args.warmup), "ms_per_step": round(total_ms / args.steps, 4), "higher_is_better": False,
            "scaling": "weak", "vs_baseline": None, "dtype": DTYPE + " (activations as 3 exact e5m2 planes; norm-fed GEMMs of 128+ tokens: 2 e4m3 planes with a per-row power-of-two scale)",
            "data": "synthetic", "config": _config(args.batch, world),
            "run": {"cuda_graph": True, "overlap_step0": not args.no_overlap, "vision_tower": args.vision_precision,
                    "adarms_folded": adarms_folded},
            "chunks_per_s": round(world * args.batch / (total_ms / args.steps) * 1e3, 2),
            "clocks": clocks, "gpu_launches": launches_per_chunk * args.steps,
            "e2e": {"value": round(e2e_p50, 4), "unit": "ms", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
            "parity": parity, "roofline": roof, "cpu_baseline": cpu, "extra": extra,
        }
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def run_dit_ffn(args, rank: int, world: int) -> None:
    """Secondary workload: the FFN tail of one fastWAM-class DiT block (hidden 3072, ffn 14336,
    4096 + 50 tokens), tensor-parallel over N GPUs with one NCCL all-reduce per call (strong
    scaling: the work is fixed, the weights are sharded)."""
    import torch.distributed as dist

    from tybok_b200 import ops
    from tybok_b200.dit import DiTFFN
    from tybok_b200.shapes import DIT_FULL as S

    local = int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    peaks, peaks_kind = _peaks()
    g = torch.Generator(device="cuda").manual_seed(0)  # same weights on every rank
    rn = lambda *sh, std=1.0: torch.empty(*sh, device="cuda").normal_(0, std, generator=g)  # noqa: E731
    nblk = 6  # rotating blocks: 6 x 88 MB of e4m3 weights > L2
    blocks = [DiTFFN(rn(S.ffn, S.hidden, std=0.02), rn(S.ffn, std=0.1), rn(S.hidden, S.ffn, std=0.02),
                     rn(S.hidden, std=0.1), device=f"cuda:{local}", rank=rank, world=world) for _ in range(nblk)]
    x = rn(S.seq, S.hidden).to(torch.bfloat16)
    shift, scale, gate = (rn(S.hidden, std=0.5).to(torch.bfloat16) for _ in range(3))
    for i in range(max(3, args.warmup)):
        blocks[i % nblk](x, shift, scale, gate)
    sampler = ClockSampler(local)
    sampler.start()
    for i in range(30):  # keeps the device busy while the sampling child comes up
        blocks[i % nblk](x, shift, scale, gate)
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    sampler.mark()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(args.steps):
        y = blocks[i % nblk](x, shift, scale, gate)
    e1.record()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    clocks = sampler.stop()
    ms = e0.elapsed_time(e1) / args.steps
    if world > 1:
        t = torch.tensor([ms], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t[0])
    ops.check_status()
    flops = 4.0 * S.seq * S.hidden * S.ffn
    if rank == 0:
        print(json.dumps({
            "metric": "dit_ffn_tail_ms_per_block", "value": round(ms, 4), "unit": "ms", "n_gpus": world,
            "steps": args.steps, "warmup": max(3, args.warmup), "ms_per_step": round(ms, 4), "higher_is_better": False,
            "scaling": "strong", "vs_baseline": None, "dtype": DTYPE,
            "data": "synthetic", "config": {"workload": "dit_ffn: hidden 3072, ffn 14336, 4146 tokens, TP over N GPUs",
                                            "l2": "6 rotating blocks (528 MB of weights) exceed L2"},
            "clocks": clocks, "gpu_launches": 3 * args.steps,
            "roofline": {"bound": "tensor", "achieved": round(flops / ms / 1e9, 1), "peak": peaks["bf16_tflops"] * world,
                         "unit": "TFLOP/s", "frac": round(flops / ms / 1e9 / (peaks["bf16_tflops"] * world), 4),
                         "traffic": None, "peak_source": peaks_kind},
            "finite": bool(torch.isfinite(y.float()).all()),
        }), flush=True)
    if world > 1:
        dist.destroy_process_group()


# ------------------------------------------------------------------------------------ DiT denoiser
DIT_METRIC = "dit_fp8_denoise_ms"
DIT_WORKLOAD = ("fastWAM-class DiT denoiser: 30 blocks, hidden 3072, 24 heads x 128, FFN 14336; 4096 latent-video + 50 "
                "action tokens, 129-token context (128 text embeddings + 1 proprio token from a 14-dim state), 4 steps")


def _dit_inputs(S, device, seed: int = 0):
    """Seeded inputs of the denoiser: tokens ~N(0,1), a context of 128 text embeddings plus one
    proprio token ``Linear(14 -> hidden)(state)`` with the last four text tokens masked, per-step
    modulation tables, the dense rotary table, the shifted flow schedule's step sizes."""
    from oracle.dit_ref import sampling_deltas  # schedule arithmetic only (a few floats)

    g = torch.Generator().manual_seed(seed)
    x = torch.empty(S.seq, S.hidden).normal_(0, 1, generator=g).to(torch.bfloat16)
    text = torch.empty(S.context_len - 1, S.hidden).normal_(0, 1, generator=g)
    state = torch.empty(S.state_dim).normal_(0, 1, generator=g)
    proprio = torch.empty(S.hidden, S.state_dim).normal_(0, 0.3, generator=g) @ state
    context = torch.cat([text, proprio[None]]).to(torch.bfloat16)
    mask = torch.ones(S.context_len, dtype=torch.bool)
    mask[S.context_len - 5 : S.context_len - 1] = False
    t_mods = torch.empty(S.steps, 6, S.hidden).normal_(0, 0.5, generator=g).to(torch.bfloat16)
    ang = torch.outer(torch.arange(S.seq, dtype=torch.float64),
                      1.0 / torch.pow(10000, torch.arange(0, S.head_dim, 2, dtype=torch.float64) / S.head_dim))
    freqs = torch.polar(torch.ones_like(ang), ang)[:, None, :]
    return {"x": x, "context": context, "mask": mask, "t_mods": t_mods, "freqs": freqs, "deltas": sampling_deltas(S.steps)}


def _dit_flops(S) -> float:
    """Dense flops of one pass (all steps): projections + FFN + self-attention + cross-attention."""
    a = S.heads * S.head_dim
    lin = 2.0 * S.seq * (3 * a * S.hidden + a * S.hidden + 2 * a * S.hidden + 2 * S.hidden * S.ffn)
    attn = 4.0 * S.seq * S.seq * S.head_dim * S.heads + 4.0 * S.seq * S.context_len * S.head_dim * S.heads
    return S.steps * S.blocks * (lin + attn)


def _dit_cpu_block(S, inp, bp_cpu, reps: int):
    """One block of the denoiser on the CPU oracle at the full sequence length; returns (times ms, output)."""
    from oracle import dit_ref

    times, y = [], None
    for i in range(1 + reps):
        t0 = time.perf_counter()
        y = dit_ref.block_forward(bp_cpu, S.heads, inp["x"][None], inp["context"][None], inp["t_mods"][0][None], inp["freqs"],
                                  inp["mask"][None])
        if i:
            times.append((time.perf_counter() - t0) * 1e3)
    return times, y


def run_dit_reference(args, rank: int) -> None:
    """Reference arm of the DiT workload: the CPU oracle on ONE block at the full sequence length
    (a bounded sample), extrapolated to blocks x steps; rank 0 only, nothing on a GPU."""
    if rank != 0:
        return
    from tybok_b200.shapes import DIT_FULL as S
    from tybok_b200.weights import quantize_dit_block, random_dit_block_params

    cores = _all_host_threads()
    bp = quantize_dit_block(random_dit_block_params(S, seed=0, device="cpu"))
    inp = _dit_inputs(S, "cpu")
    times, _ = _dit_cpu_block(S, inp, bp, max(1, min(args.steps, 5)))
    blk = statistics.median(times)
    value = blk * S.blocks * S.steps
    print(json.dumps({
        "impl": "reference", "metric": DIT_METRIC, "value": round(value, 1), "unit": "ms", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(value, 1), "higher_is_better": False,
        "scaling": "strong", "vs_baseline": None, "dtype": DTYPE + " (weights dequantised to bf16, fp32 attention)",
        "data": "synthetic", "config": {"workload": DIT_WORKLOAD, "tensor_parallel_ffn": args.gpus},
        "cpu_baseline": {"value": round(value, 1), "unit": "ms", "cores": cores, "kind": "port",
                         "sample": f"one block at 4146 tokens timed {len(times)}x after 1 warm-up ({blk:.0f} ms median, "
                                   f"oracle/dit_ref.py), extrapolated x {S.blocks} blocks x {S.steps} steps"},
        "e2e": {"value": round(value, 1), "unit": "ms", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0}), flush=True)


def run_dit(args, rank: int, world: int) -> None:
    """The whole DiT denoiser: one "step" of this workload is one denoise pass (4 flow steps x 30
    blocks) over one 4146-token sequence.  With N > 1 the FFN of every block is tensor-parallel over
    the ranks (one NCCL all-reduce per block and step); attention and projections are replicated.
    Strong scaling: the work is fixed."""
    import torch.distributed as dist

    from tybok_b200 import ops
    from tybok_b200.dit import DiTDenoiser, rotary_parts
    from tybok_b200.shapes import DIT_FULL as S
    from tybok_b200.weights import quantize_dit_block, random_dit_block_params

    local = int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    dev = f"cuda:{local}"
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    peaks, peaks_kind = _peaks()
    if os.environ.get("TYBOK_BENCH_DUMP_AFTER"):  # debugging aid: where do this rank's kernels stand after N seconds
        counters = torch.zeros(128, dtype=torch.int32, device=dev)
        ops._lib.load().tybok_debug_set_counters(counters.data_ptr())
        side = torch.cuda.Stream(device=dev)

        def _watch():
            time.sleep(int(os.environ["TYBOK_BENCH_DUMP_AFTER"]) + 2)
            with torch.cuda.stream(side):
                c = counters.cpu().view(16, 8)
            names = {0: "gemm8", 1: "gemm16", 2: "gemm_pair", 6: "prefill128", 7: "qknorm", 8: "norm"}
            print(f"rank {rank} launches {ops.launch_count()} status {int(ops.status_word(torch.device(dev)).cpu().item())} " +
                  " | ".join(f"{n}: in {c[k][0]} setup {c[k][1]} awaited {c[k][2]} main {c[k][3]} out {c[k][4]}"
                             for k, n in names.items()), file=sys.stderr, flush=True)

        threading.Thread(target=_watch, daemon=True).start()
    den = DiTDenoiser([], S, device=dev, rank=rank, world=world)
    from tybok_b200.dit import DiTBlock

    bp0 = None
    for i in range(S.blocks):  # the same seeded weights on every rank; bf16 masters are dropped block by block
        bp = quantize_dit_block(random_dit_block_params(S, seed=i, device=dev))
        if i == 0 and rank == 0 and world == 1 and not args.no_cpu_baseline:  # CPU leg at N = 1 only
            bp0 = {k: v.cpu() for k, v in bp.items()}
        den.blocks.append(DiTBlock(bp, S, device=dev, rank=rank, world=world))
        del bp
    torch.cuda.empty_cache()
    inp = _dit_inputs(S, dev)
    pinned = {k: inp[k].pin_memory() for k in ("x", "context", "t_mods")}
    cos, sin = rotary_parts(inp["freqs"], dev)
    den.prepare_context(inp["context"].to(dev), inp["mask"])
    x_d, tm_d = inp["x"].to(dev), inp["t_mods"].to(dev)

    def one_pass(x):
        return den.denoise(x, tm_d, cos, sin, inp["deltas"])

    sampler = ClockSampler(local)
    sampler.start()
    for _ in range(max(1, min(args.warmup, 3))):
        one_pass(x_d)
    torch.cuda.synchronize()
    launches_per_pass = None
    n0 = ops.launch_count()
    one_pass(x_d)
    launches_per_pass = ops.launch_count() - n0
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    steps = max(1, min(args.steps, 10))
    sampler.mark()
    evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(steps)]
    for e0, e1 in evs:
        e0.record()
        out = one_pass(x_d)
        e1.record()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    clocks = sampler.stop()
    ms = statistics.median(a.elapsed_time(b) for a, b in evs)
    # end to end from host buffers: tokens, context and modulation tables up, the denoised tokens down
    e2e = []
    host_out = torch.empty(inp["x"].shape, dtype=torch.bfloat16).pin_memory()
    for _ in range(min(3, steps)):
        t0 = time.perf_counter()
        xd = pinned["x"].to(dev, non_blocking=True)
        den.prepare_context(pinned["context"].to(dev, non_blocking=True), inp["mask"])
        tm = pinned["t_mods"].to(dev, non_blocking=True)
        host_out.copy_(den.denoise(xd, tm, cos, sin, inp["deltas"]), non_blocking=True)
        torch.cuda.synchronize()
        e2e.append((time.perf_counter() - t0) * 1e3)
    e2e_ms = statistics.median(e2e)
    if world > 1:
        t = torch.tensor([ms, e2e_ms], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms, e2e_ms = float(t[0]), float(t[1])
    ops.check_status()
    flops = _dit_flops(S)
    if rank == 0:
        cpu = parity = None
        if bp0 is not None:
            from oracle import w8_ref

            cores = _all_host_threads()
            times, ref = _dit_cpu_block(S, inp, bp0, 2)
            # Only rank 0 is in this branch: with a sharded FFN a block's forward holds an all-reduce
            # that every rank must enter, so the block-level parity is computed by the N = 1 run only.
            if world == 1:
                got = den.blocks[0].forward(x_d, den.blocks[0].modulations(tm_d[0]), cos, sin, den._cache(S.seq), 0,
                                            den._cross[0], den._ctx_valid)
                parity = {"rel_l2": round(w8_ref.rel_l2(got.float().cpu()[None], ref.float()), 6), "tolerance_rel_l2": 1e-2,
                          "what": "block 0 at 4146 tokens on the GPU vs oracle/dit_ref.block_forward, same weights and inputs"}
            blk = statistics.median(times)
            cpu = {"value": round(blk * S.blocks * S.steps, 1), "unit": "ms", "cores": cores, "kind": "port",
                   "sample": f"one block at 4146 tokens timed {len(times)}x after 1 warm-up ({blk:.0f} ms median), "
                             f"extrapolated x {S.blocks} blocks x {S.steps} steps"}
        tf = flops / ms / 1e9
        peak = peaks.get("bf16_tflops_sustained", peaks["bf16_tflops"]) * world
        print(json.dumps({
            "metric": DIT_METRIC, "value": round(ms, 3), "unit": "ms", "n_gpus": world, "steps": steps,
            "warmup": max(1, min(args.warmup, 3)), "ms_per_step": round(ms, 3), "higher_is_better": False,
            "scaling": "strong", "vs_baseline": None, "dtype": DTYPE + " (norm-fed GEMMs: 2 e4m3 planes with a per-row power-of-two scale, others 3 exact e5m2 planes), bf16 attention",
            "data": "synthetic", "config": {"workload": DIT_WORKLOAD, "tensor_parallel_ffn": world},
            "run": {"cuda_graph": False, "l2": "4.3 GB of e4m3 weights per step exceed the 126 MB L2"},
            "clocks": clocks, "gpu_launches": launches_per_pass * steps,
            "e2e": {"value": round(e2e_ms, 3), "unit": "ms", "h2d_bytes_per_step": sum(v.numel() * 2 for v in pinned.values()),
                    "d2h_bytes_per_step": host_out.numel() * 2},
            "parity": parity,
            "roofline": {"bound": "tensor", "kernel": "whole pass (w8_gemm_kernel pairs + attention_prefill_kernel<128>)",
                         "achieved": round(tf, 1), "peak": peak, "unit": "TFLOP/s", "frac": round(tf / peak, 4),
                         "traffic": None, "peak_source": peaks_kind + " (sustained bf16 x ranks; only the FFN is sharded)",
                         "flops_per_pass": flops},
            "cpu_baseline": cpu, "finite": bool(torch.isfinite(out.float()).all()),
            # the denoised tokens' mean magnitude: equal across N up to the all-reduce's summation order
            "out_abs_mean": round(float(out.float().abs().mean()), 6),
        }), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()



def run_profile_case(args) -> None:
    """Small fixed workloads for profiler captures: a few launches over a few hundred MB.

    ``--workload gemm --m 50 --n 1024 --k 4096 [--launches 6] [--gated]``: the W8 GEMM over rotating
    weight copies whose total exceeds the 126 MB L2, so the DRAM counters of a captured launch mean
    what they mean inside a chunk.  ``--workload attention --tokens 50 --prefix 544 [--head-dim 256]``:
    six launches of the attention kernel."""
    from tybok_b200 import ops

    dev = torch.device("cuda")
    if args.workload == "gemm":
        n = 2 * args.n if args.gated else args.n
        nbuf = max(2, int(260e6 // (n * args.k)) + 1)
        ws = [torch.randint(0, 120, (n, args.k), dtype=torch.uint8, device=dev).view(torch.float8_e4m3fn) for _ in range(nbuf)]
        sc = torch.rand(n, device=dev)
        x = torch.randn(args.m, args.k, device=dev).to(torch.bfloat16)
        xp = ops.split3(x, 4)
        if args.two_plane:
            x2, rs = ops.norm_planes2(x, ops.NORM_RMS, torch.ones(args.k, device=dev))
        for i in range(nbuf + args.launches):
            if args.two_plane:
                ops.w8x2_gemm(x2, rs, ws[i % nbuf], sc, epilogue=ops.EPI_GEGLU_PACKED if args.gated else ops.EPI_NONE,
                              out_bf16=not args.gated, out_planes=args.gated)
            elif args.gated:
                ops.w8x3_geglu_packed(xp, 4, ws[i % nbuf], sc, out_bf16=False, out_planes=True)
            else:
                ops.w8x3_linear(xp, 4, ws[i % nbuf], sc)
        launches = nbuf + args.launches + 1 + int(args.two_plane)
        what = {"workload": f"gemm M={args.m} N={args.n} K={args.k} gated={args.gated} two_plane={args.two_plane}",
                "weight_copies": nbuf}
    else:
        d, lk, heads = args.head_dim, args.prefix + args.tokens, args.heads
        kv_heads = heads if args.mha else 1
        kc = torch.randn(1, kv_heads, lk + 8, d, device=dev).to(torch.bfloat16)
        vc = torch.randn(1, kv_heads, lk + 8, d, device=dev).to(torch.bfloat16)
        q = torch.randn(args.tokens, heads * d, device=dev).to(torch.bfloat16)
        for _ in range(args.launches):
            ops.attention(q, kc, vc, None, tokens=args.tokens, keys=lk, scale=d**-0.5, out_bf16=False, out_planes=True)
        launches = args.launches
        what = {"workload": f"attention tokens={args.tokens} keys={lk} heads={heads} kv_heads={kv_heads} head_dim={d}"}
    ops.check_status()
    print(json.dumps({"metric": "profile_case", "config": what, "gpu_launches": launches}), flush=True)


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--no-cpu-baseline", action="store_true", help="skip the CPU oracle leg (and with it the parity field)")
    ap.add_argument("--no-extras", action="store_true", help="skip the W8 sweep, the batch sweep and the tensor-parallel extra")
    ap.add_argument("--no-overlap", action="store_true", help="run the first denoise step after the prefix, not behind it")
    ap.add_argument("--vision-precision", default="fp16", choices=["fp16", "tf32", "bf16", "fp32"],
                    help="SigLIP tower: fp16 operands with an fp32 residual stream (default), fp32 activations with TF32 "
                         "GEMMs, bf16 operands, or plain fp32")
    ap.add_argument("--workload", default="pi05_chunk", choices=["pi05_chunk", "dit", "dit_ffn", "gemm", "attention"])
    for name, default in (("m", 50), ("n", 16384), ("k", 2048), ("launches", 6), ("tokens", 50), ("prefix", 544),
                          ("head-dim", 256), ("heads", 8)):
        ap.add_argument(f"--{name}", type=int, default=default)
    ap.add_argument("--gated", action="store_true")
    ap.add_argument("--mha", action="store_true")
    ap.add_argument("--no-fold", action="store_true",
                    help="pi05_chunk: run the expert's AdaRMS norms as kernels instead of folding them into the GEMMs around them")
    ap.add_argument("--two-plane", action="store_true", help="gemm workload: the two-plane e4m3 activation form")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", 0))
    world = int(os.environ.get("WORLD_SIZE", 1))
    if os.environ.get("TYBOK_BENCH_DUMP_AFTER"):  # debugging aid: python stacks of every thread after N seconds
        import faulthandler

        faulthandler.dump_traceback_later(int(os.environ["TYBOK_BENCH_DUMP_AFTER"]), exit=False)
    if args.impl == "reference":
        (run_dit_reference if args.workload == "dit" else run_reference)(args, rank)
        return
    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device -- the product path has no CPU fallback (use --impl reference "
                         "for the CPU oracle timing)")
    if args.workload in ("gemm", "attention"):
        run_profile_case(args)
    elif args.workload == "dit_ffn":
        run_dit_ffn(args, rank, world)
    elif args.workload == "dit":
        run_dit(args, rank, world)
    else:
        run_ours(args, rank, world)


if __name__ == "__main__":
    main()
