"""Benchmark of the fp8 hot path: pi0.5-shaped action-chunk latency on B200 (BASELINE config 2).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--batch B]
    torchrun --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...

One "step" = one action chunk (prefix prefill + 10 denoise steps) of the pi0.5-shaped random-init
fp8 policy on synthetic inputs.  ``value`` is the p50 of K CUDA-event-timed graph replays with
inputs resident in HBM; ``e2e`` is the same chunk through ``engine.predict_action_chunk`` from
host frames (pinned H2D of images/tokens/noise and D2H of the chunk inside the timed region).
With N > 1 every rank runs an independent replica (no data-path collective); the time is the
max over ranks.  ``--impl reference`` times the CPU oracle (the reference's eager torch path on
dequantised weights) on the host cores.  Prints one JSON line on rank 0.
"""

from __future__ import annotations

import argparse
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


def _peaks() -> tuple[dict, str]:
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        return json.load(open(path)), "measured"
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}, "fallback"


class ClockSampler(threading.Thread):
    """Samples SM clock and throttle reasons of one GPU through NVML while the timed region runs."""

    def __init__(self, index: int):
        super().__init__(daemon=True)
        self.index, self.samples, self.reasons, self.max_mhz, self._halt = index, [], set(), None, threading.Event()

    def run(self):
        try:
            import pynvml as nv

            nv.nvmlInit()
            h = nv.nvmlDeviceGetHandleByIndex(self.index)
            self.max_mhz = nv.nvmlDeviceGetMaxClockInfo(h, nv.NVML_CLOCK_SM)
            names = {nv.nvmlClocksEventReasonHwSlowdown: "hw_slowdown",
                     nv.nvmlClocksEventReasonHwThermalSlowdown: "hw_thermal_slowdown",
                     nv.nvmlClocksEventReasonSwThermalSlowdown: "sw_thermal_slowdown",
                     nv.nvmlClocksEventReasonSwPowerCap: "sw_power_cap"}
            while not self._halt.is_set():
                self.samples.append(nv.nvmlDeviceGetClockInfo(h, nv.NVML_CLOCK_SM))
                mask = nv.nvmlDeviceGetCurrentClocksEventReasons(h)
                self.reasons |= {n for bit, n in names.items() if mask & bit}
                time.sleep(0.02)
        except Exception as e:  # NVML missing: report that instead of clocks
            self.reasons.add(f"nvml_unavailable:{type(e).__name__}")

    def stop(self) -> dict:
        self._halt.set()
        self.join(timeout=2)
        med = statistics.median(self.samples) if self.samples else None
        return {"sm_mhz": med, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons)}


def _synthetic_frame(engine, seed: int):
    spec = engine.describe()
    g = torch.Generator().manual_seed(seed)
    images = {c: torch.rand(3, spec["resize"][1], spec["resize"][0], generator=g).pin_memory() for c in spec["cameras"]}
    frame = engine.make_frame(images, torch.randn(8, generator=g), "pick up the red block")
    s = engine.config.shape
    frame["observation.language.tokens"] = torch.randint(0, s.vocab, (s.lang_len,), generator=g)
    frame["observation.language.attention_mask"] = torch.ones(s.lang_len, dtype=torch.bool)
    return frame


NCU_TRAFFIC_DOWN_PROJ = 4859136  # bytes per launch, from the committed ncu summary


def _gemm_roofline(engine, peaks, peaks_kind) -> dict:
    """Roofline of the dominant kernel (``w8_gemm_kernel``), measured live: every GEMM call
    signature of one chunk is replayed as a CUDA graph of back-to-back launches over rotating
    weight copies (> 3x L2, so weights stream from HBM as they do inside the chunk) and timed
    with CUDA events on the launching stream.  Algorithmic bytes per launch =
    nw*(N*K + 4N) + 2*M*K + 2*M*N (nw = 2 for the gated form), flops = 2*nw*M*N*K.
    ``achieved`` aggregates the action-expert launches (M = 50*batch, HBM-bound, 720 of the 792
    launches of a chunk); the prefix launches (M = 544*batch, tensor-bound) are reported beside."""
    from tybok_b200 import ops

    s = engine.config.shape
    dev = engine.device
    b = engine.batch_size

    def shapes(spec, m, layers, reps):
        hd, kvd = spec.num_heads * spec.head_dim, spec.num_kv_heads * spec.head_dim
        return [("qkv", m, hd + 2 * kvd, spec.width, 1, layers * reps), ("o", m, spec.width, hd, 1, layers * reps),
                ("geglu", m, spec.mlp_dim, spec.width, 2, layers * reps),
                ("down", m, spec.width, spec.mlp_dim, 1, layers * reps)]

    groups = {"expert": shapes(s.expert, b * s.chunk, s.expert.depth, s.steps),
              "prefix": shapes(s.vlm, b * s.prefix_len, s.vlm.depth, 1)}
    out = {}
    for gname, lst in groups.items():
        rows = []
        for name, m, n, k, nw, count in lst:
            nbuf = min(48, max(4, int(400e6 // (nw * n * k)) + 1))
            # the gated form streams gate and up as one interleaved [2N, K] matrix
            ws = [[torch.randint(0, 120, (nw * n, k), dtype=torch.uint8, device=dev).view(torch.float8_e4m3fn)]
                  for _ in range(nbuf)]
            sc = torch.rand(nw * n, device=dev)
            xp = ops.split3(torch.randn(m, k, device=dev).to(torch.bfloat16), 4)
            res = torch.randn(m, n, device=dev).to(torch.bfloat16)

            def call(i):
                w = ws[i % nbuf]
                if nw == 2:
                    return ops.w8x3_geglu_packed(xp, 4, w[0], sc, out_bf16=False, out_planes=True)
                if name == "qkv":
                    return ops.w8x3_linear(xp, 4, w[0], sc)
                return ops.w8x3_linear(xp, 4, w[0], sc, epilogue=ops.EPI_RESIDUAL, residual=res)

            for i in range(3):
                call(i)
            torch.cuda.synchronize()
            iters = 2 * nbuf
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
            byts = nw * (n * k + 4 * n) + 2 * m * k + 2 * m * n
            rows.append({"gemm": name, "M": m, "N": n, "K": k, "nw": nw, "us": round(best, 2), "count": count,
                         "GBps": round(byts / best / 1e3, 1), "TFps": round(2.0 * nw * m * n * k / best / 1e6, 1),
                         "bytes": byts, "flops": 2.0 * nw * m * n * k})
            del ws, graph
        out[gname] = rows
    torch.cuda.empty_cache()

    def agg(rows, key):
        return sum(r["count"] * r[key] for r in rows) / sum(r["count"] * r["us"] for r in rows)

    hbm = agg(out["expert"], "bytes") / 1e3  # bytes/us -> GB/s
    tc = agg(out["prefix"], "flops") / 1e6  # flops/us -> TFLOP/s
    strip = lambda rows: [{k: v for k, v in r.items() if k not in ("bytes", "flops")} for r in rows]  # noqa: E731
    return {
        "bound": "hbm", "kernel": "w8_gemm_kernel (action-expert launches, M=%d)" % (b * s.chunk),
        "achieved": round(hbm, 1), "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": round(hbm / peaks["hbm_gbs"], 4),
        # dram__bytes_read + write of one captured launch of the expert down projection (M=50, N=1024,
        # K=4096; profiles/w8_gemm_m50_n1024_k4096.md) against its 4,710,400 algorithmic bytes
        "traffic": NCU_TRAFFIC_DOWN_PROJ if (b * s.chunk, s.expert.width, s.expert.mlp_dim) == (50, 1024, 4096) else None,
        "traffic_case": "M=50 N=1024 K=4096: 4859136 B measured (ncu) vs 4710400 B algorithmic per launch",
        "peak_source": peaks_kind, "per_shape": strip(out["expert"]),
        "prefix": {"bound": "tensor", "achieved": round(tc, 1), "peak": peaks["bf16_tflops"], "unit": "TFLOP/s",
                   "frac": round(tc / peaks["bf16_tflops"], 4), "per_shape": strip(out["prefix"])},
    }


def _cpu_chunk_times(reps: int, seed: int = 0) -> tuple[list[float], dict]:
    """Time the CPU oracle (reference eager path on dequantised weights) on the full config."""
    from oracle import pi05_ref
    from tybok_b200.shapes import PI05_FULL
    from tybok_b200.weights import quantize_hot_linears, random_pi05_params

    # every host thread this process may use (a torchrun launch sets OMP_NUM_THREADS=1 for its ranks)
    try:
        torch.set_num_threads(max(1, len(os.sched_getaffinity(0))))
    except (AttributeError, RuntimeError):
        torch.set_num_threads(max(1, os.cpu_count() or 1))
    dev = "cuda" if torch.cuda.is_available() else "cpu"  # weights are generated where it is fast
    params = quantize_hot_linears(random_pi05_params(PI05_FULL, seed=seed, device=dev), PI05_FULL)
    params = {k: v.cpu() for k, v in params.items()}
    if dev == "cuda":
        torch.cuda.empty_cache()
    s = PI05_FULL
    g = torch.Generator().manual_seed(seed)
    images = [torch.rand(1, 3, 224, 224, generator=g) * 2 - 1 for _ in range(s.n_cams)]
    img_masks = [torch.ones(1, dtype=torch.bool) for _ in range(s.n_cams)]
    tokens = torch.randint(0, s.vocab, (1, s.lang_len), generator=g)
    masks = torch.ones(1, s.lang_len, dtype=torch.bool)
    noise = torch.randn(1, s.chunk, s.max_action_dim, generator=g)
    # dequantise once (what the reference's loader does), then time the unmodified eager math
    from oracle import w8_ref
    deq = {}
    for k, v in params.items():
        if k.endswith(".scale_weight"):
            continue
        deq[k] = w8_ref.dequant_w8(v, params[k[: -len("weight")] + "scale_weight"]) if v.dtype == torch.float8_e4m3fn else v
    del params
    times = []
    pi05_ref.sample_actions(deq, s, images, img_masks, tokens, masks, noise)  # warm-up
    for _ in range(reps):
        t0 = time.perf_counter()
        pi05_ref.sample_actions(deq, s, images, img_masks, tokens, masks, noise)
        times.append((time.perf_counter() - t0) * 1e3)
    info = {"cores": torch.get_num_threads(), "nproc": os.cpu_count(), "torch": torch.__version__}
    return times, info


def run_reference(args, rank: int) -> None:
    if rank != 0:
        return
    times, info = _cpu_chunk_times(max(1, args.steps))
    p50 = statistics.median(times)
    line = {
        "impl": "reference", "metric": METRIC, "value": round(p50, 2), "unit": "ms", "n_gpus": args.gpus,
        "steps": len(times), "warmup": 1, "ms_per_step": round(sum(times) / len(times), 2), "higher_is_better": False,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16 activations x e4m3 weights dequantised to bf16, fp32 accumulate",
        "data": "synthetic", "config": {"workload": WORKLOAD, "batch": 1},
        "cpu_baseline": {"value": round(p50, 2), "unit": "ms", "cores": info["cores"], "kind": "port",
                         "sample": f"{len(times)} full chunks of the config (oracle/pi05_ref.py, torch {info['torch']}, "
                                   f"{info['nproc']} logical CPUs)"},
        "e2e": {"value": round(p50, 2), "unit": "ms", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def run_ours(args, rank: int, world: int) -> None:
    import torch.distributed as dist

    from tybok_b200 import ops
    from tybok_b200.engine import PI05B200Engine

    local = int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    peaks, peaks_kind = _peaks()

    l0 = ops.launch_count()
    engine = PI05B200Engine(f"synthetic:pi05_full@{rank}", device=f"cuda:{local}", graph=False, warmup=True,
                            seed=rank, batch_size=args.batch, overlap=not args.no_overlap)
    l1 = ops.launch_count()
    engine._capture()
    launches_per_chunk = ops.launch_count() - l1
    launches_per_chunk //= 3  # two warm-up passes + the captured pass
    del l0

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    graph = engine._graph
    for _ in range(max(3, args.warmup)):
        graph.replay()
    barrier()
    sampler = ClockSampler(local)
    sampler.start()
    evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(args.steps)]
    t_all0, t_all1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t_all0.record()
    for e0, e1 in evs:
        e0.record()
        graph.replay()
        e1.record()
    t_all1.record()
    barrier()
    clocks = sampler.stop()
    per = sorted(a.elapsed_time(b) for a, b in evs)
    p50 = statistics.median(per)
    total_ms = t_all0.elapsed_time(t_all1)
    if world > 1:
        t = torch.tensor([p50, total_ms], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        p50, total_ms = float(t[0]), float(t[1])

    # end to end through the public call: host frame -> numpy chunk
    frames = [_synthetic_frame(engine, 100 + i) for i in range(4)]
    for i in range(3):
        engine.predict_action_chunk(frames[i % 4])
    barrier()
    e2e = []
    for i in range(args.steps):
        t0 = time.perf_counter()
        engine.predict_action_chunk(frames[i % 4])
        e2e.append((time.perf_counter() - t0) * 1e3)
    e2e_p50 = statistics.median(e2e)
    if world > 1:
        t = torch.tensor([e2e_p50], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_p50 = float(t[0])
    s = engine.config.shape
    h2d = s.n_cams * 3 * 224 * 224 * 4 + s.n_cams + s.lang_len * 9 + s.chunk * s.max_action_dim * 4
    d2h = s.chunk * engine.config.action_dim * 4

    line = None
    if rank == 0:
        roof = _gemm_roofline(engine, peaks, peaks_kind) if world == 1 else None
        ops.check_status()
        cpu = None
        if world == 1 and not args.no_cpu_baseline:
            del engine
            torch.cuda.empty_cache()
            times, info = _cpu_chunk_times(2)
            cpu = {"value": round(statistics.median(times), 1), "unit": "ms", "cores": info["cores"], "kind": "port",
                   "sample": f"2 full chunks of the same config after 1 warm-up (oracle/pi05_ref.py, {info['nproc']} logical CPUs)"}
        line = {
            "metric": METRIC, "value": round(p50, 4), "unit": "ms", "n_gpus": world, "steps": args.steps,
            "warmup": max(3, args.warmup), "ms_per_step": round(total_ms / args.steps, 4), "higher_is_better": False,
            "scaling": "weak", "vs_baseline": None, "dtype": "e4m3 weights x bf16 activations (3 exact e5m2 planes), fp32 accumulate",
            "data": "synthetic",
            "config": {"workload": WORKLOAD, "batch_per_gpu": args.batch, "replicas": world, "cuda_graph": True, "overlap_step0": not args.no_overlap,
                       "l2": "weights streamed per chunk (3.4 GB) exceed the 126 MB L2"},
            "chunks_per_s": round(world * args.batch / (total_ms / args.steps) * 1e3, 2),
            "clocks": clocks, "gpu_launches": launches_per_chunk * args.steps,
            "e2e": {"value": round(e2e_p50, 4), "unit": "ms", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
            "roofline": roof, "cpu_baseline": cpu,
        }
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def run_dit_ffn(args, rank: int, world: int) -> None:
    """Secondary workload (BASELINE config 3): the FFN tail of one fastWAM-class DiT block
    (hidden 3072, ffn 14336, 4096+50 tokens), tensor-parallel over N GPUs with one NCCL
    all-reduce per call (strong scaling: the work is fixed, the weights are sharded)."""
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
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    sampler = ClockSampler(local)
    sampler.start()
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
            "scaling": "strong", "vs_baseline": None, "dtype": "e4m3 weights x bf16 activations, fp32 accumulate",
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


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-overlap", action="store_true", help="run the first denoise step after the prefix, not behind it")
    ap.add_argument("--workload", default="pi05_chunk", choices=["pi05_chunk", "dit_ffn"])
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", 0))
    world = int(os.environ.get("WORLD_SIZE", 1))
    if args.impl == "reference":
        run_reference(args, rank)
        return
    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device -- the product path has no CPU fallback (use --impl reference "
                         "for the CPU oracle timing)")
    if args.workload == "dit_ffn":
        run_dit_ffn(args, rank, world)
        return
    run_ours(args, rank, world)


if __name__ == "__main__":
    main()
