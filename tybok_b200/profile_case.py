"""Small fixed workloads for profiler captures (a few launches, a few hundred MB on the device).

    python -m tybok_b200.profile_case gemm --m 50 --n 16384 --k 2048 [--launches 6]
    python -m tybok_b200.profile_case attention --tokens 50 --prefix 544

``gemm`` runs the W8 GEMM over rotating weight copies whose total exceeds the 126 MB L2, so the
DRAM counters of a captured launch mean what they mean inside a real chunk.
"""

from __future__ import annotations

import argparse

import torch

from . import ops


def run_gemm(m: int, n: int, k: int, launches: int, dual: bool) -> None:
    dev = torch.device("cuda")
    nbuf = max(2, int(260e6 // (n * k)) + 1)
    ws = [torch.randint(0, 120, (n, k), dtype=torch.uint8, device=dev).view(torch.float8_e4m3fn) for _ in range(nbuf)]
    sc = torch.rand(n, device=dev)
    xp = ops.split3(torch.randn(m, k, device=dev).to(torch.bfloat16), 4)
    for i in range(nbuf + launches):
        if dual:
            ops.w8x3_geglu(xp, 4, ws[i % nbuf], sc, ws[(i + 1) % nbuf], sc)
        else:
            ops.w8x3_linear(xp, 4, ws[i % nbuf], sc)
    ops.check_status()


def run_attention(tokens: int, prefix: int, heads: int = 8) -> None:
    dev = torch.device("cuda")
    d, lk = 256, prefix + tokens
    kc = torch.randn(1, 1, lk + 8, d, device=dev).to(torch.bfloat16)
    vc = torch.randn(1, 1, lk + 8, d, device=dev).to(torch.bfloat16)
    q = torch.randn(tokens, heads * d, device=dev).to(torch.bfloat16)
    for _ in range(6):
        ops.attention(q, kc, vc, None, tokens=tokens, keys=lk, scale=d**-0.5, out_bf16=False, out_planes=True)
    ops.check_status()


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("case", choices=["gemm", "attention"])
    ap.add_argument("--m", type=int, default=50)
    ap.add_argument("--n", type=int, default=16384)
    ap.add_argument("--k", type=int, default=2048)
    ap.add_argument("--launches", type=int, default=6)
    ap.add_argument("--dual", action="store_true")
    ap.add_argument("--tokens", type=int, default=50)
    ap.add_argument("--prefix", type=int, default=544)
    a = ap.parse_args()
    if a.case == "gemm":
        run_gemm(a.m, a.n, a.k, a.launches, a.dual)
    else:
        run_attention(a.tokens, a.prefix)


if __name__ == "__main__":
    main()
