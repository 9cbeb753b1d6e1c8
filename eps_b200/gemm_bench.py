"""Timing of the FP8 grouped GEMM alone, at benchmark shapes.

  python -m eps_b200.gemm_bench [--mode down|plain|gateup|bf16] [--experts 256] [--rows 128] [--jitter 0]
                                [--N 7168] [--K 2048] [--iters 10] [--single]

--rows is the mean row count per expert, --jitter the standard deviation of a seeded normal spread around it
(the routed layer at 4096 tokens, top-8, 256 experts has 128 +- 11).  --mode bf16 times the bf16 x bf16 grouped
GEMM (the reference's aok_run), the others the FP8 block-scaled one.  Prints one JSON line: CUDA-event time
per launch, weight bytes per second and FLOP/s.  This is the command the ncu summaries of the GEMM kernels
were taken from.
"""
from __future__ import annotations

import argparse
import json

import torch

from . import ops

MODES = {"plain": ops.GEMM_PLAIN, "gateup": ops.GEMM_GATEUP, "down": ops.GEMM_DOWN, "bf16": -1}


def make_problem(experts, rows, jitter, N, K, dev, seed=1):
    g = torch.Generator().manual_seed(seed)
    if jitter:
        r = (rows + torch.randn(experts, generator=g) * jitter).round().clamp(min=0).int()
    else:
        r = torch.full((experts,), rows, dtype=torch.int32)
    D = int(r.sum())
    excl = torch.cat([torch.zeros(1, dtype=torch.int32), r.cumsum(0).int()]).to(dev).contiguous()
    A = torch.randint(0, 120, (D, K), dtype=torch.uint8, device=dev)
    a_s = torch.rand((D, K // 128), device=dev) + 0.5
    B = torch.randint(0, 120, (experts, N, K), dtype=torch.uint8, device=dev)
    b_s = torch.rand((experts, N // 128, K // 128), device=dev) + 0.5
    return D, excl, A, a_s, B, b_s


def run(mode, experts, rows, jitter, N, K, iters, single=False):
    dev = torch.device("cuda")
    D, excl, A, a_s, B, b_s = make_problem(experts, rows, jitter, N, K, dev)
    if mode == -1:
        A = torch.randn((D, K), device=dev).to(torch.bfloat16)
        B = (torch.randn((experts, N, K), device=dev) * 0.05).to(torch.bfloat16)
    status = torch.zeros(4, dtype=torch.int32, device=dev)
    if mode == ops.GEMM_GATEUP:
        out = torch.empty((D, N // 2), dtype=torch.uint8, device=dev)
        outs = torch.empty((D, N // 256), device=dev)
    else:
        out = torch.empty((D, N), dtype=torch.bfloat16, device=dev)
        outs = None
    row_w = torch.rand(D, device=dev) if mode == ops.GEMM_DOWN else None

    def launch():
        if mode == -1:
            ops.grouped_gemm_bf16(A, B, excl, out=out, status=status, rows_hint=1 if single else D)
        else:
            ops.grouped_gemm_fp8(mode, A, a_s, B, b_s, excl, out=out, out_scales=outs, row_w=row_w, status=status)

    for _ in range(3):
        launch()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        launch()
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / iters
    st = status.tolist()
    if st[0] != 0:
        raise RuntimeError(f"bounded wait expired in the GEMM kernel: code {st[0]} on CTA {st[1]}")
    return {"kernel": "grouped_gemm_bf16" if mode == -1 else "grouped_gemm_fp8", "experts": experts, "rows_total": D,
            "rows_mean": rows, "rows_sd": jitter, "N": N, "K": K, "ms": round(ms, 4),
            "weight_GBps": round(experts * N * K * (2 if mode == -1 else 1) / ms / 1e6, 1),
            "TFLOPs": round(2.0 * D * N * K / ms / 1e9, 1)}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--mode", choices=sorted(MODES), default="down")
    ap.add_argument("--experts", type=int, default=256)
    ap.add_argument("--rows", type=int, default=128)
    ap.add_argument("--jitter", type=float, default=0.0)
    ap.add_argument("--N", type=int, default=7168)
    ap.add_argument("--K", type=int, default=2048)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--single", action="store_true", help="bf16: 128-row tiles on single CTAs even for large experts")
    a = ap.parse_args()
    print(json.dumps(run(MODES[a.mode], a.experts, a.rows, a.jitter, a.N, a.K, a.iters, a.single)))


if __name__ == "__main__":
    main()
