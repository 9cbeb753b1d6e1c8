"""Per-kernel timing of the bandwidth-bound kernels of the path (quant, gathers, reductions) at benchmark sizes.

  python -m eps_b200.kernel_bench [--rows 32768] [--hidden 7168] [--iters 20]

Prints one JSON line per kernel with the algorithmic bytes, the CUDA-event time and GB/s, then the plan kernels'
times at cluster sizes 1 and 8.  Inputs are larger than
L2 (126 MB) at the default sizes.  This is the command the ncu summaries of these kernels were taken from.
"""
from __future__ import annotations

import argparse
import json

import torch

from . import ops


def _time(fn, iters):
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--rows", type=int, default=32768)
    ap.add_argument("--hidden", type=int, default=7168)
    ap.add_argument("--topk", type=int, default=8)
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--experts", type=int, default=256)
    a = ap.parse_args()
    dev = torch.device("cuda")
    R, H, k = a.rows, a.hidden, a.topk
    T = R // k
    out = []

    x = torch.randn((R, H), device=dev, dtype=torch.bfloat16)
    q = torch.empty((R, H), dtype=torch.uint8, device=dev)
    s = torch.empty((R, H // 128), dtype=torch.float32, device=dev)
    ms = _time(lambda: ops.per_token_group_quant_fp8(x, out=q, out_scales=s), a.iters)
    out.append(("quant_1x128", R * H * (2 + 1 + 4 / 128), ms))

    ms = _time(lambda: ops.per_token_group_dequant_fp8(q, s), a.iters)
    out.append(("dequant_1x128", R * H * (2 + 1 + 4 / 128), ms))

    perm = torch.randperm(R, device=dev, dtype=torch.int32)
    dst = torch.empty_like(q)
    ms = _time(lambda: ops.gather_rows(q, dst, perm), a.iters)
    out.append(("gather_rows(e4m3 rows, random permutation)", 2.0 * R * H, ms))

    # expand-for-GEMM shape: T source rows each read k times (L2 serves the repeats)
    src = q[:T]
    m2 = (torch.randint(0, T, (R,), device=dev, dtype=torch.int32) * k)
    ms = _time(lambda: ops.gather_rows(src, dst, m2, map_div=k), a.iters)
    out.append(("gather_rows(expand for GEMM, k reads per source row)", 1.0 * R * H + T * H, ms))

    # single-rank combine: T output rows, k bf16 rows each
    y = torch.randn((R, H), device=dev, dtype=torch.bfloat16)
    red = torch.randperm(R, device=dev, dtype=torch.int32).reshape(T, k).contiguous()
    glob = torch.arange(T, device=dev, dtype=torch.int32)
    ret = torch.tensor([T], device=dev, dtype=torch.int32)
    o = torch.empty((T, H), dtype=torch.bfloat16, device=dev)
    ms = _time(lambda: ops.reduce_ep1(y, red, glob, ret, 1, k, o), a.iters)
    out.append(("reduce_ep1(k rows -> 1)", (R + T) * H * 2.0, ms))

    send = torch.empty((T, H), dtype=torch.bfloat16, device=dev)
    ms = _time(lambda: ops.local_reduce(y, red, ret, k, 1, 1, -1, send), a.iters)
    out.append(("local_reduce(fp32 accumulate)", (R + T) * H * 2.0, ms))

    w = torch.rand((T, k), device=dev)
    ms = _time(lambda: ops.fastep_reduce(y, x[:T], w, red.reshape(-1), o), a.iters)
    out.append(("fastep_reduce", (R + T) * H * 2.0, ms))

    gu = torch.randn((R // 2, 4096), device=dev, dtype=torch.bfloat16)
    act = torch.empty((R // 2, 2048), device=dev, dtype=torch.bfloat16)
    ms = _time(lambda: ops.silu_run(gu, act), a.iters)
    out.append(("silu_run (unfused)", (R // 2) * 2048 * 6.0, ms))

    for name, nbytes, ms in out:
        print(json.dumps({"kernel": name, "algorithmic_bytes": nbytes, "ms": ms, "GB_per_s": nbytes / ms / 1e6}))

    xn = torch.randn((R, H), device=dev, dtype=torch.bfloat16)
    scn = torch.ones(H, device=dev, dtype=torch.bfloat16)
    on = torch.empty_like(xn)
    ms = _time(lambda: ops.rms_norm(xn, scn, 1e-6, out=on), a.iters)
    print(json.dumps({"kernel": "rms_norm (bf16 rows)", "algorithmic_bytes": 4.0 * R * H, "ms": ms,
                      "GB_per_s": 4.0 * R * H / ms / 1e6}))

    # router: T tokens x `--experts` logits, 8 groups of which 4 stay, top-k
    logits = torch.randn((T, a.experts), device=dev, dtype=torch.bfloat16)
    rbias = torch.randn(a.experts, device=dev) * 0.1
    ms = _time(lambda: ops.topk_sigmoid(logits, rbias, 8, 4, k, 2.5), a.iters)
    print(json.dumps({"kernel": "router topk_sigmoid", "tokens": T, "experts": a.experts, "top_k": k,
                      "algorithmic_bytes": T * (a.experts * 2 + k * 8), "us": round(ms * 1e3, 1)}))

    # plan kernels (latency-bound): one rank's routing of T tokens over `--experts` experts, and the expert-side
    # plans of the W * T tokens a rank of an EP group of W receives, at cluster sizes 1 and 8
    E = a.experts
    g = torch.Generator(device="cpu").manual_seed(1)
    for W, Tt in ((1, T), (8, T)):
        idx = torch.stack([torch.randperm(E, generator=g)[:k] for _ in range(Tt)]).to(torch.int32).to(dev)
        wts = torch.rand((Tt, k), device=dev)
        R = Tt * W if W == 1 else int(Tt * W * 0.66)          # tokens received: all of them, or ~2/3 at W = 8
        ridx = torch.randint(0, E, (R, k), dtype=torch.int32, device=dev)
        recv_incl = torch.tensor([R * (i + 1) // W for i in range(W)], dtype=torch.int32, device=dev)
        for c in (1, 8):
            ms_s = _time(lambda: ops.source_plans(idx, wts, E, W, 1, max_cluster=c), a.iters)
            ms_e = _time(lambda: ops.expert_plans(ridx, recv_incl, k, 0, E // W, W, 1, Tt, R, max_cluster=c), a.iters)
            print(json.dumps({"kernel": "plans", "tokens": Tt, "experts": E, "top_k": k, "ep_world": W,
                              "received_tokens": R, "max_cluster": c, "source_plans_us": round(ms_s * 1e3, 1),
                              "expert_plans_us": round(ms_e * 1e3, 1)}))


if __name__ == "__main__":
    main()
