"""Per-kernel timing of the bandwidth-bound kernels of the path (quant, gathers, reductions) at benchmark sizes.

  python -m eps_b200.kernel_bench [--rows 32768] [--hidden 7168] [--iters 20]

Prints one JSON line per kernel with the algorithmic bytes, the CUDA-event time and GB/s, then the plan kernels'
times at cluster sizes 1 and 8, then the device-side exchange's put and reduce-put kernels with 8 ranks emulated on
this GPU.  Inputs are larger than L2 (126 MB) at the default sizes.  This is the command the ncu summaries of these kernels were taken from.
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
    ap.add_argument("--no-exchange", action="store_true", help="skip the 8-rank exchange emulation (needs ~9 GB)")
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


    if not a.no_exchange:
        exchange_bench(dev, 8, T, E, k, H, max(a.iters // 4, 3))


def exchange_bench(dev, W, T, E, k, H, iters):
    """The device-side exchange at benchmark size with all W ranks emulated on THIS GPU: W exchange objects whose
    regions all live here, every phase run for all ranks before the next (so each flag is set before a kernel waits
    for it).  Times rank 0's permute-on-send put and its fused local-reduce + store; the stores land in local HBM, so
    the figures bound what the kernels can feed into NVLink (770 GB/s per direction measured on this pool)."""
    import ctypes

    from . import _lib
    from ._lib import call, ptr, stream_ptr

    sd, EL = H // 128, E // W
    nbytes = ctypes.c_int64()
    call("epsb_exchange_region_bytes", W, T, 1, k, H, 1, sd, ctypes.byref(nbytes))
    regions, xs_ = [], []
    for _ in range(W):
        pr = ctypes.c_void_p()
        call("epsb_symm_alloc", nbytes.value, ctypes.byref(pr), (ctypes.c_uint8 * 64)())
        regions.append(pr.value)
    for r in range(W):
        x = ctypes.c_void_p()
        call("epsb_exchange_create", r, W, T, 1, k, H, 1, sd, (ctypes.c_void_p * W)(*regions), ctypes.byref(x))
        xs_.append(x)
    try:
        g = torch.Generator(device="cpu").manual_seed(7)
        idx = [torch.stack([torch.randperm(E, generator=g)[:k] for _ in range(T)]).to(torch.int32).to(dev)
               for _ in range(W)]
        wts = [torch.rand((T, k), device=dev) for _ in range(W)]
        xq = torch.randint(0, 255, (T, H), dtype=torch.uint8, device=dev)
        xsc = torch.rand((T, sd), device=dev)
        status = torch.zeros(4, dtype=torch.int32, device=dev)
        src = [ops.source_plans(idx[r], wts[r], E, W, 1) for r in range(W)]
        rows = T * W
        y_rows = (T * k * 3) // 2   # a rank computes about T * k rows of the W * T * k routed ones
        y = torch.randn((y_rows, H), device=dev, dtype=torch.bfloat16)
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(4)]
        t_put = t_red = 0.0
        sent = ret_rows = gemm_rows = 0
        for it in range(iters + 2):
            e = ctypes.c_int()
            for r in range(W):
                call("epsb_exchange_begin", xs_[r], ctypes.byref(e))
                call("epsb_exchange_publish_plans", xs_[r], ptr(src[r][1]), ptr(src[r][3]), 1, stream_ptr())
            recv_incl = []
            for r in range(W):
                ri = torch.empty((W,), dtype=torch.int32, device=dev)
                call("epsb_exchange_recv_plans", xs_[r], 1, ptr(ri), ptr(status), 0, stream_ptr())
                recv_incl.append(ri)
            for r in range(W):
                if r == 0:
                    ev[0].record()
                call("epsb_exchange_put", xs_[r], 1, -1, 7, ptr(idx[r]), ptr(wts[r]), ptr(xq), ptr(xsc), ptr(src[r][0]),
                     ptr(src[r][1]), T, 1, stream_ptr())
                if r == 0:
                    ev[1].record()
            plans = []
            torch.cuda.synchronize()
            for r in range(W):
                call("epsb_exchange_wait", xs_[r], 1, ptr(status), 0, stream_ptr())
                pa = ctypes.c_void_p()
                call("epsb_exchange_arena", xs_[r], 0, e.value & 1, ctypes.byref(pa))
                from .scheduler import device_view
                ridx = device_view(pa.value, (rows, k), torch.int32, dev)
                plans.append(ops.expert_plans(ridx, recv_incl[r], k, r * EL, (r + 1) * EL, W, 1, T, rows))
                if int(plans[r][0][-1]) >= y_rows:
                    raise RuntimeError("routing put more rows on a rank than the benchmark's row buffer holds")
            for r in range(W):
                if r == 0:
                    ev[2].record()
                call("epsb_exchange_local_reduce_put", xs_[r], 3, ptr(y), ptr(plans[r][4]), ptr(plans[r][5]), 1, -1,
                     rows, stream_ptr())
                if r == 0:
                    ev[3].record()
            for r in range(W):
                call("epsb_exchange_wait", xs_[r], 3, ptr(status), 0, stream_ptr())
            torch.cuda.synchronize()
            if status.tolist()[0] != 0:
                raise RuntimeError(f"exchange status {status.tolist()}")
            if it >= 2:
                t_put += ev[0].elapsed_time(ev[1])
                t_red += ev[2].elapsed_time(ev[3])
            sent = int(src[0][1][-1])
            ret_rows = int(plans[0][5][-1])
            gemm_rows = int(plans[0][0][-1])
        row_b = H + sd * 4 + k * 8
        ms_put, ms_red = t_put / iters, t_red / iters
        b_put = 2.0 * sent * row_b
        b_red = (gemm_rows + ret_rows) * H * 2.0
        print(json.dumps({"kernel": "exchange put (permute-on-send: ids, gate weights, e4m3 rows, scales)", "ep_world": W,
                          "rows_sent": sent, "algorithmic_bytes": b_put, "ms": ms_put, "GB_per_s": b_put / ms_put / 1e6,
                          "note": "all ranks emulated on one GPU: stores land in local HBM"}))
        print(json.dumps({"kernel": "exchange local_reduce_put (weighted rows -> source rank's collect arena)",
                          "ep_world": W, "gemm_rows": gemm_rows, "rows_returned": ret_rows, "algorithmic_bytes": b_red,
                          "ms": ms_red, "GB_per_s": b_red / ms_red / 1e6,
                          "note": "all ranks emulated on one GPU: stores land in local HBM"}))
    finally:
        torch.cuda.synchronize()
        for x in xs_:
            call("epsb_exchange_destroy", x)
        for pr in regions:
            call("epsb_symm_free", pr)


if __name__ == "__main__":
    main()
