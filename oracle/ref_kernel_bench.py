"""Times the REFERENCE's own arch-agnostic kernels (oracle/_ref/libeps_ref.so, compiled from its sources) beside this
repository's kernels for the same step, at the benchmark's sizes, with CUDA events: the per-kernel speed bar.

  python -m oracle.ref_kernel_bench [--iters 10]

TEST INFRASTRUCTURE ONLY: a measurement helper beside the witness library; nothing in the product imports it.
Both libraries launch on the default stream; every timing is the mean over --iters launches after 2 warm-ups.
One JSON line per step: {"step", "size", "reference_us", "here_us", "speedup"}.
"""
from __future__ import annotations

import argparse
import ctypes
import json

import numpy as np
import torch

from eps_b200 import ops

from . import ref_kernels as ref


def _time(fn, iters):
    for _ in range(2):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters * 1e3


def _line(step, size, t_ref, t_here):
    print(json.dumps({"step": step, "size": size, "reference_us": round(t_ref, 1), "here_us": round(t_here, 1),
                      "speedup": round(t_ref / t_here, 2)}), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--iters", type=int, default=10)
    a = ap.parse_args()
    if not ref.available():
        raise SystemExit("oracle/_ref/libeps_ref.so is missing: run oracle/build_ref.py where the reference checkout is")
    dev = torch.device("cuda")
    L, P = ref.lib(), ref._p
    ll = ctypes.c_longlong
    T, k, E, H, I = 4096, 8, 256, 7168, 2048
    R = T * k
    g = torch.Generator().manual_seed(5)

    # ---- Q1: 1x128 quantisation of the GEMM-order rows
    x = torch.randn((R, H), device=dev, dtype=torch.bfloat16)
    q = torch.empty((R, H), dtype=torch.uint8, device=dev)
    s = torch.empty((R, H // 128), dtype=torch.float32, device=dev)
    t_ref = _time(lambda: L.ref_quant_1x128(P(x), ll(R), ll(H), P(q), P(s)), a.iters)
    t_here = _time(lambda: ops.per_token_group_quant_fp8(x, out=q, out_scales=s), a.iters)
    _line("Q1 per_token_group_quant_fp8", f"{R} x {H}", t_ref, t_here)

    # ---- S1 + S5 + S6 (source-side plans) and S3 + S4 (expert-side plans): a world of one, and one rank of eight
    idx = torch.stack([torch.randperm(E, generator=g)[:k] for _ in range(T)]).to(torch.int32).to(dev)
    wts = torch.rand((T, k), device=dev)
    for W in (1, 8):
        lead = torch.empty((T * W,), dtype=torch.int32, device=dev)
        smap = torch.empty((T * W,), dtype=torch.int32, device=dev)
        sincl = torch.zeros((W,), dtype=torch.int32, device=dev)
        tail = torch.empty((T * W,), dtype=torch.int32, device=dev)
        glob = torch.empty((T * W,), dtype=torch.int32, device=dev)
        coll = torch.zeros((W,), dtype=torch.int32, device=dev)
        z = torch.zeros((T,), dtype=torch.float32, device=dev)

        def ref_source():
            sincl.zero_()
            coll.zero_()
            L.ref_comm_plan(P(idx), P(lead), P(smap), P(sincl), T, k, E, 1, W)
            L.ref_global_reduce_plan(P(idx), P(tail), P(glob), P(coll), P(smap), P(sincl), T, E, 1, k, W)
            L.ref_zero_plan(P(idx), P(wts), T, k, P(z))

        t_ref = _time(ref_source, a.iters)
        t_here = _time(lambda: ops.source_plans(idx, wts, E, W, 1), a.iters)
        _line("S1+S5+S6 source-side plans", f"T={T} k={k} E={E} W={W}", t_ref, t_here)

        Rr = T if W == 1 else int(T * W * 0.66)     # tokens a rank receives
        EL = E // W
        ridx = torch.randint(0, E, (Rr, k), dtype=torch.int32, device=dev)
        recv_incl = torch.tensor([Rr * (i + 1) // W for i in range(W)], dtype=torch.int32, device=dev)
        gmap = torch.empty((Rr * k,), dtype=torch.int32, device=dev)
        excl = torch.zeros((EL + 1,), dtype=torch.int32, device=dev)
        t1, t2 = (torch.empty((Rr,), dtype=torch.int32, device=dev) for _ in range(2))
        red = torch.empty((Rr * k,), dtype=torch.int32, device=dev)
        scm = torch.empty((Rr,), dtype=torch.int32, device=dev)
        ret = torch.zeros((W,), dtype=torch.int32, device=dev)

        def ref_expert():
            excl.zero_()
            ret.zero_()
            L.ref_gemm_plan(P(ridx), P(recv_incl), P(gmap), P(excl), 0, EL, E, 1, k, W, ll(T))
            L.ref_local_reduce_plan(P(ridx), P(t1), P(t2), P(recv_incl), P(red), P(scm), P(ret), P(gmap), P(excl), 0, EL, E,
                                    1, k, W, ll(T), T * W)

        t_ref = _time(ref_expert, a.iters)
        t_here = _time(lambda: ops.expert_plans(ridx, recv_incl, k, 0, EL, W, 1, T, Rr), a.iters)
        _line("S3+S4 expert-side plans", f"received tokens={Rr} k={k} local experts={EL} W={W}", t_ref, t_here)

    # ---- A1: SwiGLU on ragged rows (unfused form; the FP8 path fuses it into the gate/up GEMM)
    rows = R // 2
    gu = torch.randn((rows, 2 * I), device=dev, dtype=torch.bfloat16)
    act = torch.empty((rows, I), device=dev, dtype=torch.bfloat16)
    ex1 = torch.tensor([0, rows], dtype=torch.int32, device=dev)
    t_ref = _time(lambda: L.ref_silu(P(gu), P(act), P(ex1), 1, 2 * I, rows), a.iters)
    t_here = _time(lambda: ops.silu_run(gu, act, ex1, 1), a.iters)
    _line("A1 silu_activate", f"{rows} x {2 * I}", t_ref, t_here)

    # ---- P3: localReduce (k weighted rows -> 1), a world of one
    y = torch.randn((R, H), device=dev, dtype=torch.bfloat16)
    red_map = torch.randperm(R, device=dev, dtype=torch.int32)
    scale_map = torch.arange(T, device=dev, dtype=torch.int32)
    ret_incl = torch.tensor([T], device=dev, dtype=torch.int32)
    send = torch.empty((T, H), dtype=torch.bfloat16, device=dev)
    t_ref = _time(lambda: L.ref_local_reduce(P(red_map), P(scale_map), P(ret_incl), 1, k, 1, ll(H), P(y), P(send), P(wts),
                                             ll(T), 0), a.iters)
    t_here = _time(lambda: ops.local_reduce_ref(y, wts, scale_map, red_map, ret_incl, k, 1, 1, 0, send), a.iters)
    _line("P3 localReduce (reference arithmetic)", f"{R} rows -> {T}, H={H}", t_ref, t_here)

    # ---- router and rms_norm (callers of the path)
    logits = torch.randn((T, E), device=dev)
    bias = torch.randn(E, device=dev) * 0.1
    t_ref = _time(lambda: ref.topk_sigmoid(logits, bias, 8, 4, k, 2.5), a.iters)     # includes its output allocation
    t_here = _time(lambda: ops.topk_sigmoid(logits, bias, 8, 4, k, 2.5), a.iters)
    _line("router topk_sigmoid (wrapper calls: allocation + synchronisation included on the reference side)",
          f"{T} x {E}", t_ref, t_here)
    scale = torch.ones(H, device=dev, dtype=torch.bfloat16)
    t_ref = _time(lambda: ref.rms_norm(x, scale, 1e-6), max(a.iters // 2, 2))
    out = torch.empty_like(x)
    t_here = _time(lambda: ops.rms_norm(x, scale, 1e-6, out=out), a.iters)
    _line("rms_norm (wrapper calls: allocation + synchronisation included on the reference side)", f"{R} x {H}", t_ref,
          t_here)

    # ---- F1: fast_ep expandPlan (the reference scans all T*k entries once per expert)
    t_ref = _time(lambda: ref.fastep_expand_plan(idx, E), a.iters)
    t_here = _time(lambda: ops.fastep_expand_plan(idx, E), a.iters)
    _line("F1 fast_ep expandPlan (wrapper calls)", f"T={T} k={k} E={E}", t_ref, t_here)


if __name__ == "__main__":
    main()
