"""Benchmark of the FP8 MoE expert layer (the hot path) on N B200s of one node.

  python bench.py [--gpus N] [--steps K] [--warmup W] [--cfg C] [--impl ours|reference]

A "step" is one pass of the layer over one batch of synthetic tokens per rank (workload = benchmark
configuration `--cfg`, default 1: DeepSeek-V3-shaped prefill, 4096 tokens per GPU, 256 experts sharded
over the N ranks, weak scaling).  Rank 0 prints ONE JSON line.

`value` is measured with the inputs resident in HBM; `e2e` is measured through the same public call with
host (pinned) inputs and a host copy of the result inside the timed region.  `roofline` describes the
dominant kernel (the gate/up grouped GEMM), timed with CUDA events inside the timed region.  `cpu_baseline`
times the CPU oracle on a bounded sample of the same workload (rank 0, N=1 only).
`--impl reference` times the CPU oracle alone (the reference has no CPU implementation of this path and its
sm_90a GEMM cannot run on B200; the oracle is the CPU restatement of its semantics).
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

METRIC = "fp8_moe_layer_tokens_per_s"
UNIT = "tokens/s"


def _peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return {"hbm_gbs": p["hbm_gbs"], "bf16_tflops": p["bf16_tflops"], "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu = gpu_index
        self.proc = None
        self.lines: list[str] = []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "200", "-i",
                 str(self.gpu)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._pump, daemon=True).start()
        except Exception:
            self.proc = None

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.25)
        self.proc.terminate()
        sm, mx, reasons = [], [], set()
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                mx.append(float(f[2]))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


class CpuLayerSample:
    """The CPU oracle on a bounded sample of one step of `cfg`: the rows routed to the first `n_exp` experts.
    Weights are generated and quantised once (outside any timed region); `run()` times one pass with all host
    threads and returns tokens/s scaled by the fraction of (token, expert) pairs the sample holds."""

    def __init__(self, cfg, n_exp):
        import numpy as np
        import torch

        from eps_b200 import workloads
        from oracle import oracle as orc

        self.orc, self.cfg, self.n_exp = orc, cfg, n_exp
        T = cfg.tokens_per_rank
        x = workloads.make_tokens(cfg)
        idx, w = workloads.make_routing(cfg)
        idx_n = idx.numpy()
        self.xb = x.view(torch.int16).numpy().view(np.uint16)
        self.total_pairs = int((idx_n >= 0).sum())
        gq, gs, dq, ds = [], [], [], []
        for e in range(n_exp):
            a, b = workloads.make_expert_weights(cfg, e)
            q1, s1 = orc.quant_block128(a.float().numpy())
            q2, s2 = orc.quant_block128(b.float().numpy())
            gq.append(q1); gs.append(s1); dq.append(q2); ds.append(s2)
        self.w = (np.stack(gq), np.stack(gs), np.stack(dq), np.stack(ds))
        in_sample = (idx_n >= 0) & (idx_n < n_exp)
        self.pairs = int(in_sample.sum())
        # slots outside the sample get an id no sampled expert has and weight 0, so they cost and add nothing
        self.sel = np.where(in_sample, idx_n, n_exp + 5).astype(np.int32)
        self.sel_w = np.where(in_sample, w.numpy(), 0).astype(np.float32)

    def run(self):
        t0 = time.perf_counter()
        self.orc.moe_layer_fp32(self.xb, self.sel, self.sel_w, *self.w)
        dt = time.perf_counter() - t0
        T = self.cfg.tokens_per_rank
        frac = self.pairs / max(self.total_pairs, 1)
        desc = (f"rows routed to the first {self.n_exp} of {self.cfg.num_experts} experts ({self.pairs} of "
                f"{self.total_pairs} (token,expert) pairs = {frac:.3f} of one {T}-token step, {dt:.1f} s of CPU time; "
                f"shared expert excluded)")
        return T * frac / dt, self.orc.num_threads(), desc


def cpu_sample_experts(cfg):
    return max(1, cfg.num_experts // 4)


def config_dict(cfg, world, stages, gemm_rows):
    """The workload description both arms print (same keys, same values for the same command line)."""
    return {"workload": f"cfg{cfg.cfg_id}:{cfg.name}", "tokens_per_gpu": cfg.tokens_per_rank,
            "global_tokens": cfg.tokens_per_rank * world, "hidden": cfg.hidden, "inter": cfg.inter,
            "experts": cfg.num_experts, "experts_per_gpu": cfg.num_experts // world, "top_k": cfg.top_k,
            "shared_inter": cfg.shared_inter, "parallelism": f"ep{world}", "stages": stages,
            "l2": "inputs larger than L2 (expert weights per GPU >> 126 MB); no flush",
            "gemm_rows_per_gpu": gemm_rows}


def run_reference(args, cfg, rank):
    """The CPU arm: the oracle (CPU restatement of the reference's layer semantics), all host threads."""
    if rank != 0:
        return
    vals = []
    desc, cores = "", 1
    sample = CpuLayerSample(cfg, cpu_sample_experts(cfg))
    for _ in range(min(args.warmup, 1)):
        sample.run()
    for _ in range(max(1, min(args.steps, 3))):   # every "step" is one pass over the bounded sample
        v, cores, desc = sample.run()
        vals.append(v)
    v = statistics.median(vals)
    line = {
        "impl": "reference", "metric": METRIC, "value": v, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": cfg.tokens_per_rank / v * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "fp8_e4m3(fp32 accumulate)", "data": "synthetic",
        "config": config_dict(cfg, max(args.gpus, 1), args.stages if args.stages else 1,
                              cfg.tokens_per_rank * cfg.top_k),
        "cpu_baseline": {"value": v, "unit": UNIT, "cores": cores, "kind": "port", "sample": desc},
        "e2e": {"value": v, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def build_layer(cfg, comm, dev, torch, stages=1):
    """Random-init expert weights of the configuration's architecture, generated and block-quantised on the GPU."""
    from eps_b200 import ops, workloads
    from eps_b200.layer import MoELayerFP8

    W, rank = comm.getWorldSize(), comm.getRank()
    EL = cfg.num_experts // W
    H, I = cfg.hidden, cfg.inter
    wgu = torch.empty((EL, 2 * I, H), dtype=torch.uint8, device=dev)
    wgu_s = torch.empty((EL, 2 * I // 128, H // 128), dtype=torch.float32, device=dev)
    wd = torch.empty((EL, H, I), dtype=torch.uint8, device=dev)
    wd_s = torch.empty((EL, H // 128, I // 128), dtype=torch.float32, device=dev)
    for le in range(EL):
        a, b = workloads.make_expert_weights(cfg, rank * EL + le, device=dev)
        q, s = ops.quant_block128(a)
        wgu[le], wgu_s[le] = q, s
        q, s = ops.quant_block128(b)
        wd[le], wd_s[le] = q, s
    shared = None
    if cfg.shared_inter:
        a, b = workloads.make_expert_weights(cfg, -1, device=dev, inter=cfg.shared_inter)
        q1, s1 = ops.quant_block128(a.unsqueeze(0))
        q2, s2 = ops.quant_block128(b.unsqueeze(0))
        shared = (q1, s1, q2, s2)
    torch.cuda.synchronize()
    layer = MoELayerFP8(H, I, cfg.num_experts, cfg.top_k, cfg.tokens_per_rank, wgu, wgu_s, wd, wd_s, comm=comm,
                        shared=shared, num_stages=stages)
    return layer


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--cfg", type=int, default=1)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--tokens", type=int, default=None, help="override tokens per GPU (diagnostics only)")
    ap.add_argument("--experts", type=int, default=None, help="override the expert count (diagnostics only)")
    ap.add_argument("--stages", type=int, default=None, help="EPS stages (default 1; 1/2 stages measured 3.82/4.09 ms at 2 GPUs and 1/2/4 stages 4.59/5.54/6.03 ms at 8)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    args = ap.parse_args()

    from eps_b200 import workloads

    cfg = workloads.CONFIGS[args.cfg]
    if args.tokens:
        cfg = cfg.scaled(tokens_per_rank=args.tokens)
    if args.experts:
        cfg = cfg.scaled(num_experts=args.experts)
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if args.impl == "reference":
        run_reference(args, cfg, rank)
        return

    import torch
    import torch.distributed as dist

    from eps_b200 import _lib
    from eps_b200.communication import Communicator, CommunicatorParams

    _lib.lib()  # fail loudly if the CUDA library is missing
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)
        comm = Communicator(None, CommunicatorParams(rank, world, world))
    else:
        comm = Communicator(None, CommunicatorParams(0, 1, 1))
    if cfg.num_experts % world:
        raise SystemExit(f"{cfg.num_experts} experts do not shard over {world} ranks")

    stages = args.stages if args.stages else 1
    layer = build_layer(cfg, comm, dev, torch, stages)
    T, H, k = cfg.tokens_per_rank, cfg.hidden, cfg.top_k
    x_h = workloads.make_tokens(cfg, rank).pin_memory()
    idx_h, w_h = workloads.make_routing(cfg, rank)
    idx_h, w_h = idx_h.pin_memory(), w_h.pin_memory()
    out_h = torch.empty((T, H), dtype=torch.bfloat16).pin_memory()
    x_d, idx_d, w_d = x_h.to(dev), idx_h.to(dev), w_h.to(dev)
    out_d = torch.empty((T, H), dtype=torch.bfloat16, device=dev)
    Tg = T * world

    gemm_events = []

    def step_resident(timed=False):
        if timed:
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            layer.gateup_events = (e0, e1)
            gemm_events.append((e0, e1))
        else:
            layer.gateup_events = None
        layer.forward(x_d, idx_d, w_d, Tg, out=out_d)

    def step_e2e():
        # the public host-buffer call: pinned inputs in, pinned result out; copies of neighbouring steps overlap compute
        layer.gateup_events = None
        layer.forward_host(x_h, idx_h, w_h, out_h, Tg)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, steps, host_path=False):
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            fn()
        if host_path:
            layer.synchronize_host()   # drain the copy streams of the host-buffer path
        e1.record()
        barrier()
        ms = e0.elapsed_time(e1)
        if world > 1:
            t = torch.tensor([ms], dtype=torch.float64, device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms

    for _ in range(max(args.warmup, 3)):
        step_resident()
    for _ in range(3):
        step_e2e()
    layer.synchronize_host()
    barrier()
    layer.check_status()

    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    ms_total = timed(lambda: step_resident(True), args.steps)
    ms_e2e_total = timed(step_e2e, args.steps, host_path=True)
    clocks = sampler.stop() if rank == 0 else None
    layer.check_status()

    ms_step = ms_total / args.steps
    value = Tg / (ms_step * 1e-3)
    e2e_value = Tg / (ms_e2e_total / args.steps * 1e-3)

    # ---- roofline of the dominant kernel: the gate/up grouped GEMM of the routed experts
    gemm_ms = statistics.mean(a.elapsed_time(b) for a, b in gemm_events) if gemm_events else None
    ctx = layer.sched.context
    excl = ctx.excl.cpu().numpy()
    D = int(excl[-1])
    EL = cfg.num_experts // world
    live = int(((excl[1:] - excl[:-1]) > 0).sum())
    I = cfg.inter
    w_bytes = live * (2 * I * H + (2 * I // 128) * (H // 128) * 4)
    a_bytes = D * (H + H // 128 * 4)
    o_bytes = D * (I + I // 128 * 4)
    algo_bytes = w_bytes + a_bytes + o_bytes
    flops = 2.0 * D * 2 * I * H
    peaks = _peaks()
    roofline = None
    # DRAM bytes of one launch: one ncu capture of this kernel on a 32-expert, 512-token cut of the same configuration
    # (128 rows per expert, inputs larger than L2) read 1.030 x its algorithmic bytes; the traffic is weight streaming
    # and grows with the expert count like the algorithmic bytes do, so the ratio is applied to the full launch.
    traffic = int(1.030 * algo_bytes) if (world == 1 and cfg.cfg_id == 1) else None
    if gemm_ms:
        t_hbm = algo_bytes / (peaks["hbm_gbs"] * 1e9)
        t_tc = flops / (2 * peaks["bf16_tflops"] * 1e12)  # dense FP8 peak taken as 2 x the measured bf16 figure
        if t_hbm >= t_tc:
            ach = algo_bytes / (gemm_ms * 1e-3) / 1e9
            roofline = {"kernel": "grouped_gemm_fp8<gate/up+SwiGLU+requant>", "bound": "hbm", "achieved": ach,
                        "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": ach / peaks["hbm_gbs"], "traffic": traffic,
                        "traffic_source": "ncu dram bytes of a 32-expert cut, scaled by algorithmic bytes" if traffic else None,
                        "peak_source": peaks["source"], "ms_per_launch": gemm_ms, "algorithmic_bytes": algo_bytes,
                        "tflops": flops / (gemm_ms * 1e-3) / 1e12}
        else:
            ach = flops / (gemm_ms * 1e-3) / 1e12
            pk = 2 * peaks["bf16_tflops"]
            roofline = {"kernel": "grouped_gemm_fp8<gate/up+SwiGLU+requant>", "bound": "tensor", "achieved": ach,
                        "peak": pk, "unit": "TFLOP/s", "frac": ach / pk, "traffic": None,
                        "peak_source": peaks["source"] + " (2 x bf16)", "ms_per_launch": gemm_ms,
                        "algorithmic_bytes": algo_bytes, "gbs": algo_bytes / (gemm_ms * 1e-3) / 1e9}

    if roofline is not None:
        roofline["gemm_rows"] = D
    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        try:
            v, cores, desc = CpuLayerSample(cfg, cpu_sample_experts(cfg)).run()
            cpu = {"value": v, "unit": UNIT, "cores": cores, "kind": "port", "sample": desc}
        except Exception as exc:  # the baseline is a report, not a gate
            cpu = {"value": None, "unit": UNIT, "cores": 0, "kind": "port", "sample": f"failed: {exc}"}

    if rank == 0:
        h2d = x_h.numel() * 2 + idx_h.numel() * 4 + w_h.numel() * 4
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "fp8_e4m3(fp32 accumulate)", "data": "synthetic",
            "config": config_dict(cfg, world, stages, T * k),   # nominal rows; rank 0's actual count is in roofline
            "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": h2d * world,
                    "d2h_bytes_per_step": out_h.numel() * 2 * world, "ms_per_step": ms_e2e_total / args.steps},
            "gpu_launches": layer.kernel_launches * args.steps,
            "roofline": roofline, "cpu_baseline": cpu, "clocks": clocks,
        }
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
