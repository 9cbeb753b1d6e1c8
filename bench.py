"""Benchmark of the FP8 MoE expert layer (the hot path) on N B200s of one node.

  python bench.py [--gpus N] [--steps K] [--warmup W] [--cfg C] [--impl ours|reference]

A "step" is one pass of the layer over one batch of synthetic tokens per rank (workload = benchmark
configuration `--cfg`, default 1: DeepSeek-V3-shaped prefill, 4096 tokens per GPU, 256 experts sharded
over the N ranks, weak scaling).  Rank 0 prints ONE JSON line.

`value` is measured with the inputs resident in HBM; `e2e` is measured through the same public call with
host (pinned) inputs and a host copy of the result inside the timed region.  Both are timed as blocks of
`--steps` steps (CUDA events, barrier + synchronize on both sides, max over ranks); blocks are repeated until
the timed region has lasted at least `--min-seconds` (default 2 s, so that the board has settled under its
power cap) and the MEDIAN block is reported (`timed_blocks`, `timed_region_s` say how many and how long).
`roofline` describes the dominant kernel (the gate/up grouped GEMM), timed with CUDA events inside the timed
region.  `parity` is checked after the timed regions: every rank compares a seeded sample of 64 of its output
rows with the CPU oracle; a failure makes the exit code non-zero.  `cpu_baseline` times the CPU oracle on a
bounded sample of the same workload (rank 0, N=1 only).
`--impl reference` times the CPU oracle alone (the reference has no CPU implementation of this path and its
sm_90a GEMM cannot run on B200; the oracle is the CPU restatement of its semantics): every step is one pass over
a bounded sample of the workload, with all host cores, on rank 0.
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
        return {"hbm_gbs": p["hbm_gbs"], "bf16_tflops": p["bf16_tflops"],
                "bf16_tflops_sustained": p.get("bf16_tflops_sustained", p["bf16_tflops"]), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


def _traffic_ratio():
    """DRAM bytes over algorithmic bytes of the gate/up GEMM, read from the committed ncu summary of the kernel
    (one capture on a 32-expert cut of cfg1; the traffic is weight streaming and grows with the expert count like
    the algorithmic bytes, so the ratio carries over to the full launch).  None when the summary has no such line."""
    import re

    path = os.path.join(ROOT, "profiles", "grouped_gemm_gateup_cfg1_small.md")
    try:
        with open(path) as f:
            m = re.search(r"traffic / algorithmic = ([0-9.]+)", f.read())
        return float(m.group(1)) if m else None
    except OSError:
        return None


def host_cores() -> int:
    try:
        return len(os.sched_getaffinity(0))
    except AttributeError:
        return os.cpu_count() or 1


def bind_to_gpu_numa_node(device_index: int):
    """One process per GPU: keep this process (and so the pinned host buffers it allocates next) on the CPUs of the NUMA
    node the GPU hangs off, as a deployment would.  Only narrows the affinity when the host reports such a node and it is
    a proper subset of the CPUs the process may use; returns what it did for the JSON line, or None."""
    try:
        p = torch.cuda.get_device_properties(device_index)
        path = f"/sys/bus/pci/devices/{p.pci_domain_id:04x}:{p.pci_bus_id:02x}:{p.pci_device_id:02x}.0/local_cpulist"
        cpus = set()
        for part in open(path).read().strip().split(","):
            if not part:
                continue
            lo, _, hi = part.partition("-")
            cpus.update(range(int(lo), int(hi or lo) + 1))
        allowed = os.sched_getaffinity(0)
        local = cpus & allowed
        if len(local) < 2 or local == allowed:
            return None
        os.sched_setaffinity(0, local)
        return {"cpus": len(local), "of": len(allowed)}
    except Exception:   # no sysfs node information, no permission: run unbound
        return None


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
    """The CPU oracle on a bounded sample of one step of `cfg`: the (token, expert) pairs routed to the first
    `n_exp` experts plus, when the configuration has a shared expert, that expert on the same fraction of the
    tokens.  Weights are generated and quantised once (outside any timed region); `run()` times one pass with the
    oracle's current thread count and returns tokens/s scaled by the fraction of the step the sample holds."""

    def __init__(self, cfg, n_exp):
        import numpy as np
        import torch

        from eps_b200 import workloads
        from oracle import oracle as orc

        self.orc, self.cfg, self.n_exp = orc, cfg, n_exp
        x = workloads.make_tokens(cfg)
        idx, w = workloads.make_routing(cfg)
        idx_n = idx.numpy()
        self.xb = x.view(torch.int16).numpy().view(np.uint16)
        self.total_pairs = int((idx_n >= 0).sum())

        def codes(e, inter=None):
            a, b = workloads.make_expert_weights(cfg, e, inter=inter)
            return orc.quant_block128(a.float().numpy()) + orc.quant_block128(b.float().numpy())

        per = [codes(e) for e in range(n_exp)]
        self.w = tuple(np.stack([p[i] for p in per]) for i in range(4))
        in_sample = (idx_n >= 0) & (idx_n < n_exp)
        self.pairs = int(in_sample.sum())
        self.frac = self.pairs / max(self.total_pairs, 1)
        # slots outside the sample get an id no sampled expert has and weight 0, so they cost and add nothing
        self.sel = np.where(in_sample, idx_n, n_exp + 5).astype(np.int32)
        self.sel_w = np.where(in_sample, w.numpy(), 0).astype(np.float32)
        self.shared, self.shared_tokens = None, 0
        if cfg.shared_inter:
            self.shared = tuple(t[None] for t in codes(-1, cfg.shared_inter))
            self.shared_tokens = max(1, int(round(cfg.tokens_per_rank * self.frac)))

    def run(self):
        import numpy as np

        t0 = time.perf_counter()
        self.orc.moe_layer_fp32(self.xb, self.sel, self.sel_w, *self.w)
        if self.shared is not None:   # the always-on expert on the same fraction of the tokens
            n = self.shared_tokens
            none = np.full((n, 1), -1, dtype=np.int32)
            self.orc.moe_layer_fp32_sampled(self.xb[:n], none, np.zeros((n, 1), np.float32), None, shared=self.shared)
        dt = time.perf_counter() - t0
        T = self.cfg.tokens_per_rank
        desc = (f"rows routed to the first {self.n_exp} of {self.cfg.num_experts} experts ({self.pairs} of "
                f"{self.total_pairs} (token,expert) pairs = {self.frac:.3f} of one {T}-token step"
                + (f", plus the shared expert on {self.shared_tokens} tokens" if self.shared is not None else "")
                + f"; {dt:.1f} s of CPU time per pass)")
        return T * self.frac / dt, self.orc.num_threads(), desc, dt


def cpu_sample_experts(cfg, per_pass_budget_s=3.0):
    """Experts in the CPU sample: about `per_pass_budget_s` of work on this host.  One expert row costs
    6*H*I flops; the blocked oracle sustains roughly 10 GFLOP/s per core."""
    rows_per_expert = cfg.tokens_per_rank * cfg.top_k / max(cfg.num_experts + cfg.num_zero_experts, 1)
    sec_per_expert = rows_per_expert * 6.0 * cfg.hidden * cfg.inter / (10e9 * host_cores()) + 0.02
    return int(max(1, min(cfg.num_experts // 4, per_pass_budget_s / sec_per_expert)))


def config_dict(cfg, world, stages, gemm_rows):
    """The workload description both arms print (same keys, same values for the same command line)."""
    return {"workload": f"cfg{cfg.cfg_id}:{cfg.name}", "tokens_per_gpu": cfg.tokens_per_rank,
            "global_tokens": cfg.tokens_per_rank * world, "hidden": cfg.hidden, "inter": cfg.inter,
            "experts": cfg.num_experts, "experts_per_gpu": cfg.num_experts // world, "top_k": cfg.top_k,
            "shared_inter": cfg.shared_inter, "parallelism": f"ep{world}", "stages": stages,
            "l2": "inputs larger than L2 (expert weights per GPU >> 126 MB); no flush",
            "gemm_rows_per_gpu": gemm_rows}


def run_reference(args, cfg, rank):
    """The CPU arm: the oracle (CPU restatement of the reference's layer semantics) on rank 0 with every host core
    (a launcher's OMP_NUM_THREADS=1 is overridden: the other ranks do no work).  A step is one pass over the
    bounded sample; `steps` passes are timed and the median is reported."""
    if rank != 0:
        return
    from oracle import oracle as orc

    cores = orc.set_num_threads(host_cores())
    # keep warm-up + steps within about two minutes whatever K is
    budget = max(0.5, min(4.0, 100.0 / max(args.steps + args.warmup, 1)))
    sample = CpuLayerSample(cfg, cpu_sample_experts(cfg, budget))
    for _ in range(args.warmup):
        sample.run()
    vals, dts, desc = [], [], ""
    for _ in range(max(1, args.steps)):   # every step is one pass over the bounded sample
        v, cores, desc, dt = sample.run()
        vals.append(v)
        dts.append(dt)
    v = statistics.median(vals)
    world = max(int(os.environ.get("WORLD_SIZE", "1")), args.gpus, 1)
    line = {
        "impl": "reference", "metric": METRIC, "value": v, "unit": UNIT, "n_gpus": args.gpus, "steps": len(vals),
        "warmup": args.warmup, "ms_per_step": statistics.median(dts) * 1e3,
        "ms_per_full_step_extrapolated": cfg.tokens_per_rank / v * 1e3, "step_fraction_of_workload": sample.frac,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "fp8_e4m3(fp32 accumulate)",
        "data": "synthetic",
        "config": config_dict(cfg, world, args.stages if args.stages else 1, cfg.tokens_per_rank * cfg.top_k),
        "cpu_baseline": {"value": v, "unit": UNIT, "cores": cores, "kind": "port", "sample": desc},
        "e2e": {"value": v, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--cfg", type=int, default=1)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--tokens", type=int, default=None, help="override tokens per GPU (diagnostics only)")
    ap.add_argument("--experts", type=int, default=None, help="override the expert count (diagnostics only)")
    ap.add_argument("--stages", type=int, default=None, help="EPS stages (default 1)")
    ap.add_argument("--graph", action="store_true",
                    help="diagnostics (N=1): also time the resident step replayed as one CUDA graph (key cuda_graph)")
    ap.add_argument("--no-numa-bind", action="store_true",
                    help="N > 1: do not bind the rank to the CPUs of its GPU's NUMA node before allocating pinned buffers")
    ap.add_argument("--shared-late", action="store_true",
                    help="diagnostics: run the shared expert after the routed experts instead of under the dispatch")
    ap.add_argument("--min-seconds", type=float, default=2.0,
                    help="repeat the timed block of --steps steps until this much time has been timed")
    ap.add_argument("--parity-tokens", type=int, default=64, help="output rows per rank checked against the oracle")
    ap.add_argument("--transport", default="auto", choices=["auto", "ipc", "nccl"],
                    help="expert-parallel transport at N > 1: this library's peer-store kernels (ipc, the default) "
                         "or grouped NCCL send/recv")
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
    host_binding = bind_to_gpu_numa_node(local_rank) if (world > 1 and not args.no_numa_bind) else None
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)
        comm = Communicator(None, CommunicatorParams(rank, world, world), transport=args.transport)
    else:
        comm = Communicator(None, CommunicatorParams(0, 1, 1))
    if cfg.num_experts % world:
        raise SystemExit(f"{cfg.num_experts} experts do not shard over {world} ranks")

    stages = args.stages if args.stages else 1
    from eps_b200.layer import build_synthetic_layer, synthetic_expert_codes

    layer = build_synthetic_layer(cfg, comm, dev, stages)
    layer.shared_under_dispatch = not args.shared_late
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

    # The ranks build their experts' weights at their own pace; the device-side exchange bounds every wait for a
    # peer, so they enter the first step together, and the bound is generous here (first launches load modules).
    if getattr(layer.sched, "peer", None) is not None:
        layer.sched.peer.timeout_ns = 20_000_000_000
    barrier()
    for _ in range(max(args.warmup, 3)):
        step_resident()
    for _ in range(3):
        step_e2e()
    layer.synchronize_host()
    barrier()
    layer.check_status()

    def timed_blocks(fn, host_path=False):
        """Blocks of --steps steps until --min-seconds have been timed (every rank sees the same max-over-ranks
        block times, so every rank stops after the same block); returns the block times in ms."""
        out, total = [], 0.0
        while True:
            ms = timed(fn, args.steps, host_path)
            out.append(ms)
            total += ms
            if total >= args.min_seconds * 1e3 or len(out) >= 1000:
                return out

    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    layer.exchange_events = [] if world > 1 else None     # (kind, start, end, bytes out, bytes in) per exchange
    blocks = timed_blocks(lambda: step_resident(True))
    layer.exchange_events_done = layer.exchange_events
    layer.exchange_events = None
    blocks_e2e = timed_blocks(step_e2e, host_path=True)
    graph_info = None
    if args.graph and world == 1:
        # the same resident step replayed as one CUDA graph (diagnostics: what the host's launch work costs)
        captured = layer.capture(x_d, idx_d, w_d, out_d, Tg)
        blocks_g = timed_blocks(captured.replay)
        graph_info = {"ms_per_step": statistics.median(blocks_g) / args.steps, "timed_blocks": len(blocks_g),
                      "kernels_in_graph": captured.kernel_launches}
    clocks = sampler.stop() if rank == 0 else None
    layer.check_status()

    ms_step = statistics.median(blocks) / args.steps
    ms_e2e_step = statistics.median(blocks_e2e) / args.steps
    value = Tg / (ms_step * 1e-3)
    e2e_value = Tg / (ms_e2e_step * 1e-3)

    # ---- parity: a seeded sample of this rank's output rows against the CPU oracle (outside every timed region)
    parity = None
    if args.parity_tokens > 0:
        import numpy as np

        from oracle import layer_check
        from oracle import oracle as orc

        orc.set_num_threads(max(1, host_cores() // world))
        layer.forward(x_d, idx_d, w_d, Tg, out=out_d)
        torch.cuda.synchronize()
        layer.check_status()
        sample = layer_check.sample_tokens(T, args.parity_tokens, seed=4242 + rank)
        sel = torch.from_numpy(sample)
        xb = x_h[sel].view(torch.int16).numpy().view(np.uint16)
        got = out_d[sel.to(dev)].float().cpu().numpy()
        got_h = out_h[sel].float().numpy()    # what the host-buffer path delivered in its last step

        def expert_weights(e):   # any expert's weights can be regenerated from its seed on this GPU
            return tuple(t.cpu().numpy() for t in synthetic_expert_codes(cfg, e, dev))

        shared = None
        if cfg.shared_inter:
            shared = tuple(t.cpu().numpy()[None] for t in synthetic_expert_codes(cfg, -1, dev, inter=cfg.shared_inter))
        res = layer_check.check_rows(xb, idx_h[sel].numpy(), w_h[sel].numpy(), got, expert_weights, shared=shared,
                                     bf16_stores=2 if world == 1 else 3)
        same_host = bool(np.array_equal(got, got_h))
        mine = torch.tensor([res["worst_ratio"], res["worst_ratio_bf16"], 0.0 if (res["ok"] and same_host) else 1.0],
                            dtype=torch.float64, device=dev)
        n_checked = torch.tensor([res["checked_tokens"]], dtype=torch.int64, device=dev)
        if world > 1:
            dist.all_reduce(mine, op=dist.ReduceOp.MAX)
            dist.all_reduce(n_checked, op=dist.ReduceOp.SUM)
        parity = {"checked_tokens": int(n_checked.item()), "worst_ratio": float(mine[0].item()),
                  "worst_ratio_bf16": float(mine[1].item()), "ok": bool(mine[2].item() == 0.0),
                  "bound": "worst_ratio = max|err| / (2e-2 x RMS); worst_ratio_bf16 adds half a bf16 ulp of |want| per bf16 "
                           "store on the value's way (2 in a world of one: weighted GEMM row, output; 3 with expert "
                           "parallelism: + the partial row on the link); ok = worst_ratio_bf16 <= 1 on every rank and "
                           "the host-buffer path returned the same rows", "oracle": "fp32 dequantised CPU oracle on the sampled tokens"}

    # ---- roofline of the dominant kernel: the gate/up grouped GEMM of the routed experts
    gemm_ms = statistics.mean(a.elapsed_time(b) for a, b in gemm_events) if gemm_events else None
    ctx = layer.sched.context
    excl = ctx.excl.cpu().numpy()
    EL = cfg.num_experts // world
    # the timed launch is the FIRST stage's gate/up GEMM: its experts are the first EL / stages of the rank
    excl = excl[:EL // stages + 1]
    D = int(excl[-1])
    live = int(((excl[1:] - excl[:-1]) > 0).sum())
    I = cfg.inter
    w_bytes = live * (2 * I * H + (2 * I // 128) * (H // 128) * 4)
    a_bytes = D * (H + H // 128 * 4)
    o_bytes = D * (I + I // 128 * 4)
    algo_bytes = w_bytes + a_bytes + o_bytes
    flops = 2.0 * D * 2 * I * H
    peaks = _peaks()
    roofline = None
    # DRAM bytes of one launch: ESTIMATED as (dram bytes / algorithmic bytes of the committed ncu capture of this
    # kernel on a small cut of cfg1) x this launch's algorithmic bytes
    ratio = _traffic_ratio() if (world == 1 and cfg.cfg_id == 1) else None
    traffic = int(ratio * algo_bytes) if ratio else None
    if gemm_ms:
        t_hbm = algo_bytes / (peaks["hbm_gbs"] * 1e9)
        # dense FP8 peak taken as 2 x the measured SUSTAINED bf16 figure: the kernel is timed inside a seconds-long region
        t_tc = flops / (2 * peaks["bf16_tflops_sustained"] * 1e12)
        if t_hbm >= t_tc:
            ach = algo_bytes / (gemm_ms * 1e-3) / 1e9
            roofline = {"kernel": "grouped_gemm_fp8<gate/up+SwiGLU+requant>", "bound": "hbm", "achieved": ach,
                        "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": ach / peaks["hbm_gbs"], "traffic": traffic,
                        "traffic_source": ("estimated: dram/algorithmic ratio of the ncu capture in profiles/"
                                           "grouped_gemm_gateup_cfg1_small.md x algorithmic bytes") if traffic else None,
                        "peak_source": peaks["source"], "ms_per_launch": gemm_ms, "algorithmic_bytes": algo_bytes,
                        "tflops": flops / (gemm_ms * 1e-3) / 1e12}
        else:
            ach = flops / (gemm_ms * 1e-3) / 1e12
            pk = 2 * peaks["bf16_tflops_sustained"]
            roofline = {"kernel": "grouped_gemm_fp8<gate/up+SwiGLU+requant>", "bound": "tensor", "achieved": ach,
                        "peak": pk, "unit": "TFLOP/s", "frac": ach / pk, "traffic": None,
                        "peak_source": peaks["source"] + " (2 x sustained bf16)", "ms_per_launch": gemm_ms,
                        "algorithmic_bytes": algo_bytes, "gbs": algo_bytes / (gemm_ms * 1e-3) / 1e9}

    if roofline is not None:
        roofline["gemm_rows"] = D
    # ---- exchange bandwidth (N > 1): bytes a rank moves in a dispatch / combine over the CUDA-event time of the
    # exchange on the stream it runs on, max(out, in) as the bus figure, against 900 GB/s per direction (nominal NVLink 5)
    ev = getattr(layer, "exchange_events_done", None)
    if ev and roofline is not None:
        bus = {}
        for kind in ("dispatch", "combine"):
            rows = [a.elapsed_time(b) for k_, a, b, st_ in ev if k_ == kind]
            if rows:
                ms = statistics.median(rows)
                # the routing is the same in every step: bytes of the last call's plans, all stages
                byt = max(layer.sched.exchange_bytes(-1, combine=kind == "combine"))
                bus[kind] = {"ms": ms * stages, "bytes": int(byt), "gbs": byt / (ms * stages * 1e-3) / 1e9}
        if bus:
            t = torch.tensor([bus.get("dispatch", {}).get("gbs", 0.0), bus.get("combine", {}).get("gbs", 0.0)],
                             dtype=torch.float64, device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MIN)
            roofline["bus_gbs"] = {"dispatch": float(t[0].item()), "combine": float(t[1].item()), "peak": 900.0,
                                   "rank0": bus, "note": "min over ranks of max(bytes out, bytes in) / CUDA-event time of the exchange on its stream"
                                           "; with the device-side transport the dispatch time covers plan exchange + "
                                           "permute-on-send (+ the flag wait when there is no shared expert to run "
                                           "under it), the combine time the fused local reduce + store",
                                   "transport": comm.transport}
    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        try:
            from oracle import oracle as orc

            orc.set_num_threads(host_cores())
            v, cores, desc, _ = CpuLayerSample(cfg, cpu_sample_experts(cfg, 10.0)).run()
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
                    "d2h_bytes_per_step": out_h.numel() * 2 * world, "ms_per_step": ms_e2e_step,
                    "timed_blocks": len(blocks_e2e)},
            "timed_blocks": len(blocks), "timed_region_s": sum(blocks) * 1e-3,
            "timing": f"median of {len(blocks)} blocks of {args.steps} steps (blocks repeated until "
                      f"{args.min_seconds:g} s were timed); block ms min/median/max = {min(blocks):.2f}/"
                      f"{statistics.median(blocks):.2f}/{max(blocks):.2f}",
            "gpu_launches": layer.kernel_launches * args.steps,
            "roofline": roofline, "parity": parity, "cpu_baseline": cpu, "clocks": clocks,
        }
        if graph_info is not None:
            line["cuda_graph"] = graph_info
        if world > 1:
            line["host_binding"] = host_binding if host_binding is not None else "unbound"
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()
    if parity is not None and not parity["ok"]:
        raise SystemExit(3)


if __name__ == "__main__":
    main()
