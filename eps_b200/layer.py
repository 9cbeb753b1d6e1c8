"""The FP8 MoE expert layer on one rank of an expert-parallel group: the hot path end to end.

  tokens bf16 --quant 1x128--> fp8 + scales --dispatch (unique token per rank)--> expert-contiguous rows
  --grouped GEMM gate/up + SwiGLU + requant (tcgen05)--> fp8 activations
  --grouped GEMM down x gate weight (tcgen05)--> bf16 rows --local reduce--> combine --global reduce
  (+ identity experts, + shared expert)--> bf16 output

It drives the same objects a caller of the reference would drive (Scheduler + a grouped-GEMM executor,
reference python/eps/scheduler/scheduler.py and python/eps/executor/aok_grouped_gemm.py), staged the same way.
"""
from __future__ import annotations

import torch

from . import ops
from ._lib import EpsError
from .communication import Communicator
from .scheduler import Scheduler


class MoELayerFP8:
    def __init__(self, hidden: int, inter: int, num_experts: int, top_k: int, max_tokens_per_gpu: int,
                 w_gate_up, w_gate_up_scale, w_down, w_down_scale, comm: Communicator | None = None,
                 shared=None, num_stages: int = 1, max_gemm_rows: int | None = None, device=None):
        """w_gate_up [EL, 2I, H] e4m3 codes (gate rows first), w_gate_up_scale [EL, 2I/128, H/128] fp32,
        w_down [EL, H, I], w_down_scale [EL, H/128, I/128]: this rank's experts.
        shared: optional (w_gate_up [1, 2Is, H], scale, w_down [1, H, Is], scale) of an always-on expert."""
        self.comm = comm if comm is not None else Communicator()
        self.W = self.comm.getWorldSize()
        self.H, self.I, self.E, self.k = hidden, inter, num_experts, top_k
        self.EL = num_experts // self.W
        self.S = num_stages
        self.max_tok = max_tokens_per_gpu
        self.dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        self.num_sms = torch.cuda.get_device_properties(self.dev).multi_processor_count
        if hidden % 128 or inter % 128:
            raise EpsError("hidden and intermediate sizes must be multiples of 128")
        if tuple(w_gate_up.shape) != (self.EL, 2 * inter, hidden) or tuple(w_down.shape) != (self.EL, hidden, inter):
            raise EpsError("expert weight shapes do not match (EL, 2I, H) / (EL, H, I)")
        self.wgu, self.wgu_s, self.wd, self.wd_s = w_gate_up, w_gate_up_scale, w_down, w_down_scale
        self.shared = shared
        self.sched = Scheduler(top_k, num_experts, hidden, hidden // 128, max_tokens_per_gpu, self.comm, self.EL,
                               input_dtype=torch.uint8, device=self.dev)
        worst = max_tokens_per_gpu * self.W * min(top_k, self.EL)
        # Like the reference's arenas (src/communication/msccl_comm.cu:191-199) the GEMM-side buffers are sized for
        # the worst routing by default: every token of every rank lands here with min(k, EL) of its slots.  The
        # host only learns the number of received TOKENS before it launches the GEMMs (the row count stays on the
        # device), so a smaller capacity is checked against tokens * min(k, EL), which over-counts by up to k.
        self.max_gemm_rows = min(worst, max_gemm_rows) if max_gemm_rows is not None else worst
        D = max(self.max_gemm_rows, 1)
        dev = self.dev
        # With the device-side exchange (and in a world of one) every GEMM row knows its source row (the arena, or the
        # caller's own quantised tokens): ONE gather brings the rows into expert order, nothing is staged for sending.
        self.direct_sources = self.W == 1 or self.sched.peer is not None
        # True: the gate/up GEMM fetches those rows itself (TMA gather4 in its producer) and the gather pass goes too.
        # Measured on cfg1 this is slower (32 four-row loads per stage instead of one box load: 3.4 vs 2.1 ms), so it is
        # off; small-row workloads may set it.
        self.gemm_gathers_rows = False
        self.A = torch.empty((D, hidden), dtype=torch.uint8, device=dev)
        self.A_s = torch.empty((D, hidden // 128), dtype=torch.float32, device=dev)
        self.act = torch.empty((D, inter), dtype=torch.uint8, device=dev)
        self.act_s = torch.empty((D, inter // 128), dtype=torch.float32, device=dev)
        self.Y = torch.empty((D, hidden), dtype=torch.bfloat16, device=dev)
        self.status = torch.zeros(4, dtype=torch.int32, device=dev)
        T = max(max_tokens_per_gpu, 1)
        self.xq = torch.empty((T, hidden), dtype=torch.uint8, device=dev)
        self.xs = torch.empty((T, hidden // 128), dtype=torch.float32, device=dev)
        if shared is not None:
            Is = shared[2].shape[2]
            self.sh_act = torch.empty((T, Is), dtype=torch.uint8, device=dev)
            self.sh_act_s = torch.empty((T, Is // 128), dtype=torch.float32, device=dev)
            self.sh_out = torch.empty((T, hidden), dtype=torch.bfloat16, device=dev)
            self._sh_excl = {}
        self.kernel_launches = 0
        self.shared_sm_reserve = 4   # SMs the shared expert's GEMMs leave to the plan and gather kernels (EP=1)
        # device-side exchange: run the shared expert between this rank's put and the wait for the peers' rows
        self.shared_under_dispatch = True
        self.gateup_events = None  # optional (start, end) torch.cuda.Event pair recorded around the gate/up GEMM
        # optional list; with ep_world_size > 1 every exchange appends (kind, start event, end event, stage) so that a
        # caller can report bus bandwidth (bytes per exchange: Scheduler.exchange_bytes, after the timed region)
        self.exchange_events = None

    def forward(self, x: torch.Tensor, expert_indices: torch.Tensor, expert_weights: torch.Tensor,
                num_global_tokens: int | None = None, out: torch.Tensor | None = None) -> torch.Tensor:
        """x [T, H] bf16, expert_indices [T, k] int32 (negative = identity expert), expert_weights [T, k] fp32."""
        T = x.shape[0]
        if T > self.max_tok:
            raise EpsError(f"{T} tokens exceed max_tokens_per_gpu {self.max_tok}")
        sched, S, EL = self.sched, self.S, self.EL
        n = 0
        xq, xs = ops.per_token_group_quant_fp8(x, out=self.xq[:T], out_scales=self.xs[:T])
        n += 1
        Tg = num_global_tokens if num_global_tokens is not None else T * self.W
        shared_out, shared_done = None, None
        if self.W == 1 and self.shared is not None and T > 0:
            # The shared expert needs only the quantised tokens, while the routed path first runs its plan kernels
            # (single CTAs, ~0.2 ms): run the two side by side.  The GEMMs leave a few SMs to the plan kernels,
            # which could not start otherwise (a GEMM CTA owns all registers of its SM).
            main = torch.cuda.current_stream()
            side = self._comm_stream()
            side.wait_stream(main)
            with torch.cuda.stream(side):
                shared_out = self._shared_expert(xq, xs, T, sm_count=max(self.num_sms - self.shared_sm_reserve, 1))
                shared_done = torch.cuda.Event()
                shared_done.record(side)
        # next to the shared expert's GEMMs (which occupy all but four SMs) a plan must fit into single free SMs
        # device-side exchange with one stage: the FP8 rows and their scales travel with the expert ids
        eager = sched.peer is not None and S == 1
        mark = self._exchange_mark("dispatch", 0, torch.cuda.current_stream()) if eager else None
        early = []   # device-side exchange: the shared expert runs while the peers' rows are on their way
        marks = [mark]

        def shared_under_dispatch():
            # the exchange's own time ends with this rank's put; what follows is compute, then the flag wait
            self._exchange_done(marks[0], torch.cuda.current_stream())
            marks[0] = None
            early.append(self._shared_expert(xq, xs, T))

        excl, n_recv = sched.rendezvous_and_plan(
            expert_indices, expert_weights, Tg, S, True, host_sync=self.W > 1,
            max_cluster=1 if shared_done is not None else 0, payload=(xq, xs) if eager else None,
            after_put=shared_under_dispatch if (self.shared_under_dispatch and sched.peer is not None
                                                and self.shared is not None and T > 0) else None)
        self._exchange_done(marks[0], torch.cuda.current_stream())
        # source plans, expert plans + (NCCL transport: index gather, receive plan | device-side exchange: publish,
        # receive plans, put, wait) or the index gather of a world of one
        n += 2 + (4 if sched.peer is not None else (2 if self.W > 1 else 1))
        rows_k = max(sched.context.rows_bound, 0) * min(self.k, EL)
        if rows_k > self.max_gemm_rows:
            raise EpsError(f"{rows_k} possible GEMM rows exceed max_gemm_rows {self.max_gemm_rows}")
        D = max(rows_k, 1)
        a_rows = src_h = src_s = None
        if self.W == 1:
            # nothing is staged: the GEMM reads the quantised tokens through the composed plans
            sched.context.raw_input = x
            a_rows, row_w, src_h, src_s = sched.gemm_sources(expert_weights, xq, xs)
            n += 1
        else:
            sched.prologue(expert_weights, xq, xs, None if self.direct_sources else self.A_s[:D], raw_input=x,
                           defer_exchange=True)
            # NCCL transport: gate weights, hidden rows, scales to send order; scales to GEMM order; GEMM-row gate
            # weights.  Device-side exchange: nothing is staged, only the per-GEMM-row sources.
            n += 1 if self.direct_sources else 5
            row_w = None
        eps_ = EL // S

        def stage_gemms(s):
            ex = excl[s * eps_:(s + 1) * eps_ + 1]
            ev = self.gateup_events if s == 0 else None
            if ev is not None:
                ev[0].record()
            if self.direct_sources and self.gemm_gathers_rows:
                ops.grouped_gemm_fp8(ops.GEMM_GATEUP, src_h, src_s, self.wgu[s * eps_:(s + 1) * eps_],
                                     self.wgu_s[s * eps_:(s + 1) * eps_], ex, out=self.act[:D],
                                     out_scales=self.act_s[:D], status=self.status, a_rows=a_rows[:D])
            else:
                if self.direct_sources:   # one gather from the source rows into expert order (rows and their scales)
                    b0, b1 = s * eps_, (s + 1) * eps_
                    ops.gather_rows(src_h, self.A[:D], a_rows, 1, ops.INT32_MAX, bounds=excl, b0=b0, b1=b1)
                    ops.gather_rows(src_s, self.A_s[:D], a_rows, 1, ops.INT32_MAX, bounds=excl, b0=b0, b1=b1)
                ops.grouped_gemm_fp8(ops.GEMM_GATEUP, self.A[:D], self.A_s[:D], self.wgu[s * eps_:(s + 1) * eps_],
                                     self.wgu_s[s * eps_:(s + 1) * eps_], ex, out=self.act[:D],
                                     out_scales=self.act_s[:D], status=self.status)
            if ev is not None:
                ev[1].record()
            ops.grouped_gemm_fp8(ops.GEMM_DOWN, self.act[:D], self.act_s[:D], self.wd[s * eps_:(s + 1) * eps_],
                                 self.wd_s[s * eps_:(s + 1) * eps_], ex, out=self.Y[:D], row_w=row_w,
                                 status=self.status)

        if self.W == 1:
            for s in range(S):
                stage_gemms(s)
                n += 2 if self.gemm_gathers_rows else 4
        else:
            # Stage pipeline on two streams (the reference leaves this to its caller): all dispatches are queued on
            # the communication stream up front, each combine as soon as its stage has been reduced, so the exchange
            # of stage s+1 / s-1 runs under the GEMMs of stage s.
            main = torch.cuda.current_stream()
            comm_stream = self._comm_stream()
            ready = torch.cuda.Event()
            ready.record(main)
            disp_done = [torch.cuda.Event() for _ in range(S)]
            red_done = [torch.cuda.Event() for _ in range(S)]
            with torch.cuda.stream(comm_stream):
                comm_stream.wait_event(ready)
                for s in range(S):
                    mark = None if eager else self._exchange_mark("dispatch", s, comm_stream)
                    sched.dispatch(s)
                    self._exchange_done(mark, comm_stream)
                    disp_done[s].record(comm_stream)
            for s in range(S):
                main.wait_event(disp_done[s])
                if s == 0:  # the first dispatch carried the gate weights and the input scales
                    if self.direct_sources:
                        a_rows, row_w, src_h, src_s = sched.gemm_sources(expert_weights, xq, xs)
                    else:
                        sched.finish_prologue()
                        row_w = sched.gemm_row_weights()
                if not self.direct_sources:
                    sched.gemm_expand(self.A[:D], s)
                stage_gemms(s)
                mark_lr = self._exchange_mark("combine", s, main) if sched.peer is not None else None
                sched.local_reduce(self.Y[:D], s, pre_weighted=True)   # device-side exchange: reduce + store at the source
                self._exchange_done(mark_lr, main)
                red_done[s].record(main)
                with torch.cuda.stream(comm_stream):
                    comm_stream.wait_event(red_done[s])
                    mark = self._exchange_mark("combine", s, comm_stream) if sched.peer is None else None
                    sched.combine(s)
                    self._exchange_done(mark, comm_stream)
                n += 4 if (self.gemm_gathers_rows or not self.direct_sources) else 6
            all_back = torch.cuda.Event()
            all_back.record(comm_stream)
        if self.W > 1:
            shared_out = early[0] if early else self._shared_expert(xq, xs, T)
        if out is None:
            out = torch.empty((T, self.H), dtype=torch.bfloat16, device=x.device)
        if self.W > 1:
            torch.cuda.current_stream().wait_event(all_back)  # the shared expert above ran under the last combine
            sched.epilogue(out, shared=shared_out, ref_arith=False)
        else:
            if shared_done is not None:
                torch.cuda.current_stream().wait_event(shared_done)
            sched.reduce_single_rank(self.Y[:D], out, shared=shared_out)
        n += 1 + (2 if shared_out is not None else 0)
        self.kernel_launches = n
        return out

    def capture(self, x: torch.Tensor, expert_indices: torch.Tensor, expert_weights: torch.Tensor, out: torch.Tensor,
                num_global_tokens: int | None = None) -> "CapturedStep":
        """One layer step as a CUDA graph over these four tensors: `replay()` runs the step on whatever they hold
        then.  For steps whose time is the host's launch work rather than the GPU's (decode-sized batches: ten
        launches of a few microseconds of GPU time each).  World of one only: the device-side exchange numbers its
        calls on the host."""
        return CapturedStep(self, x, expert_indices, expert_weights, out, num_global_tokens)

    def forward_routed(self, x: torch.Tensor, router_logits: torch.Tensor, router_bias: torch.Tensor | None,
                       num_expert_groups: int = 1, topk_groups: int = 1, route_scale: float = 1.0,
                       num_zero_experts: int = 0, out: torch.Tensor | None = None) -> torch.Tensor:
        """The layer fed by the router: router_logits [T, num_experts + num_zero_experts] (fp32 or bf16) go through
        topk_sigmoid (reference utils/topk_sigmoid), whose indices and weights are what `forward` reads; the last
        num_zero_experts ids are identity experts."""
        idx, w = ops.topk_sigmoid(router_logits, router_bias, num_expert_groups, topk_groups, self.k, route_scale,
                                  num_ffn_experts=router_logits.shape[1] - num_zero_experts)
        return self.forward(x, idx, w, out=out)

    def _shared_expert(self, xq, xs, T, sm_count=0):
        """The always-on expert on the quantised tokens; returns its [T, H] bf16 output (None without one)."""
        if self.shared is None or T == 0:
            return None
        sgu, sgu_s, sd, sd_s = self.shared
        if T not in self._sh_excl:
            self._sh_excl[T] = torch.tensor([0, T], dtype=torch.int32, device=self.dev)
        sh_excl = self._sh_excl[T]
        ops.grouped_gemm_fp8(ops.GEMM_GATEUP, xq, xs, sgu, sgu_s, sh_excl, out=self.sh_act[:T],
                             out_scales=self.sh_act_s[:T], status=self.status, sm_count=sm_count)
        return ops.grouped_gemm_fp8(ops.GEMM_DOWN, self.sh_act[:T], self.sh_act_s[:T], sd, sd_s, sh_excl,
                                    out=self.sh_out[:T], status=self.status, sm_count=sm_count)

    def _exchange_mark(self, kind, stage, stream):
        if self.exchange_events is None:
            return None
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        return (kind, e0, e1, stage)

    def _exchange_done(self, mark, stream):
        if mark is not None:
            mark[2].record(stream)
            self.exchange_events.append(mark)

    def _comm_stream(self):
        if getattr(self, "_cs", None) is None:
            self._cs = torch.cuda.Stream(device=self.dev)
        return self._cs

    # ------------------------------------------------------------------ host-buffer entry point

    def _host_pipeline(self):
        if getattr(self, "_hp", None) is None:
            T, H, k = max(self.max_tok, 1), self.H, self.k
            dev = self.dev
            self._hp = dict(
                h2d=torch.cuda.Stream(device=dev), d2h=torch.cuda.Stream(device=dev), slot=0,
                x=[torch.empty((T, H), dtype=torch.bfloat16, device=dev) for _ in range(2)],
                idx=[torch.empty((T, k), dtype=torch.int32, device=dev) for _ in range(2)],
                w=[torch.empty((T, k), dtype=torch.float32, device=dev) for _ in range(2)],
                out=[torch.empty((T, H), dtype=torch.bfloat16, device=dev) for _ in range(2)],
                in_ready=[torch.cuda.Event() for _ in range(2)], in_free=[None, None],
                out_ready=[torch.cuda.Event() for _ in range(2)], out_free=[None, None])
        return self._hp

    def forward_host(self, x_host: torch.Tensor, idx_host: torch.Tensor, w_host: torch.Tensor,
                     out_host: torch.Tensor, num_global_tokens: int | None = None) -> None:
        """Same layer for HOST (pinned) tensors.  Asynchronous: the inputs are copied to one of two device slots on a
        copy stream, the layer runs on the current stream, the result is copied into `out_host` on a second copy
        stream; consecutive calls overlap (copy-in of call i+1 and copy-out of call i-1 with the compute of call i).
        Call `synchronize_host()` before reading `out_host`."""
        hp = self._host_pipeline()
        T = x_host.shape[0]
        i = hp["slot"]
        hp["slot"] = 1 - i
        main = torch.cuda.current_stream()
        with torch.cuda.stream(hp["h2d"]):
            if hp["in_free"][i] is not None:
                hp["h2d"].wait_event(hp["in_free"][i])     # the call that last used this slot has consumed it
            hp["idx"][i][:T].copy_(idx_host, non_blocking=True)
            hp["w"][i][:T].copy_(w_host, non_blocking=True)
            hp["x"][i][:T].copy_(x_host, non_blocking=True)
            hp["in_ready"][i].record(hp["h2d"])
        main.wait_event(hp["in_ready"][i])
        if hp["out_free"][i] is not None:
            main.wait_event(hp["out_free"][i])             # the previous result in this slot has left the device
        self.forward(hp["x"][i][:T], hp["idx"][i][:T], hp["w"][i][:T], num_global_tokens, out=hp["out"][i][:T])
        done = torch.cuda.Event()
        done.record(main)
        hp["in_free"][i] = done
        hp["out_ready"][i].record(main)
        with torch.cuda.stream(hp["d2h"]):
            hp["d2h"].wait_event(hp["out_ready"][i])
            out_host.copy_(hp["out"][i][:T], non_blocking=True)
            free = torch.cuda.Event()
            free.record(hp["d2h"])
            hp["out_free"][i] = free

    def synchronize_host(self) -> None:
        hp = self._host_pipeline()
        hp["h2d"].synchronize()
        torch.cuda.current_stream().synchronize()
        hp["d2h"].synchronize()

    def check_status(self) -> None:
        """Raises if a bounded device-side wait of a GEMM kernel or of the exchange expired (synchronises)."""
        if self.sched.peer is not None:
            self.sched.peer.check_status()
        st = self.status.cpu().tolist()
        if st[0] != 0:
            raise EpsError(f"grouped GEMM gave up on a bounded wait (code {st[0]}, CTA {st[1]})")


class CapturedStep:
    """A captured MoELayerFP8.forward (see MoELayerFP8.capture).  The graph holds the plan and GEMM buffers of its
    step; the layer's eager entry points stay usable beside it, but not while a replay is in flight."""

    def __init__(self, layer: MoELayerFP8, x, expert_indices, expert_weights, out, num_global_tokens=None):
        if layer.W != 1:
            raise EpsError("a layer step can be captured in a world of one only")
        if out is None or out.shape != (x.shape[0], layer.H) or out.dtype != torch.bfloat16:
            raise EpsError("capture needs the output tensor [T, H] bfloat16 the replays will write")
        self.layer, self.out = layer, out
        self.inputs = (x, expert_indices, expert_weights)
        ev, gev = layer.exchange_events, layer.gateup_events
        layer.exchange_events = layer.gateup_events = None   # timing events cannot be recorded inside a graph
        try:
            for _ in range(2):   # first-call set-up (function attributes, cached bounds, the side stream) stays outside
                layer.forward(x, expert_indices, expert_weights, num_global_tokens, out=out)
            torch.cuda.synchronize()
            layer.check_status()
            self.graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(self.graph):
                layer.forward(x, expert_indices, expert_weights, num_global_tokens, out=out)
            self.kernel_launches = layer.kernel_launches
        finally:
            layer.exchange_events, layer.gateup_events = ev, gev

    def replay(self) -> torch.Tensor:
        self.graph.replay()
        return self.out


def synthetic_expert_codes(cfg, expert: int, device, inter: int | None = None):
    """Random-init weights of one expert of a workloads.MoEConfig, generated (seeded by the expert id) and
    block-quantised on `device`: (W_gate_up codes [2I,H], scales, W_down codes [H,I], scales).  expert -1 is the
    shared expert (pass inter=cfg.shared_inter)."""
    from . import workloads

    a, b = workloads.make_expert_weights(cfg, expert, device=device, inter=inter)
    q1, s1 = ops.quant_block128(a)
    q2, s2 = ops.quant_block128(b)
    return q1, s1, q2, s2


def build_synthetic_layer(cfg, comm: Communicator | None = None, device=None, num_stages: int = 1, **kw) -> MoELayerFP8:
    """The layer of a benchmark configuration with random-init weights of that architecture: this rank's block of
    experts (rank * E/W ...) and the shared expert if the configuration has one."""
    comm = comm if comm is not None else Communicator()
    W, rank = comm.getWorldSize(), comm.getRank()
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    EL = cfg.num_experts // W
    H, I = cfg.hidden, cfg.inter
    wgu = torch.empty((EL, 2 * I, H), dtype=torch.uint8, device=dev)
    wgu_s = torch.empty((EL, 2 * I // 128, H // 128), dtype=torch.float32, device=dev)
    wd = torch.empty((EL, H, I), dtype=torch.uint8, device=dev)
    wd_s = torch.empty((EL, H // 128, I // 128), dtype=torch.float32, device=dev)
    for le in range(EL):
        wgu[le], wgu_s[le], wd[le], wd_s[le] = synthetic_expert_codes(cfg, rank * EL + le, dev)
    shared = None
    if cfg.shared_inter:
        shared = tuple(t.unsqueeze(0) for t in synthetic_expert_codes(cfg, -1, dev, inter=cfg.shared_inter))
    torch.cuda.synchronize(dev)
    return MoELayerFP8(H, I, cfg.num_experts, cfg.top_k, cfg.tokens_per_rank, wgu, wgu_s, wd, wd_s, comm=comm,
                       shared=shared, num_stages=num_stages, device=dev, **kw)
