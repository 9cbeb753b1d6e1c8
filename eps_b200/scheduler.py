"""Staged EPS scheduler: the host-side mirror of the reference's `Scheduler`
(python/eps/scheduler/scheduler.py:19-122 over src/scheduler/scheduler.cu:30-353).

Same constructor, same methods, same index layouts and stage semantics:
  rendezvous_and_plan -> prologue -> for each stage: dispatch, gemm_expand, <GEMMs>, local_reduce, combine
  -> epilogue.
What differs is underneath: plans come from two single-launch kernels (source side, expert side), rows move
with grid-filling gathers, and the exchanges are grouped NCCL send/recv (Communicator.exchange).  The FP8
path uses the slots the reference already has: `input_quanted`, `input_scales`, `recv_input_scales`.
"""
from __future__ import annotations

import numpy as np
import torch

from . import ops
from ._lib import EpsError
from .communication import Communicator


class Context:
    """Per-call plans (reference: Scheduler::Context, src/scheduler/context.cu)."""

    def __init__(self, num_tokens, num_global_tokens, num_stages, input_quanted):
        self.num_tokens = num_tokens
        self.num_global_tokens = num_global_tokens
        self.num_stages = num_stages
        self.input_quanted = input_quanted
        self.n_recv = None            # rows received (host int) once known
        self.host_dispatch = None     # (send_excl, send_incl, recv_excl, recv_incl) numpy, world > 1
        self.host_combine = None      # (ret_excl, ret_incl, coll_excl, coll_incl) numpy, world > 1


def _excl(incl: np.ndarray) -> np.ndarray:
    out = np.zeros_like(incl)
    out[1:] = incl[:-1]
    return out


def dispatch_windows(gathered: np.ndarray, rank: int, W: int, S: int):
    """Host view of one exchange from the all-gathered inclusive send plans `gathered[W, W*S]`:
    (send_excl, send_incl, recv_excl, recv_incl) as int64 arrays of W*S entries, rows counted in this rank's send
    order and receive order (source-major, then stage — reference alltoall_runner.cu:60-101)."""
    g = np.asarray(gathered, dtype=np.int64).reshape(W, W * S)
    send_incl = g[rank]
    counts = np.zeros((W, S), dtype=np.int64)  # rows rank r sends me at stage s
    for r in range(W):
        for s in range(S):
            i = rank * S + s
            counts[r, s] = g[r, i] - (g[r, i - 1] if i > 0 else 0)
    recv_incl = np.cumsum(counts.reshape(-1))
    return _excl(send_incl), send_incl, _excl(recv_incl), recv_incl


def stage_slices(windows, W: int, S: int, stage: int):
    """Per peer p: ((send_begin, send_end), (recv_begin, recv_end)) row ranges of one stage (stage < 0: all stages)."""
    s_ex, s_in, r_ex, r_in = windows
    out = []
    for p in range(W):
        if stage < 0:
            out.append(((int(s_ex[p * S]), int(s_in[p * S + S - 1])), (int(r_ex[p * S]), int(r_in[p * S + S - 1]))))
        else:
            i = p * S + stage
            out.append(((int(s_ex[i]), int(s_in[i])), (int(r_ex[i]), int(r_in[i]))))
    return out


class Scheduler:
    def __init__(self, top_k: int, num_experts: int, hidden_size: int, input_scales_dim: int,
                 max_num_tokens_per_gpu: int, comm: Communicator | None, local_num_experts: int,
                 input_dtype: torch.dtype = torch.bfloat16, device=None) -> None:
        self.comm = comm if comm is not None else Communicator()
        self.W = self.comm.getWorldSize()
        self.rank = self.comm.getRank()
        self.top_k, self.num_experts, self.hidden = top_k, num_experts, hidden_size
        self.scales_dim = input_scales_dim
        self.max_tok = max_num_tokens_per_gpu
        if num_experts % self.W != 0:
            raise EpsError(f"num_experts {num_experts} is not divisible by ep_world_size {self.W}")
        self.local_num_experts = num_experts // self.W
        # local_num_experts is what the reference passes on as max_num_stages (scheduler.py:37 vs
        # scheduler_ops.cu:25,35): an upper bound only, nothing is sized from it here
        self.lo = self.rank * self.local_num_experts
        self.hi = self.lo + self.local_num_experts
        self.device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        self.input_dtype = input_dtype
        rows = max(1, self.max_tok * self.W)   # reference arena sizing: max_tok * W rows each way (msccl_comm.cu:191-199)
        self.arena_rows = rows
        dev = self.device
        in_dt = torch.uint8 if input_dtype in (torch.uint8, torch.float8_e4m3fn) else input_dtype

        def pair(cols, dtype):
            s = torch.empty((rows, cols), dtype=dtype, device=dev)
            return s, (s if self.W == 1 else torch.empty((rows, cols), dtype=dtype, device=dev))

        self.send_idx, self.recv_idx = pair(top_k, torch.int32)
        self.send_w, self.recv_w = pair(top_k, torch.float32)
        self.send_hidden, self.recv_hidden = pair(hidden_size, in_dt)
        self.send_out, self.recv_out = pair(hidden_size, torch.bfloat16)
        if input_scales_dim > 0:
            self.send_scales, self.recv_scales = pair(input_scales_dim, torch.float32)
        else:
            self.send_scales = self.recv_scales = None
        self.context: Context | None = None

    def destroy(self) -> None:
        """The reference frees its C++ object here; this object owns only tensors, which the allocator reclaims."""
        self.context = None

    # ------------------------------------------------------------------ plans

    def get_context(self, num_tokens, num_global_tokens, num_stages, input_quanted) -> Context:
        if num_stages <= 0 or self.local_num_experts % num_stages != 0:
            raise EpsError(f"Invalid num_stages: {num_stages} for local_num_experts: {self.local_num_experts}")
        if num_tokens > self.max_tok:
            raise EpsError(f"num_tokens {num_tokens} exceeds max_num_tokens_per_gpu {self.max_tok}")
        return Context(num_tokens, num_global_tokens, num_stages, input_quanted)

    def rendezvous_and_plan(self, expert_indices: torch.Tensor, expert_scales: torch.Tensor, num_global_tokens,
                            num_stages, input_quanted, host_sync: bool = True, max_cluster: int = 0):
        """-> (exclusive_sum [EL+1] int32 on the device, number of unique rows this rank receives).

        With a world of one and host_sync=False nothing is copied to the host and the second value is the
        upper bound num_tokens (every later step reads its bounds on the device).
        max_cluster caps the CTAs of the plan kernels (0 = up to 8)."""
        T = expert_indices.shape[0]
        ctx = self.context = self.get_context(T, num_global_tokens, num_stages, input_quanted)
        W, S, k = self.W, num_stages, self.top_k
        # --- rendezvous (reference scheduler.cu:231-283): dispatch plan, plan exchange, receive count
        (ctx.send_map, ctx.send_incl, ctx.glob_map, ctx.coll_incl, ctx.zero_scale, ctx.send_bounds) = ops.source_plans(
            expert_indices, expert_scales, self.num_experts, W, S, with_bounds=True, max_cluster=max_cluster)
        if W == 1:
            ctx.recv_incl = ctx.send_incl
            if host_sync:
                ctx.n_recv = int(ctx.send_incl[-1].item())
                rows_bound = ctx.n_recv
            else:
                ctx.n_recv = None
                rows_bound = T
        else:
            # One all-gather carries both inclusive plans of every rank: what it sends (dispatch) and what it will
            # collect back (combine).  The rows this rank returns to peer p are the rows p collects from it, so the
            # host gets the combine windows from the same single read and never waits for the expert plans.
            both = self.comm.all_gather(torch.cat([ctx.send_incl, ctx.coll_incl]))   # [W, 2*W*S] on the device
            gathered = both[:, :W * S].contiguous()
            ctx.recv_incl, ctx.remote_offset = ops.recv_plan(gathered, self.rank, W, S)
            g2 = both.cpu().numpy()                                      # the one host read of the rendezvous
            g = g2[:, :W * S]
            ctx.host_dispatch = dispatch_windows(g, self.rank, W, S)
            coll = dispatch_windows(g2[:, W * S:], self.rank, W, S)      # (coll_excl, coll_incl, ret_excl, ret_incl)
            ctx.host_combine = (coll[2], coll[3], coll[0], coll[1])
            ctx.n_recv = int(ctx.host_dispatch[3][-1])
            rows_bound = ctx.n_recv
            if ctx.n_recv > self.arena_rows:
                raise EpsError("received rows exceed the arena")
        ctx.rows_bound = rows_bound
        # --- plan (reference scheduler.cu:286-353)
        self._expand_for_comm(expert_indices, self.send_idx, ctx)
        self._all2all(self.send_idx, self.recv_idx, ctx, -1, combine=False)
        (ctx.excl, ctx.gemm_map, ctx.inv_gemm, ctx.scale_map, ctx.red_map, ctx.ret_incl) = ops.expert_plans(
            self.recv_idx, ctx.recv_incl, k, self.lo, self.hi, W, S, self.max_tok, max(rows_bound, 0),
            max_cluster=max_cluster)
        return ctx.excl, (ctx.n_recv if ctx.n_recv is not None else rows_bound)

    # ------------------------------------------------------------------ data path

    def _expand_for_comm(self, src: torch.Tensor, dst: torch.Tensor, ctx: Context) -> None:
        """dst[i] = src[send_map[i] % T] for the rows that will be sent (reference expandForComm)."""
        T = ctx.num_tokens
        if T == 0:
            return
        bound = min(T * min(self.W, self.top_k), dst.shape[0])
        ops.gather_rows(src, dst[:bound], ctx.send_map, 1, T, bounds=ctx.send_bounds, b0=0,
                        b1=self.W * ctx.num_stages)

    def _all2all(self, send: torch.Tensor, recv: torch.Tensor, ctx: Context, stage: int, combine: bool) -> None:
        self._all2all_many([(send, recv, stage)], ctx, combine)

    def _all2all_many(self, items, ctx: Context, combine: bool) -> None:
        """One grouped exchange for several (send arena, receive arena, stage) triples."""
        if self.W == 1:
            return  # recv aliases send
        W, S = self.W, ctx.num_stages
        sends = [[] for _ in range(W)]
        recvs = [[] for _ in range(W)]
        for send, recv, stage in items:
            sl = stage_slices(ctx.host_combine if combine else ctx.host_dispatch, W, S, stage)
            for p, ((a, b), (c, d)) in enumerate(sl):
                sends[p].append(send[a:b])
                recvs[p].append(recv[c:d])
        self.comm.exchange(sends, recvs)

    def exchange_bytes(self, stage: int, combine: bool):
        """(bytes this rank sends to its peers, bytes it receives from them) in the exchange of one stage, from the
        host view of the plans; rows that stay on this rank are not counted.  A dispatched row is its FP8 (or bf16)
        hidden row + its scales + k expert ids + k gate weights; a returned row is bf16 hidden."""
        ctx = self.context
        if self.W == 1 or ctx is None or ctx.host_dispatch is None:
            return 0, 0
        sl = stage_slices(ctx.host_combine if combine else ctx.host_dispatch, self.W, ctx.num_stages, stage)
        out_rows = sum(b - a for p, ((a, b), _) in enumerate(sl) if p != self.rank)
        in_rows = sum(d - c for p, (_, (c, d)) in enumerate(sl) if p != self.rank)
        if combine:
            row = self.hidden * 2
        else:
            row = self.hidden * self.send_hidden.element_size() + self.scales_dim * 4 + self.top_k * 8
        return out_rows * row, in_rows * row

    def prologue(self, expert_scales: torch.Tensor, hidden_states: torch.Tensor, input_scales=None,
                 recv_input_scales=None, raw_input: torch.Tensor | None = None, defer_exchange: bool = False) -> None:
        """raw_input: the bf16 tokens the identity (zero-computation) experts pass through; defaults to
        hidden_states when that is bf16 (reference ZeroReducePlan::setRawInput, scheduler.cu:76).
        defer_exchange=True (world > 1): the gate weights and the input scales are not exchanged here but ride in
        the same grouped exchange as the first `dispatch`; `finish_prologue()` must follow that dispatch."""
        ctx = self.context
        ctx.raw_input = raw_input if raw_input is not None else hidden_states
        defer = defer_exchange and self.W > 1
        ctx.deferred = [] if defer else None
        self._expand_for_comm(expert_scales, self.send_w, ctx)
        if defer:
            ctx.deferred.append((self.send_w, self.recv_w, -1))
        else:
            self._all2all(self.send_w, self.recv_w, ctx, -1, combine=False)
        h = hidden_states.view(torch.uint8) if hidden_states.dtype == torch.float8_e4m3fn else hidden_states
        if h.dtype != self.send_hidden.dtype:
            raise EpsError(f"hidden_states must have dtype {self.send_hidden.dtype}, got {h.dtype}")
        self._expand_for_comm(h, self.send_hidden, ctx)
        if ctx.input_quanted:
            if input_scales is None or recv_input_scales is None or self.send_scales is None:
                raise EpsError("input_quanted needs input_scales, recv_input_scales and input_scales_dim > 0")
            self._expand_for_comm(input_scales, self.send_scales, ctx)
            if defer:
                ctx.deferred.append((self.send_scales, self.recv_scales, -1))
                ctx.deferred_scales_out = recv_input_scales
                return
            self._all2all(self.send_scales, self.recv_scales, ctx, -1, combine=False)
            ops.gather_rows(self.recv_scales, recv_input_scales, ctx.gemm_map, self.top_k, ops.INT32_MAX,
                            bounds=ctx.excl, b0=0, b1=self.local_num_experts)

    def finish_prologue(self) -> None:
        """After the dispatch that carried a deferred prologue: the received input scales go to GEMM order."""
        ctx = self.context
        out = getattr(ctx, "deferred_scales_out", None)
        if out is not None:
            ops.gather_rows(self.recv_scales, out, ctx.gemm_map, self.top_k, ops.INT32_MAX, bounds=ctx.excl, b0=0,
                            b1=self.local_num_experts)
            ctx.deferred_scales_out = None

    def dispatch(self, stage_idx: int) -> None:
        ctx = self.context
        items = [(self.send_hidden, self.recv_hidden, stage_idx)]
        if getattr(ctx, "deferred", None):
            items = ctx.deferred + items      # gate weights and input scales of ALL stages go with the first dispatch
            ctx.deferred = None
        self._all2all_many(items, ctx, combine=False)

    def gemm_expand(self, gemm_input: torch.Tensor, stage_idx: int) -> None:
        """gemm_input[p] = received row gemm_map[p] / top_k for the stage's experts (reference expandForGemm)."""
        ctx = self.context
        eps_ = self.local_num_experts // ctx.num_stages
        b0, b1 = (0, self.local_num_experts) if stage_idx < 0 else (eps_ * stage_idx, eps_ * (stage_idx + 1))
        g = gemm_input.view(torch.uint8) if gemm_input.dtype == torch.float8_e4m3fn else gemm_input
        ops.gather_rows(self.recv_hidden, g, ctx.gemm_map, self.top_k, ops.INT32_MAX, bounds=ctx.excl, b0=b0, b1=b1)

    def local_reduce(self, gemm_output: torch.Tensor, stage_idx: int, pre_weighted: bool = False) -> None:
        """Sums the rows of each received token over this rank's experts into the return buffer.
        pre_weighted=False: reference arithmetic (bf16(weight) * row, bf16 accumulate, local_reducer.cu:103-181).
        pre_weighted=True : rows already carry their gate weight (fused down-GEMM epilogue); fp32 accumulate."""
        ctx = self.context
        if pre_weighted:
            ops.local_reduce(gemm_output, ctx.red_map, ctx.ret_incl, self.top_k, self.W, ctx.num_stages, stage_idx,
                             self.send_out, max_rows=max(ctx.rows_bound, 0))
        else:
            ops.local_reduce_ref(gemm_output, self.recv_w, ctx.scale_map, ctx.red_map, ctx.ret_incl, self.top_k,
                                 self.W, ctx.num_stages, stage_idx, self.send_out, max_rows=max(ctx.rows_bound, 0))

    def combine(self, stage_idx: int) -> None:
        self._all2all(self.send_out, self.recv_out, self.context, stage_idx, combine=True)

    def epilogue(self, output: torch.Tensor, shared: torch.Tensor | None = None, ref_arith: bool = True) -> None:
        """output[t] = (shared[t] +) sum over ranks of the returned partial rows + x[t] * zero_scale[t]
        (reference globalReduce + zeroReduce, scheduler.cu:205-228).  ref_arith=False accumulates in fp32."""
        ctx = self.context
        x = ctx.raw_input
        zero = ctx.zero_scale if (x is not None and x.dtype == torch.bfloat16) else None
        ops.global_reduce(self.recv_out, ctx.glob_map, output, self.W, shared=shared, x=x if zero is not None else None,
                          zero_scale=zero, ref_arith=ref_arith)

    def reduce_single_rank(self, gemm_output: torch.Tensor, output: torch.Tensor, shared=None) -> None:
        """ep_world_size == 1 only: local_reduce(all stages) + combine + epilogue in one kernel, rows pre-weighted."""
        if self.W != 1:
            raise EpsError("reduce_single_rank needs ep_world_size == 1")
        ctx = self.context
        x = ctx.raw_input
        zero = ctx.zero_scale if (x is not None and x.dtype == torch.bfloat16) else None
        ops.reduce_ep1(gemm_output, ctx.red_map, ctx.glob_map, ctx.ret_incl, ctx.num_stages, self.top_k, output,
                       shared=shared, x=x if zero is not None else None, zero_scale=zero)

    # helper used by the fused layer
    def gemm_row_weights(self) -> torch.Tensor:
        ctx = self.context
        return ops.gather_row_weights(self.recv_w, ctx.gemm_map, ctx.excl, self.local_num_experts,
                                      max(ctx.rows_bound, 0) * self.top_k)
