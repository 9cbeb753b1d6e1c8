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

import ctypes
import sys

import numpy as np
import torch

from . import _lib, ops
from ._lib import EpsError
from .communication import Communicator, SymmetricMemoryUnavailable

ARENA_IDX, ARENA_WEIGHTS, ARENA_HIDDEN, ARENA_SCALES, ARENA_OUT, ARENA_RECV_PLAN = range(6)
PUT_META, PUT_SCALES, PUT_HIDDEN = 1, 2, 4
FLAG_META = 1


class _RawDeviceMemory:
    """Lets torch view device memory this package allocated itself (zero-copy, not owning)."""

    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 2}


def device_view(ptr: int, shape, dtype: torch.dtype, device) -> torch.Tensor:
    n = int(np.prod(shape)) * torch.empty((), dtype=dtype).element_size()
    flat = torch.as_tensor(_RawDeviceMemory(ptr, max(n, 1)), device=device)
    return flat[:n].view(dtype).view(*shape)


class PeerExchange:
    """This rank's end of the device-side exchange (include/eps_b200.h, "Expert-parallel exchange over peer
    memory"): the symmetric region, the C handle and torch views of the receive arenas."""

    def __init__(self, comm: Communicator, max_tok: int, S_max: int, k: int, H: int, hidden_elem: int,
                 scales_dim: int, device):
        self.comm, self.S_max = comm, S_max
        W = comm.getWorldSize()
        nbytes = ctypes.c_int64()
        _lib.call("epsb_exchange_region_bytes", W, max_tok, S_max, k, H, hidden_elem, scales_dim, ctypes.byref(nbytes))
        self.local, peers = comm.symm_alloc(nbytes.value)
        arr = (ctypes.c_void_p * W)(*peers)
        h = ctypes.c_void_p()
        _lib.call("epsb_exchange_create", comm.getRank(), W, max_tok, S_max, k, H, hidden_elem, scales_dim, arr,
                  ctypes.byref(h))
        self.handle = h
        self.epoch = 0
        rows = max(max_tok, 1) * W
        hid_dt = torch.uint8 if hidden_elem == 1 else torch.bfloat16

        def arena(which, par, shape, dtype):
            p = ctypes.c_void_p()
            _lib.call("epsb_exchange_arena", self.handle, which, par, ctypes.byref(p))
            return device_view(p.value, shape, dtype, device)

        self.recv_idx = [arena(ARENA_IDX, par, (rows, k), torch.int32) for par in (0, 1)]
        self.recv_w = [arena(ARENA_WEIGHTS, par, (rows, k), torch.float32) for par in (0, 1)]
        self.recv_hidden = [arena(ARENA_HIDDEN, par, (rows, H), hid_dt) for par in (0, 1)]
        self.recv_scales = ([arena(ARENA_SCALES, par, (rows, scales_dim), torch.float32) for par in (0, 1)]
                            if scales_dim > 0 else [None, None])
        self.recv_out = arena(ARENA_OUT, 0, (rows, H), torch.bfloat16)
        self.recv_plan = arena(ARENA_RECV_PLAN, 0, (W * S_max,), torch.int32)
        self.status = torch.zeros(4, dtype=torch.int32, device=device)
        self.timeout_ns = 0   # 0 = the library's default (2 s)

    def begin(self) -> int:
        e = ctypes.c_int()
        _lib.call("epsb_exchange_begin", self.handle, ctypes.byref(e))
        self.epoch = e.value
        return self.epoch

    @property
    def par(self) -> int:
        return self.epoch & 1

    def flag_dispatch(self, stage: int) -> int:
        return 2 + max(stage, 0)

    def flag_combine(self, stage: int) -> int:
        return 2 + self.S_max + max(stage, 0)

    def publish_plans(self, send_incl, coll_incl, S):
        _lib.call("epsb_exchange_publish_plans", self.handle, _lib.ptr(send_incl), _lib.ptr(coll_incl), S,
                  _lib.stream_ptr())

    def recv_plans(self, S, recv_incl):
        _lib.call("epsb_exchange_recv_plans", self.handle, S, _lib.ptr(recv_incl), _lib.ptr(self.status),
                  self.timeout_ns, _lib.stream_ptr())

    def put(self, flag_slot, stage, mask, idx, w, hidden, scales, send_map, send_incl, T, S):
        _lib.call("epsb_exchange_put", self.handle, flag_slot, stage, mask, _lib.ptr(idx), _lib.ptr(w),
                  _lib.ptr(hidden), _lib.ptr(scales), _lib.ptr(send_map), _lib.ptr(send_incl), T, S,
                  _lib.stream_ptr())

    def wait(self, flag_slot):
        _lib.call("epsb_exchange_wait", self.handle, flag_slot, _lib.ptr(self.status), self.timeout_ns,
                  _lib.stream_ptr())

    def local_reduce_put(self, flag_slot, y, red_map, ret_incl, S, stage, max_rows):
        _lib.call("epsb_exchange_local_reduce_put", self.handle, flag_slot, _lib.ptr(y), _lib.ptr(red_map),
                  _lib.ptr(ret_incl), S, stage, max_rows, _lib.stream_ptr())

    def check_status(self) -> None:
        st = self.status.cpu().tolist()
        if st[0] != 0:
            raise EpsError(f"expert-parallel exchange failed (code {st[0]}, peer {st[1]})")

    def destroy(self) -> None:
        if self.handle is not None:
            self.comm.symm_free(self.local)
            _lib.call("epsb_exchange_destroy", self.handle)
            self.handle = None


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

        self.peer = None
        self.hidden_dtype = in_dt
        if self.W > 1 and self.comm.transport == "ipc":
            # device-side exchange: the receive arenas live in the symmetric region, nothing is staged for sending
            try:
                self.peer = PeerExchange(self.comm, self.max_tok, self.local_num_experts, top_k, hidden_size,
                                         torch.empty((), dtype=in_dt).element_size(), input_scales_dim, dev)
            except SymmetricMemoryUnavailable as e:
                # raised on every rank together; a transport the caller did not insist on gives way to the other one
                if not self.comm.transport_is_a_choice:
                    raise
                print(f"eps_b200: {e}; expert-parallel exchange falls back to the NCCL transport", file=sys.stderr)
                self.comm.transport = "nccl"
        if self.peer is not None:
            self.recv_out = self.peer.recv_out
            self._select_arenas()
        else:
            self.send_idx, self.recv_idx = pair(top_k, torch.int32)
            self.send_w, self.recv_w = pair(top_k, torch.float32)
            self.send_hidden, self.recv_hidden = pair(hidden_size, in_dt)
            self.send_out, self.recv_out = pair(hidden_size, torch.bfloat16)
            if input_scales_dim > 0:
                self.send_scales, self.recv_scales = pair(input_scales_dim, torch.float32)
            else:
                self.send_scales = self.recv_scales = None
        self.context: Context | None = None

    def _select_arenas(self) -> None:
        """The dispatch arenas of the current call (they alternate with the exchange's epoch)."""
        pe, par = self.peer, self.peer.par
        self.recv_idx, self.recv_w = pe.recv_idx[par], pe.recv_w[par]
        self.recv_hidden, self.recv_scales = pe.recv_hidden[par], pe.recv_scales[par]

    def destroy(self) -> None:
        """Collective when the device-side exchange is in use (the symmetric region is unmapped everywhere)."""
        self.context = None
        if self.peer is not None:
            self.peer.destroy()
            self.peer = None

    # ------------------------------------------------------------------ plans

    def get_context(self, num_tokens, num_global_tokens, num_stages, input_quanted) -> Context:
        if num_stages <= 0 or self.local_num_experts % num_stages != 0:
            raise EpsError(f"Invalid num_stages: {num_stages} for local_num_experts: {self.local_num_experts}")
        if num_tokens > self.max_tok:
            raise EpsError(f"num_tokens {num_tokens} exceeds max_num_tokens_per_gpu {self.max_tok}")
        return Context(num_tokens, num_global_tokens, num_stages, input_quanted)

    def rendezvous_and_plan(self, expert_indices: torch.Tensor, expert_scales: torch.Tensor, num_global_tokens,
                            num_stages, input_quanted, host_sync: bool = True, max_cluster: int = 0,
                            payload=None, after_put=None):
        """-> (exclusive_sum [EL+1] int32 on the device, number of unique rows this rank receives).

        With a world of one and host_sync=False nothing is copied to the host and the second value is the
        upper bound num_tokens (every later step reads its bounds on the device).
        max_cluster caps the CTAs of the plan kernels (0 = up to 8).
        With the device-side exchange nothing is read on the host either: the second value is the arena size, and
        `payload` = (hidden_states, input_scales) lets the rows travel in the same launch as the expert ids
        (`dispatch` is then a no-op); `after_put` is called between this rank's put and the wait for the peers'
        rows, so that work which needs no peer (the shared expert) runs while those rows are on their way."""
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
        elif self.peer is not None:
            pe = self.peer
            if S > pe.S_max:
                raise EpsError(f"Invalid num_stages: {S} for local_num_experts: {self.local_num_experts}")
            pe.begin()
            self._select_arenas()
            pe.publish_plans(ctx.send_incl, ctx.coll_incl, S)
            ctx.recv_incl = torch.empty((W * S,), dtype=torch.int32, device=self.device)
            pe.recv_plans(S, ctx.recv_incl)
            mask = PUT_META
            ctx.eager = payload is not None
            hidden = scales = None
            if ctx.eager:
                hidden, scales = payload
                hidden = hidden.view(torch.uint8) if hidden.dtype == torch.float8_e4m3fn else hidden
                if hidden.dtype != self.hidden_dtype:
                    raise EpsError(f"hidden_states must have dtype {self.hidden_dtype}, got {hidden.dtype}")
                mask |= PUT_HIDDEN | (PUT_SCALES if scales is not None else 0)
            pe.put(FLAG_META, -1, mask, expert_indices, expert_scales, hidden, scales, ctx.send_map, ctx.send_incl, T, S)
            if after_put is not None:
                after_put()
            pe.wait(FLAG_META)
            ctx.n_recv = None
            rows_bound = self.arena_rows
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
        if self.peer is None:
            self._expand_for_comm(expert_indices, self.send_idx, ctx)
            self._all2all(self.send_idx, self.recv_idx, ctx, -1, combine=False)
        (ctx.excl, ctx.gemm_map, ctx.inv_gemm, ctx.scale_map, ctx.red_map, ctx.ret_incl) = ops.expert_plans(
            self.recv_idx, ctx.recv_incl, k, self.lo, self.hi, W, S, self.max_tok, max(rows_bound, 0),
            status=self.peer.status[2:] if self.peer is not None else None, max_cluster=max_cluster)
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
        if self.W == 1 or ctx is None:
            return 0, 0
        if ctx.host_dispatch is None:
            # device-side exchange: the plans never came to the host; read them now (synchronises: not for hot paths)
            if self.peer is None:
                return 0, 0
            W, S = self.W, ctx.num_stages
            if combine:
                mine, theirs = ctx.ret_incl.cpu().numpy(), ctx.coll_incl.cpu().numpy()
            else:
                mine, theirs = ctx.send_incl.cpu().numpy(), ctx.recv_incl.cpu().numpy()
            win = (_excl(mine.astype(np.int64)), mine.astype(np.int64), _excl(theirs.astype(np.int64)),
                   theirs.astype(np.int64))
            sl = stage_slices(win, W, S, stage)
        else:
            sl = stage_slices(ctx.host_combine if combine else ctx.host_dispatch, self.W, ctx.num_stages, stage)
        return self._bytes_of(sl, combine)

    def _bytes_of(self, sl, combine: bool):
        out_rows = sum(b - a for p, ((a, b), _) in enumerate(sl) if p != self.rank)
        in_rows = sum(d - c for p, (_, (c, d)) in enumerate(sl) if p != self.rank)
        if combine:
            row = self.hidden * 2
        else:
            elem = torch.empty((), dtype=self.hidden_dtype).element_size()
            row = self.hidden * elem + self.scales_dim * 4 + self.top_k * 8
        return out_rows * row, in_rows * row

    def prologue(self, expert_scales: torch.Tensor, hidden_states: torch.Tensor, input_scales=None,
                 recv_input_scales=None, raw_input: torch.Tensor | None = None, defer_exchange: bool = False) -> None:
        """raw_input: the bf16 tokens the identity (zero-computation) experts pass through; defaults to
        hidden_states when that is bf16 (reference ZeroReducePlan::setRawInput, scheduler.cu:76).
        defer_exchange=True (world > 1): the gate weights and the input scales are not exchanged here but ride in
        the same grouped exchange as the first `dispatch`; `finish_prologue()` must follow that dispatch."""
        ctx = self.context
        ctx.raw_input = raw_input if raw_input is not None else hidden_states
        if self.peer is not None:
            # device-side exchange: rows are read through the dispatch plan when they are sent; nothing to stage
            h = hidden_states.view(torch.uint8) if hidden_states.dtype == torch.float8_e4m3fn else hidden_states
            if h.dtype != self.hidden_dtype:
                raise EpsError(f"hidden_states must have dtype {self.hidden_dtype}, got {h.dtype}")
            if ctx.input_quanted and (input_scales is None or self.scales_dim == 0):
                raise EpsError("input_quanted needs input_scales and input_scales_dim > 0")
            # recv_input_scales may be None: a GEMM with index-driven A loads reads the scales where they arrive
            ctx.src_hidden, ctx.src_scales = h, (input_scales if ctx.input_quanted else None)
            ctx.src_idx_w = None
            ctx.scales_out = recv_input_scales if ctx.input_quanted else None
            return
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
        if self.peer is not None:
            if getattr(ctx, "eager", False):
                return   # the rows travelled with the expert ids
            pe = self.peer
            mask = PUT_HIDDEN | (PUT_SCALES if ctx.src_scales is not None else 0)
            pe.put(pe.flag_dispatch(stage_idx), stage_idx, mask, None, None, ctx.src_hidden, ctx.src_scales,
                   ctx.send_map, ctx.send_incl, ctx.num_tokens, ctx.num_stages)
            pe.wait(pe.flag_dispatch(stage_idx))
            return
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
        if self.peer is not None and getattr(ctx, "scales_out", None) is not None:
            # the stage's input scales arrived with its rows: bring them to GEMM order too
            ops.gather_rows(self.recv_scales, ctx.scales_out, ctx.gemm_map, self.top_k, ops.INT32_MAX,
                            bounds=ctx.excl, b0=b0, b1=b1)

    def local_reduce(self, gemm_output: torch.Tensor, stage_idx: int, pre_weighted: bool = False) -> None:
        """Sums the rows of each received token over this rank's experts into the return buffer.
        pre_weighted=False: reference arithmetic (bf16(weight) * row, bf16 accumulate, local_reducer.cu:103-181).
        pre_weighted=True : rows already carry their gate weight (fused down-GEMM epilogue); fp32 accumulate."""
        ctx = self.context
        if self.peer is not None:
            if not pre_weighted:
                raise EpsError("the device-side exchange returns pre-weighted rows (pre_weighted=True); the reference's "
                               "bf16 arithmetic is available with transport 'nccl'")
            pe = self.peer
            pe.local_reduce_put(pe.flag_combine(stage_idx), gemm_output, ctx.red_map, ctx.ret_incl, ctx.num_stages,
                                stage_idx, max(ctx.rows_bound, 0))
            return
        if pre_weighted:
            ops.local_reduce(gemm_output, ctx.red_map, ctx.ret_incl, self.top_k, self.W, ctx.num_stages, stage_idx,
                             self.send_out, max_rows=max(ctx.rows_bound, 0))
        else:
            ops.local_reduce_ref(gemm_output, self.recv_w, ctx.scale_map, ctx.red_map, ctx.ret_incl, self.top_k,
                                 self.W, ctx.num_stages, stage_idx, self.send_out, max_rows=max(ctx.rows_bound, 0))

    def combine(self, stage_idx: int) -> None:
        if self.peer is not None:
            self.peer.wait(self.peer.flag_combine(stage_idx))   # the rows were stored by the peers' local_reduce
            return
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

    def gemm_sources(self, expert_scales: torch.Tensor, hidden: torch.Tensor, scales: torch.Tensor | None):
        """For GEMMs with index-driven A loads (no expandForGemm pass): -> (a_rows int32 [GEMM rows], row_w fp32,
        source rows, source scales).  GEMM row d reads row a_rows[d] of the source: the receive arena, or in a world of
        one the caller's own `hidden` / `scales` (the receive order is the send order there, so nothing is staged at
        all).  row_w[d] is the row's gate weight."""
        ctx = self.context
        EL, k = self.local_num_experts, self.top_k
        n = max(ctx.rows_bound, 0) * min(k, EL)
        if self.W == 1:
            T = ctx.num_tokens
            a_rows, row_w = ops.gemm_row_sources(ctx.gemm_map, ctx.excl, EL, k, n, w_src=expert_scales,
                                                 send_map=ctx.send_map if T > 0 else None, T=T)
            return a_rows, row_w, hidden, scales
        a_rows, row_w = ops.gemm_row_sources(ctx.gemm_map, ctx.excl, EL, k, n, w_src=self.recv_w)
        return a_rows, row_w, self.recv_hidden, self.recv_scales

    # helper used by the fused layer
    def gemm_row_weights(self) -> torch.Tensor:
        ctx = self.context
        return ops.gather_row_weights(self.recv_w, ctx.gemm_map, ctx.excl, self.local_num_experts,
                                      max(ctx.rows_bound, 0) * self.top_k)
