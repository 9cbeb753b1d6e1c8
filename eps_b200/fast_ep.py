"""Non-staged expert-parallel dispatch / combine: the host-side mirror of the reference's fast_ep `AllToAll`
(python/eps/fast_ep/all_to_all.py:8-68 over src/fast_ep/all_to_all/fast_ep.cu:63-215).

dispatch: count-sort the (token, slot) pairs by GLOBAL expert (rows of one expert in descending pair index, the
reference's order), scatter the token rows into send order, exchange, regroup [source][expert] -> [expert][source].
combine: the inverse regroup and exchange, then the fp32-accumulated weighted sum over the k slots, where a
zero-computation slot reads the raw input token.
"""
from __future__ import annotations

import numpy as np
import torch

from . import ops
from ._lib import EpsError
from .communication import Communicator


class AllToAll:
    def __init__(self, top_k: int, num_experts: int, hidden_size: int, max_num_global_tokens: int,
                 comm: Communicator | None, dtype: torch.dtype = torch.bfloat16, device=None) -> None:
        self.comm = comm if comm is not None else Communicator()
        self.W, self.rank = self.comm.getWorldSize(), self.comm.getRank()
        if num_experts % self.W:
            raise EpsError(f"num_experts {num_experts} is not divisible by ep_world_size {self.W}")
        self.k, self.E, self.H = top_k, num_experts, hidden_size
        self.EL = num_experts // self.W
        self.dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        rows = max(1, max_num_global_tokens * top_k)   # reference arena: every pair may land on one rank
        self.rows = rows
        self.send = torch.empty((rows, hidden_size), dtype=dtype, device=self.dev)
        self.recv = self.send if self.W == 1 else torch.empty((rows, hidden_size), dtype=dtype, device=self.dev)
        self.ctx = None

    def destroy(self) -> None:
        """The reference frees its C++ object here; this object owns only tensors."""

    def dispatch(self, out_exclusive_sum: torch.Tensor, out_expert_x: torch.Tensor, dp_x: torch.Tensor,
                 indices: torch.Tensor, num_global_tokens: int) -> None:
        T = indices.shape[0]
        W, EL = self.W, self.EL
        if T * self.k > self.rows:
            raise EpsError("tokens exceed max_num_global_tokens")
        excl, mapping = ops.fastep_expand_plan(indices, self.E)
        if T > 0:
            ops.scatter_rows(dp_x, self.send, mapping, self.k, T * self.k)
        ag = self.comm.all_gather(excl)                                   # [W, E+1]
        plan = ops.fastep_plan(ag, self.rank, W, self.E, gemm_plan=out_exclusive_sum)
        remote_recv, local_send, _, arr_src, arr_rows, arr_dst = plan
        host = None
        if W > 1:
            g = ag.cpu().numpy().astype(np.int64)                         # the one host read
            send_b = g[self.rank, np.arange(W) * EL]
            send_e = g[self.rank, (np.arange(W) + 1) * EL]
            cnt_in = g[:, (self.rank + 1) * EL] - g[:, self.rank * EL]    # rows each source sends me
            recv_e = np.cumsum(cnt_in)
            recv_b = recv_e - cnt_in
            host = (send_b, send_e, recv_b, recv_e, g)
            if int(recv_e[-1]) > self.rows or int(recv_e[-1]) > out_expert_x.shape[0]:
                raise EpsError("received rows exceed the buffers")
            self.comm.exchange([self.send[int(a):int(b)] for a, b in zip(send_b, send_e)],
                               [self.recv[int(a):int(b)] for a, b in zip(recv_b, recv_e)])
        ops.arrange_rows(self.recv, out_expert_x, arr_src, arr_rows, arr_dst, EL * W, out_expert_x.shape[0])
        self.ctx = dict(T=T, mapping=mapping, dp_x=dp_x, arr=(arr_src, arr_rows, arr_dst), host=host)

    def combine(self, out_tokens: torch.Tensor, weights: torch.Tensor, expert_y: torch.Tensor,
                num_global_tokens: int, shared: torch.Tensor | None = None) -> None:
        c = self.ctx
        if c is None:
            raise EpsError("combine called before dispatch")
        W, EL = self.W, self.EL
        arr_src, arr_rows, arr_dst = c["arr"]
        # inverse regroup: [expert][source] -> [source][expert] in the return-send buffer (the receive buffer of dispatch)
        ops.arrange_rows(expert_y, self.recv, arr_dst, arr_rows, arr_src, EL * W, expert_y.shape[0])
        if W > 1:
            send_b, send_e, recv_b, recv_e, _ = c["host"]
            # what I received from p goes back to p and lands where p sent it from
            self.comm.exchange([self.recv[int(a):int(b)] for a, b in zip(recv_b, recv_e)],
                               [self.send[int(a):int(b)] for a, b in zip(send_b, send_e)])
        ops.fastep_reduce(self.send, c["dp_x"], weights, c["mapping"], out_tokens, shared=shared)
