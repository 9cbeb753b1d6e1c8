"""Expert-parallel communicator: the transport under Scheduler and fast_ep.AllToAll.

Mirrors the surface of the reference's MscclppCommunicator (python/eps/communication/__init__.py:35-71,
src/communication/msccl_comm.cuh:14): create from a unique id + (rank, world, ranks_per_node), barrier,
rank/world queries.  The reference moves bytes with mscclpp SM-copy kernels over CUDA-IPC arenas; here
two transports exist.  "ipc" (the default on GPUs): every rank's receive arenas live in a symmetric region that
all ranks of the box map through CUDA IPC, and the exchange is done by this library's own kernels storing rows
straight into the destination's arena (see Scheduler and include/eps_b200.h, "Expert-parallel exchange over peer
memory"); torch.distributed only carries the 64-byte memory handles at set-up.  "nccl": the variable-size
all-to-all is one grouped NCCL send/recv per call (gloo on CPU for tests), launched through torch.distributed,
with one host read of the exchanged plans per call.  A world of one never touches a process group.
"""
from __future__ import annotations

from dataclasses import dataclass

import ctypes

import torch
import torch.distributed as dist

from . import _lib


@dataclass
class CommunicatorParams:
    rank: int
    ep_world_size: int
    num_ranks_per_node: int


class SymmetricMemoryUnavailable(RuntimeError):
    """Raised by Communicator.symm_alloc on EVERY rank when any rank could not allocate or map the shared regions."""


class Communicator:
    """One expert-parallel group.  `group` is a torch.distributed process group (None = default group)."""

    def __init__(self, unique_id=None, p: CommunicatorParams | None = None, group=None, transport: str = "auto"):
        if p is None:
            if dist.is_available() and dist.is_initialized():
                p = CommunicatorParams(dist.get_rank(group), dist.get_world_size(group), dist.get_world_size(group))
            else:
                p = CommunicatorParams(0, 1, 1)
        self.rank = int(p.rank)
        self.world = int(p.ep_world_size)
        self.num_ranks_per_node = int(p.num_ranks_per_node)
        self.group = group
        if self.world > 1:
            if not dist.is_initialized():
                raise RuntimeError("ep_world_size > 1 needs an initialised torch.distributed process group")
            if dist.get_world_size(group) != self.world or dist.get_rank(group) != self.rank:
                raise RuntimeError("rank/world of the process group do not match the communicator parameters")
            if self.world != self.num_ranks_per_node:
                raise RuntimeError("multi-node expert parallelism is not supported: one NVSwitch box only")
        if transport not in ("auto", "ipc", "nccl"):
            raise RuntimeError(f"transport must be 'auto', 'ipc' or 'nccl', got {transport!r}")
        self.transport_is_a_choice = transport == "auto"   # "auto" may fall back from "ipc" to "nccl" (all ranks together)
        if transport == "auto":
            on_gpu = self.world > 1 and dist.get_backend(group) == "nccl"
            transport = "ipc" if on_gpu and self.world <= 8 else "nccl"
        self.transport = transport
        self._regions = []   # (local pointer, [mapped peer pointers]) of every symmetric allocation

    # reference API names
    @staticmethod
    def createUniqueId():
        """The reference ships a TCP bootstrap id from rank 0; the rendezvous here belongs to torch.distributed."""
        return torch.zeros(128, dtype=torch.uint8)

    def getRank(self) -> int:
        return self.rank

    def getWorldSize(self) -> int:
        return self.world

    def getNumRanksPerNode(self) -> int:
        return self.num_ranks_per_node

    def barrier(self) -> None:
        if self.world > 1:
            dist.barrier(group=self.group)

    # ---- symmetric memory (transport "ipc")

    def symm_alloc(self, nbytes: int):
        """Collective.  Allocates `nbytes` of zeroed device memory on every rank and maps every rank's block into
        every process: -> (this rank's pointer, [pointer of rank r's block in this process for r in range(world)]).
        If any rank cannot allocate or map (no peer access, no IPC between the processes), every rank releases what
        it holds and raises SymmetricMemoryUnavailable, so that all ranks take the same decision."""
        local = ctypes.c_void_p()
        handle = (ctypes.c_uint8 * 64)()
        err = None
        try:
            _lib.call("epsb_symm_alloc", int(nbytes), ctypes.byref(local), handle)
        except _lib.EpsError as e:
            err = e
            local = ctypes.c_void_p(0)
        peers = [local.value] * self.world
        if self.world > 1:
            on_gpu = dist.get_backend(self.group) == "nccl"    # the handles travel on the group's own device type
            dev = torch.device("cuda", torch.cuda.current_device()) if on_gpu else torch.device("cpu")
            mine = torch.tensor(list(handle), dtype=torch.uint8, device=dev)
            allh = torch.empty((self.world, 64), dtype=torch.uint8, device=dev)
            ok = torch.tensor([0 if err is not None else 1], dtype=torch.int32, device=dev)
            dist.all_gather_into_tensor(allh.view(-1), mine, group=self.group)
            dist.all_reduce(ok, op=dist.ReduceOp.MIN, group=self.group)
            opened = []
            if int(ok.item()) == 1:
                allh = allh.cpu()
                for r in range(self.world):
                    if r == self.rank:
                        continue
                    h = (ctypes.c_uint8 * 64)(*allh[r].tolist())
                    p = ctypes.c_void_p()
                    try:
                        _lib.call("epsb_symm_open", h, ctypes.byref(p))
                    except _lib.EpsError as e:
                        err = e
                        break
                    peers[r] = p.value
                    opened.append(p.value)
            ok = torch.tensor([0 if err is not None else 1], dtype=torch.int32, device=dev)
            dist.all_reduce(ok, op=dist.ReduceOp.MIN, group=self.group)   # doubles as the barrier after the opens
            if int(ok.item()) == 0:
                for p in opened:
                    _lib.call("epsb_symm_close", p)
                dist.barrier(group=self.group)
                if local.value:
                    _lib.call("epsb_symm_free", local.value)
                raise SymmetricMemoryUnavailable(
                    f"symmetric memory over CUDA IPC is not available on every rank ({err or 'a peer failed'})")
        elif err is not None:
            raise err
        self._regions.append((local.value, peers))
        return local.value, peers

    def symm_free(self, local_ptr: int) -> None:
        """Collective.  Unmaps the peers' blocks and frees this rank's; no rank may still be writing to it."""
        for i, (loc, peers) in enumerate(self._regions):
            if loc == local_ptr:
                if self.world > 1:
                    torch.cuda.synchronize()
                    dist.barrier(group=self.group)
                    for r, p in enumerate(peers):
                        if r != self.rank:
                            _lib.call("epsb_symm_close", p)
                    dist.barrier(group=self.group)
                _lib.call("epsb_symm_free", loc)
                del self._regions[i]
                return

    # ---- collectives used by the plans

    def all_gather(self, t: torch.Tensor) -> torch.Tensor:
        """[n] -> [world, n] (every rank's copy of `t`)."""
        if self.world == 1:
            return t.reshape(1, -1)
        out = torch.empty((self.world, t.numel()), dtype=t.dtype, device=t.device)
        dist.all_gather_into_tensor(out.view(-1), t.contiguous().view(-1), group=self.group)
        return out

    def exchange(self, sends, recvs) -> None:
        """Variable-size all-to-all: sends[p] goes to peer p, recvs[p] is filled by peer p.  An entry is a
        contiguous row slice (possibly empty or None) or a list of such slices (several arrays exchanged in one
        grouped call; both sides list them in the same order); the entry for this rank itself is copied locally."""
        def as_list(x):
            return [] if x is None else (list(x) if isinstance(x, (list, tuple)) else [x])

        me = self.rank
        for snd, rcv in zip(as_list(sends[me]), as_list(recvs[me])):
            if snd is not None and rcv is not None and snd.numel() and rcv.data_ptr() != snd.data_ptr():
                rcv.copy_(snd)
        if self.world == 1:
            return
        ops = []
        for step in range(1, self.world):
            dst = (me + step) % self.world
            src = (me - step) % self.world
            for t in as_list(sends[dst]):
                if t is not None and t.numel():
                    ops.append(dist.P2POp(dist.isend, t, self._global(dst), group=self.group))
            for t in as_list(recvs[src]):
                if t is not None and t.numel():
                    ops.append(dist.P2POp(dist.irecv, t, self._global(src), group=self.group))
        if ops:
            for w in dist.batch_isend_irecv(ops):
                w.wait()

    def _global(self, group_rank: int) -> int:
        return group_rank if self.group is None else dist.get_global_rank(self.group, group_rank)


# The reference's class name, so that code written against python/eps keeps importing.
MscclppCommunicator = Communicator
MscclppCommunicatorParams = CommunicatorParams
