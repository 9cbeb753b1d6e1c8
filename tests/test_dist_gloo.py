"""World-size-2 (and 3) host logic of the expert-parallel exchange on CPU ranks over gloo: the Communicator's
variable-size all-to-all and all-gather, and the window arithmetic the Scheduler derives from the gathered plans.
The device kernels are replaced here by the CPU oracle (test infrastructure), which produces the same plans."""
import os
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))


def _worker(rank, world, port, S, E, k, T, q):
    try:
        os.environ["MASTER_ADDR"] = "127.0.0.1"
        os.environ["MASTER_PORT"] = str(port)
        dist.init_process_group("gloo", rank=rank, world_size=world)
        from helpers import random_routing, simulate_eps
        from oracle import oracle as orc

        from eps_b200.communication import Communicator, CommunicatorParams
        from eps_b200.scheduler import dispatch_windows, stage_slices

        comm = Communicator(None, CommunicatorParams(rank, world, world))
        # every rank builds the same global routing so that it can check what it receives
        rng = np.random.default_rng(1234)
        Ts = [T + 7 * r for r in range(world)]
        routing = [random_routing(rng, Ts[r], k, E, 2) for r in range(world)]
        ranks = simulate_eps(orc, [rt[0] for rt in routing], E, world, S, max(Ts))
        me = ranks[rank]
        # 1. plan exchange
        gathered = comm.all_gather(torch.from_numpy(me["send_incl"]))
        assert np.array_equal(gathered.numpy(), np.stack([ranks[r]["send_incl"] for r in range(world)]))
        win = dispatch_windows(gathered.numpy(), rank, world, S)
        assert np.array_equal(win[3], me["recv_incl"]) and int(win[3][-1]) == me["R"]
        # 2. one-shot exchange of the index rows, then stage by stage of a "hidden" payload
        idx = routing[rank][0]
        send_idx = torch.from_numpy(idx[me["send_map"] % Ts[rank]].copy())
        recv_idx = torch.full((me["R"], k), -9, dtype=torch.int32)
        sl = stage_slices(win, world, S, -1)
        comm.exchange([send_idx[a:b] for (a, b), _ in sl], [recv_idx[c:d] for _, (c, d) in sl])
        assert np.array_equal(recv_idx.numpy(), me["ridx"])
        payload = torch.from_numpy((me["send_map"] % Ts[rank]).astype(np.int64) + 100000 * rank).reshape(-1, 1).contiguous()
        got = torch.full((me["R"], 1), -1, dtype=torch.int64)
        for st in range(S):
            sl = stage_slices(win, world, S, st)
            comm.exchange([payload[a:b] for (a, b), _ in sl], [got[c:d] for _, (c, d) in sl])
        want = me["src_of"][:, 1] + 100000 * me["src_of"][:, 0]
        assert np.array_equal(got.numpy().reshape(-1), want)
        # 2b. two arrays in ONE grouped exchange (what the first dispatch of the layer does)
        recv_idx2 = torch.full((me["R"], k), -9, dtype=torch.int32)
        got2 = torch.full((me["R"], 1), -1, dtype=torch.int64)
        sl = stage_slices(win, world, S, -1)
        comm.exchange([[send_idx[a:b], payload[a:b]] for (a, b), _ in sl],
                      [[recv_idx2[c:d], got2[c:d]] for _, (c, d) in sl])
        assert np.array_equal(recv_idx2.numpy(), me["ridx"]) and np.array_equal(got2.numpy().reshape(-1), want)
        # 3. combine direction: windows from the return plan (sender side) and the collect plan (receiver side)
        ret, coll = me["ret_incl"].astype(np.int64), me["coll_incl"].astype(np.int64)
        ex = lambda a: np.concatenate([[0], a[:-1]])
        cwin = (ex(ret), ret, ex(coll), coll)
        # ... which the host can derive from the all-gathered collect plans alone: the rows this rank returns to
        # peer p are the rows p collects from it (Scheduler.rendezvous_and_plan relies on this)
        gcoll = comm.all_gather(torch.from_numpy(me["coll_incl"]))
        cw = dispatch_windows(gcoll.numpy(), rank, world, S)
        assert np.array_equal(cw[3], ret) and np.array_equal(cw[1], coll)
        back = torch.arange(me["R"], dtype=torch.int64).reshape(-1, 1) + 1000000 * rank
        collected = torch.full((int(coll[-1]), 1), -1, dtype=torch.int64)
        for st in range(S):
            sl = stage_slices(cwin, world, S, st)
            comm.exchange([back[a:b] for (a, b), _ in sl], [collected[c:d] for _, (c, d) in sl])
        assert int(coll[-1]) == int(me["send_incl"][-1]) and bool((collected >= 0).all())
        # every collected row came from the rank the global-reduce plan expects
        glob = me["glob_map"]
        for t in range(Ts[rank]):
            for ep in range(world):
                if glob[t, ep] < Ts[rank] * world:
                    assert int(collected[glob[t, ep], 0]) // 1000000 == ep
        comm.barrier()
        dist.destroy_process_group()
        q.put((rank, "ok"))
    except Exception as exc:  # surfaced by the parent
        import traceback

        q.put((rank, traceback.format_exc()))


@pytest.mark.parametrize("world,S,E,k,T", [(2, 1, 8, 2, 40), (2, 2, 16, 4, 64), (3, 2, 12, 3, 33)])
def test_exchange_over_gloo(world, S, E, k, T):
    from oracle import oracle as orc

    orc.build()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29500 + (os.getpid() + world * 7 + S) % 2000
    procs = [ctx.Process(target=_worker, args=(r, world, port, S, E, k, T, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = [q.get(timeout=180) for _ in range(world)]
    for p in procs:
        p.join(timeout=60)
    for rank, msg in results:
        assert msg == "ok", f"rank {rank}: {msg}"


def _symm_worker(rank, world, port, q):
    try:
        os.environ["MASTER_ADDR"] = "127.0.0.1"
        os.environ["MASTER_PORT"] = str(port)
        dist.init_process_group("gloo", rank=rank, world_size=world)
        from eps_b200 import _lib
        from eps_b200.communication import Communicator, CommunicatorParams, SymmetricMemoryUnavailable

        comm = Communicator(None, CommunicatorParams(rank, world, world), transport="ipc")
        real = _lib.call
        opened, freed = [], []

        def fake(name, *args):
            # rank 0 allocates and opens fine; rank 1 cannot open its peer's handle (the failure is made on the host)
            if name == "epsb_symm_alloc":
                args[1]._obj.value = 0x1000 * (rank + 1)
                return 0
            if name == "epsb_symm_open":
                if rank == 1:
                    raise _lib.EpsError("epsb_symm_open: peer access is not available (code 2)")
                args[1]._obj.value = 0x9000
                opened.append(0x9000)
                return 0
            if name == "epsb_symm_close":
                opened.remove(args[0])
                return 0
            if name == "epsb_symm_free":
                freed.append(args[0])
                return 0
            return real(name, *args)

        _lib.call = fake
        try:
            comm.symm_alloc(4096)
            q.put((rank, "symm_alloc did not raise"))
            return
        except SymmetricMemoryUnavailable:
            pass          # on BOTH ranks, although only rank 1 failed
        finally:
            _lib.call = real
        assert opened == [] and freed == [0x1000 * (rank + 1)], (opened, freed)
        assert comm._regions == []
        dist.barrier()
        dist.destroy_process_group()
        q.put((rank, "ok"))
    except Exception:
        import traceback

        q.put((rank, traceback.format_exc()))


def test_symmetric_memory_failure_is_collective():
    """One rank cannot map its peer's region: every rank releases what it holds and raises the same exception (the
    caller's fall-back to the other transport is then the same decision on all ranks).  The failure is injected on the
    host; no GPU is involved."""
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29500 + (os.getpid() + 911) % 2000
    procs = [ctx.Process(target=_symm_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    results = [q.get(timeout=180) for _ in range(2)]
    for p in procs:
        p.join(timeout=60)
    for rank, msg in results:
        assert msg == "ok", f"rank {rank}: {msg}"


def test_single_rank_never_touches_a_process_group():
    from eps_b200.communication import Communicator, CommunicatorParams

    comm = Communicator(None, CommunicatorParams(0, 1, 1))
    a = torch.arange(6).reshape(3, 2)
    b = torch.zeros_like(a)
    comm.exchange([a], [b])
    assert torch.equal(a, b)
    assert comm.all_gather(torch.arange(4)).shape == (1, 4)
    comm.barrier()
    with pytest.raises(RuntimeError):
        Communicator(None, CommunicatorParams(0, 2, 2))
