"""Expert parallelism over 2 GPUs, both transports (this library's peer-store kernels over CUDA IPC, and grouped NCCL
send/recv): every rank's layer output against the fp32 oracle of the global layer.
Skipped on machines with fewer than two GPUs."""
import os
import sys

import numpy as np
import pytest
import torch
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, case, transport, q):
    try:
        sys.path.insert(0, ROOT)
        sys.path.insert(0, os.path.join(ROOT, "tests"))
        os.environ["MASTER_ADDR"] = "127.0.0.1"
        os.environ["MASTER_PORT"] = str(port)
        os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
        import torch.distributed as dist

        torch.cuda.set_device(rank)
        dev = torch.device("cuda", rank)
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
        from oracle import oracle as orc

        from eps_b200 import ops, workloads
        from eps_b200.communication import Communicator, CommunicatorParams
        from eps_b200.layer import MoELayerFP8

        T, H, I, E, k, nz, sh, S = case
        cfg = workloads.CONFIGS[0].scaled(tokens_per_rank=T, hidden=H, inter=I, num_experts=E, top_k=k,
                                          num_zero_experts=nz, shared_inter=sh, bias="normal" if nz else "none")
        EL = E // world
        gu = torch.stack([workloads.make_expert_weights(cfg, e)[0] for e in range(E)])
        dn = torch.stack([workloads.make_expert_weights(cfg, e)[1] for e in range(E)])
        lo, hi = rank * EL, (rank + 1) * EL
        gq, gs = ops.quant_block128(gu[lo:hi].to(dev))
        dq, ds = ops.quant_block128(dn[lo:hi].to(dev))
        shared = ref_shared = None
        if sh:
            a, b = workloads.make_expert_weights(cfg, -1, inter=sh)
            shared = (*ops.quant_block128(a.unsqueeze(0).to(dev)), *ops.quant_block128(b.unsqueeze(0).to(dev)))
            ref_shared = (*orc.quant_block128(a.unsqueeze(0).float().numpy()), *orc.quant_block128(b.unsqueeze(0).float().numpy()))
        comm = Communicator(None, CommunicatorParams(rank, world, world), transport=transport)
        assert comm.transport == transport
        Tr = T + 5 * rank   # ragged token counts per rank
        layer = MoELayerFP8(H, I, E, k, T + 5 * world, gq, gs, dq, ds, comm=comm, shared=shared, num_stages=S)
        x = workloads.make_tokens(cfg, rank, Tr)
        idx, w = workloads.make_routing(cfg, rank, Tr)
        for _ in range(3):  # later calls reuse the arenas (both parities of the device-side exchange) and plan buffers
            out = layer.forward(x.to(dev), idx.to(dev), w.to(dev))
            ctx = layer.sched.context
            if transport == "nccl":
                # the combine windows the host derived from the all-gathered plans == the device's return plan
                assert np.array_equal(ctx.ret_incl.cpu().numpy(), ctx.host_combine[1]), "return plan mismatch"
                assert np.array_equal(ctx.coll_incl.cpu().numpy(), ctx.host_combine[3]), "collect plan mismatch"
        torch.cuda.synchronize()
        layer.check_status()
        rq, rs = orc.quant_block128(gu.float().numpy())
        rdq, rds = orc.quant_block128(dn.float().numpy())
        want = orc.moe_layer_fp32(x.view(torch.int16).numpy().view(np.uint16), idx.numpy(), w.numpy(), rq, rs, rdq, rds,
                                  shared=ref_shared)
        got = out.float().cpu().numpy()
        rms = float(np.sqrt(np.mean(want ** 2)))
        worst = float(np.max(np.abs(got - want) / (2e-2 * rms + 2.0 ** -8 * np.abs(want))))
        layer.sched.destroy()
        dist.barrier()
        dist.destroy_process_group()
        q.put((rank, "ok" if worst <= 1.0 else f"worst err/bound {worst:.3f}"))
    except Exception:
        import traceback

        q.put((rank, traceback.format_exc()))


@pytest.mark.parametrize("transport", ["ipc", "nccl"])
@pytest.mark.parametrize("case", [(64, 512, 256, 8, 2, 0, 0, 1), (100, 1024, 512, 8, 4, 4, 256, 2), (200, 2048, 1408, 16, 4, 0, 0, 4)])
def test_layer_ep2_vs_oracle(case, transport):
    if not torch.cuda.is_available() or torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    from eps_b200 import build
    from oracle import oracle as orc

    build.build()
    orc.build()
    world = 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29700 + (os.getpid() + case[0] + (700 if transport == "ipc" else 0)) % 1500
    procs = [ctx.Process(target=_worker, args=(r, world, port, case, transport, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = [q.get(timeout=300) for _ in range(world)]
    for p in procs:
        p.join(timeout=60)
    for rank, msg in results:
        assert msg == "ok", f"rank {rank}: {msg}"


def _fastep_worker(rank, world, port, q):
    try:
        sys.path.insert(0, ROOT)
        sys.path.insert(0, os.path.join(ROOT, "tests"))
        os.environ["MASTER_ADDR"] = "127.0.0.1"
        os.environ["MASTER_PORT"] = str(port)
        os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
        import torch.distributed as dist

        torch.cuda.set_device(rank)
        dev = torch.device("cuda", rank)
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
        from helpers import random_routing
        from oracle import oracle as orc

        from eps_b200.communication import Communicator, CommunicatorParams
        from eps_b200.fast_ep import AllToAll

        T, k, E, H = 90 + 11 * rank, 4, 16, 1024
        EL = E // world
        rng = np.random.default_rng(50 + rank)
        idx, w = random_routing(rng, T, k, E, 3)
        x = torch.randn((T, H), generator=torch.Generator().manual_seed(rank)).to(torch.bfloat16)
        comm = Communicator(None, CommunicatorParams(rank, world, world), transport="nccl")
        a2a = AllToAll(k, E, H, 256, comm)
        excl = torch.empty((EL + 1,), dtype=torch.int32, device=dev)
        expert_x = torch.zeros((256 * k, H), dtype=torch.bfloat16, device=dev)
        a2a.dispatch(excl, expert_x, x.to(dev), torch.from_numpy(idx).to(dev), 256)
        ex = excl.cpu().numpy()
        y = torch.zeros_like(expert_x)
        for le in range(EL):   # expert e scales its rows by (1 + e/8)
            e = rank * EL + le
            y[ex[le]:ex[le + 1]] = (expert_x[ex[le]:ex[le + 1]].float() * (1 + e / 8)).to(torch.bfloat16)
        out = torch.empty((T, H), dtype=torch.bfloat16, device=dev)
        a2a.combine(out, torch.from_numpy(w).to(dev), y, 256)
        torch.cuda.synchronize()
        _, rmap = orc.fastep_expand_plan(idx, E)
        rows = torch.zeros((T * k, H), dtype=torch.bfloat16)
        for i in range(T * k):
            if rmap[i] < 1000000:
                rows[rmap[i]] = (x[i // k].float() * (1 + idx.reshape(-1)[i] / 8)).to(torch.bfloat16)
        b = lambda t: t.view(torch.int16).cpu().numpy().view(np.uint16)
        want = orc.fastep_reduce(b(rows), b(x), w, rmap)
        ok = np.array_equal(b(out), want)
        dist.barrier()
        dist.destroy_process_group()
        q.put((rank, "ok" if ok else "fast_ep output differs from the oracle"))
    except Exception:
        import traceback

        q.put((rank, traceback.format_exc()))


def test_fastep_ep2_bit_exact():
    if not torch.cuda.is_available() or torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    from eps_b200 import build
    from oracle import oracle as orc

    build.build()
    orc.build()
    world = 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29900 + os.getpid() % 1000
    procs = [ctx.Process(target=_fastep_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = [q.get(timeout=300) for _ in range(world)]
    for p in procs:
        p.join(timeout=60)
    for rank, msg in results:
        assert msg == "ok", f"rank {rank}: {msg}"
