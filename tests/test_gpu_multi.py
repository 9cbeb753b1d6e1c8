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


def _native_worker(rank, world, uid, q):
    """The C++ stack on 2 GPUs through the drop-in `eps` package: communicator created from a unique id (NCCL carries
    the set-up, the data moves through this library's peer-store kernels), the FP8 layer driven through the scheduler
    and executor ops, fast_ep, fast_oep and the TP<->DP convertor."""
    try:
        sys.path.insert(0, ROOT)
        sys.path.insert(0, os.path.join(ROOT, "tests"))
        sys.path.insert(0, os.path.join(ROOT, "eps_b200"))
        os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
        torch.cuda.set_device(rank)
        dev = torch.device("cuda", rank)
        from eps.communication import MscclppCommunicator, MscclppCommunicatorParams, TPDPConvertor
        from eps.executor import AokGroupedGemm
        from eps.executor.silu import per_token_group_quant_fp8
        from eps.fast_ep import AllToAll as FastEP
        from eps.fast_oep import AllToAll as FastOEP
        from eps.scheduler import Scheduler
        from helpers import random_routing
        from oracle import oracle as orc

        from eps_b200 import ops, workloads

        comm = MscclppCommunicator(uid, MscclppCommunicatorParams(rank, world, world))
        comm.barrier()
        msgs = []

        # ---- FP8 expert layer, EP2, through the ops
        T, H, I, E, k, nz, sh = 100, 1024, 512, 8, 4, 4, 256
        cfg = workloads.CONFIGS[0].scaled(tokens_per_rank=T, hidden=H, inter=I, num_experts=E, top_k=k,
                                          num_zero_experts=nz, shared_inter=sh, bias="normal")
        EL = E // world
        gu = torch.stack([workloads.make_expert_weights(cfg, e)[0] for e in range(E)])
        dn = torch.stack([workloads.make_expert_weights(cfg, e)[1] for e in range(E)])
        lo, hi = rank * EL, (rank + 1) * EL
        gq, gs = ops.quant_block128(gu[lo:hi].to(dev))
        dq, ds = ops.quant_block128(dn[lo:hi].to(dev))
        a, b = workloads.make_expert_weights(cfg, -1, inter=sh)
        shared = (*ops.quant_block128(a.unsqueeze(0).to(dev)), *ops.quant_block128(b.unsqueeze(0).to(dev)))
        ref_shared = (*orc.quant_block128(a.unsqueeze(0).float().numpy()), *orc.quant_block128(b.unsqueeze(0).float().numpy()))
        Tr = T + 5 * rank
        max_tok = T + 5 * world
        x = workloads.make_tokens(cfg, rank, Tr).to(dev)
        idx, w = (t.to(dev) for t in workloads.make_routing(cfg, rank, Tr))
        sched = Scheduler(k, E, H, H // 128, max_tok, comm, EL, fp8_hidden=True)
        gemm, g1 = AokGroupedGemm(EL), AokGroupedGemm(1)
        status = torch.zeros(4, dtype=torch.int32, device=dev)
        for _ in range(3):
            xq, xs = per_token_group_quant_fp8(x)
            one = torch.tensor([0, Tr], dtype=torch.int32, device=dev)
            aq, a_s = g1.run_gate_up_swiglu(xq, xs, shared[0], shared[1], one, status=status)
            shared_out = g1.run_down_weighted(aq, a_s, shared[2], shared[3], one, status=status)
            excl, bound = sched.rendezvous_and_plan(idx, w, Tr * world, 1, True, host_sync=False, payload=(xq, xs))
            D = bound * min(k, EL)
            A = torch.empty((D, H), dtype=torch.uint8, device=dev)
            A_s = torch.empty((D, H // 128), dtype=torch.float32, device=dev)
            sched.prologue(w, xq, xs, A_s, raw_input=x)
            row_w = sched.gemm_row_weights()
            sched.dispatch(0)
            sched.gemm_expand(A, 0)
            act, act_s = gemm.run_gate_up_swiglu(A, A_s, gq, gs, excl, status=status)
            Y = gemm.run_down_weighted(act, act_s, dq, ds, excl, row_weights=row_w, status=status)
            sched.local_reduce(Y, 0, pre_weighted=True)
            sched.combine(0)
            out = torch.empty((Tr, H), dtype=torch.bfloat16, device=dev)
            sched.epilogue(out, shared=shared_out, ref_arith=False)
        torch.cuda.synchronize()
        sched.check_status()
        rq, rs = orc.quant_block128(gu.float().numpy())
        rdq, rds = orc.quant_block128(dn.float().numpy())
        want = orc.moe_layer_fp32(x.cpu().view(torch.int16).numpy().view(np.uint16), idx.cpu().numpy(), w.cpu().numpy(),
                                  rq, rs, rdq, rds, shared=ref_shared)
        got = out.float().cpu().numpy()
        rms = float(np.sqrt(np.mean(want ** 2)))
        worst = float(np.max(np.abs(got - want) / (2e-2 * rms + 2.0 ** -8 * np.abs(want))))
        if worst > 1.0 or status.tolist()[0] != 0:
            msgs.append(f"layer through the ops: worst err/bound {worst:.3f}, status {status.tolist()}")
        sched.destroy()

        # ---- fast_ep, EP2, bit-exact
        T2, k2, E2, H2 = 90 + 11 * rank, 4, 16, 1024
        EL2 = E2 // world
        rng = np.random.default_rng(50 + rank)
        idx2, w2 = random_routing(rng, T2, k2, E2, 3)
        x2 = torch.randn((T2, H2), generator=torch.Generator().manual_seed(rank)).to(torch.bfloat16)
        a2a = FastEP(k2, E2, H2, 256, comm)
        excl2 = torch.empty((EL2 + 1,), dtype=torch.int32, device=dev)
        expert_x = torch.zeros((256 * k2, H2), dtype=torch.bfloat16, device=dev)
        x2_dev = x2.to(dev)   # combine reads the raw tokens again (identity experts): the caller keeps them alive
        a2a.dispatch(excl2, expert_x, x2_dev, torch.from_numpy(idx2).to(dev), 256)
        ex = excl2.cpu().numpy()
        y = torch.zeros_like(expert_x)
        for le in range(EL2):
            e = rank * EL2 + le
            y[ex[le]:ex[le + 1]] = (expert_x[ex[le]:ex[le + 1]].float() * (1 + e / 8)).to(torch.bfloat16)
        out2 = torch.empty((T2, H2), dtype=torch.bfloat16, device=dev)
        a2a.combine(out2, torch.from_numpy(w2).to(dev), y, 256)
        torch.cuda.synchronize()
        _, rmap = orc.fastep_expand_plan(idx2, E2)
        rows = torch.zeros((T2 * k2, H2), dtype=torch.bfloat16)
        for i in range(T2 * k2):
            if rmap[i] < 1000000:
                rows[rmap[i]] = (x2[i // k2].float() * (1 + idx2.reshape(-1)[i] / 8)).to(torch.bfloat16)
        bts = lambda t: t.view(torch.int16).cpu().numpy().view(np.uint16)
        if not np.array_equal(bts(out2), orc.fastep_reduce(bts(rows), bts(x2), w2, rmap)):
            msgs.append("fast_ep output differs from the oracle")
        a2a.destroy()

        # ---- fast_oep, table sharded over the two ranks
        Dm, size = 256, 300
        table = torch.randn((world * size, Dm), generator=torch.Generator().manual_seed(7)).to(torch.bfloat16)
        g = torch.Generator().manual_seed(100 + rank)
        ids = torch.randint(0, world * size, (40 + 3 * rank, 2), generator=g, dtype=torch.int32)
        ids[torch.rand(ids.shape, generator=g) < 0.1] = -1
        oep = FastOEP(Dm, size, 512, comm)
        for _ in range(2):
            oep.dispatch(ids.to(dev))
            out3 = torch.full((ids.numel(), Dm), 3.0, dtype=torch.bfloat16, device=dev)
            oep.combine(out3, 0, 2, False, table[rank * size:(rank + 1) * size].contiguous().to(dev))
        torch.cuda.synchronize()
        flat = ids.reshape(-1)
        want3 = torch.full((ids.numel(), Dm), 3.0, dtype=torch.bfloat16)
        want3[flat >= 0] = table[flat[flat >= 0].long()]
        if not torch.equal(out3.cpu(), want3):
            msgs.append("fast_oep rows differ from the table")
        oep.destroy()

        # ---- TP <-> DP convertor, a TP group of two
        tokens, hid = 37, 512
        tpdp = TPDPConvertor(TPDPConvertor.Params(rank, 32, world, hid, comm))
        for _ in range(2):
            ag = tpdp.get_all_gather_context(tokens, 256)
            n_mine, off = ag.input().shape[0], ag.input_row_offset
            full = torch.arange(tokens * 256, dtype=torch.float32).reshape(tokens, 256).remainder(251).to(torch.bfloat16)
            ag.input().copy_(full[off:off + n_mine].to(dev))
            tpdp.all_gather(ag, None)
            torch.cuda.synchronize()
            if not torch.equal(ag.output().cpu(), full):
                msgs.append("all_gather output differs")
            rs = tpdp.get_reduce_scatter_context(tokens)
            parts = [torch.randn((tokens, hid), generator=torch.Generator().manual_seed(r)).to(torch.bfloat16)
                     for r in range(world)]
            rs.input().copy_(parts[rank].to(dev))
            tpdp.reduce_scatter(rs, None)
            torch.cuda.synchronize()
            o, n_o = rs.output_row_offset, rs.output().shape[0]
            want_rs = (parts[0].float() + parts[1].float()).to(torch.bfloat16)[o:o + n_o]
            if not torch.equal(rs.output().cpu(), want_rs):
                msgs.append("reduce_scatter output differs")
        del tpdp
        comm.barrier()
        q.put((rank, "ok" if not msgs else "; ".join(msgs)))
    except Exception:
        import traceback

        q.put((rank, traceback.format_exc()))


def test_native_stack_ep2():
    if not torch.cuda.is_available() or torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    from eps_b200 import build
    from oracle import oracle as orc

    build.build_torch_ops()
    orc.build()
    sys.path.insert(0, os.path.join(ROOT, "eps_b200"))
    from eps.communication import MscclppCommunicator

    uid = MscclppCommunicator.createUniqueId()
    world = 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_native_worker, args=(r, world, uid, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = [q.get(timeout=600) for _ in range(world)]
    for p in procs:
        p.join(timeout=60)
    for rank, msg in results:
        assert msg == "ok", f"rank {rank}: {msg}"
