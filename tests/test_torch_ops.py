"""The six torch-op libraries (libscheduler_.so, libexecutor_.so, libfast_ep.so, libfast_oep.so, libcommunication_.so,
libutils_.so) and the drop-in `eps` package on top of them: the reference's namespaces, op names and argument lists
(CPU part), and on the GPU the whole expert layer driven purely through the ops, bit for bit against MoELayerFP8."""
import os
import sys

import numpy as np
import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def eps_pkg():
    """The drop-in package: `import eps` with <repo>/eps_b200 on sys.path, as a user of the reference would."""
    from eps_b200 import build

    build.build_torch_ops()
    path = os.path.join(ROOT, "eps_b200")
    if path not in sys.path:
        sys.path.insert(0, path)
    import eps

    return eps


REFERENCE_OPS = {
    "scheduler": ["eps_create", "eps_destroy", "eps_get_context", "eps_destroy_context",
                  "eps_get_workspace_size_context", "eps_set_ws_context", "eps_rendezvous", "eps_plan", "eps_prologue",
                  "eps_dispatch", "eps_gemm_expand", "eps_local_reduce", "eps_combine", "eps_epilogue"],
    "executor": ["aok_create", "aok_get_workspace_size", "aok_run", "aok_destroy", "silu_run"],
    "fast_ep": ["all_to_all_create", "all_to_all_destroy", "all_to_all_dispatch", "all_to_all_combine"],
    "fast_oep": ["all_to_all_create", "all_to_all_destroy", "all_to_all_dispatch", "all_to_all_combine"],
    "communication": ["eps_comm_create_unique_id", "eps_comm_create", "eps_comm_destroy", "eps_comm_barrier",
                      "sync_check_cuda_error_eps", "eps_tpdp_create", "eps_tpdp_destroy",
                      "eps_tpdp_get_reduce_scatter_input", "eps_tpdp_get_reduce_scatter_output",
                      "eps_tpdp_get_reduce_scatter_output_row_offset", "eps_tpdp_reduce_scatter",
                      "eps_tpdp_get_all_gather_input", "eps_tpdp_get_all_gather_output",
                      "eps_tpdp_get_all_gather_input_row_offset", "eps_tpdp_all_gather"],
    "utils": ["topk_sigmoid", "rms_norm_op"],
}


def _schema(ns, op):
    return str(getattr(getattr(torch.ops, ns), op).default._schema)


def test_ops_are_registered_with_reference_names_and_schemas(eps_pkg):
    for ns, names in REFERENCE_OPS.items():
        for name in names:
            assert hasattr(getattr(torch.ops, ns), name), f"{ns}.{name}"
    for name in REFERENCE_OPS["scheduler"]:   # the C++ registers them under `eps`, python/eps reads `scheduler`
        assert hasattr(torch.ops.eps, name), f"eps.{name}"
    # argument lists as torch infers them from the reference's C++ signatures (ints are int64, handles are ints)
    assert _schema("scheduler", "eps_create").count("int") == 8            # 7 arguments + the handle returned
    s = _schema("scheduler", "eps_prologue")
    assert s.count("Tensor?") == 2 and s.count("Tensor") == 4
    s = _schema("executor", "aok_run")
    assert s.count("Tensor") == 5 and s.count("int") >= 3
    s = _schema("utils", "topk_sigmoid")
    assert s.count("Tensor") == 4 and s.count("int") == 5 and "float" in s
    s = _schema("fast_oep", "all_to_all_combine")
    assert s.count("Tensor") == 2 and "bool" in s
    assert _schema("communication", "eps_tpdp_all_gather").count("int") == 5


def test_handles_and_errors_need_no_gpu(eps_pkg):
    ex = torch.ops.executor
    h = ex.aok_create(8, 148)
    assert h != 0 and ex.aok_get_workspace_size(h, 7168, 4096) == 0   # the tile list is built inside the kernel
    t = torch.zeros((1, 1))
    with pytest.raises(RuntimeError, match="CUDA tensor"):
        ex.aok_run(h, t, torch.zeros((1, 1, 1)), t, torch.zeros(2, dtype=torch.int32), 0, 0, t)
    ex.aok_destroy(h)
    with pytest.raises(RuntimeError, match="context handle is null"):
        torch.ops.scheduler.eps_get_workspace_size_context(0)


# ---------------------------------------------------------------------------------------------------- GPU

def _bits(t):
    return t.view(torch.int16).cpu().numpy().view(np.uint16)


@pytest.mark.gpu
def test_executor_ops(cuda, oracle, eps_pkg):
    from eps.executor import AokGroupedGemm, silu
    from eps.executor.silu import per_token_group_quant_fp8

    from eps_b200 import ops

    x = torch.randn((64, 512), generator=torch.Generator().manual_seed(1)).to(torch.bfloat16).to(cuda)
    q, s = per_token_group_quant_fp8(x)
    q2, s2 = ops.per_token_group_quant_fp8(x)
    assert torch.equal(q, q2) and torch.equal(s, s2)
    gu = torch.randn((40, 512), generator=torch.Generator().manual_seed(2)).to(torch.bfloat16).to(cuda)
    excl = torch.tensor([0, 40], dtype=torch.int32, device=cuda)
    r2 = torch.zeros((40, 256), dtype=torch.bfloat16, device=cuda)
    ops.silu_run(gu, r2, excl, 1)
    assert torch.equal(silu(gu, excl, 40), r2)
    # the reference's call: bf16 x bf16 grouped GEMM, B_scale None
    g = torch.Generator().manual_seed(3)
    A = torch.randn((100, 256), generator=g).to(torch.bfloat16).to(cuda)
    B = (torch.randn((2, 384, 256), generator=g) * 0.05).to(torch.bfloat16).to(cuda)
    ex2 = torch.tensor([0, 60, 100], dtype=torch.int32, device=cuda)
    gemm = AokGroupedGemm(2)
    C = gemm.run(A, B, None, ex2, 100)
    for e, (a, b) in enumerate([(0, 60), (60, 100)]):
        want = A[a:b].float() @ B[e].float().t()
        assert torch.all((C[a:b].float() - want).abs() <= 2.0 ** -8 * want.abs() + 1e-3)
    with pytest.raises(RuntimeError, match="experts"):
        gemm.run(A, B[:1].contiguous(), None, ex2, 100)
    with pytest.raises(RuntimeError, match="K ="):
        gemm.run(A[:, :128].contiguous(), B, None, ex2, 100)
    # FP8 path against the oracle
    rng = np.random.default_rng(0)
    a = oracle.bf16_bits(rng.standard_normal((100, 256)).astype(np.float32))
    Aq, a_s = oracle.quant_1x128(a)
    wq, w_s = oracle.quant_block128((rng.standard_normal((2, 256, 256)) * 0.02).astype(np.float32))
    dv = lambda t: torch.from_numpy(np.ascontiguousarray(t)).to(cuda)
    C8 = gemm.run(dv(Aq), dv(wq), dv(w_s), ex2, 100, A_scale=dv(a_s))
    want = oracle.grouped_gemm_fp8(Aq, a_s, wq, w_s, ex2.cpu().numpy())
    got = C8.float().cpu().numpy()
    assert np.all(np.abs(got - want) <= 2.0 ** -8 * np.abs(want) + 1e-6)
    gemm.destroy()


@pytest.mark.gpu
def test_ffn_executors_behind_the_contract_types(cuda, oracle, eps_pkg):
    """GemmExecutor / SharedExperts / dense / batched GEMM / dense SwiGLU (the reference's contract types
    GemmExecutorInterface, SharedExpertsInterface, DenseGemmInterface, BatchedGemmInterface, DenseActivationInterface)
    give bit for bit what the same kernels give when called one by one, and the FFN agrees with the oracle."""
    from eps.executor import GemmExecutor, SharedExperts, batched_gemm_fp8, dense_gemm_fp8, dense_silu

    from eps_b200 import ops

    rng = np.random.default_rng(11)
    E, H, I = 4, 512, 256
    rows = [130, 0, 64, 7]
    D = sum(rows)
    excl = torch.tensor([0] + list(np.cumsum(rows)), dtype=torch.int32, device=cuda)
    dv = lambda t: torch.from_numpy(np.ascontiguousarray(t)).to(cuda)
    a = oracle.bf16_bits(rng.standard_normal((D, H)).astype(np.float32))
    Aq, a_s = oracle.quant_1x128(a)
    wgu, wgu_s = oracle.quant_block128((rng.standard_normal((E, 2 * I, H)) * 0.03).astype(np.float32))
    wd, wd_s = oracle.quant_block128((rng.standard_normal((E, H, I)) * 0.03).astype(np.float32))
    row_w = rng.random(D).astype(np.float32)
    A, As = dv(Aq), dv(a_s)
    # the kernels one by one
    act, act_s = ops.grouped_gemm_fp8(ops.GEMM_GATEUP, A, As, dv(wgu), dv(wgu_s), excl)
    want = ops.grouped_gemm_fp8(ops.GEMM_DOWN, act, act_s, dv(wd), dv(wd_s), excl, row_w=dv(row_w))
    ex = GemmExecutor(dv(wgu), dv(wgu_s), dv(wd), dv(wd_s))
    got = ex.run(A, As, excl, row_weights=dv(row_w))
    torch.cuda.synchronize()
    assert ex.status().tolist()[0] == 0
    assert torch.equal(got[:D], want[:D])
    # two stages: each stage writes its own experts' rows
    out2 = torch.zeros_like(got)
    for s in range(2):
        ex.run(A, As, excl, num_stages=2, stage_idx=s, row_weights=dv(row_w), out=out2)
    assert torch.equal(out2[:D], want[:D])
    with pytest.raises(RuntimeError, match="Invalid num_stages"):
        ex.run(A, As, excl, num_stages=3)
    ex.destroy()
    # against the oracle: the down GEMM of the requantised activation, x the row's weight (the gate/up half has its
    # own oracle test in test_gpu_gemm.py)
    y = oracle.grouped_gemm_fp8(act.cpu().numpy(), act_s.cpu().numpy(), wd, wd_s, excl.cpu().numpy()) * row_w[:, None]
    rms = float(np.sqrt(np.mean(y ** 2)))
    assert np.all(np.abs(got[:D].float().cpu().numpy() - y) <= 2e-2 * rms + 2.0 ** -8 * np.abs(y))
    # shared expert = one expert over all rows
    sh = SharedExperts(dv(wgu[:1]), dv(wgu_s[:1]), dv(wd[:1]), dv(wd_s[:1]))
    e1 = torch.tensor([0, D], dtype=torch.int32, device=cuda)
    a1, a1s = ops.grouped_gemm_fp8(ops.GEMM_GATEUP, A, As, dv(wgu[:1]), dv(wgu_s[:1]), e1)
    w1 = ops.grouped_gemm_fp8(ops.GEMM_DOWN, a1, a1s, dv(wd[:1]), dv(wd_s[:1]), e1)
    assert torch.equal(sh.run(A, As), w1)
    sh.destroy()
    # dense and batched GEMM = the grouped kernel on one / G equal row ranges
    Bq, Bs = dv(wd[0]), dv(wd_s[0])          # [H, I] as a dense [N, K] weight
    X, Xs = act[:D].contiguous(), act_s[:D].contiguous()
    dense = dense_gemm_fp8(X, Xs, Bq, Bs)
    ref = ops.grouped_gemm_fp8(ops.GEMM_PLAIN, X, Xs, dv(wd[:1]), dv(wd_s[:1]), e1)
    assert torch.equal(dense, ref)
    G, M = 3, 40
    Xb, Xbs = X[:G * M].reshape(G, M, I).contiguous(), Xs[:G * M].reshape(G, M, I // 128).contiguous()
    bat = batched_gemm_fp8(Xb, Xbs, dv(wd[:G]), dv(wd_s[:G]))
    eb = torch.tensor([0, M, 2 * M, 3 * M], dtype=torch.int32, device=cuda)
    refb = ops.grouped_gemm_fp8(ops.GEMM_PLAIN, X[:G * M].contiguous(), Xs[:G * M].contiguous(), dv(wd[:G]),
                                dv(wd_s[:G]), eb)
    assert torch.equal(bat.reshape(G * M, H), refb)
    gu_bf = torch.randn((33, 512), generator=torch.Generator().manual_seed(5)).to(torch.bfloat16).to(cuda)
    r = torch.zeros((33, 256), dtype=torch.bfloat16, device=cuda)
    ops.silu_run(gu_bf, r, torch.tensor([0, 33], dtype=torch.int32, device=cuda), 1)
    assert torch.equal(dense_silu(gu_bf), r)


@pytest.mark.gpu
def test_utils_ops(cuda, eps_pkg):
    from eps.utils import ops as uops

    from eps_b200 import ops

    g = torch.Generator().manual_seed(5)
    x = torch.randn((33, 1024), generator=g).to(torch.bfloat16).to(cuda)
    scale = torch.randn((1024,), generator=g).to(torch.bfloat16).to(cuda)
    out = torch.empty_like(x)
    uops._ops.rms_norm_op(out, x, scale, 1e-6)
    assert torch.equal(out, ops.rms_norm(x, scale, 1e-6))
    logits = torch.randn((50, 256), generator=g).to(torch.bfloat16).to(cuda)
    bias = torch.randn((256,), generator=g).to(cuda)
    es = torch.empty((50, 8), dtype=torch.float32, device=cuda)
    ei = torch.empty((50, 8), dtype=torch.int32, device=cuda)
    uops._ops.topk_sigmoid(logits, bias, es, ei, 50, 256, 8, 4, 8, 2.5)
    i2, s2 = ops.topk_sigmoid(logits, bias, 8, 4, 8, 2.5)
    assert torch.equal(ei, i2) and torch.equal(es, s2)


@pytest.mark.gpu
@pytest.mark.parametrize("case", [(96, 512, 256, 8, 2, 0, 0), (300, 1024, 512, 16, 4, 4, 256)])
def test_whole_layer_through_the_ops_matches_the_layer_bit_for_bit(cuda, oracle, eps_pkg, case):
    """The EP=1 expert layer driven purely through torch.ops.scheduler.* and torch.ops.executor.* (via the drop-in
    `eps` classes): quantise, plans, gathers, both grouped GEMMs, fused reduce.  Same kernels, same arguments: the
    output equals MoELayerFP8.forward bit for bit."""
    from eps.executor import AokGroupedGemm
    from eps.executor.silu import per_token_group_quant_fp8
    from eps.scheduler import Scheduler

    from eps_b200 import workloads
    from eps_b200.layer import MoELayerFP8, synthetic_expert_codes

    T, H, I, E, k, nz, sh = case
    cfg = workloads.CONFIGS[0].scaled(tokens_per_rank=T, hidden=H, inter=I, num_experts=E, top_k=k,
                                      num_zero_experts=nz, shared_inter=sh, bias="normal" if nz else "none")
    per = [synthetic_expert_codes(cfg, e, cuda) for e in range(E)]
    wgu, wgu_s, wd, wd_s = (torch.stack([p[i] for p in per]) for i in range(4))
    shared = tuple(t.unsqueeze(0) for t in synthetic_expert_codes(cfg, -1, cuda, inter=sh)) if sh else None
    x = workloads.make_tokens(cfg).to(cuda)
    idx, w = (t.to(cuda) for t in workloads.make_routing(cfg))
    layer = MoELayerFP8(H, I, E, k, T, wgu, wgu_s, wd, wd_s, shared=shared)
    want = layer.forward(x, idx, w)
    torch.cuda.synchronize()

    sched = Scheduler(k, E, H, H // 128, T, None, E, fp8_hidden=True)
    gemm = AokGroupedGemm(E)
    status = torch.zeros(4, dtype=torch.int32, device=cuda)
    for _ in range(2):   # the second call reuses the arenas
        xq, xs = per_token_group_quant_fp8(x)
        shared_out = None
        if sh:
            one = torch.tensor([0, T], dtype=torch.int32, device=cuda)
            g1 = AokGroupedGemm(1)
            aq, a_s = g1.run_gate_up_swiglu(xq, xs, shared[0], shared[1], one, status=status)
            shared_out = g1.run_down_weighted(aq, a_s, shared[2], shared[3], one, status=status)
        excl, n_recv = sched.rendezvous_and_plan(idx, w, T, 1, True, host_sync=False)
        D = n_recv * min(k, E)
        A = torch.empty((D, H), dtype=torch.uint8, device=cuda)
        A_s = torch.empty((D, H // 128), dtype=torch.float32, device=cuda)
        sched.prologue(w, xq, xs, A_s, raw_input=x)
        row_w = sched.gemm_row_weights()
        sched.dispatch(0)
        sched.gemm_expand(A, 0)
        act, act_s = gemm.run_gate_up_swiglu(A, A_s, wgu, wgu_s, excl, status=status)
        Y = gemm.run_down_weighted(act, act_s, wd, wd_s, excl, row_weights=row_w, status=status)
        out = torch.empty((T, H), dtype=torch.bfloat16, device=cuda)
        sched.reduce_single_rank(Y, out, shared=shared_out)
        torch.cuda.synchronize()
        sched.check_status()
        assert status.tolist()[0] == 0
        assert torch.equal(out, want)
    # and with the host read of the row count the reference's rendezvous does
    excl2, n2 = sched.rendezvous_and_plan(idx, w, T, 1, True)
    assert torch.equal(excl2, excl) and n2 == int((idx >= 0).any(dim=1).sum())
    sched.destroy()


@pytest.mark.gpu
def test_scheduler_reference_flow_bf16_through_the_ops(cuda, oracle, eps_pkg):
    """The reference's own calling sequence (bf16 rows, no scales, stages) with the expert FFN replaced by the
    identity: output[t] = sum_j w[t,j] * x[t]; plans against the oracle."""
    from eps.scheduler import Scheduler
    from helpers import random_routing

    T, H, E, k, S = 150, 2048, 16, 4, 2
    rng = np.random.default_rng(0)
    idx, w = random_routing(rng, T, k, E, 4)
    x = torch.randn((T, H), generator=torch.Generator().manual_seed(0)).to(torch.bfloat16).to(cuda)
    d_idx, d_w = torch.from_numpy(idx).to(cuda), torch.from_numpy(w).to(cuda)
    sched = Scheduler(k, E, H, 0, T, None, E)
    excl, n_recv = sched.rendezvous_and_plan(d_idx, d_w, T, S, False)
    send_map, send_incl = oracle.comm_plan(idx, E, 1, S)
    assert n_recv == send_incl[-1]
    rexcl, _ = oracle.gemm_plan(idx[send_map % T], k, 0, E, T, 1)
    assert np.array_equal(excl.cpu().numpy(), rexcl)
    sched.prologue(d_w, x)
    gemm_in = torch.zeros((int(rexcl[-1]), H), dtype=torch.bfloat16, device=cuda)
    for s in range(S):
        sched.dispatch(s)
        sched.gemm_expand(gemm_in, s)
        sched.local_reduce(gemm_in, s)   # identity FFN
        sched.combine(s)
    out = torch.empty((T, H), dtype=torch.bfloat16, device=cuda)
    sched.epilogue(out)
    torch.cuda.synchronize()
    want = x.float().cpu().numpy() * w.sum(1, keepdims=True)
    assert np.max(np.abs(out.float().cpu().numpy() - want)) <= 3e-2 * np.abs(want).max()
    with pytest.raises(RuntimeError, match="Invalid num_stages"):
        sched.rendezvous_and_plan(d_idx, d_w, T, 3, False)


@pytest.mark.gpu
def test_fast_ep_ops_bit_exact(cuda, oracle, eps_pkg):
    from eps.fast_ep import AllToAll
    from helpers import random_routing

    T, k, E, H = 90, 4, 16, 1024
    rng = np.random.default_rng(50)
    idx, w = random_routing(rng, T, k, E, 3)
    x = torch.randn((T, H), generator=torch.Generator().manual_seed(9)).to(torch.bfloat16)
    a2a = AllToAll(k, E, H, 256, None)
    excl = torch.empty((E + 1,), dtype=torch.int32, device=cuda)
    expert_x = torch.zeros((256 * k, H), dtype=torch.bfloat16, device=cuda)
    x_dev = x.to(cuda)   # combine reads the raw tokens again (identity experts): the caller keeps them alive
    a2a.dispatch(excl, expert_x, x_dev, torch.from_numpy(idx).to(cuda), 256)
    ex = excl.cpu().numpy()
    rexcl, rmap = oracle.fastep_expand_plan(idx, E)
    assert np.array_equal(ex, rexcl)
    y = torch.zeros_like(expert_x)
    for e in range(E):   # expert e scales its rows by (1 + e/8)
        y[ex[e]:ex[e + 1]] = (expert_x[ex[e]:ex[e + 1]].float() * (1 + e / 8)).to(torch.bfloat16)
    out = torch.empty((T, H), dtype=torch.bfloat16, device=cuda)
    a2a.combine(out, torch.from_numpy(w).to(cuda), y, 256)
    torch.cuda.synchronize()
    rows = torch.zeros((T * k, H), dtype=torch.bfloat16)
    for i in range(T * k):
        if rmap[i] < 1000000:
            rows[rmap[i]] = (x[i // k].float() * (1 + idx.reshape(-1)[i] / 8)).to(torch.bfloat16)
    want = oracle.fastep_reduce(_bits(rows), _bits(x), w, rmap)
    assert np.array_equal(_bits(out), want)


@pytest.mark.gpu
@pytest.mark.parametrize("D", [256, 512])
def test_fast_oep_ops(cuda, eps_pkg, D):
    """Lookups in a (here one-rank) sharded table: out[i] = table[id_i], negative ids leave their rows untouched; with
    do_permute the rows land n-gram-major."""
    from eps.fast_oep import AllToAll

    B, n, size = 37, 3, 500
    g = torch.Generator().manual_seed(D)
    table = torch.randn((size, D), generator=g).to(torch.bfloat16).to(cuda)
    ids = torch.randint(0, size, (B, n), generator=g, dtype=torch.int32)
    ids[torch.rand((B, n), generator=g) < 0.1] = -1
    ids = ids.to(cuda)
    a2a = AllToAll(D, size, 4096, None)
    for do_permute in (False, True):
        a2a.dispatch(ids)
        out = torch.full((B, n, D), 9.0, dtype=torch.bfloat16, device=cuda)
        a2a.combine(out, B * n, n, do_permute, table)
        torch.cuda.synchronize()
        flat = ids.reshape(-1)
        want = torch.full((B * n, D), 9.0, dtype=torch.bfloat16, device=cuda)
        for i in range(B * n):
            if flat[i] >= 0:
                d = i // n + (i % n) * B if do_permute else i
                want[d] = table[flat[i]]
        assert torch.equal(out.reshape(B * n, D), want)


@pytest.mark.gpu
def test_communication_ops_world_of_one(cuda, eps_pkg):
    from eps.communication import (MscclppCommunicator, MscclppCommunicatorParams, TPDPConvertor,
                                   sync_check_cuda_error_eps)

    uid = MscclppCommunicator.createUniqueId()
    assert uid.dtype == torch.uint8 and uid.device.type == "cpu" and uid.numel() == 128
    comm = MscclppCommunicator(uid, MscclppCommunicatorParams(0, 1, 1))
    assert int(comm) != 0
    comm.barrier()
    tpdp = TPDPConvertor(TPDPConvertor.Params(0, 64, 1, 512, comm))
    ctx = tpdp.get_all_gather_context(40, 256)
    assert ctx.input_row_offset == 0 and tuple(ctx.input().shape) == (40, 256) and tuple(ctx.output().shape) == (40, 256)
    ctx.input().copy_(torch.arange(40 * 256, device=cuda).reshape(40, 256).to(torch.bfloat16))
    tpdp.all_gather(ctx, None)
    rs = tpdp.get_reduce_scatter_context(40)
    before = rs.input().clone()
    tpdp.reduce_scatter(rs, torch.cuda.current_stream())
    sync_check_cuda_error_eps()
    assert torch.equal(rs.output(), before)    # a group of one: the sum over one rank
    with pytest.raises(RuntimeError, match="should be smaller than or equal to"):
        tpdp.get_all_gather_context(40, 1024).input()
    del tpdp
    with pytest.raises(RuntimeError, match="multi-node"):
        MscclppCommunicator(uid, MscclppCommunicatorParams(0, 2, 1))
