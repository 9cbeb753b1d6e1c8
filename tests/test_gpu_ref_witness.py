"""The reference's OWN kernels (compiled from its sources into oracle/_ref/) run on the GPU beside
the oracle and this repository's kernels.  Skipped where the prebuilt library is absent."""
import numpy as np
import pytest
import torch

from helpers import random_routing, simulate_eps

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ref():
    from oracle import ref_kernels

    if not ref_kernels.available():
        pytest.skip("oracle/_ref/libeps_ref.so was not built (needs the reference checkout)")
    return ref_kernels


CASES = [(1, 1, 8, 2, 37, 0, 64), (2, 2, 16, 4, 300, 2, 512), (4, 2, 32, 8, 129, 4, 256), (8, 4, 256, 8, 128, 0, 128)]


@pytest.mark.parametrize("W,S,E,k,T,nz,max_tok", CASES)
def test_reference_plan_kernels_agree_with_oracle(cuda, oracle, ref, W, S, E, k, T, nz, max_tok):
    rng = np.random.default_rng(77 + W)
    Ts = [max(1, T - 5 * r) for r in range(W)]
    routing = [random_routing(rng, Ts[r], k, E, nz) for r in range(W)]
    ranks = simulate_eps(oracle, [rt[0] for rt in routing], E, W, S, max_tok)
    EL = E // W
    for r in range(W):
        idx, w = routing[r]
        rk = ranks[r]
        d_idx = torch.from_numpy(idx).to(cuda)
        send_map, send_incl = ref.comm_plan(d_idx, E, W, S)
        n = int(rk["send_incl"][-1])
        assert np.array_equal(send_incl.cpu().numpy(), rk["send_incl"])
        assert np.array_equal(send_map.cpu().numpy()[:n], rk["send_map"])
        glob, coll = ref.global_reduce_plan(d_idx, send_map, send_incl, E, W, S)
        assert np.array_equal(glob.cpu().numpy()[:Ts[r] * W].reshape(Ts[r], W), rk["glob_map"])
        assert np.array_equal(coll.cpu().numpy(), rk["coll_incl"])
        z = ref.zero_plan(d_idx, torch.from_numpy(w).to(cuda))
        assert np.array_equal(z.cpu().numpy()[:Ts[r]], oracle.zero_plan(idx, w))
        R = rk["R"]
        if R == 0:
            continue
        d_ridx = torch.from_numpy(rk["ridx"]).to(cuda)
        d_recv = torch.from_numpy(rk["recv_incl"]).to(cuda)
        excl, gmap = ref.gemm_plan(d_ridx, d_recv, k, r * EL, (r + 1) * EL, E, W, S, max_tok)
        D = int(rk["excl"][-1])
        assert np.array_equal(excl.cpu().numpy(), rk["excl"])
        assert np.array_equal(gmap.cpu().numpy()[:D], rk["gemm_map"])
        for ngt in (sum(Ts), 16):
            scale_map, red_map, ret_incl = ref.local_reduce_plan(d_ridx, d_recv, gmap, excl, k, r * EL, (r + 1) * EL,
                                                                 E, W, S, max_tok, ngt)
            assert np.array_equal(scale_map.cpu().numpy()[:R], rk["scale_map"])
            assert np.array_equal(red_map.cpu().numpy()[:R * k].reshape(R, k), rk["red_map"])
            assert np.array_equal(ret_incl.cpu().numpy(), rk["ret_incl"])


def test_reference_quant_kernel(cuda, oracle, ref):
    from eps_b200 import ops

    x = torch.randn((300, 2048), generator=torch.Generator().manual_seed(3)).to(torch.bfloat16)
    x[3, 128:256] = 0
    xd = x.to(cuda)
    rq, rs = ref.quant_1x128(xd)
    q1, s1 = ops.per_token_group_quant_fp8(xd, div_mode=1)
    assert torch.equal(s1, rs) and torch.equal(q1, rq), "div_mode=1 must reproduce the reference kernel bit for bit"
    q0, s0 = ops.per_token_group_quant_fp8(xd, div_mode=0)
    ulp = (s0.view(torch.int32) - rs.view(torch.int32)).abs().max().item()
    assert ulp <= 2
    frac_scale = (s0 != rs).float().mean().item()
    frac_code = (q0 != rq).float().mean().item()
    print(f"IEEE vs div.full: {frac_scale:.2%} of scales differ (max {ulp} ulp), {frac_code:.4%} of codes differ")
    assert frac_code < 0.02


def test_reference_silu_kernel(cuda, ref):
    from eps_b200 import ops

    gu = torch.randn((77, 2 * 2048), generator=torch.Generator().manual_seed(5)).to(torch.bfloat16).to(cuda)
    excl = torch.tensor([0, 30, 77], dtype=torch.int32, device=cuda)
    want = ref.silu(gu, excl, 2, 77)
    got = torch.zeros_like(want)
    ops.silu_run(gu, got, excl, 2)
    assert torch.equal(got, want)


def test_reference_reduce_kernels(cuda, oracle, ref):
    from eps_b200 import ops

    W, S, E, k, T, max_tok, H = 2, 2, 16, 4, 200, 256, 2048
    rng = np.random.default_rng(11)
    routing = [random_routing(rng, T, k, E, 2) for _ in range(W)]
    ranks = simulate_eps(oracle, [rt[0] for rt in routing], E, W, S, max_tok)
    rk = ranks[0]
    R, D = rk["R"], int(rk["excl"][-1])
    g = torch.Generator().manual_seed(1)
    y = torch.randn((D, H), generator=g).to(torch.bfloat16).to(cuda)
    w_recv = torch.rand((R, k), generator=g).to(cuda)
    dv = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(cuda)
    red_map, scale_map, ret_incl = dv(rk["red_map"].reshape(-1)), dv(rk["scale_map"]), dv(rk["ret_incl"])
    for stage in range(S):
        want = torch.zeros((R, H), dtype=torch.bfloat16, device=cuda)
        ref.local_reduce(red_map, scale_map, ret_incl, S, k, W, y, want, w_recv, T * W * k // W, stage)
        got = torch.zeros((R, H), dtype=torch.bfloat16, device=cuda)
        ops.local_reduce_ref(y, w_recv, scale_map, red_map, ret_incl, k, W, S, stage, got)
        torch.cuda.synchronize()
        assert torch.equal(got, want), f"local_reduce_ref differs from the reference kernel at stage {stage}"
    # global reduce + zero reduce
    n_sent = int(rk["send_incl"][-1])
    recv = torch.randn((n_sent, H), generator=g).to(torch.bfloat16).to(cuda)
    x = torch.randn((T, H), generator=g).to(torch.bfloat16).to(cuda)
    shared = torch.randn((T, H), generator=g).to(torch.bfloat16).to(cuda)
    idx, w = routing[0]
    zs = dv(oracle.zero_plan(idx, w))
    glob = dv(rk["glob_map"].reshape(-1))
    for sh in (None, shared):
        want = torch.zeros((T, H), dtype=torch.bfloat16, device=cuda)
        ref.global_reduce(glob, W, recv, want, sh)
        ref.zero_reduce(zs, x, want)
        got = torch.zeros((T, H), dtype=torch.bfloat16, device=cuda)
        ops.global_reduce(recv, glob, got, W, shared=sh, x=x, zero_scale=zs, ref_arith=True)
        torch.cuda.synchronize()
        assert torch.equal(got, want)


@pytest.mark.parametrize("T,k,E,W,nz", [(300, 8, 256, 8, 0), (77, 4, 32, 2, 3), (150, 6, 24, 4, 4), (4096, 8, 128, 4, 0)])
def test_reference_fastep_kernels(cuda, oracle, ref, T, k, E, W, nz):
    """fast_ep's own kernels (expandPlan, expand, allGatherPlan's plan kernels, arrange, reduce) from the reference's
    sources, beside this repository's and the oracle: plans bit for bit (both of the reference's code paths: the
    per-expert-count instantiations for E in {512, 256, 128, 32} and the generic block kernel), rows bit for bit."""
    from eps_b200 import ops

    H = 2048    # a hidden size the reference instantiates
    rng = np.random.default_rng(T + E)
    idx, w = random_routing(rng, T, k, E, nz)
    d_idx = torch.from_numpy(idx).to(cuda)
    # F1: expand plan
    r_excl, r_map = ref.fastep_expand_plan(d_idx, E)
    excl, mapping = ops.fastep_expand_plan(d_idx, E)
    o_excl, o_map = oracle.fastep_expand_plan(idx, E)
    torch.cuda.synchronize()
    assert np.array_equal(r_excl.cpu().numpy(), o_excl) and torch.equal(excl, r_excl)
    assert np.array_equal(r_map.cpu().numpy()[:T * k], o_map) and torch.equal(mapping[:T * k], r_map[:T * k])
    # F3: expand (scatter into send order)
    x = torch.randn((T, H), generator=torch.Generator().manual_seed(T)).to(torch.bfloat16).to(cuda)
    want = ref.fastep_expand(x, d_idx, r_excl, r_map, E)
    got = torch.zeros_like(want)
    ops.scatter_rows(x, got, mapping, k, T * k)
    torch.cuda.synchronize()
    assert torch.equal(got, want)
    # F2: plans from an all-gathered count table (this rank's column-block of every rank's counts)
    ag = np.zeros((W, E + 1), dtype=np.int32)
    for r in range(W):
        idx_r, _ = random_routing(np.random.default_rng(1000 * r + T), T - 7 * r, k, E, nz)
        ag[r] = oracle.fastep_expand_plan(idx_r, E)[0]
    d_ag = torch.from_numpy(ag).to(cuda)
    for rank in (0, W - 1):
        r_plan = ref.fastep_plan(d_ag.clone(), rank, W, E)
        m_plan = ops.fastep_plan(d_ag, rank, W, E)
        o_plan = oracle.fastep_plan(ag, rank, W, E)
        torch.cuda.synchronize()
        for name, a, b, c in zip(("remote_recv", "local_send", "gemm_plan", "arr_src", "arr_rows", "arr_dst"), r_plan,
                                 m_plan, o_plan):
            n = len(c)
            assert np.array_equal(a.cpu().numpy()[:n], c), f"reference vs oracle: {name}"
            assert np.array_equal(b.cpu().numpy()[:n], c), f"this repository vs oracle: {name}"
    # F3: arrange [source][expert] -> [expert][source] with rank 0's plan
    _, _, gplan, a_src, a_rows, a_dst = ops.fastep_plan(d_ag, 0, W, E)
    R = int(gplan[-1])
    rows_in = torch.randn((R + 3, H), generator=torch.Generator().manual_seed(1)).to(torch.bfloat16).to(cuda)
    want = torch.zeros((R + 3, H), dtype=torch.bfloat16, device=cuda)
    ref.fastep_arrange(rows_in, want, W, E, a_src, a_rows, a_dst, R)
    got = torch.zeros_like(want)
    ops.arrange_rows(rows_in, got, a_src, a_rows, a_dst, (E // W) * W, R + 3)
    torch.cuda.synchronize()
    assert torch.equal(got, want)
    # F3: reduce (weighted combine, identity-expert slots read the raw token, optional shared-expert rows)
    y = torch.randn((T * k, H), generator=torch.Generator().manual_seed(2)).to(torch.bfloat16).to(cuda)
    d_w = torch.from_numpy(w).to(cuda)
    shared = torch.randn((T, H), generator=torch.Generator().manual_seed(3)).to(torch.bfloat16).to(cuda)
    for sh in (None, shared):
        want = ref.fastep_reduce(y, x, d_w, d_idx, r_excl, r_map, E, shared=sh)
        got = torch.zeros((T, H), dtype=torch.bfloat16, device=cuda)
        ops.fastep_reduce(y, x, d_w, mapping, got, shared=sh)
        torch.cuda.synchronize()
        assert torch.equal(got, want[:T])
