"""The oracle's plan chain (S1..S6, F1, F2): a hand-worked case and end-to-end routing consistency."""
import numpy as np
import pytest

from helpers import random_routing, simulate_eps


def test_comm_plan_hand_worked(oracle):
    # 6 tokens, 4 experts, 2 ranks (2 experts each), 1 stage, top-2.  NT = ceil(6/16) = 1 thread.
    idx = np.array([[0, 2], [1, 0], [3, 2], [2, 1], [0, 1], [3, -1]], dtype=np.int32)
    send_map, incl = oracle.comm_plan(idx, E=4, W=2, S=1)
    # rank 0 (experts 0,1): leading expert per token: t0:0 t1:0 t3:1 t4:0 -> bucket 0: t0,t1,t4 ; bucket 1: t3
    # rank 1 (experts 2,3): t0:lead 0(e2) t2:0 (min(3,2)=2 -> local 0) t3:0 t5:1 -> bucket 0: t0,t2,t3 ; bucket 1: t5
    assert send_map.tolist() == [0, 1, 4, 3, 6 + 0, 6 + 2, 6 + 3, 6 + 5]
    assert incl.tolist() == [4, 8]
    glob, coll = oracle.global_reduce_plan(idx, send_map, incl, E=4, W=2, S=1)
    # rank-0 block (send rows 0..3 = t0,t1,t4,t3), tailing experts: t0:0 t1:1 t4:1 t3:1 -> order t0 | t1,t4,t3
    assert glob[0, 0] == 0 and glob[1, 0] == 1 and glob[4, 0] == 2 and glob[3, 0] == 3
    # rank-1 block (rows 4..7 = t0,t2,t3,t5), tails: t0:0 t2:1 t3:0 t5:1 -> t0,t3 | t2,t5
    assert glob[0, 1] == 4 and glob[3, 1] == 5 and glob[2, 1] == 6 and glob[5, 1] == 7
    assert glob[1, 1] == 12 and glob[2, 0] == 12 and glob[5, 0] == 12  # sentinel T*W
    assert coll.tolist() == [4, 8]
    z = oracle.zero_plan(idx, np.full((6, 2), 0.5, dtype=np.float32))
    assert z.tolist() == [0, 0, 0, 0, 0, 0.5]


def test_comm_plan_two_stages(oracle):
    idx = np.array([[0, 3], [2, 1], [3, 1]], dtype=np.int32)  # 1 rank, 4 experts, 2 stages of 2
    send_map, incl = oracle.comm_plan(idx, E=4, W=1, S=2)
    # leads: t0:0 t1:1 t2:1 -> stage 0 holds all three; tails: t0:3 t1:2 t2:3 -> all return in stage 1
    assert send_map.tolist() == [0, 1, 2] and incl.tolist() == [3, 3]
    glob, coll = oracle.global_reduce_plan(idx, send_map, incl, E=4, W=1, S=2)
    assert coll.tolist() == [0, 3]
    assert glob[:, 0].tolist() == [1, 0, 2]  # stable by tail: t1 (tail 2) first, then t0, t2 (tail 3)


def test_strided_thread_order(oracle):
    # 40 tokens all routed to expert 0: NT = ceil(40/16) = 3 threads; order is tid-major
    idx = np.zeros((40, 1), dtype=np.int32)
    send_map, _ = oracle.comm_plan(idx, E=2, W=1, S=1)
    expect = [t for tid in range(3) for t in range(tid, 40, 3)]
    assert send_map.tolist() == expect
    excl, gmap = oracle.gemm_plan(idx, 1, 0, 2, max_tok_per_gpu=40, W=1)
    assert gmap.tolist() == expect and excl.tolist() == [0, 40, 40]
    # with a larger max_tok_per_gpu the GEMM plan's thread count differs from the comm plan's
    excl, gmap = oracle.gemm_plan(idx, 1, 0, 2, max_tok_per_gpu=4096, W=1)
    assert gmap.tolist() == [t for tid in range(128) for t in range(tid, 40, 128)]


def test_empty_and_degenerate(oracle):
    send_map, incl = oracle.comm_plan(np.zeros((0, 4), dtype=np.int32), E=8, W=2, S=2)
    assert send_map.size == 0 and incl.tolist() == [0, 0, 0, 0]
    # every slot an identity expert: nothing is sent
    idx = -np.ones((5, 2), dtype=np.int32)
    send_map, incl = oracle.comm_plan(idx, E=4, W=2, S=1)
    assert send_map.size == 0 and incl.tolist() == [0, 0]
    excl, mp = oracle.fastep_expand_plan(idx, 4)
    assert excl.tolist() == [0] * 5 and mp.tolist() == [1000000 + t for t in range(5) for _ in range(2)]


def test_fastep_expand_descending(oracle):
    idx = np.array([[1, 0], [1, 2], [0, 1]], dtype=np.int32)
    excl, mp = oracle.fastep_expand_plan(idx, 3)
    assert excl.tolist() == [0, 2, 5, 6]
    # expert 1 slots i=0,2,5 get rows 4,3,2 (handed out from the end); expert 0: i=1->1, i=4->0
    assert mp.tolist() == [4, 1, 3, 5, 0, 2]


@pytest.mark.parametrize("W,S,E,k,T,nz", [(1, 1, 8, 2, 37, 0), (2, 2, 16, 4, 50, 0), (4, 1, 32, 8, 33, 4),
                                           (8, 4, 64, 6, 20, 8), (2, 1, 8, 3, 300, 0)])
def test_eps_chain_routes_every_pair(oracle, W, S, E, k, T, nz):
    """Push a per-(token, expert) value through dispatch -> GEMM order -> local reduce -> combine ->
    global reduce using only the plans; the result must equal the direct weighted sum."""
    rng = np.random.default_rng(100 * W + S)
    Ts = [T + 3 * r for r in range(W)]
    routing = [random_routing(rng, Ts[r], k, E, nz) for r in range(W)]
    ranks = simulate_eps(oracle, [rt[0] for rt in routing], E, W, S, max(Ts))
    EL = E // W

    def f(rank, tok, expert):  # the "expert output" for a (global token, expert) pair
        return (rank * 1000 + tok) * 1.0 + 0.001 * (expert + 1)

    # expert side
    for d in range(W):
        rk = ranks[d]
        R, D = rk["R"], rk["excl"][-1]
        assert D == len(rk["gemm_map"])
        y = np.zeros(D)
        for e in range(EL):
            for p in range(rk["excl"][e], rk["excl"][e + 1]):
                row, slot = divmod(int(rk["gemm_map"][p]), k)
                assert rk["ridx"][row, slot] == d * EL + e
                s, tok = rk["src_of"][row]
                y[p] = f(s, tok, d * EL + e)
        # received gate weights travel like the indices
        wrecv = np.stack([routing[s][1][tok] for s, tok in rk["src_of"]]) if R else np.zeros((0, k))
        send = np.zeros(R)
        for q in range(R):
            r = rk["scale_map"][q]
            for j in range(k):
                p = rk["red_map"][q, j]
                if p < R * k:
                    send[q] += wrecv[r, j] * y[p]
        rk["ret"] = send
        assert rk["ret_incl"][-1] == R
    # combine exchange: the return buffer of rank d is cut by (source, stage) like a dispatch in reverse
    gathered = np.stack([ranks[d]["ret_incl"] for d in range(W)], 0)
    for s in range(W):
        recv_incl, remote, total = oracle.recv_plan(gathered, s, W, S)
        assert total == ranks[s]["send_incl"][-1]
        assert np.array_equal(recv_incl, ranks[s]["coll_incl"])
        ranks[s]["coll_remote"] = remote
    for s in range(W):
        ranks[s]["collected"] = np.zeros(ranks[s]["send_incl"][-1])
    for d in range(W):
        inc = ranks[d]["ret_incl"]
        for s in range(W):
            for st in range(S):
                i = s * S + st
                b = 0 if i == 0 else inc[i - 1]
                e = inc[i]
                off = ranks[d]["coll_remote"][s * S + st]
                ranks[s]["collected"][off:off + e - b] = ranks[d]["ret"][b:e]
    for s in range(W):
        idx, w = routing[s]
        for t in range(Ts[s]):
            got = sum(ranks[s]["collected"][ranks[s]["glob_map"][t, ep]] for ep in range(W)
                      if ranks[s]["glob_map"][t, ep] < Ts[s] * W)
            want = sum(w[t, j] * f(s, t, idx[t, j]) for j in range(k) if idx[t, j] >= 0)
            assert abs(got - want) < 1e-6 * max(1.0, abs(want))


@pytest.mark.parametrize("W,E,k,T", [(1, 8, 2, 19), (2, 8, 3, 40), (4, 32, 4, 25)])
def test_fastep_chain(oracle, W, E, k, T):
    rng = np.random.default_rng(7 + W)
    EL = E // W
    routing = [random_routing(rng, T + r, k, E, 2) for r in range(W)]
    plans = [oracle.fastep_expand_plan(rt[0], E) for rt in routing]
    ag = np.stack([p[0] for p in plans], 0)
    for d in range(W):
        remote, send, gplan, src, rows, dst = oracle.fastep_plan(ag, d, W, E)
        # rows received by d, source-major then local expert; after arrange expert-major
        tot = sum(ag[s][(d + 1) * EL] - ag[s][d * EL] for s in range(W))
        assert gplan[-1] == tot and send[-1] == tot
        cover = np.zeros(tot, dtype=int)
        for p in range(EL * W):
            cover[dst[p]:dst[p] + rows[p]] += 1
        assert np.all(cover == 1)
        for s in range(W):
            assert remote[s] == sum(ag[j][(s + 1) * EL] - ag[j][s * EL] for j in range(d))
