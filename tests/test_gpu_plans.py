"""CUDA plan kernels against the CPU oracle: every index array bit-exact."""
import numpy as np
import pytest
import torch

from helpers import random_routing, simulate_eps

pytestmark = pytest.mark.gpu

CASES = [
    # W, S, E, k, T, n_zero, max_tok
    (1, 1, 8, 2, 1, 0, 1),
    (1, 1, 8, 2, 3, 0, 3),
    (1, 1, 16, 4, 17, 0, 17),
    (1, 2, 16, 4, 256, 0, 256),
    (2, 1, 8, 3, 40, 2, 64),
    (2, 2, 16, 4, 300, 0, 512),
    (4, 2, 32, 8, 129, 4, 256),
    (8, 4, 256, 8, 128, 0, 128),
    (8, 1, 256, 8, 520, 0, 4096),
    (8, 2, 512, 12, 96, 256, 128),
    (1, 1, 128, 8, 2100, 0, 8192),
    (1, 1, 256, 8, 4096, 0, 4096),      # benchmark size on one rank
    (8, 2, 256, 8, 1024, 0, 4096),      # 8 ranks, 32 experts each, 2 stages
    (8, 1, 256, 8, 4096, 0, 4096),      # benchmark size on eight ranks: every rank receives ~21 600 tokens
    (4, 1, 768, 12, 300, 256, 512),     # 512 FFN + 256 identity experts would be E=512; here E=768 FFN stresses the bucket count
]


def _dev(a, cuda):
    return torch.from_numpy(np.ascontiguousarray(a)).to(cuda)


@pytest.mark.parametrize("W,S,E,k,T,nz,max_tok", CASES)
def test_eps_plans_bit_exact(cuda, oracle, W, S, E, k, T, nz, max_tok):
    from eps_b200 import ops

    rng = np.random.default_rng(W * 1000 + T)
    Ts = [max(0, T - 5 * r) for r in range(W)]
    routing = [random_routing(rng, Ts[r], k, E, nz) for r in range(W)]
    ranks = simulate_eps(oracle, [rt[0] for rt in routing], E, W, S, max_tok)
    EL = E // W
    for r in range(W):
        rk = ranks[r]
        idx, w = routing[r]
        if Ts[r] == 0:
            continue
        send_map, send_incl, glob_map, coll_incl, zero = ops.source_plans(_dev(idx, cuda), _dev(w, cuda), E, W, S)
        torch.cuda.synchronize()
        n = int(rk["send_incl"][-1])
        assert np.array_equal(send_incl.cpu().numpy(), rk["send_incl"])
        assert np.array_equal(send_map.cpu().numpy()[:n], rk["send_map"])
        assert np.array_equal(glob_map.cpu().numpy()[:Ts[r] * W].reshape(Ts[r], W), rk["glob_map"])
        assert np.array_equal(coll_incl.cpu().numpy(), rk["coll_incl"])
        assert np.array_equal(zero.cpu().numpy()[:Ts[r]], oracle.zero_plan(idx, w))
    gathered = np.stack([ranks[r]["send_incl"] for r in range(W)], 0)
    for r in range(W):
        rk = ranks[r]
        total = torch.full((1,), -1, dtype=torch.int32, device=cuda)
        recv_incl, remote = ops.recv_plan(_dev(gathered, cuda), r, W, S, total_rows=total)
        torch.cuda.synchronize()
        assert np.array_equal(recv_incl.cpu().numpy(), rk["recv_incl"])
        assert np.array_equal(remote.cpu().numpy(), rk["remote"])
        assert total.item() == rk["R"]
        R = rk["R"]
        max_rows = max(R, 1) + 3
        ridx = np.full((max_rows, k), -7, dtype=np.int32)
        ridx[:R] = rk["ridx"]
        excl, gemm_map, inv_gemm, scale_map, red_map, ret_incl = ops.expert_plans(
            _dev(ridx, cuda), recv_incl, k, r * EL, (r + 1) * EL, W, S, max_tok, max_rows)
        torch.cuda.synchronize()
        D = int(rk["excl"][-1])
        assert np.array_equal(excl.cpu().numpy(), rk["excl"])
        assert np.array_equal(gemm_map.cpu().numpy()[:D], rk["gemm_map"])
        assert np.array_equal(scale_map.cpu().numpy()[:R], rk["scale_map"])
        assert np.array_equal(red_map.cpu().numpy()[:R * k].reshape(R, k), rk["red_map"])
        assert np.array_equal(ret_incl.cpu().numpy(), rk["ret_incl"])
        inv = inv_gemm.cpu().numpy()[:R * k]
        ok = inv < R * k
        assert ok.sum() == D and np.array_equal(gemm_map.cpu().numpy()[inv[ok]], np.nonzero(ok)[0])


def test_plans_same_for_every_cluster_size(cuda):
    """The plans are launched as clusters of 1..8 CTAs; the index arrays must not depend on the cluster size."""
    from eps_b200 import ops

    rng = np.random.default_rng(7)
    E, k, T, W, S = 64, 6, 3000, 2, 2
    idx, w = random_routing(rng, T, k, E, 3)
    outs = []
    for c in (1, 2, 4, 8):
        src = ops.source_plans(_dev(idx, cuda), _dev(w, cuda), E, W, S, max_cluster=c)
        recv_incl = torch.tensor([T // 2, T, T, T], dtype=torch.int32, device=cuda)  # two sources, two stages
        ridx = _dev(np.where(idx < 0, -1, idx).astype(np.int32), cuda)
        exp = ops.expert_plans(ridx, recv_incl, k, 0, E // W, W, S, T, T, max_cluster=c)
        torch.cuda.synchronize()
        outs.append([t.cpu().numpy().copy() for t in list(src[:4]) + list(exp)])
    n_sent = int(outs[0][1][-1])
    D = int(outs[0][4][-1])
    n_red = int(outs[0][9][-1])
    for o in outs[1:]:
        assert np.array_equal(o[1], outs[0][1]) and np.array_equal(o[3], outs[0][3])       # send_incl, coll_incl
        assert np.array_equal(o[0][:n_sent], outs[0][0][:n_sent])                           # send_map
        assert np.array_equal(o[2][:T * W], outs[0][2][:T * W])                             # glob_map
        assert np.array_equal(o[4], outs[0][4]) and np.array_equal(o[5][:D], outs[0][5][:D])  # excl, gemm_map
        assert np.array_equal(o[7][:n_red], outs[0][7][:n_red])
        assert np.array_equal(o[8][:n_red * k], outs[0][8][:n_red * k])
        assert np.array_equal(o[9], outs[0][9])
    with pytest.raises(Exception):
        ops.source_plans(_dev(idx, cuda), _dev(w, cuda), E, W, S, max_cluster=3)


def test_expert_plans_refuse_more_rows_than_promised(cuda):
    """A receive plan that claims more rows than max_rows (what every buffer was sized from) is not followed:
    the kernel compares and returns, the plans come out empty, the status word names the count, and the maps
    stay as they were."""
    from eps_b200 import ops

    k, EL, W, S, max_rows = 4, 8, 1, 1, 64
    ridx = torch.randint(0, EL, (max_rows, k), dtype=torch.int32, device=cuda)
    for claimed in (max_rows + 1, 5 * max_rows, -3):
        recv_incl = torch.tensor([claimed], dtype=torch.int32, device=cuda)
        status = torch.zeros(2, dtype=torch.int32, device=cuda)
        n = max_rows * k
        excl = torch.full((EL + 1,), 7, dtype=torch.int32, device=cuda)
        gemm_map, inv_gemm, red_map = (torch.full((n,), -9, dtype=torch.int32, device=cuda) for _ in range(3))
        scale_map = torch.full((max_rows,), -9, dtype=torch.int32, device=cuda)
        ret_incl = torch.full((W * S,), 7, dtype=torch.int32, device=cuda)
        from eps_b200._lib import call, ptr, stream_ptr
        call("epsb_expert_plans", ptr(ridx), ptr(recv_incl), k, 0, EL, W, S, max_rows, max_rows, ptr(excl),
             ptr(gemm_map), ptr(inv_gemm), ptr(scale_map), ptr(red_map), ptr(ret_incl), ptr(status), 0, stream_ptr())
        torch.cuda.synchronize()
        assert status.tolist() == [ops.PLAN_ROWS_EXCEEDED, claimed]
        assert excl.tolist() == [0] * (EL + 1) and ret_incl.tolist() == [0]
        for t in (gemm_map, inv_gemm, red_map, scale_map):
            assert bool((t == -9).all())
    # a count within the promise leaves the status word alone
    status = torch.zeros(2, dtype=torch.int32, device=cuda)
    recv_incl = torch.tensor([max_rows], dtype=torch.int32, device=cuda)
    out = ops.expert_plans(ridx, recv_incl, k, 0, EL, W, S, max_rows, max_rows, status=status)
    torch.cuda.synchronize()
    assert status.tolist() == [0, 0] and int(out[0][-1]) == max_rows * k


def test_source_plans_empty_tokens(cuda):
    from eps_b200 import ops

    idx = torch.empty((0, 4), dtype=torch.int32, device=cuda)
    w = torch.empty((0, 4), dtype=torch.float32, device=cuda)
    _, send_incl, _, coll_incl, _ = ops.source_plans(idx, w, 16, 2, 2)
    assert send_incl.cpu().tolist() == [0, 0, 0, 0] and coll_incl.cpu().tolist() == [0, 0, 0, 0]


def test_plan_errors(cuda):
    from eps_b200 import ops
    from eps_b200._lib import EpsError

    idx = torch.zeros((4, 2), dtype=torch.int32, device=cuda)
    w = torch.ones((4, 2), dtype=torch.float32, device=cuda)
    with pytest.raises(EpsError, match="Invalid num_stages"):
        ops.source_plans(idx, w, 12, 2, 4)
    with pytest.raises(EpsError):
        ops.source_plans(idx, w, 4096, 2, 1)


@pytest.mark.parametrize("E,k,T,nz", [(8, 2, 5, 0), (32, 4, 100, 0), (256, 8, 4096, 0), (512, 12, 700, 256), (24, 3, 64, 5)])
def test_fastep_expand_plan_bit_exact(cuda, oracle, E, k, T, nz):
    from eps_b200 import ops

    idx, _ = random_routing(np.random.default_rng(E + T), T, k, E, nz)
    excl, mapping = ops.fastep_expand_plan(_dev(idx, cuda), E)
    torch.cuda.synchronize()
    rex, rmap = oracle.fastep_expand_plan(idx, E)
    assert np.array_equal(excl.cpu().numpy(), rex)
    assert np.array_equal(mapping.cpu().numpy()[:T * k], rmap)


@pytest.mark.parametrize("W,E,k,T", [(1, 8, 2, 19), (2, 8, 3, 40), (4, 32, 4, 25), (8, 256, 8, 300)])
def test_fastep_plan_bit_exact(cuda, oracle, W, E, k, T):
    from eps_b200 import ops

    rng = np.random.default_rng(9 * W)
    ag = np.stack([oracle.fastep_expand_plan(random_routing(rng, T + r, k, E)[0], E)[0] for r in range(W)], 0)
    for d in range(W):
        got = ops.fastep_plan(_dev(ag, cuda), d, W, E)
        torch.cuda.synchronize()
        want = oracle.fastep_plan(ag, d, W, E)
        for g, w_ in zip(got, want):
            assert np.array_equal(g.cpu().numpy(), w_)
