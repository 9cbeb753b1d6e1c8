"""Shared test helpers: a multi-rank simulation of the EPS plan chain on the CPU oracle."""
import numpy as np


def random_routing(rng, T, k, E, n_zero=0, p_zero=0.0):
    """Distinct top-k ids per token out of E (+ optional negative ids for identity experts)."""
    idx = np.empty((T, k), dtype=np.int32)
    total = E + n_zero
    for t in range(T):
        idx[t] = rng.choice(total, size=k, replace=False)
    idx = np.where(idx >= E, -(idx - E) - 1, idx).astype(np.int32)
    w = rng.random((T, k)).astype(np.float32) + 0.1
    w /= w.sum(1, keepdims=True)
    return idx, w.astype(np.float32)


def simulate_eps(orc, idx_per_rank, E, W, S, max_tok):
    """Runs S1..S5 of every rank on the oracle and the two exchanges in numpy.

    Returns per-rank dicts with every plan plus the received index rows."""
    k = idx_per_rank[0].shape[1]
    EL = E // W
    ranks = []
    for r in range(W):
        send_map, send_incl = orc.comm_plan(idx_per_rank[r], E, W, S)
        ranks.append(dict(idx=idx_per_rank[r], T=idx_per_rank[r].shape[0], send_map=send_map, send_incl=send_incl))
    gathered = np.stack([ranks[r]["send_incl"] for r in range(W)], 0)
    for r in range(W):
        recv_incl, remote, total = orc.recv_plan(gathered, r, W, S)
        ranks[r].update(recv_incl=recv_incl, remote=remote, R=total)
    # dispatch of the index rows: sender s, dest d, stage st -> rows [b, e) of the send order
    for d in range(W):
        ridx = np.zeros((ranks[d]["R"], k), dtype=np.int32)
        src_of = np.zeros((ranks[d]["R"], 2), dtype=np.int64)  # (source rank, source token)
        for s in range(W):
            inc = ranks[s]["send_incl"]
            T_s = ranks[s]["T"]
            for st in range(S):
                i = d * S + st
                b = 0 if i == 0 else inc[i - 1]
                e = inc[i]
                off = ranks[s]["remote"][d * S + st]
                toks = ranks[s]["send_map"][b:e] % max(T_s, 1)
                ridx[off:off + (e - b)] = ranks[s]["idx"][toks]
                src_of[off:off + (e - b), 0] = s
                src_of[off:off + (e - b), 1] = toks
        ranks[d].update(ridx=ridx, src_of=src_of)
    for r in range(W):
        lo, hi = r * EL, (r + 1) * EL
        excl, gemm_map = orc.gemm_plan(ranks[r]["ridx"], k, lo, hi, max_tok, W)
        scale_map, red_map, ret_incl = orc.local_reduce_plan(ranks[r]["ridx"], ranks[r]["recv_incl"], gemm_map, excl,
                                                             k, lo, hi, W, S)
        glob_map, coll_incl = orc.global_reduce_plan(ranks[r]["idx"], ranks[r]["send_map"], ranks[r]["send_incl"], E,
                                                     W, S)
        ranks[r].update(excl=excl, gemm_map=gemm_map, scale_map=scale_map, red_map=red_map, ret_incl=ret_incl,
                        glob_map=glob_map, coll_incl=coll_incl)
    return ranks
