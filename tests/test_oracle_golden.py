"""The oracle's parity pin: golden vectors recorded from the REFERENCE's own kernels (compiled from
the reference sources and run on a B200 by tests/golden/make_ref_fixtures.py)."""
import os

import numpy as np
import pytest

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def _load(name):
    path = os.path.join(GOLD, name)
    if not os.path.exists(path):
        pytest.fail(f"golden fixture {name} is missing")
    return np.load(path)


def test_plans_match_reference_kernels(oracle):
    g = _load("ref_plans.npz")
    n_checked = 0
    for ci, (W, S, E, k, T, nz, max_tok) in enumerate(g["plan_cases"].tolist()):
        EL = E // W
        for r in range(W):
            pre = f"c{ci}_r{r}_"
            idx, w = g[pre + "idx"], g[pre + "w"]
            send_map, send_incl = oracle.comm_plan(idx, E, W, S)
            assert np.array_equal(send_map, g[pre + "send_map"])
            assert np.array_equal(send_incl, g[pre + "send_incl"])
            glob, coll = oracle.global_reduce_plan(idx, send_map, send_incl, E, W, S)
            assert np.array_equal(glob, g[pre + "glob_map"])
            assert np.array_equal(coll, g[pre + "coll_incl"])
            assert np.array_equal(oracle.zero_plan(idx, w), g[pre + "zero_scale"])
            if pre + "ridx" not in g:
                continue
            ridx, recv_incl = g[pre + "ridx"], g[pre + "recv_incl"]
            excl, gmap = oracle.gemm_plan(ridx, k, r * EL, (r + 1) * EL, max_tok, W)
            assert np.array_equal(excl, g[pre + "excl"])
            assert np.array_equal(gmap, g[pre + "gemm_map"])
            scale_map, red_map, ret_incl = oracle.local_reduce_plan(ridx, recv_incl, gmap, excl, k, r * EL,
                                                                    (r + 1) * EL, W, S)
            for tag in ("thr_", "dec_"):  # the reference's threaded kernel and its one-thread decode kernel
                if pre + tag + "scale_map" in g:
                    assert np.array_equal(scale_map, g[pre + tag + "scale_map"])
                    assert np.array_equal(red_map, g[pre + tag + "red_map"])
                    assert np.array_equal(ret_incl, g[pre + tag + "ret_incl"])
                    n_checked += 1
    assert n_checked >= 20


def test_quant_matches_reference_kernel(oracle):
    g = _load("ref_quant.npz")
    q, s = oracle.quant_1x128(g["x"], div_mode=1)
    assert np.array_equal(s.view(np.uint32), g["s"].view(np.uint32))
    assert np.array_equal(q, g["q"])
    # the IEEE variant differs from the reference kernel by at most 1 ulp in the scale
    _, s0 = oracle.quant_1x128(g["x"], div_mode=0)
    assert np.max(np.abs(s0.view(np.int32).astype(np.int64) - g["s"].view(np.int32))) <= 1


def test_swiglu_matches_reference_kernel(oracle):
    g = _load("ref_silu.npz")
    gu = oracle.bf16_to_f32(g["gu"])
    act = oracle.bf16_to_f32(oracle.bf16_bits(oracle.swiglu(gu)))
    ref = oracle.bf16_to_f32(g["act"])
    # the reference uses __expf (a few ulp off expf): allow one bf16 ulp, and require most outputs identical
    assert np.all(np.abs(act - ref) <= np.abs(ref) * 2.0 ** -7 + 1e-30)
    assert np.mean(act == ref) > 0.99


def test_router_matches_reference_kernel(oracle):
    """The oracle's router against vectors recorded from the reference's topk_sigmoid kernel on a B200.  The device's
    expf and numpy's exp may differ in the last place, so the scales are compared to a few ulp and a differing index
    must sit at a tie of the biased scores."""
    if not os.path.exists(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "ref_router.npz")):
        pytest.skip("tests/golden/ref_router.npz has not been recorded")
    g = _load("ref_router.npz")
    for tag, scores in (("", g["scores"]), ("_bf16", oracle.bf16_to_f32(g["scores_bf16"]))):
        idx, w, biased = oracle.topk_sigmoid(scores, g["bias"], 8, 4, 8, 2.5)
        ref_idx, ref_w = g["idx" + tag], g["w" + tag]
        diff = idx != ref_idx
        if diff.any():
            rows = np.nonzero(diff)[0]
            a, b = biased[rows, idx[diff]], biased[rows, ref_idx[diff]]
            assert np.all(np.abs(a - b) <= 4 * np.finfo(np.float32).eps * np.abs(b))
        same = ~diff.any(axis=1)
        assert same.mean() > 0.95
        assert np.allclose(w[same], ref_w[same], rtol=2e-6, atol=0)



def test_fastep_matches_reference_kernels(oracle):
    """fast_ep's expand plan, the plans derived from the all-gathered counts and the weighted combine against vectors
    recorded from the reference's own kernels (both its per-expert-count instantiations and its generic kernels)."""
    if not os.path.exists(os.path.join(GOLD, "ref_fastep.npz")):
        pytest.skip("tests/golden/ref_fastep.npz has not been recorded")
    g = _load("ref_fastep.npz")
    for ci, (T, k, E, W, nz) in enumerate(g["cases"].tolist()):
        pre = f"c{ci}_"
        idx, w = g[pre + "idx"], g[pre + "w"]
        excl, mapping = oracle.fastep_expand_plan(idx, E)
        assert np.array_equal(excl, g[pre + "excl"]) and np.array_equal(mapping, g[pre + "mapping"])
        ag = g[pre + "all_gathered"]
        for r in range(W):   # the table rows are expand plans too
            assert ag[r, 0] == 0 and np.all(np.diff(ag[r]) >= 0)
        for rank in (0, W - 1):
            plan = oracle.fastep_plan(ag, rank, W, E)
            for name, mine in zip(("remote_recv", "local_send", "gemm_plan", "arr_src", "arr_rows", "arr_dst"), plan):
                assert np.array_equal(mine, g[pre + f"r{rank}_" + name][:len(mine)]), (ci, rank, name)
        if pre + "reduce_rows" in g:
            rows, m = g[pre + "reduce_rows"], g[pre + "reduce_map"]
            n, H = len(rows), g[pre + "reduce_x"].shape[1]
            # the sampled tokens as a little problem of their own: row j of token i sits at position i*k + j
            ys = g[pre + "reduce_y"].reshape(n * k, H)
            local_map = np.where(m < 1000000, np.arange(n * k).reshape(n, k), 1000000 + np.arange(n)[:, None])
            out = oracle.fastep_reduce(ys, g[pre + "reduce_x"], w[rows], local_map.reshape(-1).astype(np.int32))
            assert np.array_equal(out, g[pre + "reduce_out"])
