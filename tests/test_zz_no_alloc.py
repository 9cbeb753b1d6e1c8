"""epsb_expert_plans_noalloc: the expert-side plans for hosts that may not allocate device memory.

Some hosts of this library get every buffer handed to them before they start and must never call the device
allocator afterwards (a serving loop with a fixed memory plan, a plug-in inside a runtime that owns the arena).  They
cannot supply the kernel's private scratch, so this entry point keeps it in a fixed array inside the library.  The
test drives it through the C ABI twice in a row with different inputs — the array is shared by all calls and keeps
the previous call's contents — and requires every output to equal the allocating entry point's, bit for bit.

Collected last on purpose (file name), so that a run stopping at the first failure has run every other test first.
"""
import numpy as np
import pytest
import torch

from helpers import random_routing, simulate_eps

pytestmark = pytest.mark.gpu


def _plans_both_ways(cuda, oracle, seed, W, S, E, k, T, max_tok):
    from eps_b200._lib import call, ptr, stream_ptr

    rng = np.random.default_rng(seed)
    routing = [random_routing(rng, T, k, E, 2) for _ in range(W)]
    ranks = simulate_eps(oracle, [rt[0] for rt in routing], E, W, S, max_tok)
    EL = E // W
    for r in range(W):
        rk = ranks[r]
        R = rk["R"]
        max_rows = R + 2
        ridx = torch.full((max_rows, k), -5, dtype=torch.int32, device=cuda)
        ridx[:R] = torch.from_numpy(rk["ridx"]).to(cuda)
        recv_incl = torch.from_numpy(rk["recv_incl"]).to(cuda)

        def outputs():
            n = max_rows * k
            return [torch.full((EL + 1,), -1, dtype=torch.int32, device=cuda),   # excl
                    torch.full((n,), -1, dtype=torch.int32, device=cuda),        # gemm_map
                    torch.full((max_rows,), -1, dtype=torch.int32, device=cuda), # scale_map
                    torch.full((n,), -1, dtype=torch.int32, device=cuda),        # red_map
                    torch.full((W * S,), -1, dtype=torch.int32, device=cuda)]    # ret_incl

        a, b = outputs(), outputs()
        inv = torch.empty((max_rows * k,), dtype=torch.int32, device=cuda)
        call("epsb_expert_plans", ptr(ridx), ptr(recv_incl), k, r * EL, (r + 1) * EL, W, S, max_tok, max_rows,
             ptr(a[0]), ptr(a[1]), ptr(inv), ptr(a[2]), ptr(a[3]), ptr(a[4]), None, 0, stream_ptr())
        call("epsb_expert_plans_noalloc", ptr(ridx), ptr(recv_incl), k, r * EL, (r + 1) * EL, W, S, max_tok,
             max_rows, ptr(b[0]), ptr(b[1]), ptr(b[2]), ptr(b[3]), ptr(b[4]), None, 0, stream_ptr())
        torch.cuda.synchronize()
        D = int(rk["excl"][-1])
        for x, y in zip(a, b):
            assert torch.equal(x, y)   # integer plans: exact, including the untouched padding
        assert np.array_equal(b[0].cpu().numpy(), rk["excl"])
        assert np.array_equal(b[1].cpu().numpy()[:D], rk["gemm_map"])
        assert np.array_equal(b[3].cpu().numpy()[:R * k].reshape(R, k), rk["red_map"])


def test_noalloc_matches_allocating_entry_point_twice_in_a_row(cuda, oracle):
    # two calls back to back on the shared array: a larger problem first, then a smaller one with other routing,
    # so the second call runs over the first call's leftovers
    _plans_both_ways(cuda, oracle, seed=1, W=2, S=2, E=16, k=4, T=300, max_tok=512)
    _plans_both_ways(cuda, oracle, seed=2, W=4, S=1, E=32, k=8, T=90, max_tok=128)


def test_noalloc_rejects_sizes_beyond_the_built_in_scratch(cuda):
    from eps_b200._lib import EpsError, call

    with pytest.raises(EpsError, match="exceeds the built-in scratch"):
        call("epsb_expert_plans_noalloc", None, None, 8, 0, 8, 1, 1, 4096, (1 << 20) // 8 + 1, None, None, None, None,
             None, None, 0, None)
