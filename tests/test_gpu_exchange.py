"""The device-side expert-parallel exchange (publish / receive plans, permute-on-send put, flag waits, fused local
reduce + store) on ONE GPU: W ranks are emulated by W exchange objects whose regions all live on this device, and the
phases run in lock step (every rank publishes, then every rank receives, ...), so every flag a kernel waits for is
already set when the kernel starts.  Checked against the CPU oracle's multi-rank simulation of the plan chain."""
import ctypes

import numpy as np
import pytest
import torch

from helpers import random_routing, simulate_eps

pytestmark = pytest.mark.gpu

PUT_META, PUT_SCALES, PUT_HIDDEN = 1, 2, 4
FLAG_META = 1


class Rank:
    pass


def _make_ranks(cuda, W, max_tok, S_max, k, H, elem, sd):
    from eps_b200 import _lib
    from eps_b200.scheduler import device_view

    nbytes = ctypes.c_int64()
    _lib.call("epsb_exchange_region_bytes", W, max_tok, S_max, k, H, elem, sd, ctypes.byref(nbytes))
    regions = []
    for _ in range(W):
        p = ctypes.c_void_p()
        h = (ctypes.c_uint8 * 64)()
        _lib.call("epsb_symm_alloc", nbytes.value, ctypes.byref(p), h)
        regions.append(p.value)
    ranks = []
    rows = max_tok * W
    for r in range(W):
        rk = Rank()
        arr = (ctypes.c_void_p * W)(*regions)
        x = ctypes.c_void_p()
        _lib.call("epsb_exchange_create", r, W, max_tok, S_max, k, H, elem, sd, arr, ctypes.byref(x))
        rk.x, rk.region = x, regions[r]
        rk.status = torch.zeros(4, dtype=torch.int32, device=cuda)

        def arena(which, par, shape, dtype, x=x):
            p = ctypes.c_void_p()
            _lib.call("epsb_exchange_arena", x, which, par, ctypes.byref(p))
            return device_view(p.value, shape, dtype, cuda)

        hid = torch.uint8 if elem == 1 else torch.bfloat16
        rk.idx = [arena(0, par, (rows, k), torch.int32) for par in (0, 1)]
        rk.w = [arena(1, par, (rows, k), torch.float32) for par in (0, 1)]
        rk.hidden = [arena(2, par, (rows, H), hid) for par in (0, 1)]
        rk.scales = [arena(3, par, (rows, sd), torch.float32) for par in (0, 1)]
        rk.out = arena(4, 0, (rows, H), torch.bfloat16)
        ranks.append(rk)
    return ranks, regions


def _free(ranks, regions):
    from eps_b200 import _lib

    torch.cuda.synchronize()
    for rk in ranks:
        _lib.call("epsb_exchange_destroy", rk.x)
    for p in regions:
        _lib.call("epsb_symm_free", p)


@pytest.mark.parametrize("W,S,E,k,T", [(2, 1, 8, 2, 37), (4, 2, 32, 4, 150), (8, 1, 64, 8, 64), (3, 3, 27, 5, 0),
                                       (8, 2, 256, 8, 700)])   # the last: plans as multi-CTA clusters, 32 experts per rank
def test_exchange_lock_step(cuda, oracle, W, S, E, k, T):
    from eps_b200 import _lib, ops
    from eps_b200._lib import call, ptr, stream_ptr

    H, sd, max_tok = 256, 3, max(T, 1) + 5
    EL = E // W
    ranks, regions = _make_ranks(cuda, W, max_tok, EL, k, H, 2, sd)
    rng = np.random.default_rng(100 * W + S)
    try:
        for call_no in range(3):   # three calls: both parities of the double-buffered arenas, then the first again
            Ts = [T if r != 1 else max(T - 3, 0) for r in range(W)]          # ragged token counts
            routing = [random_routing(rng, Ts[r], k, E, 2) for r in range(W)]
            sim = simulate_eps(oracle, [rt[0] for rt in routing], E, W, S, max_tok)
            xs = [torch.from_numpy(rng.integers(-1, 2, (Ts[r], H)).astype(np.float32)).to(torch.bfloat16).to(cuda)
                  for r in range(W)]
            scl = [torch.from_numpy(rng.random((Ts[r], sd)).astype(np.float32)).to(cuda) for r in range(W)]
            d_idx = [torch.from_numpy(routing[r][0]).to(cuda) for r in range(W)]
            d_w = [torch.from_numpy(routing[r][1]).to(cuda) for r in range(W)]
            src = []
            for r, rk in enumerate(ranks):
                src.append(ops.source_plans(d_idx[r], d_w[r], E, W, S))
                e = ctypes.c_int()
                call("epsb_exchange_begin", rk.x, ctypes.byref(e))
                rk.epoch = e.value
                call("epsb_exchange_publish_plans", rk.x, ptr(src[r][1]), ptr(src[r][3]), S, stream_ptr())
            recv_incl = []
            for r, rk in enumerate(ranks):
                ri = torch.empty((W * S,), dtype=torch.int32, device=cuda)
                call("epsb_exchange_recv_plans", rk.x, S, ptr(ri), ptr(rk.status), 0, stream_ptr())
                recv_incl.append(ri)
            for r, rk in enumerate(ranks):
                call("epsb_exchange_put", rk.x, FLAG_META, -1, PUT_META | PUT_SCALES | PUT_HIDDEN, ptr(d_idx[r]),
                     ptr(d_w[r]), ptr(xs[r]), ptr(scl[r]), ptr(src[r][0]), ptr(src[r][1]), Ts[r], S, stream_ptr())
            for rk in ranks:
                call("epsb_exchange_wait", rk.x, FLAG_META, ptr(rk.status), 0, stream_ptr())
            torch.cuda.synchronize()
            par = ranks[0].epoch & 1
            exp_plans = []
            for d, rk in enumerate(ranks):
                assert rk.status.tolist()[0] == 0
                sd_ = sim[d]
                R = sd_["R"]
                assert np.array_equal(recv_incl[d].cpu().numpy(), sd_["recv_incl"])
                assert np.array_equal(rk.idx[par][:R].cpu().numpy(), sd_["ridx"])
                so = sd_["src_of"]
                for i in range(R):
                    s_rank, tok = int(so[i, 0]), int(so[i, 1])
                    assert torch.equal(rk.hidden[par][i], xs[s_rank][tok])
                    assert torch.equal(rk.scales[par][i], scl[s_rank][tok])
                    assert torch.equal(rk.w[par][i], d_w[s_rank][tok])
                # expert side: plans on the received ids, then rows whose value encodes (token row, expert)
                pl = ops.expert_plans(rk.idx[par], recv_incl[d], k, d * EL, (d + 1) * EL, W, S, max_tok, max_tok * W)
                exp_plans.append(pl)
                assert np.array_equal(pl[0].cpu().numpy(), sd_["excl"])
            ys = []
            for d, rk in enumerate(ranks):
                excl, gemm_map = exp_plans[d][0], exp_plans[d][1]
                D = int(excl[-1])
                gm = gemm_map[:D].long()
                factor = (rk.idx[par].flatten()[gm] % 2 + 1).float()
                y = (rk.hidden[par][gm // k].float() * factor[:, None]).to(torch.bfloat16)
                ys.append(torch.cat([y, torch.zeros((1, H), dtype=torch.bfloat16, device=cuda)]))
            slot = 2 + EL   # the first combine flag of an exchange created for EL stages
            for d, rk in enumerate(ranks):
                call("epsb_exchange_local_reduce_put", rk.x, slot, ptr(ys[d]), ptr(exp_plans[d][4]),
                     ptr(exp_plans[d][5]), S, -1, max_tok * W, stream_ptr())
            for rk in ranks:
                call("epsb_exchange_wait", rk.x, slot, ptr(rk.status), 0, stream_ptr())
            for r, rk in enumerate(ranks):
                if Ts[r] == 0:
                    continue
                out = torch.empty((Ts[r], H), dtype=torch.bfloat16, device=cuda)
                ops.global_reduce(rk.out, src[r][2], out, W)
                idx_n = routing[r][0]
                mult = np.where(idx_n >= 0, idx_n % 2 + 1, 0).sum(1).astype(np.float32)
                want = xs[r].float().cpu().numpy() * mult[:, None]
                torch.cuda.synchronize()
                assert rk.status.tolist()[0] == 0
                assert np.array_equal(out.float().cpu().numpy(), want)
    finally:
        _free(ranks, regions)


def test_exchange_waits_are_bounded(cuda):
    """A peer that never shows up: the receive-plan kernel and the data wait give up after their (millisecond) limit,
    report which peer they waited for, and leave an empty exchange behind; the device stays usable."""
    from eps_b200._lib import call, ptr, stream_ptr

    W, S, k, H = 2, 1, 2, 128
    ranks, regions = _make_ranks(cuda, W, 16, 4, k, H, 1, 1)
    try:
        rk = ranks[0]
        plan = torch.tensor([3, 5], dtype=torch.int32, device=cuda)
        call("epsb_exchange_begin", rk.x, None)
        call("epsb_exchange_publish_plans", rk.x, ptr(plan), ptr(plan), S, stream_ptr())   # rank 1 never publishes
        recv_incl = torch.full((W * S,), 99, dtype=torch.int32, device=cuda)
        call("epsb_exchange_recv_plans", rk.x, S, ptr(recv_incl), ptr(rk.status), 2_000_000, stream_ptr())
        torch.cuda.synchronize()
        assert rk.status.tolist()[:2] == [61, 1]                  # EPSB_EXCHANGE_TIMEOUT_PLANS, waiting for peer 1
        assert recv_incl.tolist() == [0, 0]
        rk.status.zero_()
        call("epsb_exchange_wait", rk.x, 1, ptr(rk.status), 2_000_000, stream_ptr())        # nobody ever put
        torch.cuda.synchronize()
        st = rk.status.tolist()
        assert st[0] == 70 + 1 and st[1] in (0, 1)
        assert int(torch.ones(4, device=cuda).sum().item()) == 4   # the context is alive
    finally:
        _free(ranks, regions)


def test_exchange_argument_errors(cuda):
    from eps_b200._lib import EpsError, call

    n = ctypes.c_int64()
    with pytest.raises(EpsError, match="ep_world_size"):
        call("epsb_exchange_region_bytes", 9, 16, 1, 2, 128, 1, 1, ctypes.byref(n))
    with pytest.raises(EpsError, match="multiple of 16"):
        call("epsb_exchange_region_bytes", 2, 16, 1, 2, 100, 1, 1, ctypes.byref(n))
    call("epsb_exchange_region_bytes", 2, 16, 1, 2, 128, 1, 1, ctypes.byref(n))
    assert n.value > 0 and n.value % 256 == 0
