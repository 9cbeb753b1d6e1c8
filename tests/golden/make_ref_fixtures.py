"""Records golden vectors from the REFERENCE's own kernels (oracle/_ref/libeps_ref.so) on a GPU.

Run on a B200:  python tests/golden/make_ref_fixtures.py [OUT_DIR] [--router-only | --fastep-only]
(OUT_DIR defaults to this directory, tests/golden/).  The CPU test tests/test_oracle_golden.py checks the oracle
against these files, which is the oracle's parity pin.
"""
import os
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

from helpers import random_routing, simulate_eps  # noqa: E402
from oracle import oracle as orc  # noqa: E402
from oracle import ref_kernels as ref  # noqa: E402

# W, S, E, k, T, n_zero, max_tok   (sizes keep the reference kernels' shared memory under the limit)
PLAN_CASES = [
    (1, 1, 8, 2, 37, 0, 64),
    (1, 2, 16, 4, 256, 0, 256),
    (2, 2, 16, 4, 300, 2, 512),
    (4, 2, 32, 8, 129, 4, 256),
    (8, 4, 256, 8, 128, 0, 128),
    (8, 1, 64, 6, 520, 8, 1024),
]


def record_router(out_dir, dev):
    """Router: the one shape the reference instantiates (256 experts, 8 groups, 4 of them kept, top-8)."""
    g = torch.Generator().manual_seed(123)
    scores = torch.randn((96, 256), generator=g)
    bias = torch.randn(256, generator=g) * 0.1
    idx, w = ref.topk_sigmoid(scores.to(dev), bias.to(dev), 8, 4, 8, 2.5)
    sb = scores.to(torch.bfloat16)
    idx_b, w_b = ref.topk_sigmoid(sb.to(dev), bias.to(dev), 8, 4, 8, 2.5)
    np.savez_compressed(os.path.join(out_dir, "ref_router.npz"), scores=scores.numpy(), bias=bias.numpy(),
                        idx=idx.cpu().numpy(), w=w.cpu().numpy(),
                        scores_bf16=sb.view(torch.int16).numpy().view(np.uint16), idx_bf16=idx_b.cpu().numpy(),
                        w_bf16=w_b.cpu().numpy())


# T, k, E, W, n_zero: E in {256, 32, 128} take the reference's per-expert-count kernels, 24 its generic block kernels
FASTEP_CASES = [(300, 8, 256, 8, 0), (77, 4, 32, 2, 3), (150, 6, 24, 4, 4), (1000, 8, 128, 4, 0)]


def record_fastep(out_dir, dev):
    """fast_ep: expand plan, the plans derived from an all-gathered count table, and the weighted combine, from the
    reference's own kernels (src/fast_ep/all_to_all/fast_ep_kernels.cu)."""
    blob = {"cases": np.array(FASTEP_CASES, dtype=np.int64)}
    H = 2048
    for ci, (T, k, E, W, nz) in enumerate(FASTEP_CASES):
        rng = np.random.default_rng(900 + ci)
        pre = f"c{ci}_"
        idx, w = random_routing(rng, T, k, E, nz)
        d_idx = torch.from_numpy(idx).to(dev)
        excl, mapping = ref.fastep_expand_plan(d_idx, E)
        blob[pre + "idx"], blob[pre + "w"] = idx, w
        blob[pre + "excl"], blob[pre + "mapping"] = excl.cpu().numpy(), mapping.cpu().numpy()[:T * k]
        ag = np.zeros((W, E + 1), dtype=np.int32)
        for r in range(W):
            idx_r, _ = random_routing(np.random.default_rng(5000 + 10 * ci + r), max(1, T - 7 * r), k, E, nz)
            ag[r] = ref.fastep_expand_plan(torch.from_numpy(idx_r).to(dev), E)[0].cpu().numpy()
        blob[pre + "all_gathered"] = ag
        for rank in (0, W - 1):
            plan = ref.fastep_plan(torch.from_numpy(ag).to(dev), rank, W, E)
            for name, t in zip(("remote_recv", "local_send", "gemm_plan", "arr_src", "arr_rows", "arr_dst"), plan):
                blob[pre + f"r{rank}_" + name] = t.cpu().numpy()
        if ci < 3:   # combine on a few rows of a hidden size the reference instantiates
            g = torch.Generator().manual_seed(ci)
            x = torch.randn((T, H), generator=g).to(torch.bfloat16)
            y = torch.randn((T * k, H), generator=g).to(torch.bfloat16)
            out = ref.fastep_reduce(y.to(dev), x.to(dev), torch.from_numpy(w).to(dev), d_idx, excl, mapping, E)
            rows = np.sort(np.random.default_rng(ci).choice(T, size=8, replace=False))
            b = lambda t: t.view(torch.int16).numpy().view(np.uint16)
            blob[pre + "reduce_rows"] = rows
            blob[pre + "reduce_x"] = b(x)[rows]
            blob[pre + "reduce_out"] = b(out.cpu())[rows]
            # the rows of y the sampled tokens read, by position in the send order
            m = mapping.cpu().numpy()[:T * k].reshape(T, k)[rows]
            blob[pre + "reduce_map"] = m
            ys = b(y)
            blob[pre + "reduce_y"] = np.stack([[ys[j] if j < 1000000 else np.zeros(H, np.uint16) for j in row] for row in m])
    np.savez_compressed(os.path.join(out_dir, "ref_fastep.npz"), **blob)


def main(out_dir):
    os.makedirs(out_dir, exist_ok=True)
    dev = torch.device("cuda:0")
    blob = {}
    for ci, (W, S, E, k, T, nz, max_tok) in enumerate(PLAN_CASES):
        rng = np.random.default_rng(4242 + ci)
        Ts = [max(1, T - 5 * r) for r in range(W)]
        routing = [random_routing(rng, Ts[r], k, E, nz) for r in range(W)]
        ranks = simulate_eps(orc, [rt[0] for rt in routing], E, W, S, max_tok)
        EL = E // W
        for r in range(W):
            idx, w = routing[r]
            d_idx = torch.from_numpy(idx).to(dev)
            send_map, send_incl = ref.comm_plan(d_idx, E, W, S)
            glob, coll = ref.global_reduce_plan(d_idx, send_map, send_incl, E, W, S)
            zero = ref.zero_plan(d_idx, torch.from_numpy(w).to(dev))
            n = int(send_incl[-1].item())
            pre = f"c{ci}_r{r}_"
            blob[pre + "idx"] = idx
            blob[pre + "w"] = w
            blob[pre + "send_map"] = send_map.cpu().numpy()[:n]
            blob[pre + "send_incl"] = send_incl.cpu().numpy()
            blob[pre + "glob_map"] = glob.cpu().numpy()[:Ts[r] * W].reshape(Ts[r], W)
            blob[pre + "coll_incl"] = coll.cpu().numpy()
            blob[pre + "zero_scale"] = zero.cpu().numpy()[:Ts[r]]
            # expert side: inputs are the rows this rank receives (built with the oracle's dispatch, which the
            # source-side fixtures above pin)
            rk = ranks[r]
            R = rk["R"]
            if R == 0:
                continue
            d_ridx = torch.from_numpy(rk["ridx"]).to(dev)
            d_recv = torch.from_numpy(rk["recv_incl"]).to(dev)
            excl, gmap = ref.gemm_plan(d_ridx, d_recv, k, r * EL, (r + 1) * EL, E, W, S, max_tok)
            D = int(excl[-1].item())
            for ngt in (sum(Ts), 16):  # the threaded kernel and the one-thread "decode" kernel
                if ngt * k <= 4096 and R > 4096:
                    continue
                scale_map, red_map, ret_incl = ref.local_reduce_plan(d_ridx, d_recv, gmap, excl, k, r * EL,
                                                                     (r + 1) * EL, E, W, S, max_tok, ngt)
                tag = "dec_" if ngt * k <= 4096 else "thr_"
                blob[pre + tag + "scale_map"] = scale_map.cpu().numpy()[:R]
                blob[pre + tag + "red_map"] = red_map.cpu().numpy()[:R * k].reshape(R, k)
                blob[pre + tag + "ret_incl"] = ret_incl.cpu().numpy()
            blob[pre + "ridx"] = rk["ridx"]
            blob[pre + "recv_incl"] = rk["recv_incl"]
            blob[pre + "excl"] = excl.cpu().numpy()
            blob[pre + "gemm_map"] = gmap.cpu().numpy()[:D]
    blob["plan_cases"] = np.array(PLAN_CASES, dtype=np.int64)
    np.savez_compressed(os.path.join(out_dir, "ref_plans.npz"), **blob)

    # quantisation: the reference kernel uses an approximate divide for the scale; record codes and scales
    g = torch.Generator().manual_seed(99)
    x = torch.randn((64, 1024), generator=g).to(torch.bfloat16)
    x[3, 128:256] = 0
    x[5] *= 1e-5
    q, s = ref.quant_1x128(x.to(dev))
    np.savez_compressed(os.path.join(out_dir, "ref_quant.npz"), x=x.view(torch.int16).numpy().view(np.uint16),
                        q=q.cpu().numpy(), s=s.cpu().numpy())

    # SwiGLU
    gu = torch.randn((40, 2 * 1408), generator=g).to(torch.bfloat16)
    excl = torch.tensor([0, 40], dtype=torch.int32)
    act = ref.silu(gu.to(dev), excl.to(dev), 1, 40)
    np.savez_compressed(os.path.join(out_dir, "ref_silu.npz"), gu=gu.view(torch.int16).numpy().view(np.uint16),
                        act=act.cpu().view(torch.int16).numpy().view(np.uint16))
    record_router(out_dir, dev)
    record_fastep(out_dir, dev)
    print("wrote fixtures to", out_dir, {k: v.shape for k, v in list(blob.items())[:4]})


if __name__ == "__main__":
    args = [a for a in sys.argv[1:] if not a.startswith("--")]
    out = args[0] if args else os.path.dirname(os.path.abspath(__file__))
    if "--router-only" in sys.argv:      # adds ref_router.npz without re-recording the other files
        os.makedirs(out, exist_ok=True)
        record_router(out, torch.device("cuda:0"))
    elif "--fastep-only" in sys.argv:    # adds ref_fastep.npz without re-recording the other files
        os.makedirs(out, exist_ok=True)
        record_fastep(out, torch.device("cuda:0"))
    else:
        main(out)
