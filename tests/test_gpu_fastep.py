"""fast_ep AllToAll (dispatch / combine) and the executor classes on one GPU."""
import numpy as np
import pytest
import torch

from helpers import random_routing

pytestmark = pytest.mark.gpu


def _bits(t):
    return t.view(torch.int16).cpu().numpy().view(np.uint16)


@pytest.mark.parametrize("T,k,E,H,nz", [(37, 2, 8, 256, 0), (300, 8, 32, 2048, 4), (64, 12, 24, 512, 8)])
def test_fastep_roundtrip_single_rank(cuda, oracle, T, k, E, H, nz):
    from eps_b200.fast_ep import AllToAll

    rng = np.random.default_rng(T)
    idx, w = random_routing(rng, T, k, E, nz)
    x = torch.randn((T, H), generator=torch.Generator().manual_seed(T)).to(torch.bfloat16).to(cuda)
    a2a = AllToAll(k, E, H, T, None)
    excl = torch.empty((E + 1,), dtype=torch.int32, device=cuda)
    expert_x = torch.zeros((T * k, H), dtype=torch.bfloat16, device=cuda)
    a2a.dispatch(excl, expert_x, x, torch.from_numpy(idx).to(cuda), T)
    torch.cuda.synchronize()
    rex, rmap = oracle.fastep_expand_plan(idx, E)
    assert np.array_equal(excl.cpu().numpy(), rex)
    # rows of expert e are the tokens routed to it, in descending pair index
    xe = expert_x.cpu()
    xc = x.cpu()
    for i in range(T * k):
        if rmap[i] < 1000000:
            assert torch.equal(xe[rmap[i]], xc[i // k])
    # "expert" = multiply by (1 + expert id / 8) in bf16
    y = torch.zeros_like(expert_x)
    yc = torch.zeros((T * k, H), dtype=torch.bfloat16)
    for e in range(E):
        yc[rex[e]:rex[e + 1]] = (xe[rex[e]:rex[e + 1]].float() * (1 + e / 8)).to(torch.bfloat16)
    y.copy_(yc)
    out = torch.empty((T, H), dtype=torch.bfloat16, device=cuda)
    a2a.combine(out, torch.from_numpy(w).to(cuda), y, T)
    want = oracle.fastep_reduce(_bits(y), _bits(x), w, rmap)
    assert np.array_equal(_bits(out), want)


def test_executor_classes(cuda, oracle):
    from eps_b200._lib import EpsError
    from eps_b200.executor import AokGroupedGemm, silu

    rng = np.random.default_rng(0)
    rows = [70, 0, 130]
    E, N, K = 3, 256, 256
    excl = np.concatenate([[0], np.cumsum(rows)]).astype(np.int32)
    a = oracle.bf16_bits(rng.standard_normal((excl[-1], K)).astype(np.float32))
    A, a_s = oracle.quant_1x128(a)
    wq, w_s = oracle.quant_block128(oracle.bf16_to_f32(oracle.bf16_bits((rng.standard_normal((E, N, K)) * 0.02).astype(np.float32))))
    dv = lambda t: torch.from_numpy(np.ascontiguousarray(t)).to(cuda)
    gemm = AokGroupedGemm(E)
    assert gemm.get_workspace_size(K, excl[-1]) == 0
    C = gemm.run(dv(A), dv(wq), dv(w_s), dv(excl), int(excl[-1]), A_scale=dv(a_s))
    want = oracle.grouped_gemm_fp8(A, a_s, wq, w_s, excl)
    rms = np.sqrt(np.mean(want ** 2))
    assert np.max(np.abs(C.float().cpu().numpy() - want)) <= 2e-2 * rms
    # without B_scale the reference's bf16 x bf16 GEMM runs: e4m3 codes are the wrong operands for it
    with pytest.raises(EpsError, match="must have dtype torch.bfloat16"):
        gemm.run(dv(A), dv(wq), None, dv(excl), 0)
    Ab = torch.from_numpy(oracle.bf16_to_f32(a)).to(torch.bfloat16).to(cuda)
    Bb = (torch.randn((E, N, K), generator=torch.Generator().manual_seed(1)) * 0.05).to(torch.bfloat16).to(cuda)
    Cb = gemm.run(Ab, Bb, None, dv(excl), int(excl[-1]))
    for e in range(E):
        lo, hi = int(excl[e]), int(excl[e + 1])
        want_b = Ab[lo:hi].float() @ Bb[e].float().t()
        assert torch.all((Cb[lo:hi].float() - want_b).abs() <= 2.0 ** -8 * want_b.abs() + 1e-3)
    gu = C  # [rows, 256] bf16 -> act [rows, 128]
    act = silu(gu, dv(excl), int(excl[-1]))
    g, u = gu[:, :128].float(), gu[:, 128:].float()
    ref = (g / (1 + torch.exp(-g))) * u
    assert bool(((act.float() - ref).abs() <= ref.abs() * 2.0 ** -7 + 1e-30).all())
