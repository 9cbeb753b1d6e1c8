"""Router (group-limited top-k over sigmoid scores) against the CPU oracle and, for the one shape the reference
instantiates (256 experts, 8 groups, top-8), bit-exact against the reference's own kernel on the GPU."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

CASES = [
    # T, E, groups, topk_groups, k, zero experts (mapped to negative ids), route_scale, bias
    (64, 256, 8, 4, 8, 0, 2.5, True),        # DeepSeek-V3 routing, the reference's instantiation
    (300, 256, 8, 4, 8, 0, 1.0, False),
    (17, 32, 1, 1, 4, 0, 1.0, True),         # no groups
    (128, 768, 8, 8, 12, 256, 1.0, True),    # 512 FFN + 256 identity experts, every group stays
    (50, 96, 3, 2, 5, 0, 1.0, True),         # groups that do not align with lanes (3 experts per lane, 32 per group)
    (33, 1024, 32, 5, 32, 0, 1.0, True),     # the limits: 1024 experts, 32 groups, top-32
    (1, 64, 2, 1, 1, 0, 1.0, False),
]


def _check_against_oracle(got_idx, got_w, oracle, scores, bias, g, tg, k, scale, nf):
    idx, w, biased = oracle.topk_sigmoid(scores, bias, g, tg, k, scale, nf)
    E = scores.shape[1]
    unmap = lambda a: np.where(a < 0, nf + (-1 - a), a)
    gi, oi = unmap(got_idx), unmap(idx)
    # expf on the device and exp in numpy may differ in the last place: an index may differ only where the two
    # candidates' biased scores are (nearly) equal
    diff = gi != oi
    if diff.any():
        rows = np.nonzero(diff)[0]
        a = biased[rows, gi[diff]]
        b = biased[rows, oi[diff]]
        assert np.all(np.abs(a - b) <= 4 * np.finfo(np.float32).eps * np.abs(b)), "selection differs beyond a tie"
        # the same SET must still be chosen unless the tie sits at the cut
    same = ~diff.any(axis=1)
    assert same.mean() > 0.99
    assert np.allclose(got_w[same], w[same], rtol=2e-6, atol=1e-9)
    assert np.allclose(got_w.sum(1), scale, rtol=1e-5)
    assert (got_idx < nf).all() and (got_idx >= -(E - nf)).all()


@pytest.mark.parametrize("T,E,g,tg,k,nz,scale,with_bias", CASES)
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_router_vs_oracle(cuda, oracle, T, E, g, tg, k, nz, scale, with_bias, dtype):
    from eps_b200 import ops

    gen = torch.Generator().manual_seed(T * 7 + E)
    scores = torch.randn((T, E), generator=gen).to(dtype)
    bias = (torch.randn(E, generator=gen) * 0.1) if with_bias else None
    nf = E - nz
    idx, w = ops.topk_sigmoid(scores.to(cuda), None if bias is None else bias.to(cuda), g, tg, k, scale, nf)
    torch.cuda.synchronize()
    _check_against_oracle(idx.cpu().numpy(), w.cpu().numpy(), oracle, scores.float().numpy(),
                          None if bias is None else bias.numpy(), g, tg, k, scale, nf)
    # every chosen expert lies in one of at most `tg` groups, no expert twice
    sel = np.where(idx.cpu().numpy() < 0, nf + (-1 - idx.cpu().numpy()), idx.cpu().numpy())
    assert all(len(set(r)) == k for r in sel)
    assert all(len(set(r // (E // g))) <= tg for r in sel)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("T", [1, 77, 4096])
def test_router_bit_exact_against_reference_kernel(cuda, T, dtype):
    from eps_b200 import ops
    from oracle import ref_kernels

    if not ref_kernels.available():
        pytest.skip("reference witness library not built")
    gen = torch.Generator().manual_seed(T)
    scores = torch.randn((T, 256), generator=gen).to(dtype).to(cuda)
    bias = (torch.randn(256, generator=gen) * 0.1).to(cuda)
    ref = ref_kernels.topk_sigmoid(scores, bias, 8, 4, 8, 2.5)
    assert ref is not None
    idx, w = ops.topk_sigmoid(scores, bias, 8, 4, 8, 2.5)
    torch.cuda.synchronize()
    assert torch.equal(idx, ref[0])
    assert torch.equal(w, ref[1])
    # a shape the reference refuses ("Not supported num_experts: ...") runs here
    assert ref_kernels.topk_sigmoid(scores[:, :128].contiguous(), bias[:128].contiguous(), 8, 4, 8, 1.0) is None
    ops.topk_sigmoid(scores[:, :128].contiguous(), bias[:128].contiguous(), 8, 4, 8, 1.0)
    torch.cuda.synchronize()


def test_router_feeds_the_plans(cuda, oracle):
    """The router's output is what Scheduler.rendezvous_and_plan reads: run the source plans on it."""
    from eps_b200 import ops

    gen = torch.Generator().manual_seed(3)
    scores = torch.randn((200, 96), generator=gen).to(cuda)
    idx, w = ops.topk_sigmoid(scores, None, 3, 2, 4, 1.0, num_ffn_experts=64)   # ids 64..95 -> identity experts
    send_map, send_incl, glob_map, coll_incl, zero = ops.source_plans(idx, w, 64, 2, 1)
    torch.cuda.synchronize()
    rmap, rincl = oracle.comm_plan(idx.cpu().numpy(), 64, 2, 1)
    assert np.array_equal(send_incl.cpu().numpy(), rincl)
    assert np.array_equal(zero.cpu().numpy(), oracle.zero_plan(idx.cpu().numpy(), w.cpu().numpy()))


@pytest.mark.parametrize("T,E,k", [(128, 128, 8), (64, 256, 8), (40, 512, 12)])
def test_router_softmax_matches_torch_topk(cuda, oracle, T, E, k):
    """Softmax scores, no groups, no bias: the plain top-k softmax router (what eps_b200.workloads generates its
    routing with): indices == torch.topk, weights == softmax probabilities renormalised over the chosen experts."""
    from eps_b200 import ops

    gen = torch.Generator().manual_seed(E + k)
    logits = torch.randn((T, E), generator=gen)
    idx, w = ops.topk_sigmoid(logits.to(cuda), None, 1, 1, k, 1.0, score_func="softmax")
    torch.cuda.synchronize()
    top = torch.topk(logits, k, dim=1)
    probs = torch.softmax(logits, dim=1).gather(1, top.indices)
    want_w = probs / probs.sum(dim=1, keepdim=True)
    assert torch.equal(idx.cpu().long(), top.indices)
    assert torch.allclose(w.cpu(), want_w, rtol=1e-5, atol=1e-8)
    oi, ow, _ = oracle.topk_sigmoid(logits.numpy(), None, 1, 1, k, 1.0, score_func="softmax")
    assert np.array_equal(oi, idx.cpu().numpy()) and np.allclose(ow, w.cpu().numpy(), rtol=1e-5)
    # with groups and bias the oracle is the checker
    bias = torch.randn(E, generator=gen) * 0.01
    idx, w = ops.topk_sigmoid(logits.to(cuda), bias.to(cuda), 8, 4, k, 2.0, score_func="softmax")
    oi, ow, biased = oracle.topk_sigmoid(logits.numpy(), bias.numpy(), 8, 4, k, 2.0, score_func="softmax")
    same = (oi == idx.cpu().numpy()).all(axis=1)
    assert same.mean() > 0.95 and np.allclose(ow[same], w.cpu().numpy()[same], rtol=2e-5)


def test_layer_fed_by_the_router(cuda, oracle):
    """forward_routed == router + forward, and both match the fp32 oracle run on the oracle's own routing."""
    from eps_b200 import ops, workloads
    from eps_b200.layer import MoELayerFP8

    T, H, I, E, k, nz = 48, 512, 256, 32, 4, 32
    cfg = workloads.CONFIGS[0].scaled(tokens_per_rank=T, hidden=H, inter=I, num_experts=E, top_k=k)
    x = workloads.make_tokens(cfg)
    gu = torch.stack([workloads.make_expert_weights(cfg, e)[0] for e in range(E)])
    d = torch.stack([workloads.make_expert_weights(cfg, e)[1] for e in range(E)])
    gq, gs = ops.quant_block128(gu.to(cuda))
    dq, ds = ops.quant_block128(d.to(cuda))
    layer = MoELayerFP8(H, I, E, k, T, gq, gs, dq, ds)
    gen = torch.Generator().manual_seed(9)
    logits = torch.randn((T, E + nz), generator=gen)
    bias = torch.randn(E + nz, generator=gen) * 0.1
    out = layer.forward_routed(x.to(cuda), logits.to(cuda), bias.to(cuda), 4, 2, 1.5, num_zero_experts=nz)
    idx, w = ops.topk_sigmoid(logits.to(cuda), bias.to(cuda), 4, 2, k, 1.5, num_ffn_experts=E)
    out2 = layer.forward(x.to(cuda), idx, w)
    torch.cuda.synchronize()
    layer.check_status()
    assert torch.equal(out, out2)
    assert (idx < 0).any() and (idx >= 0).any()      # both identity and FFN experts are routed to
    want = oracle.moe_layer_fp32(x.view(torch.int16).numpy().view(np.uint16), idx.cpu().numpy(), w.cpu().numpy(),
                                 *oracle.quant_block128(gu.float().numpy()), *oracle.quant_block128(d.float().numpy()))
    got = out.float().cpu().numpy()
    rms = float(np.sqrt(np.mean(want ** 2)))
    assert np.all(np.abs(got - want) <= 2e-2 * rms + 2.0 ** -8 * np.abs(want))


def test_router_errors(cuda):
    from eps_b200 import ops
    from eps_b200._lib import EpsError

    s = torch.zeros((4, 100), device=cuda)
    with pytest.raises(EpsError):
        ops.topk_sigmoid(s, None, 4, 2, 2)            # 100 experts: not a multiple of 32
    s = torch.zeros((4, 64), device=cuda)
    with pytest.raises(EpsError):
        ops.topk_sigmoid(s, None, 3, 2, 2)            # 3 groups do not divide 64
    with pytest.raises(EpsError):
        ops.topk_sigmoid(s, None, 4, 1, 17)           # top-17 out of one group of 16
