"""The sampled form of the layer oracle equals the whole-layer oracle on the sampled rows (CPU only)."""
import numpy as np
import torch


def test_sampled_layer_oracle_equals_full(oracle):
    from eps_b200 import workloads
    from oracle import layer_check

    cfg = workloads.CONFIGS[0].scaled(tokens_per_rank=40, hidden=256, inter=128, num_experts=6, top_k=3,
                                      num_zero_experts=2, shared_inter=128, bias="normal")
    x = workloads.make_tokens(cfg)
    idx, w = workloads.make_routing(cfg)

    def codes(e, inter=None):
        a, b = workloads.make_expert_weights(cfg, e, inter=inter)
        return oracle.quant_block128(a.float().numpy()) + oracle.quant_block128(b.float().numpy())

    ws = [codes(e) for e in range(6)]
    full = tuple(np.stack([ws[e][i] for e in range(6)]) for i in range(4))
    sh = tuple(t[None] for t in codes(-1, 128))
    xb = x.view(torch.int16).numpy().view(np.uint16)
    want = oracle.moe_layer_fp32(xb, idx.numpy(), w.numpy(), *full, shared=sh)
    s = layer_check.sample_tokens(40, 16, 3)
    asked = []

    def expert_weights(e):
        asked.append(e)
        return ws[e]

    got = oracle.moe_layer_fp32_sampled(xb[s], idx.numpy()[s], w.numpy()[s], expert_weights, shared=sh)
    assert np.array_equal(got, want[s])
    assert sorted(asked) == sorted(set(int(e) for e in idx.numpy()[s].ravel() if e >= 0))   # each expert once
    res = layer_check.check_rows(xb[s], idx.numpy()[s], w.numpy()[s], want[s] * 1.5, expert_weights, shared=sh)
    assert not res["ok"] and res["worst_ratio"] > 1.0
    assert oracle.set_num_threads(2) == 2
    oracle.set_num_threads(8)


def test_bf16_stores_alone_exceed_the_plain_tolerance_on_decode_routing(oracle):
    """The decode configuration at EP8 with EXACT fp32 arithmetic, rounded to bf16 only where the path stores bf16 (the
    down GEMM's weighted row, the rank's partial row on the link, the output): the format alone puts the worst element
    beyond 2e-2 x RMS (its elements reach 6 x RMS, and half an ulp of bf16 there is 1.2e-2 x RMS per store), and stays
    inside the bound that adds half an ulp per store.  This is why layer_check reports both ratios."""
    from eps_b200 import workloads
    from oracle import layer_check

    cfg, W = workloads.CONFIGS[2], 8
    x = workloads.make_tokens(cfg, 0)
    idx, w = workloads.make_routing(cfg, 0)
    s = layer_check.sample_tokens(x.shape[0], 16, seed=1)
    xb = x.view(torch.int16).numpy().view(np.uint16)[s]
    idx, w = idx.numpy()[s], w.numpy()[s]

    def bf(a):
        return oracle.bf16_to_f32(oracle.bf16_bits(a.astype(np.float32)))

    def codes(e, inter=None):
        a, b = workloads.make_expert_weights(cfg, e, inter=inter)
        return oracle.quant_block128(a.float().numpy()) + oracle.quant_block128(b.float().numpy())

    shared = tuple(t[None] for t in codes(-1, cfg.shared_inter)) if cfg.shared_inter else None
    want, mag = oracle.moe_layer_fp32_sampled(xb, idx, w, codes, shared=shared, return_magnitude=True)
    # the same sum with the path's three stores: per-expert rows, per-rank partials, output
    EL = cfg.num_experts // W
    n, H = want.shape
    part = np.zeros((W, n, H), dtype=np.float32)
    for e in np.unique(idx[idx >= 0]):
        tt, jj = np.nonzero(idx == e)
        row, _ = oracle.moe_layer_fp32_sampled(xb[tt], np.full((len(tt), 1), e, dtype=np.int32), w[tt, jj][:, None],
                                               codes, return_magnitude=True)
        np.add.at(part[e // EL], tt, bf(row))
    got = sum(bf(part[r]) for r in range(W))
    if shared is not None:
        only_shared, _ = oracle.moe_layer_fp32_sampled(xb, np.full((n, 1), -1, dtype=np.int32),
                                                       np.zeros((n, 1), dtype=np.float32), codes, shared=shared,
                                                       return_magnitude=True)
        got = got + bf(only_shared)
    got = bf(got)
    rms = float(np.sqrt(np.mean(want.astype(np.float64) ** 2)))
    err = np.abs(got - want)
    strict = float(err.max() / (2e-2 * rms))
    per_store = float(np.max(err / (2e-2 * rms + 3 * 2.0 ** -9 * mag)))
    assert strict > 1.0, strict
    assert per_store <= 1.0, per_store
