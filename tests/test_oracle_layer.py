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
