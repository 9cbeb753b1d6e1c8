"""Seeded synthetic MoE-layer inputs with the shapes and value distributions of the five benchmark
configurations (no dataset or checkpoint is involved; everything is generated).

Tokens and routing are generated on the CPU with a counter-based torch.Generator so that a CPU
checker and the GPU path see identical bits; expert weights are generated per expert (seeded by
the expert id) on whatever device is asked for, so a rank can materialise only its own experts.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, replace

import torch

BASE_SEED = 20251125


@dataclass(frozen=True)
class MoEConfig:
    cfg_id: int
    name: str
    tokens_per_rank: int
    hidden: int
    inter: int
    num_experts: int          # routed FFN experts
    top_k: int
    num_zero_experts: int = 0  # identity ("zero-computation") experts appended after the FFN experts
    shared_inter: int = 0      # always-on shared expert (0 = none)
    bias: str = "none"         # "none" | "zipf" (s=1.2 over a seeded permutation) | "normal" (sigma 0.5)

    def scaled(self, **kw) -> "MoEConfig":
        return replace(self, **kw)


CONFIGS = {
    0: MoEConfig(0, "small", 256, 2048, 1408, 16, 4),
    1: MoEConfig(1, "dsv3-prefill", 4096, 7168, 2048, 256, 8, shared_inter=2048),
    2: MoEConfig(2, "dsv3-decode-zipf", 128, 7168, 2048, 256, 8, bias="zipf"),
    3: MoEConfig(3, "qwen3-235b-prefill", 8192, 4096, 1536, 128, 8),
    4: MoEConfig(4, "longcat-flash-zero-experts", 4096, 6144, 2048, 512, 12, num_zero_experts=256, bias="normal"),
}


def _gen(cfg: MoEConfig, stream: int) -> torch.Generator:
    g = torch.Generator(device="cpu")
    g.manual_seed((BASE_SEED + cfg.cfg_id) * 1000 + stream)
    return g


def expert_bias(cfg: MoEConfig) -> torch.Tensor:
    """Additive per-expert router bias (same on every rank)."""
    n = cfg.num_experts + cfg.num_zero_experts
    g = _gen(cfg, 999)
    if cfg.bias == "zipf":
        perm = torch.randperm(n, generator=g)
        b = torch.empty(n, dtype=torch.float32)
        b[perm] = -1.2 * torch.log(torch.arange(1, n + 1, dtype=torch.float32))
        return b
    if cfg.bias == "normal":
        return torch.randn(n, generator=g, dtype=torch.float32) * 0.5
    return torch.zeros(n, dtype=torch.float32)


def make_tokens(cfg: MoEConfig, rank: int = 0, tokens: int | None = None) -> torch.Tensor:
    T = cfg.tokens_per_rank if tokens is None else tokens
    return torch.randn((T, cfg.hidden), generator=_gen(cfg, 2 * rank), dtype=torch.float32).to(torch.bfloat16)


def make_routing(cfg: MoEConfig, rank: int = 0, tokens: int | None = None):
    """-> (indices int32 [T,k], weights fp32 [T,k]).  Top-k is taken on logits+bias (ties are
    measure-zero); weights are the softmax over all logits gathered at the top-k and renormalised
    to sum 1.  Ids >= num_experts become negative (-1 - zero_expert_id), the reference's
    convention for zero-computation experts."""
    T = cfg.tokens_per_rank if tokens is None else tokens
    n = cfg.num_experts + cfg.num_zero_experts
    logits = torch.randn((T, n), generator=_gen(cfg, 2 * rank + 1), dtype=torch.float32) + expert_bias(cfg)
    top = torch.topk(logits, cfg.top_k, dim=1)
    probs = torch.softmax(logits, dim=1).gather(1, top.indices)
    weights = (probs / probs.sum(dim=1, keepdim=True)).to(torch.float32)
    idx = top.indices.to(torch.int32)
    idx = torch.where(idx >= cfg.num_experts, -(idx - cfg.num_experts) - 1, idx)
    return idx.contiguous(), weights.contiguous()


def make_expert_weights(cfg: MoEConfig, expert: int, device="cpu", inter: int | None = None):
    """bf16 (W_gate_up [2I, H] with gate first, W_down [H, I]) ~ N(0, 0.02) of one expert.
    expert == -1 is the shared expert."""
    I = cfg.inter if inter is None else inter
    g = torch.Generator(device=device)
    g.manual_seed((BASE_SEED + cfg.cfg_id) * 1000003 + 7 * (expert + 2))
    wgu = (torch.randn((2 * I, cfg.hidden), generator=g, device=device, dtype=torch.float32) * 0.02).to(torch.bfloat16)
    wd = (torch.randn((cfg.hidden, I), generator=g, device=device, dtype=torch.float32) * 0.02).to(torch.bfloat16)
    return wgu, wd


def layer_flops(cfg: MoEConfig, routed_pairs: int, tokens: int) -> float:
    """6*rows*H*I for the routed pairs plus the shared expert."""
    return 6.0 * routed_pairs * cfg.hidden * cfg.inter + 6.0 * tokens * cfg.hidden * cfg.shared_inter


def describe(cfg: MoEConfig, world: int) -> str:
    return (f"cfg{cfg.cfg_id}:{cfg.name} T/rank={cfg.tokens_per_rank} H={cfg.hidden} I={cfg.inter} "
            f"E={cfg.num_experts}+{cfg.num_zero_experts}z top{cfg.top_k} shared_I={cfg.shared_inter} EP{world}")
