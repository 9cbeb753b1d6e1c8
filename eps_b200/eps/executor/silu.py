import torch

from .ops import _ops


def silu(gate_up: torch.Tensor, exclusive_sum: torch.Tensor, num_tokens_hint):
    """act = silu(gate) * up over rows [exclusive_sum[0], exclusive_sum[-1]) (reference python/eps/executor/silu.py)."""
    assert gate_up.dtype == torch.bfloat16
    result = torch.empty((gate_up.shape[0], gate_up.shape[1] // 2), dtype=gate_up.dtype, device=gate_up.device)
    _ops.silu_run(gate_up, result, exclusive_sum, num_tokens_hint)
    return result


def per_token_group_quant_fp8(x: torch.Tensor, div_mode: int = 1):
    """x [rows, cols] bf16 -> (e4m3 codes uint8, fp32 scales [rows, cols/128])."""
    q = torch.empty(x.shape, dtype=torch.uint8, device=x.device)
    s = torch.empty((x.shape[0], x.shape[1] // 128), dtype=torch.float32, device=x.device)
    _ops.per_token_group_quant_fp8(x, q, s, div_mode)
    return q, s
