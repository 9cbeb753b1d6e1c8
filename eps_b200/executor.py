"""Executors: the host-side mirror of python/eps/executor (AokGroupedGemm, silu).

The reference's `AokGroupedGemm.run(A, B, B_scale, exclusive_sum, num_tokens_hint)` asserts `B_scale is None`
(bf16 x bf16 on sm_90a).  Here `B_scale is None` runs the bf16 tcgen05 grouped GEMM, and a `B_scale` selects the FP8
block-scaled one (A as e4m3 codes + `A_scale`).
"""
from __future__ import annotations

import torch

from . import ops
from ._lib import EpsError


class AokGroupedGemm:
    def __init__(self, num_local_experts: int) -> None:
        self.num_local_experts = num_local_experts
        self.status = None

    def destroy(self) -> None:
        """The reference frees its C++ object here; this object owns only tensors."""

    def get_workspace_size(self, cols, max_num_tokens) -> int:
        return 0  # the tile list is built inside the kernel; no workspace (reference: aok_get_workspace_size)

    def run(self, A: torch.Tensor, B: torch.Tensor, B_scale: torch.Tensor, exclusive_sum: torch.Tensor,
            num_tokens_hint: int, A_scale: torch.Tensor | None = None) -> torch.Tensor:
        """C[rows of expert e] = A[rows] @ B[e]^T -> bf16 [max_num_tokens, N]; bf16 operands when B_scale is None,
        e4m3 codes with 1x128 / 128x128 scales otherwise."""
        if B.shape[0] != self.num_local_experts:
            raise EpsError(f"B holds {B.shape[0]} experts, executor was created for {self.num_local_experts}")
        if self.status is None or self.status.device != A.device:
            self.status = torch.zeros(4, dtype=torch.int32, device=A.device)
        if B_scale is None:
            return ops.grouped_gemm_bf16(A, B, exclusive_sum, status=self.status, rows_hint=int(num_tokens_hint or 0))
        if A_scale is None:
            raise EpsError("the FP8 grouped GEMM needs A_scale next to B_scale")
        return ops.grouped_gemm_fp8(ops.GEMM_PLAIN, A, A_scale, B, B_scale, exclusive_sum, status=self.status)

    def run_gate_up_swiglu(self, A, A_scale, B, B_scale, exclusive_sum):
        """Fused gate/up GEMM + SwiGLU + 1x128 requantisation -> (e4m3 [rows, I], scales [rows, I/128])."""
        if self.status is None or self.status.device != A.device:
            self.status = torch.zeros(4, dtype=torch.int32, device=A.device)
        return ops.grouped_gemm_fp8(ops.GEMM_GATEUP, A, A_scale, B, B_scale, exclusive_sum, status=self.status)

    def run_down_weighted(self, A, A_scale, B, B_scale, exclusive_sum, row_weights=None):
        """Down GEMM whose epilogue multiplies every row by its gate weight (fp32) -> bf16 [rows, H]."""
        if self.status is None or self.status.device != A.device:
            self.status = torch.zeros(4, dtype=torch.int32, device=A.device)
        return ops.grouped_gemm_fp8(ops.GEMM_DOWN, A, A_scale, B, B_scale, exclusive_sum, row_w=row_weights,
                                    status=self.status)


def silu(gate_up: torch.Tensor, exclusive_sum: torch.Tensor, num_tokens_hint):
    """act = silu(gate) * up over rows [exclusive_sum[0], exclusive_sum[-1]) (python/eps/executor/silu.py:5-11)."""
    assert gate_up.dtype == torch.bfloat16
    result = torch.empty((gate_up.shape[0], gate_up.shape[1] // 2), dtype=gate_up.dtype, device=gate_up.device)
    ops.silu_run(gate_up, result, exclusive_sum, exclusive_sum.numel() - 1)
    return result
