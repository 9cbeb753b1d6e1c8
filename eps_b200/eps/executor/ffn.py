"""FP8 FFN executors behind the contract types the reference declares without an implementation
(src/scheduler/gemm_executor_interface.cuh:50-151: GemmExecutorInterface, SharedExpertsInterface, DenseGemmInterface,
BatchedGemmInterface, DenseActivationInterface).  Weights are e4m3 codes with one fp32 scale per 128 x 128 block:
gate_up [E, 2I, H] (gate rows first), down [E, H, I]."""
from typing import Optional

import torch

from .ops import _ops


class _Ffn:
    def __init__(self, ptr: int) -> None:
        self._ptr = ptr
        self._ws = None

    def _workspace(self, nbytes: int, device) -> torch.Tensor:
        if self._ws is None or self._ws.numel() < nbytes or self._ws.device != device:
            self._ws = torch.empty((max(nbytes, 256),), dtype=torch.uint8, device=device)
        return self._ws

    def status(self) -> torch.Tensor:
        """int32[4] on the device; word 0 is non-zero after a bounded wait inside a kernel gave up."""
        return _ops.ffn_status(self._ptr)

    def destroy(self) -> None:
        if getattr(self, "_ptr", None) is not None:
            _ops.ffn_destroy(self._ptr)
            self._ptr = None

    def __del__(self) -> None:
        self.destroy()


class GemmExecutor(_Ffn):
    """The routed experts of a rank: run(stage) computes gate/up + SwiGLU + requantisation + down for the experts of
    that stage on rows already in expert order (`exclusive_sum` [E+1] int32 on the device)."""

    def __init__(self, gate_up, gate_up_scales, down, down_scales, sm_count: int = 0) -> None:
        super().__init__(_ops.gemm_executor_create(gate_up, gate_up_scales, down, down_scales, sm_count))

    def get_workspace_size(self, max_num_tokens: int) -> int:
        return _ops.gemm_executor_get_workspace_size(self._ptr, max_num_tokens)

    def run(self, input, input_scales, exclusive_sum, num_stages: int = 1, stage_idx: int = 0,
            num_tokens_hint: int = 0, row_weights: Optional[torch.Tensor] = None, out=None) -> torch.Tensor:
        rows = input.shape[0]
        if out is None:
            out = torch.empty((rows, input.shape[1]), dtype=torch.bfloat16, device=input.device)
        ws = self._workspace(self.get_workspace_size(rows), input.device)
        _ops.gemm_executor_run(self._ptr, input, input_scales, out, exclusive_sum, num_stages, stage_idx,
                               num_tokens_hint, rows, row_weights, ws)
        return out


class SharedExperts(_Ffn):
    """The shared expert: the same FFN on every token of the rank."""

    def __init__(self, gate_up, gate_up_scales, down, down_scales, sm_count: int = 0) -> None:
        super().__init__(_ops.shared_experts_create(gate_up, gate_up_scales, down, down_scales, sm_count))

    def get_workspace_size(self, num_tokens: int) -> int:
        return _ops.shared_experts_get_workspace_size(self._ptr, num_tokens)

    def run(self, input, input_scales, out=None) -> torch.Tensor:
        rows = input.shape[0]
        if out is None:
            out = torch.empty((rows, input.shape[1]), dtype=torch.bfloat16, device=input.device)
        ws = self._workspace(self.get_workspace_size(rows), input.device)
        _ops.shared_experts_run(self._ptr, input, input_scales, out, rows, ws)
        return out


def dense_gemm_fp8(A, A_scale, B, B_scale, sm_count: int = 0) -> torch.Tensor:
    """C [M, N] bf16 = A [M, K] * B [N, K]^T on e4m3 codes, scales [M, K/128] and [N/128, K/128]."""
    C = torch.empty((A.shape[0], B.shape[0]), dtype=torch.bfloat16, device=A.device)
    _ops.dense_gemm_fp8(A, A_scale, B, B_scale, C, sm_count)
    return C


def batched_gemm_fp8(A, A_scale, B, B_scale, sm_count: int = 0) -> torch.Tensor:
    """C [G, M, N] bf16 = A [G, M, K] * B [G, N, K]^T per g, scales [G, M, K/128] and [G, N/128, K/128]."""
    C = torch.empty((A.shape[0], A.shape[1], B.shape[1]), dtype=torch.bfloat16, device=A.device)
    _ops.batched_gemm_fp8(A, A_scale, B, B_scale, C, sm_count)
    return C


def dense_silu(gate_up: torch.Tensor) -> torch.Tensor:
    """silu(gate) * up on dense rows: [rows, 2I] bf16 -> [rows, I] bf16."""
    out = torch.empty((gate_up.shape[0], gate_up.shape[1] // 2), dtype=torch.bfloat16, device=gate_up.device)
    _ops.dense_silu_run(gate_up, out)
    return out
