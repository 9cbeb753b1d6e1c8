"""`AokGroupedGemm` (reference python/eps/executor/aok_grouped_gemm.py:10-58): `run(A, B, None, exclusive_sum, hint)` is
the bf16 grouped GEMM; a `B_scale` (with `A_scale`) selects the FP8 block-scaled one."""
from typing import Optional

import torch

from .ops import _ops

SM_COUNT: Optional[int] = None


class AokGroupedGemm:
    def __init__(self, num_local_experts: int) -> None:
        global SM_COUNT
        if SM_COUNT is None:
            SM_COUNT = torch.cuda.get_device_properties(torch.cuda.current_device()).multi_processor_count
        self._ptr = _ops.aok_create(num_local_experts, SM_COUNT)
        assert self._ptr != 0

    def __del__(self) -> None:
        self.destroy()

    def get_workspace_size(self, cols, max_num_tokens):
        return _ops.aok_get_workspace_size(self._ptr, cols, max_num_tokens)

    def run(self, A: torch.Tensor, B: torch.Tensor, B_scale: torch.Tensor, exclusive_sum: torch.Tensor,
            num_tokens_hint: int, A_scale: Optional[torch.Tensor] = None) -> torch.Tensor:
        assert self._ptr is not None
        max_num_tokens, K = A.shape
        ws = torch.empty((1, self.get_workspace_size(K, max_num_tokens) * 2), dtype=torch.uint8, device=A.device)
        C = torch.empty((max_num_tokens, B.shape[1]), dtype=torch.bfloat16, device=A.device)
        if B_scale is None:
            _ops.aok_run(self._ptr, A, B, C, exclusive_sum, num_tokens_hint, max_num_tokens, ws)
        else:
            assert A_scale is not None, "the FP8 grouped GEMM needs A_scale next to B_scale"
            _ops.aok_run_fp8(self._ptr, A, A_scale, B, B_scale, C, exclusive_sum, num_tokens_hint, max_num_tokens, ws)
        return C

    def run_gate_up_swiglu(self, A, A_scale, B, B_scale, exclusive_sum, out=None, out_scales=None, status=None):
        """gate/up GEMM + SwiGLU + 1x128 requantisation -> (e4m3 codes [rows, I], fp32 scales [rows, I/128])."""
        rows, inter = A.shape[0], B.shape[1] // 2
        C = out if out is not None else torch.empty((rows, inter), dtype=torch.uint8, device=A.device)
        Cs = out_scales if out_scales is not None else torch.empty((rows, inter // 128), dtype=torch.float32, device=A.device)
        _ops.aok_run_gate_up_fp8(self._ptr, A, A_scale, B, B_scale, C, Cs, exclusive_sum, rows, status)
        return C, Cs

    def run_down_weighted(self, A, A_scale, B, B_scale, exclusive_sum, row_weights=None, out=None, status=None):
        """down GEMM whose rows leave multiplied by their gate weight (fp32) -> bf16 [rows, N]."""
        rows = A.shape[0]
        C = out if out is not None else torch.empty((rows, B.shape[1]), dtype=torch.bfloat16, device=A.device)
        _ops.aok_run_down_fp8(self._ptr, A, A_scale, B, B_scale, C, row_weights, exclusive_sum, rows, status)
        return C

    def destroy(self) -> None:
        if getattr(self, "_ptr", None) is not None:
            _ops.aok_destroy(self._ptr)
            self._ptr = None
