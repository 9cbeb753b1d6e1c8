"""`Scheduler`: the staged EPS driver with the reference's constructor and methods
(reference python/eps/scheduler/scheduler.py:19-122), over the ops of libscheduler_.so.

The reference's calls work unchanged (bf16 rows, reference arithmetic).  The keyword arguments and the `*_fp8` /
`*_weighted` / `*_fused` methods are additions for the FP8 path: e4m3 hidden rows with 1x128 scales, GEMM rows that
leave the down GEMM already multiplied by their gate weight, fp32 accumulation in the reductions."""
import torch

from .ops import _ops


class ContextWrapper:
    """Owns the context handle and the workspace tensor its plan buffers live in."""

    def __init__(self, context):
        self._context = context
        ws_size = _ops.eps_get_workspace_size_context(context)
        self.ws = torch.empty((1, ws_size), dtype=torch.uint8, device="cuda")
        _ops.eps_set_ws_context(context, self.ws)

    def __del__(self) -> None:
        _ops.eps_destroy_context(self._context)


class Scheduler:
    def __init__(self, top_k: int, num_experts: int, hidden_size: int, input_scales_dim: int,
                 max_num_tokens_per_gpu: int, comm, local_num_experts: int, fp8_hidden: bool = False) -> None:
        comm_ptr = int(comm) if comm is not None else 0
        create = _ops.eps_create_fp8 if fp8_hidden else _ops.eps_create
        # as in the reference, local_num_experts is what the C++ side receives as max_num_stages
        self._ptr = create(top_k, num_experts, hidden_size, input_scales_dim, max_num_tokens_per_gpu, comm_ptr,
                           local_num_experts)
        assert self._ptr != 0
        self.local_num_experts = local_num_experts
        self.context = None

    def __del__(self) -> None:
        self.destroy()

    def get_context(self, num_tokens, num_global_tokens, num_stages, input_quanted):
        return ContextWrapper(_ops.eps_get_context(self._ptr, num_tokens, num_global_tokens, num_stages, input_quanted))

    def rendezvous_and_plan(self, expert_indices: torch.Tensor, expert_scales: torch.Tensor, num_global_tokens,
                            num_stages, input_quanted, host_sync: bool = True, max_cluster: int = 0, payload=None):
        """-> (exclusive_sum [local_num_experts + 1] int32 on the device, rows this rank will receive).
        host_sync=False: the count is not read on the host and an upper bound is returned instead."""
        num_tokens = expert_indices.shape[0]
        self.context = self.get_context(num_tokens, num_global_tokens, num_stages, input_quanted)
        if host_sync:
            n_recv = _ops.eps_rendezvous(self._ptr, expert_indices, self.context._context)
        else:
            n_recv = _ops.eps_rendezvous_async(self._ptr, expert_indices, self.context._context, max_cluster)
        exclusive_sum = torch.empty((self.local_num_experts + 1,), dtype=torch.int32, device=expert_indices.device)
        if payload is None and max_cluster == 0:
            _ops.eps_plan(self._ptr, expert_indices, expert_scales, exclusive_sum, self.context._context)
        else:
            hidden, scales = payload if payload is not None else (None, None)
            _ops.eps_plan_fp8(self._ptr, expert_indices, expert_scales, exclusive_sum, self.context._context, hidden,
                              scales, max_cluster)
        return exclusive_sum, n_recv

    def prologue(self, expert_scales: torch.Tensor, hidden_states: torch.Tensor, input_scales=None,
                 recv_input_scales=None, raw_input=None) -> None:
        assert self._ptr is not None
        if raw_input is not None:
            _ops.eps_prologue_fp8(self._ptr, expert_scales, hidden_states, input_scales, recv_input_scales, raw_input,
                                  self.context._context)
        else:
            _ops.eps_prologue(self._ptr, expert_scales, hidden_states, input_scales, recv_input_scales,
                              self.context._context)

    def dispatch(self, stage_idx: int) -> None:
        assert self._ptr is not None
        _ops.eps_dispatch(self._ptr, self.context._context, stage_idx)

    def gemm_expand(self, gemm_input: torch.Tensor, stage_idx: int):
        _ops.eps_gemm_expand(self._ptr, gemm_input, self.context._context, stage_idx)

    def local_reduce(self, gemm_output: torch.Tensor, stage_idx: int, pre_weighted: bool = False):
        if pre_weighted:
            _ops.eps_local_reduce_weighted(self._ptr, gemm_output, self.context._context, stage_idx)
        else:
            _ops.eps_local_reduce(self._ptr, gemm_output, self.context._context, stage_idx)

    def combine(self, stage_idx: int) -> None:
        assert self._ptr is not None
        _ops.eps_combine(self._ptr, self.context._context, stage_idx)

    def epilogue(self, output: torch.Tensor, shared=None, ref_arith: bool = True) -> None:
        assert self._ptr is not None
        if ref_arith and shared is None:
            _ops.eps_epilogue(self._ptr, output, self.context._context)
        else:
            _ops.eps_epilogue_fused(self._ptr, output, shared, self.context._context)

    # ---- additions for the FP8 path

    def gemm_row_weights(self) -> torch.Tensor:
        """fp32 gate weight of every GEMM row (a view into the context's workspace)."""
        return _ops.eps_gemm_row_weights(self._ptr, self.context._context)

    def reduce_single_rank(self, gemm_output: torch.Tensor, output: torch.Tensor, shared=None) -> None:
        _ops.eps_reduce_single_rank(self._ptr, gemm_output, output, shared, self.context._context)

    def check_status(self) -> None:
        _ops.eps_check_status(self._ptr, self.context._context)

    def destroy(self) -> None:
        if getattr(self, "_ptr", None) is not None:
            self.context = None
            _ops.eps_destroy(self._ptr)
            self._ptr = None
