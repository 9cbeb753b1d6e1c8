"""Tensor-level operators over the C ABI (include/eps_b200.h).

Each function checks its tensors the way the reference's bindings do
(device / contiguity / dtype, reference src/common/torch_utils.h:39-44), passes
raw pointers to libeps_b200.so and launches on the current CUDA stream
(reference bindings use at::cuda::getCurrentCUDAStream()).  torch is used for
device memory and streams only.
"""
from __future__ import annotations

import torch

from ._lib import EpsError, call, ptr, stream_ptr

GEMM_PLAIN, GEMM_GATEUP, GEMM_DOWN = 0, 1, 2
ZC_MARK = 1000000
PLAN_ROWS_EXCEEDED = 51
INT32_MAX = 2**31 - 1


def _check(t: torch.Tensor, name: str, dtype=None, dim=None):
    if not t.is_cuda:
        raise EpsError(f"{name} must be a CUDA tensor")
    if not t.is_contiguous():
        raise EpsError(f"{name} must be contiguous")
    if dtype is not None and t.dtype not in (dtype if isinstance(dtype, tuple) else (dtype,)):
        raise EpsError(f"{name} must have dtype {dtype}, got {t.dtype}")
    if dim is not None and t.dim() != dim:
        raise EpsError(f"{name} must have {dim} dimensions, got {t.dim()}")


_FP8 = (torch.uint8, torch.float8_e4m3fn)

# ------------------------------------------------------------------ quantisation


def per_token_group_quant_fp8(x, exclusive_sum=None, num_experts=0, div_mode=1, out=None, out_scales=None):
    """x [rows, cols] bf16 -> (codes uint8 [rows, cols], scales fp32 [rows, cols/128]).

    div_mode 1 (default) computes the scale exactly like the reference kernel (div.full.f32, which on
    B200 equals amax * fl(1/448)); div_mode 0 uses the IEEE quotient amax/448.
    With `exclusive_sum` only rows [exclusive_sum[0], exclusive_sum[num_experts]) are written
    (reference PerTokenGroupQuantFP8Params, src/quant/fp8.cuh:43-57)."""
    _check(x, "x", torch.bfloat16, 2)
    rows, cols = x.shape
    q = out if out is not None else torch.empty((rows, cols), dtype=torch.uint8, device=x.device)
    s = out_scales if out_scales is not None else torch.empty((rows, cols // 128), dtype=torch.float32, device=x.device)
    if exclusive_sum is None:
        call("epsb_quant_1x128", ptr(x), rows, cols, ptr(q), ptr(s), div_mode, stream_ptr())
    else:
        _check(exclusive_sum, "exclusive_sum", torch.int32, 1)
        call("epsb_quant_1x128_ragged", ptr(x), ptr(exclusive_sum), num_experts, cols, ptr(q), ptr(s), rows,
             div_mode, stream_ptr())
    return q, s


def per_token_group_dequant_fp8(q, scales):
    _check(q, "q", _FP8, 2)
    _check(scales, "scales", torch.float32, 2)
    rows, cols = q.shape
    x = torch.empty((rows, cols), dtype=torch.bfloat16, device=q.device)
    call("epsb_dequant_1x128", ptr(q), ptr(scales), rows, cols, ptr(x), stream_ptr())
    return x


def quant_block128(w):
    """w [n_mats, n, k] (or [n, k]) bf16 -> (codes uint8, scales fp32 [n_mats, ceil(n/128), ceil(k/128)])."""
    _check(w, "w", torch.bfloat16)
    squeeze = w.dim() == 2
    w3 = w.unsqueeze(0) if squeeze else w
    m, n, k = w3.shape
    q = torch.empty((m, n, k), dtype=torch.uint8, device=w.device)
    s = torch.empty((m, (n + 127) // 128, (k + 127) // 128), dtype=torch.float32, device=w.device)
    call("epsb_quant_block128", ptr(w3), m, n, k, ptr(q), ptr(s), stream_ptr())
    return (q[0], s[0]) if squeeze else (q, s)


# ------------------------------------------------------------------ plans


def source_plans(idx, weights, E, W, S, want_global=True, want_zero=True, with_bounds=False, max_cluster=0):
    """Source-side plans.  with_bounds=True also returns send_bounds = [0, send_incl...] (one buffer, so the
    gathers can read their [begin, end) window from the device)."""
    _check(idx, "expert_indices", torch.int32, 2)
    T, k = idx.shape
    dev = idx.device
    send_map = torch.empty((max(T * W, 1),), dtype=torch.int32, device=dev)
    send_bounds = torch.zeros((W * S + 1,), dtype=torch.int32, device=dev)
    send_incl = send_bounds[1:]
    glob_map = torch.empty((max(T * W, 1),), dtype=torch.int32, device=dev) if want_global else None
    coll_incl = torch.empty((W * S,), dtype=torch.int32, device=dev) if want_global else None
    zero_scale = None
    if want_zero and weights is not None:
        _check(weights, "expert_scales", torch.float32, 2)
        zero_scale = torch.empty((max(T, 1),), dtype=torch.float32, device=dev)
    call("epsb_source_plans", ptr(idx), ptr(weights), T, k, E, W, S, ptr(send_map), ptr(send_incl), ptr(glob_map),
         ptr(coll_incl), ptr(zero_scale), int(max_cluster), stream_ptr())
    if with_bounds:
        return send_map, send_incl, glob_map, coll_incl, zero_scale, send_bounds
    return send_map, send_incl, glob_map, coll_incl, zero_scale


def recv_plan(gathered, my_rank, W, S, total_rows=None):
    _check(gathered, "gathered_send_plan", torch.int32)
    dev = gathered.device
    recv_incl = torch.empty((W * S,), dtype=torch.int32, device=dev)
    remote_offset = torch.empty((W * S,), dtype=torch.int32, device=dev)
    call("epsb_recv_plan", ptr(gathered), my_rank, W, S, ptr(recv_incl), ptr(remote_offset), ptr(total_rows),
         stream_ptr())
    return recv_incl, remote_offset


def expert_plans(ridx, recv_incl, k, lo, hi, W, S, max_tok_per_gpu, max_rows, want_reduce=True, status=None,
                 max_cluster=0):
    """status: optional int32[2] device tensor; word 0 becomes PLAN_ROWS_EXCEEDED when the device-side row count
    exceeds max_rows (the plans then come out empty instead of running past their buffers)."""
    _check(ridx, "recv_expert_indices", torch.int32)
    _check(recv_incl, "recv_plan", torch.int32, 1)
    dev = ridx.device
    EL = hi - lo
    n = max(max_rows * k, 1)
    excl = torch.empty((EL + 1,), dtype=torch.int32, device=dev)
    gemm_map = torch.empty((n,), dtype=torch.int32, device=dev)
    inv_gemm = torch.empty((n,), dtype=torch.int32, device=dev)
    scale_map = red_map = ret_incl = None
    if want_reduce:
        scale_map = torch.empty((max(max_rows, 1),), dtype=torch.int32, device=dev)
        red_map = torch.empty((n,), dtype=torch.int32, device=dev)
        ret_incl = torch.empty((W * S,), dtype=torch.int32, device=dev)
    call("epsb_expert_plans", ptr(ridx), ptr(recv_incl), k, lo, hi, W, S, max_tok_per_gpu, max_rows, ptr(excl),
         ptr(gemm_map), ptr(inv_gemm), ptr(scale_map), ptr(red_map), ptr(ret_incl), ptr(status), int(max_cluster),
         stream_ptr())
    return excl, gemm_map, inv_gemm, scale_map, red_map, ret_incl


def fastep_expand_plan(idx, E, excl=None):
    _check(idx, "expert_indices", torch.int32, 2)
    T, k = idx.shape
    if excl is None:
        excl = torch.empty((E + 1,), dtype=torch.int32, device=idx.device)
    mapping = torch.empty((max(T * k, 1),), dtype=torch.int32, device=idx.device)
    call("epsb_fastep_expand_plan", ptr(idx), T, k, E, ptr(excl), ptr(mapping), stream_ptr())
    return excl, mapping


def fastep_plan(all_gathered, my_rank, W, E, gemm_plan=None):
    _check(all_gathered, "all_gathered", torch.int32)
    dev = all_gathered.device
    EL = E // W
    remote_recv = torch.empty((W,), dtype=torch.int32, device=dev)
    local_send = torch.empty((W + 1,), dtype=torch.int32, device=dev)
    if gemm_plan is None:
        gemm_plan = torch.empty((EL + 1,), dtype=torch.int32, device=dev)
    arr = torch.empty((3, EL * W), dtype=torch.int32, device=dev)
    call("epsb_fastep_plan", ptr(all_gathered), my_rank, W, E, ptr(remote_recv), ptr(local_send), ptr(gemm_plan),
         ptr(arr[0]), ptr(arr[1]), ptr(arr[2]), stream_ptr())
    return remote_recv, local_send, gemm_plan, arr[0], arr[1], arr[2]


# ------------------------------------------------------------------ row movement


def _row_bytes(t):
    return t.shape[-1] * t.element_size()


def gather_rows(src, dst, mapping, map_div=1, map_mod=INT32_MAX, bounds=None, b0=0, b1=0, n_rows=None):
    """dst[i] = src[(mapping[i] // map_div) % map_mod]; rows [bounds[b0], bounds[b1]) or [0, n_rows)."""
    _check(src, "src")
    _check(dst, "dst")
    if _row_bytes(src) != _row_bytes(dst):
        raise EpsError("src and dst rows differ in size")
    max_rows = dst.shape[0]
    n = max_rows if n_rows is None else n_rows
    call("epsb_gather_rows", ptr(src), ptr(dst), ptr(mapping), map_div, map_mod, ptr(bounds), b0, b1, n, max_rows,
         _row_bytes(src), stream_ptr())
    return dst


def scatter_rows(src, dst, mapping, div, n):
    _check(src, "src")
    _check(dst, "dst")
    call("epsb_scatter_rows", ptr(src), ptr(dst), ptr(mapping), div, n, _row_bytes(src), stream_ptr())
    return dst


def arrange_rows(src, dst, src_off, rows, dst_off, n_seg, max_rows):
    _check(src, "src")
    _check(dst, "dst")
    call("epsb_arrange_rows", ptr(src), ptr(dst), ptr(src_off), ptr(rows), ptr(dst_off), n_seg, max_rows,
         _row_bytes(src), stream_ptr())
    return dst


def gather_row_weights(w_recv, gemm_map, excl, num_experts, max_rows):
    row_w = torch.empty((max(max_rows, 1),), dtype=torch.float32, device=w_recv.device)
    call("epsb_gather_row_weights", ptr(w_recv), ptr(gemm_map), ptr(excl), num_experts, max_rows, ptr(row_w),
         stream_ptr())
    return row_w


# ------------------------------------------------------------------ reductions


def local_reduce_ref(y, w_recv, scale_map, red_map, ret_incl, k, W, S, stage, send, max_rows=None):
    _check(y, "gemm_output", torch.bfloat16, 2)
    _check(send, "send_buf", torch.bfloat16, 2)
    H = y.shape[1]
    call("epsb_local_reduce_ref", ptr(y), ptr(w_recv), ptr(scale_map), ptr(red_map), ptr(ret_incl), k, W, S, stage,
         send.shape[0] if max_rows is None else max_rows, H, ptr(send), stream_ptr())
    return send


def local_reduce(y, red_map, ret_incl, k, W, S, stage, send, max_rows=None):
    _check(y, "gemm_output", torch.bfloat16, 2)
    _check(send, "send_buf", torch.bfloat16, 2)
    H = y.shape[1]
    call("epsb_local_reduce", ptr(y), ptr(red_map), ptr(ret_incl), k, W, S, stage,
         send.shape[0] if max_rows is None else max_rows, H, ptr(send), stream_ptr())
    return send


def global_reduce(recv, glob_map, out, W, shared=None, x=None, zero_scale=None, ref_arith=False):
    _check(out, "output", torch.bfloat16, 2)
    T, H = out.shape
    name = "epsb_global_reduce_ref" if ref_arith else "epsb_global_reduce"
    call(name, ptr(recv), ptr(glob_map), ptr(shared), ptr(x), ptr(zero_scale), T, W, H, ptr(out), stream_ptr())
    return out


def reduce_ep1(y, red_map, glob_map, ret_incl, S, k, out, shared=None, x=None, zero_scale=None):
    """ep_world_size == 1: out[t] = sum_j y[red_map[glob_map[t], j]] (+shared) (+x*zero_scale), fp32, one rounding."""
    _check(y, "gemm_output", torch.bfloat16, 2)
    _check(out, "output", torch.bfloat16, 2)
    T, H = out.shape
    call("epsb_reduce_ep1", ptr(y), ptr(red_map), ptr(glob_map), ptr(ret_incl), S, ptr(shared), ptr(x),
         ptr(zero_scale), T, k, H, ptr(out), stream_ptr())
    return out


def fastep_reduce(rows, raw, w, mapping, out, shared=None):
    _check(out, "out_tokens", torch.bfloat16, 2)
    _check(w, "weights", torch.float32, 2)
    T, H = out.shape
    k = w.shape[1]
    call("epsb_fastep_reduce", ptr(rows), ptr(raw), ptr(shared), ptr(w), ptr(mapping), T, k, H, ptr(out),
         stream_ptr())
    return out


def silu_run(gate_up, result, exclusive_sum=None, num_experts=0):
    _check(gate_up, "gate_up", torch.bfloat16, 2)
    _check(result, "result", torch.bfloat16, 2)
    rows, two_i = gate_up.shape
    call("epsb_silu_run", ptr(gate_up), ptr(result), ptr(exclusive_sum), num_experts, rows, two_i // 2, stream_ptr())
    return result


# ------------------------------------------------------------------ grouped GEMM


def topk_sigmoid(scores, bias, num_expert_groups, topk_groups, topk, route_scale=1.0, num_ffn_experts=None,
                 expert_indices=None, expert_scales=None, score_func="sigmoid"):
    """Router (reference utils/topk_sigmoid): scores [T, E] fp32 or bf16 logits, bias [E] fp32 or None ->
    (expert_indices [T, topk] int32, expert_scales [T, topk] fp32) in the layout the Scheduler reads."""
    if scores.dtype not in (torch.float32, torch.bfloat16):
        raise EpsError(f"scores must be float32 or bfloat16, got {scores.dtype}")
    _check(scores, "scores", scores.dtype, 2)
    T, E = scores.shape
    if bias is not None:
        _check(bias, "bias", torch.float32, 1)
        if bias.numel() != E:
            raise EpsError(f"bias must have {E} entries")
    dev = scores.device
    if expert_indices is None:
        expert_indices = torch.empty((T, topk), dtype=torch.int32, device=dev)
    if expert_scales is None:
        expert_scales = torch.empty((T, topk), dtype=torch.float32, device=dev)
    if score_func not in ("sigmoid", "softmax"):
        raise EpsError(f"score_func must be 'sigmoid' or 'softmax', got {score_func!r}")
    call("epsb_router_topk", int(score_func == "softmax"), ptr(scores), int(scores.dtype == torch.bfloat16), ptr(bias), T, E,
         int(num_expert_groups), int(topk_groups), int(topk), float(route_scale),
         int(E if num_ffn_experts is None else num_ffn_experts), ptr(expert_indices), ptr(expert_scales), stream_ptr())
    return expert_indices, expert_scales


def rms_norm(input, scale, eps, out=None):
    """out = (input * rsqrt(mean(input^2, dim=1) + eps)) * scale, bf16 rows (reference utils.rms_norm_op)."""
    _check(input, "input", torch.bfloat16, 2)
    _check(scale, "scale", torch.bfloat16, 1)
    m, n = input.shape
    if scale.numel() != n:
        raise EpsError(f"scale must have {n} entries")
    if out is None:
        out = torch.empty_like(input)
    else:
        _check(out, "output", torch.bfloat16, 2)
    call("epsb_rms_norm", ptr(out), ptr(input), ptr(scale), float(eps), m, n, stream_ptr())
    return out


def gemm_row_sources(gemm_map, excl, num_experts, k, max_rows, w_src=None, send_map=None, T=0):
    """-> (a_rows int32 [max_rows], row_w fp32 [max_rows] or None): source row and gate weight of every GEMM row."""
    dev = gemm_map.device
    a_rows = torch.empty((max(max_rows, 1),), dtype=torch.int32, device=dev)
    row_w = torch.empty((max(max_rows, 1),), dtype=torch.float32, device=dev) if w_src is not None else None
    call("epsb_gemm_row_sources", ptr(gemm_map), ptr(excl), num_experts, k, ptr(send_map), int(T), ptr(w_src), max_rows,
         ptr(a_rows), ptr(row_w), stream_ptr())
    return a_rows, row_w


def grouped_gemm_fp8(mode, A, a_s, B, b_s, excl, out=None, out_scales=None, row_w=None, status=None,
                     sm_count=0, a_rows=None):
    """FP8 block-scaled grouped GEMM; see include/eps_b200.h for the three modes.

    a_rows: optional int32 [rows]; GEMM row m then reads row a_rows[m] of A / a_s (index-driven A loads), and the
    outputs have a_rows.numel() rows.

    sm_count: SMs this launch may occupy (0 = all), the sm_count of the reference's aok_create.
    """
    _check(A, "A", _FP8, 2)
    _check(a_s, "A_scale", torch.float32, 2)
    _check(B, "B", _FP8, 3)
    _check(b_s, "B_scale", torch.float32, 3)
    _check(excl, "exclusive_sum", torch.int32, 1)
    src_rows, K = A.shape
    max_rows = src_rows if a_rows is None else a_rows.numel()
    E, N, K2 = B.shape
    if K2 != K:
        raise EpsError(f"A has K={K} but B has K={K2}")
    if excl.numel() != E + 1:
        raise EpsError(f"exclusive_sum must have {E + 1} entries")
    dev = A.device
    if mode == GEMM_GATEUP:
        I = N // 2
        C = out if out is not None else torch.empty((max_rows, I), dtype=torch.uint8, device=dev)
        c_s = out_scales if out_scales is not None else torch.empty((max_rows, I // 128), dtype=torch.float32, device=dev)
    else:
        C = out if out is not None else torch.empty((max_rows, N), dtype=torch.bfloat16, device=dev)
        c_s = None
    if a_rows is not None:
        _check(a_rows, "a_rows", torch.int32, 1)
        call("epsb_grouped_gemm_fp8_gather", mode, ptr(A), ptr(a_s), src_rows, ptr(a_rows), ptr(B), ptr(b_s), ptr(excl),
             E, max_rows, N, K, ptr(C), ptr(c_s), ptr(row_w), ptr(status), int(sm_count), stream_ptr())
        return (C, c_s) if mode == GEMM_GATEUP else C
    call("epsb_grouped_gemm_fp8", mode, ptr(A), ptr(a_s), ptr(B), ptr(b_s), ptr(excl), E, max_rows, N, K, ptr(C),
         ptr(c_s), ptr(row_w), ptr(status), int(sm_count), stream_ptr())
    return (C, c_s) if mode == GEMM_GATEUP else C


def grouped_gemm_bf16(A, B, excl, out=None, status=None, sm_count=0, rows_hint=0):
    """bf16 x bf16 -> bf16 grouped GEMM (the reference's aok_run): A [max_rows, K], B [E, N, K], excl [E+1] int32;
    rows [excl[e], excl[e+1]) of A times B[e]^T, fp32 accumulation.  rows_hint = expected number of rows (the
    reference's num_tokens_hint; 0 = unknown): picks 256-row tiles on CTA pairs for large experts."""
    _check(A, "A", torch.bfloat16, 2)
    _check(B, "B", torch.bfloat16, 3)
    _check(excl, "exclusive_sum", torch.int32, 1)
    max_rows, K = A.shape
    E, N, K2 = B.shape
    if K2 != K:
        raise EpsError(f"A has K={K} but B has K={K2}")
    if excl.numel() != E + 1:
        raise EpsError(f"exclusive_sum must have {E + 1} entries")
    C = out if out is not None else torch.empty((max_rows, N), dtype=torch.bfloat16, device=A.device)
    call("epsb_grouped_gemm_bf16", ptr(A), ptr(B), ptr(excl), E, max_rows, int(rows_hint), N, K, ptr(C), ptr(status),
         int(sm_count), stream_ptr())
    return C
