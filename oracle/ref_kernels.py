"""ctypes face of oracle/_ref/libeps_ref.so: the REFERENCE's own kernels, run on the GPU.

TEST INFRASTRUCTURE ONLY (second witness for the oracle and generator of tests/golden fixtures).
All arguments are torch CUDA tensors; every call synchronises before returning.
"""
from __future__ import annotations

import ctypes
import os

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB = os.path.join(_HERE, "_ref", "libeps_ref.so")
_lib = None


def available() -> bool:
    return os.path.exists(LIB)


def lib():
    global _lib
    if _lib is None:
        _lib = ctypes.CDLL(LIB)
    return _lib


def _p(t):
    return ctypes.c_void_p(None if t is None else t.data_ptr())


def _sync():
    rc = lib().ref_sync()
    if rc != 0:
        raise RuntimeError(f"reference kernel failed: cudaError {rc}")


def _i32(n, dev, fill=None):
    t = torch.empty((max(int(n), 1),), dtype=torch.int32, device=dev)
    if fill is not None:
        t.fill_(fill)
    return t


def comm_plan(idx, E, W, S):
    T, k = idx.shape
    dev = idx.device
    lead = _i32(T * W, dev)
    mapping = _i32(T * W, dev, -1)
    incl = _i32(W * S, dev, 0)
    lib().ref_comm_plan(_p(idx), _p(lead), _p(mapping), _p(incl), T, k, E, S, W)
    _sync()
    return mapping, incl


def gemm_plan(ridx, recv_incl, k, lo, hi, E, W, S, max_tok):
    dev = ridx.device
    R = ridx.shape[0]
    mapping = _i32(R * k, dev, -1)
    excl = _i32(hi - lo + 1, dev, 0)
    lib().ref_gemm_plan(_p(ridx), _p(recv_incl), _p(mapping), _p(excl), lo, hi, E, S, k, W,
                        ctypes.c_longlong(max_tok))
    _sync()
    return excl, mapping


def local_reduce_plan(ridx, recv_incl, gemm_map, excl, k, lo, hi, E, W, S, max_tok, num_global_tokens):
    dev = ridx.device
    R = ridx.shape[0]
    tail, stail = _i32(R, dev), _i32(R, dev)
    red_map, scale_map, ret_incl = _i32(R * k, dev, -1), _i32(R, dev, -1), _i32(W * S, dev, 0)
    lib().ref_local_reduce_plan(_p(ridx), _p(tail), _p(stail), _p(recv_incl), _p(red_map), _p(scale_map),
                                _p(ret_incl), _p(gemm_map), _p(excl), lo, hi, E, S, k, W,
                                ctypes.c_longlong(max_tok), num_global_tokens)
    _sync()
    return scale_map, red_map, ret_incl


def global_reduce_plan(idx, send_map, send_incl, E, W, S):
    T, k = idx.shape
    dev = idx.device
    tail = _i32(T * W, dev)
    glob, coll = _i32(T * W, dev, -1), _i32(W * S, dev, 0)
    lib().ref_global_reduce_plan(_p(idx), _p(tail), _p(glob), _p(coll), _p(send_map), _p(send_incl), T, E, S, k, W)
    _sync()
    return glob, coll


def zero_plan(idx, w):
    T, k = idx.shape
    z = torch.zeros((max(T, 1),), dtype=torch.float32, device=idx.device)
    lib().ref_zero_plan(_p(idx), _p(w), T, k, _p(z))
    _sync()
    return z


def zero_reduce(zero_scale, x, out):
    T, H = x.shape
    lib().ref_zero_reduce(_p(zero_scale), T, ctypes.c_longlong(H), _p(x), _p(out))
    _sync()
    return out


def local_reduce(red_map, scale_map, ret_incl, S, k, W, y, send, w_recv, hint, stage):
    H = y.shape[1]
    lib().ref_local_reduce(_p(red_map), _p(scale_map), _p(ret_incl), S, k, W, ctypes.c_longlong(H), _p(y), _p(send),
                           _p(w_recv), ctypes.c_longlong(hint), stage)
    _sync()
    return send


def global_reduce(glob_map, W, recv, out, shared=None):
    T, H = out.shape
    lib().ref_global_reduce(_p(glob_map), T, W, ctypes.c_longlong(H), _p(recv), _p(out), _p(shared))
    _sync()
    return out


def quant_1x128(x):
    rows, cols = x.shape
    q = torch.empty((rows, cols), dtype=torch.uint8, device=x.device)
    s = torch.empty((rows, cols // 128), dtype=torch.float32, device=x.device)
    lib().ref_quant_1x128(_p(x), ctypes.c_longlong(rows), ctypes.c_longlong(cols), _p(q), _p(s))
    _sync()
    return q, s


def silu(gate_up, excl, num_experts, hint):
    rows, two_i = gate_up.shape
    act = torch.zeros((rows, two_i // 2), dtype=torch.bfloat16, device=gate_up.device)
    lib().ref_silu(_p(gate_up), _p(act), _p(excl), num_experts, two_i, hint)
    _sync()
    return act


def topk_sigmoid(scores, bias, n_groups, topk_groups, topk, route_scale=1.0):
    """The reference router (utils/topk_sigmoid.cu); returns None for shapes it does not instantiate."""
    T, E = scores.shape
    dev = scores.device
    w = torch.empty((T, topk), dtype=torch.float32, device=dev)
    idx = torch.empty((T, topk), dtype=torch.int32, device=dev)
    fn = lib().ref_topk_sigmoid_bf16 if scores.dtype == torch.bfloat16 else lib().ref_topk_sigmoid_f32
    rc = fn(_p(scores), _p(bias), _p(w), _p(idx), T, E, n_groups, topk_groups, topk, ctypes.c_float(route_scale))
    if rc != 0:
        return None
    _sync()
    return idx, w


def rms_norm(x, scale, eps):
    """The reference rms_norm on bf16 rows; None if it refuses the shape (odd row length)."""
    out = torch.empty_like(x)
    rc = lib().ref_rms_norm_bf16(_p(out), _p(x), _p(scale), ctypes.c_float(eps), x.shape[0], x.shape[1])
    if rc != 0:
        return None
    _sync()
    return out



# ------------------------------------------------------------------ fast_ep (src/fast_ep/all_to_all/fast_ep_kernels.cu)

def _ll(v):
    return ctypes.c_longlong(int(v))


def fastep_expand_plan(idx, E):
    """expandPlan: -> (exclusive_sum [E+1], mapping [T*k])."""
    T, k = idx.shape
    dev = idx.device
    excl = _i32(E + 1, dev, 0)
    mapping = _i32(T * k, dev, -1)
    lib().ref_fastep_expand_plan(_p(idx), _p(excl), _p(mapping), _ll(T), _ll(k), _ll(E))
    _sync()
    return excl, mapping


def fastep_expand(x, idx, excl, mapping, E):
    """expand: rows of x scattered into send order -> [T*k, H] bf16 (H must be a hidden size the reference lists)."""
    T, k = idx.shape
    dst = torch.zeros((max(T * k, 1), x.shape[1]), dtype=torch.bfloat16, device=x.device)
    rc = lib().ref_fastep_expand(_p(x), _p(dst), _ll(x.shape[1]), _p(idx), _p(excl), _p(mapping), _ll(T), _ll(k), _ll(E))
    if rc:
        raise RuntimeError("the reference does not instantiate this hidden size")
    _sync()
    return dst


def fastep_reduce(rows, raw, w, idx, excl, mapping, E, shared=None):
    """reduce: weighted combine of the k slots per token -> [T, H] bf16."""
    T, k = idx.shape
    out = torch.zeros((max(T, 1), rows.shape[1]), dtype=torch.bfloat16, device=rows.device)
    rc = lib().ref_fastep_reduce(_p(rows), _p(out), _p(shared), _p(raw), _p(w), _ll(rows.shape[1]), _p(idx), _p(excl),
                                 _p(mapping), _ll(T), _ll(k), _ll(E))
    if rc:
        raise RuntimeError("the reference does not instantiate this hidden size")
    _sync()
    return out


def fastep_plan(all_gathered, my_rank, W, E):
    """allGatherPlan on a pre-filled table [W, E+1]: -> (remote_recv [W], local_send [W+1], gemm_plan [EL+1],
    arr_src, arr_rows, arr_dst [EL*W])."""
    dev = all_gathered.device
    EL = E // W
    remote, send, gplan = _i32(W, dev, 0), _i32(W + 1, dev, 0), _i32(EL + 1, dev, 0)
    src, rows, dst = _i32(EL * W, dev, 0), _i32(EL * W, dev, 0), _i32(EL * W, dev, 0)
    lib().ref_fastep_plan(_p(all_gathered), _ll(my_rank), _ll(W), _ll(E), _p(remote), _p(send), _p(gplan), _p(src),
                          _p(rows), _p(dst))
    _sync()
    return remote, send, gplan, src, rows, dst


def fastep_arrange(src_rows, out_rows, W, E, arr_src, arr_rows, arr_dst, num_tokens_hint):
    rc = lib().ref_fastep_arrange(_p(src_rows), _p(out_rows), _ll(W), _ll(E), _ll(src_rows.shape[1]), _p(arr_src),
                                  _p(arr_rows), _p(arr_dst), _ll(num_tokens_hint))
    if rc:
        raise RuntimeError("the reference does not instantiate this hidden size")
    _sync()
    return out_rows
