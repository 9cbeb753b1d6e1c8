"""numpy face of the CPU oracle (oracle/eps_oracle.c).

TEST INFRASTRUCTURE ONLY: imported by tests/, by __graft_entry__.smoke() and by
bench.py's cpu_baseline / reference arm.  The eps_b200 package never imports it.

Parity pin: the reference has no tests or golden vectors for this path; the pin
is the reference's own kernels compiled from its sources (ref_harness.cu ->
oracle/_ref/) and the fixtures recorded from them in tests/golden/.
"""
from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SRC = os.path.join(_HERE, "eps_oracle.c")
_BUILD = os.path.join(_HERE, "_build")
_LIB = os.path.join(_BUILD, "libeps_oracle.so")
ZC_MARK = 1000000

_lib = None


def build(force: bool = False) -> str:
    os.makedirs(_BUILD, exist_ok=True)
    if force or not os.path.exists(_LIB) or os.path.getmtime(_LIB) < os.path.getmtime(_SRC):
        cmd = ["gcc", "-O3", "-march=native", "-fopenmp", "-fPIC", "-shared", "-std=c11", "-ffp-contract=off",
               _SRC, "-o", _LIB, "-lm"]
        subprocess.run(cmd, check=True)
    return _LIB


def _p(a):
    return None if a is None else a.ctypes.data_as(ctypes.c_void_p)


def lib():
    global _lib
    if _lib is None:
        _lib = ctypes.CDLL(build())
        _lib.orc_num_threads.restype = ctypes.c_int
        _lib.orc_f32_to_e4m3.restype = ctypes.c_uint8
        _lib.orc_f32_to_e4m3.argtypes = [ctypes.c_float]
        _lib.orc_e4m3_to_f32.restype = ctypes.c_float
        _lib.orc_e4m3_to_f32.argtypes = [ctypes.c_uint8]
        _lib.orc_f32_to_bf16.restype = ctypes.c_uint16
        _lib.orc_f32_to_bf16.argtypes = [ctypes.c_float]
        for name in ("orc_comm_plan", "orc_recv_plan", "orc_gemm_plan"):
            getattr(_lib, name).restype = ctypes.c_int
    return _lib


def num_threads() -> int:
    return lib().orc_num_threads()


def set_num_threads(n: int) -> int:
    """OpenMP threads of the oracle's loops from now on (a launcher such as torch.distributed.run exports
    OMP_NUM_THREADS=1 to its children; a caller that owns the host's cores sets the count itself)."""
    lib().orc_set_num_threads(int(max(1, n)))
    return num_threads()


def _i32(a):
    return np.ascontiguousarray(a, dtype=np.int32)


def _L(v):
    return ctypes.c_int64(int(v))


# ------------------------------------------------------------------ formats

def e4m3_table() -> np.ndarray:
    t = np.empty(256, dtype=np.float32)
    lib().orc_e4m3_table(_p(t))
    return t


def f32_to_e4m3(x: float) -> int:
    return int(lib().orc_f32_to_e4m3(ctypes.c_float(x)))


def bf16_bits(x_f32: np.ndarray) -> np.ndarray:
    """fp32 -> bf16 bit patterns (uint16), round to nearest even."""
    u = np.ascontiguousarray(x_f32, dtype=np.float32).view(np.uint32).astype(np.uint64)
    nan = (u & 0x7fffffff) > 0x7f800000
    r = ((u + 0x7fff + ((u >> 16) & 1)) >> 16).astype(np.uint16)
    r[nan] = ((u[nan] >> 16) | 0x40).astype(np.uint16)
    return r


def bf16_to_f32(bits: np.ndarray) -> np.ndarray:
    return (np.ascontiguousarray(bits, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)


# ------------------------------------------------------------------ quant

def quant_1x128(x_bits: np.ndarray, div_mode: int = 0):
    """div_mode 0: scale = amax/448 (IEEE); 1: the reference kernel's div.full.f32 (= amax * fl(1/448))."""
    x_bits = np.ascontiguousarray(x_bits, dtype=np.uint16)
    rows, cols = x_bits.shape
    q = np.empty((rows, cols), dtype=np.uint8)
    s = np.empty((rows, cols // 128), dtype=np.float32)
    lib().orc_quant_1x128_mode(_p(x_bits), _L(rows), _L(cols), _p(q), _p(s), int(div_mode))
    return q, s


def quant_1x128_f32(x: np.ndarray):
    x = np.ascontiguousarray(x, dtype=np.float32)
    rows, cols = x.shape
    q = np.empty((rows, cols), dtype=np.uint8)
    s = np.empty((rows, cols // 128), dtype=np.float32)
    lib().orc_quant_1x128_f32(_p(x), _L(rows), _L(cols), _p(q), _p(s))
    return q, s


def dequant_1x128(q, s):
    q = np.ascontiguousarray(q, dtype=np.uint8)
    s = np.ascontiguousarray(s, dtype=np.float32)
    rows, cols = q.shape
    x = np.empty((rows, cols), dtype=np.uint16)
    lib().orc_dequant_1x128(_p(q), _p(s), _L(rows), _L(cols), _p(x))
    return x


def quant_block128(w: np.ndarray):
    """w [..., n, k] fp32 -> codes uint8 same shape, scales [..., ceil(n/128), ceil(k/128)]."""
    w = np.ascontiguousarray(w, dtype=np.float32)
    lead = w.shape[:-2]
    n, k = w.shape[-2:]
    w3 = w.reshape((-1, n, k))
    q = np.empty(w3.shape, dtype=np.uint8)
    nb, kb = (n + 127) // 128, (k + 127) // 128
    s = np.empty((w3.shape[0], nb, kb), dtype=np.float32)
    for m in range(w3.shape[0]):
        lib().orc_quant_block128(_p(w3[m]), _L(n), _L(k), _p(q[m]), _p(s[m]))
    return q.reshape(lead + (n, k)), s.reshape(lead + (nb, kb))


# ------------------------------------------------------------------ plans

def comm_plan(idx, E, W, S):
    idx = _i32(idx)
    T, k = idx.shape
    mapping = np.full(max(T * W, 1), -1, dtype=np.int32)
    incl = np.zeros(W * S, dtype=np.int32)
    n = lib().orc_comm_plan(_p(idx), T, k, E, W, S, _p(mapping), _p(incl))
    return mapping[:n].copy(), incl


def recv_plan(gathered, my_rank, W, S):
    gathered = _i32(gathered)
    recv = np.zeros(W * S, dtype=np.int32)
    remote = np.zeros(W * S, dtype=np.int32)
    total = lib().orc_recv_plan(_p(gathered), my_rank, W, S, _p(recv), _p(remote))
    return recv, remote, total


def gemm_plan(ridx, k, lo, hi, max_tok_per_gpu, W):
    ridx = _i32(ridx).reshape(-1, k)
    R = ridx.shape[0]
    excl = np.zeros(hi - lo + 1, dtype=np.int32)
    mapping = np.full(max(R * k, 1), -1, dtype=np.int32)
    D = lib().orc_gemm_plan(_p(ridx), R, k, lo, hi, max_tok_per_gpu, W, _p(excl), _p(mapping))
    return excl, mapping[:D].copy()


def local_reduce_plan(ridx, recv_incl, gemm_map, excl, k, lo, hi, W, S):
    ridx = _i32(ridx).reshape(-1, k)
    recv_incl = _i32(recv_incl)
    R = int(recv_incl[-1])
    scale_map = np.full(max(R, 1), -1, dtype=np.int32)
    red_map = np.full(max(R * k, 1), -1, dtype=np.int32)
    ret_incl = np.zeros(W * S, dtype=np.int32)
    lib().orc_local_reduce_plan(_p(ridx), _p(recv_incl), _p(_i32(gemm_map)), _p(_i32(excl)), k, lo, hi, W, S,
                                _p(scale_map), _p(red_map), _p(ret_incl))
    return scale_map[:R].copy(), red_map[:R * k].reshape(R, k).copy(), ret_incl


def global_reduce_plan(idx, send_map, send_incl, E, W, S):
    idx = _i32(idx)
    T, k = idx.shape
    glob = np.full(max(T * W, 1), -1, dtype=np.int32)
    coll = np.zeros(W * S, dtype=np.int32)
    lib().orc_global_reduce_plan(_p(idx), _p(_i32(send_map)), _p(_i32(send_incl)), T, k, E, W, S, _p(glob), _p(coll))
    return glob[:T * W].reshape(T, W).copy(), coll


def zero_plan(idx, w):
    idx = _i32(idx)
    w = np.ascontiguousarray(w, dtype=np.float32)
    T, k = idx.shape
    z = np.zeros(max(T, 1), dtype=np.float32)
    lib().orc_zero_plan(_p(idx), _p(w), T, k, _p(z))
    return z[:T]


def topk_sigmoid(scores, bias, n_groups, topk_groups, topk, route_scale=1.0, num_ffn_experts=None,
                 score_func="sigmoid"):
    """Router, restating reference src/utils/topk_sigmoid.cu:158-262 in fp32 numpy (vectorised over tokens).

    score = 1/(1+exp(-x)) (:181-184 `sigmoid`, fp32), biased = score + bias (:211-216); group score = sum of the
    group's two largest biased scores (:65-102); the topk_groups best groups stay (:104-118); topk times the largest
    biased score among their experts (:120-156); scales = score * (route_scale / sum of chosen scores) (:236-244).
    Ties go to the lower id, as the reference's strict `>` does.  numpy's exp may differ from the device's expf in
    the last place, so callers compare the scales with a tolerance and treat index differences at equal scores as ties.
    -> (indices int32 [T, topk] with ids >= num_ffn_experts mapped to -1-(id-num_ffn), scales fp32 [T, topk],
        biased scores fp32 [T, E] for the callers' tie check)."""
    x = np.asarray(scores, dtype=np.float32)
    T, E = x.shape
    one = np.float32(1.0)
    if score_func == "softmax":   # not in the reference: softmax over the token's logits, fp32
        ex = np.exp(x - x.max(axis=1, keepdims=True), dtype=np.float32)
        orig = (ex / ex.sum(axis=1, keepdims=True, dtype=np.float32)).astype(np.float32)
    else:
        orig = (one / (one + np.exp(-x, dtype=np.float32))).astype(np.float32)
    biased = orig if bias is None else (orig + np.asarray(bias, dtype=np.float32)[None, :]).astype(np.float32)
    gsize = E // n_groups
    neg = np.float32(-np.finfo(np.float32).max)
    grp = biased.reshape(T, n_groups, gsize)
    # two largest of each group, ties to the lower index (stable argsort on the negated score)
    order = np.argsort(-grp, axis=2, kind="stable")
    first = np.take_along_axis(grp, order[:, :, :1], 2)[:, :, 0]
    second = np.take_along_axis(grp, order[:, :, 1:2], 2)[:, :, 0] if gsize > 1 else np.full((T, n_groups), neg)
    gscore = (first + second).astype(np.float32)
    gorder = np.argsort(-gscore, axis=1, kind="stable")[:, :topk_groups]
    gmask = np.zeros((T, n_groups), dtype=bool)
    np.put_along_axis(gmask, gorder, True, 1)
    cand = np.where(np.repeat(gmask, gsize, axis=1), biased, neg)
    sel = np.argsort(-cand, axis=1, kind="stable")[:, :topk]
    chosen = np.take_along_axis(orig, sel, 1)
    total = np.zeros(T, dtype=np.float32)
    for j in range(topk):                      # the reference sums in selection order
        total = (total + chosen[:, j]).astype(np.float32)
    rescale = (np.float32(route_scale) / total).astype(np.float32)
    scales = (chosen * rescale[:, None]).astype(np.float32)
    idx = sel.astype(np.int32)
    nf = E if num_ffn_experts is None else num_ffn_experts
    idx = np.where(idx >= nf, -1 - (idx - nf), idx).astype(np.int32)
    return idx, scales, biased


def rms_norm(x_bits, scale_bits, eps):
    """RMS normalisation of bf16 rows, restating reference src/utils/rms_norm.cu:103-140: the sum of squares in fp32
    (here accumulated in float64 and rounded once: the reference's order is a block reduction), inv = rsqrt(.5 * sum
    / (n/2) + eps) in fp32, out = bf16((x * inv) * scale).  -> bf16 bits [m, n]."""
    x = bf16_to_f32(np.asarray(x_bits))
    sc = bf16_to_f32(np.asarray(scale_bits))
    n = x.shape[1]
    total = (x.astype(np.float64) ** 2).sum(axis=1).astype(np.float32)
    inv = (np.float32(1.0) / np.sqrt(np.float32(0.5) * total / np.float32(n // 2) + np.float32(eps), dtype=np.float32))
    out = ((x * inv.astype(np.float32)[:, None]).astype(np.float32) * sc[None, :]).astype(np.float32)
    return bf16_bits(out)


def fastep_expand_plan(idx, E):
    idx = _i32(idx)
    T, k = idx.shape
    excl = np.zeros(E + 1, dtype=np.int32)
    mapping = np.zeros(max(T * k, 1), dtype=np.int32)
    lib().orc_fastep_expand_plan(_p(idx), T, k, E, _p(excl), _p(mapping))
    return excl, mapping[:T * k]


def fastep_plan(all_gathered, my_rank, W, E):
    ag = _i32(all_gathered)
    EL = E // W
    remote = np.zeros(W, dtype=np.int32)
    send = np.zeros(W + 1, dtype=np.int32)
    gplan = np.zeros(EL + 1, dtype=np.int32)
    src = np.zeros(EL * W, dtype=np.int32)
    rows = np.zeros(EL * W, dtype=np.int32)
    dst = np.zeros(EL * W, dtype=np.int32)
    lib().orc_fastep_plan(_p(ag), my_rank, W, E, _p(remote), _p(send), _p(gplan), _p(src), _p(rows), _p(dst))
    return remote, send, gplan, src, rows, dst


# ------------------------------------------------------------------ compute

def grouped_gemm_fp8(A, a_s, B, b_s, excl):
    A = np.ascontiguousarray(A, dtype=np.uint8)
    B = np.ascontiguousarray(B, dtype=np.uint8)
    a_s = np.ascontiguousarray(a_s, dtype=np.float32)
    b_s = np.ascontiguousarray(b_s, dtype=np.float32)
    excl = _i32(excl)
    E, N, K = B.shape
    C = np.zeros((A.shape[0], N), dtype=np.float32)
    lib().orc_grouped_gemm_fp8(_p(A), _p(a_s), _p(B), _p(b_s), _p(excl), E, _L(N), _L(K), _p(C))
    return C


def swiglu(gate_up):
    gate_up = np.ascontiguousarray(gate_up, dtype=np.float32)
    rows, two_i = gate_up.shape
    act = np.empty((rows, two_i // 2), dtype=np.float32)
    lib().orc_swiglu(_p(gate_up), _L(rows), _L(two_i // 2), _p(act))
    return act


def fastep_reduce(rows_bits, raw_bits, w, mapping, shared_bits=None):
    rows_bits = np.ascontiguousarray(rows_bits, dtype=np.uint16)
    raw_bits = np.ascontiguousarray(raw_bits, dtype=np.uint16)
    w = np.ascontiguousarray(w, dtype=np.float32)
    T, k = w.shape
    H = raw_bits.shape[1]
    out = np.empty((T, H), dtype=np.uint16)
    sh = None if shared_bits is None else np.ascontiguousarray(shared_bits, dtype=np.uint16)
    lib().orc_fastep_reduce(_p(rows_bits), _p(raw_bits), _p(sh), _p(w), _p(_i32(mapping)), T, k, _L(H), _p(out))
    return out


# ------------------------------------------------------------------ whole-layer semantics (single process, W ranks simulated)

def moe_layer_fp32(x_bits, idx, w, Wgu_q, Wgu_s, Wd_q, Wd_s, requant_act=True, shared=None):
    """The layer's numerical standard: fp32 dequantised expert FFN over the routed (token, slot)
    pairs, fp32 weighted sum, identity experts (idx < 0) pass x scaled by their weight, one bf16
    rounding at the end.  Routing-order independent, so it is the same for the staged EPS path and
    for fast_ep.  Weights are the global [E, 2I, H] / [E, H, I] code tensors.
    `shared` = (Wgu_q, Wgu_s, Wd_q, Wd_s) of an always-on expert with leading dimension 1."""
    idx = _i32(idx)
    T, k = idx.shape
    E, two_i, H = Wgu_q.shape
    xq, xs = quant_1x128(x_bits, div_mode=1)
    order = []
    for e in range(E):
        tt, jj = np.nonzero(idx == e)
        order.append(np.stack([tt, jj], 1))
    excl = np.zeros(E + 1, dtype=np.int32)
    excl[1:] = np.cumsum([len(o) for o in order])
    pairs = np.concatenate(order, 0) if len(order) else np.zeros((0, 2), dtype=np.int64)
    A = xq[pairs[:, 0]]
    A_s = xs[pairs[:, 0]]
    gu = grouped_gemm_fp8(A, A_s, Wgu_q, Wgu_s, excl)
    act = swiglu(gu)
    if requant_act:
        aq, a_s = quant_1x128_f32(act)
    else:
        raise NotImplementedError
    y = grouped_gemm_fp8(aq, a_s, Wd_q, Wd_s, excl)
    out = np.zeros((T, H), dtype=np.float32)
    np.add.at(out, pairs[:, 0], y * w[pairs[:, 0], pairs[:, 1]][:, None])
    xf = bf16_to_f32(x_bits)
    zs = np.where(idx < 0, w, 0).sum(1).astype(np.float32)
    out += xf * zs[:, None]
    if shared is not None:
        sgu_q, sgu_s, sd_q, sd_s = shared
        ex1 = np.array([0, T], dtype=np.int32)
        sg = grouped_gemm_fp8(xq, xs, sgu_q, sgu_s, ex1)
        sa_q, sa_s = quant_1x128_f32(swiglu(sg))
        out += grouped_gemm_fp8(sa_q, sa_s, sd_q, sd_s, ex1)
    return out


def moe_layer_fp32_sampled(x_bits, idx, w, expert_weights, shared=None, return_magnitude=False):
    """The standard of moe_layer_fp32 evaluated on a SAMPLE of tokens: rows of x_bits / idx / w are the sampled
    tokens only.  expert_weights(e) -> (Wgu_q [2I,H], Wgu_s [2I/128,H/128], Wd_q [H,I], Wd_s [H/128,I/128]) is
    asked once for every FFN expert the sample routes to, so a layer with hundreds of experts costs the oracle
    only the experts (and rows) of the sample.  shared as in moe_layer_fp32.  Returns fp32 [n, H]; with
    return_magnitude also the sum of the ABSOLUTE values of the terms each output element is the sum of (weighted expert
    rows, identity term, shared expert's row): what the roundings of stored intermediate values scale with."""
    idx = _i32(idx)
    w = np.ascontiguousarray(w, dtype=np.float32)
    n, k = idx.shape
    xq, xs = quant_1x128(x_bits, div_mode=1)
    H = xq.shape[1]
    out = np.zeros((n, H), dtype=np.float32)
    mag = np.zeros((n, H), dtype=np.float32)
    for e in np.unique(idx[idx >= 0]):
        tt, jj = np.nonzero(idx == e)
        gu_q, gu_s, d_q, d_s = expert_weights(int(e))
        ex = np.array([0, len(tt)], dtype=np.int32)
        gu = grouped_gemm_fp8(xq[tt], xs[tt], gu_q[None], gu_s[None], ex)
        aq, a_s = quant_1x128_f32(swiglu(gu))
        y = grouped_gemm_fp8(aq, a_s, d_q[None], d_s[None], ex) * w[tt, jj][:, None]
        np.add.at(out, tt, y)
        np.add.at(mag, tt, np.abs(y))
    zs = np.where(idx < 0, w, 0).sum(1).astype(np.float32)
    ident = bf16_to_f32(x_bits) * zs[:, None]
    out += ident
    mag += np.abs(ident)
    if shared is not None:
        sgu_q, sgu_s, sd_q, sd_s = shared
        ex1 = np.array([0, n], dtype=np.int32)
        sg = grouped_gemm_fp8(xq, xs, sgu_q, sgu_s, ex1)
        sa_q, sa_s = quant_1x128_f32(swiglu(sg))
        sh = grouped_gemm_fp8(sa_q, sa_s, sd_q, sd_s, ex1)
        out += sh
        mag += np.abs(sh)
    return (out, mag) if return_magnitude else out
