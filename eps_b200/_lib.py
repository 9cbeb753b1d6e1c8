"""ctypes binding of libeps_b200.so (the C ABI declared in include/eps_b200.h).

There is no fallback: if the shared library is missing, `lib()` raises, and every
operator of this package raises with it.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import c_char_p, c_float, c_int, c_int32, c_int64, c_void_p

_HERE = os.path.dirname(os.path.abspath(__file__))
# EPS_B200_LIB selects another build of the same library (kernel A/B comparisons).
LIB_PATH = os.environ.get("EPS_B200_LIB") or os.path.join(_HERE, "libeps_b200.so")

_P = c_void_p
_I = c_int
_L = c_int64

# name -> argtypes; every function returns int (EPSB_OK == 0).
SIGNATURES = {
    "epsb_quant_1x128": [_P, _L, _L, _P, _P, _I, _P],
    "epsb_quant_1x128_ragged": [_P, _P, _I, _L, _P, _P, _L, _I, _P],
    "epsb_dequant_1x128": [_P, _P, _L, _L, _P, _P],
    "epsb_quant_block128": [_P, _L, _L, _L, _P, _P, _P],
    "epsb_source_plans": [_P, _P, _I, _I, _I, _I, _I, _P, _P, _P, _P, _P, _I, _P],
    "epsb_zero_plan": [_P, _P, _I, _I, _P, _P],
    "epsb_recv_plan": [_P, _I, _I, _I, _P, _P, _P, _P],
    "epsb_expert_plans": [_P, _P, _I, _I, _I, _I, _I, _I, _L, _P, _P, _P, _P, _P, _P, _P, _I, _P],
    "epsb_expert_plans_noalloc": [_P, _P, _I, _I, _I, _I, _I, _I, _L, _P, _P, _P, _P, _P, _P, _I, _P],
    "epsb_fastep_expand_plan": [_P, _I, _I, _I, _P, _P, _P],
    "epsb_fastep_plan": [_P, _I, _I, _I, _P, _P, _P, _P, _P, _P, _P],
    "epsb_gather_rows": [_P, _P, _P, c_int32, c_int32, _P, _I, _I, _L, _L, _L, _P],
    "epsb_scatter_rows": [_P, _P, _P, c_int32, _L, _L, _P],
    "epsb_arrange_rows": [_P, _P, _P, _P, _P, _I, _L, _L, _P],
    "epsb_local_reduce_ref": [_P, _P, _P, _P, _P, _I, _I, _I, _I, _L, _L, _P, _P],
    "epsb_local_reduce": [_P, _P, _P, _I, _I, _I, _I, _L, _L, _P, _P],
    "epsb_global_reduce_ref": [_P, _P, _P, _P, _P, _I, _I, _L, _P, _P],
    "epsb_global_reduce": [_P, _P, _P, _P, _P, _I, _I, _L, _P, _P],
    "epsb_reduce_ep1": [_P, _P, _P, _P, _I, _P, _P, _P, _I, _I, _L, _P, _P],
    "epsb_fastep_reduce": [_P, _P, _P, _P, _P, _I, _I, _L, _P, _P],
    "epsb_silu_run": [_P, _P, _P, _I, _L, _L, _P],
    "epsb_grouped_gemm_fp8": [_I, _P, _P, _P, _P, _P, _I, _L, _L, _L, _P, _P, _P, _P, _I, _P],
    "epsb_rms_norm": [_P, _P, _P, c_float, _L, _L, _P],
    "epsb_router_topk_sigmoid": [_P, _I, _P, _I, _I, _I, _I, _I, c_float, _I, _P, _P, _P],
    "epsb_router_topk": [_I, _P, _I, _P, _I, _I, _I, _I, _I, c_float, _I, _P, _P, _P],
    "epsb_grouped_gemm_fp8_gather": [_I, _P, _P, _L, _P, _P, _P, _P, _I, _L, _L, _L, _P, _P, _P, _P, _I, _P],
    "epsb_gemm_row_sources": [_P, _P, _I, _I, _P, _I, _P, _L, _P, _P, _P],
    "epsb_grouped_gemm_bf16": [_P, _P, _P, _I, _L, _L, _L, _L, _P, _P, _I, _P],
    "epsb_gather_row_weights": [_P, _P, _P, _I, _L, _P, _P],
    "epsb_oep_arrange_plan": [_P, _L, _L, _I, _P, _P, _P, _P],
    "epsb_exchange_put_ids": [_P, _I, _P, _P, _P, _L, _P],
    "epsb_exchange_lookup_put": [_P, _I, _P, _L, _L, _P],
    "epsb_oep_scatter": [_P, _P, _L, _L, _L, _I, _P, _P],
    "epsb_tpdp_region_bytes": [_L, _L, _P],
    "epsb_tpdp_signal": [_P, _I, _I, _L, _L, _I, _I, _P],
    "epsb_tpdp_wait": [_P, _I, _L, _L, _I, _I, _P, _L, _P],
    "epsb_tpdp_all_gather_put": [_P, _I, _I, _L, _L, _L, _L, _I, _I, _P],
    "epsb_tpdp_reduce_scatter_sum": [_P, _I, _I, _L, _L, _L, _L, _I, _I, _P],
    "epsb_symm_alloc": [_L, _P, _P],
    "epsb_symm_open": [_P, _P],
    "epsb_symm_close": [_P],
    "epsb_symm_free": [_P],
    "epsb_exchange_region_bytes": [_I, _I, _I, _I, _L, _I, _I, _P],
    "epsb_exchange_create": [_I, _I, _I, _I, _I, _L, _I, _I, _P, _P],
    "epsb_exchange_destroy": [_P],
    "epsb_exchange_begin": [_P, _P],
    "epsb_exchange_arena": [_P, _I, _I, _P],
    "epsb_exchange_publish_plans": [_P, _P, _P, _I, _P],
    "epsb_exchange_recv_plans": [_P, _I, _P, _P, _L, _P],
    "epsb_exchange_put": [_P, _I, _I, _I, _P, _P, _P, _P, _P, _P, _I, _I, _P],
    "epsb_exchange_wait": [_P, _I, _P, _L, _P],
    "epsb_exchange_local_reduce_put": [_P, _I, _P, _P, _P, _I, _I, _L, _P],
}

_lib = None


class EpsError(RuntimeError):
    """Raised for any non-zero status of the C ABI (the reference throws std::runtime_error)."""


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise EpsError(
                f"{LIB_PATH} is missing: build it with `python -m eps_b200.build` "
                "(this package has no CPU or PyTorch fallback)")
        handle = ctypes.CDLL(LIB_PATH)
        handle.epsb_last_error.restype = c_char_p
        handle.epsb_last_error.argtypes = []
        handle.epsb_version.restype = c_int
        handle.epsb_version.argtypes = []
        for name, args in SIGNATURES.items():
            fn = getattr(handle, name)
            fn.restype = c_int
            fn.argtypes = args
        _lib = handle
    return _lib


def ptr(t) -> int | None:
    """Device (or host) address of a torch tensor, None for None."""
    if t is None:
        return None
    return t.data_ptr()


def stream_ptr(stream=None) -> int:
    import torch

    s = stream if stream is not None else torch.cuda.current_stream()
    return s.cuda_stream


def call(name: str, *args) -> None:
    h = lib()
    rc = getattr(h, name)(*args)
    if rc != 0:
        raise EpsError(f"{name}: {h.epsb_last_error().decode()} (code {rc})")
