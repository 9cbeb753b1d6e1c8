"""Checks rows of an MoE-layer output against the CPU oracle on a seeded sample of tokens.

TEST INFRASTRUCTURE ONLY (like everything under oracle/): used by the GPU tests and by bench.py's parity block,
outside every timed region.  A full-size layer (hundreds of experts, thousands of tokens) is far too much for the
fp32 oracle as a whole; a sample of tokens needs only the experts those tokens route to, each asked for once.

Two ratios are reported for the same errors:
  worst_ratio       max |got - want| / (2e-2 x RMS(want))                     the layer's arithmetic tolerance as stated
  worst_ratio_bf16  max |got - want| / (2e-2 x RMS(want) + n x 2^-9 x mag)    the same plus half an ulp of bf16 for every
                                                                              time a value is STORED as bf16 on its way;
                                                                              mag = sum of |terms| of the element >= |want|
n = 2 in a world of one (the down GEMM's weighted row, the output) and 3 with expert parallelism (the rank's partial row
crosses the link as bf16 too) - the stores the reference's own path has (GEMM output, localReduce output, output).
A CPU emulation that rounds exact fp32 values at just those three points reaches worst_ratio 2.0 on the decode
configuration at EP8 (elements of 6 x RMS), so the format's own rounding cannot be charged to the kernels.
`ok` is worst_ratio_bf16 <= 1.
"""
from __future__ import annotations

import numpy as np

from . import oracle as orc


def sample_tokens(num_tokens: int, n: int, seed: int) -> np.ndarray:
    """Sorted seeded sample of min(n, num_tokens) distinct token ids."""
    rng = np.random.default_rng(seed)
    n = min(n, num_tokens)
    return np.sort(rng.choice(num_tokens, size=n, replace=False)) if n > 0 else np.zeros(0, dtype=np.int64)


def check_rows(x_bits, idx, w, got_rows, expert_weights, shared=None, rms_rows=None, bf16_stores=2):
    """x_bits [n,H] uint16 (bf16 bits), idx [n,k] int32, w [n,k] fp32: the sampled tokens; got_rows [n,H] fp32: the
    layer's output rows for them.  expert_weights(e) as in oracle.moe_layer_fp32_sampled.  RMS is taken over the
    oracle's rows (a sample of >= 64 rows x thousands of columns estimates the full output's RMS to well under 1 %)."""
    want, mag = orc.moe_layer_fp32_sampled(x_bits, idx, w, expert_weights, shared=shared, return_magnitude=True)
    got = np.asarray(got_rows, dtype=np.float32)
    n = want.shape[0]
    if n == 0:
        return {"checked_tokens": 0, "worst_ratio": 0.0, "worst_ratio_bf16": 0.0, "ok": True}
    rms = float(np.sqrt(np.mean(want.astype(np.float64) ** 2)))
    err = np.abs(got - want)
    finite = bool(np.isfinite(got).all())
    strict = float(np.max(err) / (2e-2 * rms)) if rms > 0 else float(np.max(err) > 0)
    amended = float(np.max(err / (2e-2 * rms + bf16_stores * 2.0 ** -9 * mag))) if rms > 0 else strict
    return {"checked_tokens": int(n), "worst_ratio": strict, "worst_ratio_bf16": amended, "rms": rms,
            "bf16_stores": int(bf16_stores), "ok": bool(finite and amended <= 1.0)}
