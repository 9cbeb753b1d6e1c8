"""rms_norm of bf16 rows against the CPU oracle and against the reference's own kernel on the GPU.

The three implementations sum the squares in different orders, so 1/rms may differ in the last place of fp32 and an
output may land on the neighbouring bf16 value: the bound is one bf16 ulp, with nearly all outputs identical."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _bits(t):
    return t.view(torch.int16).cpu().numpy().view(np.uint16)


def _close(a_bits, b_bits, oracle):
    a, b = oracle.bf16_to_f32(a_bits), oracle.bf16_to_f32(b_bits)
    assert np.all(np.abs(a - b) <= np.abs(b) * 2.0 ** -7 + 1e-30)
    assert np.mean(a_bits == b_bits) > 0.98


@pytest.mark.parametrize("m,n", [(1, 2), (7, 64), (33, 1030), (64, 2048), (16, 7168), (5, 16384), (3, 16400), (4, 20480)])
def test_rms_norm_vs_oracle_and_reference(cuda, oracle, m, n):
    from eps_b200 import ops
    from oracle import ref_kernels

    g = torch.Generator().manual_seed(m * 131 + n)
    x = (torch.randn((m, n), generator=g) * 3).to(torch.bfloat16)
    sc = (1 + 0.1 * torch.randn(n, generator=g)).to(torch.bfloat16)
    out = ops.rms_norm(x.to(cuda), sc.to(cuda), 1e-6)
    torch.cuda.synchronize()
    _close(_bits(out), oracle.rms_norm(_bits(x), _bits(sc), 1e-6), oracle)
    if ref_kernels.available():
        ref = ref_kernels.rms_norm(x.to(cuda), sc.to(cuda), 1e-6)
        assert ref is not None
        _close(_bits(out), _bits(ref), oracle)


def test_rms_norm_zero_rows_and_errors(cuda):
    from eps_b200 import ops
    from eps_b200._lib import EpsError

    sc = torch.ones(8, dtype=torch.bfloat16, device=cuda)
    x = torch.zeros((2, 8), dtype=torch.bfloat16, device=cuda)
    assert torch.equal(ops.rms_norm(x, sc, 1e-6), x)              # 0 * rsqrt(eps) = 0
    assert ops.rms_norm(x[:0], sc, 1e-6).shape == (0, 8)
    with pytest.raises(EpsError, match="not divisible by 2"):
        ops.rms_norm(torch.zeros((2, 7), dtype=torch.bfloat16, device=cuda), sc[:7].contiguous(), 1e-6)
