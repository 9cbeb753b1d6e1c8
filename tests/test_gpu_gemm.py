"""tcgen05 FP8 block-scaled grouped GEMM against the fp32 dequantised oracle."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _dev(a, cuda):
    return torch.from_numpy(np.ascontiguousarray(a)).to(cuda)


def _make(oracle, rng, rows_per_expert, N, K, pad_rows=5):
    E = len(rows_per_expert)
    excl = np.zeros(E + 1, dtype=np.int32)
    excl[1:] = np.cumsum(rows_per_expert)
    D = int(excl[-1])
    max_rows = D + pad_rows
    a = oracle.bf16_bits(rng.standard_normal((max_rows, K)).astype(np.float32))
    A, a_s = oracle.quant_1x128(a)
    w = (rng.standard_normal((E, N, K)) * 0.02).astype(np.float32)
    w = oracle.bf16_to_f32(oracle.bf16_bits(w))
    B, b_s = oracle.quant_block128(w)
    return excl, D, max_rows, A, a_s, B, b_s


def _check_status(status):
    st = status.cpu().tolist()
    assert st[0] == 0, f"bounded wait expired in the GEMM kernel: code {st[0]} on CTA {st[1]}"


GEMM_CASES = [
    ([128], 256, 128),
    ([1], 256, 256),
    ([130, 0, 7], 256, 512),
    ([64] * 16, 2048, 1408 - 1408 % 128),
    ([300, 5, 0, 129, 128, 1, 77, 256], 512, 2048),
    # tail tiles (remainders of 1..64 rows run with the operand roles swapped), N % 256 == 128
    ([129, 160, 33, 64, 65, 32, 193, 31], 384, 256),
]


@pytest.mark.parametrize("rows,N,K", GEMM_CASES)
def test_gemm_plain(cuda, oracle, rows, N, K):
    from eps_b200 import ops

    rng = np.random.default_rng(N + K + len(rows))
    excl, D, max_rows, A, a_s, B, b_s = _make(oracle, rng, rows, N, K)
    status = torch.zeros(4, dtype=torch.int32, device=cuda)
    C = torch.full((max_rows, N), 7.0, dtype=torch.bfloat16, device=cuda)
    ops.grouped_gemm_fp8(ops.GEMM_PLAIN, _dev(A, cuda), _dev(a_s, cuda), _dev(B, cuda), _dev(b_s, cuda),
                         _dev(excl, cuda), out=C, status=status)
    torch.cuda.synchronize()
    _check_status(status)
    want = oracle.grouped_gemm_fp8(A, a_s, B, b_s, excl)
    got = C.float().cpu().numpy()
    rms = np.sqrt(np.mean(want[:D] ** 2)) if D else 1.0
    # bf16 output rounding (2^-9 relative) + fp32 summation-order differences; tolerance stated vs RMS
    # fp32 summation-order differences (vs RMS) plus the bf16 rounding of the output itself (2^-8 relative)
    assert np.all(np.abs(got[:D] - want[:D]) <= 2e-2 * rms + 2.0 ** -8 * np.abs(want[:D]))
    assert np.max(np.abs(got[:D] - want[:D]) / (np.abs(want[:D]) + rms)) <= 2 ** -7
    assert np.all(got[D:] == 7.0), "rows outside every expert must not be written"


@pytest.mark.parametrize("rows,I,K", [([128], 128, 128), ([5, 140], 256, 512), ([64] * 16, 1408 - 1408 % 128, 2048),
                                       ([200, 0, 3, 131], 2048, 1024),
                                       ([129, 160, 33, 64, 65, 32, 193, 31, 0, 16], 256, 384)])
def test_gemm_gateup_swiglu_requant(cuda, oracle, rows, I, K):
    from eps_b200 import ops

    rng = np.random.default_rng(I + K)
    excl, D, max_rows, A, a_s, B, b_s = _make(oracle, rng, rows, 2 * I, K)
    status = torch.zeros(4, dtype=torch.int32, device=cuda)
    q = torch.full((max_rows, I), 0xAA, dtype=torch.uint8, device=cuda)
    s = torch.full((max_rows, I // 128), -1.0, dtype=torch.float32, device=cuda)
    ops.grouped_gemm_fp8(ops.GEMM_GATEUP, _dev(A, cuda), _dev(a_s, cuda), _dev(B, cuda), _dev(b_s, cuda),
                         _dev(excl, cuda), out=q, out_scales=s, status=status)
    torch.cuda.synchronize()
    _check_status(status)
    act = oracle.swiglu(oracle.grouped_gemm_fp8(A, a_s, B, b_s, excl))
    gq, gs = q.cpu().numpy(), s.cpu().numpy()
    assert np.all(gq[D:] == 0xAA) and np.all(gs[D:] == -1.0)
    deq = oracle.e4m3_table()[gq[:D]] * np.repeat(gs[:D], 128, axis=1)
    rms = np.sqrt(np.mean(act[:D] ** 2))
    # the requantised activation carries half an e4m3 ulp (2^-4 of the group amax) of error by design
    amax = np.abs(act[:D]).reshape(D, I // 128, 128).max(-1)
    assert np.all(np.abs(gs[:D] - amax / 448.0) <= np.abs(amax / 448.0) * 1e-3 + 1e-12)
    bound = np.repeat(amax, 128, axis=1) * (2.0 ** -4) * 1.05 + 1e-3 * rms
    assert np.all(np.abs(deq - act[:D]) <= bound)


@pytest.mark.parametrize("rows,N,K", [([128], 256, 128), ([9, 250, 0, 40], 512, 1408 - 1408 % 128),
                                       ([130, 64, 33, 1, 161], 384, 256)])
def test_gemm_down_weighted(cuda, oracle, rows, N, K):
    from eps_b200 import ops

    rng = np.random.default_rng(N * 3 + K)
    excl, D, max_rows, A, a_s, B, b_s = _make(oracle, rng, rows, N, K)
    row_w = rng.random(max_rows).astype(np.float32)
    status = torch.zeros(4, dtype=torch.int32, device=cuda)
    C = ops.grouped_gemm_fp8(ops.GEMM_DOWN, _dev(A, cuda), _dev(a_s, cuda), _dev(B, cuda), _dev(b_s, cuda),
                             _dev(excl, cuda), row_w=_dev(row_w, cuda), status=status)
    torch.cuda.synchronize()
    _check_status(status)
    want = oracle.grouped_gemm_fp8(A, a_s, B, b_s, excl) * row_w[:, None]
    got = C.float().cpu().numpy()
    rms = np.sqrt(np.mean(want[:D] ** 2))
    # fp32 summation-order differences (vs RMS) plus the bf16 rounding of the output itself (2^-8 relative)
    assert np.all(np.abs(got[:D] - want[:D]) <= 2e-2 * rms + 2.0 ** -8 * np.abs(want[:D]))
    assert np.max(np.abs(got[:D] - want[:D]) / (np.abs(want[:D]) + rms)) <= 2 ** -7


def test_gemm_sm_count_limit(cuda, oracle):
    """The sm_count argument (the sm_count of the reference's aok_create) changes the grid, not the result."""
    from eps_b200 import ops
    from eps_b200._lib import EpsError

    rng = np.random.default_rng(5)
    excl, D, max_rows, A, a_s, B, b_s = _make(oracle, rng, [200, 17, 0, 129], 512, 256)
    args = (_dev(A, cuda), _dev(a_s, cuda), _dev(B, cuda), _dev(b_s, cuda), _dev(excl, cuda))
    status = torch.zeros(4, dtype=torch.int32, device=cuda)
    full = ops.grouped_gemm_fp8(ops.GEMM_PLAIN, *args, status=status)
    few = ops.grouped_gemm_fp8(ops.GEMM_PLAIN, *args, status=status, sm_count=3)
    torch.cuda.synchronize()
    _check_status(status)
    assert torch.equal(full[:D], few[:D])
    with pytest.raises(EpsError):
        ops.grouped_gemm_fp8(ops.GEMM_PLAIN, *args, status=status, sm_count=-1)


def test_gemm_errors(cuda):
    from eps_b200 import ops
    from eps_b200._lib import EpsError

    A = torch.zeros((4, 100), dtype=torch.uint8, device=cuda)
    with pytest.raises(EpsError):
        ops.grouped_gemm_fp8(ops.GEMM_PLAIN, A, torch.zeros((4, 1), device=cuda), torch.zeros((1, 128, 100), dtype=torch.uint8, device=cuda),
                             torch.zeros((1, 1, 1), device=cuda), torch.zeros(2, dtype=torch.int32, device=cuda))


@pytest.mark.parametrize("pairs", [False, True])
@pytest.mark.parametrize("rows,N,K", [([200, 17, 0, 129], 512, 256), ([1, 128, 300], 384, 192), ([64] * 8, 1024, 2048),
                                      ([700], 256, 64), ([300, 257, 256, 1, 0, 511], 512, 256),
                                      ([1024, 1000, 1030], 256, 128)])
def test_grouped_gemm_bf16_vs_fp32_reference(cuda, rows, N, K, pairs):
    """The bf16 grouped GEMM (the reference's aok_run) against a plain fp32 matmul of the same bf16 operands: fp32
    accumulation and one rounding on both sides, so the results agree to one bf16 ulp (summation order differs).
    pairs: the row hint promises experts large enough for 256-row tiles on CTA pairs (cta_group::2); N % 256 != 0
    keeps single CTAs either way."""
    from eps_b200 import ops

    g = torch.Generator().manual_seed(len(rows) * 1000 + N)
    E, D = len(rows), sum(rows)
    max_rows = max(D + 5, E * 512) if pairs else D + 5
    excl = torch.tensor([0] + list(np.cumsum(rows)), dtype=torch.int32, device=cuda)
    A = torch.randn((max_rows, K), generator=g).to(torch.bfloat16).to(cuda)
    B = (torch.randn((E, N, K), generator=g) * 0.05).to(torch.bfloat16).to(cuda)
    status = torch.zeros(4, dtype=torch.int32, device=cuda)
    out = torch.full((max_rows, N), 7.0, dtype=torch.bfloat16, device=cuda)
    ops.grouped_gemm_bf16(A, B, excl, out=out, status=status, rows_hint=max_rows if pairs else 1)
    torch.cuda.synchronize()
    _check_status(status)
    ex = excl.cpu().numpy()
    for e in range(E):
        a, b = int(ex[e]), int(ex[e + 1])
        if b == a:
            continue
        want = A[a:b].float() @ B[e].float().t()
        got = out[a:b].float()
        assert torch.all((got - want).abs() <= 2.0 ** -8 * want.abs() + 1e-3), f"expert {e}"
    assert torch.all(out[D:] == 7.0)   # rows outside every expert are not touched


@pytest.mark.parametrize("mode", ["plain", "gateup", "down"])
@pytest.mark.parametrize("rows", [[128], [130, 0, 7, 33, 64, 65, 200], [64] * 5 + [129, 1, 257]])
def test_gemm_index_driven_a_loads_equal_a_gathered_copy(cuda, oracle, rows, mode):
    """GEMM row m read through a_rows[m] from a source matrix (TMA gather4 in the kernel) gives bit for bit what the
    same kernel gives on a pre-gathered copy of those rows; rows may repeat (a token routed to several experts)."""
    from eps_b200 import ops

    rng = np.random.default_rng(len(rows) * 7 + len(mode))
    N, K = (512, 384) if mode != "gateup" else (512, 256)
    E, D = len(rows), int(sum(rows))
    excl = np.zeros(E + 1, dtype=np.int32)
    excl[1:] = np.cumsum(rows)
    S = 97                                                   # source rows: fewer than GEMM rows, so they repeat
    src = oracle.bf16_bits(rng.standard_normal((S, K)).astype(np.float32))
    A_src, as_src = oracle.quant_1x128(src)
    a_rows = rng.integers(0, S, size=D + 3).astype(np.int32)
    w = oracle.bf16_to_f32(oracle.bf16_bits((rng.standard_normal((E, N, K)) * 0.02).astype(np.float32)))
    B, b_s = oracle.quant_block128(w)
    d = lambda t: _dev(t, cuda)
    m = {"plain": ops.GEMM_PLAIN, "gateup": ops.GEMM_GATEUP, "down": ops.GEMM_DOWN}[mode]
    row_w = d(rng.random(D + 3).astype(np.float32)) if mode == "down" else None
    status = torch.zeros(4, dtype=torch.int32, device=cuda)
    got = ops.grouped_gemm_fp8(m, d(A_src), d(as_src), d(B), d(b_s), d(excl), row_w=row_w, status=status,
                               a_rows=d(a_rows))
    want = ops.grouped_gemm_fp8(m, d(A_src[a_rows]), d(as_src[a_rows]), d(B), d(b_s), d(excl), row_w=row_w,
                                status=status)
    torch.cuda.synchronize()
    _check_status(status)
    if mode == "gateup":
        assert torch.equal(got[0][:D], want[0][:D]) and torch.equal(got[1][:D], want[1][:D])
    else:
        assert torch.equal(got[:D], want[:D])
