"""Row movement, reductions and SwiGLU against numpy / the oracle."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _bits(t):
    return t.view(torch.int16).cpu().numpy().view(np.uint16)


def _dev(a, cuda):
    return torch.from_numpy(np.ascontiguousarray(a)).to(cuda)


@pytest.mark.parametrize("rows,row_bytes", [(1, 16), (7, 32), (100, 7168), (64, 224), (33, 14336), (5, 4096 + 16), (9, 8), (50, 12), (31, 48 + 4)])
def test_gather_rows(cuda, rows, row_bytes):
    from eps_b200 import ops

    rng = np.random.default_rng(rows)
    T = rows + 3
    src = rng.integers(0, 256, (T, row_bytes), dtype=np.uint8)
    mapping = rng.integers(0, 4 * T, rows).astype(np.int32)  # ep*T + src style markers
    dst = torch.zeros((rows, row_bytes), dtype=torch.uint8, device=cuda)
    ops.gather_rows(_dev(src, cuda), dst, _dev(mapping, cuda), map_div=1, map_mod=T)
    assert np.array_equal(dst.cpu().numpy(), src[mapping % T])
    # expand-for-gemm form: mapping = row*k + slot, window from a prefix sum
    k = 4
    m2 = (rng.integers(0, T, rows) * k + rng.integers(0, k, rows)).astype(np.int32)
    bounds = np.array([0, rows // 3, rows // 3, rows], dtype=np.int32)
    dst2 = torch.full((rows, row_bytes), 0x55, dtype=torch.uint8, device=cuda)
    ops.gather_rows(_dev(src, cuda), dst2, _dev(m2, cuda), map_div=k, bounds=_dev(bounds, cuda), b0=1, b1=3)
    want = np.full((rows, row_bytes), 0x55, dtype=np.uint8)
    want[rows // 3:] = src[m2[rows // 3:] // k]
    assert np.array_equal(dst2.cpu().numpy(), want)


def test_scatter_and_arrange(cuda):
    from eps_b200 import ops

    rng = np.random.default_rng(3)
    T, k, rb = 50, 3, 512
    src = rng.integers(0, 256, (T, rb), dtype=np.uint8)
    perm = rng.permutation(T * k).astype(np.int32)
    zc = rng.random(T * k) < 0.2
    mapping = np.where(zc, 1000000 + np.arange(T * k) // k, perm).astype(np.int32)
    dst = torch.zeros((T * k, rb), dtype=torch.uint8, device=cuda)
    ops.scatter_rows(_dev(src, cuda), dst, _dev(mapping, cuda), k, T * k)
    want = np.zeros((T * k, rb), dtype=np.uint8)
    for i in range(T * k):
        if mapping[i] < 1000000:
            want[mapping[i]] = src[i // k]
    assert np.array_equal(dst.cpu().numpy(), want)
    # arrange: segments
    rows = np.array([3, 0, 10, 1, 7], dtype=np.int32)
    src_off = np.concatenate([[0], np.cumsum(rows)[:-1]]).astype(np.int32)
    order = np.array([2, 0, 4, 1, 3])
    dst_off = np.zeros(5, dtype=np.int32)
    acc = 0
    for p in order:
        dst_off[p] = acc
        acc += rows[p]
    a = rng.integers(0, 256, (rows.sum(), rb), dtype=np.uint8)
    out = torch.zeros((rows.sum(), rb), dtype=torch.uint8, device=cuda)
    ops.arrange_rows(_dev(a, cuda), out, _dev(src_off, cuda), _dev(rows, cuda), _dev(dst_off, cuda), 5, int(rows.sum()))
    want = np.zeros_like(a)
    for p in range(5):
        want[dst_off[p]:dst_off[p] + rows[p]] = a[src_off[p]:src_off[p] + rows[p]]
    assert np.array_equal(out.cpu().numpy(), want)


@pytest.mark.parametrize("T,k,H,shared", [(5, 2, 256, False), (64, 8, 7168, True), (33, 12, 6144, False), (1, 1, 128, True)])
def test_fastep_reduce_bit_exact(cuda, oracle, T, k, H, shared):
    from eps_b200 import ops

    rng = np.random.default_rng(T + k)
    rows = oracle.bf16_bits(rng.standard_normal((T * k, H)).astype(np.float32))
    raw = oracle.bf16_bits(rng.standard_normal((T, H)).astype(np.float32))
    sh = oracle.bf16_bits(rng.standard_normal((T, H)).astype(np.float32)) if shared else None
    w = rng.random((T, k)).astype(np.float32)
    mapping = rng.permutation(T * k).astype(np.int32)
    zc = rng.random(T * k) < 0.25
    mapping = np.where(zc, 1000000 + np.arange(T * k) // k, mapping).astype(np.int32)
    out = torch.empty((T, H), dtype=torch.bfloat16, device=cuda)
    ops.fastep_reduce(_dev(rows.view(np.int16), cuda).view(torch.bfloat16), _dev(raw.view(np.int16), cuda).view(torch.bfloat16),
                      _dev(w, cuda), _dev(mapping, cuda), out,
                      shared=None if sh is None else _dev(sh.view(np.int16), cuda).view(torch.bfloat16))
    want = oracle.fastep_reduce(rows, raw, w, mapping, sh)
    assert np.array_equal(_bits(out), want)


def _local_reduce_case(rng, R, k, H, W, S):
    D = R * 2
    red_map = np.full((R, k), R * k, dtype=np.int32)
    perm = rng.permutation(D)
    p = 0
    for q in range(R):
        n = rng.integers(1, min(k, 2) + 1)
        for j in rng.choice(k, n, replace=False):
            red_map[q, j] = perm[p]
            p += 1
    cuts = np.sort(rng.integers(0, R + 1, W * S - 1))
    ret_incl = np.concatenate([cuts, [R]]).astype(np.int32)
    return D, red_map, ret_incl


@pytest.mark.parametrize("R,k,H,W,S", [(10, 4, 256, 2, 2), (200, 8, 7168, 4, 1), (37, 6, 2048, 1, 4)])
def test_local_reduce_fp32(cuda, oracle, R, k, H, W, S):
    from eps_b200 import ops

    rng = np.random.default_rng(R)
    D, red_map, ret_incl = _local_reduce_case(rng, R, k, H, W, S)
    y = torch.randn((D, H), generator=torch.Generator().manual_seed(R)).to(torch.bfloat16)
    yf = y.float().numpy()
    want = np.zeros((R, H), dtype=np.float32)
    for q in range(R):
        acc = np.zeros(H, dtype=np.float32)
        for j in range(k):
            if red_map[q, j] < R * k:
                acc = acc + yf[red_map[q, j]]
        want[q] = acc
    want_bits = oracle.bf16_bits(want)
    # all stages at once
    send = torch.zeros((R, H), dtype=torch.bfloat16, device=cuda)
    ops.local_reduce(y.to(cuda), _dev(red_map, cuda), _dev(ret_incl, cuda), k, W, S, -1, send)
    assert np.array_equal(_bits(send), want_bits)
    # stage by stage: each stage writes only its windows
    send2 = torch.zeros((R, H), dtype=torch.bfloat16, device=cuda)
    for st in range(S):
        ops.local_reduce(y.to(cuda), _dev(red_map, cuda), _dev(ret_incl, cuda), k, W, S, st, send2)
        done = np.zeros(R, dtype=bool)
        for d in range(W):
            for s2 in range(st + 1):
                i = d * S + s2
                b = 0 if i == 0 else ret_incl[i - 1]
                done[b:ret_incl[i]] = True
        got = _bits(send2)
        assert np.array_equal(got[done], want_bits[done])
        assert np.all(got[~done] == 0)


def test_local_reduce_ref_arithmetic(cuda, oracle):
    """bf16 multiply / bf16 accumulate like the reference kernel: within 2 bf16 ulp of the
    unfused restatement (the reference leaves mul+add contraction to the compiler)."""
    from eps_b200 import ops

    R, k, H, W, S = 50, 8, 2048, 2, 1
    rng = np.random.default_rng(4)
    D, red_map, ret_incl = _local_reduce_case(rng, R, k, H, W, S)
    y = torch.randn((D, H), generator=torch.Generator().manual_seed(1)).to(torch.bfloat16)
    w = torch.rand((R, k), generator=torch.Generator().manual_seed(2))
    scale_map = rng.permutation(R).astype(np.int32)
    send = torch.zeros((R, H), dtype=torch.bfloat16, device=cuda)
    ops.local_reduce_ref(y.to(cuda), w.to(cuda), _dev(scale_map, cuda), _dev(red_map, cuda), _dev(ret_incl, cuda), k,
                         W, S, -1, send)
    acc = torch.zeros((R, H), dtype=torch.bfloat16)
    for q in range(R):
        for j in range(k):
            if red_map[q, j] < R * k:
                prod = y[red_map[q, j]] * w[scale_map[q], j].to(torch.bfloat16)
                acc[q] = acc[q] + prod
    diff = (send.cpu().float() - acc.float()).abs()
    tol = acc.float().abs() * 2.0 ** -7 + 1e-6
    assert bool((diff <= tol).all())


@pytest.mark.parametrize("T,W,H,shared,zero", [(9, 2, 256, False, False), (130, 8, 7168, True, True), (40, 4, 4096, False, True), (7, 20, 512, True, True)])
def test_global_reduce(cuda, oracle, T, W, H, shared, zero):
    from eps_b200 import ops

    rng = np.random.default_rng(T * W)
    n_recv = T * 2
    glob = np.full((T, W), T * W, dtype=np.int32)
    perm = rng.permutation(n_recv)
    p = 0
    for t in range(T):
        for ep in rng.choice(W, rng.integers(0, min(W, 2) + 1), replace=False):
            glob[t, ep] = perm[p]
            p += 1
    recv = torch.randn((n_recv, H), generator=torch.Generator().manual_seed(T)).to(torch.bfloat16)
    x = torch.randn((T, H), generator=torch.Generator().manual_seed(T + 1)).to(torch.bfloat16)
    sh = torch.randn((T, H), generator=torch.Generator().manual_seed(T + 2)).to(torch.bfloat16) if shared else None
    zs = torch.rand((T,), generator=torch.Generator().manual_seed(T + 3)) if zero else None
    out = torch.empty((T, H), dtype=torch.bfloat16, device=cuda)
    ops.global_reduce(recv.to(cuda), _dev(glob, cuda), out, W, shared=None if sh is None else sh.to(cuda),
                      x=x.to(cuda), zero_scale=None if zs is None else zs.to(cuda))
    want = np.zeros((T, H), dtype=np.float32)
    rf = recv.float().numpy()
    for t in range(T):
        acc = np.zeros(H, dtype=np.float32)
        for ep in range(W):
            if glob[t, ep] < T * W:
                acc = acc + rf[glob[t, ep]]
        if shared:
            acc = acc + sh[t].float().numpy()
        if zero:
            acc = (x[t].float().numpy().astype(np.float64) * np.float64(zs[t].item()) + acc.astype(np.float64))
            acc = acc.astype(np.float32)  # fma: one rounding
        want[t] = acc
    assert np.array_equal(_bits(out), oracle.bf16_bits(want))
    # reference-arithmetic variant: bf16 adds; compare with the same sequence in torch bf16
    out2 = torch.empty((T, H), dtype=torch.bfloat16, device=cuda)
    ops.global_reduce(recv.to(cuda), _dev(glob, cuda), out2, W, shared=None if sh is None else sh.to(cuda),
                      x=x.to(cuda), zero_scale=None if zs is None else zs.to(cuda), ref_arith=True)
    acc = torch.zeros((T, H), dtype=torch.bfloat16)
    for t in range(T):
        for ep in range(W):
            if glob[t, ep] < T * W:
                acc[t] = acc[t] + recv[glob[t, ep]]
        if shared:
            acc[t] = sh[t] + acc[t]
        if zero:
            acc[t] = acc[t] + (x[t].float() * zs[t]).to(torch.bfloat16)
    assert torch.equal(out2.cpu(), acc)


@pytest.mark.parametrize("rows,I", [(3, 128), (50, 1408), (129, 2048)])
def test_silu(cuda, rows, I):
    from eps_b200 import ops

    gu = torch.randn((rows, 2 * I), generator=torch.Generator().manual_seed(rows)).to(torch.bfloat16)
    out = torch.zeros((rows, I), dtype=torch.bfloat16, device=cuda)
    excl = torch.tensor([1, rows - 1], dtype=torch.int32, device=cuda)
    ops.silu_run(gu.to(cuda), out, excl, 1)
    g, u = gu[:, :I].float(), gu[:, I:].float()
    want = ((g / (1 + torch.exp(-g))) * u)
    got = out.cpu().float()
    assert torch.all(got[0] == 0) and torch.all(got[-1] == 0)
    # __expf is within a few ulp of expf; one bf16 ulp of slack
    assert bool(((got[1:-1] - want[1:-1]).abs() <= want[1:-1].abs() * 2.0 ** -7 + 1e-30).all())


@pytest.mark.parametrize("T,k,H,S,shared,zero", [(40, 4, 512, 2, True, True), (300, 8, 7168, 1, False, False), (9, 12, 256, 3, True, False)])
def test_reduce_ep1_matches_two_pass_semantics(cuda, oracle, T, k, H, S, shared, zero):
    """World of one: the fused pass equals sum over the token's GEMM rows (+shared, +x*zero_scale) in fp32."""
    from eps_b200 import ops

    rng = np.random.default_rng(T + k)
    R = T - 2                         # two tokens have only identity experts: no return row
    D = R * 2
    red_map = np.full((R, k), R * k, dtype=np.int32)
    perm = rng.permutation(D)
    p = 0
    for q in range(R):
        for j in rng.choice(k, rng.integers(1, min(k, 2) + 1), replace=False):
            red_map[q, j] = perm[p]
            p += 1
    ret_incl = np.sort(np.concatenate([rng.integers(0, R + 1, S - 1), [R]])).astype(np.int32)
    glob = np.full(T, T, dtype=np.int32)
    toks = rng.permutation(T)[:R]
    glob[toks] = np.arange(R)
    y = torch.randn((D, H), generator=torch.Generator().manual_seed(T)).to(torch.bfloat16)
    x = torch.randn((T, H), generator=torch.Generator().manual_seed(T + 1)).to(torch.bfloat16)
    sh = torch.randn((T, H), generator=torch.Generator().manual_seed(T + 2)).to(torch.bfloat16) if shared else None
    zs = torch.rand((T,), generator=torch.Generator().manual_seed(T + 3)) if zero else None
    out = torch.empty((T, H), dtype=torch.bfloat16, device=cuda)
    ops.reduce_ep1(y.to(cuda), _dev(red_map, cuda), _dev(glob, cuda), _dev(ret_incl, cuda), S, k, out,
                   shared=None if sh is None else sh.to(cuda), x=x.to(cuda), zero_scale=None if zs is None else zs.to(cuda))
    yf = y.float().numpy()
    want = np.zeros((T, H), dtype=np.float32)
    for t in range(T):
        acc = np.zeros(H, dtype=np.float32)
        if glob[t] < T:
            for j in range(k):
                if red_map[glob[t], j] < R * k:
                    acc = acc + yf[red_map[glob[t], j]]
        if shared:
            acc = acc + sh[t].float().numpy()
        if zero:
            acc = (x[t].float().numpy().astype(np.float64) * np.float64(zs[t].item()) + acc.astype(np.float64)).astype(np.float32)
        want[t] = acc
    assert np.array_equal(_bits(out), oracle.bf16_bits(want))
