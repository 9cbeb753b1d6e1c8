"""The TORCH_LIBRARY registration (libexecutor_.so): op names and schemas of the reference's `executor` namespace."""
import numpy as np
import pytest
import torch


@pytest.fixture(scope="module")
def ex_ops():
    from eps_b200 import build

    build.build_torch_ops()
    return build.load_torch_ops()


def test_ops_are_registered_with_reference_names(ex_ops):
    for name in ("aok_create", "aok_get_workspace_size", "aok_run", "aok_destroy", "silu_run", "aok_run_fp8",
                 "per_token_group_quant_fp8"):
        assert hasattr(ex_ops, name), name
    h = ex_ops.aok_create(8, 148)
    assert h != 0 and ex_ops.aok_get_workspace_size(h, 7168, 4096) == 0
    # reference schema of aok_run: (int ptr, Tensor A, Tensor B, Tensor C, Tensor exclusive_sum, int hint, int max, Tensor ws)
    schema = str(torch.ops.executor.aok_run.default._schema)
    assert schema.count("Tensor") == 5 and schema.count("int") >= 3
    with pytest.raises(RuntimeError, match="not part of this build"):
        t = torch.zeros(1)
        ex_ops.aok_run(h, t, t, t, t, 0, 0, t)
    ex_ops.aok_destroy(h)
    # the router sits in the reference's `utils` library (src/utils/bindings/bindings.cpp:6-9) with ten arguments
    schema = str(torch.ops.utils.topk_sigmoid.default._schema)
    assert schema.count("Tensor") == 4 and schema.count("int") == 5 and "float" in schema


@pytest.mark.gpu
def test_torch_ops_run_on_gpu(cuda, oracle, ex_ops):
    from eps_b200 import ops

    x = torch.randn((64, 512), generator=torch.Generator().manual_seed(1)).to(torch.bfloat16).to(cuda)
    q = torch.empty((64, 512), dtype=torch.uint8, device=cuda)
    s = torch.empty((64, 4), dtype=torch.float32, device=cuda)
    ex_ops.per_token_group_quant_fp8(x, q, s, 1)
    q2, s2 = ops.per_token_group_quant_fp8(x)
    assert torch.equal(q, q2) and torch.equal(s, s2)
    gu = torch.randn((40, 512), generator=torch.Generator().manual_seed(2)).to(torch.bfloat16).to(cuda)
    excl = torch.tensor([0, 40], dtype=torch.int32, device=cuda)
    r1 = torch.zeros((40, 256), dtype=torch.bfloat16, device=cuda)
    r2 = torch.zeros_like(r1)
    ex_ops.silu_run(gu, r1, excl, 40)
    ops.silu_run(gu, r2, excl, 1)
    assert torch.equal(r1, r2)
    rng = np.random.default_rng(0)
    a = oracle.bf16_bits(rng.standard_normal((100, 256)).astype(np.float32))
    A, a_s = oracle.quant_1x128(a)
    wq, w_s = oracle.quant_block128((rng.standard_normal((2, 256, 256)) * 0.02).astype(np.float32))
    ex = np.array([0, 60, 100], dtype=np.int32)
    dv = lambda t: torch.from_numpy(np.ascontiguousarray(t)).to(cuda)
    C = torch.zeros((100, 256), dtype=torch.bfloat16, device=cuda)
    h = ex_ops.aok_create(2, 148)
    ex_ops.aok_run_fp8(h, dv(A), dv(a_s), dv(wq), dv(w_s), C, dv(ex), 100, 100, torch.zeros((1, 1), dtype=torch.uint8, device=cuda))
    ex_ops.aok_destroy(h)
    want = oracle.grouped_gemm_fp8(A, a_s, wq, w_s, ex)
    assert np.max(np.abs(C.float().cpu().numpy() - want)) <= 2e-2 * np.sqrt(np.mean(want ** 2))
    with pytest.raises(RuntimeError, match="not divisible by 128"):
        ex_ops.aok_run_fp8(0, dv(A)[:, :100].contiguous(), dv(a_s), dv(wq)[:, :, :100].contiguous(), dv(w_s), C, dv(ex), 100, 100, C)


@pytest.mark.gpu
def test_torch_router_op(cuda, ex_ops):
    from eps_b200 import ops

    gen = torch.Generator().manual_seed(11)
    scores = torch.randn((40, 256), generator=gen).to(torch.bfloat16).to(cuda)
    bias = (torch.randn(256, generator=gen) * 0.1).to(cuda)
    w = torch.empty((40, 8), dtype=torch.float32, device=cuda)
    idx = torch.empty((40, 8), dtype=torch.int32, device=cuda)
    torch.ops.utils.topk_sigmoid(scores, bias, w, idx, 40, 256, 8, 4, 8, 2.5)
    idx2, w2 = ops.topk_sigmoid(scores, bias, 8, 4, 8, 2.5)
    torch.cuda.synchronize()
    assert torch.equal(idx, idx2) and torch.equal(w, w2)
    with pytest.raises(RuntimeError, match="Not supported expert_indices data type"):
        torch.ops.utils.topk_sigmoid(scores, bias, w, idx.to(torch.int64), 40, 256, 8, 4, 8, 2.5)


@pytest.mark.gpu
def test_torch_rms_norm_op(cuda, ex_ops):
    from eps_b200 import ops

    x = torch.randn((9, 512), generator=torch.Generator().manual_seed(2)).to(torch.bfloat16).to(cuda)
    sc = torch.ones(512, dtype=torch.bfloat16, device=cuda)
    out = torch.empty_like(x)
    torch.ops.utils.rms_norm_op(out, x, sc, 1e-6)
    torch.cuda.synchronize()
    assert torch.equal(out, ops.rms_norm(x, sc, 1e-6))
    with pytest.raises(RuntimeError, match="dim must be 2"):
        torch.ops.utils.rms_norm_op(out, x[0], sc, 1e-6)

