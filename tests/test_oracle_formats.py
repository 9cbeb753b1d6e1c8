"""Known-answer tests that pin the oracle's number formats (CPU only)."""
import numpy as np
import pytest
import torch


def test_e4m3_all_codes_roundtrip(oracle):
    table = oracle.e4m3_table()
    for c in range(256):
        v = table[c]
        if np.isnan(v):
            assert c in (0x7F, 0xFF)
            continue
        assert oracle.f32_to_e4m3(float(v)) == c or (v == 0 and c == 0x80 and oracle.f32_to_e4m3(float(v)) in (0x00, 0x80))


def test_e4m3_known_values(oracle):
    kat = {0.0: 0x00, 1.0: 0x38, -1.0: 0xB8, 448.0: 0x7E, -448.0: 0xFE, 2.0 ** -6: 0x08, 2.0 ** -9: 0x01,
           7 * 2.0 ** -9: 0x07, 1.5: 0x3C, 240.0: 0x77, 0.5: 0x30}
    for v, c in kat.items():
        assert oracle.f32_to_e4m3(v) == c, (v, hex(c))


def test_e4m3_ties_saturation_subnormals(oracle):
    f = oracle.f32_to_e4m3
    # ties to even between 1.0 (0x38) and 1.125 (0x39) -> 1.0; between 1.125 and 1.25 (0x3A) -> 1.25
    assert f(1.0625) == 0x38
    assert f(1.1875) == 0x3A
    # just above/below a tie
    assert f(np.nextafter(np.float32(1.0625), np.float32(2))) == 0x39
    assert f(np.nextafter(np.float32(1.1875), np.float32(0))) == 0x39
    # saturation (satfinite): everything >= 448 and +inf -> 0x7E; NaN -> 0x7F
    assert f(464.0) == 0x7E and f(1e30) == 0x7E and f(float("inf")) == 0x7E
    assert f(-1e30) == 0xFE
    assert f(float("nan")) & 0x7F == 0x7F
    # 432 is the tie between 416 (0x7D) and 448 (0x7E): even mantissa is 448
    assert f(432.0) == 0x7E
    # subnormal grid 2^-9; 2^-10 ties to even (0); 1.5*2^-9 ties to 2*2^-9
    assert f(2.0 ** -10) == 0x00
    assert f(1.5 * 2.0 ** -9) == 0x02
    assert f(np.nextafter(np.float32(2.0 ** -10), np.float32(1))) == 0x01
    # largest subnormal / smallest normal boundary
    assert f(7.5 * 2.0 ** -9) == 0x08


def test_e4m3_matches_torch_in_range(oracle):
    rng = np.random.default_rng(1)
    x = np.concatenate([rng.standard_normal(20000).astype(np.float32) * s for s in (1e-3, 0.05, 1.0, 60.0)])
    x = x[np.abs(x) <= 448]
    ref = torch.from_numpy(x).to(torch.float8_e4m3fn).view(torch.uint8).numpy()
    got = np.array([oracle.f32_to_e4m3(float(v)) for v in x], dtype=np.uint8)
    assert np.array_equal(got, ref)
    back = torch.from_numpy(got).view(torch.float8_e4m3fn).to(torch.float32).numpy()
    assert np.array_equal(back, oracle.e4m3_table()[got])


def test_bf16_rounding_matches_torch(oracle):
    rng = np.random.default_rng(2)
    x = (rng.standard_normal(50000) * 10).astype(np.float32)
    ref = torch.from_numpy(x).to(torch.bfloat16).view(torch.int16).numpy().view(np.uint16)
    assert np.array_equal(oracle.bf16_bits(x), ref)
    got_c = np.array([oracle.lib().orc_f32_to_bf16(float(v)) for v in x[:2000]], dtype=np.uint16)
    assert np.array_equal(got_c, ref[:2000])


def test_quant_1x128_definition(oracle):
    """orc_quant_1x128 against a direct numpy statement of amax/448, 1/scale, clamp, RN-even."""
    rng = np.random.default_rng(3)
    x = oracle.bf16_bits(rng.standard_normal((7, 384)).astype(np.float32))
    x[2, 128:256] = 0  # an all-zero group: scale 0, codes 0x7E (0*inf = NaN dropped by fmin/fmax)
    q, s = oracle.quant_1x128(x)
    xf = oracle.bf16_to_f32(x).reshape(7, 3, 128)
    amax = np.abs(xf).max(-1)
    scale = (amax / np.float32(448.0)).astype(np.float32)
    assert np.array_equal(s, scale)
    assert np.all(q[2, 128:256] == 0x7E) and s[2, 1] == 0
    with np.errstate(divide="ignore", invalid="ignore"):
        inv = (np.float32(1.0) / scale).astype(np.float32)
        v = (xf * inv[..., None]).astype(np.float32)
    ok = scale > 0
    ref = torch.from_numpy(np.clip(v[ok], -448, 448)).to(torch.float8_e4m3fn).view(torch.uint8).numpy()
    assert np.array_equal(q.reshape(7, 3, 128)[ok], ref)
    # dequantised error bound: half an e4m3 ulp of the group's amax
    deq = oracle.bf16_to_f32(oracle.dequant_1x128(q, s)).reshape(7, 3, 128)
    assert np.all(np.abs(deq - xf) <= amax[..., None] * (2.0 ** -4) + 1e-30)


def test_quant_block128_definition(oracle):
    rng = np.random.default_rng(4)
    w = oracle.bf16_to_f32(oracle.bf16_bits((rng.standard_normal((2, 200, 256)) * 0.02).astype(np.float32)))
    q, s = oracle.quant_block128(w)
    assert q.shape == (2, 200, 256) and s.shape == (2, 2, 2)
    for m in range(2):
        for bi in range(2):
            for bj in range(2):
                blk = w[m, bi * 128:(bi + 1) * 128, bj * 128:(bj + 1) * 128]
                sc = np.float32(np.abs(blk).max()) / np.float32(448.0)
                assert s[m, bi, bj] == sc
                ref = torch.from_numpy(np.clip(blk * (np.float32(1.0) / sc), -448, 448).astype(np.float32)).to(
                    torch.float8_e4m3fn).view(torch.uint8).numpy()
                assert np.array_equal(q[m, bi * 128:(bi + 1) * 128, bj * 128:(bj + 1) * 128], ref)
