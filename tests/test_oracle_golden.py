"""The numpy oracle must reproduce every byte the reference quantisers produced (fixtures made by
tests/golden/gen_golden.py from the reference's quant_ref.py / fp4_ref.py on the host cores)."""
import numpy as np
import pytest

from oracle import quant_oracle as qo

CASES = ["normal_37x256", "heavy_130x768", "mk_65x1024", "wide_33x512", "zeros_16x128", "c1_bf16_96x1024",
         "rowout_40x256", "mid_e2m1_4x64", "mid_e4m3_2x128"]


@pytest.mark.parametrize("name", CASES)
def test_mx8_bytes(golden, name):
    x = golden[f"{name}/x"]
    q, s = qo.mx8_quantize(x)
    assert np.array_equal(q, golden[f"{name}/mx8_q"])
    assert np.array_equal(s, golden[f"{name}/mx8_s"])
    assert np.array_equal(qo.to_blocked(s), golden[f"{name}/mx8_sb"])
    if f"{name}/mx8_dq" in golden:
        assert np.array_equal(qo.mx8_dequant(q, s), golden[f"{name}/mx8_dq"])


@pytest.mark.parametrize("name", CASES)
def test_nv4_bytes(golden, name):
    x = golden[f"{name}/x"]
    q, s, ts = qo.nv4_quantize(x)
    assert np.array_equal(ts, golden[f"{name}/nv4_ts"])
    assert np.array_equal(s, golden[f"{name}/nv4_s"])
    assert np.array_equal(q, golden[f"{name}/nv4_q"])
    assert np.array_equal(qo.to_blocked(s), golden[f"{name}/nv4_sb"])
    if f"{name}/nv4_dq" in golden:
        assert np.array_equal(qo.nv4_dequant(q, s, ts), golden[f"{name}/nv4_dq"])
    # static (calibrated, headroom 2) per-tensor scale
    q2, s2, _ = qo.nv4_quantize(x, golden[f"{name}/nv4h_ts"])
    assert np.array_equal(s2, golden[f"{name}/nv4h_s"])
    assert np.array_equal(q2, golden[f"{name}/nv4h_q"])


@pytest.mark.parametrize("name", CASES)
def test_mx4_bytes(golden, name):
    x = golden[f"{name}/x"]
    q, s = qo.mx4_quantize(x)
    assert np.array_equal(s, golden[f"{name}/mx4_s"])
    assert np.array_equal(q, golden[f"{name}/mx4_q"])
    if f"{name}/mx4_dq" in golden:
        assert np.array_equal(qo.mx4_dequant(q, s), golden[f"{name}/mx4_dq"])


@pytest.mark.parametrize("fmt", ["mx8", "nv4", "mx4"])
def test_c1_gemm_slice(golden, fmt):
    """dequantise-then-fp32-matmul of the config-1 slice: same operands bit for bit, product within fp32 summation noise."""
    x, w, b = golden["c1gemm/x"], golden["c1gemm/w"], golden["c1gemm/bias"]
    y = qo.qdq(x, fmt).astype(np.float64) @ qo.qdq(w, fmt).astype(np.float64).T + b
    ref = golden[f"c1gemm/{fmt}_y"].astype(np.float64)
    assert np.linalg.norm(y - ref) / np.linalg.norm(ref) < 1e-6


def test_blocked_roundtrip_and_offsets():
    rng = np.random.default_rng(0)
    for R, nb in ((1, 4), (130, 24), (257, 8), (1605, 32)):
        s = rng.integers(0, 256, (R, nb), dtype=np.uint8)
        blk = qo.to_blocked(s)
        assert blk.shape == (-(-R // 128), nb // 4, 32, 4, 4)
        assert np.array_equal(qo.from_blocked(blk, R, nb), s)
        flat = blk.reshape(-1)
        for row, kb in ((0, 0), (R - 1, nb - 1), (R // 2, nb // 2)):
            off = ((row // 128) * (nb // 4) + kb // 4) * 512 + (row % 32) * 16 + ((row // 32) % 4) * 4 + kb % 4
            assert flat[off] == s[row, kb]
        assert flat.size == qo.sf_bytes(R, nb * 32, "mx8")


def test_e2m1_grid_fixed_point_and_e4m3_exhaustive():
    codes = np.arange(16, dtype=np.uint8)
    assert np.array_equal(qo.e2m1_rn(qo.e2m1_value(codes)) & 7, codes & 7)
    b = np.array([i for i in range(256) if (i & 0x7F) != 0x7F], dtype=np.uint8)
    assert np.array_equal(qo.f32_to_e4m3_bits(qo.e4m3_bits_to_f32(b)) & 0x7F, b & 0x7F)
    # against torch's own cast on a dense sweep (torch is plumbing here, not the oracle)
    import torch

    v = torch.linspace(-448, 448, 200001)
    assert np.array_equal(qo.f32_to_e4m3_bits(v.numpy()), v.to(torch.float8_e4m3fn).view(torch.uint8).numpy())
    v = torch.randn(100000) * 0.01
    assert np.array_equal(qo.f32_to_e4m3_bits(v.numpy()), v.to(torch.float8_e4m3fn).view(torch.uint8).numpy())


def test_bf16_round():
    import torch

    v = torch.randn(50000) * 37
    assert np.array_equal(qo.bf16_round(v.numpy()), v.to(torch.bfloat16).float().numpy())


def test_non_finite_inputs_follow_the_reference(golden):
    """NaN and +-Inf in different blocks: the scale bytes (255 / 254 / 0x7f) and codes the reference quantisers produce."""
    import warnings

    x = golden["nonfinite/x"]
    with warnings.catch_warnings():
        warnings.simplefilter("ignore")
        q, s = qo.mx8_quantize(x)
        assert np.array_equal(q, golden["nonfinite/mx8_q"]) and np.array_equal(s, golden["nonfinite/mx8_s"])
        q, s = qo.mx4_quantize(x)
        assert np.array_equal(q, golden["nonfinite/mx4_q"]) and np.array_equal(s, golden["nonfinite/mx4_s"])
        q, s, _ = qo.nv4_quantize(x, golden["nonfinite/nv4h_ts"])
        assert np.array_equal(q, golden["nonfinite/nv4h_q"]) and np.array_equal(s, golden["nonfinite/nv4h_s"])
