"""GPU parity of the quantiser kernels (through the C-ABI) against the numpy oracle and the golden fixtures:
codes, scales and the blocked scale tensor must match byte for byte."""
import numpy as np
import pytest
import torch

from oracle import quant_oracle as qo

pytestmark = pytest.mark.gpu

FMTS = ["mx8", "nv4", "mx4"]
GOLDEN_CASES = ["normal_37x256", "heavy_130x768", "mk_65x1024", "wide_33x512", "zeros_16x128", "c1_bf16_96x1024",
                "rowout_40x256", "mid_e4m3_2x128"]


def _ops():
    from lightly_trian_quant_b200 import ops

    return ops


def _run_quant(x_t, fmt, ts=None, **kw):
    ops = _ops()
    M, K = x_t.shape
    buf = ops.ActBuf(M, K, fmt, device="cuda")
    buf.q.fill_(0xAA)
    buf.sf.fill_(0xAA)
    if fmt == "nv4":
        buf.ts.copy_(torch.from_numpy(np.asarray(ts, dtype=np.float32)))
    ops.quant_rows(x_t, buf, **kw)
    torch.cuda.synchronize()
    return buf.q.cpu().numpy(), buf.sf.cpu().numpy()


def _expect(x_np, fmt, ts=None):
    q, s, _ = qo.quantize(x_np, fmt, ts)
    return q, qo.to_blocked(s).reshape(-1)


@pytest.mark.parametrize("fmt", FMTS)
@pytest.mark.parametrize("name", GOLDEN_CASES)
def test_quant_rows_golden(golden, name, fmt):
    x = golden[f"{name}/x"]
    if x.shape[1] % 128:
        pytest.skip("K not a multiple of 128")
    ts = golden[f"{name}/nv4_ts"] if fmt == "nv4" else None
    q, sf = _run_quant(torch.from_numpy(x).cuda(), fmt, ts)
    key = {"mx8": "mx8", "nv4": "nv4", "mx4": "mx4"}[fmt]
    assert np.array_equal(q, golden[f"{name}/{key}_q"])
    sb = golden[f"{name}/{key}_sb"].reshape(-1) if f"{name}/{key}_sb" in golden else qo.to_blocked(golden[f"{name}/{key}_s"]).reshape(-1)
    assert np.array_equal(sf, sb)
    if fmt == "nv4":    # static calibrated scale (headroom 2)
        q2, sf2 = _run_quant(torch.from_numpy(x).cuda(), fmt, golden[f"{name}/nv4h_ts"])
        assert np.array_equal(q2, golden[f"{name}/nv4h_q"])
        assert np.array_equal(sf2, qo.to_blocked(golden[f"{name}/nv4h_s"]).reshape(-1))


@pytest.mark.parametrize("fmt", FMTS)
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
@pytest.mark.parametrize("shape", [(1, 128), (130, 768), (1605, 1024), (257, 4096)])
def test_quant_rows_vs_oracle(fmt, dtype, shape):
    g = torch.Generator().manual_seed(hash((fmt, shape)) % 1000)
    M, K = shape
    x = torch.randn(M, K, generator=g)
    x[:, 5] *= 30
    x[:, K // 3] *= 12
    if M > 8:
        x[7] = 0
    x = x.to(dtype)
    xn = x.float().numpy()
    ts = qo.nv4_ts(xn) if fmt == "nv4" else None
    q, sf = _run_quant(x.cuda(), fmt, ts)
    eq, esf = _expect(xn, fmt, ts)
    assert np.array_equal(sf, esf)
    assert np.array_equal(q, eq)


@pytest.mark.parametrize("fmt", FMTS)
def test_quant_rows_strided_and_gelu(fmt):
    g = torch.Generator().manual_seed(3)
    M, K = 200, 512
    base = torch.randn(M, 2 * K, generator=g).to(torch.bfloat16)
    bias = (torch.randn(K, generator=g) * 0.1)
    x = base[:, :K]                                       # row stride 2K
    gx = torch.nn.functional.gelu(x.float() + bias)       # erf GELU in fp32
    # the GPU erff differs from the host erf in the last ulp: compare on the bf16-rounded values both sides compute
    gx_b = gx.to(torch.bfloat16).float().numpy()
    ts = qo.nv4_ts(gx_b) if fmt == "nv4" else None
    q, sf = _run_quant(x.cuda(), fmt, ts, bias=bias.cuda(), gelu=True, round_bf16=True)
    eq, esf = _expect(gx_b, fmt, ts)
    agree = (q == eq).mean()
    assert agree > 0.9995, agree                           # bf16 ties of GELU values that differ by an ulp of erff
    assert (sf == esf).mean() > 0.999
    # plain strided input: exact
    xn = x.float().numpy()
    ts = qo.nv4_ts(xn) if fmt == "nv4" else None
    q, sf = _run_quant(x.cuda(), fmt, ts)
    eq, esf = _expect(xn, fmt, ts)
    assert np.array_equal(q, eq) and np.array_equal(sf, esf)


@pytest.mark.parametrize("fmt", FMTS)
@pytest.mark.parametrize("d", [768, 1024])
@pytest.mark.parametrize("round_bf16", [False, True])
def test_ln_quant(fmt, d, round_bf16):
    """LN fused with quantisation: bit-exact against the oracle quantiser applied to the kernel's own LN output,
    and the LN values themselves within fp32 rounding of a float64 LayerNorm."""
    ops = _ops()
    g = torch.Generator().manual_seed(11)
    M = 301
    x = torch.randn(M, d, generator=g) * 3 + 0.5
    x[:, 17] *= 40
    x[:5] *= 100
    w = torch.rand(d, generator=g) + 0.5
    b = torch.randn(d, generator=g) * 0.1
    eps = 1e-5
    y_ref = qo.layernorm(x.numpy(), w.numpy(), b.numpy(), eps)
    if round_bf16:
        y_ref = qo.bf16_round(y_ref)
    buf = ops.ActBuf(M, d, fmt, device="cuda")
    buf.sf.fill_(0xAA)
    ts = qo.nv4_ts(y_ref) * 2.0 if fmt == "nv4" else None
    if fmt == "nv4":
        buf.ts.copy_(torch.from_numpy(ts))
    y_dbg = torch.empty(M, d, device="cuda")
    ops.ln_quant(x.cuda(), w.cuda(), b.cuda(), eps, buf, round_bf16=round_bf16, y_dbg=y_dbg)
    torch.cuda.synchronize()
    y = y_dbg.cpu().numpy()
    tol = 2e-2 if round_bf16 else 2e-5
    assert np.max(np.abs(y - y_ref) / (np.abs(y_ref) + 1.0)) < tol
    eq, esf = _expect(y, fmt, ts)
    assert np.array_equal(buf.q.cpu().numpy(), eq)
    assert np.array_equal(buf.sf.cpu().numpy(), esf)
    # against the oracle LN: nearly all bytes agree (summation order differs)
    eq2, esf2 = _expect(y_ref, fmt, ts)
    assert (buf.q.cpu().numpy() == eq2).mean() > 0.999
    # without the debug output: identical bytes
    buf2 = ops.ActBuf(M, d, fmt, device="cuda", ts=buf.ts)
    ops.ln_quant(x.cuda(), w.cuda(), b.cuda(), eps, buf2, round_bf16=round_bf16)
    assert torch.equal(buf2.q, buf.q) and torch.equal(buf2.sf, buf.sf)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_ln_rows(dtype):
    ops = _ops()
    g = torch.Generator().manual_seed(5)
    x = torch.randn(77, 1024, generator=g) * 2
    w = torch.rand(1024, generator=g) + 0.5
    b = torch.randn(1024, generator=g) * 0.1
    y = ops.ln_rows(x.cuda(), w.cuda(), b.cuda(), 1e-5, dtype).float().cpu()
    ref = torch.from_numpy(qo.layernorm(x.numpy(), w.numpy(), b.numpy(), 1e-5)).to(dtype).float()
    assert (y - ref).abs().max() <= 2 * torch.finfo(dtype).eps * ref.abs().max()


def test_recip_div_mode_same_mx_bytes():
    """MX scale bytes do not depend on true division vs reciprocal multiply."""
    x = (torch.randn(512, 1024, generator=torch.Generator().manual_seed(2)) * 7).cuda()
    for fmt in ("mx8", "mx4"):
        a = _run_quant(x, fmt)
        b = _run_quant(x, fmt, recip_div=True)
        assert np.array_equal(a[0], b[0]) and np.array_equal(a[1], b[1])


def test_fast_reciprocal_is_correctly_rounded_for_every_significand():
    """the three-instruction reciprocal the NVFP4 quantisers divide by (approximate reciprocal + one Newton step) equals
    __frcp_rn for all 2^23 - 1 significands (all ones excluded by contract), both signs, at several exponents of its range."""
    import ctypes as C

    from lightly_trian_quant_b200 import _lib, ops

    cnt = torch.zeros(1, dtype=torch.int32, device="cuda")
    for e in (-59, -17, -1, 0, 1, 23, 59):
        _lib.check(_lib.lib().kf_selftest_rcp(e, C.c_void_p(cnt.data_ptr()), C.c_void_p(torch.cuda.current_stream().cuda_stream)), "kf_selftest_rcp")
    torch.cuda.synchronize()
    ops.check_device_error()
    assert int(cnt.item()) == 0, f"{int(cnt.item())} significands differ from __frcp_rn"


@pytest.mark.parametrize("fmt", ["mx8", "mx4", "nv4"])
def test_non_finite_inputs_follow_the_reference(golden, fmt):
    """a NaN or an infinity in a block reaches the scale byte and the codes exactly as in the reference quantiser (its
    maxima propagate NaN): nothing is silently quantised as a finite value."""
    from lightly_trian_quant_b200 import ops

    x = torch.from_numpy(golden["nonfinite/x"]).cuda()
    a = ops.ActBuf(x.shape[0], x.shape[1], fmt, device="cuda")
    key = "nv4h" if fmt == "nv4" else fmt
    if fmt == "nv4":
        a.ts.copy_(torch.from_numpy(golden["nonfinite/nv4h_ts"]))
    ops.quant_rows(x, a)
    ops.check_device_error()
    assert np.array_equal(a.q.cpu().numpy(), golden[f"nonfinite/{key}_q"])
    nb = x.shape[1] // qo.VEC[fmt]
    s2 = qo.from_blocked(a.sf.cpu().numpy().reshape(1, -(-nb // 4), 32, 4, 4), x.shape[0], nb)
    assert np.array_equal(s2, golden[f"nonfinite/{key}_s"])
