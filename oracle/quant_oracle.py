"""CPU oracle for the block-scaled quantisers (MXFP8 / NVFP4 / MXFP4): test infrastructure, not product code.

Only the tests, the smoke check and the CPU-baseline leg of the benchmark may import this module; the product
path never does.  It restates, in numpy with explicit bit arithmetic (no torch float8 casts), the algorithm of
the reference's single bit-exact quantiser specification:

  infer-opt/round10_lowp_probe/impl/quant_ref.py
      _rceil_byte :92-97      mx8_quantize :100-109    mx8_dequant :112-115
      _nv4_ts     :119-121    _nv4_sf      :124-125    nv4_quantize :128-137   nv4_dequant :140-143
      mx4_quantize:146-154    mx4_dequant  :157-159    e2m1_rn :39-43   pack_nibbles :52-53
      to_blocked  :224-230    from_blocked :233-236    qdq :202-221
  train-opt/round20_fp4_probe/impl/fp4_ref.py  (the same FP4 rules; quantize_matrix :169-188, dequant_copy :263-273)

Parity is pinned: the golden fixtures under tests/golden/ were produced by importing the reference's quant_ref.py
and fp4_ref.py unmodified (tests/golden/gen_golden.py) and this module reproduces every byte of them
(tests/test_oracle_golden.py).

All divisions by python scalars are IEEE fp32 divisions, which is what the reference computes when it runs on the
host cores.
"""
from __future__ import annotations

import numpy as np

VEC = {"mx8": 32, "nv4": 16, "mx4": 32}
E2M1_GRID = np.array([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0], dtype=np.float32)
F8_MAX = np.float32(448.0)
f32 = np.float32


# ------------------------------------------------------------------------------------------------ element formats
def f32_to_e4m3_bits(v: np.ndarray) -> np.ndarray:
    """fp32 -> e4m3 (fn) byte, round-to-nearest-even, |v| saturated at 448 (the reference clamps before it casts,
    quant_ref.py:107,125).  Exact: computed in float64 on the e4m3 lattice."""
    v = np.asarray(v, dtype=np.float32)
    sign = np.signbit(v).astype(np.uint8) << 7
    a = np.minimum(np.abs(v).astype(np.float64), 448.0)
    _, ex = np.frexp(a)                                   # a = m * 2^ex, m in [0.5, 1)
    e = np.maximum(ex - 1, -6)                            # unbiased exponent, clamped to the subnormal quantum
    q = np.ldexp(1.0, e - 3)                              # lattice spacing
    val = np.rint(a / q) * q                              # rint = round half to even; a/q is exact
    # encode val (exactly representable): subnormal -> val * 2^9, normal -> ((E) << 3) | M
    m2, ex2 = np.frexp(val)
    E = ex2 - 1 + 7
    M = np.rint((m2 * 2.0 - 1.0) * 8.0).astype(np.int64)
    normal = (E.astype(np.int64) << 3) | M
    sub = np.rint(val * 512.0).astype(np.int64)
    bits = np.where(val < 2.0 ** -6, sub, normal)
    bits = np.where(val == 0, 0, bits)
    bits = np.where(np.isnan(v), 0x7F, bits)              # e4m3fn has one NaN pattern per sign (the torch cast gives 0x7f)
    return (bits.astype(np.uint8) | sign).astype(np.uint8)


def e4m3_bits_to_f32(b: np.ndarray) -> np.ndarray:
    b = np.asarray(b, dtype=np.uint8).astype(np.int32)
    s = np.where(b & 0x80, -1.0, 1.0)
    E = (b >> 3) & 0xF
    M = b & 7
    normal = np.ldexp(1.0 + M / 8.0, E - 7)
    sub = np.ldexp(M / 8.0, -6)
    out = np.where(E == 0, sub, normal)
    out = np.where((E == 15) & (M == 7), np.nan, out)
    return (s * out).astype(np.float32)


def e2m1_rn(v: np.ndarray) -> np.ndarray:
    """fp32 -> e2m1 code (bit 3 = sign taken from signbit, so -0 -> 0x8), RN-even thresholds, saturating at 6
    (quant_ref.py:39-43)."""
    v = np.asarray(v, dtype=np.float32)
    a = np.abs(v)
    code = ((a > 0.25).astype(np.uint8) + (a >= 0.75) + (a > 1.25) + (a >= 1.75) + (a > 2.5) + (a >= 3.5)
            + (a > 5.0)).astype(np.uint8)
    return code | (np.signbit(v).astype(np.uint8) << 3)


def e2m1_value(code: np.ndarray) -> np.ndarray:
    code = np.asarray(code, dtype=np.uint8)
    val = E2M1_GRID[(code & 7).astype(np.int64)]
    return np.where((code & 8) != 0, -val, val).astype(np.float32)


def pack_nibbles(codes: np.ndarray) -> np.ndarray:
    """[..., C] codes -> [..., C/2] bytes, even element index in the low nibble (quant_ref.py:52-53)."""
    return np.ascontiguousarray(codes[..., 0::2] | (codes[..., 1::2] << 4)).astype(np.uint8)


def unpack_nibbles(b: np.ndarray) -> np.ndarray:
    b = np.asarray(b, dtype=np.uint8)
    return np.stack([b & 0xF, b >> 4], axis=-1).reshape(*b.shape[:-1], b.shape[-1] * 2)


# ------------------------------------------------------------------------------------------------ scale rules
def rceil_byte(amax: np.ndarray, denom: float, max_byte: int) -> np.ndarray:
    """ue8m0 byte = biased_exp(fl32(amax/denom)) + (mantissa != 0), clamped (quant_ref.py:92-97)."""
    r = (np.asarray(amax, dtype=np.float32) / f32(denom)).astype(np.float32)
    bits = np.ascontiguousarray(r).view(np.int32)
    e = (bits >> 23) & 0xFF
    frac = ((bits & 0x7FFFFF) != 0).astype(np.int32)
    return np.minimum(e + frac, max_byte).astype(np.int32)


def _exp2_f32(k: np.ndarray) -> np.ndarray:
    """2^k as fp32 for integer k in [-127, 127] (k = -127 is the subnormal 2^-127, as torch.exp2 returns)."""
    return np.ldexp(np.float64(1.0), np.asarray(k, dtype=np.int64)).astype(np.float32)


def mx8_quantize(x: np.ndarray):
    """x [R, C] (C % 32 == 0) -> (q [R, C] uint8 e4m3 bytes, byte [R, C/32] uint8).  quant_ref.py:100-109."""
    x = np.asarray(x)
    R, C = x.shape
    xf = x.astype(np.float32).reshape(R, C // 32, 32)
    amax = np.abs(xf).max(-1)
    byte = rceil_byte(amax, 448.0, 255)
    inv = _exp2_f32(127 - np.where(byte == 0, 1, byte))
    v = np.clip((xf * inv[..., None]).astype(np.float32), -F8_MAX, F8_MAX)
    return f32_to_e4m3_bits(v).reshape(R, C), byte.astype(np.uint8)


def mx8_dequant(q: np.ndarray, byte: np.ndarray) -> np.ndarray:
    R, C = q.shape
    s = np.ldexp(np.float64(1.0), byte.astype(np.int64) - 127).astype(np.float32)
    return (e4m3_bits_to_f32(q).reshape(R, C // 32, 32) * s[..., None]).reshape(R, C).astype(np.float32)


def nv4_ts(x: np.ndarray) -> np.ndarray:
    """per-tensor scale amax/(6*448), 1 when the tensor is all zero (quant_ref.py:119-121)."""
    amax = np.abs(np.asarray(x).astype(np.float32)).max()
    return np.array([amax / f32(6.0 * 448.0) if amax > 0 else 1.0], dtype=np.float32)


def nv4_quantize(x: np.ndarray, ts: np.ndarray | None = None):
    """x [R, C] (C % 16 == 0) -> (q [R, C/2] uint8, sf [R, C/16] uint8 e4m3 bytes, ts [1] fp32).
    quant_ref.py:128-137; a given ts is a static calibrated scale."""
    x = np.asarray(x)
    R, C = x.shape
    xf = np.ascontiguousarray(x.astype(np.float32))
    ts = nv4_ts(xf) if ts is None else np.asarray(ts, dtype=np.float32).reshape(1)
    amax_b = np.abs(xf.reshape(R, C // 16, 16)).max(-1)
    t = ((amax_b / f32(6.0)).astype(np.float32) / ts[0]).astype(np.float32)
    sf8 = f32_to_e4m3_bits(np.minimum(t, F8_MAX))
    denom = (e4m3_bits_to_f32(sf8) * ts[0]).astype(np.float32).reshape(R, C // 16, 1)
    ok = denom > 0
    with np.errstate(divide="ignore", invalid="ignore"):
        v = (xf.reshape(R, C // 16, 16) / np.where(ok, denom, f32(1.0))).astype(np.float32)
    v = np.where(ok, v, f32(0.0)).reshape(R, C)
    return pack_nibbles(e2m1_rn(v)), sf8, ts


def nv4_dequant(q, sf8, ts) -> np.ndarray:
    vals = e2m1_value(unpack_nibbles(q))
    s = (e4m3_bits_to_f32(sf8) * np.asarray(ts, dtype=np.float32).reshape(1)[0]).astype(np.float32)
    return (vals * np.repeat(s, 16, axis=1)).astype(np.float32)


def mx4_quantize(x: np.ndarray):
    """x [R, C] (C % 32 == 0) -> (q [R, C/2] uint8, byte [R, C/32] uint8).  quant_ref.py:146-154."""
    x = np.asarray(x)
    R, C = x.shape
    xf = np.ascontiguousarray(x.astype(np.float32))
    amax = np.abs(xf.reshape(R, C // 32, 32)).max(-1)
    byte = rceil_byte(amax, 6.0, 254)
    inv = _exp2_f32(127 - byte).reshape(R, C // 32, 1)
    v = (xf.reshape(R, C // 32, 32) * inv).astype(np.float32).reshape(R, C)
    return pack_nibbles(e2m1_rn(v)), byte.astype(np.uint8)


def mx4_dequant(q, byte) -> np.ndarray:
    vals = e2m1_value(unpack_nibbles(q))
    s = np.ldexp(np.float64(1.0), byte.astype(np.int64) - 127).astype(np.float32)
    return (vals * np.repeat(s, 32, axis=1)).astype(np.float32)


# ------------------------------------------------------------------------------------------------ scale layout
def to_blocked(sf2d: np.ndarray) -> np.ndarray:
    """uint8 [R, nb] -> [ceil(R/128), ceil(nb/4), 32, 4, 4]: the 128x4 blocked scale layout, zero padded
    (quant_ref.py:224-230).  Byte of (row, kb) sits at
    ((row/128)*(nb/4) + kb/4)*512 + (row%32)*16 + ((row/32)%4)*4 + kb%4."""
    sf2d = np.asarray(sf2d, dtype=np.uint8)
    R, nb = sf2d.shape
    rm, rk = -(-R // 128), -(-nb // 4)
    pad = np.zeros((rm * 128, rk * 4), dtype=np.uint8)
    pad[:R, :nb] = sf2d
    t = pad.reshape(rm, 128, rk, 4).transpose(0, 2, 1, 3).reshape(rm, rk, 4, 32, 4).transpose(0, 1, 3, 2, 4)
    return np.ascontiguousarray(t)


def from_blocked(sf: np.ndarray, R: int, nb: int) -> np.ndarray:
    sf = np.asarray(sf, dtype=np.uint8)
    rm, rk = sf.shape[:2]
    t = sf.reshape(rm, rk, 32, 4, 4).transpose(0, 1, 3, 2, 4).reshape(rm, rk, 128, 4).transpose(0, 2, 1, 3)
    return np.ascontiguousarray(t.reshape(rm * 128, rk * 4)[:R, :nb])


def sf_bytes(R: int, K: int, fmt: str) -> int:
    """size in bytes of the blocked scale tensor of an [R, K] operand."""
    nb = K // VEC[fmt]
    return -(-R // 128) * -(-nb // 4) * 512


# ------------------------------------------------------------------------------------------------ one-call helpers
def quantize(x: np.ndarray, fmt: str, ts=None):
    """-> (codes, scales2d uint8, ts or None) in the row-major 2-D scale form."""
    if fmt == "mx8":
        q, s = mx8_quantize(x)
        return q, s, None
    if fmt == "nv4":
        return nv4_quantize(x, ts)
    if fmt == "mx4":
        q, s = mx4_quantize(x)
        return q, s, None
    raise ValueError(fmt)


def dequant(q, s2d, ts, fmt: str) -> np.ndarray:
    if fmt == "mx8":
        return mx8_dequant(q, s2d)
    if fmt == "nv4":
        return nv4_dequant(q, s2d, ts)
    if fmt == "mx4":
        return mx4_dequant(q, s2d)
    raise ValueError(fmt)


def qdq(x: np.ndarray, fmt: str, ts=None) -> np.ndarray:
    """fp32 values the tensor core multiplies for x quantised in fmt (nv4: ts folded in).  quant_ref.py:202-221."""
    q, s, t = quantize(x, fmt, ts)
    return dequant(q, s, t, fmt)


def bf16_round(x: np.ndarray) -> np.ndarray:
    """fp32 -> nearest bf16 (RN-even) returned as fp32."""
    b = np.ascontiguousarray(np.asarray(x, dtype=np.float32)).view(np.uint32).astype(np.uint64)
    r = ((b + 0x7FFF + ((b >> 16) & 1)) >> 16) << 16
    return r.astype(np.uint32).view(np.float32)


def layernorm(x: np.ndarray, w: np.ndarray, b: np.ndarray, eps: float) -> np.ndarray:
    """fp32 two-pass LayerNorm over the last axis: mean, centred variance, rsqrt(var+eps), affine
    (infer-opt/round13_mxfp8_full/impl/mx13.cu:104-130).  Accumulated in float64 then rounded, so it is a
    tolerance reference for the LN statistics, not a bit reference (summation order differs on the GPU)."""
    xd = np.asarray(x, dtype=np.float64)
    mean = xd.mean(-1, keepdims=True)
    var = ((xd - mean) ** 2).mean(-1, keepdims=True)
    y = (xd - mean) / np.sqrt(var + eps) * np.asarray(w, dtype=np.float64) + np.asarray(b, dtype=np.float64)
    return y.astype(np.float32)
