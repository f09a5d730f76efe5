"""CPU oracle of the block-scaled GEMM and its fused epilogues: test infrastructure, not product code.

The GEMM reference is the reference's own gate: the product of the DEQUANTISED operands in high precision
(fp32 gate / fp64 report), as in
    infer-opt/round13_mxfp8_full/tests/test13a.py:75-89      (cuBLASLt / own MXFP8 GEMM vs dequant product)
    infer-opt/round14_fp4_full/tests/t_gemm.py:54-68         (check(): FP4 GEMM vs the fp64 product)
Epilogues follow
    RoPE + [3,B,N,H,64] relayout   infer-opt/round13_mxfp8_full/tests/test_mgx.py:46-57 (rope_ref), mgx_core.cu:391-426
    residual                       mgx_core.cu:370-382   out = R + gamma * (acc + bias)
    GELU (erf) + quantise-out      mgx_core.cu:308-360, fp4g_core.cu:309-382
Parity of this file is pinned through tolerance (rel. Frobenius <= 2e-3 for 16-bit outputs), exactly as the reference
pins its own GEMMs; the operands themselves are pinned bit for bit by quant_oracle.
"""
from __future__ import annotations

import math

import numpy as np

from . import quant_oracle as qo


def dequant_operand(q, sf_blocked, ts, fmt: str, R: int, K: int) -> np.ndarray:
    """fp32 [R, K] from codes + the blocked scale tensor (flat or 5-D) (+ ts for nv4)."""
    nb = K // qo.VEC[fmt]
    s2 = qo.from_blocked(np.asarray(sf_blocked, dtype=np.uint8).reshape(-(-R // 128), -(-nb // 4), 32, 4, 4), R, nb)
    return qo.dequant(q, s2, ts, fmt)


def matmul_ref(a: np.ndarray, w: np.ndarray) -> np.ndarray:
    """a [M,K] @ w [N,K]^T in float64."""
    return a.astype(np.float64) @ w.astype(np.float64).T


def gelu_erf(x: np.ndarray) -> np.ndarray:
    from scipy.special import erf

    x = np.asarray(x, dtype=np.float64)
    return 0.5 * x * (1.0 + erf(x / math.sqrt(2.0)))


def epi_res(acc, bias, gamma, R):
    return np.asarray(R, dtype=np.float64) + np.asarray(gamma, dtype=np.float64) * (acc + np.asarray(bias, dtype=np.float64))


def epi_rope(y, sin, cos, Ntok: int, prefix: int, H: int) -> np.ndarray:
    """y [M, 3*H*64] (bias already added) -> [3, B, Ntok, H, 64] with rotary embedding on q, k of tokens >= prefix:
    x*cos + rotate_half(x)*sin, rotate_half = cat(-x[32:], x[:32])."""
    M = y.shape[0]
    B = M // Ntok
    t = np.asarray(y, dtype=np.float64).reshape(B, Ntok, 3, H, 64).transpose(2, 0, 1, 3, 4).copy()
    s = np.asarray(sin, dtype=np.float64)[: Ntok - prefix, None, :]
    c = np.asarray(cos, dtype=np.float64)[: Ntok - prefix, None, :]
    for which in (0, 1):
        x = t[which][:, prefix:]
        rot = np.concatenate([-x[..., 32:], x[..., :32]], axis=-1)
        t[which][:, prefix:] = x * c + rot * s
    return t


def rel_fro(a, b) -> float:
    a = np.asarray(a, dtype=np.float64)
    b = np.asarray(b, dtype=np.float64)
    return float(np.linalg.norm(a - b) / max(np.linalg.norm(b), 1e-30))
