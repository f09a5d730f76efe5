"""Operator layer: quantised operand containers and the fused operators, mirroring the reference's L6 surface.

Reference counterparts (paths relative to the reference checkout):
    ActBuf / act_buf / MXW            infer-opt/round13_mxfp8_full/impl/mx13.py:53-84
    ln_mx8 / quant_rows / gelu_quant  infer-opt/round13_mxfp8_full/impl/mx13.cu:299-330
    lnq / quantx                      infer-opt/round14_fp4_full/impl/lnq14.cu:158-188
    ln_bf16                           infer-opt/round14_fp4_full/impl/ln14.cu:67
    FQ / Site / Calib                 infer-opt/round14_fp4_full/impl/fp4util.py:47-77

Every operator launches on torch's current CUDA stream through the C-ABI, never synchronises and never
falls back to another implementation: a missing library or a failed launch raises KfError.
torch is used for device memory and streams only.
"""
from __future__ import annotations

from typing import Optional

import torch

from . import _lib
from ._lib import KF_DT, KF_FMT, KF_Q_GELU, KF_Q_RECIP_DIV, KF_Q_ROUND_BF16, KfError, check

VEC = {"mx8": 32, "nv4": 16, "mx4": 32}
_DT = {torch.float32: KF_DT["f32"], torch.bfloat16: KF_DT["bf16"], torch.float16: KF_DT["f16"]}


def pad128(n: int) -> int:
    return -(-n // 128) * 128


def sf_bytes(R: int, K: int, fmt: str) -> int:
    n = _lib.lib().kf_sf_bytes(R, K, KF_FMT[fmt])
    if n < 0:
        check(int(n), "kf_sf_bytes")
    return int(n)


def code_cols(K: int, fmt: str) -> int:
    return K if fmt == "mx8" else K // 2


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _ptr(t: Optional[torch.Tensor]) -> int:
    return 0 if t is None else t.data_ptr()


def _need_cuda(*ts):
    for t in ts:
        if t is not None and not t.is_cuda:
            raise KfError("operands must live on a CUDA device (there is no CPU path)")


class ActBuf:
    """Quantised [M, K] operand: codes q (uint8, [M, K] for mx8, [M, K/2] packed nibbles for nv4 / mx4), blocked
    scales sf (uint8, [ceil(M/128), K/(4 vec), 32, 4, 4] flattened) and, for nv4, the fp32 per-tensor scale ts [1]."""

    __slots__ = ("M", "K", "fmt", "q", "sf", "ts")

    def __init__(self, M: int, K: int, fmt: str = "mx8", device="cuda", ts: Optional[torch.Tensor] = None):
        self.M, self.K, self.fmt = M, K, fmt
        self.q = torch.empty(M, code_cols(K, fmt), dtype=torch.uint8, device=device)
        self.sf = torch.empty(sf_bytes(M, K, fmt), dtype=torch.uint8, device=device)
        self.ts = ts if ts is not None else (torch.ones(1, dtype=torch.float32, device=device) if fmt == "nv4" else None)


FQ = ActBuf   # the FP4 stacks call the same container FQ (fp4util.py:54-58)

_POOL: dict = {}


def act_buf(M: int, K: int, fmt: str = "mx8", device="cuda", slot: int = 0) -> ActBuf:
    """persistent operand buffer shared by every layer of one shape (the stream is sequential)."""
    key = (M, K, fmt, slot, str(device))
    if key not in _POOL:
        _POOL[key] = ActBuf(M, K, fmt, device)
    return _POOL[key]


def _flags(gelu=False, round_bf16=False, recip_div=False) -> int:
    return (KF_Q_GELU if gelu else 0) | (KF_Q_ROUND_BF16 if round_bf16 else 0) | (KF_Q_RECIP_DIV if recip_div else 0)


def quant_rows(x: torch.Tensor, out: ActBuf, *, bias: Optional[torch.Tensor] = None, gelu: bool = False,
               round_bf16: bool = False, recip_div: bool = False) -> ActBuf:
    """x [M, K] f32 | bf16 | f16 (last dim contiguous) -> out (codes + blocked scales), format out.fmt.
    gelu=True applies gelu_erf(x + bias) first (the reference's gelu_quant)."""
    _need_cuda(x, out.q, bias)
    if x.dim() != 2 or x.stride(1) != 1 or x.shape != (out.M, out.K):
        raise KfError(f"quant_rows: x must be [M={out.M}, K={out.K}] with a contiguous last dim, got {tuple(x.shape)}")
    if x.dtype not in _DT:
        raise KfError(f"quant_rows: unsupported dtype {x.dtype}")
    st = _lib.lib().kf_quant_rows(KF_FMT[out.fmt], _DT[x.dtype], x.data_ptr(), x.stride(0), out.M, out.K, _ptr(out.ts),
                                  _ptr(bias), _flags(gelu, round_bf16, recip_div), out.q.data_ptr(), out.sf.data_ptr(), _stream())
    check(st, "kf_quant_rows")
    return out


def gelu_quant(y: torch.Tensor, bias: torch.Tensor, out: ActBuf, **kw) -> ActBuf:
    return quant_rows(y, out, bias=bias, gelu=True, **kw)


def quantx(x: torch.Tensor, out: ActBuf, **kw) -> ActBuf:
    return quant_rows(x, out, **kw)


def ln_quant(x: torch.Tensor, w: torch.Tensor, b: torch.Tensor, eps: float, out: ActBuf, *, round_bf16: bool = False,
             recip_div: bool = False, y_dbg: Optional[torch.Tensor] = None) -> ActBuf:
    """LayerNorm of the fp32 residual stream x [..., d] fused with quantisation into out (ln_mx8 / lnq)."""
    _need_cuda(x, w, b, out.q)
    d = x.shape[-1]
    M = x.numel() // d
    if x.dtype != torch.float32 or not x.is_contiguous() or (M, d) != (out.M, out.K):
        raise KfError(f"ln_quant: x must be contiguous fp32 [M={out.M}, d={out.K}], got {tuple(x.shape)} {x.dtype}")
    st = _lib.lib().kf_ln_quant(KF_FMT[out.fmt], x.data_ptr(), w.data_ptr(), b.data_ptr(), float(eps), M, d, _ptr(out.ts),
                                _flags(False, round_bf16, recip_div), out.q.data_ptr(), out.sf.data_ptr(), _ptr(y_dbg), _stream())
    check(st, "kf_ln_quant")
    return out


def ln_mx8(x, w, b, out: ActBuf, eps: float, **kw) -> ActBuf:
    return ln_quant(x, w, b, eps, out, **kw)


def lnq(x, w, b, eps: float, out: ActBuf, **kw) -> ActBuf:
    return ln_quant(x, w, b, eps, out, **kw)


def ln_rows(x: torch.Tensor, w: torch.Tensor, b: torch.Tensor, eps: float, dtype=torch.bfloat16) -> torch.Tensor:
    """LayerNorm of fp32 x [..., d] to a bf16 / f16 tensor of the same shape (ln_bf16 / ln16)."""
    _need_cuda(x, w, b)
    d = x.shape[-1]
    M = x.numel() // d
    if x.dtype != torch.float32 or not x.is_contiguous():
        raise KfError("ln_rows: x must be contiguous fp32")
    y = torch.empty(x.shape, dtype=dtype, device=x.device)
    st = _lib.lib().kf_ln_rows(x.data_ptr(), w.data_ptr(), b.data_ptr(), float(eps), M, d, _DT[dtype], y.data_ptr(), _stream())
    check(st, "kf_ln_rows")
    return y


ln_bf16 = ln_rows
