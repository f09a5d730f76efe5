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
from ._lib import KF_DT, KF_EPI, KF_FMT, KF_G_GELU, KF_Q_GELU, KF_Q_RECIP_DIV, KF_Q_ROUND_BF16, GemmParams, KfError, check

VEC = {"mx8": 32, "nv4": 16, "mx4": 32}

# Launch accounting used by the benchmark: LAUNCHES counts every kernel launched through this module; when TIMING is
# a dict every launch is bracketed by CUDA events on the launching stream under its kernel-class name and BYTES
# accumulates the algorithmic bytes of the memory-bound classes.
LAUNCHES = 0
TIMING = None
BYTES: dict = {}


def _run(name: str, call, nbytes: int = 0) -> None:
    global LAUNCHES
    LAUNCHES += 1
    if TIMING is not None:
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        st = call()
        e1.record()
        TIMING.setdefault(name, []).append((e0, e1))
        if nbytes:
            BYTES[name] = BYTES.get(name, 0) + nbytes
    else:
        st = call()
    check(st, name)
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
        self.sf = torch.zeros(sf_bytes(M, K, fmt), dtype=torch.uint8, device=device)   # padded rows stay zero
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
    _run("quant_rows", lambda: _lib.lib().kf_quant_rows(KF_FMT[out.fmt], _DT[x.dtype], x.data_ptr(), x.stride(0), out.M, out.K, _ptr(out.ts),
                                                        _ptr(bias), _flags(gelu, round_bf16, recip_div), out.q.data_ptr(), out.sf.data_ptr(), _stream()),
         x.numel() * x.element_size() + out.q.numel() + out.sf.numel())
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
    _run("ln_quant", lambda: _lib.lib().kf_ln_quant(KF_FMT[out.fmt], x.data_ptr(), w.data_ptr(), b.data_ptr(), float(eps), M, d, _ptr(out.ts),
                                                    _flags(False, round_bf16, recip_div), out.q.data_ptr(), out.sf.data_ptr(), _ptr(y_dbg), _stream()),
         x.numel() * 4 + out.q.numel() + out.sf.numel())
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
    _run("ln_rows", lambda: _lib.lib().kf_ln_rows(x.data_ptr(), w.data_ptr(), b.data_ptr(), float(eps), M, d, _DT[dtype], y.data_ptr(), _stream()))
    return y


ln_bf16 = ln_rows


# ------------------------------------------------------------------------------------------------ weights and GEMMs
def set_pdl(on: bool) -> None:
    """Programmatic dependent launch for the block kernels (off by default); results are the same either way.
    Counterpart: set_pdl (infer-opt/round13_mxfp8_full/impl/mx13.cu:282)."""
    check(_lib.lib().kf_set_pdl(1 if on else 0), "kf_set_pdl")


def check_device_error() -> None:
    """synchronises and raises if a kernel's bounded wait ran out (no reference counterpart)."""
    check(_lib.lib().kf_check_device_error(), "kf_check_device_error")


class QWeight:
    """Weight [N, K] (nn.Linear layout) quantised once along K with 1-D block scales; fmt "bf16" keeps a bf16 copy.
    nv4: exact per-tensor scale ts = amax/(6*448) computed once on the host cores (IEEE division).
    Counterparts: MXW (infer-opt/round13_mxfp8_full/impl/mx13.py:74-84), Lin / FP4Linear weights
    (infer-opt/round14_fp4_full/impl/stack14b.py:55-66, fp4util.py:114-131)."""

    def __init__(self, W: torch.Tensor, fmt: str, ts: Optional[torch.Tensor] = None):
        _need_cuda(W)
        self.N, self.K = W.shape
        self.fmt = fmt
        if fmt == "bf16":
            self.q = W.to(torch.bfloat16).contiguous()
            self.sf = None
            self.ts = None
            return
        Wf = W.float().contiguous()
        buf = ActBuf(self.N, self.K, fmt, device=W.device)
        if fmt == "nv4":
            if ts is None:
                import numpy as np

                amax = np.float32(Wf.abs().amax().item())
                ts = torch.tensor([amax / np.float32(2688.0) if amax > 0 else 1.0], dtype=torch.float32)
            buf.ts.copy_(ts.reshape(1))
        quant_rows(Wf, buf)
        self.q, self.sf, self.ts = buf.q, buf.sf, buf.ts


MXW = QWeight


def _gemm(a, W: QWeight, epi: str, *, bias=None, gamma=None, R=None, C=None, sin=None, cos=None, out: Optional[ActBuf] = None,
          out_dtype=torch.bfloat16, gelu=False, round_bf16=False, recip_div=False, Ntok=0, prefix=0, H=0, tag="block", pre_round=False,
          fast_nv4=False, y_dbg=None, rope_half=False, row_map=None):
    p = GemmParams()
    if isinstance(a, ActBuf):
        if a.fmt != W.fmt or a.K != W.K:
            raise KfError(f"gemm: operand mismatch A {a.fmt} K={a.K} vs W {W.fmt} K={W.K}")
        M = a.M
        p.A, p.SFA, p.ts_a = a.q.data_ptr(), a.sf.data_ptr(), _ptr(a.ts)
    else:
        if W.fmt != "bf16" or a.dtype != torch.bfloat16 or a.dim() != 2 or not a.is_contiguous() or a.shape[1] != W.K:
            raise KfError("gemm: a plain tensor operand must be contiguous bf16 [M, K] with a bf16 weight")
        _need_cuda(a)
        M = a.shape[0]
        p.A = a.data_ptr()
    p.fmt, p.epi, p.M, p.N, p.K = KF_FMT[W.fmt], KF_EPI[epi], M, W.N, W.K
    p.W, p.SFW, p.ts_w = W.q.data_ptr(), _ptr(W.sf), _ptr(W.ts)
    p.out_dtype = _DT[out_dtype]
    p.flags = (KF_G_GELU if gelu else 0) | (KF_Q_ROUND_BF16 if round_bf16 else 0) | (KF_Q_RECIP_DIV if recip_div else 0) \
        | (_lib.KF_G_PRE_ROUND_BF16 if pre_round else 0) | (_lib.KF_Q_FAST_NV4 if fast_nv4 else 0) | (_lib.KF_G_ROPE_HALF if rope_half else 0)
    p.Ntok, p.prefix, p.H = Ntok, prefix, H
    _need_cuda(bias, gamma, R, C, sin, cos, y_dbg)
    p.bias, p.gamma, p.R, p.sin, p.cos, p.C = _ptr(bias), _ptr(gamma), _ptr(R), _ptr(sin), _ptr(cos), _ptr(C)
    p.y_dbg = _ptr(y_dbg)
    if row_map is not None:
        p.out_row_group, p.out_row_stride, p.out_row_offset = row_map
    if out is not None:
        p.out_fmt, p.Qo, p.SFo, p.tso = KF_FMT[out.fmt], out.q.data_ptr(), out.sf.data_ptr(), _ptr(out.ts)
    _run(f"gemm_{tag}_{W.fmt}", lambda: _lib.lib().kf_gemm_bs(p, _stream()))


def _f32c(t, n, what):
    if t is not None and (t.dtype != torch.float32 or not t.is_contiguous() or t.numel() != n):
        raise KfError(f"gemm: {what} must be contiguous fp32 with {n} elements")


def gemm_plain(a, W: QWeight, bias=None, *, gelu: bool = False, out_dtype=torch.bfloat16, out: Optional[torch.Tensor] = None,
               tag: str = "block", pre_round: bool = False) -> torch.Tensor:
    """[M, N] = act(a @ W^T (* ts) + bias) in bf16 / f16 / f32 (mm, gemm_plain, fwd_bias, fwd_gelu, fwd_plain)."""
    M = a.M if isinstance(a, ActBuf) else a.shape[0]
    _f32c(bias, W.N, "bias")
    if out is None:
        out = torch.empty(M, W.N, dtype=out_dtype, device=W.q.device)
    _gemm(a, W, "plain", bias=bias, C=out, out_dtype=out.dtype, gelu=gelu, tag=tag, pre_round=pre_round)
    return out


mm = gemm_plain


def bmm_nt(a: torch.Tensor, w: torch.Tensor, out: Optional[torch.Tensor] = None, tag: str = "mask") -> torch.Tensor:
    """out[b] = a[b] @ w[b]^T for bf16 a [B, Q, K] and w [B, P, K] in one launch (P a multiple of 128): the mask product
    torch.bmm(h, u.transpose(1, 2)) of the head (infer-opt/round11_attn_tier0/impl/head11.py:95).  Bit-identical to B
    gemm_plain calls; one launch fills the SMs where a single image leaves a partial round of tiles."""
    _need_cuda(a, w)
    if a.dim() != 3 or w.dim() != 3 or a.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or not a.is_contiguous() or not w.is_contiguous() \
            or a.shape[0] != w.shape[0] or a.shape[2] != w.shape[2]:
        raise KfError("bmm_nt: a [B, Q, K] and w [B, P, K] must be contiguous bf16 with equal B and K")
    B, Q, K = a.shape
    P = w.shape[1]
    if out is None:
        out = torch.empty(B, Q, P, dtype=torch.bfloat16, device=a.device)
    elif out.shape != (B, Q, P) or out.dtype != torch.bfloat16 or not out.is_contiguous():
        raise KfError(f"bmm_nt: out must be contiguous bf16 [{B}, {Q}, {P}]")
    p = GemmParams()
    p.fmt, p.epi, p.M, p.N, p.K = KF_FMT["bf16"], KF_EPI["plain"], B * Q, P, K
    p.A, p.W, p.C = a.data_ptr(), w.data_ptr(), out.data_ptr()
    p.out_dtype = _DT[torch.bfloat16]
    p.batch, p.a_rows_per_batch, p.w_rows_per_batch = B, Q, P
    _run(f"gemm_{tag}_bf16", lambda: _lib.lib().kf_gemm_bs(p, _stream()))
    return out


def gemm_res(a, W: QWeight, bias, gamma, res: torch.Tensor, out: Optional[torch.Tensor] = None, row_map=None) -> torch.Tensor:
    """fp32 [M, N] = res + gamma * (a @ W^T (* ts) + bias)   (proj / fc2; gemm_res, fwd_res).
    row_map = (group, stride, offset): row m of the result goes to row (m // group) * stride + offset + m % group of `out`
    (a longer token stream: the rows of each image land behind `offset` rows that are filled separately); not in place."""
    M = a.M if isinstance(a, ActBuf) else a.shape[0]
    _f32c(bias, W.N, "bias")
    _f32c(gamma, W.N, "gamma")
    _f32c(res, M * W.N, "res")
    if out is None:
        if row_map is not None:
            raise KfError("gemm_res: a row mapping needs the output tensor")
        out = torch.empty_like(res)
    if out.dtype != torch.float32 or not out.is_contiguous():
        raise KfError("gemm_res: out must be contiguous fp32")
    if row_map is not None:
        group, stride, offset = row_map
        if M % group or out.numel() != (M // group) * stride * W.N or offset + group > stride:
            raise KfError(f"gemm_res: row mapping {row_map} does not fit M={M} rows into {out.numel() // W.N} output rows")
    _gemm(a, W, "res", bias=bias, gamma=gamma, R=res, C=out, out_dtype=torch.float32, row_map=row_map)
    return out


def broadcast_rows(src: torch.Tensor, dst: torch.Tensor, row_offset: int) -> torch.Tensor:
    """dst[b, row_offset : row_offset + R, :] = src [R, d] for every image b of the fp32 token stream dst [B, Ntok, d]."""
    _need_cuda(src, dst)
    if src.dtype != torch.float32 or dst.dtype != torch.float32 or not src.is_contiguous() or not dst.is_contiguous() or dst.dim() != 3 or src.shape[-1] != dst.shape[2]:
        raise KfError("broadcast_rows: src [R, d] and dst [B, Ntok, d] must be contiguous fp32")
    R = src.numel() // dst.shape[2]
    _run("broadcast_rows", lambda: _lib.lib().kf_broadcast_rows(src.data_ptr(), dst.data_ptr(), R, dst.shape[2], dst.shape[0], dst.shape[1] * dst.shape[2], row_offset, _stream()))
    return dst


def rope_tables_are_half(sin: torch.Tensor, cos: torch.Tensor) -> bool:
    """True when columns 32..63 of both tables repeat columns 0..31 (the axial tables of DINOv3: the angle vector concatenated
    with itself).  A host-side check (it synchronises): call it once when the tables are built, not per launch."""
    return bool(torch.equal(sin[:, :32], sin[:, 32:]) and torch.equal(cos[:, :32], cos[:, 32:]))


def qkv_rope(a, W: QWeight, bias, sin, cos, Ntok: int, prefix: int, H: int, out_dtype=torch.bfloat16, half_tables: bool = False) -> torch.Tensor:
    """a [M=B*Ntok, d] -> physical [3, B, Ntok, H, 64] (bias + RoPE in fp32 on q and k of tokens >= prefix).
    half_tables=True promises rope_tables_are_half(sin, cos): the kernel then keeps a tile's table rows in shared memory."""
    M = a.M if isinstance(a, ActBuf) else a.shape[0]
    _f32c(bias, W.N, "bias")
    if sin.dtype != torch.float32 or cos.dtype != torch.float32 or not sin.is_contiguous() or not cos.is_contiguous() \
            or sin.shape[-1] != 64 or sin.shape[0] < Ntok - prefix or cos.shape != sin.shape:
        raise KfError("qkv_rope: sin / cos must be contiguous fp32 [>= Ntok - prefix, 64]")
    if M % Ntok:
        raise KfError("qkv_rope: M must be a multiple of Ntok")
    out = torch.empty(3, M // Ntok, Ntok, H, 64, dtype=out_dtype, device=W.q.device)
    _gemm(a, W, "rope", bias=bias, sin=sin, cos=cos, C=out, out_dtype=out_dtype, Ntok=Ntok, prefix=prefix, H=H, rope_half=half_tables)
    return out


def gemm_gelu_q(a, W: QWeight, bias, out: ActBuf, *, round_bf16: bool = False, recip_div: bool = False, fast_nv4: bool = False,
                y_dbg: Optional[torch.Tensor] = None) -> ActBuf:
    """out = quantise(gelu(a @ W^T (* ts) + bias)) in out.fmt: fc1 writes fc2's operand and blocked scales directly.
    The quantisation follows the bit specification (IEEE divisions); fast_nv4=True selects approximate reciprocals for an
    nv4 output.  y_dbg (fp32 [M, N], optional) receives the values that were quantised."""
    M = a.M if isinstance(a, ActBuf) else a.shape[0]
    _f32c(bias, W.N, "bias")
    if (out.M, out.K) != (M, W.N):
        raise KfError(f"gemm_gelu_q: out must be [{M}, {W.N}], got [{out.M}, {out.K}]")
    _f32c(y_dbg, M * W.N, "y_dbg")
    _gemm(a, W, "quant", bias=bias, out=out, round_bf16=round_bf16, recip_div=recip_div, fast_nv4=fast_nv4, y_dbg=y_dbg)
    return out


# ------------------------------------------------------------------------------------------------ attention
def attn_fwd(qkv: torch.Tensor, pre: float = 1.0, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """qkv contiguous [3, B, N, H, 64] bf16 | f16 (RoPE applied) -> O [B, N, H*64] of the same dtype.
    Counterpart: attn16_fwd(qkv, kind, pre) (infer-opt/round12_lowp_stack/impl/attn16o.cu:389-404)."""
    _need_cuda(qkv)
    if qkv.dim() != 5 or qkv.shape[0] != 3 or qkv.shape[4] != 64 or not qkv.is_contiguous() or qkv.dtype not in (torch.bfloat16, torch.float16):
        raise KfError("attn_fwd: qkv must be contiguous [3, B, N, H, 64] bf16 or f16")
    _, B, N, H, _ = qkv.shape
    if out is None:
        out = torch.empty(B, N, H * 64, dtype=qkv.dtype, device=qkv.device)
    _run("attn_fwd", lambda: _lib.lib().kf_attn_fwd(_DT[qkv.dtype], qkv.data_ptr(), out.data_ptr(), B, N, H, float(pre), _stream()))
    return out


attn16_fwd = attn_fwd


def attn_fwd_quant(qkv: torch.Tensor, out: ActBuf, pre: float = 1.0, recip_div: bool = False) -> ActBuf:
    """attention forward whose output is written directly as the quantised [B*N, H*64] operand `out` (codes + blocked
    scales; out.ts is the static nv4 scale): attn16_fwd + quant_rows in one kernel."""
    _need_cuda(qkv, out.q)
    if qkv.dim() != 5 or qkv.shape[0] != 3 or qkv.shape[4] != 64 or not qkv.is_contiguous() or qkv.dtype not in (torch.bfloat16, torch.float16):
        raise KfError("attn_fwd_quant: qkv must be contiguous [3, B, N, H, 64] bf16 or f16")
    _, B, N, H, _ = qkv.shape
    if (out.M, out.K) != (B * N, H * 64):
        raise KfError(f"attn_fwd_quant: out must be [{B * N}, {H * 64}], got [{out.M}, {out.K}]")
    _run("attn_fwd", lambda: _lib.lib().kf_attn_fwd_quant(_DT[qkv.dtype], qkv.data_ptr(), B, N, H, float(pre), KF_FMT[out.fmt], out.q.data_ptr(),
                                                          out.sf.data_ptr(), _ptr(out.ts), KF_Q_RECIP_DIV if recip_div else 0, _stream()))
    return out


# ------------------------------------------------------------------------------------------------ patch embed / head / pre / post
def gemm_tokens(a: torch.Tensor, W: QWeight, bias, out: torch.Tensor, rows_per_image: int, tokens_per_image: int, row_offset: int,
                round_bf16: bool = False) -> torch.Tensor:
    """patch-embed GEMM: a bf16 [B*P, K] @ W^T + bias written as fp32 rows row_offset.. of every image of the token
    stream out [B, tokens_per_image, N] (counterpart: PatchEmbedGemm, infer-opt/round11_attn_tier0/impl/patch_embed.py:34-53)."""
    if out.dtype != torch.float32 or not out.is_contiguous():
        raise KfError("gemm_tokens: out must be contiguous fp32")
    p = GemmParams()
    p.fmt, p.epi, p.M, p.N, p.K = KF_FMT["bf16"], KF_EPI["plain"], a.shape[0], W.N, W.K
    p.A, p.W, p.bias, p.C = a.data_ptr(), W.q.data_ptr(), _ptr(bias), out.data_ptr()
    p.out_dtype = KF_DT["f32"]
    p.flags = _lib.KF_G_ROUND_BF16 if round_bf16 else 0
    p.out_row_group, p.out_row_stride, p.out_row_offset = rows_per_image, tokens_per_image, row_offset
    _run("gemm_patch_bf16", lambda: _lib.lib().kf_gemm_bs(p, _stream()))
    return out


PATCH_STATIC_MAX_ROWS = 4096


def patch_embed_static(x: torch.Tensor, W: QWeight, bias, out: torch.Tensor, row_offset: int, round_bf16: bool = False) -> torch.Tensor:
    """Patch embedding for callers that must not allocate: x bf16 [B, 3, S, S] -> rows row_offset.. of every image of the fp32
    token stream out [B, tokens_per_image, d], through the library's built-in scratch array instead of an im2col tensor
    (the same bits as gemm_tokens(im2col_patch16(x), ...)).  At most PATCH_STATIC_MAX_ROWS patch rows per call; calls that
    overlap on the GPU race on the shared array; the first call on a device should come before any stream capture."""
    _need_cuda(x, W.q, bias, out)
    if x.dtype != torch.bfloat16 or x.dim() != 4 or x.shape[1] != 3 or x.shape[2] != x.shape[3] or not x.is_contiguous():
        raise KfError("patch_embed_static: x must be contiguous bf16 [B, 3, S, S]")
    if W.fmt != "bf16" or W.K != 768 or out.dtype != torch.float32 or not out.is_contiguous() or out.dim() != 3 or out.shape[2] != W.N:
        raise KfError("patch_embed_static: W must be a bf16 [d, 768] weight and out contiguous fp32 [B, tokens_per_image, d]")
    B, _, S, _ = x.shape
    _run("patch_embed_static", lambda: _lib.lib().kf_patch_embed_static(x.data_ptr(), W.q.data_ptr(), _ptr(bias), out.data_ptr(), B, S, W.N, out.shape[1], row_offset,
                                                                        _lib.KF_G_ROUND_BF16 if round_bf16 else 0, _stream()))
    return out


def im2col_patch16(x: torch.Tensor) -> torch.Tensor:
    """x bf16 [B, 3, S, S] -> bf16 [B*(S/16)^2, 768]."""
    _need_cuda(x)
    if x.dtype != torch.bfloat16 or x.dim() != 4 or x.shape[1] != 3 or x.shape[2] != x.shape[3] or not x.is_contiguous():
        raise KfError("im2col_patch16: x must be contiguous bf16 [B, 3, S, S]")
    B, _, S, _ = x.shape
    out = torch.empty(B * (S // 16) ** 2, 768, dtype=torch.bfloat16, device=x.device)
    _run("im2col_patch16", lambda: _lib.lib().kf_im2col_patch16(x.data_ptr(), out.data_ptr(), B, S, _stream()))
    return out


def ln_tail(x: torch.Tensor, w, b, eps: float, Q: int, npre: int, wcls: Optional[torch.Tensor] = None, bcls: Optional[torch.Tensor] = None):
    """final LayerNorm + gather: x fp32 [B, Ntok, d] -> (queries bf16 [B*Q, d], patches bf16 [B*(Ntok-Q-npre), d]), and with
    wcls bf16 [ncls1, d] / bcls fp32 [ncls1] the class logits bf16 [B*Q, ncls1] of the query rows as a third result."""
    _need_cuda(x, w, b, wcls, bcls)
    B, Ntok, d = x.shape
    if x.dtype != torch.float32 or not x.is_contiguous():
        raise KfError("ln_tail: x must be contiguous fp32")
    qb = torch.empty(B * Q, d, dtype=torch.bfloat16, device=x.device)
    xb = torch.empty(B * (Ntok - Q - npre), d, dtype=torch.bfloat16, device=x.device)
    cl, ncls1 = None, 0
    if wcls is not None:
        if wcls.dtype != torch.bfloat16 or not wcls.is_contiguous() or wcls.shape[1] != d or bcls is None or bcls.dtype != torch.float32 or bcls.numel() != wcls.shape[0]:
            raise KfError("ln_tail: wcls must be contiguous bf16 [ncls1, d] and bcls fp32 [ncls1]")
        ncls1 = wcls.shape[0]
        cl = torch.empty(B * Q, ncls1, dtype=torch.bfloat16, device=x.device)
    _run("ln_tail", lambda: _lib.lib().kf_ln_tail(x.data_ptr(), w.data_ptr(), b.data_ptr(), float(eps), B, Ntok, Q, npre, d, qb.data_ptr(), xb.data_ptr(),
                                                  _ptr(wcls), _ptr(bcls), ncls1, _ptr(cl), _stream()))
    return (qb, xb) if wcls is None else (qb, xb, cl)


def dw_ln(g: torch.Tensor, bias, dww, lnw, lnb, B: int, Hs: int, Ws: int, eps: float, pre_act: bool = False) -> torch.Tensor:
    """ScaleBlock tail: g bf16 [B*Hs*Ws, 4C] -> bf16 [B, 2Hs, 2Ws, C] (dw_ln_launch, head11.py:60-67).
    pre_act=True: g already is bf16(gelu(conv + bias)) (fused into the GEMM epilogue), bias may be None."""
    C = g.shape[1] // 4
    _need_cuda(g, dww, lnw, lnb)
    if g.dtype != torch.bfloat16 or not g.is_contiguous() or g.shape[0] != B * Hs * Ws or dww.shape != (9, C) or (bias is None and not pre_act):
        raise KfError("dw_ln: g must be contiguous bf16 [B*Hs*Ws, 4C] and dww fp32 [9, C]")
    out = torch.empty(B, 2 * Hs, 2 * Ws, C, dtype=torch.bfloat16, device=g.device)
    _run("dw_ln", lambda: _lib.lib().kf_dw_ln(g.data_ptr(), _ptr(bias), dww.data_ptr(), lnw.data_ptr(), lnb.data_ptr(), out.data_ptr(), B, Hs, Ws, C,
                                              float(eps), 1 if pre_act else 0, _stream()))
    return out


def semantic(mask_logits: torch.Tensor, class_logits: torch.Tensor, want_scores: bool = False):
    """mask_logits bf16 [B, Q, h, w], class_logits bf16 [B, Q, ncls+1] -> (labels uint8 [B, h, w], scores fp32 [B, ncls+1, h, w] | None)."""
    _need_cuda(mask_logits, class_logits)
    B, Q, h, w = mask_logits.shape
    ncls1 = class_logits.shape[-1]
    if mask_logits.dtype != torch.bfloat16 or class_logits.dtype != torch.bfloat16 or not mask_logits.is_contiguous() or not class_logits.is_contiguous():
        raise KfError("semantic: logits must be contiguous bf16")
    labels = torch.empty(B, h, w, dtype=torch.uint8, device=mask_logits.device)
    scores = torch.empty(B, ncls1, h, w, dtype=torch.float32, device=mask_logits.device) if want_scores else None
    _run("semantic", lambda: _lib.lib().kf_semantic(mask_logits.data_ptr(), class_logits.data_ptr(), B, Q, ncls1 - 1, h * w, _ptr(scores),
                                                    labels.data_ptr(), _stream()))
    return labels, scores


IMAGENET_MEAN = (0.485, 0.456, 0.406)
IMAGENET_STD = (0.229, 0.224, 0.225)


def resize_norm(frames: torch.Tensor, size: int, mean=IMAGENET_MEAN, std=IMAGENET_STD, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """frames uint8 [B, Hi, Wi, 3] -> bf16 [B, 3, size, size] (antialiased bilinear + normalisation)."""
    import ctypes as C

    _need_cuda(frames)
    if frames.dtype != torch.uint8 or frames.dim() != 4 or frames.shape[3] != 3 or not frames.is_contiguous():
        raise KfError("resize_norm: frames must be contiguous uint8 [B, H, W, 3]")
    B, Hi, Wi, _ = frames.shape
    if out is None:
        out = torch.empty(B, 3, size, size, dtype=torch.bfloat16, device=frames.device)
    m, s = (C.c_float * 3)(*mean), (C.c_float * 3)(*std)
    _run("resize_norm", lambda: _lib.lib().kf_resize_norm(frames.data_ptr(), out.data_ptr(), B, Hi, Wi, size, m, s, _stream()))
    return out


def tensor_peak_tflops(fmt: str, n: int = 256, iters: int = 4096, reps: int = 5, sf_copies: int = 0) -> float:
    """measured tcgen05 instruction-rate ceiling (TFLOP/s) for operand format fmt at M=128, N=n (best of reps)."""
    import ctypes as C

    fl = C.c_double(0.0)
    L = _lib.lib()
    best = 0.0
    for _ in range(reps + 1):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        check(L.kf_tensor_peak_probe(KF_FMT[fmt], n, iters, sf_copies, C.byref(fl), _stream()), "kf_tensor_peak_probe")
        e1.record()
        e1.synchronize()
        best = max(best, fl.value / (e0.elapsed_time(e1) * 1e-3) / 1e12)
    return best


def smem_fill_rate_gbs(span_bytes: int, stage_bytes: int = 49152, iters: int = 2048, reps: int = 5) -> float:
    """measured rate (GB/s, all SMs together) at which bulk copies fill shared memory from a window of span_bytes of
    global memory that fits L2 (best of reps)."""
    import ctypes as C

    src = torch.empty(span_bytes, dtype=torch.uint8, device="cuda").zero_()
    nb = C.c_double(0.0)
    L = _lib.lib()
    best = 0.0
    for _ in range(reps + 1):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        check(L.kf_fill_rate_probe(src.data_ptr(), span_bytes, stage_bytes, iters, C.byref(nb), _stream()), "kf_fill_rate_probe")
        e1.record()
        e1.synchronize()
        best = max(best, nb.value / (e0.elapsed_time(e1) * 1e-3) / 1e9)
    check_device_error()
    return best
