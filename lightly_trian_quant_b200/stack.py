"""Stack plugin: whole-model low-precision model_fn for DINOv3 ViT + EoMT on B200, one variant per format.

Plugin contract of the reference's speed harness (infer-opt/round12_lowp_stack/speed12.py:5-9,45-50;
infer-opt/round13_mxfp8_full/plug13.py:12-17; infer-opt/round14_fp4_full/plug14.py:10-15):

    PREFIXES = ("b200",)
    make_variant(name, model, variant) -> (model_fn, pipeline_cls)
    model_fn(x: bf16 [B, 3, S, S]) -> (mask_logits bf16 [B, Q, S/4, S/4], class_logits bf16 [B, Q, classes+1])
        capture-safe after the first (eager) call, no host sync, static shapes; model_fn._keepalive holds the weights

Variant grammar  base[+flag...]:   base in b200_mx8 | b200_nv4 | b200_mx4 | b200_bf16
    +s<N>      input side in pixels (default 640)
    +fp32pts   quantise the fp32 LN / GELU values directly (the rounding points of the reference's own-kernel stacks,
               infer-opt/round13_mxfp8_full/impl/stack13.py:93-121); default = round to bf16 first, the rounding points of the
               emulated model (infer-opt/round10_lowp_probe/impl/emu.py:260-333)
    +f16attn   q, k, v and the attention output in fp16 instead of bf16
    +bf16head  keep the two ConvTranspose GEMMs of the head in bf16 instead of the block-scaled format

Kernel sequence per block (7 launches), the decomposition of infer-opt/round14_fp4_full/impl/stack14b.py:85-130:
    ln_quant | qkv GEMM (+bias +RoPE +[3,B,N,H,64]) | attention (+quantise-out) | proj GEMM (+bias, gamma, residual) |
    ln_quant | fc1 GEMM (+bias +GELU +quantise-out) | fc2 GEMM (+bias, gamma, residual)
NVFP4 activations use static per-tensor scales measured on the first call (headroom 2,
infer-opt/round14_fp4_full/impl/fp4util.py:41,68-75; stack14b.py:49-52); that call must run eagerly.
"""
from __future__ import annotations

import copy

import torch

from . import ops
from ._lib import KfError

PREFIXES = ("b200",)
HEADROOM = 2.0
BF, F16, F32 = torch.bfloat16, torch.float16, torch.float32


# ------------------------------------------------------------------------------------------------ weight extraction
@torch.no_grad()
def prepare_block_weights(block) -> dict:
    """bf16-rounded weights, fp32 biases (bf16-rounded values, K third of the qkv bias zeroed), fp32 LayerScale and LN
    parameters of one SelfAttentionBlock (infer-opt/round5_gemm_sm120/impl/ops.py:204-233 with ln_fold=False)."""
    f = lambda t: t.detach().float().contiguous()  # noqa: E731
    b16 = lambda t: t.detach().to(BF)  # noqa: E731
    qkv = block.attn.qkv
    bq = qkv.bias.detach().float().clone()
    o = qkv.out_features
    if hasattr(qkv, "bias_mask"):
        bq = torch.nan_to_num(bq * qkv.bias_mask.float(), nan=0.0)
        bq[o // 3: 2 * o // 3] = 0
    return dict(
        Wqkv=b16(qkv.weight), Wproj=b16(block.attn.proj.weight), W1=b16(block.mlp.fc1.weight), W2=b16(block.mlp.fc2.weight),
        bqkv=b16(bq).float().contiguous(), bproj=b16(block.attn.proj.bias).float().contiguous(),
        b1=b16(block.mlp.fc1.bias).float().contiguous(), b2=b16(block.mlp.fc2.bias).float().contiguous(),
        g1=f(block.ls1.gamma), g2=f(block.ls2.gamma),
        ln1_w=f(block.norm1.weight), ln1_b=f(block.norm1.bias), ln1_eps=block.norm1.eps,
        ln2_w=f(block.norm2.weight), ln2_b=f(block.norm2.bias), ln2_eps=block.norm2.eps,
    )


class Calib:
    """True during the first eager call of a model_fn (static NVFP4 scales are measured), False afterwards."""

    def __init__(self):
        self.on = True


def _site_ts(fmt, dev):
    return torch.ones(1, dtype=F32, device=dev) if fmt == "nv4" else None


def set_ts(ts_dev: torch.Tensor, x: torch.Tensor) -> None:
    """static per-tensor scale of an nv4 activation site: HEADROOM * amax / 2688, computed on the device without a
    host sync (stack14b.py:49-52).  Calibration only; not on the steady-state path."""
    amax = x.float().abs().amax()
    ts_dev.copy_(torch.where(amax > 0, amax * (HEADROOM / 2688.0), torch.ones_like(amax)).reshape(1))


def _with_ts(buf: ops.ActBuf, ts) -> ops.ActBuf:
    b = copy.copy(buf)
    b.ts = ts
    return b


class Layer:
    """quantised weights and activation-site scales of one block."""

    def __init__(self, block, fmt: str):
        w = prepare_block_weights(block)
        dev = w["Wqkv"].device
        self.fmt = fmt
        self.qkv, self.proj, self.fc1, self.fc2 = (ops.QWeight(w[k].float(), fmt) for k in ("Wqkv", "Wproj", "W1", "W2"))
        for k in ("bqkv", "bproj", "b1", "b2", "g1", "g2", "ln1_w", "ln1_b", "ln2_w", "ln2_b"):
            setattr(self, k, w[k])
        self.ln1_eps, self.ln2_eps = w["ln1_eps"], w["ln2_eps"]
        self.ts_ln1, self.ts_o, self.ts_ln2, self.ts_g = (_site_ts(fmt, dev) for _ in range(4))


def block_fwd(x: torch.Tensor, L: Layer, sin, cos, prefix: int, heads: int, calib: Calib, *, round_bf16: bool, attn_dtype, half_tables: bool = False,
              grow_into: torch.Tensor = None) -> torch.Tensor:
    """x fp32 [B, N, d] (updated in place) -> x.  grow_into (fp32 [B, N + Q, d], optional): the block's result is written
    behind the first Q rows of every image of this longer stream instead (the fc2 epilogue maps the rows), which is then
    returned: how the query tokens join the stream without a copy of it."""
    B, N, d = x.shape
    M = B * N
    ff = L.fc1.N
    fmt = L.fmt
    nv4, cal = fmt == "nv4", calib.on
    x2 = x.view(M, d)
    if fmt == "bf16":
        h = ops.ln_rows(x, L.ln1_w, L.ln1_b, L.ln1_eps, BF).view(M, d)
        qkv = ops.qkv_rope(h, L.qkv, L.bqkv, sin, cos, N, prefix, heads, out_dtype=attn_dtype, half_tables=half_tables)
        o = ops.attn_fwd(qkv).view(M, d)
        ops.gemm_res(o if o.dtype == BF else o.to(BF), L.proj, L.bproj, L.g1, x2, out=x2)
        h = ops.ln_rows(x, L.ln2_w, L.ln2_b, L.ln2_eps, BF).view(M, d)
        a = ops.gemm_plain(h, L.fc1, L.b1, gelu=True)
        return _fc2(a, L, x, x2, grow_into)
    # ---- LN1 + quant -> qkv (bias + RoPE + layout) -> attention
    if cal and nv4:
        set_ts(L.ts_ln1, ops.ln_rows(x, L.ln1_w, L.ln1_b, L.ln1_eps, BF))
    a = _with_ts(ops.act_buf(M, d, fmt, x.device, 0), L.ts_ln1)
    ops.ln_quant(x, L.ln1_w, L.ln1_b, L.ln1_eps, a, round_bf16=round_bf16)
    qkv = ops.qkv_rope(a, L.qkv, L.bqkv, sin, cos, N, prefix, heads, out_dtype=attn_dtype, half_tables=half_tables)
    # ---- attention with its output quantised in the epilogue -> proj (gamma + residual, in place on the stream)
    if cal and nv4:
        set_ts(L.ts_o, ops.attn_fwd(qkv))
    a2 = _with_ts(ops.act_buf(M, d, fmt, x.device, 1), L.ts_o)
    ops.attn_fwd_quant(qkv, a2)
    ops.gemm_res(a2, L.proj, L.bproj, L.g1, x2, out=x2)
    # ---- LN2 + quant -> fc1 (GELU + quantise-out) -> fc2 (gamma + residual)
    if cal and nv4:
        set_ts(L.ts_ln2, ops.ln_rows(x, L.ln2_w, L.ln2_b, L.ln2_eps, BF))
    a = _with_ts(a, L.ts_ln2)
    ops.ln_quant(x, L.ln2_w, L.ln2_b, L.ln2_eps, a, round_bf16=round_bf16)
    if cal and nv4:
        set_ts(L.ts_g, ops.gemm_plain(a, L.fc1, L.b1, gelu=True))
    f = _with_ts(ops.act_buf(M, ff, fmt, x.device, 0), L.ts_g)
    ops.gemm_gelu_q(a, L.fc1, L.b1, f, round_bf16=round_bf16)
    return _fc2(f, L, x, x2, grow_into)


def _fc2(f, L: Layer, x, x2, grow_into):
    if grow_into is None:
        ops.gemm_res(f, L.fc2, L.b2, L.g2, x2, out=x2)
        return x
    N, Nbig = x.shape[1], grow_into.shape[1]
    ops.gemm_res(f, L.fc2, L.b2, L.g2, x2, out=grow_into, row_map=(N, Nbig, Nbig - N))
    return grow_into


# ------------------------------------------------------------------------------------------------ patch embed and head
class PatchEmbed:
    """Conv2d(3, d, 16, 16) as a bf16 tcgen05 GEMM over gathered patches, written straight into the token stream behind
    the cls / register rows (infer-opt/round11_attn_tier0/impl/patch_embed.py:34-53)."""

    def __init__(self, bb, round_bf16: bool):
        pw = bb.patch_embed.proj.weight.detach()
        self.d = pw.shape[0]
        if bb.patch_size != 16 or pw.shape[1:] != (3, 16, 16):
            raise KfError("patch embed: only 3-channel 16x16 patches are supported")
        self.W = ops.QWeight(pw.reshape(self.d, 768), "bf16")
        self.bias = bb.patch_embed.proj.bias.detach().to(BF).float().contiguous()
        self.prefix = torch.cat((bb.cls_token.detach().float(), bb.storage_tokens.detach().float()), dim=1).contiguous()   # [1, 1+S, d]
        self.npre = self.prefix.shape[1]
        self.round_bf16 = round_bf16

    def __call__(self, x: torch.Tensor) -> torch.Tensor:
        B, _, S, _ = x.shape
        P = (S // 16) ** 2
        t = torch.empty(B, self.npre + P, self.d, dtype=F32, device=x.device)
        ops.broadcast_rows(self.prefix, t, 0)
        ops.gemm_tokens(ops.im2col_patch16(x), self.W, self.bias, t, P, self.npre + P, self.npre, round_bf16=self.round_bf16)
        return t


class Head:
    """EoMT prediction head: final LN + gather, class head, mask MLP, two ScaleBlocks (ConvTranspose as a GEMM in the
    block-scaled format + fused bias/GELU/pixel-shuffle/depthwise/LayerNorm2D), mask product of all images as one batched bf16 GEMM launch
    (task_model.py:636-651; infer-opt/round11_attn_tier0/impl/head11.py:42-96; stack13.py:124-148)."""

    def __init__(self, model, fmt: str, calib: Calib):
        bb = model.backbone
        self.fmt, self.calib = fmt, calib
        self.Q, self.npre = model.num_queries, 1 + bb.n_storage_tokens
        f = lambda t: t.detach().float().contiguous()  # noqa: E731
        self.ln_w, self.ln_b, self.ln_eps = f(bb.norm.weight), f(bb.norm.bias), bb.norm.eps
        C = bb.embed_dim
        self.C = C
        dev = bb.norm.weight.device
        ncls1 = model.class_head.out_features
        self.ncls1 = ncls1
        self.Wcls = model.class_head.weight.detach().to(BF).contiguous()                 # the class head runs inside the final LayerNorm kernel
        self.bcls = model.class_head.bias.detach().to(BF).float().contiguous()
        self.mh = [(ops.QWeight(m.weight.detach(), "bf16"), m.bias.detach().to(BF).float().contiguous())
                   for m in model.mask_head if isinstance(m, torch.nn.Linear)]
        self.stages = []
        for blk in model.upscale:
            c1, c2, nrm = blk.conv1, blk.conv2, blk.norm
            # ConvTranspose2d weight [Cin, Cout, 2, 2] -> GEMM weight [(dy, dx, Cout), Cin]
            wr = c1.weight.detach().permute(2, 3, 1, 0).reshape(4 * C, C).to(BF)
            self.stages.append(dict(
                W=ops.QWeight(wr.float() if fmt != "bf16" else wr, fmt), bias4=c1.bias.detach().to(BF).float().repeat(4).contiguous(),
                dww=c2.weight.detach().reshape(C, 9).t().to(BF).float().contiguous(), g=f(nrm.weight), b=f(nrm.bias), eps=nrm.eps,
                ts=_site_ts(fmt, dev)))

    def __call__(self, t: torch.Tensor, grid):
        B, Ntok, C = t.shape
        Q, (Hs, Ws) = self.Q, grid
        qb, xb, cl = ops.ln_tail(t, self.ln_w, self.ln_b, self.ln_eps, Q, self.npre, self.Wcls, self.bcls)
        cl = cl.view(B, Q, self.ncls1)
        z = xb
        for st in self.stages:
            if self.fmt == "bf16":
                g = ops.gemm_plain(z, st["W"], st["bias4"], gelu=True, pre_round=True, tag="head")
            else:
                if self.calib.on and self.fmt == "nv4":
                    set_ts(st["ts"], z)
                a = _with_ts(ops.act_buf(z.shape[0], C, self.fmt, z.device, 2), st["ts"])
                ops.quant_rows(z, a)
                g = ops.gemm_plain(a, st["W"], st["bias4"], gelu=True, pre_round=True, tag="head")
            u = ops.dw_ln(g, None, st["dww"], st["g"], st["b"], B, Hs, Ws, st["eps"], pre_act=True)
            z = u.view(B * 4 * Hs * Ws, C)
            Hs, Ws = 2 * Hs, 2 * Ws
        h = qb
        for i, (W, b) in enumerate(self.mh):
            h = ops.gemm_plain(h, W, b, gelu=i < len(self.mh) - 1, tag="head")
        ml = ops.bmm_nt(h.view(B, Q, C), u.view(B, Hs * Ws, C))          # all images in one launch
        return ml.view(B, Q, Hs, Ws), cl


# ------------------------------------------------------------------------------------------------ model_fn
def make_model_fn(model, fmt: str, *, image_size: int = 640, round_bf16: bool = True, attn_dtype=BF, head_fmt=None):
    bb = model.backbone
    heads = bb.blocks[0].attn.num_heads
    nb = len(bb.blocks)
    calib = Calib()
    layers = [Layer(b, fmt) for b in bb.blocks]
    grid = (image_size // bb.patch_size, image_size // bb.patch_size)
    with torch.no_grad():
        sin, cos = bb.rope_embed(H=grid[0], W=grid[1])
    sin, cos = sin.float().contiguous(), cos.float().contiguous()
    half_tables = ops.rope_tables_are_half(sin, cos)       # checked once here, on the host
    queries = model.queries.weight.detach().float().contiguous()
    Q = queries.shape[0]
    first_joint = nb - model.num_joint_blocks
    pe = PatchEmbed(bb, round_bf16)
    head = Head(model, head_fmt or fmt, calib)
    P = grid[0] * grid[1]

    @torch.no_grad()
    def model_fn(x: torch.Tensor):
        if x.dtype != BF or x.dim() != 4 or x.shape[2] != image_size or x.shape[3] != image_size:
            raise KfError(f"model_fn: x must be bf16 [B, 3, {image_size}, {image_size}], got {tuple(x.shape)} {x.dtype}")
        if calib.on and fmt == "nv4" and torch.cuda.is_current_stream_capturing():
            raise RuntimeError("the first call (static-scale calibration) must run eagerly, before CUDA graph capture")
        t = pe(x.contiguous())
        for i in range(nb):
            grow = None
            if i + 1 == first_joint and first_joint < nb:     # the next block sees the queries: this block's fc2 writes the longer stream
                grow = torch.empty(t.shape[0], Q + t.shape[1], t.shape[2], dtype=F32, device=t.device)
                ops.broadcast_rows(queries, grow, 0)
            elif i == first_joint == 0:                   # every block is a joint block: no fc2 in front to do the move
                t = torch.cat((queries[None].expand(t.shape[0], -1, -1), t), dim=1).contiguous()
            t = block_fwd(t, layers[i], sin, cos, t.shape[1] - P, heads, calib, round_bf16=round_bf16, attn_dtype=attn_dtype, half_tables=half_tables,
                          grow_into=grow)
        out = head(t, grid)
        calib.on = False
        return out

    model_fn._keepalive = (layers, pe, head, calib, sin, cos, queries)
    model_fn.calib = calib
    return model_fn


class FramePipeline:
    """uint8 frames -> resize + normalise -> model_fn -> per-pixel labels, all on the current stream
    (the GPU part of VideoPipeline, infer-opt/round9_integration/video_infer.py:87-320)."""

    def __init__(self, model, model_fn, image_size: int = 640):
        self.model_fn, self.image_size = model_fn, image_size

    def __call__(self, frames_u8: torch.Tensor):
        x = ops.resize_norm(frames_u8, self.image_size)
        ml, cl = self.model_fn(x)
        labels, _ = ops.semantic(ml, cl)
        return labels


def make_variant(name, model, variant: str):
    """-> (model_fn, pipeline_cls) for variant strings like "b200_nv4", "b200_mx8+s1024+fp32pts"."""
    parts = variant.split("+")
    base, flags = parts[0], set(parts[1:])
    fmts = {"b200_mx8": "mx8", "b200_nv4": "nv4", "b200_mx4": "mx4", "b200_bf16": "bf16"}
    if base not in fmts:
        raise ValueError(variant)
    size = 640
    for f in list(flags):
        if f.startswith("s") and f[1:].isdigit():
            size = int(f[1:])
            flags.discard(f)
    unknown = flags - {"fp32pts", "f16attn", "bf16head"}
    if unknown:
        raise ValueError(f"unknown variant flags {sorted(unknown)}")
    fn = make_model_fn(model, fmts[base], image_size=size, round_bf16="fp32pts" not in flags,
                       attn_dtype=F16 if "f16attn" in flags else BF, head_fmt="bf16" if "bf16head" in flags else None)
    return fn, FramePipeline
