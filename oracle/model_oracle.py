"""CPU oracle of the emulated low-precision model: test infrastructure, not product code.

Restates, with torch CPU ops and the numpy quantiser oracle, the reference's emulated path EmuNet
(infer-opt/round10_lowp_probe/impl/emu.py:260-333 gemm/block/forward, :356-397 head) with the model semantics of
    src/lightly_train/_task_models/dinov3_eomt_semantic_segmentation/task_model.py:416-508 (forward_train),
    :636-651 (_predict), :674-698 (_attn); scale_block.py:19-56
and the rounding points of its right-hand dataflow: the LN output, the attention output and the GELU output are
rounded to bf16 before they are quantised-dequantised; q, k, v are bf16; the residual stream is fp32; weights are the
bf16-rounded module weights quantised-dequantised once.  The input size is a parameter (the reference hard-codes 512).

Pinning: the model semantics (token order, RoPE tables and placement, qkv split, K-masked bias, LayerScale / residual
order, ScaleBlock layout) are pinned to the reference's own DinoVisionTransformer / SelfAttentionBlock / ScaleBlock through
tests/golden/model_golden.npz (tests/test_model_pin_cpu.py runs this file's block at format "bf16" against the reference
block's output); the quantiser it calls is bit-exact against the reference's quant_ref.py.  EmuNet itself cannot run
outside an sm_120a GPU (emu.py:25-33), so the PLACEMENT of its rounding points (which tensors are rounded to bf16 and
quantised-dequantised, emu.py:260-333) is restated from the source and is the one part that stays "parity unpinned".
"""
from __future__ import annotations

import math

import numpy as np
import torch
import torch.nn.functional as F

from . import quant_oracle as qo

BF = torch.bfloat16


def _bf(t: torch.Tensor) -> torch.Tensor:
    return t.to(BF).float()


def qdq_t(x: torch.Tensor, fmt: str, ts=None) -> torch.Tensor:
    """fp32 [R, C] -> the dequantised values of its quantisation in fmt ("bf16": bf16 rounding)."""
    if fmt == "bf16":
        return _bf(x)
    return torch.from_numpy(qo.qdq(x.detach().float().numpy(), fmt, None if ts is None else np.asarray(ts, dtype=np.float32)))


def static_ts(x: torch.Tensor, headroom: float = 2.0) -> np.ndarray:
    amax = np.float32(x.detach().abs().max().item())
    return np.array([amax * np.float32(headroom / 2688.0) if amax > 0 else 1.0], dtype=np.float32)


class EmuModel:
    """model: a DINOv3EoMTSemanticSegmentation-like module on CPU (fp32 parameters).  ts: optional dict
    {(layer, site) -> float32 [1]} of static NVFP4 activation scales ("ln1", "o", "ln2", "g"; ("head", j) for the
    ConvTranspose inputs); missing entries are measured on the first call with headroom 2."""

    def __init__(self, model, fmt: str, head_fmt=None, ts=None, round_bf16: bool = True, attn_dtype=BF):
        self.m, self.fmt, self.head_fmt = model, fmt, head_fmt or fmt
        self.attn_dtype = attn_dtype                  # 16-bit type of q, k, v and of the attention output (bf16 | f16)
        self.ts = dict(ts or {})
        self.round = round_bf16
        self._w = {}

    def _ts(self, key, x):
        if key not in self.ts:
            self.ts[key] = static_ts(x)
        return self.ts[key]

    def _wq(self, key, W, fmt):
        if key not in self._w:
            self._w[key] = qdq_t(_bf(W.detach()), fmt)
        return self._w[key]

    def _lin(self, key, site, X, lin, fmt, bias=None):
        """X [M, K] fp32 values already at their rounding point -> qdq(X) @ qdq(W)^T + bias (fp32)."""
        Xq = qdq_t(X, fmt, self._ts((key[0], site), X) if fmt == "nv4" else None)
        Wq = self._wq(key, lin.weight, fmt)
        y = Xq @ Wq.t()
        if bias is not None:
            y = y + bias
        return y

    @torch.no_grad()
    def block(self, i, blk, x, sin, cos, prefix):
        B, N, d = x.shape
        H = blk.attn.num_heads
        rp = _bf if self.round else (lambda t: t)
        h = rp(F.layer_norm(x, (d,), blk.norm1.weight, blk.norm1.bias, blk.norm1.eps)).reshape(B * N, d)
        bq = blk.attn.qkv.bias.detach().clone()
        bq[d: 2 * d] = 0
        y = self._lin((i, "qkv"), "ln1", h, blk.attn.qkv, self.fmt, _bf(bq))
        q, k, v = y.reshape(B, N, 3, H, 64).permute(2, 0, 3, 1, 4)        # [B, H, N, 64]

        def rope(t):
            r = t[:, :, prefix:]
            rot = torch.cat([-r[..., 32:], r[..., :32]], dim=-1)
            return torch.cat((t[:, :, :prefix], r * cos + rot * sin), dim=2)

        r16 = lambda t: t.to(self.attn_dtype).float()  # noqa: E731
        q, k, v = r16(rope(q)), r16(rope(k)), r16(v)
        s = (q @ k.transpose(-1, -2)) * 0.125
        o = r16((torch.softmax(s, dim=-1) @ v).transpose(1, 2).reshape(B * N, d))
        y = self._lin((i, "proj"), "o", o, blk.attn.proj, self.fmt, _bf(blk.attn.proj.bias.detach()))
        x = x + (y * blk.ls1.gamma).reshape(B, N, d)
        h = rp(F.layer_norm(x, (d,), blk.norm2.weight, blk.norm2.bias, blk.norm2.eps)).reshape(B * N, d)
        a = self._lin((i, "fc1"), "ln2", h, blk.mlp.fc1, self.fmt, _bf(blk.mlp.fc1.bias.detach()))
        a = rp(F.gelu(a))
        y = self._lin((i, "fc2"), "g", a, blk.mlp.fc2, self.fmt, _bf(blk.mlp.fc2.bias.detach()))
        return x + (y * blk.ls2.gamma).reshape(B, N, d)

    @torch.no_grad()
    def head(self, t, grid):
        m, bb = self.m, self.m.backbone
        B, Ntok, C = t.shape
        Q, npre = m.num_queries, 1 + bb.n_storage_tokens
        xn = F.layer_norm(t, (C,), bb.norm.weight, bb.norm.bias, bb.norm.eps)
        qb = _bf(xn[:, :Q]).reshape(B * Q, C)
        z = _bf(xn[:, Q + npre:]).reshape(-1, C)
        cl = _bf(qb @ _bf(m.class_head.weight.detach()).t() + _bf(m.class_head.bias.detach())).reshape(B, Q, -1)
        Hs, Ws = grid
        for j, blk in enumerate(m.upscale):
            wr = blk.conv1.weight.detach().permute(2, 3, 1, 0).reshape(4 * C, C)          # [(dy,dx,co), ci]
            Xq = qdq_t(z, self.head_fmt, self._ts(("head", j), z) if self.head_fmt == "nv4" else None)
            Wq = self._wq(("head", j), wr, self.head_fmt)
            g = _bf(Xq @ Wq.t())                                                         # [B*Hs*Ws, 4C] bf16
            g = g.reshape(B, Hs, Ws, 2, 2, C).permute(0, 1, 3, 2, 4, 5).reshape(B, 2 * Hs, 2 * Ws, C)
            a = _bf(F.gelu(g + _bf(blk.conv1.bias.detach())))
            dw = _bf(blk.conv2.weight.detach())                                          # [C, 1, 3, 3]
            o = _bf(F.conv2d(a.permute(0, 3, 1, 2), dw, padding=1, groups=C)).permute(0, 2, 3, 1)
            u = _bf(F.layer_norm(o, (C,), blk.norm.weight, blk.norm.bias, blk.norm.eps))
            Hs, Ws = 2 * Hs, 2 * Ws
            z = u.reshape(-1, C)
        h = qb
        lins = [l for l in m.mask_head if isinstance(l, torch.nn.Linear)]
        for j, l in enumerate(lins):
            h = h @ _bf(l.weight.detach()).t() + _bf(l.bias.detach())
            if j < len(lins) - 1:
                h = F.gelu(h)
            h = _bf(h)
        ml = _bf(torch.bmm(h.reshape(B, Q, C), u.reshape(B, Hs * Ws, C).transpose(1, 2)))
        return ml.reshape(B, Q, Hs, Ws), cl

    @torch.no_grad()
    def __call__(self, x_img: torch.Tensor):
        """x_img bf16-representable [B, 3, S, S] -> (mask_logits, class_logits) as fp32 tensors holding bf16 values."""
        m, bb = self.m, self.m.backbone
        x = _bf(x_img.float())
        pw = _bf(bb.patch_embed.proj.weight.detach())
        pb = _bf(bb.patch_embed.proj.bias.detach())
        tok = F.conv2d(x, pw, pb, stride=bb.patch_size).permute(0, 2, 3, 1)
        B, gh, gw, d = tok.shape
        tok = tok.reshape(B, gh * gw, d)
        if self.round:
            tok = _bf(tok)
        t = torch.cat([bb.cls_token.detach().float().expand(B, -1, -1), bb.storage_tokens.detach().float().expand(B, -1, -1), tok], dim=1)
        sin, cos = bb.rope_embed(H=gh, W=gw)
        nb = len(bb.blocks)
        for i, blk in enumerate(bb.blocks):
            if i == nb - m.num_joint_blocks:
                t = torch.cat((m.queries.weight.detach().float()[None].expand(B, -1, -1), t), dim=1)
            t = self.block(i, blk, t, sin.float(), cos.float(), t.shape[1] - gh * gw)
        return self.head(t, (gh, gw))


def cosine(a, b) -> float:
    a = torch.as_tensor(a).detach().double().flatten()
    b = torch.as_tensor(b).detach().double().flatten()
    return float((a @ b) / (a.norm() * b.norm()).clamp_min(1e-300))
