"""Module-level Linear swap: patch selected (layer, kind) units of a DINOv3 model so its own forward runs the
block-scaled GEMMs, keeping everything else (attention, residuals, head) as the model defines it.

Same surface as the reference (infer-opt/round6_low_precision/impl/mxlinear.py:68-149):

    enable(model, units, fmt="mx8")    units = [(layer_idx, "qkv" | "proj" | "fc1" | "fc2"), ...]
    disable(model)

enable() sets instance-level `.forward` on model.backbone.blocks[i].{norm1, attn.qkv, attn.proj, norm2, mlp.fc1,
mlp.act, mlp.fc2}: the LayerNorm / GELU patches run the fused quantiser, stash the quantised operand under the unit key
and return an empty tensor; the Linear patch pops the stash (or quantises its own input) and runs the tcgen05 GEMM with
bias, returning bf16 in the input's leading shape.  disable() removes the instance attributes.

Differences from the reference, both deliberate: the quantisers behind the swap are the bit-exact ones (the reference's
first-generation mx_ext.cu computes the scale with exp2f(ceilf(log2f(.))), mx_ext.cu:24-26); padded scale rows are
written as zero rather than 127 (either is valid: mxlinear.py:46 vs mx13.py:56-61).  NVFP4 units use a dynamic per-call
per-tensor scale measured on the device (no host sync) because a swapped Linear has no calibration pass.
"""
from __future__ import annotations

import torch

from . import ops

BF = torch.bfloat16


class _Ctx:
    def __init__(self, fmt):
        self.fmt, self.buf = fmt, {}

    def get(self, M, K, device, slot=0) -> ops.ActBuf:
        key = (M, K, str(device), slot)
        if key not in self.buf:
            self.buf[key] = ops.ActBuf(M, K, self.fmt, device)
        return self.buf[key]


def _dyn_ts(buf: ops.ActBuf, x: torch.Tensor) -> None:
    if buf.fmt == "nv4":
        amax = x.float().abs().amax()
        buf.ts.copy_(torch.where(amax > 0, amax / 2688.0, torch.ones_like(amax)).reshape(1))


def enable(model, units, fmt: str = "mx8") -> None:
    """Patch the selected (layer, qkv|proj|fc1|fc2) units of model.backbone.blocks."""
    units = set(map(tuple, units))
    ctx = _Ctx(fmt)
    stash, leads, patched = {}, {}, []
    for i, blk in enumerate(model.backbone.blocks):
        types = {t for li, t in units if li == i}
        if not types:
            continue

        def make_lin(lin, key):
            W = ops.QWeight(lin.weight.detach().to(BF).float(), fmt)
            bias = None
            if lin.bias is not None:
                b = lin.bias.detach().float()
                if hasattr(lin, "bias_mask"):
                    b = torch.nan_to_num(b * lin.bias_mask.float(), nan=0.0)
                bias = b.to(BF).float().contiguous()
            N = lin.weight.shape[0]

            def fwd(x):
                if key in stash:
                    a = stash.pop(key)
                    lead = leads.pop(key)
                else:
                    K = x.shape[-1]
                    lead = x.shape[:-1]
                    x2 = x.reshape(-1, K)
                    if x2.dtype not in (torch.float32, BF, torch.float16) or x2.stride(-1) != 1:
                        x2 = x2.float().contiguous()
                    a = ctx.get(x2.shape[0], K, x.device, 1)
                    _dyn_ts(a, x2)
                    ops.quant_rows(x2, a)
                return ops.gemm_plain(a, W, bias, out_dtype=BF).view(*lead, N)

            lin.forward = fwd
            patched.append(lin)

        def make_ln(norm, key):
            g = norm.weight.detach().float().contiguous()
            b = norm.bias.detach().float().contiguous()

            def fwd(x):
                K = x.shape[-1]
                x2 = x.reshape(-1, K).float().contiguous()
                a = ctx.get(x2.shape[0], K, x.device, 0)
                if fmt == "nv4":
                    _dyn_ts(a, ops.ln_rows(x2, g, b, norm.eps, BF))
                ops.ln_quant(x2, g, b, norm.eps, a, round_bf16=True)
                stash[key] = a
                leads[key] = x.shape[:-1]
                return x.new_empty(0)

            norm.forward = fwd
            patched.append(norm)

        def make_gelu(act, key):
            def fwd(x):
                K = x.shape[-1]
                x2 = x.reshape(-1, K)
                if x2.stride(-1) != 1:
                    x2 = x2.contiguous()
                a = ctx.get(x2.shape[0], K, x.device, 2)
                zero = torch.zeros(K, dtype=torch.float32, device=x.device)
                if fmt == "nv4":
                    _dyn_ts(a, torch.nn.functional.gelu(x2.float()))
                ops.quant_rows(x2, a, bias=zero, gelu=True, round_bf16=True)
                stash[key] = a
                leads[key] = x.shape[:-1]
                return x.new_empty(0)

            act.forward = fwd
            patched.append(act)

        if "qkv" in types:
            make_ln(blk.norm1, (i, "qkv"))
            make_lin(blk.attn.qkv, (i, "qkv"))
        if "proj" in types:
            make_lin(blk.attn.proj, (i, "proj"))
        if "fc1" in types:
            make_ln(blk.norm2, (i, "fc1"))
            make_lin(blk.mlp.fc1, (i, "fc1"))
        if "fc2" in types:
            make_gelu(blk.mlp.act, (i, "fc2"))
            make_lin(blk.mlp.fc2, (i, "fc2"))
    model._kf_patched = patched


def disable(model) -> None:
    for m in getattr(model, "_kf_patched", []):
        m.__dict__.pop("forward", None)
    model._kf_patched = []
