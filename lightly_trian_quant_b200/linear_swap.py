"""Module-level Linear swap: selected (layer, kind) units of a DINOv3 model run their Linear on the block-scaled
tcgen05 GEMM while everything else (attention, residuals, head) stays as the model defines it.

Surface of the reference's swap (infer-opt/round6_low_precision/impl/mxlinear.py:68-149):

    enable(model, units, fmt="mx8")    units = [(layer_idx, "qkv" | "proj" | "fc1" | "fc2"), ...]
    disable(model)

Behaviour kept from that contract: enable() installs instance-level `forward` callables on
model.backbone.blocks[i].{norm1, attn.qkv, attn.proj, norm2, mlp.fc1, mlp.act, mlp.fc2}; a LayerNorm / GELU in front of a
swapped Linear runs the fused quantiser, leaves the quantised operand in a hand-over slot keyed by the unit and returns
an EMPTY tensor; the Linear takes the operand from its slot (or quantises the tensor it was given when the slot is
empty), runs the GEMM with its bias and returns bf16 in the caller's leading shape; disable() removes the instance
attributes so the class forwards are back, bit for bit.

Differences from the reference, both deliberate: the quantisers behind the swap are the bit-exact ones (the reference's
first-generation mx_ext.cu computes the scale with exp2f(ceilf(log2f(.))), mx_ext.cu:24-26); padded scale rows are
written as zero rather than 127 (either is valid: mxlinear.py:46 vs mx13.py:56-61).  NVFP4 units use a dynamic per-call
per-tensor scale measured on the device (no host sync) because a swapped Linear has no calibration pass.

Structure: one `_Swap` session per enable() call owns the operand pool and the hand-over slots; every patched module
gets one small callable object (`_Feeder` for LayerNorm / GELU, `_QLinear` for the Linear); which sub-modules a unit
kind touches is the table `_UNIT_PLAN`.
"""
from __future__ import annotations

from typing import Callable, Dict, List, Optional, Tuple

import torch

from . import ops

BF = torch.bfloat16
_ATTR = "_kf_patched"

# unit kind -> (path of the module that feeds the Linear or None, how it feeds, path of the Linear)
_UNIT_PLAN: Dict[str, Tuple[Optional[str], Optional[str], str]] = {
    "qkv": ("norm1", "ln", "attn.qkv"),
    "proj": (None, None, "attn.proj"),
    "fc1": ("norm2", "ln", "mlp.fc1"),
    "fc2": ("mlp.act", "gelu", "mlp.fc2"),
}


def _resolve(root, dotted: str):
    for name in dotted.split("."):
        root = getattr(root, name)
    return root


def _rows(t: torch.Tensor) -> torch.Tensor:
    """[..., K] -> [M, K] with a contiguous last dimension in a dtype the quantisers take."""
    flat = t.reshape(-1, t.shape[-1])
    if flat.dtype not in (torch.float32, BF, torch.float16):
        flat = flat.float()
    return flat if flat.stride(-1) == 1 else flat.contiguous()


class _Swap:
    """State shared by the patched modules of one enable() call."""

    def __init__(self, fmt: str):
        self.fmt = fmt
        self.pool: Dict[tuple, ops.ActBuf] = {}      # persistent operands per (rows, K, device, role)
        self.slots: Dict[tuple, tuple] = {}          # unit -> (operand, leading shape) waiting for its Linear
        self.modules: List[torch.nn.Module] = []

    def operand(self, rows: int, K: int, device, role: str) -> ops.ActBuf:
        key = (rows, K, str(device), role)
        buf = self.pool.get(key)
        if buf is None:
            buf = self.pool[key] = ops.ActBuf(rows, K, self.fmt, device)
        return buf

    def set_dynamic_scale(self, buf: ops.ActBuf, values: torch.Tensor) -> None:
        """nv4 only: per-tensor scale amax / (6 * 448) of the values about to be quantised, on the device."""
        if self.fmt != "nv4":
            return
        peak = values.float().abs().amax()
        buf.ts.copy_(torch.where(peak > 0, peak / 2688.0, torch.ones_like(peak)).reshape(1))

    def install(self, module: torch.nn.Module, fn: Callable) -> None:
        module.forward = fn                          # instance attribute: shadows the class forward until disable()
        self.modules.append(module)


class _Feeder:
    """forward of a LayerNorm ("ln") or GELU ("gelu") whose only consumer is a swapped Linear: quantise, park, return empty."""

    def __init__(self, swap: _Swap, unit: tuple, how: str, module: torch.nn.Module):
        self.swap, self.unit, self.how = swap, unit, how
        if how == "ln":
            self.w = module.weight.detach().float().contiguous()
            self.b = module.bias.detach().float().contiguous()
            self.eps = module.eps
        self.no_bias: Dict[tuple, torch.Tensor] = {}   # the GELU quantiser wants a bias vector: zeros, made once per width

    def __call__(self, x: torch.Tensor) -> torch.Tensor:
        sw = self.swap
        if self.how == "ln":
            src = x.reshape(-1, x.shape[-1]).float().contiguous()
            buf = sw.operand(src.shape[0], src.shape[1], x.device, "ln")
            if sw.fmt == "nv4":
                sw.set_dynamic_scale(buf, ops.ln_rows(src, self.w, self.b, self.eps, BF))
            ops.ln_quant(src, self.w, self.b, self.eps, buf, round_bf16=True)
        else:
            src = _rows(x)
            buf = sw.operand(src.shape[0], src.shape[1], x.device, "gelu")
            zkey = (src.shape[1], str(x.device))
            if zkey not in self.no_bias:
                self.no_bias[zkey] = torch.zeros(src.shape[1], dtype=torch.float32, device=x.device)
            if sw.fmt == "nv4":
                sw.set_dynamic_scale(buf, torch.nn.functional.gelu(src.float()))
            ops.quant_rows(src, buf, bias=self.no_bias[zkey], gelu=True, round_bf16=True)
        sw.slots[self.unit] = (buf, tuple(x.shape[:-1]))
        return x.new_empty(0)


class _QLinear:
    """forward of a swapped nn.Linear: weight quantised once, activation from the unit's slot or quantised here."""

    def __init__(self, swap: _Swap, unit: tuple, lin: torch.nn.Linear):
        self.swap, self.unit = swap, unit
        self.out_features = lin.weight.shape[0]
        self.weight = ops.QWeight(lin.weight.detach().to(BF).float(), swap.fmt)
        self.bias = None
        if lin.bias is not None:
            b = lin.bias.detach().float()
            if hasattr(lin, "bias_mask"):          # the qkv projection masks the K third of its bias
                b = torch.nan_to_num(b * lin.bias_mask.float(), nan=0.0)
            self.bias = b.to(BF).float().contiguous()

    def __call__(self, x: torch.Tensor) -> torch.Tensor:
        sw = self.swap
        parked = sw.slots.pop(self.unit, None)
        if parked is not None:
            buf, lead = parked
        else:
            src = _rows(x)
            lead = tuple(x.shape[:-1])
            buf = sw.operand(src.shape[0], src.shape[1], x.device, "lin")
            sw.set_dynamic_scale(buf, src)
            ops.quant_rows(src, buf)
        y = ops.gemm_plain(buf, self.weight, self.bias, out_dtype=BF)
        return y.view(*lead, self.out_features)


def enable(model, units, fmt: str = "mx8") -> None:
    """Patch the selected (layer, qkv|proj|fc1|fc2) units of model.backbone.blocks."""
    wanted = {(int(layer), str(kind)) for layer, kind in units}
    for _, kind in wanted:
        if kind not in _UNIT_PLAN:
            raise ValueError(f"unknown unit kind {kind!r}: expected one of {sorted(_UNIT_PLAN)}")
    disable(model)
    swap = _Swap(fmt)
    blocks = model.backbone.blocks
    for layer, kind in sorted(wanted):
        feeder_path, how, linear_path = _UNIT_PLAN[kind]
        block = blocks[layer]
        unit = (layer, kind)
        if feeder_path is not None:
            feeder = _resolve(block, feeder_path)
            swap.install(feeder, _Feeder(swap, unit, how, feeder))
        lin = _resolve(block, linear_path)
        swap.install(lin, _QLinear(swap, unit, lin))
    setattr(model, _ATTR, swap.modules)


def disable(model) -> None:
    """Remove every instance-level forward that enable() installed."""
    for module in getattr(model, _ATTR, None) or []:
        vars(module).pop("forward", None)
    setattr(model, _ATTR, [])
