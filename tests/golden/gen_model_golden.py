"""Generates tests/golden/model_golden.npz by running the REFERENCE backbone and ScaleBlock, imported unmodified.

Run once, in a container where the reference checkout is mounted (pass its root as argv[1]); the GPU box never
runs this.  The reference package cannot be imported as a whole offline (it pulls albumentations, pytorch_lightning,
omegaconf), so a stub top-level package whose __path__ points at <ref>/src/lightly_train makes the sub-packages that
only need torch importable:
    <ref>/src/lightly_train/_models/dinov3/dinov3_src/models/vision_transformer.py    DinoVisionTransformer
    <ref>/src/lightly_train/_models/dinov3/dinov3_src/layers/{attention,block,rope_position_encoding,...}.py
    <ref>/src/lightly_train/_models/dinov3/dinov3_src/hub/backbones.py                dinov3_vitb16 / dinov3_vitl16 configs
    <ref>/src/lightly_train/_task_models/dinov3_eomt_semantic_segmentation/scale_block.py   ScaleBlock

What is stored (all fp32, host cores):
    hub_*            the constructor facts of dinov3_vitb16 / dinov3_vitl16 (depth, width, heads, MLP width, storage
                     tokens, LN eps, LayerScale init, RoPE periods) that modeldef.VIT_B / VIT_L restate
    rope_*           rope_embed(H, W) sin / cos for 40x40 (640 px), 64x64 (1024 px) and a non-square 5x7 grid
    small backbone   embed_dim 128, 2 heads (head dim 64), depth 2, 4 storage tokens, K-masked qkv bias, LayerScale,
                     LN eps 1e-5, built with the hub's keyword values; its parameters are drawn from a seeded generator in
                     state-dict order (param_spec) so the test regenerates them instead of storing them.
                     Outputs: prepare_tokens_with_masks, each block's output, the final norm
    scale block      ScaleBlock(128) on a [2, 128, 5, 7] input
"""
from __future__ import annotations

import json
import sys
import types
from pathlib import Path

import numpy as np
import torch

SMALL = dict(embed_dim=128, depth=2, num_heads=2, n_storage_tokens=4)
IMG = (48, 80)          # -> a 3 x 5 patch grid (non-square on purpose)


def stub_reference(ref_root: Path):
    pkg = types.ModuleType("lightly_train")
    pkg.__path__ = [str(ref_root / "src" / "lightly_train")]
    sys.modules["lightly_train"] = pkg


def seeded_params(named_shapes, seed: int):
    """the deterministic parameter recipe shared by this generator and the test: for every (name, shape) in order,
    randn * scale(name) + offset(name) from one seeded CPU generator."""
    g = torch.Generator().manual_seed(seed)
    out = {}
    for name, shape in named_shapes:
        t = torch.randn(*shape, generator=g)
        if name.endswith("bias_mask") or name.endswith("periods"):
            continue                                    # buffers keep the values the reference gives them
        if name.endswith(".gamma"):
            t = 0.5 + 0.25 * t.abs()                    # LayerScale large enough for block errors to show
        elif "norm" in name and name.endswith(".weight"):
            t = 1.0 + 0.2 * t
        elif name.endswith(".weight"):
            t = t * (1.0 / max(shape[-1], 1)) ** 0.5
        else:
            t = t * 0.1
        out[name] = t
    return out


def main(ref_root: Path, out_path: Path):
    torch.set_grad_enabled(False)
    torch.manual_seed(0)
    stub_reference(ref_root)
    from lightly_train._models.dinov3.dinov3_src.hub import backbones
    from lightly_train._models.dinov3.dinov3_src.models.vision_transformer import DinoVisionTransformer
    from lightly_train._task_models.dinov3_eomt_semantic_segmentation.scale_block import ScaleBlock

    out = {}
    # ---- hub configurations the model definition restates
    for tag, ctor in (("vitb16", backbones.dinov3_vitb16), ("vitl16", backbones.dinov3_vitl16)):
        m = ctor(pretrained=False)
        m.init_weights()
        m.eval()                                        # inference: no coordinate shift / jitter / rescale in rope_embed
        b0 = m.blocks[0]
        facts = dict(depth=len(m.blocks), embed_dim=m.embed_dim, heads=b0.attn.num_heads, ffn=b0.mlp.fc1.out_features,
                     n_storage_tokens=m.n_storage_tokens, patch_size=m.patch_size, ln_eps=b0.norm1.eps, final_ln_eps=m.norm.eps,
                     layerscale_init=float(b0.ls1.gamma[0]), qkv_class=type(b0.attn.qkv).__name__,
                     k_bias_mask_zero=bool((b0.attn.qkv.bias_mask[m.embed_dim: 2 * m.embed_dim] == 0).all()),
                     act=type(b0.mlp.act).__name__, rope_dtype=str(m.rope_embed.periods.dtype))
        out[f"hub_{tag}_facts"] = np.frombuffer(json.dumps(facts, sort_keys=True).encode(), dtype=np.uint8)
        out[f"hub_{tag}_periods"] = m.rope_embed.periods.float().numpy()
        if tag == "vitl16":
            for H, W in ((40, 40), (64, 64), (5, 7)):
                sin, cos = m.rope_embed(H=H, W=W)
                out[f"rope_sin_{H}x{W}"] = sin.float().numpy()
                out[f"rope_cos_{H}x{W}"] = cos.float().numpy()
        del m

    # ---- small backbone with the hub's keyword values (hub/backbones.py: dinov3_vitb16 / dinov3_vitl16)
    bb = DinoVisionTransformer(img_size=224, patch_size=16, pos_embed_rope_base=100, pos_embed_rope_normalize_coords="separate",
                               pos_embed_rope_rescale_coords=2, pos_embed_rope_dtype="fp32", ffn_ratio=4, qkv_bias=True,
                               layerscale_init=1.0e-05, norm_layer="layernormbf16", ffn_layer="mlp", ffn_bias=True, proj_bias=True,
                               mask_k_bias=True, **SMALL)
    bb.init_weights()
    bb.eval()
    spec = [(k, tuple(v.shape)) for k, v in bb.state_dict().items()]
    out["param_spec"] = np.frombuffer(json.dumps(spec).encode(), dtype=np.uint8)
    sd = bb.state_dict()
    for k, v in seeded_params(spec, seed=1234).items():
        sd[k].copy_(v)
    g = torch.Generator().manual_seed(7)
    x = torch.rand(2, 3, *IMG, generator=g)
    out["image"] = x.numpy()
    t, (gh, gw) = bb.prepare_tokens_with_masks(x)
    out["tokens"] = t.numpy()
    out["grid"] = np.array([gh, gw])
    rope = bb.rope_embed(H=gh, W=gw)
    for i, blk in enumerate(bb.blocks):
        t = blk(t, rope)
        out[f"block{i}_out"] = t.numpy()
    out["final_norm"] = bb.norm(t).numpy()
    # the K third of the qkv bias has no effect: a control that the mask is what the reference applies
    out["qkv_bias_masked"] = (bb.blocks[0].attn.qkv.bias * bb.blocks[0].attn.qkv.bias_mask).numpy()

    # ---- ScaleBlock
    sb = ScaleBlock(SMALL["embed_dim"]).eval()
    sspec = [(k, tuple(v.shape)) for k, v in sb.state_dict().items()]
    out["scale_param_spec"] = np.frombuffer(json.dumps(sspec).encode(), dtype=np.uint8)
    ssd = sb.state_dict()
    for k, v in seeded_params(sspec, seed=4321).items():
        ssd[k].copy_(v)
    z = torch.randn(2, SMALL["embed_dim"], 5, 7, generator=g)
    out["scale_in"] = z.numpy()
    out["scale_out"] = sb(z).numpy()
    np.savez_compressed(out_path, **out)
    print(f"wrote {out_path}: {len(out)} arrays, {out_path.stat().st_size / 1024:.0f} KiB")


if __name__ == "__main__":
    root = Path(sys.argv[1] if len(sys.argv) > 1 else "/root/reference")
    main(root, Path(__file__).resolve().parent / "model_golden.npz")
