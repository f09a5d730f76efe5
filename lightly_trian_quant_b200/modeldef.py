"""Minimal torch definition of DINOv3 ViT + EoMT semantic segmentation with the reference's attribute names.

It stands in for the reference's nn.Module where that package is not installed (the GPU box): the stack plugin
(`stack.make_variant(name, model, variant)`) and the Linear swap (`linear_swap.enable(model, units)`) address weights
and sub-modules exactly as they do on the reference model, so either object can be passed:

    model.backbone.patch_embed.proj / cls_token / storage_tokens / rope_embed / blocks[i] / norm / patch_size / n_storage_tokens
    blocks[i].norm1 / attn.qkv (K third of the bias masked) / attn.proj / attn.num_heads / ls1.gamma / norm2 / mlp.fc1 / mlp.act / mlp.fc2 / ls2.gamma
    model.queries / class_head / mask_head / upscale[j].conv1 / conv2 / norm / num_queries / num_joint_blocks

Reference definitions (paths relative to the reference checkout):
    src/lightly_train/_models/dinov3/dinov3_src/models/vision_transformer.py:74-251, hub/backbones.py:270-330 (ViT-B/L configs)
    src/lightly_train/_models/dinov3/dinov3_src/layers/{attention.py:37-110, rope_position_encoding.py:62-127, layer_scale.py}
    src/lightly_train/_task_models/dinov3_eomt_semantic_segmentation/{task_model.py:175-215,416-508,636-698, scale_block.py:19-56}

The forward here is plain torch in the module's dtype (no autocast); it is the unquantised baseline the low-precision
variants are compared with, not a compute path of the library.
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch
import torch.nn.functional as F
from torch import nn


@dataclass
class EoMTConfig:
    dim: int = 1024
    depth: int = 24
    heads: int = 16
    ffn: int = 4096
    n_storage_tokens: int = 4
    patch_size: int = 16
    num_queries: int = 200
    num_joint_blocks: int = 4
    num_classes: int = 2
    ln_eps: float = 1e-5
    layerscale_init: float = 1e-5
    rope_base: float = 100.0


VIT_L = EoMTConfig()
VIT_B = EoMTConfig(dim=768, depth=12, heads=12, ffn=3072)


class LinearKMaskedBias(nn.Linear):
    """qkv projection whose K third of the bias is multiplied by zero (attention.py:37-53)."""

    def __init__(self, *a, **kw):
        super().__init__(*a, **kw)
        self.register_buffer("bias_mask", torch.ones_like(self.bias))
        o = self.out_features
        self.bias_mask[o // 3: 2 * o // 3] = 0

    def forward(self, x):
        return F.linear(x, self.weight, self.bias * self.bias_mask.to(self.bias.dtype))


class LayerScale(nn.Module):
    def __init__(self, dim, init):
        super().__init__()
        self.gamma = nn.Parameter(torch.full((dim,), float(init)))

    def forward(self, x):
        return x * self.gamma


class RopePositionEmbedding(nn.Module):
    """axial 2-D RoPE tables, eval mode (rope_position_encoding.py:62-127): coords (i+0.5)/H mapped to [-1,1],
    periods base^(2t/(D/2)), angles 2*pi*coord/period, [h-angles | w-angles] repeated twice -> sin, cos [HW, D]."""

    def __init__(self, head_dim: int, base: float):
        super().__init__()
        self.register_buffer("periods", base ** (2 * torch.arange(head_dim // 4, dtype=torch.float32) / (head_dim // 2)))

    def forward(self, *, H: int, W: int):
        dd = dict(device=self.periods.device, dtype=torch.float32)
        ch = torch.arange(0.5, H, **dd) / H
        cw = torch.arange(0.5, W, **dd) / W
        coords = torch.stack(torch.meshgrid(ch, cw, indexing="ij"), dim=-1).flatten(0, 1)
        coords = 2.0 * coords - 1.0
        angles = 2 * math.pi * coords[:, :, None] / self.periods[None, None, :]
        angles = angles.flatten(1, 2)
        angles = torch.cat((angles, angles), dim=-1)
        return torch.sin(angles), torch.cos(angles)


def rope_apply(x, sin, cos):
    x1, x2 = x.chunk(2, dim=-1)
    return x * cos + torch.cat([-x2, x1], dim=-1) * sin


class SelfAttention(nn.Module):
    def __init__(self, dim, heads):
        super().__init__()
        self.num_heads = heads
        self.qkv = LinearKMaskedBias(dim, 3 * dim, bias=True)
        self.proj = nn.Linear(dim, dim, bias=True)


class Mlp(nn.Module):
    def __init__(self, dim, ffn):
        super().__init__()
        self.fc1 = nn.Linear(dim, ffn)
        self.act = nn.GELU()
        self.fc2 = nn.Linear(ffn, dim)

    def forward(self, x):
        return self.fc2(self.act(self.fc1(x)))


class SelfAttentionBlock(nn.Module):
    def __init__(self, cfg: EoMTConfig):
        super().__init__()
        self.norm1 = nn.LayerNorm(cfg.dim, eps=cfg.ln_eps)
        self.attn = SelfAttention(cfg.dim, cfg.heads)
        self.ls1 = LayerScale(cfg.dim, cfg.layerscale_init)
        self.norm2 = nn.LayerNorm(cfg.dim, eps=cfg.ln_eps)
        self.mlp = Mlp(cfg.dim, cfg.ffn)
        self.ls2 = LayerScale(cfg.dim, cfg.layerscale_init)


class PatchEmbed(nn.Module):
    def __init__(self, cfg: EoMTConfig):
        super().__init__()
        self.proj = nn.Conv2d(3, cfg.dim, kernel_size=cfg.patch_size, stride=cfg.patch_size)

    def forward(self, x):
        return self.proj(x).permute(0, 2, 3, 1)     # [B, gh, gw, d]


class DinoVisionTransformer(nn.Module):
    def __init__(self, cfg: EoMTConfig):
        super().__init__()
        self.embed_dim, self.patch_size, self.n_storage_tokens = cfg.dim, cfg.patch_size, cfg.n_storage_tokens
        self.patch_embed = PatchEmbed(cfg)
        self.cls_token = nn.Parameter(torch.zeros(1, 1, cfg.dim))
        self.storage_tokens = nn.Parameter(torch.zeros(1, cfg.n_storage_tokens, cfg.dim))
        self.mask_token = nn.Parameter(torch.zeros(1, cfg.dim), requires_grad=False)
        self.rope_embed = RopePositionEmbedding(cfg.dim // cfg.heads, cfg.rope_base)
        self.blocks = nn.ModuleList(SelfAttentionBlock(cfg) for _ in range(cfg.depth))
        self.norm = nn.LayerNorm(cfg.dim, eps=cfg.ln_eps)

    def prepare_tokens_with_masks(self, x):
        x = self.patch_embed(x)
        B, H, W, _ = x.shape
        x = x.flatten(1, 2)
        x = torch.cat([self.cls_token.to(x.dtype).expand(B, -1, -1), self.storage_tokens.to(x.dtype).expand(B, -1, -1), x], dim=1)
        return x, (H, W)


class LayerNorm2D(nn.LayerNorm):
    def forward(self, x):
        return super().forward(x.permute(0, 2, 3, 1)).permute(0, 3, 1, 2)


class ScaleBlock(nn.Module):
    def __init__(self, dim):
        super().__init__()
        self.conv1 = nn.ConvTranspose2d(dim, dim, kernel_size=2, stride=2)
        self.act = nn.GELU()
        self.conv2 = nn.Conv2d(dim, dim, kernel_size=3, padding=1, groups=dim, bias=False)
        self.norm = LayerNorm2D(dim)

    def forward(self, x):
        return self.norm(self.conv2(self.act(self.conv1(x))))


class DINOv3EoMTSemanticSegmentation(nn.Module):
    def __init__(self, cfg: EoMTConfig):
        super().__init__()
        self.cfg = cfg
        self.backbone = DinoVisionTransformer(cfg)
        self.num_queries, self.num_joint_blocks = cfg.num_queries, cfg.num_joint_blocks
        self.queries = nn.Embedding(cfg.num_queries, cfg.dim)
        self.class_head = nn.Linear(cfg.dim, cfg.num_classes + 1)
        self.mask_head = nn.Sequential(nn.Linear(cfg.dim, cfg.dim), nn.GELU(), nn.Linear(cfg.dim, cfg.dim), nn.GELU(), nn.Linear(cfg.dim, cfg.dim))
        self.upscale = nn.Sequential(*[ScaleBlock(cfg.dim) for _ in range(max(1, math.ceil(math.log2(16)) - 2))])

    def _attn(self, module: SelfAttention, x, rope):
        qkv = module.qkv(x)
        B, N, _ = qkv.shape
        C = module.qkv.in_features
        q, k, v = torch.unbind(qkv.reshape(B, N, 3, module.num_heads, C // module.num_heads), 2)
        q, k, v = [t.transpose(1, 2) for t in (q, k, v)]
        sin, cos = rope
        prefix = N - sin.shape[-2]
        q = torch.cat((q[:, :, :prefix], rope_apply(q[:, :, prefix:].float(), sin, cos).to(q.dtype)), dim=2)
        k = torch.cat((k[:, :, :prefix], rope_apply(k[:, :, prefix:].float(), sin, cos).to(k.dtype)), dim=2)
        x = F.scaled_dot_product_attention(q, k, v)
        return module.proj(x.transpose(1, 2).reshape(B, N, C))

    def _predict(self, x, grid_size):
        q = x[:, : self.num_queries]
        class_logits = self.class_head(q)
        x = x[:, self.num_queries + 1 + self.backbone.n_storage_tokens:]
        x = x.transpose(1, 2).reshape(x.shape[0], -1, *grid_size)
        mask_logits = torch.einsum("bqc,bchw->bqhw", self.mask_head(q), self.upscale(x))
        return mask_logits, class_logits

    def forward(self, x):
        """x [B, 3, S, S] -> (mask_logits [B, Q, S/4, S/4], class_logits [B, Q, classes+1]) of the last layer
        (forward_train without per-layer logits, task_model.py:416-508)."""
        bb = self.backbone
        _, _, H, W = x.shape
        grid = (H // bb.patch_size, W // bb.patch_size)
        t, (gh, gw) = bb.prepare_tokens_with_masks(x)
        rope = bb.rope_embed(H=gh, W=gw)
        nb = len(bb.blocks)
        for i, blk in enumerate(bb.blocks):
            if i == nb - self.num_joint_blocks:
                t = torch.cat((self.queries.weight[None].to(t.dtype).expand(t.shape[0], -1, -1), t), dim=1)
            t = t + blk.ls1(self._attn(blk.attn, blk.norm1(t), rope))
            t = t + blk.ls2(blk.mlp(blk.norm2(t)))
        return self._predict(bb.norm(t), grid)


@torch.no_grad()
def init_weights(model: DINOv3EoMTSemanticSegmentation, seed: int = 0, mode: str = "upstream") -> DINOv3EoMTSemanticSegmentation:
    """Seeded random initialisation.
    mode "upstream": the reference's own init (vision_transformer.py:55-72,211-217: trunc_normal(0.02) linears, zero
        biases, LayerScale 1e-5, cls / storage tokens N(0, 0.02)); every block then contributes ~1e-5 of its output, so
        this mode alone cannot reveal a broken GEMM.
    mode "stress": LayerScale ~ U(0.5, 1.5)/sqrt(depth), LN affine ~ U(0.5, 1.5) / N(0, 0.1), biases N(0, 0.02) and 1 % of
        the patch-embed output channels scaled x20, so quantisation error propagates through the network."""
    g = torch.Generator().manual_seed(seed)
    cfg = model.cfg

    def tn(t, std=0.02):
        t.copy_(torch.nn.init.trunc_normal_(torch.empty(t.shape), std=std, generator=g))

    for m in model.modules():
        if isinstance(m, nn.Linear):
            tn(m.weight)
            m.bias.zero_()
        elif isinstance(m, nn.LayerNorm):
            m.weight.fill_(1.0)
            m.bias.zero_()
        elif isinstance(m, LayerScale):
            m.gamma.fill_(cfg.layerscale_init)
        elif isinstance(m, (nn.Conv2d, nn.ConvTranspose2d)):
            fan = m.weight[0].numel() if isinstance(m, nn.Conv2d) else m.weight.shape[0] * 4
            m.weight.copy_((torch.rand(m.weight.shape, generator=g) * 2 - 1) / math.sqrt(fan))
            if m.bias is not None:
                m.bias.copy_((torch.rand(m.bias.shape, generator=g) * 2 - 1) / math.sqrt(fan))
    model.backbone.cls_token.copy_(torch.randn(model.backbone.cls_token.shape, generator=g) * 0.02)
    model.backbone.storage_tokens.copy_(torch.randn(model.backbone.storage_tokens.shape, generator=g) * 0.02)
    model.queries.weight.copy_(torch.randn(model.queries.weight.shape, generator=g))
    if mode == "stress":
        for m in model.modules():
            if isinstance(m, nn.Linear):
                m.bias.copy_(torch.randn(m.bias.shape, generator=g) * 0.02)
            elif isinstance(m, nn.LayerNorm):
                m.weight.copy_(torch.rand(m.weight.shape, generator=g) + 0.5)
                m.bias.copy_(torch.randn(m.bias.shape, generator=g) * 0.1)
            elif isinstance(m, LayerScale):
                m.gamma.copy_((torch.rand(m.gamma.shape, generator=g) + 0.5) / math.sqrt(cfg.depth))
        pe = model.backbone.patch_embed.proj
        ch = torch.randperm(cfg.dim, generator=g)[: max(1, cfg.dim // 100)]
        pe.weight[ch] *= 20
        pe.bias[ch] *= 20
    elif mode != "upstream":
        raise ValueError(mode)
    return model


def build_model(cfg: EoMTConfig, seed: int = 0, mode: str = "upstream", device="cpu") -> DINOv3EoMTSemanticSegmentation:
    model = DINOv3EoMTSemanticSegmentation(cfg)
    init_weights(model, seed, mode)
    return model.to(device).eval()
