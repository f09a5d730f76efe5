"""CPU oracle of the attention forward: test infrastructure, not product code.

Float64 softmax attention over the physical [3, B, N, H, 64] layout, softmax scale 64^-0.5, no mask: the
reference's own check (infer-opt/round11_attn_tier0/tests/test_attn16.py:31-39, ref_attn) and the model semantics
(src/lightly_train/_task_models/dinov3_eomt_semantic_segmentation/task_model.py:686-693).  Pinned by tolerance, as in
the reference (attention is not bit-reproducible across summation orders).
"""
from __future__ import annotations

import numpy as np


def attn_ref(qkv: np.ndarray) -> np.ndarray:
    """qkv [3, B, N, H, 64] -> O [B, N, H*64] float64."""
    q, k, v = (np.asarray(qkv[i], dtype=np.float64).transpose(0, 2, 1, 3) for i in range(3))   # [B, H, N, 64]
    s = np.einsum("bhqd,bhkd->bhqk", q, k) * 0.125
    s -= s.max(-1, keepdims=True)
    p = np.exp(s)
    p /= p.sum(-1, keepdims=True)
    o = np.einsum("bhqk,bhkd->bhqd", p, v)
    B, H, N, D = o.shape
    return o.transpose(0, 2, 1, 3).reshape(B, N, H * D)
