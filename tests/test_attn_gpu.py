"""GPU parity of the tcgen05 attention forward (through the C-ABI) against the float64 softmax oracle.
Tolerance: rel. Frobenius <= 4e-3 for bf16 (P and O rounded to bf16), 1e-3 for f16; max abs error reported."""
import numpy as np
import pytest
import torch

from oracle import attn_oracle as ao
from oracle import gemm_oracle as go

pytestmark = pytest.mark.gpu


def _ops():
    from lightly_trian_quant_b200 import ops

    return ops


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("shape", [(1, 128, 1), (2, 77, 2), (1, 300, 3), (2, 1605, 2), (1, 1805, 1)])
def test_attn_vs_oracle(dtype, shape):
    ops = _ops()
    B, N, H = shape
    g = torch.Generator().manual_seed(N)
    qkv = torch.randn(3, B, N, H, 64, generator=g)
    qkv[0] *= 2.0          # sharper softmax
    qkv = qkv.to(dtype)
    out = ops.attn_fwd(qkv.cuda())
    ops.check_device_error()
    assert out.shape == (B, N, H * 64) and out.dtype == dtype
    ref = ao.attn_ref(qkv.float().numpy())
    err = go.rel_fro(out.float().cpu().numpy(), ref)
    assert err < (4e-3 if dtype == torch.bfloat16 else 1e-3), err


def test_attn_massive_activation_rows():
    """a few key rows with very large norm (the cls / register tokens of DINOv3): softmax stays finite and exact."""
    ops = _ops()
    B, N, H = 1, 517, 2
    g = torch.Generator().manual_seed(1)
    qkv = torch.randn(3, B, N, H, 64, generator=g)
    qkv[1, :, :5] *= 30
    qkv[0, :, 100:110] *= 10
    qkv = qkv.to(torch.bfloat16)
    out = ops.attn_fwd(qkv.cuda())
    ops.check_device_error()
    assert torch.isfinite(out).all()
    ref = ao.attn_ref(qkv.float().numpy())
    assert go.rel_fro(out.float().cpu().numpy(), ref) < 6e-3


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_attn_logits_growing_along_the_keys(dtype):
    """the key norm grows with the key index, so for most rows later key tiles hold far larger logits than the running
    maximum of the earlier ones (by more than 2^15 in the exponent domain for many of them, by less for others): the rows
    that have to raise their maximum late and rescale O, and the rows that do not, in the same warp."""
    ops = _ops()
    B, N, H = 1, 453, 2
    g = torch.Generator().manual_seed(7)
    qkv = torch.randn(3, B, N, H, 64, generator=g)
    qkv[0] *= 1.5
    qkv[1] *= (0.2 + torch.arange(N).float() / 30.0).view(1, N, 1, 1)
    qkv[0, :, ::3] *= 0.05                                  # every third query row stays flat: no rescale there
    qkv = qkv.to(dtype)
    out = ops.attn_fwd(qkv.cuda())
    ops.check_device_error()
    assert torch.isfinite(out).all()
    ref = ao.attn_ref(qkv.float().numpy())
    err = go.rel_fro(out.float().cpu().numpy(), ref)
    assert err < (6e-3 if dtype == torch.bfloat16 else 2e-3), err


def test_attn_permutation_of_keys_is_neutral():
    """size-independent property: permuting the keys (and values with them) leaves O unchanged up to rounding."""
    ops = _ops()
    B, N, H = 1, 1605, 4
    g = torch.Generator().manual_seed(2)
    qkv = torch.randn(3, B, N, H, 64, generator=g).to(torch.bfloat16).cuda()
    perm = torch.randperm(N, generator=g).cuda()
    o1 = ops.attn_fwd(qkv)
    qkv2 = qkv.clone()
    qkv2[1] = qkv[1][:, perm]
    qkv2[2] = qkv[2][:, perm]
    o2 = ops.attn_fwd(qkv2.contiguous())
    ops.check_device_error()
    assert go.rel_fro(o2.float().cpu().numpy(), o1.float().cpu().numpy()) < 4e-3


@pytest.mark.parametrize("fmt", ["mx8", "nv4", "mx4"])
def test_attn_fused_quantise_out(fmt):
    """attention with the output quantisation fused in: bit-exact against the oracle quantiser applied to the bf16
    output of the unfused kernel (same arithmetic up to the final rounding), scales in the blocked layout."""
    import numpy as np

    from oracle import quant_oracle as qo

    ops = _ops()
    B, N, H = 2, 333, 4
    g = torch.Generator().manual_seed(3)
    qkv = torch.randn(3, B, N, H, 64, generator=g).to(torch.bfloat16).cuda()
    o = ops.attn_fwd(qkv).view(B * N, H * 64)
    on = o.float().cpu().numpy()
    out = ops.ActBuf(B * N, H * 64, fmt, device="cuda")
    ts = None
    if fmt == "nv4":
        ts = qo.nv4_ts(on) * np.float32(2.0)
        out.ts.copy_(torch.from_numpy(ts))
    ops.attn_fwd_quant(qkv, out)
    ops.check_device_error()
    eq, es, _ = qo.quantize(on, fmt, ts)
    assert np.array_equal(out.q.cpu().numpy(), eq)
    assert np.array_equal(out.sf.cpu().numpy(), qo.to_blocked(es).reshape(-1))
