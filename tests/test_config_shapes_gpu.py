"""GPU parity at the benchmark configurations' own sizes (through the C-ABI), beyond the small cases of the other files.

  config 2   every ViT-L linear (qkv 1024->3072, proj 1024->1024, fc1 1024->4096, fc2 4096->1024) at M = 1605 x 32 = 51 360
             rows THROUGH ITS FUSED EPILOGUE (bias + RoPE + relayout / LayerScale + residual / GELU + quantise-out); one
             image's worth of rows (the last image: rows that only exist when the batch index arithmetic is right) is checked
             against the float64 oracle, and row independence ties the rest to the small-M launch
  config 5   attention at N = 4101 and 4301 tokens (1024 x 1024 input) in f16 and bf16; ViT-L/16 + EoMT with MXFP4
             linears and fp16 attention at 1024 x 1024, one frame, against the emulated model
  config 4   ViT-L/16 + EoMT NVFP4 at 640 x 640 with a batch of two frames (batch index arithmetic at Ntok = 1605 / 1805)
Tolerances as in the small tests: fp32 outputs 2e-5 / 2e-6, 16-bit outputs 2e-3 (the stated bound), codes and scale bytes exact.
"""
import numpy as np
import pytest
import torch

from oracle import attn_oracle as ao
from oracle import gemm_oracle as go
from oracle import model_oracle as mo
from oracle import quant_oracle as qo

pytestmark = pytest.mark.gpu
torch.set_grad_enabled(False)
BF = torch.bfloat16
NTOK, FRAMES = 1605, 32
SHAPES = {"qkv": (1024, 3072), "proj": (1024, 1024), "fc1": (1024, 4096), "fc2": (4096, 1024)}


def _ops():
    from lightly_trian_quant_b200 import ops

    return ops


def _big_operand(M, K, fmt, seed):
    """activation N(0,1) with 1 % of channels x20, generated on the device (51 360 x 4096 values), quantised there."""
    ops = _ops()
    g = torch.Generator(device="cuda").manual_seed(seed)
    x = torch.randn(M, K, generator=g, device="cuda")
    ch = torch.randperm(K, generator=g, device="cuda")[: K // 100]
    x[:, ch] *= 20
    x = x.to(BF)
    a = ops.ActBuf(M, K, fmt, device="cuda")
    if fmt == "nv4":
        a.ts.fill_(float(x.float().abs().max()) / 2688.0)
    ops.quant_rows(x, a)
    return x, a


def _dequant_rows(a, rows, fmt):
    M, K = a.M, a.K
    nb = K // qo.VEC[fmt]
    s2 = qo.from_blocked(a.sf.cpu().numpy().reshape(-(-M // 128), nb // 4, 32, 4, 4), M, nb)
    ts = a.ts.cpu().numpy() if a.ts is not None else None
    return qo.dequant(a.q[rows].cpu().numpy(), s2[rows], ts, fmt)


@pytest.mark.parametrize("fmt", ["nv4", "mx8"])
@pytest.mark.parametrize("kind", ["qkv", "proj", "fc1", "fc2"])
def test_vitl_linears_at_32_frames_through_their_epilogues(fmt, kind):
    ops = _ops()
    K, N = SHAPES[kind]
    M = NTOK * FRAMES
    x, a = _big_operand(M, K, fmt, 100 + len(kind))
    g = torch.Generator().manual_seed(7)
    W = ops.QWeight((torch.randn(N, K, generator=g) * 0.02).to(BF).cuda(), fmt)
    wd = go.dequant_operand(W.q.cpu().numpy(), W.sf.cpu().numpy(), None if W.ts is None else W.ts.cpu().numpy(), fmt, N, K)
    bias = (torch.randn(N, generator=g) * 0.05)
    rows = slice(M - NTOK, M)                                 # the last image
    acc = go.matmul_ref(_dequant_rows(a, rows, fmt), wd) + bias.numpy().astype(np.float64)
    if kind == "qkv":
        H, prefix = 16, 5
        sin = torch.randn(NTOK - prefix, 64, generator=g)
        cos = torch.randn(NTOK - prefix, 64, generator=g)
        out = ops.qkv_rope(a, W, bias.cuda(), sin.cuda(), cos.cuda(), NTOK, prefix, H, out_dtype=BF)
        ops.check_device_error()
        ref = go.epi_rope(acc, sin.numpy(), cos.numpy(), NTOK, prefix, H)            # [3, 1, Ntok, H, 64]
        err = go.rel_fro(out[:, FRAMES - 1].float().cpu().numpy(), ref[:, 0])
        print(f"qkv+RoPE {fmt} M={M}: bf16 rel. Frobenius {err:.3e}")
        assert err < 2e-3
        # the first image alone gives the same bits (row independence, batch index arithmetic)
        a1 = ops.ActBuf(NTOK, K, fmt, device="cuda", ts=a.ts)
        ops.quant_rows(x[:NTOK], a1)
        o1 = ops.qkv_rope(a1, W, bias.cuda(), sin.cuda(), cos.cuda(), NTOK, prefix, H, out_dtype=BF)
        assert torch.equal(o1[:, 0], out[:, 0])
    elif kind in ("proj", "fc2"):
        gamma = torch.rand(N, generator=g)
        R = torch.randn(M, N, generator=torch.Generator(device="cuda").manual_seed(3), device="cuda")
        Rw = R[rows].cpu().numpy()
        out = ops.gemm_res(a, W, bias.cuda(), gamma.cuda(), R, out=R)                    # in place, as in the block
        ops.check_device_error()
        ref = go.epi_res(acc - bias.numpy().astype(np.float64), bias.numpy(), gamma.numpy(), Rw)
        err = go.rel_fro(out[rows].cpu().numpy(), ref)
        print(f"{kind} residual {fmt} M={M}: fp32 rel. Frobenius {err:.3e}")
        assert err < 2e-6
    else:
        out = ops.ActBuf(M, N, fmt, device="cuda")
        if fmt == "nv4":
            out.ts.fill_(float(np.abs(go.gelu_erf(acc)).max()) * 2.0 / 2688.0)
        y = torch.empty(M, N, device="cuda")
        ops.gemm_gelu_q(a, W, bias.cuda(), out, round_bf16=True, y_dbg=y)
        ops.check_device_error()
        yw = y[rows].cpu().numpy()
        pre = qo.bf16_round(go.gelu_erf(acc).astype(np.float32))
        assert float((yw != pre).mean()) < 2e-3 and go.rel_fro(yw, pre) < 3e-3
        tso = out.ts.cpu().numpy() if out.ts is not None else None
        eq, es, _ = qo.quantize(yw, fmt, tso)
        assert np.array_equal(out.q[rows].cpu().numpy(), eq)
        nb = N // qo.VEC[fmt]
        s2 = qo.from_blocked(out.sf.cpu().numpy().reshape(-(-M // 128), nb // 4, 32, 4, 4), M, nb)
        assert np.array_equal(s2[rows], es)


@pytest.mark.parametrize("dtype", [torch.float16, BF])
@pytest.mark.parametrize("N", [4101, 4301])
def test_attention_at_1024px_token_counts(dtype, N):
    ops = _ops()
    B, H = 1, 2
    g = torch.Generator().manual_seed(N)
    qkv = torch.randn(3, B, N, H, 64, generator=g)
    qkv[0] *= 2.0
    qkv = qkv.to(dtype)
    out = ops.attn_fwd(qkv.cuda())
    ops.check_device_error()
    err = go.rel_fro(out.float().cpu().numpy(), ao.attn_ref(qkv.float().numpy()))
    print(f"attention N={N} {dtype}: rel. Frobenius {err:.3e}")
    assert err < (4e-3 if dtype == BF else 1e-3), err


def _collect_ts(model_fn):
    layers, head = model_fn._keepalive[0], model_fn._keepalive[2]
    ts = {}
    for i, L in enumerate(layers):
        for site in ("ln1", "o", "ln2", "g"):
            t = getattr(L, "ts_" + site)
            if t is not None:
                ts[(i, site)] = t.cpu().numpy()
    for j, st in enumerate(head.stages):
        if st["ts"] is not None:
            ts[("head", j)] = st["ts"].cpu().numpy()
    return ts


@pytest.mark.parametrize("variant,side,batch,gamma", [("b200_mx4+f16attn", 1024, 1, None), ("b200_nv4", 640, 2, None), ("b200_nv4", 640, 1, 0.1), ("b200_mx8", 640, 1, 0.1),
                                                      ("b200_mx4", 640, 1, 0.1)])
def test_vitl_end_to_end_at_config_sizes(variant, side, batch, gamma):
    """ViT-L/16 + EoMT at full width and depth against the emulated model at the same format.
    gamma None: the upstream initialisation (LayerScale 1e-5, what the benchmark configurations use): cosine >= 0.9999.
    gamma 0.1: LayerScale raised to 0.1 in every block so that the blocks' quantisation errors reach the logits (the
    upstream value hides them).  Class logits: cosine >= 0.999.  Mask logits of a random-init network are chaotic under
    quantisation, so their bound is calibrated on the emulation itself: the GPU path may differ from the emulation by no
    more than 3x what a one-bf16-ulp change of 1 % of the input pixels does to the emulation's own mask logits.  All
    measured values are printed."""
    import copy

    from lightly_trian_quant_b200 import modeldef, ops, stack

    fmt = variant.split("+")[0].split("_")[1]
    model = modeldef.build_model(modeldef.VIT_L, 0, "upstream", "cpu")
    if gamma is not None:
        for blk in model.backbone.blocks:
            blk.ls1.gamma.fill_(gamma)
            blk.ls2.gamma.fill_(gamma)
    x = torch.rand(batch, 3, side, side, generator=torch.Generator().manual_seed(21)).to(BF)
    fn, _ = stack.make_variant("vit_l", copy.deepcopy(model).cuda(), f"{variant}+s{side}")
    ml, cl = fn(x.cuda())
    ops.check_device_error()
    g = side // 4
    assert ml.shape == (batch, 200, g, g) and torch.isfinite(ml.float()).all()
    attn_dtype = torch.float16 if "f16attn" in variant else BF
    ts = _collect_ts(fn)
    ml_ref, cl_ref = mo.EmuModel(model, fmt, ts=ts, attn_dtype=attn_dtype)(x.float())
    c_ml, c_cl = mo.cosine(ml.float().cpu(), ml_ref), mo.cosine(cl.float().cpu(), cl_ref)
    msg = f"{variant} {side}px batch {batch} LayerScale {gamma or 1e-5}: mask-logit cosine {c_ml:.6f}, class-logit cosine {c_cl:.6f}"
    if gamma is None:
        print(msg)
        assert c_ml >= 0.9999 and c_cl >= 0.9999, (c_ml, c_cl)
        return
    xp = x.float().clone()
    m = torch.rand(xp.shape, generator=torch.Generator().manual_seed(1)) < 0.01
    xp[m] = (xp[m] * (1 + 2 ** -8)).to(BF).float()
    ml_p, cl_p = mo.EmuModel(model, fmt, ts=ts, attn_dtype=attn_dtype)(xp)
    sens_ml, sens_cl = 1.0 - mo.cosine(ml_p, ml_ref), 1.0 - mo.cosine(cl_p, cl_ref)
    print(msg + f"; the emulation's own 1-cos under a one-ulp input change: mask {sens_ml:.2e}, class {sens_cl:.2e}")
    assert c_cl >= 0.999, (c_cl, sens_cl)
    assert 1.0 - c_ml <= max(3.0 * sens_ml, 1e-4), (c_ml, sens_ml)
