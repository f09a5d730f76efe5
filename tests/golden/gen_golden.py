"""Generates tests/golden/quant_golden.npz by running the REFERENCE quantisers, imported unmodified.

Run once, in a container where the reference checkout is mounted (pass its root as argv[1]); the GPU box never
runs this.  Sources imported:
    <ref>/infer-opt/round10_lowp_probe/impl/quant_ref.py      mx8_quantize / nv4_quantize / mx4_quantize / to_blocked / qdq
    <ref>/train-opt/round20_fp4_probe/impl/fp4_ref.py         quantize_matrix / dequant_copy (cross-check of the FP4 rules)
Everything runs on the host cores (torch CPU), i.e. python-scalar divisions are true IEEE divisions.

Cases follow the distributions of the reference's own operator tests:
    heavy()  randn with column 5 x30, column K/3 x12, one zero row  (round14_fp4_full/tests/t_quant14.py:18-23)
    mk()     randn with every 97th column x8                         (round13_mxfp8_full/tests/test13a.py:46-50)
    normal / outlier / wide / zeros                                  (round10_lowp_probe/tests/test_quant_ref.py:29-62)
plus the first rows of the single-GEMM benchmark input (bf16, 1 % of channels x20) and lattice-midpoint probes.
"""
from __future__ import annotations

import importlib.util
import sys
from pathlib import Path

import numpy as np
import torch


def _load(path: Path, name: str):
    spec = importlib.util.spec_from_file_location(name, path)
    mod = importlib.util.module_from_spec(spec)
    sys.modules[name] = mod
    spec.loader.exec_module(mod)
    return mod


def cases():
    g = torch.Generator().manual_seed(0)
    out = {}
    out["normal_37x256"] = torch.randn(37, 256, generator=g)
    x = torch.randn(130, 768, generator=g)
    x[:, 5] *= 30
    x[:, 768 // 3] *= 12
    x[7] = 0
    out["heavy_130x768"] = x
    x = torch.randn(65, 1024, generator=g)
    x[:, ::97] *= 8
    out["mk_65x1024"] = x
    x = torch.randn(33, 512, generator=g) * torch.exp2(torch.randint(-40, 40, (33, 512 // 32, 1), generator=g).float()).expand(33, 16, 32).reshape(33, 512)
    out["wide_33x512"] = x
    x = torch.randn(16, 128, generator=g)
    x[3] = 0
    x[5, 32:64] = 0
    x[6, :16] = 0
    out["zeros_16x128"] = x
    # single-GEMM benchmark input recipe, first 96 rows: N(0,1), 1 % of channels x20, rounded to bf16
    gc = torch.Generator().manual_seed(0)
    X = torch.randn(1605, 1024, generator=gc)
    ch = torch.randperm(1024, generator=gc)[:10]
    X[:, ch] *= 20
    out["c1_bf16_96x1024"] = X[:96].to(torch.bfloat16).float()
    # row outliers: 5 prefix rows x1000 (massive activations on cls/register rows)
    x = torch.randn(40, 256, generator=g)
    x[:5] *= 1000
    out["rowout_40x256"] = x
    # lattice probes: exact e2m1 / e4m3 midpoints and neighbours after scaling by the block maximum
    mids = torch.tensor([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, 6.0, 0.0, -0.25, -0.75, -1.25, -1.75, -2.5, -3.5, -5.0])
    blk = torch.cat([mids, mids * (1 + 2 ** -20), mids * (1 - 2 ** -20), -mids])[:64]
    out["mid_e2m1_4x64"] = torch.stack([blk, blk * 2, blk * 0.5, blk * 3.0])
    e4 = torch.arange(0, 64).float()
    row = torch.cat([(e4 + 0.5) * 2.0 ** -9 * 448 / 448, 448 - e4 * 8 - 4.0])
    out["mid_e4m3_2x128"] = torch.stack([row, -row * 0.37])
    return out


def main(ref_root: str):
    ref = Path(ref_root)
    qr = _load(ref / "infer-opt/round10_lowp_probe/impl/quant_ref.py", "quant_ref")
    fr = _load(ref / "train-opt/round20_fp4_probe/impl/fp4_ref.py", "fp4_ref")
    blob = {}
    for name, x in cases().items():
        x = x.contiguous()
        blob[f"{name}/x"] = x.numpy()
        q, b = qr.mx8_quantize(x)
        blob[f"{name}/mx8_q"] = q.view(torch.uint8).numpy()
        blob[f"{name}/mx8_s"] = b.numpy()
        blob[f"{name}/mx8_sb"] = qr.to_blocked(b).numpy()
        small = x.numel() <= 16384          # dequantised tensors only for the small cases (fixture size)
        if small:
            blob[f"{name}/mx8_dq"] = qr.mx8_dequant(q, b).numpy()
        q, sf, ts = qr.nv4_quantize(x)
        blob[f"{name}/nv4_q"] = q.numpy()
        blob[f"{name}/nv4_s"] = sf.view(torch.uint8).numpy()
        blob[f"{name}/nv4_ts"] = ts.numpy()
        blob[f"{name}/nv4_sb"] = qr.to_blocked(sf.view(torch.uint8)).numpy()
        if small:
            blob[f"{name}/nv4_dq"] = qr.nv4_dequant(q, sf, ts).numpy()
        # static calibrated scale with headroom 2 (round14_fp4_full/impl/fp4util.py:41,68-75)
        amax = x.abs().amax()
        ts2 = torch.where(amax > 0, amax * (2.0 / 2688.0), torch.ones_like(amax)).reshape(1)
        q2, sf2, _ = qr.nv4_quantize(x, ts2)
        blob[f"{name}/nv4h_ts"] = ts2.numpy()
        blob[f"{name}/nv4h_q"] = q2.numpy()
        blob[f"{name}/nv4h_s"] = sf2.view(torch.uint8).numpy()
        q, b = qr.mx4_quantize(x)
        blob[f"{name}/mx4_q"] = q.numpy()
        blob[f"{name}/mx4_s"] = b.numpy()
        if small:
            blob[f"{name}/mx4_dq"] = qr.mx4_dequant(q, b).numpy()
        # cross-check with the second reference module: identical codes / blocked scales / ts
        for fmt, qq, ss in (("nv4", blob[f"{name}/nv4_q"], blob[f"{name}/nv4_sb"]), ("mx4", blob[f"{name}/mx4_q"], None)):
            fq, fsf, fts = fr.quantize_matrix(x, fmt)
            assert np.array_equal(fq.numpy(), qq), (name, fmt)
            if fmt == "nv4":
                assert np.array_equal(fsf.numpy(), ss) and np.array_equal(fts.numpy(), blob[f"{name}/nv4_ts"])
            else:
                assert np.array_equal(fsf.numpy(), qr.to_blocked(torch.from_numpy(blob[f"{name}/mx4_s"])).numpy())
    # non-finite inputs (NaN, +Inf, -Inf in different blocks): only the codes and scale bytes, with a given static nv4 scale
    # (a data-derived per-tensor scale would be NaN itself)
    gn = torch.Generator().manual_seed(5)
    xn = torch.randn(4, 128, generator=gn)
    xn[0, 3], xn[1, 40], xn[2, 100], xn[3, 127] = float("nan"), float("inf"), float("-inf"), float("nan")
    blob["nonfinite/x"] = xn.numpy()
    q, b = qr.mx8_quantize(xn)
    blob["nonfinite/mx8_q"], blob["nonfinite/mx8_s"] = q.view(torch.uint8).numpy(), b.numpy()
    q, b = qr.mx4_quantize(xn)
    blob["nonfinite/mx4_q"], blob["nonfinite/mx4_s"] = q.numpy(), b.numpy()
    tsn = torch.tensor([0.01])
    q, sf, _ = qr.nv4_quantize(xn, tsn)
    blob["nonfinite/nv4h_ts"], blob["nonfinite/nv4h_q"], blob["nonfinite/nv4h_s"] = tsn.numpy(), q.numpy(), sf.view(torch.uint8).numpy()
    # config-1 GEMM slice: dequant(X[:96]) @ dequant(W[:128])^T + bias -> fp32 and bf16 (the reference's CPU path)
    gc = torch.Generator().manual_seed(0)
    X = torch.randn(1605, 1024, generator=gc)
    ch = torch.randperm(1024, generator=gc)[:10]
    X[:, ch] *= 20
    W = (torch.randn(4096, 1024, generator=gc) * 0.02).to(torch.bfloat16)
    bias = (torch.randn(4096, generator=gc) * 0.02).to(torch.bfloat16)
    Xs, Ws, bs = X[:96].to(torch.bfloat16), W[:128], bias[:128]
    blob["c1gemm/x"] = Xs.float().numpy()
    blob["c1gemm/w"] = Ws.float().numpy()
    blob["c1gemm/bias"] = bs.float().numpy()
    for fmt in ("mx8", "nv4", "mx4"):
        y = qr.qdq(Xs.float(), fmt) @ qr.qdq(Ws.float(), fmt).t() + bs.float()
        blob[f"c1gemm/{fmt}_y"] = y.numpy()
    out = Path(__file__).resolve().parent / "quant_golden.npz"
    np.savez_compressed(out, **blob)
    print("wrote", out, out.stat().st_size, "bytes", len(blob), "arrays")


if __name__ == "__main__":
    if len(sys.argv) < 2:
        sys.exit("usage: gen_golden.py <path to the reference checkout>")
    main(sys.argv[1])
