"""Per-kernel micro-benchmarks of the hot path at the ViT shapes (CUDA events on the launching stream, rotating buffers
larger than L2 so operands come from HBM, not from cache).

    python -m lightly_trian_quant_b200.microbench gemm --fmt nv4 --kind fc1 --batch 8 [--iters 20]
    python -m lightly_trian_quant_b200.microbench lib_gemm --fmt mx8 --kind fc1 --batch 8      # cuBLASLt comparator
    python -m lightly_trian_quant_b200.microbench attn --batch 8 --tokens 1605
    python -m lightly_trian_quant_b200.microbench ln_quant --fmt mx8 --batch 8
    python -m lightly_trian_quant_b200.microbench quant_rows --fmt nv4 --batch 8 --k 1024
    python -m lightly_trian_quant_b200.microbench dw_ln --batch 14 --hs 80 --k 1024
    python -m lightly_trian_quant_b200.microbench peak --fmt nv4
    python -m lightly_trian_quant_b200.microbench sweep --fmt nv4        # quantise + GEMM over every ViT-L linear at 1 / 8 / 32 frames

`kind` selects the GEMM shape AND its fused epilogue: qkv (bias + RoPE + relayout), proj / fc2 (bias, LayerScale,
fp32 residual in place), fc1 (bias + GELU + quantise-out), plain (bf16 out).  Prints one JSON line.
Timing method after infer-opt/round10_lowp_probe/bench10.py:1-8,62-63 (cold weights: R independent copies > L2).
"""
from __future__ import annotations

import argparse
import json

import torch

from . import ops

BF = torch.bfloat16
SHAPES = {"qkv": (1024, 3072), "proj": (1024, 1024), "fc1": (1024, 4096), "fc2": (4096, 1024), "plain": (1024, 4096)}


def _time(fn, iters, warm=5):
    for i in range(warm):
        fn(i)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(iters):
        fn(warm + i)
    e1.record()
    torch.cuda.synchronize()
    ops.check_device_error()
    return e0.elapsed_time(e1) / iters * 1e-3


def _act(M, K, fmt, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    x = torch.randn(M, K, generator=g, device="cuda").to(BF)
    if fmt == "bf16":
        return x
    a = ops.ActBuf(M, K, fmt)
    if fmt == "nv4":
        a.ts.fill_(float(x.float().abs().max()) / 2688.0)
    ops.quant_rows(x, a)
    return a


def bench_gemm(args):
    K, N = SHAPES[args.kind]
    M = args.tokens * args.batch
    fmt = args.fmt
    copies = max(2, int(2 * 126e6 / (N * K)) + 1) if args.cold else 1
    g = torch.Generator(device="cuda").manual_seed(0)
    Ws = [ops.QWeight(torch.randn(N, K, generator=g, device="cuda") * 0.02, fmt) for _ in range(min(copies, 8))]
    acts = [_act(M, K, fmt, s) for s in range(2)]
    bias = torch.randn(N, device="cuda") * 0.02
    gamma = torch.rand(N, device="cuda")
    H = 16
    ang = torch.rand(args.tokens, 32, device="cuda") * 6.28                 # second half of the tables = first half, as in the model
    sin, cos = torch.sin(torch.cat((ang, ang), 1)).contiguous(), torch.cos(torch.cat((ang, ang), 1)).contiguous()    # [tokens, 64]: more rows than any prefix needs
    res = [torch.randn(M, N, device="cuda") for _ in range(args.res_copies)] if args.kind in ("proj", "fc2") else None
    outq = ops.ActBuf(M, N, fmt if fmt != "bf16" else "mx8") if args.kind == "fc1" else None
    if outq is not None and outq.fmt == "nv4":
        outq.ts.fill_(0.01)
    outb = torch.empty(M, N, device="cuda", dtype=BF) if args.kind == "plain" else None

    def fn(i):
        a, W = acts[i % 2], Ws[i % len(Ws)]
        if args.kind == "qkv":
            ops.qkv_rope(a, W, bias, sin, cos, args.tokens, args.prefix, H, half_tables=not args.general_tables)
        elif args.kind in ("proj", "fc2"):
            ops.gemm_res(a, W, bias, gamma, res[i % len(res)], out=res[i % len(res)])
        elif args.kind == "fc1":
            if fmt == "bf16":
                ops.gemm_plain(a, W, bias, gelu=True)
            else:
                ops.gemm_gelu_q(a, W, bias, outq, round_bf16=True)
        else:
            ops.gemm_plain(a, W, out=outb)

    t = _time(fn, args.iters)
    fl = 2.0 * M * N * K
    return {"kernel": f"gemm {fmt} {args.kind}", "M": M, "N": N, "K": K, "us": t * 1e6, "TFLOP/s": fl / t / 1e12}


def bench_lib_gemm(args):
    """Same-box library comparator: cuBLASLt through torch._scaled_mm (block-scaled mx8 / nv4 / mx4) or torch.matmul (bf16)
    on operands quantised by this library (its blocked scale layout is the swizzled layout cuBLASLt expects); plain bf16
    output, no fused epilogue.  M is rounded up to a multiple of 128."""
    K, N = SHAPES[args.kind]
    M = (args.tokens * args.batch + 127) // 128 * 128
    fmt = args.fmt
    g = torch.Generator(device="cuda").manual_seed(0)
    copies = max(2, int(2 * 126e6 / (N * K)) + 1)
    Ws = [ops.QWeight(torch.randn(N, K, generator=g, device="cuda") * 0.02, fmt) for _ in range(min(copies, 8))]
    acts = [_act(M, K, fmt, s) for s in range(2)]
    if fmt == "bf16":
        def fn(i):
            torch.matmul(acts[i % 2], Ws[i % len(Ws)].q.t())
    else:
        dt = torch.float8_e4m3fn if fmt == "mx8" else torch.float4_e2m1fn_x2
        st = torch.float8_e4m3fn if fmt == "nv4" else torch.float8_e8m0fnu
        A = [(a.q.view(dt), a.sf.view(st)) for a in acts]
        Wv = [(w.q.view(dt).t(), w.sf.view(st)) for w in Ws]

        def fn(i):
            a, sa = A[i % 2]
            w, sw = Wv[i % len(Wv)]
            torch._scaled_mm(a, w, scale_a=sa, scale_b=sw, out_dtype=BF)
    try:
        t = _time(fn, args.iters)
    except Exception as e:  # the library may not offer the format on this build
        return {"kernel": f"library gemm {fmt} {args.kind}", "unavailable": str(e).split("\n")[0][:300]}
    fl = 2.0 * M * N * K
    return {"kernel": f"library gemm {fmt} {args.kind} (torch._scaled_mm / matmul, bf16 out)", "M": M, "N": N, "K": K, "us": t * 1e6, "TFLOP/s": fl / t / 1e12}


def bench_attn(args):
    B, N, H = args.batch, args.tokens, 16
    dt = torch.float16 if args.dtype == "f16" else BF
    qkvs = [torch.randn(3, B, N, H, 64, device="cuda").to(dt) for _ in range(2)]
    outs = [torch.empty(B, N, H * 64, device="cuda", dtype=dt) for _ in range(2)]
    if args.quant_out:                      # the form the block uses: O quantised into the proj GEMM's operand
        bufs = [ops.ActBuf(B * N, H * 64, args.fmt, device="cuda") for _ in range(2)]
        for b in bufs:
            if b.ts is not None:
                b.ts.fill_(0.01)
        t = _time(lambda i: ops.attn_fwd_quant(qkvs[i % 2], bufs[i % 2]), args.iters)
    else:
        t = _time(lambda i: ops.attn_fwd(qkvs[i % 2], out=outs[i % 2]), args.iters)
    fl = 4.0 * B * H * N * N * 64
    tag = f" + {args.fmt} quantise-out" if args.quant_out else ""
    return {"kernel": f"attn_fwd {args.dtype}{tag}", "B": B, "N": N, "H": H, "us": t * 1e6, "TFLOP/s": fl / t / 1e12}


def bench_ln_quant(args):
    M, d = args.tokens * args.batch, args.k
    n = max(2, int(2 * 126e6 / (M * d * 4)) + 1)
    xs = [torch.randn(M, d, device="cuda") for _ in range(n)]
    bufs = [ops.ActBuf(M, d, args.fmt) for _ in range(n)]
    w, b = torch.ones(d, device="cuda"), torch.zeros(d, device="cuda")
    t = _time(lambda i: ops.ln_quant(xs[i % n], w, b, 1e-5, bufs[i % n], round_bf16=True), args.iters)
    by = M * d * 4 + bufs[0].q.numel() + bufs[0].sf.numel()
    return {"kernel": f"ln_quant {args.fmt}", "M": M, "d": d, "us": t * 1e6, "GB/s": by / t / 1e9, "bytes": by}


def bench_quant_rows(args):
    M, K = args.tokens * args.batch, args.k
    n = max(2, int(2 * 126e6 / (M * K * 2)) + 1)
    xs = [torch.randn(M, K, device="cuda").to(BF) for _ in range(n)]
    bufs = [ops.ActBuf(M, K, args.fmt) for _ in range(n)]
    t = _time(lambda i: ops.quant_rows(xs[i % n], bufs[i % n]), args.iters)
    by = M * K * 2 + bufs[0].q.numel() + bufs[0].sf.numel()
    return {"kernel": f"quant_rows bf16->{args.fmt}", "M": M, "K": K, "us": t * 1e6, "GB/s": by / t / 1e9, "bytes": by}


def bench_dw_ln(args):
    B, Hs, C = args.batch, args.hs, args.k
    n = max(2, int(2 * 126e6 / (B * Hs * Hs * 4 * C * 2)) + 1)
    gs = [torch.randn(B * Hs * Hs, 4 * C, device="cuda").to(BF) for _ in range(n)]
    dww, lnw, lnb = torch.randn(9, C, device="cuda") * 0.3, torch.ones(C, device="cuda"), torch.zeros(C, device="cuda")
    t = _time(lambda i: ops.dw_ln(gs[i % n], None, dww, lnw, lnb, B, Hs, Hs, 1e-6, pre_act=True), args.iters)
    by = 2 * gs[0].numel() * 2
    return {"kernel": "dw_ln", "B": B, "Hs": Hs, "C": C, "us": t * 1e6, "GB/s": by / t / 1e9, "bytes": by}


def bench_peak(args):
    out = {"kernel": f"tcgen05 instruction-rate probe {args.fmt}", "TFLOP/s_n128": ops.tensor_peak_tflops(args.fmt, 128),
           "TFLOP/s_n256": ops.tensor_peak_tflops(args.fmt, 256)}
    if args.fmt != "bf16":
        for c in (1, 2, 4, 8, 10, 12, 16):
            out[f"TFLOP/s_n128_sfcopies{c}"] = ops.tensor_peak_tflops(args.fmt, 128, sf_copies=c)
    return out


def bench_fill(args):
    out = {"kernel": "shared-memory fill-rate probe (bulk copies, 3-stage ring, 148 SMs)"}
    for span_mb in (4, 32, 96):            # windows that stay in L2 (126 MB): the rate a main loop re-reading its operands sees
        for stage in (16384, 32768, 49152, 65536):
            out[f"GB/s_span{span_mb}MB_stage{stage // 1024}KB"] = round(ops.smem_fill_rate_gbs(span_mb << 20, stage), 1)
    return out


def bench_sweep(args):
    """The quantise + GEMM sweep over every ViT-L/16 linear shape (qkv, proj, fc1, fc2 with their fused epilogues) at
    M = 1605 x {1, 8, 32} in one format, plus the row quantiser and the LayerNorm + quantiser at the same sizes: one JSON
    document with us, TFLOP/s and GB/s per (shape, frames)."""
    import copy

    out = {"kernel": f"sweep {args.fmt}", "tokens": args.tokens, "rows": {}}
    for frames in (1, 8, 32):
        a = copy.copy(args)
        a.batch = frames
        a.iters = max(5, min(args.iters, 200 // frames))
        row = {}
        for kind in ("qkv", "proj", "fc1", "fc2"):
            a.kind = kind
            r = bench_gemm(a)
            row[kind] = {"us": round(r["us"], 2), "TFLOP/s": round(r["TFLOP/s"], 1)}
        for k in (1024, 4096):
            a.k = k
            r = bench_quant_rows(a)
            row[f"quant_rows_k{k}"] = {"us": round(r["us"], 2), "GB/s": round(r["GB/s"], 1)}
        a.k = 1024
        r = bench_ln_quant(a)
        row["ln_quant_d1024"] = {"us": round(r["us"], 2), "GB/s": round(r["GB/s"], 1)}
        out["rows"][f"{frames}_frames_M{frames * args.tokens}"] = row
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("what", choices=["gemm", "lib_gemm", "attn", "ln_quant", "quant_rows", "dw_ln", "peak", "fill", "sweep"])
    ap.add_argument("--fmt", default="nv4")
    ap.add_argument("--kind", default="fc1", choices=list(SHAPES))
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--tokens", type=int, default=1605)
    ap.add_argument("--k", type=int, default=1024)
    ap.add_argument("--res-copies", type=int, default=2, help="gemm proj / fc2: residual buffers rotated through (1 = the stream stays where the last launch left it, as far as L2 holds it)")
    ap.add_argument("--hs", type=int, default=80, help="dw_ln: input grid side (output is 2x)")
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--cold", type=int, default=1)
    ap.add_argument("--dtype", default="bf16", choices=["bf16", "f16"])
    ap.add_argument("--quant-out", action="store_true", help="attn: fused quantisation of the output in --fmt")
    ap.add_argument("--prefix", type=int, default=5, help="gemm qkv: tokens per image that are not rotated")
    ap.add_argument("--general-tables", action="store_true", help="gemm qkv: rotary tables without the repeated-half promise (the slower general path)")
    args = ap.parse_args()
    torch.set_grad_enabled(False)
    fn = {"gemm": bench_gemm, "lib_gemm": bench_lib_gemm, "attn": bench_attn, "ln_quant": bench_ln_quant, "quant_rows": bench_quant_rows, "dw_ln": bench_dw_ln, "peak": bench_peak, "fill": bench_fill, "sweep": bench_sweep}[args.what]
    print(json.dumps(fn(args)), flush=True)


if __name__ == "__main__":
    main()
