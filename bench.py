"""Headline benchmark: ViT-L/16 + EoMT frames/s with NVFP4 linears on B200 (the 126-frame synthetic video workload, 640x640, frames sharded over the GPUs).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--batch B] [--variant b200_nv4] [--impl reference]

Workload: a seeded synthetic 126-frame uint8 1440x1900x3 video (smooth low-frequency noise + Gaussian noise sigma 8)
stands in for the reference's private clip; frames are sharded round-robin over the ranks, one process per GPU, weights
replicated (random init, upstream recipe), no collective on the data path.  One step = one micro-batch of B frames per
GPU through resize+normalise -> model_fn -> per-pixel labels.

  value  frames/s with the uint8 frames already resident in HBM (CUDA-graph replay of the step, CUDA events, max over ranks)
  e2e    frames/s through the public pipeline (lightly_trian_quant_b200.pipeline.VideoPipeline) with HOST frames: per step the
         pinned-host -> device copy of the B frames, the step, and the device -> host copy of the label maps, on separate
         copy / compute streams over a ring of slots
  video_126   wall-clock of THIS video: every rank runs its shard of the 126 frames once through VideoPipeline.run (the last
         micro-batch padded), slowest rank counts: frames/s of the fixed job, i.e. strong scaling including batch padding
  roofline / kernels   per-kernel-class durations measured live with CUDA events in an instrumented eager pass over the
         same step; the dominant class (block-scaled GEMMs) is reported against the tcgen05 instruction-rate ceiling
         measured in the same run
  cpu_baseline   the CPU oracle of the emulated model (a port of the reference's emulated path) timed on this host
--impl reference times that CPU path alone, one frame per step.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

FRAME_H, FRAME_W, N_FRAMES, SIZE = 1440, 1900, 126, 640
METRIC = "ViT-L/16+EoMT frames/s"


def synth_video(n_frames: int, device, seed: int = 0) -> torch.Tensor:
    """uint8 [n, 1440, 1900, 3]: per frame a bilinearly upsampled seeded 6x8 grid (smooth content) + N(0, 8^2) noise."""
    g = torch.Generator(device=device).manual_seed(seed)
    out = torch.empty(n_frames, FRAME_H, FRAME_W, 3, dtype=torch.uint8, device=device)
    for i in range(n_frames):
        low = torch.rand(1, 3, 6, 8, generator=g, device=device) * 255.0
        img = torch.nn.functional.interpolate(low, size=(FRAME_H, FRAME_W), mode="bilinear", align_corners=False)[0]
        img = img + torch.randn(3, FRAME_H, FRAME_W, generator=g, device=device) * 8.0
        out[i] = img.clamp(0, 255).permute(1, 2, 0).to(torch.uint8)
    return out


class ClockSampler:
    QUERY = "clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown," \
            "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap"

    def __init__(self, index: int):
        self.index, self.rows, self.proc = index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "50"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm = [float(r[0]) for r in self.rows if len(r) >= 6 and r[0].replace(".", "").isdigit()]
        mx = [float(r[1]) for r in self.rows if len(r) >= 6 and r[1].replace(".", "").isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for k, n in enumerate(names) if any(len(r) >= 6 and r[2 + k].lower().startswith("active") for r in self.rows)]
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None, "reasons": reasons, "samples": len(sm)}


def block_gemm_flops(cfg, batch: int, size: int) -> float:
    """algorithmic FLOPs of the block GEMMs (qkv, proj, fc1, fc2) of one step: 2*M*N*K summed over the layers."""
    P = (size // 16) ** 2
    d, ff = cfg.dim, cfg.ffn
    per_tok = 2.0 * (d * 3 * d + d * d + d * ff + ff * d)
    first = cfg.depth - cfg.num_joint_blocks
    return batch * per_tok * (first * (P + 5) + cfg.num_joint_blocks * (P + 5 + cfg.num_queries))


def run_reference(args, rank: int):
    """the reference's CPU path (CPU oracle port of its emulated model), one frame per step, on the host cores."""
    if rank != 0:
        return
    from lightly_trian_quant_b200 import modeldef
    from oracle import model_oracle as mo

    torch.set_grad_enabled(False)
    torch.set_num_threads(max(1, os.cpu_count() or 1))      # rank 0 alone runs this arm (the other ranks exit): every host core
    fmt = args.variant.split("+")[0].split("_")[1]
    model = modeldef.build_model(modeldef.VIT_L, seed=0, mode="upstream", device="cpu")
    g = torch.Generator().manual_seed(0)
    emu = mo.EmuModel(model, fmt)
    frames = [torch.rand(1, 3, SIZE, SIZE, generator=g).to(torch.bfloat16).float() for _ in range(2)]
    for i in range(args.warmup):
        emu(frames[i % 2])
    t0 = time.perf_counter()
    for i in range(args.steps):
        emu(frames[i % 2])
    dt = time.perf_counter() - t0
    fps = args.steps / dt
    line = {"impl": "reference", "metric": METRIC, "value": fps, "unit": "frames/s", "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": dt / args.steps * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": fmt, "data": "synthetic",
            "config": {"workload": f"DINOv3 ViT-L/16 + EoMT (200 queries, 4 joint blocks), {fmt} linears, bf16 attention, 126-frame synthetic "
                                   f"1900x1440 uint8 video -> {SIZE}x{SIZE}, sharded by frame", "variant": args.variant,
                       "sample": "CPU emulated path on the host cores, one 640x640 frame per step (a bounded sample of the same workload)"},
            "cpu_baseline": {"value": fps, "unit": "frames/s", "cores": torch.get_num_threads(), "kind": "port",
                             "sample": "1 frame (640x640, whole model) per step; the reference's sm_120a extensions cannot run on the host, so its torch "
                                       "quantiser + dequantise-then-fp32-matmul emulation is timed through the CPU oracle port"},
            "e2e": {"value": fps, "unit": "frames/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}, "gpu_launches": 0}
    print(json.dumps(line), flush=True)


def cpu_baseline_sample(fmt: str) -> dict:
    from lightly_trian_quant_b200 import modeldef
    from oracle import model_oracle as mo

    model = modeldef.build_model(modeldef.VIT_L, seed=0, mode="upstream", device="cpu")
    emu = mo.EmuModel(model, fmt)
    x = torch.rand(1, 3, SIZE, SIZE, generator=torch.Generator().manual_seed(0)).to(torch.bfloat16).float()
    t0 = time.perf_counter()
    emu(x)                      # first frame: includes the one-off weight quantisation
    t1 = time.perf_counter()
    emu(x)
    t2 = time.perf_counter()
    return {"value": 1.0 / (t2 - t1), "unit": "frames/s", "cores": torch.get_num_threads(), "kind": "port",
            "sample": f"1 frame 640x640 through the CPU oracle of the emulated ViT-L/16+EoMT {fmt} model ({t2 - t1:.1f} s; the first frame incl. "
                      f"weight quantisation took {t1 - t0:.1f} s); host {os.cpu_count()} logical cores"}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--batch", type=int, default=14, help="frames per GPU per step")
    ap.add_argument("--variant", default="b200_nv4")
    ap.add_argument("--arch", default="vit_l", choices=["vit_l", "vit_b"], help="backbone of the other benchmark configurations (default: the headline ViT-L/16)")
    ap.add_argument("--size", type=int, default=SIZE, help="input side in pixels (default 640)")
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--pdl", action="store_true", help="launch the block kernels with programmatic dependent launch (default: plain stream order)")
    args = ap.parse_args()
    rank, world, local = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1)), int(os.environ.get("LOCAL_RANK", 0))
    if args.impl == "reference":
        run_reference(args, rank)
        return
    if args.warmup < 3:
        args.warmup = 3
    torch.set_grad_enabled(False)
    torch.set_num_threads(max(1, (os.cpu_count() or 1) // max(1, world)))      # host threads are shared by the ranks of one box
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist = None
    if world > 1:
        import torch.distributed as dist_mod

        dist = dist_mod
        dist.init_process_group("nccl", device_id=dev)

    from lightly_trian_quant_b200 import modeldef, ops, sharding, stack

    ops.set_pdl(args.pdl)
    cfg = modeldef.VIT_L if args.arch == "vit_l" else modeldef.VIT_B
    size = args.size
    if size != SIZE and "+s" not in args.variant:
        args.variant += f"+s{size}"
    fmt = args.variant.split("+")[0].split("_")[1]
    model = modeldef.build_model(cfg, seed=0, mode="upstream", device=dev)
    model_fn, pipe_cls = stack.make_variant(args.arch, model, args.variant)
    pipe = pipe_cls(model, model_fn, size)
    B = args.batch

    # this rank's shard of the video: frames rank, rank+world, ...; grouped into micro-batches of B (cyclic)
    shard = sharding.shard_frames(N_FRAMES, rank, world)
    batches = sharding.micro_batches(shard, B, min_batches=2)
    n_batches = len(batches)
    video = synth_video(N_FRAMES, dev)
    dev_batches = [video[idx].contiguous() for idx in batches]
    host_batches = [b.cpu().pin_memory() for b in dev_batches]
    host_frames = {k: video[k].cpu() for k in shard}
    del video

    # the public host pipeline: warm-up = eager calibration call (static NVFP4 scales from the first batch) + one graph per slot
    from lightly_trian_quant_b200 import pipeline as host_pipeline

    vp = host_pipeline.VideoPipeline(pipe, B, FRAME_H, FRAME_W, slots=3, inflight=2, device=dev)
    vp.warmup(dev_batches[0])
    ops.check_device_error()
    nslots = len(vp.slots)

    def barrier():
        torch.cuda.synchronize()
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    def reduce_max(ms: float) -> float:
        if dist is None:
            return ms
        t = torch.tensor([ms], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    # ---------------------------------------------------------------- device-resident steps (graph replay, inputs in HBM)
    def dev_step(i):
        slot = vp.slots[i % nslots]
        slot.dev_in.copy_(dev_batches[i % n_batches], non_blocking=True)     # device-to-device: a different batch every step
        slot.graph.replay()

    with torch.cuda.stream(vp.comp):
        for i in range(args.warmup):
            dev_step(i)
    barrier()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with torch.cuda.stream(vp.comp):
        e0.record()
        for i in range(args.steps):
            dev_step(args.warmup + i)
        e1.record()
    barrier()
    ms_total = reduce_max(e0.elapsed_time(e1))
    clocks = sampler.stop() if rank == 0 else None
    fps = sharding.aggregate_fps(B, world, args.steps, ms_total)

    # ---------------------------------------------------------------- end to end with host frames through VideoPipeline.submit
    def e2e_run(n_steps, start):
        for i in range(n_steps):
            vp.submit(i % nslots, src=host_batches[(start + i) % n_batches])

    e2e_run(args.warmup, 0)
    barrier()
    s0, s1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s0.record(vp.h2d)                                   # the first copy of the timed region is enqueued behind it
    e2e_run(args.steps, args.warmup)
    vp.d2h.wait_stream(vp.comp)
    s1.record(vp.d2h)                                   # behind the last device -> host copy
    barrier()
    e2e_ms = reduce_max(s0.elapsed_time(s1))
    e2e_fps = sharding.aggregate_fps(B, world, args.steps, e2e_ms)
    h2d, d2h = vp.slots[0].dev_in.numel(), vp.slots[0].pinned_out.numel()

    # ---------------------------------------------------------------- the 126-frame video once, sharded, tail batch included
    uniq = [shard[j:j + B] for j in range(0, len(shard), B)]
    video_batches = []
    for idx in uniq:
        pad = idx + [idx[-1]] * (B - len(idx))
        video_batches.append((torch.stack([host_frames[k] for k in pad]).pin_memory(), len(idx)))
    barrier()
    t0 = time.perf_counter()
    vstats = vp.run(iter(video_batches)) if video_batches else {"frames": 0, "batches": 0}
    torch.cuda.synchronize()
    v_ms = reduce_max((time.perf_counter() - t0) * 1e3)
    v_frames = vstats["frames"]
    if dist is not None:
        tf = torch.tensor([v_frames], device=dev, dtype=torch.float64)
        dist.all_reduce(tf)
        v_frames = int(tf.item())
    video_126 = {"frames": v_frames, "seconds": v_ms * 1e-3, "frames_per_s": v_frames / (v_ms * 1e-3), "scaling": "strong",
                 "frames_on_rank0": len(shard), "batches_on_rank0": len(uniq),
                 "note": "host wall clock around VideoPipeline.run of each rank's shard (pinned frames in, labels out), slowest rank; the last micro-batch is padded to the static batch"}

    # ---------------------------------------------------------------- per-kernel-class timing (instrumented eager pass)
    kern = None
    roof = None
    if rank == 0:
        ops.TIMING, ops.BYTES = {}, {}
        ops.LAUNCHES = 0
        pipe(dev_batches[1 % n_batches])
        torch.cuda.synchronize()
        launches_per_step = ops.LAUNCHES
        classes = {}
        for name, evs in ops.TIMING.items():
            classes[name] = {"launches": len(evs), "ms": sum(a.elapsed_time(b) for a, b in evs)}
        ops.TIMING = None
        total_ms = sum(c["ms"] for c in classes.values())
        for c in classes.values():
            c["share"] = c["ms"] / total_ms
        kern = {k: {"launches": v["launches"], "ms": round(v["ms"], 4), "share": round(v["share"], 4)} for k, v in sorted(classes.items(), key=lambda kv: -kv[1]["ms"])}
        peaks = json.loads((ROOT / "MEASURED_PEAKS.json").read_text()) if (ROOT / "MEASURED_PEAKS.json").exists() else None
        gname = "gemm_block_" + fmt
        if gname in classes:
            flops = block_gemm_flops(cfg, B, size)
            achieved = flops / (classes[gname]["ms"] * 1e-3) / 1e12
            peak = ops.tensor_peak_tflops(fmt, 256)
            nominal = {"nv4": 9000.0, "mx4": 9000.0, "mx8": 4500.0, "bf16": 2250.0}[fmt]
            # DRAM bytes per launch of the dominant kernel: a profiled figure per token row, kept as data beside the profile
            # summaries, times the mean rows per launch of this run; None when this configuration has not been profiled
            rows_mean = B * ((cfg.depth - cfg.num_joint_blocks) * (5 + (size // 16) ** 2) + cfg.num_joint_blocks * (5 + (size // 16) ** 2 + cfg.num_queries)) / cfg.depth
            traffic = None
            tfile = ROOT / "profiles" / "dram_traffic.json"
            if tfile.exists():
                per_row = json.loads(tfile.read_text()).get(f"gemm_block_{fmt}_{args.arch}", {}).get("dram_bytes_per_row_per_launch")
                traffic = per_row * rows_mean if per_row else None
            roof = {"bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s", "frac": achieved / peak, "traffic": traffic,
                    "kernel": f"gemm_kernel<{fmt}> (qkv, proj, fc1, fc2 of all blocks; {classes[gname]['launches']} launches per step)",
                    "peak_source": f"tcgen05 {fmt} instruction-rate probe (M=128, N=256 as in the kernel, shared-memory-resident operands) measured in this run; "
                                   f"MEASURED_PEAKS.json has no {fmt} figure (bf16 burst {peaks['bf16_tflops'] if peaks else 'n/a'} TFLOP/s of measured); "
                                   f"nominal dense {nominal:.0f}",
                    "frac_of_nominal": achieved / nominal}
        hbm = peaks["hbm_gbs"] if peaks else 6650.0
        for qn in ("ln_quant", "quant_rows"):
            if qn in classes and qn in ops.BYTES:
                kern[qn]["GB/s"] = round(ops.BYTES[qn] / (classes[qn]["ms"] * 1e-3) / 1e9, 1)
                kern[qn]["frac_hbm"] = round(kern[qn]["GB/s"] / hbm, 3)
        kern["_hbm_peak"] = f"{hbm} GB/s ({'of measured' if peaks else 'of fallback'})"
    ops.check_device_error()

    if rank == 0:
        arch_name = "ViT-L/16" if args.arch == "vit_l" else "ViT-B/16"
        line = {"metric": METRIC if args.arch == "vit_l" else "ViT-B/16+EoMT frames/s", "value": fps, "unit": "frames/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
                "ms_per_step": ms_total / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
                "dtype": {"nv4": "nvfp4 (e2m1, ue4m3 per 16, fp32 accumulate)", "mx4": "mxfp4", "mx8": "mxfp8 (e4m3, ue8m0 per 32, fp32 accumulate)", "bf16": "bf16"}[fmt],
                "data": "synthetic",
                "config": {"workload": f"DINOv3 {arch_name} + EoMT (200 queries, 4 joint blocks), {fmt} linears, {'f16' if 'f16attn' in args.variant else 'bf16'} attention, "
                                       f"126-frame synthetic 1900x1440 uint8 video -> {size}x{size}, sharded by frame", "variant": args.variant, "frames_per_gpu_per_step": B,
                           "parallelism": f"dp{world} (replicated weights, no collective)", "l2": "inputs larger than L2: a different frame batch every step"},
                "clocks": clocks,
                "e2e": {"value": e2e_fps, "unit": "frames/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
                "gpu_launches": launches_per_step * args.steps, "roofline": roof, "kernels": kern, "video_126": video_126}
        if not args.no_cpu_baseline and world == 1:
            line["cpu_baseline"] = cpu_baseline_sample(fmt)
        print(json.dumps(line), flush=True)
    if dist is not None:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
