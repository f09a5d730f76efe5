"""Host side of the frame path: pinned ring -> H2D -> [one CUDA graph: resize + normalise + model_fn + per-pixel labels] ->
D2H -> consumer, micro-batched, with copies and compute on separate streams so that they overlap.

Behaviour of the reference's VideoPipeline (infer-opt/round9_integration/video_infer.py:87-320): a ring of pinned input /
output slots, an H2D, a compute and a D2H stream chained by events, one captured graph per slot, a bounded number of
slots in flight, a thread that waits for finished slots and hands results to a consumer in frame order.  What differs:
a slot holds a micro-batch of B frames (the reference processes one frame per slot and lists multi-frame batching as
not built, infer-opt/round14_fp4_full/NOTES.md:145), frames come from any iterable of host arrays instead of cv2, and the
result is the uint8 label map at mask resolution.

    pipe = VideoPipeline(frame_fn, batch=14, height=1440, width=1900)       # frame_fn: stack.FramePipeline instance
    pipe.warmup(first_batch)                                                # eager calibration call + graph capture
    stats = pipe.run(frames, consumer)                                      # consumer(frame_index, labels_hw_uint8_numpy)

Frames are independent units, so several processes (one per GPU) each run their own VideoPipeline over their shard of the
frame indices (sharding.shard_frames); nothing is exchanged between them.
"""
from __future__ import annotations

import queue
import threading
import time
from typing import Callable, Iterable, Optional

import torch

from . import ops
from ._lib import KfError


class _Slot:
    """buffers and events of one ring slot (a micro-batch)."""

    def __init__(self, batch, height, width, device):
        self.pinned_in = torch.empty(batch, height, width, 3, dtype=torch.uint8).pin_memory()
        self.dev_in = torch.empty(batch, height, width, 3, dtype=torch.uint8, device=device)
        self.dev_out: Optional[torch.Tensor] = None       # allocated at warm-up, when the label shape is known
        self.pinned_out: Optional[torch.Tensor] = None
        self.ev_h2d, self.ev_comp, self.ev_d2h = torch.cuda.Event(), torch.cuda.Event(), torch.cuda.Event()
        self.graph = None
        self.src = None                                    # pinned tensor the next H2D reads (the slot's own or the caller's)


class VideoPipeline:
    def __init__(self, frame_fn: Callable[[torch.Tensor], torch.Tensor], batch: int, height: int, width: int, *, slots: int = 3,
                 inflight: int = 2, use_graph: bool = True, device="cuda"):
        if batch < 1 or slots < 1 or inflight < 1:
            raise ValueError("batch, slots and inflight must be positive")
        if inflight > slots:
            raise ValueError("inflight cannot exceed the number of slots")
        self.frame_fn, self.B, self.H, self.W = frame_fn, batch, height, width
        self.device = torch.device(device)
        self.use_graph = use_graph
        self.inflight = inflight
        self.slots = [_Slot(batch, height, width, self.device) for _ in range(slots)]
        self.h2d, self.comp, self.d2h = torch.cuda.Stream(self.device), torch.cuda.Stream(self.device), torch.cuda.Stream(self.device)
        self.ready = False

    # ------------------------------------------------------------------ warm-up: calibration + capture
    @torch.no_grad()
    def warmup(self, first_batch: torch.Tensor) -> torch.Tensor:
        """first_batch uint8 [B, H, W, 3] (host or device).  Runs frame_fn eagerly (the first call measures the static NVFP4
        activation scales, so it must see real frames), then captures one graph per slot.  Returns the labels of the batch."""
        if tuple(first_batch.shape) != (self.B, self.H, self.W, 3) or first_batch.dtype != torch.uint8:
            raise KfError(f"warmup: expected uint8 [{self.B}, {self.H}, {self.W}, 3], got {tuple(first_batch.shape)} {first_batch.dtype}")
        self.comp.wait_stream(torch.cuda.current_stream(self.device))
        with torch.cuda.stream(self.comp):
            for s in self.slots:
                s.dev_in.copy_(first_batch, non_blocking=False)
            labels = self.frame_fn(self.slots[0].dev_in)
            for _ in range(2):
                labels = self.frame_fn(self.slots[0].dev_in)
            for s in self.slots:
                s.dev_out = torch.empty_like(labels)
                s.pinned_out = torch.empty(labels.shape, dtype=labels.dtype).pin_memory()
        self.comp.synchronize()
        ops.check_device_error()
        if self.use_graph:
            pool = None
            for s in self.slots:
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g, pool=pool, stream=self.comp):
                    s.dev_out.copy_(self.frame_fn(s.dev_in))
                pool = g.pool() if pool is None else pool
                s.graph = g
            torch.cuda.synchronize(self.device)
        self.ready = True
        return labels.clone()

    # ------------------------------------------------------------------ one micro-batch
    @torch.no_grad()
    def submit(self, k: int, src: Optional[torch.Tensor] = None) -> None:
        """Enqueue H2D -> graph -> D2H for slot k.  src: a pinned uint8 [B, H, W, 3] tensor to read instead of the slot's own
        pinned buffer (frames that already sit in pinned memory need no extra host copy).  Returns at once; wait on
        slots[k].ev_d2h (or use run()) before reading slots[k].pinned_out."""
        if not self.ready:
            raise KfError("VideoPipeline.submit before warmup()")
        s = self.slots[k]
        host = s.pinned_in if src is None else src
        if src is not None and (not src.is_pinned() or tuple(src.shape) != tuple(s.pinned_in.shape) or src.dtype != torch.uint8):
            raise KfError("submit: src must be a pinned uint8 tensor of the slot's shape")
        with torch.cuda.stream(self.h2d):
            self.h2d.wait_event(s.ev_comp)                  # the slot's previous compute has consumed dev_in
            s.dev_in.copy_(host, non_blocking=True)
            s.ev_h2d.record(self.h2d)
        with torch.cuda.stream(self.comp):
            self.comp.wait_event(s.ev_h2d)
            self.comp.wait_event(s.ev_d2h)                  # the slot's previous labels have left dev_out
            if s.graph is not None:
                s.graph.replay()
            else:
                s.dev_out.copy_(self.frame_fn(s.dev_in))
            s.ev_comp.record(self.comp)
        with torch.cuda.stream(self.d2h):
            self.d2h.wait_event(s.ev_comp)
            s.pinned_out.copy_(s.dev_out, non_blocking=True)
            s.ev_d2h.record(self.d2h)

    # ------------------------------------------------------------------ streaming driver
    def run(self, source: Iterable, consumer: Optional[Callable] = None) -> dict:
        """source yields uint8 host frames [H, W, 3] (numpy or torch; copied into the ring), whole pinned batches
        [B, H, W, 3] (read in place) or (pinned batch, valid) pairs for a batch of which only the first `valid` frames count.
        consumer(frame_index, labels) is called in frame order from the result thread with a numpy view [h, w] of the slot's
        pinned output; it must copy what it keeps.  A last, partial batch is padded with
        its final frame; padded frames are not reported.  Returns {"frames", "batches", "t_total", "lat_ms"}."""
        if not self.ready:
            raise KfError("VideoPipeline.run before warmup()")
        nslots = len(self.slots)
        free: "queue.Queue[int]" = queue.Queue()
        for k in range(nslots):
            free.put(k)
        filled: "queue.Queue" = queue.Queue()
        pending: "queue.Queue" = queue.Queue()
        gate = threading.Semaphore(self.inflight)
        failed: list = []
        stop = threading.Event()
        lat_ms: list = []

        def take_slot():
            while not stop.is_set():
                try:
                    return free.get(timeout=0.1)
                except queue.Empty:
                    continue
            return None

        def feed():
            try:
                idx, k, fill = 0, None, 0
                for item in source:
                    if stop.is_set():
                        break
                    valid = self.B
                    if isinstance(item, tuple):
                        item, valid = item
                    t = torch.as_tensor(item)
                    if t.dim() == 4:                       # a whole batch that already sits in pinned memory
                        if fill:
                            raise KfError("run: a batch arrived while a slot was partly filled with single frames")
                        k = take_slot()
                        if k is None:
                            break
                        self.slots[k].src = t
                        filled.put((k, idx, valid, time.perf_counter()))
                        idx += valid
                        k = None
                        continue
                    if k is None:
                        k = take_slot()
                        if k is None:
                            break
                        self.slots[k].src = None
                        t_in = time.perf_counter()
                    self.slots[k].pinned_in[fill].copy_(t)
                    fill += 1
                    if fill == self.B:
                        filled.put((k, idx, self.B, t_in))
                        idx += self.B
                        k, fill = None, 0
                if k is not None and fill and not stop.is_set():   # tail: pad with the last frame
                    buf = self.slots[k].pinned_in
                    for j in range(fill, self.B):
                        buf[j].copy_(buf[fill - 1])
                    filled.put((k, idx, fill, t_in))
            except Exception as e:  # noqa: BLE001
                failed.append(e)
                stop.set()
            finally:
                filled.put(None)

        def collect():
            try:
                while True:
                    item = pending.get()
                    if item is None:
                        return
                    k, first, valid, t_in = item
                    s = self.slots[k]
                    s.ev_d2h.synchronize()
                    gate.release()
                    lat_ms.append((time.perf_counter() - t_in) * 1e3)
                    if consumer is not None and not stop.is_set():
                        out = s.pinned_out.numpy()
                        for j in range(valid):
                            consumer(first + j, out[j])
                    free.put(k)
            except Exception as e:  # noqa: BLE001
                failed.append(e)
                stop.set()
                while True:                                 # drain so that the submitting thread cannot block
                    item = pending.get()
                    if item is None:
                        return
                    gate.release()
                    free.put(item[0])

        tf, tc = threading.Thread(target=feed, daemon=True), threading.Thread(target=collect, daemon=True)
        tf.start()
        tc.start()
        t0 = time.perf_counter()
        frames = batches = 0
        try:
            while True:
                item = filled.get()
                if item is None:
                    break
                k, first, valid, t_in = item
                if stop.is_set():
                    free.put(k)
                    continue
                gate.acquire()
                try:
                    self.submit(k, self.slots[k].src)
                except Exception:
                    gate.release()
                    free.put(k)
                    raise
                pending.put((k, first, valid, t_in))
                frames += valid
                batches += 1
        except Exception as e:  # noqa: BLE001
            failed.append(e)
            stop.set()
        finally:
            pending.put(None)
            tc.join()
            tf.join()
        if failed:
            raise failed[0]
        torch.cuda.synchronize(self.device)
        ops.check_device_error()                            # a bounded device wait that ran out would otherwise go unnoticed under graph replay
        return {"frames": frames, "batches": batches, "t_total": time.perf_counter() - t0, "lat_ms": lat_ms}
