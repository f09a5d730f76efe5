"""Frame sharding of the data-parallel video path: frames are independent units (no cross-frame state; the reference
processes them one by one, infer-opt/round9_integration/video_infer.py:195-320), so rank r of W takes frames
r, r + W, r + 2W, ... with replicated weights and no collective on the data path."""
from __future__ import annotations

from typing import List


def shard_frames(n_frames: int, rank: int, world: int) -> List[int]:
    if not (0 <= rank < world):
        raise ValueError(f"rank {rank} outside world {world}")
    return list(range(rank, n_frames, world))


def micro_batches(shard: List[int], batch: int, min_batches: int = 1) -> List[List[int]]:
    """groups a shard into micro-batches of exactly `batch` frame indices; the last batch wraps around (cyclic) so every
    batch has the static shape a captured CUDA graph needs.  Empty shards give no batches."""
    if batch <= 0:
        raise ValueError("batch must be positive")
    if not shard:
        return []
    n = max(min_batches, -(-len(shard) // batch))
    return [[shard[(j * batch + i) % len(shard)] for i in range(batch)] for j in range(n)]


def aggregate_fps(frames_per_rank_step: int, world: int, steps: int, max_ms_over_ranks: float) -> float:
    """whole-job frames/s = frames all ranks processed / the slowest rank's device time."""
    return world * frames_per_rank_step * steps / (max_ms_over_ranks * 1e-3)
