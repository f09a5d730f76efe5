"""N>1 host logic on CPU: two gloo ranks shard the video, every frame is covered exactly once, and the timing
aggregation takes the maximum over ranks (the GPU data path itself has no collective)."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from lightly_trian_quant_b200 import sharding


def test_shard_and_batches_single_process():
    all_frames = sorted(f for r in range(8) for f in sharding.shard_frames(126, r, 8))
    assert all_frames == list(range(126))
    assert [len(sharding.shard_frames(126, r, 8)) for r in range(8)] == [16] * 6 + [15] * 2
    b = sharding.micro_batches(sharding.shard_frames(126, 0, 1), 14, min_batches=2)
    assert len(b) == 9 and all(len(x) == 14 for x in b) and sorted(sum(b, [])) == list(range(126))
    b = sharding.micro_batches(sharding.shard_frames(126, 7, 8), 14, min_batches=2)      # 15 frames -> 2 batches, cyclic tail
    assert len(b) == 2 and set(sum(b, [])) == set(range(7, 126, 8))
    assert sharding.micro_batches([], 4) == []
    with pytest.raises(ValueError):
        sharding.shard_frames(10, 3, 2)
    assert sharding.aggregate_fps(14, 2, 10, 100.0) == pytest.approx(2800.0)


def _worker(rank, world, port, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    shard = sharding.shard_frames(126, rank, world)
    mine = torch.zeros(126, dtype=torch.int64)
    mine[shard] = 1
    dist.all_reduce(mine)                                   # test-only collective: coverage check
    ms = torch.tensor([10.0 + 5.0 * rank], dtype=torch.float64)
    dist.all_reduce(ms, op=dist.ReduceOp.MAX)               # the bench's max-over-ranks timing
    ret[rank] = (bool((mine == 1).all()), float(ms.item()), len(sharding.micro_batches(shard, 14, 2)))
    dist.destroy_process_group()


def test_two_ranks_gloo():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    ctx = mp.get_context("spawn")
    ret = ctx.Manager().dict()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, ret)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
        assert p.exitcode == 0
    assert ret[0] == (True, 15.0, 5) and ret[1] == (True, 15.0, 5)
