"""GPU test of the host-side frame pipeline (pinned ring, copy / compute streams, one captured graph per slot): labels from
HOST frames equal the labels of the device-resident path bit for bit, in frame order, including a padded tail batch."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
torch.set_grad_enabled(False)

TINY = dict(dim=256, depth=4, heads=4, ffn=1024, num_queries=32, num_joint_blocks=2)


def _setup(fmt):
    from lightly_trian_quant_b200 import modeldef, pipeline, stack

    cfg = modeldef.EoMTConfig(**TINY)
    model = modeldef.build_model(cfg, 0, "stress", "cuda")
    fn, pipe_cls = stack.make_variant("tiny", model, f"b200_{fmt}+s64")
    return pipeline, pipe_cls(model, fn, 64)


@pytest.mark.parametrize("fmt", ["nv4", "mx8"])
def test_host_frames_give_the_device_path_labels(fmt):
    pipeline, frame_fn = _setup(fmt)
    B, H, W, n = 3, 90, 120, 8
    g = torch.Generator().manual_seed(3)
    frames = torch.randint(0, 256, (n, H, W, 3), generator=g, dtype=torch.uint8)
    vp = pipeline.VideoPipeline(frame_fn, B, H, W, slots=3, inflight=2)
    first = vp.warmup(frames[:B])                       # calibrates the static scales on the first batch
    # device-resident reference: the same micro-batches (tail padded with its last frame), after calibration
    ref = []
    for i in range(0, n, B):
        chunk = frames[i:i + B]
        if chunk.shape[0] < B:
            chunk = torch.cat([chunk, chunk[-1:].expand(B - chunk.shape[0], -1, -1, -1)])
        ref.append(frame_fn(chunk.cuda()).cpu()[: min(B, n - i)])
    ref = torch.cat(ref).numpy()
    assert np.array_equal(first.cpu().numpy(), ref[:B])
    got = {}

    def consumer(idx, labels):
        got[idx] = labels.copy()

    stats = vp.run((frames[i].numpy() for i in range(n)), consumer)
    assert stats["frames"] == n and stats["batches"] == 3
    assert sorted(got) == list(range(n))
    for i in range(n):
        assert np.array_equal(got[i], ref[i]), i
    # a second pass reuses the slots and graphs; whole pinned batches are read in place
    pinned = [frames[i:i + B].clone().pin_memory() for i in (0, 3)]
    got.clear()
    stats = vp.run(iter(pinned), consumer)
    assert stats["frames"] == 6
    for i in range(6):
        assert np.array_equal(got[i], ref[i]), i


def test_pipeline_rejects_use_before_warmup_and_bad_shapes():
    from lightly_trian_quant_b200._lib import KfError

    pipeline, frame_fn = _setup("mx8")
    vp = pipeline.VideoPipeline(frame_fn, 2, 64, 64)
    with pytest.raises(KfError):
        vp.run(iter([]))
    with pytest.raises(KfError):
        vp.warmup(torch.zeros(1, 64, 64, 3, dtype=torch.uint8))
    with pytest.raises(ValueError):
        pipeline.VideoPipeline(frame_fn, 2, 64, 64, slots=1, inflight=2)
