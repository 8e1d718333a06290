"""Host-side logic of the multi-GPU path, on CPU: two gloo ranks shard a batch, run the
forward on their slices (the CPU checker stands in for the GPU here), and rank 0's
gathered result must equal the unsharded forward bit for bit; timing is the maximum over
ranks."""
import os
import sys

import numpy as np
import pytest
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

from darknet_b200.shard import shard_batch  # noqa: E402


def test_shard_batch_covers_every_image_once():
    for total in (0, 1, 7, 8, 64, 65):
        for world in (1, 2, 3, 4, 8):
            spans = [shard_batch(total, world, r) for r in range(world)]
            assert sum(c for _, c in spans) == total
            pos = 0
            for start, count in spans:
                assert start == pos and count >= 0
                pos += count
            counts = [c for _, c in spans]
            assert max(counts) - min(counts) <= 1
    assert [shard_batch(64, 8, r) for r in (0, 7)] == [(0, 8), (56, 8)]
    with pytest.raises(ValueError):
        shard_batch(8, 2, 2)


def _worker(rank, world, port, q):
    sys.path.insert(0, ROOT)
    import torch.distributed as dist
    from darknet_b200 import synth
    from darknet_b200.shard import gather_outputs, max_over_ranks, shard_batch
    from oracle import network as orc
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    total = 3
    cfg = synth.yolov3_tiny_cfg(batch=total, size=64)
    params = synth.seeded_params(cfg, 5)
    x = synth.seeded_input(cfg, 5)
    start, count = shard_batch(total, world, rank)
    local = orc.forward_network(cfg, params, x[start:start + count])[-1] if count else np.zeros((0,), np.float32)
    whole = gather_outputs(local, total)
    slowest = max_over_ranks(10.0 + rank)
    if rank == 0:
        full = orc.forward_network(cfg, params, x)[-1]
        q.put((bool(np.array_equal(whole, full)), slowest))
    else:
        assert whole is None
    dist.barrier()
    dist.destroy_process_group()


def test_two_ranks_shard_and_gather():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29000 + os.getpid() % 2000
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    same, slowest = q.get(timeout=120)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert same, "sharded forward differs from the unsharded one"
    assert slowest == 11.0


def test_cpus_near_gpu_decodes_the_affinity_mask():
    from darknet_b200.shard import cpus_near_gpu
    # CPUs 0-3 and 64-65 of a 128-CPU host
    assert cpus_near_gpu(0, affinity_words=[0b1111, 0b11], ncpu=128) == [0, 1, 2, 3, 64, 65]
    # CPUs beyond the host's count are dropped
    assert cpus_near_gpu(0, affinity_words=[0b1111, 0b11], ncpu=3) == [0, 1, 2]
    # without NVML (no GPU here) the query degrades to "unknown"
    assert isinstance(cpus_near_gpu(0), list)
