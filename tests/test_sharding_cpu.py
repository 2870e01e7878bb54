"""Multi-rank host logic on CPU (gloo, world_size 2): batch shards partition the global batch,
each rank's shard of a network forward equals the same rows of the single-rank result, and the
throughput aggregation takes the max time and the sum of images."""
import importlib
import os
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from helpers import ROOT

sys.path.insert(0, os.path.join(ROOT, "paddle-lite_b200"))
S = importlib.import_module("paddle-lite_b200.sharding")


def test_shards_partition_the_batch():
    for batch, world in [(1024, 8), (256, 8), (10, 4), (3, 4), (128, 1)]:
        edges = [S.shard_slice(batch, r, world) for r in range(world)]
        assert edges[0][0] == 0 and edges[-1][1] == batch
        for a, b in zip(edges, edges[1:]):
            assert a[1] == b[0]
        sizes = [e[1] - e[0] for e in edges]
        assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        S.shard_slice(8, 4, 4)


def _worker(rank, world, port, out):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import net_oracle
    N = importlib.import_module("paddle-lite_b200.networks")
    spec = dict(name="tiny", image=(3, 32, 32), ops=[
        dict(op="conv", name="conv1", src="x", dst="c1", cin=3, cout=16, k=3, s=2, p=1, act=1, out="i8"),
        dict(op="conv", name="dw", src="c1", dst="d1", cin=16, cout=16, k=3, s=1, p=1, groups=16, act=1, out="i8"),
        dict(op="conv", name="pw", src="d1", dst="p1", cin=16, cout=32, k=1, s=1, p=0, act=1, out="f32"),
        dict(op="avgpool_calib", name="pool", src="p1", dst="feat", c=32),
        dict(op="fc", name="fc", src="feat", dst="logits", k=32, n=10)])
    qnet = N.build_quantized(spec, seed=5, calib_images=4, device="cpu")  # same seed on every rank
    images = np.random.default_rng(11).standard_normal((6, 3, 32, 32)).astype(np.float32)
    lo, hi = S.shard_slice(6, rank, world)
    local = net_oracle.forward(qnet, images[lo:hi])["logits"]
    full = net_oracle.forward(qnet, images)["logits"]
    ok = np.array_equal(local, full[lo:hi])
    value, ms = S.aggregate_throughput(hi - lo, 10.0 * (rank + 1))
    out[rank] = (ok, value, ms, lo, hi)
    dist.destroy_process_group()


def test_two_ranks_gloo():
    world = 2
    port = 29500 + os.getpid() % 1000
    mgr = mp.Manager()
    out = mgr.dict()
    mp.spawn(_worker, args=(world, port, out), nprocs=world, join=True)
    assert set(out.keys()) == {0, 1}
    for rank in range(world):
        ok, value, ms, lo, hi = out[rank]
        assert ok, "rank %d: shard result differs from the rows of the full batch" % rank
        assert ms == 20.0                      # max over ranks
        assert abs(value - 6 / 0.020) < 1e-6   # all images / slowest rank
    assert out[0][3:] == (0, 3) and out[1][3:] == (3, 6)
