"""Data-parallel logic on CPU (gloo, world size 2 and 3): sharding, bucket planning and the
gradient arithmetic the GPU path relies on — each rank's cross-entropy divides by the GLOBAL
batch, the all-reduced SUM of shard gradients equals the single-process full-batch gradient
(the reference divides by the batch it sees, src/nn/loss.rs:100; it has no distributed code).
The ranks run the CPU oracle; the collective is torch.distributed over gloo on 127.0.0.1."""
import os
import socket
import sys
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parent.parent


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _rank_main(rank, world, port, out_dir):
    sys.path.insert(0, str(ROOT))
    os.environ["OMP_NUM_THREADS"] = "2"
    import torch
    import torch.distributed as dist
    from neuralrs_b200 import cuda
    from oracle import models
    from oracle.nrs_oracle import Oracle
    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
    o = Oracle("f64")
    cfg = models.SMALL_CNN
    global_batch = 10                      # not divisible by 3: uneven shards
    params = models.he_init(cfg["layers"], 99)            # identical bytes on every rank
    x, t = models.synthetic_batch(cfg, global_batch, 100, uniform01=True)
    b0, b1 = cuda.dp_shard_range(global_batch, rank, world)
    loss, grads, _ = models.forward_backward(o, cfg["layers"], params, x[b0:b1], t[b0:b1], divisor=global_batch)
    # flat gradient in parameter order, padded like the library's flat store (multiples of 4 floats)
    lens = [g.size for g in grads]
    offs = np.cumsum([0] + [(n + 3) // 4 * 4 for n in lens])
    flat = np.zeros(offs[-1], np.float32)
    for g, off in zip(grads, offs):
        flat[off:off + g.size] = g.ravel()
    buckets = cuda.dp_plan_buckets(lens, 64 * 1024)
    ft = torch.from_numpy(flat)
    for s, e in buckets:                   # one all-reduce per bucket, last bucket of the model first
        dist.all_reduce(ft[s:e], op=dist.ReduceOp.SUM)
    lt = torch.tensor([loss], dtype=torch.float64)
    dist.all_reduce(lt, op=dist.ReduceOp.SUM)
    if rank == 0:
        np.save(os.path.join(out_dir, "flat.npy"), flat)
        np.save(os.path.join(out_dir, "loss.npy"), lt.numpy())
        np.save(os.path.join(out_dir, "buckets.npy"), np.array(buckets))
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 3])
def test_sharded_gradients_sum_to_full_batch(world, tmp_path, nrs_lib):
    import torch.multiprocessing as mp
    port = _free_port()
    mp.spawn(_rank_main, args=(world, port, str(tmp_path)), nprocs=world, join=True)
    from oracle import models
    from oracle.nrs_oracle import Oracle
    o = Oracle("f64")
    cfg = models.SMALL_CNN
    params = models.he_init(cfg["layers"], 99)
    x, t = models.synthetic_batch(cfg, 10, 100, uniform01=True)
    loss, grads, _ = models.forward_backward(o, cfg["layers"], params, x, t)
    flat = np.load(tmp_path / "flat.npy")
    offs = np.cumsum([0] + [(g.size + 3) // 4 * 4 for g in grads])
    for g, off in zip(grads, offs):
        got = flat[off:off + g.size]
        assert np.linalg.norm(got - g.ravel()) <= 1e-5 * np.linalg.norm(g) + 1e-12
    assert abs(float(np.load(tmp_path / "loss.npy")[0]) - loss) <= 1e-6 * max(1.0, abs(loss))
    buckets = np.load(tmp_path / "buckets.npy")
    # buckets tile the flat gradient exactly, ordered from the END (the order backward finishes them)
    assert buckets[0][1] == offs[-1] and buckets[-1][0] == 0
    for (s0, e0), (s1, e1) in zip(buckets[:-1], buckets[1:]):
        assert e1 == s0 and s0 < e0


def test_shard_ranges_and_bucket_plan(nrs_lib):
    from neuralrs_b200 import cuda
    for gb, world in [(1024, 8), (10, 4), (7, 8), (0, 2), (1, 1)]:
        ranges = [cuda.dp_shard_range(gb, r, world) for r in range(world)]
        assert ranges[0][0] == 0 and ranges[-1][1] == gb
        for (a0, a1), (b0, b1) in zip(ranges[:-1], ranges[1:]):
            assert a1 == b0 and 0 <= a1 - a0 - (b1 - b0) <= 1          # contiguous, sizes differ by at most one
    lens = [27 * 64, 64, 64 * 64 * 9, 64, 4096 * 512, 512, 5120, 10]
    one = cuda.dp_plan_buckets(lens, 1 << 40)
    assert len(one) == 1 and one[0][0] == 0
    many = cuda.dp_plan_buckets(lens, 4)
    assert len(many) == len(lens)                                      # every tensor its own bucket
    with pytest.raises(Exception):
        cuda.dp_shard_range(8, 3, 2)
