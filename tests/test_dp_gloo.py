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


def _bn_rank(rank, world, port, out_dir):
    """Batch normalisation with statistics shared across ranks, as the device library does it: per-channel sums
    around a pivot every rank has (the running mean), summed across ranks together with the element count;
    backward sums of g and g*xhat likewise before dx, the parameter gradients summed like any other gradient."""
    sys.path.insert(0, str(ROOT))
    import torch
    import torch.distributed as dist
    from neuralrs_b200 import cuda
    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
    rng = np.random.default_rng(7)                          # identical data on every rank; each keeps its shard
    n, c, h, w = 11, 6, 5, 4
    x = (rng.normal(size=(n, c, h, w)) * 2 + np.arange(c)[None, :, None, None]).astype(np.float32)
    g = rng.normal(size=(n, c, h, w)).astype(np.float32)
    gamma, beta = rng.normal(size=c).astype(np.float32), rng.normal(size=c).astype(np.float32)
    running_mean = rng.normal(size=c).astype(np.float32)
    b0, b1 = cuda.dp_shard_range(n, rank, world)
    xs, gs = x[b0:b1].astype(np.float64), g[b0:b1].astype(np.float64)
    k = running_mean.astype(np.float64)[None, :, None, None]
    fwd = np.concatenate([(xs - k).sum(axis=(0, 2, 3)), ((xs - k) ** 2).sum(axis=(0, 2, 3)), [xs.size / c]])
    ft = torch.from_numpy(fwd)
    dist.all_reduce(ft)
    s, q, count = fwd[:c], fwd[c:2 * c], fwd[2 * c]
    mean = running_mean + s / count
    var = np.maximum(q / count - (s / count) ** 2, 0.0)
    istd = 1.0 / np.sqrt(var + 1e-5)
    xhat = (xs - mean[None, :, None, None]) * istd[None, :, None, None]
    local = np.concatenate([gs.sum(axis=(0, 2, 3)), (gs * xhat).sum(axis=(0, 2, 3))])   # dbeta, dgamma of this shard
    shared = torch.from_numpy(local.copy())
    dist.all_reduce(shared)
    sg, sgx = shared.numpy()[:c], shared.numpy()[c:]
    ga = gamma.astype(np.float64)[None, :, None, None]
    dx = istd[None, :, None, None] * (gs * ga - ga * sg[None, :, None, None] / count -
                                      xhat * ga * sgx[None, :, None, None] / count)
    # dbeta / dgamma stay this shard's own sums: they are summed across ranks with every other parameter gradient
    # (here: by the test, over the ranks' files)
    np.save(os.path.join(out_dir, f"bn_{rank}.npy"), np.concatenate([mean, var, dx.ravel(), local]))
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 3])
def test_shared_batchnorm_statistics_equal_the_full_batch(world, tmp_path, nrs_lib):
    import torch.multiprocessing as mp
    from neuralrs_b200 import cuda
    from oracle.nrs_oracle import Oracle
    mp.spawn(_bn_rank, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    o = Oracle("f64")
    rng = np.random.default_rng(7)
    n, c, h, w = 11, 6, 5, 4
    x = (rng.normal(size=(n, c, h, w)) * 2 + np.arange(c)[None, :, None, None]).astype(np.float32)
    g = rng.normal(size=(n, c, h, w)).astype(np.float32)
    gamma, beta = rng.normal(size=c).astype(np.float32), rng.normal(size=c).astype(np.float32)
    running_mean = rng.normal(size=c).astype(np.float32)
    y, xhat, istd, rm, rv = o.batchnorm_fwd(x, gamma, beta, running_mean, np.ones(c, np.float32), 1e-5, 0.0, True)
    dx, dgamma, dbeta = o.batchnorm_bwd(g, xhat, istd, gamma, True)
    # momentum 0: the oracle's running statistics after the call ARE the batch statistics
    dx_parts, dgamma_sum, dbeta_sum = [], np.zeros(c), np.zeros(c)
    for r in range(world):
        got = np.load(tmp_path / f"bn_{r}.npy")
        b0, b1 = cuda.dp_shard_range(n, r, world)
        m = (b1 - b0) * c * h * w
        assert np.allclose(got[:c], rm, rtol=1e-5, atol=1e-6) and np.allclose(got[c:2 * c], rv, rtol=1e-4, atol=1e-6)
        dx_parts.append(got[2 * c:2 * c + m].reshape(b1 - b0, c, h, w))
        dbeta_sum += got[2 * c + m:2 * c + m + c]
        dgamma_sum += got[2 * c + m + c:]
    assert np.linalg.norm(np.concatenate(dx_parts) - dx) <= 1e-5 * np.linalg.norm(dx)
    assert np.allclose(dgamma_sum, dgamma, rtol=1e-4, atol=1e-5) and np.allclose(dbeta_sum, dbeta, rtol=1e-4, atol=1e-5)


def test_a_shard_draws_its_samples_part_of_the_global_mask(nrs_lib):
    """Element i of a mask of `count` elements is word i%4 of counter block offset + i/4: a rank holding samples
    [b0, b1) of the global batch that starts its draw at block offset + b0*per/4 reproduces its rows of the mask a
    single process draws for the whole batch (what nrs_rng_window arranges on the device)."""
    from neuralrs_b200 import cuda
    from oracle.nrs_oracle import Oracle
    o = Oracle("f32")
    per, gb, seed, offset = 12, 10, 99, 5
    full = o.dropout_mask(gb * per, 0.3, seed, offset).reshape(gb, per)
    for world in (2, 3, 5):
        for r in range(world):
            b0, b1 = cuda.dp_shard_range(gb, r, world)
            assert (b0 * per) % 4 == 0
            part = o.dropout_mask((b1 - b0) * per, 0.3, seed, offset + b0 * per // 4).reshape(b1 - b0, per)
            assert np.array_equal(part, full[b0:b1])


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


# ---------------------------------------------------------------- deadlines and rank agreement
# Failure handling of the collective path, exercised on the host only: a rank that never joins a
# collective (gloo ranks on CPU) must surface as NRS_ERR_TIMEOUT through the library's deadline loop,
# and ranks that disagree about the model must be refused before anything is exchanged.

def test_watchdog_returns_when_the_poll_finishes_and_reports_failures(nrs_lib):
    from neuralrs_b200 import _lib, cuda
    calls = {"n": 0}

    def done_on_third():
        calls["n"] += 1
        return 1 if calls["n"] >= 3 else 0
    waited = cuda.watchdog_wait(done_on_third, timeout_ms=2000, interval_us=100)
    assert calls["n"] == 3 and waited < 1000
    with pytest.raises(_lib.NrsError) as e:
        cuda.watchdog_wait(lambda: -1, timeout_ms=2000)
    assert e.value.code == 5                      # NRS_ERR_NCCL: the polled operation failed
    with pytest.raises(_lib.NrsError) as e:
        cuda.watchdog_wait(lambda: 0, timeout_ms=50, interval_us=1000)
    assert e.value.code == 6                      # NRS_ERR_TIMEOUT
    polled = {"n": 0}

    def count():
        polled["n"] += 1
        return 0
    with pytest.raises(_lib.NrsError):
        cuda.watchdog_wait(count, timeout_ms=0)   # a zero deadline still polls once
    assert polled["n"] == 1


def _absent_rank_main(rank, world, port, out_dir):
    sys.path.insert(0, str(ROOT))
    import time
    import torch
    import torch.distributed as dist
    from neuralrs_b200 import _lib, cuda
    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
    flag = Path(out_dir) / "rank0_gave_up"
    if rank == 0:
        work = dist.all_reduce(torch.ones(4), async_op=True)      # rank 1 never issues its half
        t0 = time.time()
        try:
            cuda.watchdog_wait(lambda: 1 if work.is_completed() else 0, timeout_ms=400, interval_us=500)
            outcome = "completed"
        except _lib.NrsError as e:
            outcome = f"code{e.code}"
        (Path(out_dir) / "outcome.txt").write_text(f"{outcome} {time.time() - t0:.3f}")
        flag.write_text("1")
    else:
        t0 = time.time()
        while not flag.exists() and time.time() - t0 < 30:       # stays alive, never joins the collective
            time.sleep(0.02)
    os._exit(0)   # the collective can never complete: leave without tearing the group down


def test_rank_that_never_joins_a_collective_times_out(tmp_path, nrs_lib):
    import torch.multiprocessing as mp
    mp.spawn(_absent_rank_main, args=(2, _free_port(), str(tmp_path)), nprocs=2, join=True)
    outcome, seconds = (tmp_path / "outcome.txt").read_text().split()
    assert outcome == "code6"                     # NRS_ERR_TIMEOUT from the host watchdog
    assert 0.35 <= float(seconds) < 5.0


def _mismatch_rank_main(rank, world, port, out_dir):
    sys.path.insert(0, str(ROOT))
    import torch
    import torch.distributed as dist
    from neuralrs_b200 import _lib, cuda
    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
    lens = [27 * 64, 64, 4096 * 512, 512]
    results = []
    for case, mine in enumerate([lens,                                         # all ranks agree
                                 lens if rank == 0 else lens[:-1] + [513],     # rank 1 has a different layer width
                                 lens]):
        gb = 64 if (case < 2 or rank == 0) else 128                            # case 2: ranks disagree on the global batch
        fp = cuda.dp_fingerprint(mine, 1 << 20, gb, world)
        t = torch.tensor([fp & 0x7fffffff, fp >> 31 & 0x7fffffff, fp >> 62], dtype=torch.int64)
        got = [torch.zeros(3, dtype=torch.int64) for _ in range(world)]
        dist.all_gather(got, t)
        fps = [int(g[0]) | int(g[1]) << 31 | int(g[2]) << 62 for g in got]
        try:
            cuda.dp_check_fingerprints(fps)
            results.append("ok")
        except _lib.NrsError as e:
            results.append(f"code{e.code}")
    (Path(out_dir) / f"result_{rank}.txt").write_text(" ".join(results))
    dist.barrier()
    dist.destroy_process_group()


def test_ranks_that_disagree_about_the_model_are_refused_on_the_host(tmp_path, nrs_lib):
    import torch.multiprocessing as mp
    mp.spawn(_mismatch_rank_main, args=(2, _free_port(), str(tmp_path)), nprocs=2, join=True)
    for rank in range(2):
        assert (tmp_path / f"result_{rank}.txt").read_text() == "ok code2 code2"    # NRS_ERR_SHAPE on every rank
