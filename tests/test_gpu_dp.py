"""Data-parallel training step on 2 GPUs against the same step on 1 GPU (needs >= 2 devices;
skipped otherwise).  Each rank trains its shard through nrs_trainer_step with NCCL
all-reduced gradient buckets; after two steps every rank's parameters must equal the
single-GPU full-batch run up to summation order."""
import os
import sys
import time
from pathlib import Path

import numpy as np
import pytest

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent


def _worker(rank, world, tmp, bucket_bytes):
    sys.path.insert(0, str(ROOT))
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    from neuralrs_b200 import cuda
    from oracle import models      # model table and synthetic data only
    cfg = models.SMALL_CNN
    hp = models.ADAMW_HP
    gb = 64
    ctx = cuda.Context(rank)
    idf = Path(tmp) / "nccl_id.bin"
    if rank == 0:
        idf.with_suffix(".tmp").write_bytes(cuda.dp_unique_id())
        idf.with_suffix(".tmp").rename(idf)
    else:
        t0 = time.time()
        while not idf.exists():
            if time.time() - t0 > 60:
                raise RuntimeError("rank 0 never published the NCCL id")
            time.sleep(0.05)
    uid = idf.read_bytes()
    tr = cuda.Trainer(cfg["layers"], cfg["in_shape"], cfg["classes"], hp["lr"], hp["beta1"], hp["beta2"], hp["eps"],
                      hp["wd"], fuse=True, ctx=ctx)
    tr.set_params(models.he_init(cfg["layers"], 5))
    tr.enable_dp(rank, world, uid, gb, bucket_bytes)
    b0, b1 = cuda.dp_shard_range(gb, rank, world)
    losses = []
    for step in range(2):
        x, t = models.synthetic_batch(cfg, gb, 50 + step, uniform01=True)
        losses.append(tr.step(x[b0:b1], t[b0:b1]))
    np.save(Path(tmp) / f"params_{rank}.npy", np.concatenate([tr.get_param(i) for i in range(tr.n_params)]))
    np.save(Path(tmp) / f"loss_{rank}.npy", np.array(losses))
    tr.close()
    ctx.close()


@pytest.mark.parametrize("bucket_bytes", [0, 16 * 1024])
def test_two_gpu_step_matches_single_gpu(tmp_path, gpu_ctx, bucket_bytes):
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    import torch.multiprocessing as mp
    from neuralrs_b200 import cuda
    from oracle import models
    mp.spawn(_worker, args=(2, str(tmp_path), bucket_bytes), nprocs=2, join=True)
    cfg, hp, gb = models.SMALL_CNN, models.ADAMW_HP, 64
    tr = cuda.Trainer(cfg["layers"], cfg["in_shape"], cfg["classes"], hp["lr"], hp["beta1"], hp["beta2"], hp["eps"],
                      hp["wd"], fuse=True, ctx=gpu_ctx)
    tr.set_params(models.he_init(cfg["layers"], 5))
    ref_losses = []
    for step in range(2):
        x, t = models.synthetic_batch(cfg, gb, 50 + step, uniform01=True)
        ref_losses.append(tr.step(x, t))
    ref = np.concatenate([tr.get_param(i) for i in range(tr.n_params)])
    tr.close()
    p0, p1 = np.load(tmp_path / "params_0.npy"), np.load(tmp_path / "params_1.npy")
    assert np.array_equal(p0, p1)                       # replicas stay bit-identical
    # vs single GPU: summation order only.  (AdamW moves a weight by ~lr whatever the gradient's
    # size, so a near-zero gradient whose sign flips shows up as 2*lr on that one element.)
    assert np.linalg.norm(p0 - ref) <= 1e-4 * np.linalg.norm(ref)
    assert np.abs(p0 - ref).max() <= 2.5 * hp["lr"] * 2
    # each rank reports its shard's share of the global-mean loss
    l0, l1 = np.load(tmp_path / "loss_0.npy"), np.load(tmp_path / "loss_1.npy")
    assert np.abs(l0 + l1 - np.array(ref_losses)).max() <= 1e-4
