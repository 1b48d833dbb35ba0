"""Data-parallel training on 2 GPUs against the same work on 1 GPU (needs >= 2 devices; skipped otherwise).
Each rank runs its shard with NCCL all-reduced gradient buckets; after two steps every rank's parameters
must equal the single-GPU full-batch run up to summation order.  Covered: the native trainer on the small
CNN and on a token model (transformer blocks), and the operator-level entry points (nrs_dp_create,
nrs_bucket_register, nrs_backward_graph_dp) under a caller's own loop over nodes."""
import os
import sys
import time
from pathlib import Path

import numpy as np
import pytest

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent

SMALL_LM = dict(name="small_lm", in_shape=(16,), classes=50, vocab=50, token_model=True,
                layers=[("embedding", 50, 32, 16), ("transformer_block", 32, 4, 64, 2, 1), ("transformer_block", 32, 4, 64, 2, 1),
                        ("linear", 32, 50)])


# conv + BatchNorm2d + ReLU, Linear + BatchNorm + ReLU + Dropout: batch statistics couple the samples of a batch,
# and the dropout mask of a rank's samples must be the one they have in the full batch
SMALL_BN = dict(name="small_bn", in_shape=(3, 8, 8), classes=10,
                layers=[("conv", 3, 32, 3, 1, 1), ("batchnorm", 32), ("relu",), ("conv", 32, 32, 3, 1, 1), ("batchnorm", 32),
                        ("relu",), ("maxpool", 2, 2), ("flatten",), ("linear", 512, 64), ("batchnorm", 64), ("relu",),
                        ("dropout", 0.25), ("linear", 64, 10)])


def _config(kind):
    from neuralrs_b200 import workloads
    return {"lm": SMALL_LM, "bn": SMALL_BN, "bn_local": SMALL_BN}.get(kind, workloads.SMALL_CNN)


def _batch(cfg, gb, seed):
    from neuralrs_b200 import workloads
    if cfg.get("token_model"):
        ids, labels = workloads.synthetic_tokens(cfg, gb, seed)
        return ids, labels.reshape(gb, -1)
    return workloads.synthetic_batch(cfg, gb, seed, uniform01=True)


def _step(tr, cfg, x, t):
    return tr.step_tokens(x, t) if cfg.get("token_model") else tr.step(x, t)


def _rendezvous(rank, tmp):
    from neuralrs_b200 import cuda
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
    return idf.read_bytes()


def _worker(rank, world, tmp, bucket_bytes, kind):
    sys.path.insert(0, str(ROOT))
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    from neuralrs_b200 import cuda, workloads
    cfg, hp, gb = _config(kind), workloads.ADAMW_HP, 8 if kind == "lm" else 64
    ctx = cuda.Context(rank)
    uid = _rendezvous(rank, tmp)
    tr = cuda.Trainer(cfg["layers"], cfg["in_shape"], cfg["classes"], hp["lr"], hp["beta1"], hp["beta2"], hp["eps"],
                      hp["wd"], fuse=True, ctx=ctx)
    tr.set_params(workloads.he_init(cfg["layers"], 5))
    tr.set_dp_timeout_ms(120000)
    _rewind_random_stream(ctx)
    tr.enable_dp(rank, world, uid, gb, bucket_bytes)
    if kind == "bn":
        tr.set_sync_batchnorm(True)
    b0, b1 = cuda.dp_shard_range(gb, rank, world)
    losses = []
    for step in range(3):   # the third step reads weight planes restaged behind the second step's bucket updates
        x, t = _batch(cfg, gb, 50 + step)
        losses.append(_step(tr, cfg, x[b0:b1], t[b0:b1]))
    np.save(Path(tmp) / f"params_{rank}.npy", np.concatenate([tr.get_param(i) for i in range(tr.n_params)]))
    np.save(Path(tmp) / f"loss_{rank}.npy", np.array(losses))
    if tr.n_buffers:
        np.save(Path(tmp) / f"buffers_{rank}.npy", np.concatenate([tr.get_buffer(i) for i in range(tr.n_buffers)]))
    tr.close()
    ctx.close()


@pytest.mark.parametrize("kind,bucket_bytes", [("cnn", 0), ("cnn", 16 * 1024), ("lm", 8 * 1024)])
def test_two_gpu_step_matches_single_gpu(tmp_path, gpu_ctx, kind, bucket_bytes):
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    import torch.multiprocessing as mp
    from neuralrs_b200 import cuda, workloads
    mp.spawn(_worker, args=(2, str(tmp_path), bucket_bytes, kind), nprocs=2, join=True)
    cfg, hp, gb = _config(kind), workloads.ADAMW_HP, 64 if kind == "cnn" else 8
    tr = cuda.Trainer(cfg["layers"], cfg["in_shape"], cfg["classes"], hp["lr"], hp["beta1"], hp["beta2"], hp["eps"],
                      hp["wd"], fuse=True, ctx=gpu_ctx)
    tr.set_params(workloads.he_init(cfg["layers"], 5))
    ref_losses = []
    for step in range(3):   # the third step reads weight planes restaged behind the second step's bucket updates
        x, t = _batch(cfg, gb, 50 + step)
        ref_losses.append(_step(tr, cfg, x, t))
    ref = np.concatenate([tr.get_param(i) for i in range(tr.n_params)])
    tr.close()
    p0, p1 = np.load(tmp_path / "params_0.npy"), np.load(tmp_path / "params_1.npy")
    assert np.array_equal(p0, p1)                       # replicas stay bit-identical
    # vs single GPU: summation order only.  (AdamW moves a weight by ~lr whatever the gradient's
    # size, so a near-zero gradient whose sign flips shows up as 2*lr on that one element.)
    assert np.linalg.norm(p0 - ref) <= 1e-4 * np.linalg.norm(ref)
    assert np.abs(p0 - ref).max() <= 2.5 * hp["lr"] * 3
    # each rank reports its shard's share of the global-mean loss
    l0, l1 = np.load(tmp_path / "loss_0.npy"), np.load(tmp_path / "loss_1.npy")
    assert np.abs(l0 + l1 - np.array(ref_losses)).max() <= 1e-4


def _rewind_random_stream(ctx):
    """Dropout masks come from a counter stream that earlier tests on the same context have advanced: both sides of
    a comparison start it from the same seed and offset."""
    import ctypes as C
    from neuralrs_b200 import _lib
    _lib.check(ctx.h, _lib.lib().nrs_rng_seed(ctx.h, C.c_uint64(4242)))


def _bn_run(tmp_path, gpu_ctx, kind):
    import torch.multiprocessing as mp
    from neuralrs_b200 import cuda, workloads
    mp.spawn(_worker, args=(2, str(tmp_path), 4096, kind), nprocs=2, join=True)
    _rewind_random_stream(gpu_ctx)
    cfg, hp, gb = SMALL_BN, workloads.ADAMW_HP, 64
    tr = cuda.Trainer(cfg["layers"], cfg["in_shape"], cfg["classes"], hp["lr"], hp["beta1"], hp["beta2"], hp["eps"],
                      hp["wd"], fuse=True, ctx=gpu_ctx)
    tr.set_params(workloads.he_init(cfg["layers"], 5))
    ref_losses = []
    for step in range(3):
        x, t = _batch(cfg, gb, 50 + step)
        ref_losses.append(_step(tr, cfg, x, t))
    parts = [tr.get_param(i) for i in range(tr.n_params)]
    ref = np.concatenate(parts)
    ref_buf = np.concatenate([tr.get_buffer(i) for i in range(tr.n_buffers)])
    tr.close()
    # A bias in front of a BatchNorm layer has a gradient of exactly zero in real arithmetic (the layer removes
    # the mean); what is computed is rounding noise of either sign, which AdamW's normalisation turns into steps
    # of a fraction of lr.  Those three vectors are compared with that bound only.
    keep = np.concatenate([np.full(p.size, i not in (1, 5, 9)) for i, p in enumerate(parts)])
    p0, p1 = np.load(tmp_path / "params_0.npy"), np.load(tmp_path / "params_1.npy")
    b0, b1 = np.load(tmp_path / "buffers_0.npy"), np.load(tmp_path / "buffers_1.npy")
    l0, l1 = np.load(tmp_path / "loss_0.npy"), np.load(tmp_path / "loss_1.npy")
    return dict(p0=p0, p1=p1, b0=b0, b1=b1, loss=l0 + l1, ref=ref, ref_buf=ref_buf, ref_losses=np.array(ref_losses), lr=hp["lr"],
                keep=keep)


def test_shared_batchnorm_statistics_make_two_gpus_equal_one(tmp_path, gpu_ctx):
    """With nrs_trainer_set_sync_batchnorm the per-channel sums of both passes are added up across the ranks, so a
    model with BatchNorm layers trains on two GPUs exactly as on one with the full batch (up to summation order),
    running statistics included."""
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    r = _bn_run(tmp_path, gpu_ctx, "bn")
    assert np.array_equal(r["p0"], r["p1"]) and np.array_equal(r["b0"], r["b1"])
    k = r["keep"]
    assert np.linalg.norm((r["p0"] - r["ref"])[k]) <= 1e-4 * np.linalg.norm(r["ref"][k])
    assert np.abs(r["p0"] - r["ref"]).max() <= 2.5 * r["lr"] * 3
    # running means carry those biases (a few 1e-5 absolute after three steps); per-rank statistics differ by percents
    assert np.linalg.norm(r["b0"] - r["ref_buf"]) <= 1e-3 * np.linalg.norm(r["ref_buf"])
    assert np.abs(r["loss"] - r["ref_losses"]).max() <= 1e-4


def test_per_rank_batchnorm_statistics_differ_from_one_gpu(tmp_path, gpu_ctx):
    """The default (every rank normalises with its own shard's statistics, as the single-GPU reference would with
    that batch) is a different computation from the full-batch one: the running statistics differ between the
    ranks and the loss differs from the single-GPU run.  This is what the shared statistics remove."""
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    r = _bn_run(tmp_path, gpu_ctx, "bn_local")
    assert np.array_equal(r["p0"], r["p1"])                 # parameters still move together (summed gradients)
    assert not np.array_equal(r["b0"], r["b1"])             # running statistics are per rank
    assert np.abs(r["loss"] - r["ref_losses"]).max() > 1e-4


def _mlp(seed):
    rng = np.random.default_rng(seed)
    x = rng.standard_normal((16, 12)).astype(np.float32)
    t = np.eye(5, dtype=np.float32)[rng.integers(0, 5, 16)]
    ws = [rng.standard_normal((12, 20)).astype(np.float32) * 0.3, rng.standard_normal(20).astype(np.float32) * 0.1,
          rng.standard_normal((20, 5)).astype(np.float32) * 0.3, rng.standard_normal(5).astype(np.float32) * 0.1]
    return x, t, ws


def _node_loop_grads(ctx, x, t, ws, global_batch, dp):
    """The reference's user loop over nodes: forward, cross-entropy backward (dividing by the GLOBAL batch),
    backward_graph — through the data-parallel group when given."""
    import ctypes as C
    from neuralrs_b200 import _lib
    from neuralrs_b200.cuda import Node, backward_graph, graph
    from neuralrs_b200.cuda import runtime as gpu

    def on_gpu(a):
        n = Node.new(a, list(a.shape), ctx)
        gpu.to_cuda(n)
        return n
    gx, gt = on_gpu(x), on_gpu(t)
    gx.requires_grad = False
    ps = [on_gpu(w) for w in ws]
    if dp:
        dp.register(ps, 256)
    gpu.zero_grad(ps)
    logits = graph.add(graph.matmul(graph.relu(graph.add(graph.matmul(gx, ps[0]), ps[1])), ps[2]), ps[3])
    # cross_entropy_backward with the global divisor: the gradient buffer is seeded through the raw entry point
    l = _lib.lib()
    grad = np.zeros((x.shape[0], 5), np.float32)
    gpu.set_grad(logits, grad)
    loss_dev = C.c_void_p()
    _lib.check(ctx.h, l.nrs_alloc(ctx.h, 4, 1, C.byref(loss_dev)))
    _lib.check(ctx.h, l.nrs_ce_fwd_bwd(ctx.h, C.c_void_p(logits.data_ptr()), C.c_void_p(gt.data_ptr()), loss_dev,
                                       C.c_void_p(logits.grad_ptr()), x.shape[0], 5, global_batch))
    if dp:
        dp.backward_graph(logits)
        dp.host_wait()
    else:
        backward_graph(logits)
    return [gpu.read_grad(p) for p in ps]


def _node_worker(rank, world, tmp):
    sys.path.insert(0, str(ROOT))
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    from neuralrs_b200 import cuda
    ctx = cuda.Context(rank)
    uid = _rendezvous(rank, tmp)
    x, t, ws = _mlp(7)
    dp = cuda.DataParallel(rank, world, uid, 16, timeout_ms=120000, ctx=ctx)
    b0, b1 = cuda.dp_shard_range(16, rank, world)
    grads = _node_loop_grads(ctx, x[b0:b1], t[b0:b1], ws, 16, dp)
    np.save(Path(tmp) / f"grads_{rank}.npy", np.concatenate([g.ravel() for g in grads]))
    dp.close()
    ctx.close()


def test_operator_level_exchange_on_two_gpus(tmp_path, gpu_ctx):
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    import torch.multiprocessing as mp
    mp.spawn(_node_worker, args=(2, str(tmp_path)), nprocs=2, join=True)
    x, t, ws = _mlp(7)
    ref = np.concatenate([g.ravel() for g in _node_loop_grads(gpu_ctx, x, t, ws, 16, None)])
    g0, g1 = np.load(tmp_path / "grads_0.npy"), np.load(tmp_path / "grads_1.npy")
    assert np.array_equal(g0, g1)
    assert np.linalg.norm(g0 - ref) <= 1e-5 * np.linalg.norm(ref)
