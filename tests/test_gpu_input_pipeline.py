"""The device-side input pipeline: flip/shift augmentation and one-hot expansion against the CPU oracle
(bit-exact: both are gathers / comparisons), and the trainer's staged entry points that use them."""
import ctypes as C

import numpy as np
import pytest

from neuralrs_b200 import _lib, cuda
from oracle import models
from .gpu_util import Dev, call

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("n,c,h,w,shift,flip", [(16, 3, 32, 32, 4, 1), (5, 1, 7, 9, 2, 1), (3, 2, 8, 8, 0, 1),
                                                  (4, 3, 32, 32, 4, 0), (1, 1, 1, 1, 3, 1), (64, 3, 32, 32, 4, 1)])
def test_augment_flip_shift(gpu_ctx, oracle32, n, c, h, w, shift, flip):
    l = _lib.lib()
    rng = np.random.default_rng(n * 100 + h)
    x = rng.normal(size=(n, c, h, w)).astype(np.float32)
    seed = 0xABCDEF0123456789
    _lib.check(gpu_ctx.h, l.nrs_rng_seed(gpu_ctx.h, seed))
    y = Dev(gpu_ctx, shape=x.shape)
    call(gpu_ctx, "nrs_augment_flip_shift", Dev(gpu_ctx, x), y, n, c, h, w, shift, flip)
    assert np.array_equal(y.get(), oracle32.augment_batch(x, seed, 0, shift, bool(flip)))
    off = C.c_uint64()
    _lib.check(gpu_ctx.h, l.nrs_rng_offset(gpu_ctx.h, C.byref(off)))
    assert off.value == n                                  # one counter block per image
    y2 = Dev(gpu_ctx, shape=x.shape)
    call(gpu_ctx, "nrs_augment_flip_shift", Dev(gpu_ctx, x), y2, n, c, h, w, shift, flip)
    assert np.array_equal(y2.get(), oracle32.augment_batch(x, seed, n, shift, bool(flip)))


@pytest.mark.parametrize("batch,classes", [(1024, 10), (7, 3), (1, 1), (33, 1000)])
def test_onehot(gpu_ctx, batch, classes):
    rng = np.random.default_rng(batch)
    labels = rng.integers(0, classes, batch).astype(np.int32)
    if batch > 2:
        labels[1] = classes            # out of range: an all-zero row
    out = Dev(gpu_ctx, shape=(batch, classes))
    call(gpu_ctx, "nrs_onehot", Dev(gpu_ctx, labels), out, batch, classes)
    want = (labels[:, None] == np.arange(classes)[None, :]).astype(np.float32)
    assert np.array_equal(out.get(), want)


def test_trainer_indexed_labels_and_augmentation(gpu_ctx, oracle32):
    cfg = dict(in_shape=(3, 16, 16), classes=10,
               layers=[("conv", 3, 32, 3, 1, 1), ("relu",), ("maxpool", 2, 2), ("flatten",), ("linear", 2048, 10)])
    hp = models.ADAMW_HP
    params = models.he_init(cfg["layers"], 600)
    rng = np.random.default_rng(601)
    batches = []
    for i in range(3):
        x = rng.random((24,) + cfg["in_shape"], dtype=np.float32)
        labels = rng.integers(0, 10, 24).astype(np.int32)
        onehot = (labels[:, None] == np.arange(10)[None, :]).astype(np.float32)
        batches.append((x, labels, onehot))

    def make():
        tr = cuda.Trainer(cfg["layers"], cfg["in_shape"], cfg["classes"], hp["lr"], hp["beta1"], hp["beta2"], hp["eps"],
                          hp["wd"], fuse=True, ctx=gpu_ctx)
        tr.set_params(params)
        return tr

    l = _lib.lib()
    seed = 77
    # reference run: augmentation done by the oracle on the host, one-hot rows uploaded, plain steps
    plain = make()
    losses_plain = []
    for i, (x, labels, onehot) in enumerate(batches):
        losses_plain.append(plain.step(oracle32.augment_batch(x, seed, 24 * i, 4, True), onehot))
    staged = make()
    staged.set_augment(4, True)
    _lib.check(gpu_ctx.h, l.nrs_rng_seed(gpu_ctx.h, seed))
    losses_staged = []
    staged.stage_next_indexed(batches[0][0], batches[0][1])
    for i in range(3):
        if i + 1 < 3:
            staged.stage_next_indexed(batches[i + 1][0], batches[i + 1][1])
        losses_staged.append(staged.step_staged())
    assert losses_staged == losses_plain
    for i in range(plain.n_params):
        assert np.array_equal(staged.get_param(i), plain.get_param(i))
    # evaluation mode leaves the images alone
    staged.set_training(False)
    plain.set_training(False)
    staged.stage_next_indexed(batches[0][0], batches[0][1])
    assert staged.step_staged() == plain.step(batches[0][0], batches[0][2])
    plain.close()
    staged.close()


def test_lagged_loss_readback_returns_every_loss_one_step_late(gpu_ctx):
    """nrs_trainer_step_staged_lagged issues step i and returns the loss of step i-1: the sequence of losses and the
    final parameters are those of synchronous staged steps, bit for bit."""
    cfg = dict(in_shape=(3, 16, 16), classes=10,
               layers=[("conv", 3, 32, 3, 1, 1), ("relu",), ("maxpool", 2, 2), ("flatten",), ("linear", 2048, 10)])
    hp = models.ADAMW_HP
    params = models.he_init(cfg["layers"], 610)
    rng = np.random.default_rng(611)
    batches = []
    for i in range(5):
        x = rng.random((16,) + cfg["in_shape"], dtype=np.float32)
        onehot = np.eye(10, dtype=np.float32)[rng.integers(0, 10, 16)]
        batches.append((x, onehot))

    def make():
        tr = cuda.Trainer(cfg["layers"], cfg["in_shape"], cfg["classes"], hp["lr"], hp["beta1"], hp["beta2"], hp["eps"],
                          hp["wd"], fuse=True, ctx=gpu_ctx)
        tr.set_params(params)
        return tr

    sync, lag = make(), make()
    want = []
    sync.stage_next(*batches[0])
    for i in range(5):
        if i + 1 < 5:
            sync.stage_next(*batches[i + 1])
        want.append(sync.step_staged())
    got = []
    lag.stage_next(*batches[0])
    for i in range(5):
        if i + 1 < 5:
            lag.stage_next(*batches[i + 1])
        prev = lag.step_staged_lagged()
        assert (prev is None) == (i == 0)
        if prev is not None:
            got.append(prev)
    got.append(lag.last_loss())
    assert got == want
    for i in range(sync.n_params):
        assert np.array_equal(lag.get_param(i), sync.get_param(i))
    # a lagged step with nothing staged is refused like a synchronous one
    with pytest.raises(Exception):
        lag.step_staged_lagged()
    sync.close()
    lag.close()
