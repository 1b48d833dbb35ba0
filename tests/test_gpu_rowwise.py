"""The row-wise HBM-bound kernels on their register-resident (128-bit) and scalar paths: LayerNorm with the
residual add folded in, the one-launch LayerNorm backward (input gradients into one or two destinations plus
dgamma / dbeta), softmax, cross-entropy from dense one-hot rows and from int32 class indices, and the
vectorised 2x2 max-pool.  Against the f64 CPU oracle; integer output bit-exact."""
import ctypes as C

import numpy as np
import pytest

from neuralrs_b200 import _lib
from .conftest import rel_l2
from .gpu_util import Dev, call

pytestmark = pytest.mark.gpu
F = C.c_float

# widths on the vector path (1, 2, 4, 8 float4 per lane), off it (not a multiple of 4, wider than 1024)
LN_SHAPES = [(7, 8), (129, 128), (4096, 256), (300, 512), (65, 1024), (33, 1000), (5, 33), (3, 1028), (2, 2048)]


@pytest.mark.parametrize("rows,f", LN_SHAPES)
def test_layernorm_residual_matches_add_then_layernorm(gpu_ctx, oracle64, rows, f):
    rng = np.random.default_rng(rows * 7 + f)
    a = rng.normal(0.5, 2.0, size=(rows, f)).astype(np.float32)
    b = rng.normal(-0.3, 1.0, size=(rows, f)).astype(np.float32)
    gamma, beta = rng.normal(size=f).astype(np.float32), rng.normal(size=f).astype(np.float32)
    g = rng.normal(size=(rows, f)).astype(np.float32)
    x = (a + b).astype(np.float32)                        # the add kernel's f32 sum
    yr, xhr, isr = oracle64.layernorm_fwd(x, gamma, beta, 1e-5)
    dxr, dgr, dbr = oracle64.layernorm_bwd(g, xhr, isr, gamma)
    da_, db_, dga, dbe, dg_ = Dev(gpu_ctx, a), Dev(gpu_ctx, b), Dev(gpu_ctx, gamma), Dev(gpu_ctx, beta), Dev(gpu_ctx, g)
    y, xh, ist = Dev(gpu_ctx, shape=x.shape), Dev(gpu_ctx, shape=x.shape), Dev(gpu_ctx, shape=(rows,))
    call(gpu_ctx, "nrs_layernorm_residual_fwd", da_, db_, dga, dbe, y, xh, ist, rows, f, F(1e-5))
    assert np.abs(y.get() - yr).max() <= 1e-4
    assert np.abs(xh.get() - xhr).max() <= 1e-4
    # the two-kernel form gives the same bits
    s, y2, xh2, ist2 = Dev(gpu_ctx, shape=x.shape), Dev(gpu_ctx, shape=x.shape), Dev(gpu_ctx, shape=x.shape), Dev(gpu_ctx, shape=(rows,))
    call(gpu_ctx, "nrs_add", da_, db_, s, a.size)
    call(gpu_ctx, "nrs_layernorm_fwd", s, dga, dbe, y2, xh2, ist2, rows, f, F(1e-5))
    assert np.array_equal(y.get(), y2.get()) and np.array_equal(ist.get(), ist2.get())
    # backward: both addends and the parameters from one launch; first writers overwrite, then accumulate
    ga, gb2 = Dev(gpu_ctx, shape=x.shape), Dev(gpu_ctx, np.ones_like(x))
    gg, gbt = Dev(gpu_ctx, shape=(f,)), Dev(gpu_ctx, shape=(f,))
    call(gpu_ctx, "nrs_layernorm_residual_bwd", dg_, xh, ist, dga, ga, gb2, gg, gbt, rows, f, 0, 1, 0)
    assert rel_l2(ga.get(), dxr) <= 1e-5
    assert rel_l2(gb2.get() - 1.0, dxr) <= 2e-5
    assert rel_l2(gg.get(), dgr) <= 1e-5 and rel_l2(gbt.get(), dbr) <= 1e-5
    call(gpu_ctx, "nrs_layernorm_residual_bwd", dg_, xh, ist, dga, ga, None, gg, gbt, rows, f, 1, 0, 1)
    assert rel_l2(ga.get(), 2 * dxr) <= 1e-5
    assert rel_l2(gg.get(), 2 * dgr) <= 1e-5 and rel_l2(gbt.get(), 2 * dbr) <= 1e-5
    # only the second addend wants a gradient; only the parameters; run-to-run identical
    only_b = Dev(gpu_ctx, shape=x.shape)
    call(gpu_ctx, "nrs_layernorm_residual_bwd", dg_, xh, ist, dga, None, only_b, None, None, rows, f, 0, 0, 0)
    assert rel_l2(only_b.get(), dxr) <= 1e-5
    p1, p2, q1, q2 = (Dev(gpu_ctx, shape=(f,)) for _ in range(4))
    call(gpu_ctx, "nrs_layernorm_bwd", dg_, xh, ist, dga, None, p1, q1, rows, f, 0, 0)
    call(gpu_ctx, "nrs_layernorm_bwd", dg_, xh, ist, dga, None, p2, q2, rows, f, 0, 0)
    assert np.array_equal(p1.get(), p2.get()) and np.array_equal(q1.get(), q2.get())
    assert rel_l2(p1.get(), dgr) <= 1e-5


def test_layernorm_residual_graph_op_matches_two_operators(gpu_ctx):
    """TransformerBlock with the fused residual LayerNorm against the reference's add + layernorm composition,
    through the trainer (fuse on / off): identical losses and gradients up to rounding of different kernels."""
    from neuralrs_b200 import cuda, workloads
    layers = [("embedding", 40, 32, 16), ("transformer_block", 32, 4, 64, 1, 0), ("linear", 32, 40)]
    params = workloads.he_init(layers, 3)
    cfg = dict(in_shape=(16,), vocab=40)
    ids, labels = workloads.synthetic_tokens(cfg, 5, 4)
    out = []
    for fuse in (True, False):
        tr = cuda.Trainer(layers, (16,), 40, fuse=fuse, ctx=gpu_ctx)
        tr.set_params(params)
        loss = tr.forward_backward_tokens(ids, labels)
        out.append((loss, [tr.get_grad(i) for i in range(tr.n_params)]))
        tr.close()
    assert abs(out[0][0] - out[1][0]) <= 1e-5 * abs(out[1][0])
    for g0, g1 in zip(out[0][1], out[1][1]):
        assert rel_l2(g0, g1) <= 2e-5


@pytest.mark.parametrize("rows,width", [(5, 4), (1000, 128), (77, 256), (31, 512), (9, 1024), (6, 1000), (9, 33), (3, 1500)])
def test_softmax_paths(gpu_ctx, oracle64, rows, width):
    rng = np.random.default_rng(rows + width)
    x = (rng.normal(size=(rows, width)) * 3).astype(np.float32)
    x[0, :] = -1e30                                       # a fully masked row stays finite: uniform
    x[0, 0] = 0.0
    g = rng.normal(size=(rows, width)).astype(np.float32)
    yr = oracle64.softmax_fwd(x)
    y, gx = Dev(gpu_ctx, shape=x.shape), Dev(gpu_ctx, np.full(x.shape, 0.5, np.float32))
    call(gpu_ctx, "nrs_softmax_fwd", Dev(gpu_ctx, x), y, rows, width)
    assert np.abs(y.get() - yr).max() <= 1e-6
    assert np.abs(y.get().sum(1) - 1).max() <= 1e-5
    call(gpu_ctx, "nrs_softmax_bwd", y, Dev(gpu_ctx, g), gx, rows, width, 1)
    assert rel_l2(gx.get() - 0.5, oracle64.softmax_bwd(yr, g)) <= 2e-5


@pytest.mark.parametrize("batch,classes", [(16, 10), (64, 128), (33, 500), (300, 1000), (257, 1024), (9, 1001), (4, 2000)])
def test_cross_entropy_indexed_equals_one_hot(gpu_ctx, oracle64, batch, classes):
    rng = np.random.default_rng(batch + classes)
    logits = (rng.normal(size=(batch, classes)) * 3).astype(np.float32)
    labels = rng.integers(0, classes, batch).astype(np.int32)
    labels[0] = classes - 1
    labels[-1] = 0
    target = np.zeros((batch, classes), np.float32)
    target[np.arange(batch), labels] = 1
    dl, dt, dlab = Dev(gpu_ctx, logits), Dev(gpu_ctx, target), Dev(gpu_ctx, labels)
    loss_a, loss_b = Dev(gpu_ctx, shape=(1,)), Dev(gpu_ctx, shape=(1,))
    grad_a, grad_b = Dev(gpu_ctx, shape=logits.shape), Dev(gpu_ctx, shape=logits.shape)
    div = 3 * batch
    call(gpu_ctx, "nrs_ce_fwd_bwd", dl, dt, loss_a, grad_a, batch, classes, div)
    call(gpu_ctx, "nrs_ce_fwd_bwd_indexed", dl, dlab, loss_b, grad_b, batch, classes, div)
    assert np.array_equal(loss_a.get(), loss_b.get())
    assert np.array_equal(grad_a.get(), grad_b.get())
    ref = oracle64.ce_fwd(logits, target, div)
    assert abs(loss_a.get()[0] - ref) <= 1e-5 * max(1, abs(ref))
    assert rel_l2(grad_a.get(), oracle64.ce_bwd(logits, target, div)) <= 1e-5
    # an index outside [0, classes) is an all-zero target row: no loss term, gradient = softmax / divisor
    bad = labels.copy()
    bad[1 % batch] = classes
    target[1 % batch, :] = 0
    call(gpu_ctx, "nrs_ce_fwd_bwd_indexed", dl, Dev(gpu_ctx, bad), loss_b, grad_b, batch, classes, div)
    ref = oracle64.ce_fwd(logits, target, div)
    assert abs(loss_b.get()[0] - ref) <= 1e-5 * max(1, abs(ref))
    assert rel_l2(grad_b.get(), oracle64.ce_bwd(logits, target, div)) <= 1e-5


@pytest.mark.parametrize("shape", [(2, 3, 8, 8), (3, 5, 6, 12), (1, 2, 2, 4), (2, 2, 8, 6), (64, 16, 32, 32)])
def test_maxpool_2x2_vector_path(gpu_ctx, oracle32, shape):
    n, c, h, w = shape
    rng = np.random.default_rng(h * w)
    x = rng.integers(-3, 4, size=shape).astype(np.float32)      # many ties: the first maximum must win
    g = rng.normal(size=(n, c, h // 2, w // 2)).astype(np.float32)
    yr, amr = oracle32.maxpool_fwd(x, 2, 2)
    y = Dev(gpu_ctx, shape=yr.shape)
    am = Dev(gpu_ctx, shape=yr.shape, dtype=np.int32)
    call(gpu_ctx, "nrs_maxpool_fwd", Dev(gpu_ctx, x), y, am, n, c, h, w, 2, 2)
    assert np.array_equal(y.get(), yr)
    assert np.array_equal(am.get(), amr)
    y2 = Dev(gpu_ctx, shape=yr.shape)
    call(gpu_ctx, "nrs_maxpool_fwd", Dev(gpu_ctx, x), y2, None, n, c, h, w, 2, 2)       # argmax is optional
    assert np.array_equal(y2.get(), yr)
    dxr = oracle32.maxpool_bwd(g, amr, x.shape)
    gx = Dev(gpu_ctx, np.full(shape, 7.0, np.float32))
    call(gpu_ctx, "nrs_maxpool_bwd", Dev(gpu_ctx, g), am, gx, n, c, h, w, 2, 2, 0)
    assert np.array_equal(gx.get(), dxr)
    call(gpu_ctx, "nrs_maxpool_bwd", Dev(gpu_ctx, g), am, gx, n, c, h, w, 2, 2, 1)
    assert np.array_equal(gx.get(), (dxr + dxr).astype(np.float32))
