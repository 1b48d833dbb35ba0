"""GPU parity of the raw C-ABI operators against the CPU oracle (bit-exact for
integer outputs, stated tolerances for f32).  Run with -m gpu on a B200."""
import ctypes as C

import numpy as np
import pytest

from neuralrs_b200 import _lib
from .conftest import max_rel, rel_l2
from .gpu_util import Dev, call

pytestmark = pytest.mark.gpu
F = C.c_float

# Relative-error bars stated by the hot-path spec: 3xTF32 (default) and FP32 <= 1e-4, TF32 <= 1e-2.
TOL = {_lib.MATH_3XTF32: 1e-4, _lib.MATH_FP32: 1e-4, _lib.MATH_TF32: 1e-2}


@pytest.fixture(params=[_lib.MATH_FP32, _lib.MATH_3XTF32, _lib.MATH_TF32], ids=["fp32", "3xtf32", "tf32"])
def math_mode(request, gpu_ctx):
    gpu_ctx.set_math_mode(request.param)
    yield request.param
    gpu_ctx.set_math_mode(_lib.MATH_3XTF32)


GEMM_SHAPES = [(40, 32, 56), (16, 10, 24), (1, 1, 1), (129, 257, 65), (64, 128, 3136), (256, 512, 1024),
               (300, 1000, 256), (128, 128, 128), (512, 256, 8),
               (1024, 10, 512), (1024, 512, 10), (512, 10, 1024),   # classifier head: the thin-product kernels
               (515, 7, 130), (130, 16, 515), (203, 13, 1027)]      # ... with ragged rows and reduction lengths


@pytest.mark.parametrize("m,n,k", GEMM_SHAPES)
@pytest.mark.parametrize("ta,tb", [(0, 0), (0, 1), (1, 0), (1, 1)])
def test_gemm_all_transposes(gpu_ctx, oracle64, math_mode, m, n, k, ta, tb):
    rng = np.random.default_rng(m * 131 + n * 17 + k + ta * 2 + tb)
    a = rng.normal(size=(m, k)).astype(np.float32)
    b = rng.normal(size=(k, n)).astype(np.float32)
    ref = oracle64.matmul_fwd(a, b)
    da = Dev(gpu_ctx, a.T if ta else a)
    db = Dev(gpu_ctx, b.T if tb else b)
    dc = Dev(gpu_ctx, shape=(m, n))
    call(gpu_ctx, "nrs_gemm", ta, tb, m, n, k, da, db, dc, None, 0, F(0))
    assert rel_l2(dc.get(), ref) <= TOL[math_mode]


def test_gemm_epilogues(gpu_ctx, oracle64, math_mode):
    rng = np.random.default_rng(7)
    m, n, k = 96, 160, 72
    a, b = rng.normal(size=(m, k)).astype(np.float32), rng.normal(size=(k, n)).astype(np.float32)
    bias = rng.normal(size=n).astype(np.float32)
    c0 = rng.normal(size=(m, n)).astype(np.float32)
    z = oracle64.bias_add_fwd(oracle64.matmul_fwd(a, b), bias)
    da, db, dbias = Dev(gpu_ctx, a), Dev(gpu_ctx, b), Dev(gpu_ctx, bias)
    for act, ref in ((0, z), (1, oracle64.relu_fwd(z)), (2, oracle64.gelu_fwd(z))):
        dc = Dev(gpu_ctx, c0)
        call(gpu_ctx, "nrs_gemm", 0, 0, m, n, k, da, db, dc, dbias, act, F(0))
        assert rel_l2(dc.get(), ref) <= TOL[math_mode]
        dc = Dev(gpu_ctx, c0)
        call(gpu_ctx, "nrs_gemm", 0, 0, m, n, k, da, db, dc, dbias, act, F(1))   # accumulate into C
        assert rel_l2(dc.get(), ref + c0) <= TOL[math_mode]


def test_bmm(gpu_ctx, oracle64, math_mode):
    rng = np.random.default_rng(8)
    bt, m, k, n = 6, 128, 32, 128     # attention-score shape of the transformer config
    a, b = rng.normal(size=(bt, m, k)).astype(np.float32), rng.normal(size=(bt, k, n)).astype(np.float32)
    g = rng.normal(size=(bt, m, n)).astype(np.float32)
    da, db, dg = Dev(gpu_ctx, a), Dev(gpu_ctx, b), Dev(gpu_ctx, g)
    dc = Dev(gpu_ctx, shape=(bt, m, n))
    call(gpu_ctx, "nrs_bmm", 0, 0, bt, m, n, k, da, db, dc, F(0))
    assert rel_l2(dc.get(), oracle64.bmm_fwd(a, b)) <= TOL[math_mode]
    ra, rb = oracle64.bmm_bwd(a, b, g)
    dda, ddb = Dev(gpu_ctx, shape=a.shape), Dev(gpu_ctx, shape=b.shape)
    call(gpu_ctx, "nrs_bmm", 0, 1, bt, m, k, n, dg, db, dda, F(0))
    call(gpu_ctx, "nrs_bmm", 1, 0, bt, k, n, m, da, dg, ddb, F(0))
    assert rel_l2(dda.get(), ra) <= TOL[math_mode]
    assert rel_l2(ddb.get(), rb) <= TOL[math_mode]


CONV_CASES = [
    # n, ci, h, w, co, kh, kw, stride, pad
    (2, 3, 8, 8, 4, 3, 3, 1, 1),        # tests/cuda_conv2d_test.rs:17-18
    (2, 3, 7, 7, 5, 3, 3, 1, 1),        # tests/cuda_conv2d_test.rs:48-49
    (1, 1, 3, 3, 1, 2, 2, 1, 0),        # tests/nn_conv_test.rs
    (3, 2, 9, 6, 4, 2, 3, 2, 1),        # stride 2, ragged
    (4, 1, 28, 28, 32, 3, 3, 1, 1),     # small-CNN first layer
    (4, 32, 14, 14, 64, 3, 3, 1, 1),    # small-CNN second layer
    (2, 64, 32, 32, 128, 3, 3, 1, 1),   # conv microbench shape, 2 samples
    (3, 64, 16, 16, 64, 3, 3, 1, 1),
    (4, 128, 8, 8, 256, 3, 3, 1, 1),
    (2, 32, 12, 20, 48, 1, 1, 1, 0),    # 1x1
    (1, 3, 32, 32, 64, 3, 3, 1, 1),     # VGG first layer
    # row-streaming weight gradient: two channel chunks, a ragged last m-block, one-row images,
    # a 96-channel chunk, enough rows for several splits, and a shape it must leave to the general kernel
    (5, 256, 8, 8, 256, 3, 3, 1, 1),
    (3, 96, 8, 16, 160, 3, 3, 1, 1),
    (7, 32, 1, 8, 32, 3, 3, 1, 1),
    (40, 64, 16, 16, 64, 3, 3, 1, 1),
    (2, 32, 6, 12, 32, 3, 3, 1, 1),
    (2, 64, 10, 10, 64, 5, 5, 1, 2),
    (3, 32, 16, 16, 32, 3, 3, 1, 1),    # 32 / 64 output channels: two horizontal taps share the accumulator rows
    (2, 64, 8, 32, 64, 3, 3, 1, 1),
    (2, 128, 5, 64, 96, 3, 3, 1, 1),    # 64-pixel rows
]


@pytest.mark.parametrize("cfg", CONV_CASES)
def test_conv2d_fwd_bwd(gpu_ctx, oracle64, math_mode, cfg):
    n, ci, h, w, co, kh, kw, s, p = cfg
    rng = np.random.default_rng(sum(cfg))
    x = rng.normal(size=(n, ci, h, w)).astype(np.float32)
    wt = (rng.normal(size=(co, ci, kh, kw)) * np.sqrt(2.0 / (ci * kh * kw))).astype(np.float32)
    b = rng.normal(size=co).astype(np.float32) * 0.1
    yref = oracle64.conv2d_fwd(x, wt, b, s, p)
    dy = rng.normal(size=yref.shape).astype(np.float32)
    dxr, dwr, dbr = oracle64.conv2d_bwd(x, wt, dy, s, p)
    dx_, dw_, db_, dyd = Dev(gpu_ctx, x), Dev(gpu_ctx, wt), Dev(gpu_ctx, b), Dev(gpu_ctx, dy)
    y = Dev(gpu_ctx, shape=yref.shape)
    call(gpu_ctx, "nrs_conv2d_fwd", dx_, dw_, db_, y, n, ci, h, w, co, kh, kw, s, p, 0)
    tol = TOL[math_mode]
    assert rel_l2(y.get(), yref) <= tol
    call(gpu_ctx, "nrs_conv2d_fwd", dx_, dw_, db_, y, n, ci, h, w, co, kh, kw, s, p, 1)
    assert rel_l2(y.get(), np.maximum(yref, 0)) <= tol
    gx, gw, gb = Dev(gpu_ctx, shape=x.shape), Dev(gpu_ctx, shape=wt.shape), Dev(gpu_ctx, shape=b.shape)
    call(gpu_ctx, "nrs_conv2d_bwd", dx_, dw_, dyd, gx, gw, gb, n, ci, h, w, co, kh, kw, s, p, 0)
    assert rel_l2(gx.get(), dxr) <= tol
    assert rel_l2(gw.get(), dwr) <= tol
    assert rel_l2(gb.get(), dbr) <= 1e-5
    # accumulate mode adds a second copy; the weight gradient is run-to-run deterministic
    first = gw.get().copy()
    call(gpu_ctx, "nrs_conv2d_bwd", dx_, dw_, dyd, gx, gw, gb, n, ci, h, w, co, kh, kw, s, p, 1)
    assert rel_l2(gx.get(), 2 * dxr) <= tol
    assert rel_l2(gw.get(), 2 * dwr) <= tol
    gw2 = Dev(gpu_ctx, shape=wt.shape)
    call(gpu_ctx, "nrs_conv2d_bwd", dx_, dw_, dyd, None, gw2, None, n, ci, h, w, co, kh, kw, s, p, 0)
    assert np.array_equal(gw2.get(), first)


@pytest.mark.parametrize("cfg", [(6, 64, 16, 16, 128, 3, 3, 1, 1), (5, 32, 8, 8, 64, 3, 3, 1, 1), (4, 3, 12, 12, 32, 3, 3, 1, 1)])
def test_cached_operand_planes_change_nothing(gpu_ctx, math_mode, cfg):
    """nrs_planes_cache makes a tensor's tensor-core operand once; the convolutions must return the very bits they
    return when they stage it themselves, stale planes must be droppable, and the calls are no-ops where the
    tensor-core path does not apply (FP32 mode, 3 channels)."""
    n, ci, h, w, co, kh, kw, s, p = cfg
    rng = np.random.default_rng(sum(cfg) + 1)
    x = rng.normal(size=(n, ci, h, w)).astype(np.float32)
    wt = (rng.normal(size=(co, ci, kh, kw)) * 0.1).astype(np.float32)
    dy = rng.normal(size=(n, co, h, w)).astype(np.float32)
    dx_, dw_, db_, dyd = Dev(gpu_ctx, x), Dev(gpu_ctx, wt), Dev(gpu_ctx, np.zeros(co, np.float32)), Dev(gpu_ctx, dy)

    def run():
        y, gx, gw = Dev(gpu_ctx, shape=dy.shape), Dev(gpu_ctx, shape=x.shape), Dev(gpu_ctx, shape=wt.shape)
        call(gpu_ctx, "nrs_conv2d_fwd", dx_, dw_, db_, y, n, ci, h, w, co, kh, kw, s, p, 0)
        call(gpu_ctx, "nrs_conv2d_bwd", dx_, dw_, dyd, gx, gw, None, n, ci, h, w, co, kh, kw, s, p, 0)
        return y.get(), gx.get(), gw.get()
    plain = run()
    call(gpu_ctx, "nrs_planes_cache", dx_, n, ci, h, w)
    call(gpu_ctx, "nrs_planes_cache", dyd, n, co, h, w)
    cached = run()
    for a, b in zip(plain, cached):
        assert np.array_equal(a, b)
    # new contents: drop (or re-cache) first
    x2 = (x * 0.5 + 1.0).astype(np.float32)
    call(gpu_ctx, "nrs_planes_drop", dx_)
    _lib.check(gpu_ctx.h, _lib.lib().nrs_h2d(gpu_ctx.h, dx_.ptr, x2.ctypes.data_as(C.c_void_p), x2.nbytes))
    gpu_ctx.sync()
    call(gpu_ctx, "nrs_planes_cache", dx_, n, ci, h, w)
    again = run()
    call(gpu_ctx, "nrs_planes_drop", dx_)
    call(gpu_ctx, "nrs_planes_drop", dyd)
    call(gpu_ctx, "nrs_planes_drop", dyd)        # dropping twice / an unknown pointer is fine
    fresh = run()
    for a, b in zip(again, fresh):
        assert np.array_equal(a, b)
    assert not np.array_equal(again[0], plain[0])
    l = _lib.lib()
    assert l.nrs_planes_cache(gpu_ctx.h, None, n, ci, h, w) == 1
    assert l.nrs_planes_cache(gpu_ctx.h, dx_.ptr, n, 0, h, w) == 2


def test_conv2d_empty_batch_and_bad_args(gpu_ctx):
    l = _lib.lib()
    w = Dev(gpu_ctx, np.ones((4, 3, 3, 3), np.float32))
    gw = Dev(gpu_ctx, np.ones((4, 3, 3, 3), np.float32))
    call(gpu_ctx, "nrs_conv2d_bwd", None, w, None, None, gw, None, 0, 3, 8, 8, 4, 3, 3, 1, 1, 0)
    assert np.all(gw.get() == 0)
    assert l.nrs_conv2d_fwd(gpu_ctx.h, None, None, None, None, 1, 3, 2, 2, 4, 3, 3, 1, 0, 0) == 2   # kernel > input
    assert l.nrs_conv2d_fwd(gpu_ctx.h, None, w.ptr, None, None, 1, 3, 8, 8, 4, 3, 3, 1, 1, 0) == 1   # null tensor
    assert b"null" in l.nrs_last_error(gpu_ctx.h)


@pytest.mark.parametrize("n", [1, 5, 4096, 100003])
def test_elementwise(gpu_ctx, oracle32, n):
    rng = np.random.default_rng(n)
    a, b = rng.normal(size=n).astype(np.float32), rng.normal(size=n).astype(np.float32)
    da, db, do = Dev(gpu_ctx, a), Dev(gpu_ctx, b), Dev(gpu_ctx, shape=(n,))
    call(gpu_ctx, "nrs_add", da, db, do, n)
    assert np.array_equal(do.get(), a + b)
    call(gpu_ctx, "nrs_relu_fwd", da, do, n)
    assert np.array_equal(do.get(), oracle32.relu_fwd(a))
    call(gpu_ctx, "nrs_relu_bwd", da, db, do, n, 0)
    assert np.array_equal(do.get(), oracle32.relu_bwd(a, b))
    call(gpu_ctx, "nrs_relu_bwd", da, db, do, n, 1)
    assert np.allclose(do.get(), 2 * oracle32.relu_bwd(a, b))
    call(gpu_ctx, "nrs_gelu_fwd", da, do, n)
    assert np.abs(do.get() - oracle32.gelu_fwd(a)).max() <= 1e-6
    call(gpu_ctx, "nrs_gelu_bwd", da, db, do, n, 0)
    assert np.abs(do.get() - oracle32.gelu_bwd(a, b)).max() <= 1e-5
    acc = Dev(gpu_ctx, a)
    call(gpu_ctx, "nrs_accumulate", acc, db, n)
    assert np.array_equal(acc.get(), a + b)
    call(gpu_ctx, "nrs_scale", da, do, n, F(0.125), 0)
    assert np.array_equal(do.get(), a * np.float32(0.125))


@pytest.mark.parametrize("rows,cols", [(1, 1), (16, 10), (64, 128), (1000, 33), (4096, 256), (7, 1000)])
def test_bias_and_reductions(gpu_ctx, oracle64, rows, cols):
    rng = np.random.default_rng(rows * 7 + cols)
    a, bias = rng.normal(size=(rows, cols)).astype(np.float32), rng.normal(size=cols).astype(np.float32)
    da, db, do = Dev(gpu_ctx, a), Dev(gpu_ctx, bias), Dev(gpu_ctx, shape=a.shape)
    call(gpu_ctx, "nrs_bias_add", da, db, do, rows, cols)
    assert np.array_equal(do.get(), a + bias)
    out = Dev(gpu_ctx, bias)
    call(gpu_ctx, "nrs_sum_axis0", da, out, rows, cols, 0)
    _, ref = oracle64.bias_add_bwd(a)
    assert np.abs(out.get() - ref).max() <= 1e-5 * max(1.0, np.abs(ref).max())
    call(gpu_ctx, "nrs_sum_axis0", da, out, rows, cols, 1)
    assert np.abs(out.get() - 2 * ref).max() <= 2e-5 * max(1.0, np.abs(ref).max())


@pytest.mark.parametrize("n,c,plane", [(2, 5, 49), (8, 128, 1024), (64, 3, 7), (33, 64, 256)])
def test_channel_sum(gpu_ctx, n, c, plane):
    rng = np.random.default_rng(n + c + plane)
    g = rng.normal(size=(n, c, plane)).astype(np.float32)
    out = Dev(gpu_ctx, shape=(c,))
    call(gpu_ctx, "nrs_channel_sum", Dev(gpu_ctx, g), out, n, c, plane, 0)
    ref = g.astype(np.float64).sum((0, 2))
    assert np.abs(out.get() - ref).max() <= 1e-5 * max(1.0, np.abs(ref).max())


@pytest.mark.parametrize("shape,k,s", [((2, 3, 8, 8), 2, 2), ((2, 3, 7, 7), 3, 1), ((1, 1, 4, 4), 2, 2),
                                       ((4, 32, 28, 28), 2, 2), ((3, 5, 9, 9), 2, 2), ((2, 4, 10, 10), 3, 2)])
def test_maxpool(gpu_ctx, oracle32, shape, k, s):
    n, c, h, w = shape
    size = int(np.prod(shape))
    x = ((np.arange(size) * 31 + 7) % 97 * 0.05 - 2.0).astype(np.float32).reshape(shape)  # cuda_maxpool_test.rs:11
    yref, amref = oracle32.maxpool_fwd(x, k, s)
    g = (np.arange(yref.size) % 7 * 0.2 + 0.1).astype(np.float32).reshape(yref.shape)
    dxref = oracle32.maxpool_bwd(g, amref, shape)
    dx_, y, am = Dev(gpu_ctx, x), Dev(gpu_ctx, shape=yref.shape), Dev(gpu_ctx, shape=yref.shape, dtype=np.int32)
    call(gpu_ctx, "nrs_maxpool_fwd", dx_, y, am, n, c, h, w, k, s)
    assert np.array_equal(y.get(), yref)
    assert np.array_equal(am.get(), amref)          # index work: bit-exact, ties included
    gx = Dev(gpu_ctx, np.full(shape, 5.0, np.float32))
    call(gpu_ctx, "nrs_maxpool_bwd", Dev(gpu_ctx, g), am, gx, n, c, h, w, k, s, 0)
    assert np.abs(gx.get() - dxref).max() <= 1e-5
    call(gpu_ctx, "nrs_maxpool_bwd", Dev(gpu_ctx, g), am, gx, n, c, h, w, k, s, 1)
    assert np.abs(gx.get() - 2 * dxref).max() <= 1e-5


@pytest.mark.parametrize("batch,classes", [(16, 10), (1, 10), (64, 10), (300, 1000), (1024, 10)])
def test_cross_entropy(gpu_ctx, oracle64, batch, classes):
    rng = np.random.default_rng(batch + classes)
    logits = (rng.normal(size=(batch, classes)) * 3).astype(np.float32)
    target = np.zeros((batch, classes), np.float32)
    target[np.arange(batch), rng.integers(0, classes, batch)] = 1
    dl, dt = Dev(gpu_ctx, logits), Dev(gpu_ctx, target)
    loss, grad = Dev(gpu_ctx, shape=(1,)), Dev(gpu_ctx, shape=logits.shape)
    for div in (batch, 4 * batch):
        call(gpu_ctx, "nrs_ce_fwd_bwd", dl, dt, loss, grad, batch, classes, div)
        assert abs(loss.get()[0] - oracle64.ce_fwd(logits, target, div)) <= 1e-5 * max(1, abs(oracle64.ce_fwd(logits, target, div)))
        assert rel_l2(grad.get(), oracle64.ce_bwd(logits, target, div)) <= 1e-5
    row = Dev(gpu_ctx, shape=(batch,))
    call(gpu_ctx, "nrs_ce_fwd", dl, dt, loss, row, batch, classes, batch)
    assert abs(row.get().sum() / batch - loss.get()[0]) <= 1e-5 * max(1, abs(loss.get()[0]))
    call(gpu_ctx, "nrs_ce_bwd", dl, dt, grad, batch, classes, batch)
    assert rel_l2(grad.get(), oracle64.ce_bwd(logits, target)) <= 1e-5


@pytest.mark.parametrize("n", [256, 64, 1, 100003])
def test_adamw_flat(gpu_ctx, oracle32, n):
    # tests/cuda_adamw_test.rs:11-15 inputs; 10 steps with the same gradient
    p = (np.arange(n) % 17 * 0.1 - 0.8).astype(np.float32)
    g = (np.arange(n) % 11 * 0.05 - 0.25).astype(np.float32)
    lr, b1, b2, eps, wd = 0.001, 0.9, 0.999, 1e-8, 0.01
    pr, mr, vr = p.copy(), np.zeros(n, np.float32), np.zeros(n, np.float32)
    dp, dg = Dev(gpu_ctx, p), Dev(gpu_ctx, g)
    dm, dv = Dev(gpu_ctx, shape=(n,), zero=True), Dev(gpu_ctx, shape=(n,), zero=True)
    for t in range(10):
        oracle32.adamw_step(pr, g, mr, vr, lr, b1, b2, eps, wd, t)
        bc1 = np.float32(1) - np.float32(b1) ** np.int32(t + 1)
        bc2 = np.float32(1) - np.float32(b2) ** np.int32(t + 1)
        call(gpu_ctx, "nrs_adamw_step", dp, dg, dm, dv, n, F(lr), F(b1), F(b2), F(eps), F(wd), F(bc1), F(bc2), F(1.0))
    assert np.abs(dp.get() - pr).max() <= 1e-4      # bar of tests/cuda_adamw_test.rs:35
    assert np.abs(dm.get() - mr).max() <= 1e-6
    assert np.abs(dv.get() - vr).max() <= 1e-6


@pytest.mark.parametrize("rows,f", [(3, 8), (4096, 256), (17, 1000), (5, 33)])
def test_layernorm(gpu_ctx, oracle64, rows, f):
    rng = np.random.default_rng(rows + f)
    x = rng.normal(1.0, 2.0, size=(rows, f)).astype(np.float32)
    gamma, beta = rng.normal(size=f).astype(np.float32), rng.normal(size=f).astype(np.float32)
    g = rng.normal(size=(rows, f)).astype(np.float32)
    yr, xhr, isr = oracle64.layernorm_fwd(x, gamma, beta, 1e-5)
    dxr, dgr, dbr = oracle64.layernorm_bwd(g, xhr, isr, gamma)
    dx_, dga, dbe, dg_ = Dev(gpu_ctx, x), Dev(gpu_ctx, gamma), Dev(gpu_ctx, beta), Dev(gpu_ctx, g)
    y, xh, ist = Dev(gpu_ctx, shape=x.shape), Dev(gpu_ctx, shape=x.shape), Dev(gpu_ctx, shape=(rows,))
    call(gpu_ctx, "nrs_layernorm_fwd", dx_, dga, dbe, y, xh, ist, rows, f, F(1e-5))
    assert np.abs(y.get() - yr).max() <= 1e-4      # bar of tests/cuda_layers_test.rs:58-61
    gx, gg, gb = Dev(gpu_ctx, shape=x.shape), Dev(gpu_ctx, shape=(f,)), Dev(gpu_ctx, shape=(f,))
    call(gpu_ctx, "nrs_layernorm_bwd", dg_, xh, ist, dga, gx, gg, gb, rows, f, 0, 0)
    assert rel_l2(gx.get(), dxr) <= 1e-5
    assert rel_l2(gg.get(), dgr) <= 1e-5
    assert rel_l2(gb.get(), dbr) <= 1e-5


@pytest.mark.parametrize("rows,width", [(4, 3), (32768, 128), (5, 1000), (9, 33)])
def test_softmax(gpu_ctx, oracle64, rows, width):
    rng = np.random.default_rng(rows + width)
    x, g = (rng.normal(size=(rows, width)) * 2).astype(np.float32), rng.normal(size=(rows, width)).astype(np.float32)
    yr = oracle64.softmax_fwd(x)
    y, gx = Dev(gpu_ctx, shape=x.shape), Dev(gpu_ctx, shape=x.shape)
    call(gpu_ctx, "nrs_softmax_fwd", Dev(gpu_ctx, x), y, rows, width)
    assert np.abs(y.get() - yr).max() <= 1e-6
    call(gpu_ctx, "nrs_softmax_bwd", y, Dev(gpu_ctx, g), gx, rows, width, 0)
    assert rel_l2(gx.get(), oracle64.softmax_bwd(yr, g)) <= 1e-5


def test_manipulation(gpu_ctx, oracle32):
    rng = np.random.default_rng(11)
    x = rng.normal(size=(3, 37, 50)).astype(np.float32)
    y = Dev(gpu_ctx, shape=(3, 50, 37))
    call(gpu_ctx, "nrs_transpose", Dev(gpu_ctx, x), y, 3, 37, 50, 0)
    assert np.array_equal(y.get(), oracle32.transpose_fwd(x))
    s = Dev(gpu_ctx, shape=(3 * 37, 20))
    call(gpu_ctx, "nrs_slice_cols_fwd", Dev(gpu_ctx, x), s, 3 * 37, 50, 10, 30)
    assert np.array_equal(s.get(), oracle32.slice_cols_fwd(x.reshape(-1, 50), 10, 30))
    gx = Dev(gpu_ctx, shape=(3 * 37, 50), zero=True)
    call(gpu_ctx, "nrs_slice_cols_bwd", s, gx, 3 * 37, 50, 10, 30, 1)
    assert np.array_equal(gx.get(), oracle32.slice_cols_bwd(s.get(), (3 * 37, 50), 10, 30))
    out = Dev(gpu_ctx, shape=(3 * 37, 70), zero=True)
    call(gpu_ctx, "nrs_concat_write", Dev(gpu_ctx, x), out, 3 * 37, 70, 0, 50)
    call(gpu_ctx, "nrs_concat_write", s, out, 3 * 37, 70, 50, 20)
    assert np.array_equal(out.get(), np.concatenate([x.reshape(-1, 50), s.get()], 1))
    part = Dev(gpu_ctx, shape=(3 * 37, 20))
    call(gpu_ctx, "nrs_concat_read", out, part, 3 * 37, 70, 50, 20, 0)
    assert np.array_equal(part.get(), s.get())


def test_permute_heads(gpu_ctx, oracle32):
    """Head split = the reference's per-head column slices stacked along the batch
    (src/nn/multihead.rs:94-107); merge = its concat_cols; both bit-exact, merge(split(x)) == x."""
    rng = np.random.default_rng(12)
    b, s, h, dh = 3, 7, 4, 5
    x = rng.normal(size=(b, s, h * dh)).astype(np.float32)
    heads = Dev(gpu_ctx, shape=(b * h, s, dh))
    call(gpu_ctx, "nrs_permute_heads", Dev(gpu_ctx, x), heads, b, s, h, dh, 1, 0)
    want = np.stack([oracle32.slice_cols_fwd(x.reshape(-1, h * dh), k * dh, (k + 1) * dh).reshape(b, s, dh)
                     for k in range(h)], axis=1).reshape(b * h, s, dh)
    assert np.array_equal(heads.get(), want)
    back = Dev(gpu_ctx, shape=x.shape)
    call(gpu_ctx, "nrs_permute_heads", heads, back, b, s, h, dh, 0, 0)
    assert np.array_equal(back.get(), x)
    call(gpu_ctx, "nrs_permute_heads", heads, back, b, s, h, dh, 0, 1)   # accumulate
    assert np.array_equal(back.get(), 2 * x)


def test_bounded_wait_times_out_and_context_survives(gpu_ctx):
    """A device wait that runs out is reported as NRS_ERR_TIMEOUT at the next sync; nothing faults,
    and the context keeps working afterwards."""
    l = _lib.lib()
    assert l.nrs_selftest_bounded_wait(gpu_ctx.h, 200000) == 0           # ~0.1 ms on a barrier nobody completes
    assert l.nrs_sync(gpu_ctx.h) == 6                                     # NRS_ERR_TIMEOUT
    assert b"bounded wait" in l.nrs_last_error(gpu_ctx.h)
    assert l.nrs_sync(gpu_ctx.h) == 0                                     # the error word was consumed
    a = np.arange(12, dtype=np.float32).reshape(3, 4)
    out = Dev(gpu_ctx, shape=(3, 3))
    call(gpu_ctx, "nrs_gemm", 0, 1, 3, 3, 4, Dev(gpu_ctx, a), Dev(gpu_ctx, a), out, None, 0, 0.0)
    assert np.allclose(out.get(), a @ a.T)
