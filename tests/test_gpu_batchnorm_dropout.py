"""GPU parity of BatchNorm (1-D and 2-D) and Dropout / Dropout2d against the CPU oracle, through the raw
C-ABI operators and through the node-level API in the shape of the reference's tests/cuda_batchnorm_test.rs
and tests/cuda_dropout_test.rs.  Run with -m gpu on a B200."""
import ctypes as C

import numpy as np
import pytest

from neuralrs_b200 import _lib
from neuralrs_b200.cuda import Node, backward_graph, graph, nn
from neuralrs_b200.cuda import runtime as gpu
from .conftest import rel_l2
from .gpu_util import Dev, call

pytestmark = pytest.mark.gpu
F = C.c_float


def on_gpu(data, shape):
    n = Node.new(np.asarray(data, np.float32).ravel(), list(shape))
    gpu.to_cuda(n)
    return n


BN_SHAPES = [(16, 8, 1), (4, 3, 25), (3, 2, 1), (1, 5, 1), (2, 2, 4), (1024, 4096, 1), (300, 70, 1), (64, 32, 1024),
             (256, 64, 256), (33, 7, 49), (8, 512, 16), (5, 3, 2)]


@pytest.mark.parametrize("n,c,hw", BN_SHAPES)
@pytest.mark.parametrize("training", [True, False], ids=["train", "eval"])
def test_batchnorm_ops(gpu_ctx, oracle64, n, c, hw, training):
    rng = np.random.default_rng(n * 7 + c * 3 + hw)
    # per-channel offsets up to ~20 standard deviations: the raw-sum-of-squares cancellation case
    x = (rng.normal(size=(n, c, hw)) * rng.uniform(0.2, 3.0, size=(1, c, 1)) + rng.normal(size=(1, c, 1)) * 20).astype(np.float32)
    gamma, beta = rng.normal(1.0, 0.5, size=c).astype(np.float32), rng.normal(size=c).astype(np.float32)
    rm0, rv0 = rng.normal(size=c).astype(np.float32), rng.uniform(0.5, 2.0, size=c).astype(np.float32)
    g = rng.normal(size=(n, c, hw)).astype(np.float32)
    yr, xhr, isr, rmr, rvr = oracle64.batchnorm_fwd(x, gamma, beta, rm0, rv0, 1e-5, 0.9, training)
    dxr, dgr, dbr = oracle64.batchnorm_bwd(g, xhr, isr, gamma, training)

    dx_, dga, dbe, dg_ = Dev(gpu_ctx, x), Dev(gpu_ctx, gamma), Dev(gpu_ctx, beta), Dev(gpu_ctx, g)
    rm, rv = Dev(gpu_ctx, rm0), Dev(gpu_ctx, rv0)
    y, xh, ist = Dev(gpu_ctx, shape=x.shape), Dev(gpu_ctx, shape=x.shape), Dev(gpu_ctx, shape=(c,))
    call(gpu_ctx, "nrs_batchnorm_fwd", dx_, dga, dbe, rm, rv, y, xh, ist, n, c, hw, F(1e-5), F(0.9), int(training))
    if n * hw > 1 or not training:
        assert rel_l2(ist.get(), isr) <= 1e-5
        assert np.abs(xh.get() - xhr).max() <= 1e-4 * max(1.0, np.abs(xhr).max())
        assert np.abs(y.get() - yr).max() <= 1e-4 * max(1.0, np.abs(yr).max())   # bar of tests/cuda_batchnorm_test.rs:76
    assert np.abs(rm.get() - rmr).max() <= 1e-5 * max(1.0, np.abs(rmr).max())  # :79-80
    assert np.abs(rv.get() - rvr).max() <= 1e-5 * max(1.0, np.abs(rvr).max())
    # backward from the ORACLE's saved xhat/istd so that the two passes are checked independently
    xh_ref, ist_ref = Dev(gpu_ctx, xhr), Dev(gpu_ctx, isr)
    gx, gg, gb = Dev(gpu_ctx, shape=x.shape), Dev(gpu_ctx, shape=(c,)), Dev(gpu_ctx, shape=(c,))
    call(gpu_ctx, "nrs_batchnorm_bwd", dg_, xh_ref, ist_ref, dga, gx, gg, gb, n, c, hw, int(training), 0, 0)
    assert rel_l2(gg.get(), dgr) <= 1e-5
    assert rel_l2(gb.get(), dbr) <= 1e-5
    assert rel_l2(gx.get(), dxr) <= 1e-4
    # accumulate flags: a second call adds; parameter gradients alone (dx NULL) and dx alone
    call(gpu_ctx, "nrs_batchnorm_bwd", dg_, xh_ref, ist_ref, dga, gx, gg, gb, n, c, hw, int(training), 1, 1)
    assert rel_l2(gx.get(), 2 * dxr) <= 1e-4
    assert rel_l2(gg.get(), 2 * dgr) <= 1e-5
    gg2, gb2 = Dev(gpu_ctx, shape=(c,)), Dev(gpu_ctx, shape=(c,))
    call(gpu_ctx, "nrs_batchnorm_bwd", dg_, xh_ref, ist_ref, dga, None, gg2, gb2, n, c, hw, int(training), 0, 0)
    assert rel_l2(gb2.get(), dbr) <= 1e-5
    gx2 = Dev(gpu_ctx, shape=x.shape)
    call(gpu_ctx, "nrs_batchnorm_bwd", dg_, xh_ref, ist_ref, dga, gx2, None, None, n, c, hw, int(training), 0, 0)
    assert rel_l2(gx2.get(), dxr) <= 1e-4
    # bit-reproducible
    gx3 = Dev(gpu_ctx, shape=x.shape)
    call(gpu_ctx, "nrs_batchnorm_bwd", dg_, xh_ref, ist_ref, dga, gx3, None, None, n, c, hw, int(training), 0, 0)
    assert np.array_equal(gx3.get(), gx2.get())


def test_batchnorm_rejects_bad_arguments(gpu_ctx):
    l = _lib.lib()
    d = Dev(gpu_ctx, np.zeros(8, np.float32))
    assert l.nrs_batchnorm_fwd(gpu_ctx.h, d.ptr, d.ptr, d.ptr, d.ptr, d.ptr, d.ptr, d.ptr, d.ptr, 0, 2, 1, F(1e-5), F(0.9), 1) == 2
    assert l.nrs_batchnorm_fwd(gpu_ctx.h, None, d.ptr, d.ptr, d.ptr, d.ptr, d.ptr, d.ptr, d.ptr, 2, 2, 1, F(1e-5), F(0.9), 1) == 1
    assert l.nrs_batchnorm_bwd(gpu_ctx.h, d.ptr, d.ptr, d.ptr, d.ptr, d.ptr, d.ptr, None, 2, 2, 1, 1, 0, 0) == 1
    assert l.nrs_mask_mul(gpu_ctx.h, d.ptr, d.ptr, d.ptr, 7, 2, 0) == 2
    assert l.nrs_dropout_mask(gpu_ctx.h, d.ptr, 8, F(1.5)) == 1


def test_cuda_batchnorm_train_eval_backward(gpu_ctx, oracle32):
    # tests/cuda_batchnorm_test.rs:46-150: [16, 8] inputs, gamma/beta/seed formulas of the reference
    batch, features = 16, 8
    n = batch * features
    x = ((np.arange(n) * 13 + 5) % 47 * 0.1 - 2.0).astype(np.float32).reshape(batch, features)
    gamma = (0.5 + np.arange(features) % 4 * 0.3).astype(np.float32)
    beta = (np.arange(features) % 3 * 0.2 - 0.2).astype(np.float32)
    seed = (np.arange(n) % 9 * 0.15 + 0.05).astype(np.float32).reshape(batch, features)
    yr, xhr, isr, rmr, rvr = oracle32.batchnorm_fwd(x, gamma, beta, np.zeros(features), np.ones(features), 1e-5, 0.9, True)
    dxr, dgr, dbr = oracle32.batchnorm_bwd(seed, xhr, isr, gamma, True)
    gi, gg, gb = on_gpu(x, x.shape), on_gpu(gamma, [features]), on_gpu(beta, [features])
    rmean, rvar = on_gpu(np.zeros(features), [features]), on_gpu(np.ones(features), [features])
    gout = nn.batchnorm(gi, gg, gb, rmean, rvar, 0.9, 1e-5, True)
    assert np.abs(gpu.to_host(gout) - yr.ravel()).max() < 1e-4
    assert np.abs(gpu.to_host(rmean) - rmr).max() < 1e-5
    assert np.abs(gpu.to_host(rvar) - rvr).max() < 1e-5
    gpu.set_grad(gout, seed.ravel())
    backward_graph(gout)
    assert np.abs(gpu.read_grad(gg) - dgr).max() < 1e-3
    assert np.abs(gpu.read_grad(gb) - dbr).max() < 1e-3
    assert np.abs(gpu.read_grad(gi) - dxr.ravel()).max() < 1e-3
    # evaluation (:84-113): given running statistics, which stay as they are
    x2 = ((np.arange(n) * 9 + 1) % 31 * 0.1 - 1.5).astype(np.float32).reshape(batch, features)
    rm = (np.arange(features) % 5 * 0.1).astype(np.float32)
    rv = (0.5 + np.arange(features) % 3 * 0.2).astype(np.float32)
    yr2, _, _, _, _ = oracle32.batchnorm_fwd(x2, gamma, beta, rm, rv, 1e-5, 0.9, False)
    rmean2, rvar2 = on_gpu(rm, [features]), on_gpu(rv, [features])
    gout2 = nn.batchnorm(on_gpu(x2, x2.shape), gg, gb, rmean2, rvar2, 0.9, 1e-5, False)
    assert np.abs(gpu.to_host(gout2) - yr2.ravel()).max() < 1e-4
    assert np.array_equal(gpu.to_host(rmean2), rm) and np.array_equal(gpu.to_host(rvar2), rv)


def test_cuda_batchnorm2d_train_eval(gpu_ctx, oracle32):
    # tests/cuda_batchnorm_test.rs:155-232: [4, 3, 5, 5]
    shape = (4, 3, 5, 5)
    total, c = int(np.prod(shape)), shape[1]
    x = ((np.arange(total) * 13 + 5) % 47 * 0.1 - 2.0).astype(np.float32).reshape(shape)
    seed = (np.arange(total) % 9 * 0.15 + 0.05).astype(np.float32).reshape(shape)
    gamma = (0.5 + np.arange(c) % 4 * 0.3).astype(np.float32)
    beta = (np.arange(c) % 3 * 0.2 - 0.2).astype(np.float32)
    yr, xhr, isr, rmr, rvr = oracle32.batchnorm_fwd(x, gamma, beta, np.zeros(c), np.ones(c), 1e-5, 0.9, True)
    dxr, dgr, dbr = oracle32.batchnorm_bwd(seed, xhr, isr, gamma, True)
    gi, gg, gb = on_gpu(x, shape), on_gpu(gamma, [c]), on_gpu(beta, [c])
    rmean, rvar = on_gpu(np.zeros(c), [c]), on_gpu(np.ones(c), [c])
    gout = nn.batchnorm2d(gi, gg, gb, rmean, rvar, 0.9, 1e-5, True)
    assert gout.shape == list(shape)
    assert np.abs(gpu.to_host(gout) - yr.ravel()).max() < 1e-4
    gpu.set_grad(gout, seed.ravel())
    backward_graph(gout)
    assert np.abs(gpu.read_grad(gi) - dxr.ravel()).max() < 1e-3
    assert np.abs(gpu.to_host(rmean) - rmr).max() < 1e-5 and np.abs(gpu.to_host(rvar) - rvr).max() < 1e-5
    assert np.abs(gpu.read_grad(gg) - dgr).max() < 1e-3 and np.abs(gpu.read_grad(gb) - dbr).max() < 1e-3
    x2 = ((np.arange(total) * 9 + 1) % 31 * 0.1 - 1.5).astype(np.float32).reshape(shape)
    rm, rv = (np.arange(c) % 5 * 0.1).astype(np.float32), (0.5 + np.arange(c) % 3 * 0.2).astype(np.float32)
    yr2, _, _, _, _ = oracle32.batchnorm_fwd(x2, gamma, beta, rm, rv, 1e-5, 0.9, False)
    gout2 = nn.batchnorm2d(on_gpu(x2, shape), gg, gb, on_gpu(rm, [c]), on_gpu(rv, [c]), 0.9, 1e-5, False)
    assert np.abs(gpu.to_host(gout2) - yr2.ravel()).max() < 1e-4
    # wrong rank is refused like the reference's shape indexing would panic
    with pytest.raises(_lib.NrsError):
        nn.batchnorm2d(on_gpu(x2.reshape(4, 75), [4, 75]), gg, gb, rmean, rvar, 0.9, 1e-5, True)


def test_conv_batchnorm_relu_chain(gpu_ctx, oracle64):
    """conv -> BatchNorm2d -> ReLU, the block of the reference's examples/cifar_cuda.rs:44-48, against the oracle."""
    rng = np.random.default_rng(77)
    n, ci, co, h = 8, 32, 64, 16
    x = rng.normal(size=(n, ci, h, h)).astype(np.float32)
    w = (rng.normal(size=(co, ci, 3, 3)) * np.sqrt(2.0 / (ci * 9))).astype(np.float32)
    b = (rng.normal(size=co) * 0.1).astype(np.float32)
    gamma, beta = rng.normal(1.0, 0.2, size=co).astype(np.float32), (rng.normal(size=co) * 0.3).astype(np.float32)
    seed = rng.normal(size=(n, co, h, h)).astype(np.float32)
    z = oracle64.conv2d_fwd(x, w, b, 1, 1)
    yb, xh, ist, rmr, rvr = oracle64.batchnorm_fwd(z, gamma, beta, np.zeros(co), np.ones(co), 1e-5, 0.9, True)
    gi, gw, gbias = on_gpu(x, x.shape), on_gpu(w, w.shape), on_gpu(b, [co])
    gg, gb = on_gpu(gamma, [co]), on_gpu(beta, [co])
    rmean, rvar = on_gpu(np.zeros(co), [co]), on_gpu(np.ones(co), [co])
    bn = nn.batchnorm2d(nn.conv2d(gi, gw, gbias, 1, 1), gg, gb, rmean, rvar, 0.9, 1e-5, True)
    out = graph.relu(bn)
    got_bn = gpu.to_host(bn).reshape(yb.shape)
    assert rel_l2(got_bn, yb) <= 1e-4
    assert rel_l2(gpu.to_host(rvar), rvr) <= 1e-4
    gpu.set_grad(out, seed.ravel())
    backward_graph(out)
    # the oracle's backward with the DEVICE's ReLU mask (a pre-activation within rounding of zero may fall
    # on either side; the comparison is of the arithmetic, not of that coin flip)
    gmask = seed * (got_bn > 0)
    dz, dgr, dbr = oracle64.batchnorm_bwd(gmask, xh, ist, gamma, True)
    dxr, dwr, dbiasr = oracle64.conv2d_bwd(x, w, dz, 1, 1)
    assert rel_l2(gpu.read_grad(gg), dgr) <= 1e-4 and rel_l2(gpu.read_grad(gb), dbr) <= 1e-4
    assert rel_l2(gpu.read_grad(gw).reshape(w.shape), dwr) <= 1e-4
    assert rel_l2(gpu.read_grad(gi).reshape(x.shape), dxr) <= 1e-4
    # the conv bias sees a gradient that sums to ~0 per channel through BatchNorm: compare absolutely
    assert np.abs(gpu.read_grad(gbias) - dbiasr).max() <= 1e-3


@pytest.mark.parametrize("count,p", [(10000, 0.3), (7, 0.5), (1, 0.0), (4099, 1.0), (1 << 20, 0.1)])
def test_dropout_mask_matches_stream_definition(gpu_ctx, oracle32, count, p):
    """Bit-exact: the device mask is the stated function of (seed, offset), restated on the CPU."""
    l = _lib.lib()
    _lib.check(gpu_ctx.h, l.nrs_rng_seed(gpu_ctx.h, 0x1234567887654321))
    m = Dev(gpu_ctx, shape=(count,))
    call(gpu_ctx, "nrs_dropout_mask", m, count, F(p))
    assert np.array_equal(m.get(), oracle32.dropout_mask(count, p, 0x1234567887654321, 0))
    off = C.c_uint64()
    _lib.check(gpu_ctx.h, l.nrs_rng_offset(gpu_ctx.h, C.byref(off)))
    assert off.value == (count + 3) // 4
    # the next call continues the stream where this one stopped
    m2 = Dev(gpu_ctx, shape=(count,))
    call(gpu_ctx, "nrs_dropout_mask", m2, count, F(p))
    assert np.array_equal(m2.get(), oracle32.dropout_mask(count, p, 0x1234567887654321, off.value))


@pytest.mark.parametrize("total,hw", [(10000, 1), (10003, 1), (8 * 16 * 49, 49), (4 * 8 * 64, 64), (6, 2), (5, 1)])
def test_mask_mul(gpu_ctx, oracle32, total, hw):
    rng = np.random.default_rng(total + hw)
    a = rng.normal(size=total).astype(np.float32)
    mask = oracle32.dropout_mask(total // hw, 0.4, seed=total)
    want = oracle32.mask_mul(a, mask, hw)
    out = Dev(gpu_ctx, shape=(total,))
    call(gpu_ctx, "nrs_mask_mul", Dev(gpu_ctx, a), Dev(gpu_ctx, mask), out, total, hw, 0)
    assert np.array_equal(out.get(), want)                      # one multiply per element: bit-exact
    call(gpu_ctx, "nrs_mask_mul", Dev(gpu_ctx, a), Dev(gpu_ctx, mask), out, total, hw, 1)
    assert np.array_equal(out.get(), want + want)


def test_cuda_dropout_training_mechanics(gpu_ctx, oracle32):
    # tests/cuda_dropout_test.rs:8-36
    l = _lib.lib()
    n, p = 10000, 0.3
    scale = np.float32(1.0) / (np.float32(1.0) - np.float32(p))
    x = ((np.arange(n) % 50 + 1) * 0.1).astype(np.float32)
    seed = (np.arange(n) % 7 * 0.2 + 0.5).astype(np.float32)
    _lib.check(gpu_ctx.h, l.nrs_rng_seed(gpu_ctx.h, 99))
    gi = on_gpu(x, [n])
    gout = nn.dropout(gi, p, True)
    out = gpu.to_host(gout)
    gpu.set_grad(gout, seed)
    backward_graph(gout)
    igrad = gpu.read_grad(gi)
    dropped = out == 0
    assert np.abs(igrad[dropped]).max() < 1e-6
    assert np.abs(out[~dropped] - x[~dropped] * scale).max() < 1e-4
    assert np.abs(igrad[~dropped] - seed[~dropped] * scale).max() < 1e-4
    assert abs(dropped.mean() - p) < 0.05
    # and exactly the mask of the stated stream
    assert np.array_equal(out, x * oracle32.dropout_mask(n, p, 99, 0))
    # evaluation (:38-49): the very same node comes back
    ev = nn.dropout(gi, p, False)
    assert np.array_equal(gpu.to_host(ev), x)
    # a caller-supplied mask (the reference's host-drawn one) is used as given
    host_mask = np.where(np.arange(n) % 3 == 0, 0.0, scale).astype(np.float32)
    gi2 = on_gpu(x, [n])
    gout2 = nn.dropout(gi2, p, True, mask=on_gpu(host_mask, [n]))
    assert np.array_equal(gpu.to_host(gout2), x * host_mask)
    gpu.set_grad(gout2, seed)
    backward_graph(gout2)
    assert np.array_equal(gpu.read_grad(gi2), seed * host_mask)


def test_cuda_dropout2d_channel_mechanics(gpu_ctx, oracle32):
    # tests/cuda_dropout_test.rs:52-103
    l = _lib.lib()
    n, c, h, w, p = 8, 16, 7, 7, 0.4
    hw, total = h * w, n * c * h * w
    scale = np.float32(1.0) / (np.float32(1.0) - np.float32(p))
    x = ((np.arange(total) % 50 + 1) * 0.1).astype(np.float32)
    seed = (np.arange(total) % 7 * 0.2 + 0.5).astype(np.float32)
    _lib.check(gpu_ctx.h, l.nrs_rng_seed(gpu_ctx.h, 5))
    gi = on_gpu(x, [n, c, h, w])
    gout = nn.dropout2d(gi, p, True)
    out = gpu.to_host(gout).reshape(n * c, hw)
    gpu.set_grad(gout, seed)
    backward_graph(gout)
    igrad = gpu.read_grad(gi).reshape(n * c, hw)
    mask = oracle32.dropout_mask(n * c, p, 5, 0)
    assert np.array_equal(out, x.reshape(n * c, hw) * mask[:, None])
    assert np.array_equal(igrad, seed.reshape(n * c, hw) * mask[:, None])
    dropped = (out == 0).all(1)
    assert ((out == 0).any(1) == dropped).all()                # whole planes only
    assert abs(dropped.mean() - p) < 0.15
    assert np.abs(out[~dropped] - x.reshape(n * c, hw)[~dropped] * scale).max() < 1e-4
    ev = nn.dropout2d(gi, p, False)
    assert np.array_equal(gpu.to_host(ev), x)
    with pytest.raises(_lib.NrsError):
        nn.dropout2d(on_gpu(x, [total]), p, True)


@pytest.mark.parametrize("n,c,hw", [(16, 8, 1), (4, 3, 25), (64, 32, 64), (32, 64, 256), (128, 256, 16), (300, 70, 1)])
@pytest.mark.parametrize("training", [True, False], ids=["train", "eval"])
def test_batchnorm_with_fused_relu(gpu_ctx, oracle64, n, c, hw, training):
    """nrs_batchnorm_act_* with NRS_ACT_RELU against BatchNorm followed by ReLU in the oracle
    (src/autograd/graph/relu.rs:12-49: y = max(0, x), gradient passes where x > 0)."""
    rng = np.random.default_rng(n + c + hw)
    x = (rng.normal(size=(n, c, hw)) * 1.5 + rng.normal(size=(1, c, 1))).astype(np.float32)
    gamma, beta = rng.normal(1.0, 0.5, size=c).astype(np.float32), rng.normal(size=c).astype(np.float32)
    rm0, rv0 = rng.normal(size=c).astype(np.float32), rng.uniform(0.5, 2.0, size=c).astype(np.float32)
    g = rng.normal(size=(n, c, hw)).astype(np.float32)
    yr, xhr, isr, _, _ = oracle64.batchnorm_fwd(x, gamma, beta, rm0, rv0, 1e-5, 0.9, training)
    y, xh, ist = Dev(gpu_ctx, shape=x.shape), Dev(gpu_ctx, shape=x.shape), Dev(gpu_ctx, shape=(c,))
    dga, dbe = Dev(gpu_ctx, gamma), Dev(gpu_ctx, beta)
    call(gpu_ctx, "nrs_batchnorm_act_fwd", Dev(gpu_ctx, x), dga, dbe, Dev(gpu_ctx, rm0), Dev(gpu_ctx, rv0), y, xh, ist,
         n, c, hw, F(1e-5), F(0.9), int(training), _lib.ACT_RELU)
    got = y.get()
    assert (got >= 0).all()
    assert np.abs(got - oracle64.relu_fwd(yr)).max() <= 1e-4 * max(1.0, np.abs(yr).max())
    # outputs within rounding of zero may fall on either side of the ReLU: bound their share, then compare the
    # backward arithmetic under the device's own mask
    mask = got > 0
    assert ((yr > 0) != mask).mean() <= 1e-3
    dxr, dgr, dbr = oracle64.batchnorm_bwd(g * mask, xhr, isr, gamma, training)
    gx, gg, gb = Dev(gpu_ctx, shape=x.shape), Dev(gpu_ctx, shape=(c,)), Dev(gpu_ctx, shape=(c,))
    call(gpu_ctx, "nrs_batchnorm_act_bwd", Dev(gpu_ctx, g), xh, ist, dga, dbe, gx, gg, gb, n, c, hw, int(training), 0, 0,
         _lib.ACT_RELU)
    assert rel_l2(gg.get(), dgr) <= 1e-4 and rel_l2(gb.get(), dbr) <= 1e-4
    assert rel_l2(gx.get(), dxr) <= 1e-4
    # act = NONE is the plain pair of entry points, bit for bit
    y0, xh0, ist0 = Dev(gpu_ctx, shape=x.shape), Dev(gpu_ctx, shape=x.shape), Dev(gpu_ctx, shape=(c,))
    y1, xh1, ist1 = Dev(gpu_ctx, shape=x.shape), Dev(gpu_ctx, shape=x.shape), Dev(gpu_ctx, shape=(c,))
    call(gpu_ctx, "nrs_batchnorm_act_fwd", Dev(gpu_ctx, x), dga, dbe, Dev(gpu_ctx, rm0), Dev(gpu_ctx, rv0), y0, xh0, ist0,
         n, c, hw, F(1e-5), F(0.9), int(training), _lib.ACT_NONE)
    call(gpu_ctx, "nrs_batchnorm_fwd", Dev(gpu_ctx, x), dga, dbe, Dev(gpu_ctx, rm0), Dev(gpu_ctx, rv0), y1, xh1, ist1,
         n, c, hw, F(1e-5), F(0.9), int(training))
    assert np.array_equal(y0.get(), y1.get()) and np.array_equal(xh0.get(), xh1.get())


def test_batchnorm_act_graph_matches_separate_relu(gpu_ctx):
    """The fused node and batchnorm2d followed by a relu node agree bit for bit, forward and backward."""
    rng = np.random.default_rng(91)
    shape, c = (8, 16, 12, 12), 16
    x = rng.normal(size=shape).astype(np.float32)
    gamma, beta = rng.normal(1.0, 0.3, size=c).astype(np.float32), rng.normal(size=c).astype(np.float32)
    seed = rng.normal(size=shape).astype(np.float32)
    res = []
    for fused in (True, False):
        gi, gg, gb = on_gpu(x, shape), on_gpu(gamma, [c]), on_gpu(beta, [c])
        rm, rv = on_gpu(np.zeros(c), [c]), on_gpu(np.ones(c), [c])
        if fused:
            out = nn.batchnorm_act(gi, gg, gb, rm, rv, 0.9, 1e-5, True, _lib.ACT_RELU)
        else:
            out = graph.relu(nn.batchnorm2d(gi, gg, gb, rm, rv, 0.9, 1e-5, True))
        y = gpu.to_host(out)
        gpu.set_grad(out, seed.ravel())
        backward_graph(out)
        res.append((y, gpu.read_grad(gi), gpu.read_grad(gg), gpu.read_grad(gb), gpu.to_host(rm), gpu.to_host(rv)))
    for a, b in zip(*res):
        assert np.array_equal(a, b)
