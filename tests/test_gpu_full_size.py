"""The benchmark configurations at FULL size, where the CPU oracle would take minutes to hours:
parity is checked through properties that do not depend on the size —

* batch independence: a slice of the full-batch result equals the oracle run on that slice alone;
* the adjoint identities <conv(x,w), dy> = <x, dgrad(dy,w)> = <w, wgrad(x,dy)>, which tie the three
  convolution kernels to one another (and, through the slice check, to the oracle);
* linearity in the input;
* additivity of the training step over a split of the batch (gradients and loss of the whole batch
  are the means of the halves');
* run-to-run determinism (bit-identical weight gradients, losses and parameter gradients).

Tolerance: 1e-4 relative in 3xTF32 (the default mode), as for the small cases."""
import numpy as np
import pytest

from neuralrs_b200 import _lib, cuda
from oracle import models
from .conftest import rel_l2
from .gpu_util import Dev, call

pytestmark = pytest.mark.gpu


def dot(a, b):
    return float(np.dot(np.asarray(a, np.float64).ravel(), np.asarray(b, np.float64).ravel()))


def test_conv_microbench_full_size_properties(gpu_ctx, oracle64):
    """The conv microbenchmark configuration: x[256,64,32,32], w[128,64,3,3], stride 1, pad 1."""
    n, ci, h, w, co = 256, 64, 32, 32, 128
    rng = np.random.default_rng(1236)
    x = rng.standard_normal((n, ci, h, w), dtype=np.float32)
    x2 = rng.standard_normal((n, ci, h, w), dtype=np.float32)
    wt = (rng.standard_normal((co, ci, 3, 3), dtype=np.float32) * np.sqrt(2.0 / (ci * 9))).astype(np.float32)
    b = (rng.standard_normal(co, dtype=np.float32) * 0.1).astype(np.float32)
    dy = rng.standard_normal((n, co, h, w), dtype=np.float32)
    dims = (n, ci, h, w, co, 3, 3, 1, 1)
    dX, dX2, dW, dB, dDY = Dev(gpu_ctx, x), Dev(gpu_ctx, x2), Dev(gpu_ctx, wt), Dev(gpu_ctx, b), Dev(gpu_ctx, dy)
    zero_b = Dev(gpu_ctx, np.zeros(co, np.float32))
    y = Dev(gpu_ctx, shape=dy.shape)
    call(gpu_ctx, "nrs_conv2d_fwd", dX, dW, dB, y, *dims, 0)
    y_full = y.get()
    # batch independence: two images of the full-batch result against the oracle on those two alone
    for sl in (slice(0, 2), slice(n - 2, n)):
        ref = oracle64.conv2d_fwd(x[sl], wt, b, 1, 1)
        assert rel_l2(y_full[sl], ref) <= 1e-4
    # linearity in x (bias off)
    call(gpu_ctx, "nrs_conv2d_fwd", dX, dW, zero_b, y, *dims, 0)
    y1 = y.get()
    call(gpu_ctx, "nrs_conv2d_fwd", dX2, dW, zero_b, y, *dims, 0)
    y2 = y.get()
    xs = Dev(gpu_ctx, x + x2)
    call(gpu_ctx, "nrs_conv2d_fwd", xs, dW, zero_b, y, *dims, 0)
    assert rel_l2(y.get(), y1 + y2) <= 1e-4
    # adjoint identities
    gx, gw, gb = Dev(gpu_ctx, shape=x.shape), Dev(gpu_ctx, shape=wt.shape), Dev(gpu_ctx, shape=b.shape)
    call(gpu_ctx, "nrs_conv2d_bwd", dX, dW, dDY, gx, gw, gb, *dims, 0)
    lhs = dot(y1, dy)
    assert abs(dot(x, gx.get()) - lhs) <= 1e-4 * abs(lhs)
    assert abs(dot(wt, gw.get()) - lhs) <= 1e-4 * abs(lhs)
    assert rel_l2(gb.get(), dy.sum(axis=(0, 2, 3), dtype=np.float64)) <= 1e-5
    # data gradient: batch independence against the oracle
    ref_dx, _, _ = oracle64.conv2d_bwd(x[:2], wt, dy[:2], 1, 1)
    assert rel_l2(gx.get()[:2], ref_dx) <= 1e-4
    # the weight gradient (a reduction over 262144 pixels split across CTAs) is deterministic
    first = gw.get().copy()
    gw2 = Dev(gpu_ctx, shape=wt.shape)
    call(gpu_ctx, "nrs_conv2d_bwd", dX, dW, dDY, None, gw2, None, *dims, 0)
    assert np.array_equal(gw2.get(), first)


def test_vgg_full_batch_step_properties(gpu_ctx):
    """The headline configuration: the VGG-style CNN at batch 1024.  The whole-batch loss and gradients are the
    means of the two half-batch ones (cross-entropy averages over the batch), and two runs from the
    same state agree bit for bit."""
    cfg = models.VGG_CIFAR
    hp = models.ADAMW_HP
    params = models.he_init(cfg["layers"], 1237)
    x, t = models.synthetic_batch(cfg, 1024, 1238)

    def grads_of(xb, tb):
        tr = cuda.Trainer(cfg["layers"], cfg["in_shape"], cfg["classes"], hp["lr"], hp["beta1"], hp["beta2"], hp["eps"],
                          hp["wd"], fuse=True, ctx=gpu_ctx)
        tr.set_params(params)
        loss = tr.forward_backward(xb, tb)
        g = [tr.get_grad(i).copy() for i in range(len(params))]
        tr.close()
        return loss, g

    loss_full, g_full = grads_of(x, t)
    loss_again, g_again = grads_of(x, t)
    assert loss_full == loss_again
    assert all(np.array_equal(a, b) for a, b in zip(g_full, g_again))
    loss_a, g_a = grads_of(x[:512], t[:512])
    loss_b, g_b = grads_of(x[512:], t[512:])
    assert abs(loss_full - 0.5 * (loss_a + loss_b)) <= 1e-5 * abs(loss_full)
    for gf, ga, gb in zip(g_full, g_a, g_b):
        assert rel_l2(gf, 0.5 * (ga + gb)) <= 1e-4


def test_wide_mlp_layer_full_size_properties(gpu_ctx, oracle64):
    """The wide-MLP configuration's hidden layer at full size: [16384, 4096] x [4096, 4096] with bias and GELU."""
    m, k, n = 16384, 4096, 4096
    rng = np.random.default_rng(1239)
    a = rng.standard_normal((m, k), dtype=np.float32)
    wt = (rng.standard_normal((k, n), dtype=np.float32) / np.sqrt(k)).astype(np.float32)
    bias = (rng.standard_normal(n, dtype=np.float32) * 0.1).astype(np.float32)
    dA, dW, dB = Dev(gpu_ctx, a), Dev(gpu_ctx, wt), Dev(gpu_ctx, bias)
    out = Dev(gpu_ctx, shape=(m, n))
    call(gpu_ctx, "nrs_gemm", 0, 0, m, n, k, dA, dW, out, dB, _lib.ACT_GELU, 0.0)
    got = out.get()
    # row independence: a few rows against the oracle's matmul + bias + GELU on those rows alone
    rows = np.array([0, 1, 777, m - 1])
    ref = oracle64.gelu_fwd(oracle64.matmul_fwd(a[rows], wt) + bias)
    assert rel_l2(got[rows], ref) <= 1e-4
    # the products behind dX = dY W^T and dW = X^T dY satisfy <X W, dY> = <X, dY W^T> = <W, X^T dY>
    dy = rng.standard_normal((m, n), dtype=np.float32)
    dDY = Dev(gpu_ctx, dy)
    call(gpu_ctx, "nrs_gemm", 0, 0, m, n, k, dA, dW, out, None, _lib.ACT_NONE, 0.0)
    lhs = dot(out.get(), dy)
    gx = Dev(gpu_ctx, shape=(m, k))
    call(gpu_ctx, "nrs_gemm", 0, 1, m, k, n, dDY, dW, gx, None, _lib.ACT_NONE, 0.0)
    assert abs(dot(a, gx.get()) - lhs) <= 1e-4 * abs(lhs)
    gw = Dev(gpu_ctx, shape=(k, n))
    call(gpu_ctx, "nrs_gemm", 1, 0, k, n, m, dA, dDY, gw, None, _lib.ACT_NONE, 0.0)
    assert abs(dot(wt, gw.get()) - lhs) <= 1e-4 * abs(lhs)
    first = gw.get().copy()
    call(gpu_ctx, "nrs_gemm", 1, 0, k, n, m, dA, dDY, gw, None, _lib.ACT_NONE, 0.0)
    assert np.array_equal(gw.get(), first)


@pytest.mark.parametrize("shape", [(256, 64, 32, 32, 128), (1024, 64, 32, 32, 64)],
                         ids=["conv_microbench", "vgg_64to64_at_32x32_batch_1024"])
def test_full_size_weight_gradient_slices_against_the_oracle(gpu_ctx, oracle64, shape):
    """The weight gradient at the benchmark's own sizes, compared DIRECTLY with the oracle: dW[oc] depends only
    on dy[:, oc], so the oracle computes a few output channels' slices (under 3 GFLOP) while the device computes
    the whole tensor — a dropped split, a mis-ordered tap at a row-split boundary or any other error that the
    scalar identity <w, dW> = <y, dy> cannot see shows up here.  Bias gradient likewise."""
    n, ci, h, w, co = shape
    rng = np.random.default_rng(n + co)
    x = rng.standard_normal((n, ci, h, w), dtype=np.float32)
    dy = rng.standard_normal((n, co, h, w), dtype=np.float32)
    wt = np.zeros((co, ci, 3, 3), np.float32)          # not read by the weight gradient
    dims = (n, ci, h, w, co, 3, 3, 1, 1)
    gw, gb = Dev(gpu_ctx, shape=wt.shape), Dev(gpu_ctx, shape=(co,))
    call(gpu_ctx, "nrs_conv2d_bwd", Dev(gpu_ctx, x), Dev(gpu_ctx, wt), Dev(gpu_ctx, dy), None, gw, gb, *dims, 0)
    got_w, got_b = gw.get(), gb.get()
    ocs = [0, co // 2 + 1, co - 1]
    _, ref_w, ref_b = oracle64.conv2d_bwd(x, wt[ocs], np.ascontiguousarray(dy[:, ocs]), 1, 1, need_dx=False)
    for k, oc in enumerate(ocs):
        assert rel_l2(got_w[oc], ref_w[k]) <= 1e-4, f"dW[{oc}]"
        # every tap of every input channel, not only the tensor's norm
        assert np.abs(got_w[oc] - ref_w[k]).max() <= 1e-4 * np.abs(ref_w[k]).max(), f"dW[{oc}] elementwise"
    assert rel_l2(got_b[ocs], ref_b) <= 1e-5
