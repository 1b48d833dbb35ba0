"""Pins the CPU oracle (oracle/nrs_oracle.c) to the reference.

The reference crate cannot be built here (no Rust toolchain), so the pins are the
known-answer vectors its own tests assert, replayed verbatim, plus analytic
checks (finite differences as in the reference's gradcheck tests, and an
independent float64 restatement in numpy/torch).
"""
import numpy as np
import pytest

from .conftest import rel_l2


@pytest.mark.parametrize("acc", ["f32", "f64"])
def test_conv_forward_known_answers(acc):
    from oracle.nrs_oracle import Oracle
    o = Oracle(acc)
    # tests/nn_conv_test.rs:7-36 -> [12,16,24,28]
    x = np.arange(1, 10, dtype=np.float32).reshape(1, 1, 3, 3)
    y = o.conv2d_fwd(x, np.ones((1, 1, 2, 2), np.float32), np.zeros(1, np.float32), 1, 0)
    assert y.shape == (1, 1, 2, 2)
    assert y.ravel().tolist() == [12.0, 16.0, 24.0, 28.0]
    # tests/nn_conv_test.rs:39-70 -> [36,72]
    w = np.array([1] * 8 + [2] * 8, np.float32).reshape(2, 2, 2, 2)
    x = np.arange(1, 9, dtype=np.float32).reshape(1, 2, 2, 2)
    y = o.conv2d_fwd(x, w, np.zeros(2, np.float32), 1, 0)
    assert y.shape == (1, 2, 1, 1)
    assert y.ravel().tolist() == [36.0, 72.0]
    # tests/nn_conv_padding_test.rs:9-35 -> [4,6,4,6,9,6,4,6,4]
    y = o.conv2d_fwd(np.ones((1, 1, 3, 3), np.float32), np.ones((1, 1, 3, 3), np.float32), np.zeros(1, np.float32), 1, 1)
    assert y.ravel().tolist() == [4, 6, 4, 6, 9, 6, 4, 6, 4]


@pytest.mark.parametrize("acc", ["f32", "f64"])
def test_maxpool_known_answers(acc):
    from oracle.nrs_oracle import Oracle
    o = Oracle(acc)
    # tests/nn_maxpool_test.rs:7-42
    x = np.arange(1, 17, dtype=np.float32).reshape(1, 1, 4, 4)
    y, am = o.maxpool_fwd(x, 2, 2)
    assert y.ravel().tolist() == [6.0, 8.0, 14.0, 16.0]
    dx = o.maxpool_bwd(np.ones(4, np.float32), am, x.shape)
    assert dx.ravel().tolist() == [0, 0, 0, 0, 0, 1, 0, 1, 0, 0, 0, 0, 0, 1, 0, 1]
    # strict '>' : the FIRST maximum of a window wins (src/nn/maxpool.rs:51)
    y, am = o.maxpool_fwd(np.full((1, 1, 2, 2), 3.0, np.float32), 2, 2)
    assert am.ravel().tolist() == [0]


def test_linear_known_answer(oracle32):
    # tests/nn_linear_test.rs: identity weights, input [3,-2]
    y = oracle32.bias_add_fwd(oracle32.matmul_fwd([[3.0, -2.0]], [[1, 0], [0, 1]]), [0.0, 0.0])
    assert y.ravel().tolist() == [3.0, -2.0]
    da, db = oracle32.matmul_bwd([[3.0, -2.0]], [[1, 0], [0, 1]], [[1.0, 1.0]])
    assert da.ravel().tolist() == [1.0, 1.0]
    assert db.ravel().tolist() == [3.0, 3.0, -2.0, -2.0]


def test_softmax_known_properties(oracle32):
    # tests/autograd_softmax_test.rs: rows sum to 1, ordering preserved
    y = oracle32.softmax_fwd(np.array([[1.0, 2.0, 3.0], [0.0, 0.0, 0.0]], np.float32))
    assert np.allclose(y.sum(1), 1.0, atol=1e-6)
    assert y[0, 0] < y[0, 1] < y[0, 2]
    assert np.allclose(y[1], 1 / 3, atol=1e-6)


def test_layernorm_row_statistics(oracle32):
    # tests/nn_layernorm_test.rs:17-32: with gamma=1, beta=0 each row has mean ~0 and variance ~1
    rng = np.random.default_rng(0)
    x = rng.normal(2.0, 3.0, (5, 16)).astype(np.float32)
    y, xhat, istd = oracle32.layernorm_fwd(x, np.ones(16), np.zeros(16), 1e-5)
    assert np.abs(y.mean(1)).max() < 1e-5
    assert np.abs(y.var(1) - 1).max() < 1e-3


def _conv_np64(x, w, b, stride, pad):
    n, ci, h, wd = x.shape
    co, _, kh, kw = w.shape
    xp = np.zeros((n, ci, h + 2 * pad, wd + 2 * pad))
    xp[:, :, pad:pad + h, pad:pad + wd] = x
    oh, ow = (h + 2 * pad - kh) // stride + 1, (wd + 2 * pad - kw) // stride + 1
    y = np.zeros((n, co, oh, ow))
    for i in range(kh):
        for j in range(kw):
            patch = xp[:, :, i:i + stride * oh:stride, j:j + stride * ow:stride]
            y += np.einsum("nchw,oc->nohw", patch, w[:, :, i, j].astype(np.float64))
    return y + b.reshape(1, -1, 1, 1)


@pytest.mark.parametrize("cfg", [(2, 3, 8, 8, 4, 3, 3, 1, 1), (2, 3, 7, 7, 5, 3, 3, 1, 1), (3, 2, 9, 6, 4, 2, 3, 2, 1)])
def test_conv_against_independent_float64(cfg, oracle32, oracle64):
    n, ci, h, wd, co, kh, kw, s, p = cfg
    # input formulas of tests/cuda_conv2d_test.rs:21-23
    x = (np.arange(n * ci * h * wd) % 23 * 0.05 - 0.5).astype(np.float32).reshape(n, ci, h, wd)
    w = (np.arange(co * ci * kh * kw) % 13 * 0.07 - 0.4).astype(np.float32).reshape(co, ci, kh, kw)
    b = (np.arange(co) % 5 * 0.1 - 0.2).astype(np.float32)
    ref = _conv_np64(x.astype(np.float64), w, b.astype(np.float64), s, p)
    assert np.abs(oracle64.conv2d_fwd(x, w, b, s, p) - ref).max() < 1e-6
    assert np.abs(oracle32.conv2d_fwd(x, w, b, s, p) - ref).max() < 1e-4   # bar of cuda_conv2d_test.rs:40
    # backward against torch autograd in float64
    import torch
    import torch.nn.functional as F
    xt = torch.tensor(x, dtype=torch.float64, requires_grad=True)
    wt = torch.tensor(w, dtype=torch.float64, requires_grad=True)
    bt = torch.tensor(b, dtype=torch.float64, requires_grad=True)
    yt = F.conv2d(xt, wt, bt, stride=s, padding=p)
    seed = (np.arange(yt.numel()) % 7 * 0.2 + 0.1).astype(np.float32).reshape(yt.shape)   # cuda_conv2d_test.rs:66
    yt.backward(torch.tensor(seed, dtype=torch.float64))
    # f64 sums are rounded once to f32 on output: 1e-6 relative; f32 sums: the
    # reference's own absolute bar of 1e-3 (cuda_conv2d_test.rs:87-93)
    for o, tol, rel in ((oracle64, 1e-6, True), (oracle32, 1e-3, False)):
        dx, dw, db = o.conv2d_bwd(x, w, seed, s, p)
        for got, ref in ((dx, xt.grad.numpy()), (dw, wt.grad.numpy()), (db, bt.grad.numpy())):
            scale = max(1.0, np.abs(ref).max()) if rel else 1.0
            assert np.abs(got - ref).max() < tol * scale


def test_conv_gradcheck_like_reference(oracle64):
    # tests/gradcheck_conv_test.rs: loss = sum (i+1)*out_i, central differences h=1e-3, tol 1e-2..5e-2
    rng = np.random.default_rng(1)
    x = rng.normal(size=(1, 2, 5, 5)).astype(np.float32)
    w = rng.normal(size=(3, 2, 3, 3)).astype(np.float32) * 0.3
    b = rng.normal(size=3).astype(np.float32) * 0.1
    y = oracle64.conv2d_fwd(x, w, b, 1, 1)
    coeff = (np.arange(y.size) + 1).astype(np.float32).reshape(y.shape)
    dx, dw, db = oracle64.conv2d_bwd(x, w, coeff, 1, 1)
    h = 1e-3
    for idx in [(0, 0, 0, 0), (0, 1, 2, 3), (0, 0, 4, 4)]:
        xp, xm = x.copy(), x.copy()
        xp[idx] += h
        xm[idx] -= h
        num = ((oracle64.conv2d_fwd(xp, w, b, 1, 1) - oracle64.conv2d_fwd(xm, w, b, 1, 1)) * coeff).sum() / (2 * h)
        assert abs(num - dx[idx]) < 5e-2 * max(1.0, abs(num))
    for idx in [(0, 0, 0, 0), (2, 1, 2, 2)]:
        wp, wm = w.copy(), w.copy()
        wp[idx] += h
        wm[idx] -= h
        num = ((oracle64.conv2d_fwd(x, wp, b, 1, 1) - oracle64.conv2d_fwd(x, wm, b, 1, 1)) * coeff).sum() / (2 * h)
        assert abs(num - dw[idx]) < 5e-2 * max(1.0, abs(num))


def test_matmul_bmm_against_numpy(oracle32, oracle64):
    m, k, n = 40, 56, 32   # tests/cuda_matmul_resident_test.rs:10-13
    a = (np.arange(m * k) % 13 * 0.1 - 0.6).astype(np.float32).reshape(m, k)
    b = (np.arange(k * n) % 7 * 0.2 - 0.6).astype(np.float32).reshape(k, n)
    seed = (np.arange(m * n) % 5 * 0.2 + 0.1).astype(np.float32).reshape(m, n)
    a64, b64, s64 = a.astype(np.float64), b.astype(np.float64), seed.astype(np.float64)
    for o, tol in ((oracle64, 1e-6), (oracle32, 1e-3)):
        assert np.abs(o.matmul_fwd(a, b) - a64 @ b64).max() < tol
        da, db = o.matmul_bwd(a, b, seed)
        assert np.abs(da - s64 @ b64.T).max() < tol
        assert np.abs(db - a64.T @ s64).max() < tol
    rng = np.random.default_rng(2)
    A, B = rng.normal(size=(3, 5, 4)).astype(np.float32), rng.normal(size=(3, 4, 6)).astype(np.float32)
    G = rng.normal(size=(3, 5, 6)).astype(np.float32)
    assert np.abs(oracle64.bmm_fwd(A, B) - np.einsum("bmk,bkn->bmn", A.astype(np.float64), B)).max() < 1e-6
    dA, dB = oracle64.bmm_bwd(A, B, G)
    assert np.abs(dA - np.einsum("bmn,bkn->bmk", G.astype(np.float64), B)).max() < 1e-6
    assert np.abs(dB - np.einsum("bmk,bmn->bkn", A.astype(np.float64), G)).max() < 1e-6


def test_ce_against_torch(oracle32, oracle64):
    import torch
    # tests/cuda_ce_test.rs:12-19 shapes; target one-hot at b % classes
    batch, classes = 16, 10
    rng = np.random.default_rng(3)
    logits = rng.normal(size=(batch, classes)).astype(np.float32) * 3
    target = np.zeros((batch, classes), np.float32)
    target[np.arange(batch), np.arange(batch) % classes] = 1
    lt = torch.tensor(logits, dtype=torch.float64, requires_grad=True)
    loss = -(torch.tensor(target, dtype=torch.float64) * torch.log_softmax(lt, 1)).sum() / batch
    loss.backward()
    for o, tol in ((oracle64, 1e-6), (oracle32, 1e-5)):
        assert abs(o.ce_fwd(logits, target) - loss.item()) < tol
        assert np.abs(o.ce_bwd(logits, target) - lt.grad.numpy()).max() < tol
    # a data-parallel shard divides by the global batch
    half = oracle64.ce_fwd(logits[:8], target[:8], divisor=16) + oracle64.ce_fwd(logits[8:], target[8:], divisor=16)
    assert abs(half - loss.item()) < 1e-6


def test_adamw_against_closed_form(oracle32):
    # tests/cuda_adamw_test.rs:11-15: 10 steps, constant gradient; compare with a float64 restatement
    n = 256
    p = (np.arange(n) % 17 * 0.1 - 0.8).astype(np.float32)
    g = (np.arange(n) % 11 * 0.05 - 0.25).astype(np.float32)
    lr, b1, b2, eps, wd = 0.001, 0.9, 0.999, 1e-8, 0.01
    m, v = np.zeros(n, np.float32), np.zeros(n, np.float32)
    p64, m64, v64 = p.astype(np.float64), np.zeros(n), np.zeros(n)
    for t in range(10):
        oracle32.adamw_step(p, g, m, v, lr, b1, b2, eps, wd, t)
        m64 = b1 * m64 + (1 - b1) * g
        v64 = b2 * v64 + (1 - b2) * g.astype(np.float64) ** 2
        mh, vh = m64 / (1 - b1 ** (t + 1)), v64 / (1 - b2 ** (t + 1))
        p64 = p64 - lr * mh / (np.sqrt(vh) + eps) - lr * wd * p64
    assert np.abs(p - p64).max() < 1e-4     # bar of cuda_adamw_test.rs:35


def test_gelu_relu_layernorm_softmax_backward_against_torch(oracle64):
    import torch
    rng = np.random.default_rng(4)
    x = rng.normal(size=(6, 12)).astype(np.float32)
    g = rng.normal(size=(6, 12)).astype(np.float32)
    xt = torch.tensor(x, dtype=torch.float64, requires_grad=True)
    gt = torch.tensor(g, dtype=torch.float64)
    # gelu (tanh form; src/autograd/graph/gelu.rs)
    torch.nn.functional.gelu(xt, approximate="tanh").backward(gt)
    assert np.abs(oracle64.gelu_fwd(x) - torch.nn.functional.gelu(xt, approximate="tanh").detach().numpy()).max() < 1e-6
    assert np.abs(oracle64.gelu_bwd(x, g) - xt.grad.numpy()).max() < 1e-5
    xt.grad = None
    torch.relu(xt).backward(gt)
    assert np.abs(oracle64.relu_bwd(x, g) - xt.grad.numpy()).max() == 0
    xt.grad = None
    # layernorm
    gamma = rng.normal(size=12).astype(np.float32)
    beta = rng.normal(size=12).astype(np.float32)
    gm = torch.tensor(gamma, dtype=torch.float64, requires_grad=True)
    bt = torch.tensor(beta, dtype=torch.float64, requires_grad=True)
    torch.nn.functional.layer_norm(xt, (12,), gm, bt, 1e-5).backward(gt)
    y, xhat, istd = oracle64.layernorm_fwd(x, gamma, beta, 1e-5)
    assert np.abs(y - torch.nn.functional.layer_norm(xt, (12,), gm, bt, 1e-5).detach().numpy()).max() < 1e-5
    dx, dg, db = oracle64.layernorm_bwd(g, xhat, istd, gamma)
    assert np.abs(dx - xt.grad.numpy()).max() < 1e-5
    assert np.abs(dg - gm.grad.numpy()).max() < 1e-5
    assert np.abs(db - bt.grad.numpy()).max() < 1e-5
    xt.grad = None
    # softmax
    torch.softmax(xt, 1).backward(gt)
    ys = oracle64.softmax_fwd(x)
    assert np.abs(oracle64.softmax_bwd(ys, g) - xt.grad.numpy()).max() < 1e-6
    assert rel_l2(oracle64.transpose_fwd(x), x.T) == 0


def test_fast_cpu_kernels_match_the_naive_ones(oracle32):
    """The reference's fast forward kernels (matmul_simd, conv2d_im2col), restated for the timed CPU
    baseline, replaying the reference's own tests of them."""
    from oracle import nrs_oracle as no
    # tests/matmul_simd_test.rs:6-29 (tolerance 1e-3)
    m, k, n = 5, 11, 7
    a = ((np.arange(m * k) % 9).astype(np.float32) - 4.0) * np.float32(0.3)
    b = ((np.arange(k * n) % 6).astype(np.float32) - 2.0) * np.float32(0.25)
    naive = oracle32.matmul_fwd(a.reshape(m, k), b.reshape(k, n))
    assert np.abs(no.matmul_simd(a.reshape(m, k), b.reshape(k, n)) - naive).max() < 1e-3
    # tests/im2col_conv_test.rs:10-54 (tolerance 1e-4)
    nb, ci, co, h, w = 2, 2, 3, 5, 5
    wt = ((np.arange(co * ci * 9) % 7).astype(np.float32) - 3.0) * np.float32(0.1)
    bias = np.arange(co, dtype=np.float32) * np.float32(0.5)
    x = ((np.arange(nb * ci * h * w) % 11).astype(np.float32) - 5.0) * np.float32(0.2)
    direct = oracle32.conv2d_fwd(x.reshape(nb, ci, h, w), wt.reshape(co, ci, 3, 3), bias, 1, 1)
    fast = no.conv2d_im2col(x.reshape(nb, ci, h, w), wt.reshape(co, ci, 3, 3), bias, 1, 1)
    assert fast.shape == direct.shape and np.abs(fast - direct).max() < 1e-4
    # the known answers of tests/nn_conv_test.rs and nn_conv_padding_test.rs hold for the fast path too
    y = no.conv2d_im2col(np.arange(1, 10, dtype=np.float32).reshape(1, 1, 3, 3), np.ones((1, 1, 2, 2), np.float32),
                         np.zeros(1, np.float32), 1, 0)
    assert y.ravel().tolist() == [12.0, 16.0, 24.0, 28.0]
    y = no.conv2d_im2col(np.ones((1, 1, 3, 3), np.float32), np.ones((1, 1, 3, 3), np.float32), np.zeros(1, np.float32), 1, 1)
    assert y.ravel().tolist() == [4, 6, 4, 6, 9, 6, 4, 6, 4]
    # thread control used by the timed baselines
    cores = no.host_cores()
    no.set_threads(1)
    assert no.get_threads() == 1
    no.set_threads(cores)
    assert no.get_threads() == cores
