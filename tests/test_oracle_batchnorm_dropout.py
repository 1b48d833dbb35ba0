"""Pins the oracle's BatchNorm / Dropout restatement to the reference: the known answers of the
reference's own tests (tests/nn_batchnorm_test.rs, tests/batchnorm_eval_test.rs,
tests/gradcheck_batchnorm2d_test.rs, tests/dropout2d_test.rs) and an independent float64 restatement.
The mask stream (Philox-4x32-10) is pinned to the published known-answer vectors of that generator; the
augmentation restatement (examples/cifar_cuda.rs:146-169) to hand-worked cases and the reference's draw ranges."""
import numpy as np
import pytest

from .conftest import rel_l2


def _oracle(acc):
    from oracle.nrs_oracle import Oracle
    return Oracle(acc)


@pytest.mark.parametrize("acc", ["f32", "f64"])
def test_batchnorm_known_answers(acc):
    o = _oracle(acc)
    ones, zeros = np.ones(2, np.float32), np.zeros(2, np.float32)
    # tests/nn_batchnorm_test.rs:7-31: gamma=1, beta=0 -> the output has mean ~0
    y, _, _, _, _ = o.batchnorm_fwd(np.array([[1, 2], [3, 4]], np.float32), ones, zeros, zeros, ones, 1e-5, 0.9, True)
    assert y.shape == (2, 2) and abs(float(y.mean())) < 1e-5
    # tests/batchnorm_eval_test.rs:22-36: one training step from (0, 1) with momentum 0.9 -> running mean [0.4, 2.0]
    x = np.array([[2, 10], [4, 20], [6, 30]], np.float32)
    _, _, _, rm, rv = o.batchnorm_fwd(x, ones, zeros, zeros, ones, 1e-5, 0.9, True)
    assert abs(rm[0] - 0.4) < 1e-4 and abs(rm[1] - 2.0) < 1e-4
    assert np.allclose(rv, 0.9 + 0.1 * x.var(0), atol=1e-5)          # biased variance
    # tests/batchnorm_eval_test.rs:38-56: five steps, then a single sample in evaluation mode stays finite
    for _ in range(4):
        _, _, _, rm, rv = o.batchnorm_fwd(x, ones, zeros, rm, rv, 1e-5, 0.9, True)
    y, _, _, rm2, rv2 = o.batchnorm_fwd(np.array([[4, 20]], np.float32), ones, zeros, rm, rv, 1e-5, 0.9, False)
    assert y.shape == (1, 2) and np.isfinite(y).all()
    assert np.array_equal(rm2, rm) and np.array_equal(rv2, rv)       # evaluation leaves the statistics alone
    assert np.allclose(y, (np.array([[4, 20]]) - rm) / np.sqrt(rv + 1e-5), atol=1e-5)


def _bn_ref64(x, gamma, beta, eps):
    """Independent float64 restatement: [n, c, *spatial], statistics over every axis but 1."""
    x = x.astype(np.float64)
    ax = tuple(i for i in range(x.ndim) if i != 1)
    sh = [1, -1] + [1] * (x.ndim - 2)
    m, v = x.mean(ax, keepdims=True), x.var(ax, keepdims=True)
    xh = (x - m) / np.sqrt(v + eps)
    return gamma.reshape(sh) * xh + beta.reshape(sh), xh, m.ravel(), v.ravel()


@pytest.mark.parametrize("shape", [(16, 8), (4, 3, 5, 5), (2, 2, 2, 2)])
def test_batchnorm_against_float64_and_finite_differences(shape):
    o = _oracle("f64")
    rng = np.random.default_rng(len(shape) * 10 + shape[0])
    c = shape[1]
    # inputs and parameters in the style of tests/cuda_batchnorm_test.rs:15-18,49
    x = ((np.arange(int(np.prod(shape))) * 13 + 5) % 47 * 0.1 - 2.0).astype(np.float32).reshape(shape)
    gamma = (0.5 + np.arange(c) % 4 * 0.3).astype(np.float32)
    beta = (np.arange(c) % 3 * 0.2 - 0.2).astype(np.float32)
    y, xhat, istd, rm, rv = o.batchnorm_fwd(x, gamma, beta, np.zeros(c), np.ones(c), 1e-5, 0.9, True)
    yr, xhr, m, v = _bn_ref64(x, gamma, beta, 1e-5)
    assert np.abs(y - yr).max() < 1e-5
    assert np.allclose(rm, 0.1 * m, atol=1e-6) and np.allclose(rv, 0.9 + 0.1 * v, atol=1e-6)
    # backward against central differences of L = sum(seed * y), as tests/gradcheck_batchnorm2d_test.rs:6-70 does
    seed = (np.arange(x.size) % 9 * 0.15 + 0.05).astype(np.float32).reshape(shape)
    dx, dgamma, dbeta = o.batchnorm_bwd(seed, xhat, istd, gamma, True)
    loss = lambda xx, gg, bb: float((seed.astype(np.float64) * _bn_ref64(xx, gg, bb, 1e-5)[0]).sum())
    h = 1e-3
    for idx in rng.choice(x.size, size=min(12, x.size), replace=False):
        xp, xm = x.astype(np.float64).copy(), x.astype(np.float64).copy()
        xp.flat[idx] += h
        xm.flat[idx] -= h
        num = (loss(xp, gamma, beta) - loss(xm, gamma, beta)) / (2 * h)
        assert abs(num - dx.flat[idx]) < 2e-2 * max(1.0, abs(num))      # the reference's own bar (:69)
    assert rel_l2(dgamma, (seed * xhr).sum(tuple(i for i in range(x.ndim) if i != 1))) < 1e-5
    assert rel_l2(dbeta, seed.astype(np.float64).sum(tuple(i for i in range(x.ndim) if i != 1))) < 1e-6
    # evaluation mode: dx = g * gamma * istd (src/nn/batchnorm2d.rs:144-153)
    dxe, _, _ = o.batchnorm_bwd(seed, xhat, istd, gamma, False)
    sh = [1, -1] + [1] * (x.ndim - 2)
    assert np.allclose(dxe, seed * (gamma * istd).reshape(sh), atol=1e-6)


def test_philox_known_answers():
    o = _oracle("f32")
    # known-answer vectors published with the generator (Random123 kat_vectors, philox4x32 with 10 rounds)
    kat = [([0, 0, 0, 0], [0, 0], [0x6627e8d5, 0xe169c58d, 0xbc57ac4c, 0x9b00dbd8]),
           ([0xffffffff] * 4, [0xffffffff] * 2, [0x408f276d, 0x41c83b0e, 0xa20bc7c6, 0x6d5451fd]),
           ([0x243f6a88, 0x85a308d3, 0x13198a2e, 0x03707344], [0xa4093822, 0x299f31d0],
            [0xd16cfe09, 0x94fdcceb, 0x5001e420, 0x24126ea1])]
    for ctr, key, want in kat:
        assert o.philox4x32_10(ctr, key).tolist() == want


def test_dropout_mask_and_routing():
    o = _oracle("f32")
    # tests/cuda_dropout_test.rs:8-36: n = 10000, p = 0.3: dropped share near p, survivors scaled by 1/(1-p)
    n, p = 10000, 0.3
    mask = o.dropout_mask(n, p, seed=7)
    scale = np.float32(1.0) / (np.float32(1.0) - np.float32(p))
    assert set(np.unique(mask).tolist()) == {0.0, float(scale)}
    assert abs(float((mask == 0).mean()) - p) < 0.05
    # a mask is a pure function of (seed, offset): a later window of the stream equals the tail of a longer one
    assert np.array_equal(o.dropout_mask(400, p, seed=7, offset=25), mask[100:500])
    assert not np.array_equal(o.dropout_mask(n, p, seed=8), mask)
    x = ((np.arange(n) % 50 + 1) * 0.1).astype(np.float32)
    out = o.mask_mul(x, mask)
    assert np.array_equal(out, x * mask)
    # tests/dropout2d_test.rs:15-45: p = 1 drops every channel, p = 0 keeps the input bit for bit
    x4 = np.arange(1, 9, dtype=np.float32).reshape(1, 2, 2, 2)
    assert np.array_equal(o.mask_mul(x4, o.dropout_mask(2, 1.0, seed=1), hw=4), np.zeros_like(x4))
    assert np.array_equal(o.mask_mul(x4, o.dropout_mask(2, 0.0, seed=1), hw=4), x4)
    # whole-channel masking (tests/cuda_dropout_test.rs:53-88): every pixel of a plane shares its factor
    m2 = o.dropout_mask(8 * 16, 0.4, seed=3)
    x2 = ((np.arange(8 * 16 * 49) % 50 + 1) * 0.1).astype(np.float32).reshape(8, 16, 7, 7)
    out2 = o.mask_mul(x2, m2, hw=49)
    assert np.array_equal(out2, x2 * m2.reshape(8, 16, 1, 1))
    assert abs(float((m2 == 0).mean()) - 0.4) < 0.15


def test_augment_draws_cover_the_reference_range():
    """examples/cifar_cuda.rs:150-152: flip with probability 1/2, dx and dy uniform over -4..=4."""
    draws = np.array([_oracle('f32').augment_draw(11, 0, i, 4) for i in range(4000)])
    assert abs(draws[:, 0].mean() - 0.5) < 0.05
    for col in (1, 2):
        vals, counts = np.unique(draws[:, col], return_counts=True)
        assert vals.tolist() == list(range(-4, 5))
        assert np.abs(counts / 4000 - 1 / 9).max() < 0.03


def test_augment_image_known_cases():
    img = np.arange(12, dtype=np.float32).reshape(1, 3, 4)
    assert np.array_equal(_oracle('f32').augment_image(img, 0, 0, 0), img)
    assert np.array_equal(_oracle('f32').augment_image(img, 1, 0, 0), img[:, :, ::-1])
    want = np.zeros_like(img)
    want[0, 1:, 1:] = img[0, :-1, :-1]                      # dx = dy = 1 moves the content right and down
    assert np.array_equal(_oracle('f32').augment_image(img, 0, 1, 1), want)
