"""Committed fixtures under tests/golden/:

* reference_vectors.json — known-answer vectors the reference's own tests assert (each with its file:line); the CPU
  oracle must reproduce them, and so must the device through the C ABI;
* seeded_fixtures.npz — seeded inputs and the f64 oracle's outputs for the hot-path operators at small sizes; the
  oracle must still reproduce them (a regression pin of the oracle itself), and the device must match them within
  the math mode's bar.
"""
import ctypes as C
import json
from pathlib import Path

import numpy as np
import pytest

from .conftest import rel_l2

GOLDEN = Path(__file__).resolve().parent / "golden"
CASES = json.loads((GOLDEN / "reference_vectors.json").read_text())["cases"]
F = C.c_float


def _fx():
    return np.load(GOLDEN / "seeded_fixtures.npz")


def _arr(case, key):
    return np.asarray(case[key], np.float32).reshape(case[key + "_shape"]) if key + "_shape" in case else np.asarray(case[key], np.float32)


# ---------------------------------------------------------------------------------------------- CPU: the oracle

@pytest.mark.parametrize("case", CASES, ids=[c["source"] for c in CASES])
def test_oracle_reproduces_the_reference_vectors(case, oracle32, oracle64):
    for o in (oracle32, oracle64):
        op = case["op"]
        if op == "conv2d_fwd":
            y = o.conv2d_fwd(_arr(case, "x"), _arr(case, "w"), np.asarray(case["b"], np.float32), case["stride"], case["pad"])
            assert list(y.shape) == case["y_shape"] and y.ravel().tolist() == [float(v) for v in case["y"]]
        elif op == "maxpool":
            x = _arr(case, "x")
            y, am = o.maxpool_fwd(x, case["k"], case["stride"])
            assert y.ravel().tolist() == [float(v) for v in case["y"]]
            gx = o.maxpool_bwd(np.asarray(case["gy"], np.float32).reshape(y.shape), am, x.shape)
            assert gx.ravel().tolist() == [float(v) for v in case["gx"]]
        elif op == "batchnorm_running_mean":
            x = _arr(case, "x")
            c = x.shape[1]
            _, _, _, rm, _ = o.batchnorm_fwd(x, np.ones(c, np.float32), np.zeros(c, np.float32),
                                             np.asarray(case["running_mean0"], np.float32),
                                             np.asarray(case["running_var0"], np.float32), 1e-5, case["momentum"], True)
            assert np.abs(rm - np.asarray(case["running_mean"])).max() < case["tolerance"]
        elif op == "embedding_fwd":
            y = o.embedding_fwd(_arr(case, "w"), case["idx"])
            assert y.ravel().tolist() == [float(v) for v in case["y"]]
        elif op == "embedding_bwd":
            gw = o.embedding_bwd(np.asarray(case["gy"], np.float32).reshape(len(case["idx"]), case["dim"]), case["idx"], case["vocab"])
            assert gw.ravel().tolist() == [float(v) for v in case["gw"]]
        elif op == "positional_table":
            pe = o.positional_table(case["rows"], case["d_model"])
            assert np.abs(pe[0] - np.asarray(case["first_row"])).max() < 1e-5
            assert abs(pe[1, 0] - np.sin(case["row1_dim0_is_sin_of"])) < case["tolerance"]
        elif op == "matmul":
            assert o.matmul_fwd(_arr(case, "a"), _arr(case, "b")).ravel().tolist() == [float(v) for v in case["y"]]
        elif op == "linear":
            x = _arr(case, "x")
            y = o.bias_add_fwd(o.matmul_fwd(x, _arr(case, "w")), np.asarray(case["b"], np.float32))
            assert y.ravel().tolist() == [float(v) for v in case["y"]]
            _, gb = o.bias_add_bwd(np.asarray(case["gy"], np.float32).reshape(y.shape))
            assert gb.ravel().tolist() == [float(v) for v in case["gb"]]
        elif op == "slice_cols":
            x = _arr(case, "x")
            assert o.slice_cols_fwd(x, case["c0"], case["c1"]).ravel().tolist() == [float(v) for v in case["y"]]
            assert o.slice_cols_fwd(x, case["c1"], case["c2"]).ravel().tolist() == [float(v) for v in case["right"]]
        elif op == "relu_bwd":
            gx = o.relu_bwd(np.asarray(case["x"], np.float32), np.asarray(case["gy"], np.float32))
            assert gx.ravel().tolist() == [float(v) for v in case["gx"]]
        else:
            raise AssertionError(f"unknown op {op}")


def test_oracle_still_reproduces_the_seeded_fixtures(oracle64):
    o, fx = oracle64, _fx()
    close = lambda got, key: rel_l2(got, fx[key]) <= 1e-6
    assert close(o.conv2d_fwd(fx["conv_x"], fx["conv_w"], fx["conv_b"], 1, 1), "conv_y")
    dx, dw, db = o.conv2d_bwd(fx["conv_x"], fx["conv_w"], fx["conv_dy"], 1, 1)
    assert close(dx, "conv_dx") and close(dw, "conv_dw") and close(db, "conv_db")
    assert close(o.matmul_fwd(fx["mm_a"], fx["mm_b"]), "mm_c")
    da, dbm = o.matmul_bwd(fx["mm_a"], fx["mm_b"], fx["mm_dc"])
    assert close(da, "mm_da") and close(dbm, "mm_db")
    y, xhat, istd = o.layernorm_fwd(fx["ln_x"], fx["ln_gamma"], fx["ln_beta"], 1e-5)
    assert close(y, "ln_y") and close(xhat, "ln_xhat") and close(istd, "ln_istd")
    ldx, ldg, ldb = o.layernorm_bwd(fx["ln_gy"], fx["ln_xhat"], fx["ln_istd"], fx["ln_gamma"])
    assert close(ldx, "ln_dx") and close(ldg, "ln_dgamma") and close(ldb, "ln_dbeta")
    sy = o.softmax_fwd(fx["sm_x"])
    assert close(sy, "sm_y") and close(o.softmax_bwd(fx["sm_y"], fx["sm_g"]), "sm_dx")
    assert abs(o.ce_fwd(fx["ce_logits"], fx["ce_target"]) - float(fx["ce_loss"])) <= 1e-6
    assert close(o.ce_bwd(fx["ce_logits"], fx["ce_target"]), "ce_grad")
    py, pam = o.maxpool_fwd(fx["pool_x"], 2, 2)
    assert np.array_equal(py, fx["pool_y"]) and np.array_equal(pam, fx["pool_argmax"])
    assert np.array_equal(o.maxpool_bwd(fx["pool_gy"], pam, fx["pool_x"].shape), fx["pool_dx"])
    assert close(o.gelu_fwd(fx["gelu_x"]), "gelu_y") and close(o.gelu_bwd(fx["gelu_x"], fx["gelu_g"]), "gelu_dx")
    p, m, v = fx["adamw_p0"].copy(), np.zeros(200, np.float32), np.zeros(200, np.float32)
    for t in range(3):
        o.adamw_step(p, fx["adamw_grads"][t], m, v, 1e-3, 0.9, 0.999, 1e-8, 1e-4, t)
    assert close(p, "adamw_p3") and close(m, "adamw_m3") and close(v, "adamw_v3")


# ---------------------------------------------------------------------------------------------- GPU: the device

_DEVICE_OPS = ("conv2d_fwd", "maxpool", "matmul", "linear", "relu_bwd")


@pytest.mark.gpu
@pytest.mark.parametrize("case", [c for c in CASES if c["op"] in _DEVICE_OPS],
                         ids=[c["source"] for c in CASES if c["op"] in _DEVICE_OPS])
def test_device_reproduces_the_reference_vectors(case, gpu_ctx):
    from .gpu_util import Dev, call
    if case["op"] == "matmul":
        a, b = _arr(case, "a"), _arr(case, "b")
        c = Dev(gpu_ctx, shape=(a.shape[0], b.shape[1]))
        call(gpu_ctx, "nrs_gemm", 0, 0, a.shape[0], b.shape[1], a.shape[1], Dev(gpu_ctx, a), Dev(gpu_ctx, b), c, None, 0, F(0))
        assert c.get().ravel().tolist() == [float(v) for v in case["y"]]
    elif case["op"] == "linear":
        x, w = _arr(case, "x"), _arr(case, "w")
        y = Dev(gpu_ctx, shape=(x.shape[0], w.shape[1]))
        call(gpu_ctx, "nrs_gemm", 0, 0, x.shape[0], w.shape[1], x.shape[1], Dev(gpu_ctx, x), Dev(gpu_ctx, w), y,
             Dev(gpu_ctx, np.asarray(case["b"], np.float32)), 0, F(0))
        assert y.get().ravel().tolist() == [float(v) for v in case["y"]]
        gb = Dev(gpu_ctx, shape=(w.shape[1],))
        call(gpu_ctx, "nrs_sum_axis0", Dev(gpu_ctx, np.asarray(case["gy"], np.float32)), gb, x.shape[0], w.shape[1], 0)
        assert gb.get().ravel().tolist() == [float(v) for v in case["gb"]]
    elif case["op"] == "relu_bwd":
        gx = Dev(gpu_ctx, shape=(len(case["x"]),))
        call(gpu_ctx, "nrs_relu_bwd", Dev(gpu_ctx, np.asarray(case["x"], np.float32)), Dev(gpu_ctx, np.asarray(case["gy"], np.float32)),
             gx, C.c_size_t(len(case["x"])), 0)
        assert gx.get().ravel().tolist() == [float(v) for v in case["gx"]]
    elif case["op"] == "conv2d_fwd":
        x, w = _arr(case, "x"), _arr(case, "w")
        n, ci, h, wd = x.shape
        co, _, kh, kw = w.shape
        y = Dev(gpu_ctx, shape=case["y_shape"])
        call(gpu_ctx, "nrs_conv2d_fwd", Dev(gpu_ctx, x), Dev(gpu_ctx, w), Dev(gpu_ctx, np.asarray(case["b"], np.float32)), y,
             n, ci, h, wd, co, kh, kw, case["stride"], case["pad"], 0)
        assert y.get().ravel().tolist() == [float(v) for v in case["y"]]
    else:
        x = _arr(case, "x")
        n, c, h, w = x.shape
        y, am = Dev(gpu_ctx, shape=case["y_shape"]), Dev(gpu_ctx, shape=case["y_shape"], dtype=np.int32)
        call(gpu_ctx, "nrs_maxpool_fwd", Dev(gpu_ctx, x), y, am, n, c, h, w, case["k"], case["stride"])
        assert y.get().ravel().tolist() == [float(v) for v in case["y"]]
        gx = Dev(gpu_ctx, shape=x.shape)
        call(gpu_ctx, "nrs_maxpool_bwd", Dev(gpu_ctx, np.asarray(case["gy"], np.float32)), am, gx, n, c, h, w, case["k"],
             case["stride"], 0)
        assert gx.get().ravel().tolist() == [float(v) for v in case["gx"]]


@pytest.mark.gpu
@pytest.mark.parametrize("mode,tol", [(0, 1e-4), (2, 1e-4), (1, 1e-2)], ids=["3xtf32", "fp32", "tf32"])
def test_device_matches_the_seeded_fixtures(gpu_ctx, mode, tol):
    from .gpu_util import Dev, call
    fx = _fx()
    D = lambda key: Dev(gpu_ctx, fx[key])
    gpu_ctx.set_math_mode(mode)
    try:
        # convolution: forward, and the three gradients from one call
        y = Dev(gpu_ctx, shape=fx["conv_y"].shape)
        dims = (2, 32, 8, 8, 32, 3, 3, 1, 1)
        call(gpu_ctx, "nrs_conv2d_fwd", D("conv_x"), D("conv_w"), D("conv_b"), y, *dims, 0)
        assert rel_l2(y.get(), fx["conv_y"]) <= tol
        dx, dw, db = (Dev(gpu_ctx, shape=fx[k].shape) for k in ("conv_dx", "conv_dw", "conv_db"))
        call(gpu_ctx, "nrs_conv2d_bwd", D("conv_x"), D("conv_w"), D("conv_dy"), dx, dw, db, *dims, 0)
        assert rel_l2(dx.get(), fx["conv_dx"]) <= tol and rel_l2(dw.get(), fx["conv_dw"]) <= tol
        assert rel_l2(db.get(), fx["conv_db"]) <= 1e-5
        # matmul and both gradients
        c = Dev(gpu_ctx, shape=(32, 32))
        call(gpu_ctx, "nrs_gemm", 0, 0, 32, 32, 64, D("mm_a"), D("mm_b"), c, None, 0, F(0))
        assert rel_l2(c.get(), fx["mm_c"]) <= tol
        da, dbm = Dev(gpu_ctx, shape=(32, 64)), Dev(gpu_ctx, shape=(64, 32))
        call(gpu_ctx, "nrs_gemm", 0, 1, 32, 64, 32, D("mm_dc"), D("mm_b"), da, None, 0, F(0))
        call(gpu_ctx, "nrs_gemm", 1, 0, 64, 32, 32, D("mm_a"), D("mm_dc"), dbm, None, 0, F(0))
        assert rel_l2(da.get(), fx["mm_da"]) <= tol and rel_l2(dbm.get(), fx["mm_db"]) <= tol
    finally:
        gpu_ctx.set_math_mode(0)
    if mode != 0:
        return          # the rest is exact-f32 arithmetic in every mode
    ly, lxhat, listd = Dev(gpu_ctx, shape=(8, 64)), Dev(gpu_ctx, shape=(8, 64)), Dev(gpu_ctx, shape=(8,))
    call(gpu_ctx, "nrs_layernorm_fwd", D("ln_x"), D("ln_gamma"), D("ln_beta"), ly, lxhat, listd, 8, 64, F(1e-5))
    assert rel_l2(ly.get(), fx["ln_y"]) <= 1e-5 and rel_l2(lxhat.get(), fx["ln_xhat"]) <= 1e-5
    ldx, ldg, ldb = Dev(gpu_ctx, shape=(8, 64)), Dev(gpu_ctx, shape=(64,)), Dev(gpu_ctx, shape=(64,))
    call(gpu_ctx, "nrs_layernorm_bwd", D("ln_gy"), D("ln_xhat"), D("ln_istd"), D("ln_gamma"), ldx, ldg, ldb, 8, 64, 0, 0)
    assert rel_l2(ldx.get(), fx["ln_dx"]) <= 1e-5 and rel_l2(ldg.get(), fx["ln_dgamma"]) <= 1e-5
    assert rel_l2(ldb.get(), fx["ln_dbeta"]) <= 1e-5
    sy, sdx = Dev(gpu_ctx, shape=(8, 128)), Dev(gpu_ctx, shape=(8, 128))
    call(gpu_ctx, "nrs_softmax_fwd", D("sm_x"), sy, 8, 128)
    call(gpu_ctx, "nrs_softmax_bwd", D("sm_y"), D("sm_g"), sdx, 8, 128, 0)
    assert rel_l2(sy.get(), fx["sm_y"]) <= 1e-5 and rel_l2(sdx.get(), fx["sm_dx"]) <= 1e-5
    loss, grad = Dev(gpu_ctx, shape=(1,)), Dev(gpu_ctx, shape=(16, 20))
    call(gpu_ctx, "nrs_ce_fwd_bwd", D("ce_logits"), D("ce_target"), loss, grad, 16, 20, 16)
    assert abs(float(loss.get()[0]) - float(fx["ce_loss"])) <= 1e-5 and rel_l2(grad.get(), fx["ce_grad"]) <= 1e-5
    py, pam = Dev(gpu_ctx, shape=fx["pool_y"].shape), Dev(gpu_ctx, shape=fx["pool_y"].shape, dtype=np.int32)
    call(gpu_ctx, "nrs_maxpool_fwd", D("pool_x"), py, pam, 2, 4, 8, 8, 2, 2)
    assert np.array_equal(py.get(), fx["pool_y"]) and np.array_equal(pam.get(), fx["pool_argmax"])   # integer output: bit-exact
    pdx = Dev(gpu_ctx, shape=fx["pool_x"].shape)
    call(gpu_ctx, "nrs_maxpool_bwd", D("pool_gy"), pam, pdx, 2, 4, 8, 8, 2, 2, 0)
    assert np.array_equal(pdx.get(), fx["pool_dx"])
    gy, gdx = Dev(gpu_ctx, shape=(256,)), Dev(gpu_ctx, shape=(256,))
    call(gpu_ctx, "nrs_gelu_fwd", D("gelu_x"), gy, C.c_size_t(256))
    call(gpu_ctx, "nrs_gelu_bwd", D("gelu_x"), D("gelu_g"), gdx, C.c_size_t(256), 0)
    assert rel_l2(gy.get(), fx["gelu_y"]) <= 1e-5 and rel_l2(gdx.get(), fx["gelu_dx"]) <= 1e-5
    p, m, v = Dev(gpu_ctx, fx["adamw_p0"]), Dev(gpu_ctx, np.zeros(200, np.float32)), Dev(gpu_ctx, np.zeros(200, np.float32))
    for t in range(3):
        bc1, bc2 = 1.0 - 0.9 ** (t + 1), 1.0 - 0.999 ** (t + 1)
        call(gpu_ctx, "nrs_adamw_step", p, Dev(gpu_ctx, fx["adamw_grads"][t]), m, v, C.c_size_t(200), F(1e-3), F(0.9), F(0.999),
             F(1e-8), F(1e-4), F(bc1), F(bc2), F(1.0))
    assert rel_l2(p.get(), fx["adamw_p3"]) <= 1e-5 and rel_l2(m.get(), fx["adamw_m3"]) <= 1e-5
    assert rel_l2(v.get(), fx["adamw_v3"]) <= 1e-5
