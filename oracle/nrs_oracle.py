"""numpy/ctypes front end of the CPU oracle (oracle/nrs_oracle.c).

TEST INFRASTRUCTURE ONLY: imported by tests/, by __graft_entry__.smoke() and by
bench.py's CPU-baseline legs as the checker / the timed CPU baseline.  Nothing
in the neuralrs_b200 package imports it.

``Oracle("f32")`` accumulates in f32 in the reference's loop order,
``Oracle("f64")`` carries the sums in f64 (the "true value" for the error bars).
Every method follows the reference function cited beside the C routine it calls.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
LIB = HERE / "libnrs_oracle.so"
_lib = None


def build(force: bool = False) -> Path:
    src = HERE / "nrs_oracle.c"
    if force or not LIB.exists() or LIB.stat().st_mtime < src.stat().st_mtime:
        env = dict(os.environ)
        env.pop("CC", None)
        subprocess.run(["make", "-C", str(HERE), "-s"], check=True, env=env)
    return LIB


def _load():
    global _lib
    if _lib is None:
        build()
        _lib = C.CDLL(str(LIB))
    return _lib


def host_cores() -> int:
    return int(_load().nrs_oracle_host_cores())


def get_threads() -> int:
    return int(_load().nrs_oracle_get_threads())


def set_threads(n: int) -> None:
    """Threads of the OpenMP loops (the reference's Rayon pools); overrides OMP_NUM_THREADS."""
    _load().nrs_oracle_set_threads(int(n))


def matmul_simd(a, b):
    """matmul_simd (src/ops/simd.rs:42-77): the reference's AVX2 + Rayon forward matmul."""
    a, b = _f(a), _f(b)
    m, k = a.shape
    n = b.shape[1]
    c = np.empty((m, n), np.float32)
    _load().nrs_oracle_matmul_simd(_p(a), _p(b), _p(c), m, k, n)
    return c


def conv2d_im2col(x, w, b, stride=1, pad=0):
    """conv2d_im2col (src/ops/im2col.rs:59-98): the reference's im2col + matmul forward convolution."""
    x, w, b = _f(x), _f(w), _f(b)
    n, ci, h, wd = x.shape
    co, _, kh, kw = w.shape
    oh, ow = (h + 2 * pad - kh) // stride + 1, (wd + 2 * pad - kw) // stride + 1
    y = np.empty((n, co, oh, ow), np.float32)
    _load().nrs_oracle_conv2d_im2col(_p(x), _p(w), _p(b), _p(y), n, ci, h, wd, co, kh, kw, stride, pad)
    return y


def _f(a):
    return np.ascontiguousarray(np.asarray(a, dtype=np.float32))


def _p(a):
    return C.c_void_p(a.ctypes.data) if a is not None else None


class Oracle:
    def __init__(self, acc: str = "f64"):
        assert acc in ("f32", "f64")
        self.sfx = "_" + acc
        self.l = _load()

    def _fn(self, name, restype=None):
        f = getattr(self.l, name + self.sfx)
        f.restype = restype
        return f

    # ---- conv (src/nn/conv.rs:33-203)
    def conv2d_fwd(self, x, w, b, stride=1, pad=0):
        x, w, b = _f(x), _f(w), _f(b)
        n, ci, h, wd = x.shape
        co, _, kh, kw = w.shape
        oh, ow = (h + 2 * pad - kh) // stride + 1, (wd + 2 * pad - kw) // stride + 1
        y = np.empty((n, co, oh, ow), np.float32)
        self._fn("nrs_oracle_conv2d_fwd")(_p(x), _p(w), _p(b), _p(y), n, ci, h, wd, co, kh, kw, stride, pad)
        return y

    def conv2d_bwd(self, x, w, dy, stride=1, pad=0, need_dx=True):
        x, w, dy = _f(x), _f(w), _f(dy)
        n, ci, h, wd = x.shape
        co, _, kh, kw = w.shape
        dx = np.zeros_like(x) if need_dx else None
        dw = np.zeros_like(w)
        db = np.zeros(co, np.float32)
        self._fn("nrs_oracle_conv2d_bwd")(_p(x), _p(w), _p(dy), _p(dx), _p(dw), _p(db), n, ci, h, wd, co, kh, kw,
                                          stride, pad)
        return dx, dw, db

    # ---- matmul / bmm (src/autograd/graph/matmul.rs:12-66, bmm.rs:13-96)
    def matmul_fwd(self, a, b):
        a, b = _f(a), _f(b)
        m, k = a.shape
        n = b.shape[1]
        c = np.empty((m, n), np.float32)
        self._fn("nrs_oracle_matmul_fwd")(_p(a), _p(b), _p(c), m, k, n)
        return c

    def matmul_bwd(self, a, b, dc):
        a, b, dc = _f(a), _f(b), _f(dc)
        m, k = a.shape
        n = b.shape[1]
        da, db = np.zeros_like(a), np.zeros_like(b)
        self._fn("nrs_oracle_matmul_bwd")(_p(a), _p(b), _p(dc), _p(da), _p(db), m, k, n)
        return da, db

    def bmm_fwd(self, a, b):
        a, b = _f(a), _f(b)
        bt, m, k = a.shape
        n = b.shape[2]
        c = np.empty((bt, m, n), np.float32)
        self._fn("nrs_oracle_bmm_fwd")(_p(a), _p(b), _p(c), bt, m, k, n)
        return c

    def bmm_bwd(self, a, b, dc):
        a, b, dc = _f(a), _f(b), _f(dc)
        bt, m, k = a.shape
        n = b.shape[2]
        da, db = np.zeros_like(a), np.zeros_like(b)
        self._fn("nrs_oracle_bmm_bwd")(_p(a), _p(b), _p(dc), _p(da), _p(db), bt, m, k, n)
        return da, db

    # ---- add / bias (src/autograd/graph/add.rs:13-74)
    def add_fwd(self, a, b):
        a, b = _f(a), _f(b)
        out = np.empty_like(a)
        self._fn("nrs_oracle_add_fwd")(_p(a), _p(b), _p(out), C.c_size_t(a.size))
        return out

    def bias_add_fwd(self, a, bias):
        a, bias = _f(a), _f(bias)
        out = np.empty_like(a)
        self._fn("nrs_oracle_bias_add_fwd")(_p(a), _p(bias), _p(out), a.shape[0], a.shape[1])
        return out

    def bias_add_bwd(self, g):
        g = _f(g)
        da = np.zeros_like(g)
        db = np.zeros(g.shape[1], np.float32)
        self._fn("nrs_oracle_bias_add_bwd")(_p(g), _p(da), _p(db), g.shape[0], g.shape[1])
        return da, db

    # ---- activations (relu.rs:12-49, gelu.rs:9-60)
    def _unary(self, name, x):
        x = _f(x)
        y = np.empty_like(x)
        self._fn(name)(_p(x), _p(y), C.c_size_t(x.size))
        return y

    def _unary_bwd(self, name, x, g):
        x, g = _f(x), _f(g)
        dx = np.zeros_like(x)
        self._fn(name)(_p(x), _p(g), _p(dx), C.c_size_t(x.size))
        return dx

    def relu_fwd(self, x): return self._unary("nrs_oracle_relu_fwd", x)
    def relu_bwd(self, x, g): return self._unary_bwd("nrs_oracle_relu_bwd", x, g)
    def gelu_fwd(self, x): return self._unary("nrs_oracle_gelu_fwd", x)
    def gelu_bwd(self, x, g): return self._unary_bwd("nrs_oracle_gelu_bwd", x, g)

    # ---- maxpool (src/nn/maxpool.rs:20-82)
    def maxpool_fwd(self, x, k, stride):
        x = _f(x)
        n, c, h, w = x.shape
        oh, ow = (h - k) // stride + 1, (w - k) // stride + 1
        y = np.empty((n, c, oh, ow), np.float32)
        am = np.empty((n, c, oh, ow), np.int32)
        self._fn("nrs_oracle_maxpool_fwd")(_p(x), _p(y), _p(am), n, c, h, w, k, stride)
        return y, am

    def maxpool_bwd(self, g, argmax, in_shape):
        g = _f(g)
        am = np.ascontiguousarray(argmax, dtype=np.int32)
        dx = np.zeros(in_shape, np.float32)
        self._fn("nrs_oracle_maxpool_bwd")(_p(g), _p(am), _p(dx), C.c_size_t(g.size))
        return dx

    # ---- cross-entropy (src/nn/loss.rs:49-108)
    def ce_fwd(self, logits, target, divisor=None):
        logits, target = _f(logits), _f(target)
        b, c = logits.shape
        return float(self._fn("nrs_oracle_ce_fwd", C.c_float)(_p(logits), _p(target), b, c, divisor or b))

    def ce_bwd(self, logits, target, divisor=None):
        logits, target = _f(logits), _f(target)
        b, c = logits.shape
        g = np.empty_like(logits)
        self._fn("nrs_oracle_ce_bwd")(_p(logits), _p(target), _p(g), b, c, divisor or b)
        return g

    # ---- AdamW (src/optim/adamw.rs:23-46); updates p, m, v in place
    def adamw_step(self, p, g, m, v, lr, b1, b2, eps, wd, t):
        for a in (p, m, v):
            assert a.dtype == np.float32 and a.flags.c_contiguous
        g = _f(g)
        self._fn("nrs_oracle_adamw_step")(_p(p), _p(g), _p(m), _p(v), C.c_size_t(p.size), C.c_float(lr),
                                          C.c_float(b1), C.c_float(b2), C.c_float(eps), C.c_float(wd), int(t))

    # ---- layernorm (src/nn/normalization.rs:23-106)
    def layernorm_fwd(self, x, gamma, beta, eps):
        x, gamma, beta = _f(x), _f(gamma), _f(beta)
        f = x.shape[-1]
        rows = x.size // f
        y, xhat = np.empty_like(x), np.empty_like(x)
        istd = np.empty(rows, np.float32)
        self._fn("nrs_oracle_layernorm_fwd")(_p(x), _p(gamma), _p(beta), _p(y), _p(xhat), _p(istd), rows, f,
                                             C.c_float(eps))
        return y, xhat, istd

    def layernorm_bwd(self, g, xhat, istd, gamma):
        g, xhat, istd, gamma = _f(g), _f(xhat), _f(istd), _f(gamma)
        f = g.shape[-1]
        rows = g.size // f
        dx = np.zeros_like(g)
        dgamma, dbeta = np.zeros(f, np.float32), np.zeros(f, np.float32)
        self._fn("nrs_oracle_layernorm_bwd")(_p(g), _p(xhat), _p(istd), _p(gamma), _p(dx), _p(dgamma), _p(dbeta),
                                             rows, f)
        return dx, dgamma, dbeta

    # ---- batchnorm (src/nn/batchnorm.rs:28-150 with hw == 1, src/nn/batchnorm2d.rs:28-164)
    @staticmethod
    def _bn_dims(x):
        n, c = x.shape[0], x.shape[1]
        return n, c, x.size // (n * c)

    def batchnorm_fwd(self, x, gamma, beta, running_mean, running_var, eps, momentum, training):
        """Returns y, xhat, istd and the running statistics after the call (the inputs are not modified)."""
        x, gamma, beta = _f(x), _f(gamma), _f(beta)
        rm, rv = _f(running_mean).copy(), _f(running_var).copy()
        n, c, hw = self._bn_dims(x)
        y, xhat = np.empty_like(x), np.empty_like(x)
        istd = np.empty(c, np.float32)
        self._fn("nrs_oracle_batchnorm_fwd")(_p(x), _p(gamma), _p(beta), _p(rm), _p(rv), _p(y), _p(xhat), _p(istd),
                                             n, c, hw, C.c_float(eps), C.c_float(momentum), int(bool(training)))
        return y, xhat, istd, rm, rv

    def batchnorm_bwd(self, g, xhat, istd, gamma, training):
        g, xhat, istd, gamma = _f(g), _f(xhat), _f(istd), _f(gamma)
        n, c, hw = self._bn_dims(g)
        dx = np.zeros_like(g)
        dgamma, dbeta = np.zeros(c, np.float32), np.zeros(c, np.float32)
        self._fn("nrs_oracle_batchnorm_bwd")(_p(g), _p(xhat), _p(istd), _p(gamma), _p(dx), _p(dgamma), _p(dbeta),
                                             n, c, hw, int(bool(training)))
        return dx, dgamma, dbeta

    # ---- dropout (src/nn/dropout.rs:19-56, src/nn/dropout2d.rs; mask stream: the device library's own)
    def mask_mul(self, a, mask, hw=1):
        a, mask = _f(a), _f(mask)
        out = np.empty_like(a)
        self._fn("nrs_oracle_mask_mul")(_p(a), _p(mask), _p(out), C.c_size_t(a.size), int(hw), 0)
        return out

    def philox4x32_10(self, ctr, key):
        ctr = np.ascontiguousarray(ctr, np.uint32)
        key = np.ascontiguousarray(key, np.uint32)
        out = np.empty(4, np.uint32)
        self._fn("nrs_oracle_philox4x32_10")(_p(ctr), _p(key), _p(out))
        return out

    def dropout_mask(self, count, p, seed, offset=0):
        mask = np.empty(count, np.float32)
        self._fn("nrs_oracle_dropout_mask")(_p(mask), C.c_size_t(count), C.c_float(p), C.c_uint64(seed),
                                            C.c_uint64(offset))
        return mask

    # ---- input pipeline (examples/cifar_cuda.rs:148-169; draws: the device library's stream)
    def augment_image(self, img, flip, dx, dy):
        img = _f(img)
        c, h, w = img.shape
        out = np.empty_like(img)
        self._fn("nrs_oracle_augment_image")(_p(img), _p(out), c, h, w, int(flip), int(dx), int(dy))
        return out

    def augment_draw(self, seed, offset, index, max_shift):
        flip, dx, dy = C.c_int(), C.c_int(), C.c_int()
        self._fn("nrs_oracle_augment_draw")(C.c_uint64(seed), C.c_uint64(offset), C.c_uint64(index), int(max_shift),
                                            C.byref(flip), C.byref(dx), C.byref(dy))
        return flip.value, dx.value, dy.value

    def augment_batch(self, x, seed, offset, max_shift, flip=True):
        x = _f(x)
        out = np.empty_like(x)
        for i in range(x.shape[0]):
            f, dx, dy = self.augment_draw(seed, offset, i, max_shift)
            out[i] = self.augment_image(x[i], f and flip, dx, dy)
        return out

    # ---- softmax (src/autograd/graph/softmax.rs:14-64)
    def softmax_fwd(self, x):
        x = _f(x)
        w = x.shape[-1]
        y = np.empty_like(x)
        self._fn("nrs_oracle_softmax_fwd")(_p(x), _p(y), x.size // w, w)
        return y

    def softmax_bwd(self, y, g):
        y, g = _f(y), _f(g)
        w = y.shape[-1]
        dx = np.zeros_like(y)
        self._fn("nrs_oracle_softmax_bwd")(_p(y), _p(g), _p(dx), y.size // w, w)
        return dx

    # ---- manipulation (transpose.rs, scale.rs, slice_cols.rs, concat_cols.rs)
    def transpose_fwd(self, x):
        x = _f(x)
        rows, cols = x.shape[-2:]
        batch = x.size // (rows * cols)
        y = np.empty(x.shape[:-2] + (cols, rows), np.float32)
        self._fn("nrs_oracle_transpose_fwd")(_p(x), _p(y), batch, rows, cols)
        return y

    def slice_cols_fwd(self, x, c0, c1):
        x = _f(x)
        total = x.shape[-1]
        rows = x.size // total
        y = np.empty(x.shape[:-1] + (c1 - c0,), np.float32)
        self._fn("nrs_oracle_slice_cols_fwd")(_p(x), _p(y), rows, total, c0, c1)
        return y

    def slice_cols_bwd(self, g, in_shape, c0, c1):
        g = _f(g)
        total = in_shape[-1]
        dx = np.zeros(in_shape, np.float32)
        self._fn("nrs_oracle_slice_cols_bwd")(_p(g), _p(dx), dx.size // total, total, c0, c1)
        return dx

    # ---- embedding / positional encoding (src/nn/embedding.rs, src/nn/positional.rs)
    def embedding_fwd(self, weight, idx):
        weight = _f(weight)
        idx = np.ascontiguousarray(idx, dtype=np.int32).reshape(-1)
        out = np.empty((idx.size, weight.shape[1]), np.float32)
        self._fn("nrs_oracle_embedding_fwd")(_p(weight), _p(idx), _p(out), idx.size, weight.shape[1])
        return out

    def embedding_bwd(self, g, idx, vocab):
        g = _f(g)
        idx = np.ascontiguousarray(idx, dtype=np.int32).reshape(-1)
        dim = g.size // idx.size
        dw = np.zeros((vocab, dim), np.float32)
        self._fn("nrs_oracle_embedding_bwd")(_p(g), _p(idx), _p(dw), idx.size, dim, vocab)
        return dw

    def positional_table(self, max_len, d_model):
        pe = np.empty((max_len, d_model), np.float32)
        self._fn("nrs_oracle_positional_table")(_p(pe), max_len, d_model)
        return pe

    def transpose_bwd(self, g):
        # the gradient of a transpose is the transpose of the gradient (transpose.rs:45-52)
        return self.transpose_fwd(g)

    def scale_fwd(self, x, s):
        return (_f(x) * np.float32(s)).astype(np.float32)
