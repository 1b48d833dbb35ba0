"""Whole-model CPU oracle: the reference's CPU training step restated over oracle/nrs_oracle.c.

TEST INFRASTRUCTURE ONLY (same rule as nrs_oracle.py).

A model is a list of layer tuples, applied in order, exactly as the reference's
``Sequential`` walks its ``Vec<Box<dyn Module>>`` (src/nn/sequential.rs:22-30):

    ("conv", c_in, c_out, k, stride, pad)   Conv2d          src/nn/conv.rs
    ("relu",) / ("gelu",)                    activations     src/autograd/graph/{relu,gelu}.rs
    ("maxpool", k, stride)                   MaxPool2d       src/nn/maxpool.rs
    ("flatten",)                             Flatten         src/nn/flatten.rs
    ("linear", n_in, n_out)                  Linear          src/nn/linear.rs (matmul + bias add)
    ("batchnorm", c)                         BatchNorm / BatchNorm2d  src/nn/batchnorm.rs, batchnorm2d.rs
                                             (momentum 0.9, eps 1e-5 as in examples/cifar_cuda.rs:44-48)
    ("dropout", p) / ("dropout2d", p)        Dropout / Dropout2d      src/nn/dropout.rs, dropout2d.rs

Parameters are a flat list [w0, b0, w1, b1, ...] in layer order — the order
``ADAMW::step`` flattens them in (src/optim/adamw.rs:48-54); a batchnorm layer adds
[gamma, beta].  Its running statistics are buffers, not parameters: a separate list
[mean0, var0, mean1, var1, ...] that training-mode forward passes update in place.
"""
from __future__ import annotations

import numpy as np

# The benchmark configurations (input shape without batch, layers, classes).
SMALL_CNN = dict(
    name="small_cnn", in_shape=(1, 28, 28), classes=10,
    layers=[("conv", 1, 32, 3, 1, 1), ("relu",), ("maxpool", 2, 2),
            ("conv", 32, 64, 3, 1, 1), ("relu",), ("maxpool", 2, 2),
            ("flatten",), ("linear", 3136, 128), ("relu",), ("linear", 128, 10)])

VGG_CIFAR = dict(
    name="vgg_cifar", in_shape=(3, 32, 32), classes=10,
    layers=[("conv", 3, 64, 3, 1, 1), ("relu",), ("conv", 64, 64, 3, 1, 1), ("relu",), ("maxpool", 2, 2),
            ("conv", 64, 128, 3, 1, 1), ("relu",), ("conv", 128, 128, 3, 1, 1), ("relu",), ("maxpool", 2, 2),
            ("conv", 128, 256, 3, 1, 1), ("relu",), ("conv", 256, 256, 3, 1, 1), ("relu",), ("maxpool", 2, 2),
            ("flatten",), ("linear", 4096, 512), ("relu",), ("linear", 512, 10)])

# The model of the reference's examples/cifar_cuda.rs:99-136: conv + BatchNorm2d + ReLU units, and a
# Linear -> BatchNorm -> ReLU -> Dropout(0.5) -> Linear head.
def _conv_bn(ci, co):
    return [("conv", ci, co, 3, 1, 1), ("batchnorm", co), ("relu",)]


VGG_CIFAR_BN = dict(
    name="vgg_cifar_bn", in_shape=(3, 32, 32), classes=10,
    layers=_conv_bn(3, 64) + _conv_bn(64, 64) + [("maxpool", 2, 2)] + _conv_bn(64, 128) + _conv_bn(128, 128)
    + [("maxpool", 2, 2)] + _conv_bn(128, 256) + _conv_bn(256, 256) + [("maxpool", 2, 2)]
    + [("flatten",), ("linear", 4096, 512), ("batchnorm", 512), ("relu",), ("dropout", 0.5), ("linear", 512, 10)])

BN_MOMENTUM, BN_EPS = 0.9, 1e-5

WIDE_MLP = dict(
    name="wide_mlp", in_shape=(4096,), classes=1000,
    layers=[("linear", 4096, 4096), ("gelu",), ("linear", 4096, 4096), ("gelu",),
            ("linear", 4096, 4096), ("gelu",), ("linear", 4096, 4096), ("gelu",), ("linear", 4096, 1000)])

ADAMW_HP = dict(lr=1e-3, beta1=0.9, beta2=0.999, eps=1e-8, wd=1e-4)


def he_init(layers, seed: int):
    """N(0, sqrt(2/fan_in)) weights, zero biases; fan_in = c_in*k*k for conv, n_in for Linear
    (src/init/he.rs:9-21 draws the same distribution from an unseedable RNG)."""
    rng = np.random.default_rng(seed)
    params = []
    for l in layers:
        if l[0] == "conv":
            _, ci, co, k, _, _ = l
            params.append((rng.standard_normal((co, ci, k, k)) * np.sqrt(2.0 / (ci * k * k))).astype(np.float32))
            params.append(np.zeros(co, np.float32))
        elif l[0] == "linear":
            _, n_in, n_out = l
            params.append((rng.standard_normal((n_in, n_out)) * np.sqrt(2.0 / n_in)).astype(np.float32))
            params.append(np.zeros(n_out, np.float32))
        elif l[0] == "batchnorm":   # gamma = 1, beta = 0 (examples/cifar_cuda.rs:42)
            params.append(np.ones(l[1], np.float32))
            params.append(np.zeros(l[1], np.float32))
    return params


def bn_buffers(layers):
    """Running statistics of the batchnorm layers, [mean0, var0, ...], at their initial 0 / 1."""
    out = []
    for l in layers:
        if l[0] == "batchnorm":
            out += [np.zeros(l[1], np.float32), np.ones(l[1], np.float32)]
    return out


def synthetic_batch(cfg, batch: int, seed: int, uniform01: bool = False):
    """Synthetic stand-in for the dataset: N(0,1) (or U[0,1)) inputs, uniform labels as one-hot f32."""
    rng = np.random.default_rng(seed)
    shape = (batch,) + tuple(cfg["in_shape"])
    x = rng.random(shape, dtype=np.float32) if uniform01 else rng.standard_normal(shape).astype(np.float32)
    labels = rng.integers(0, cfg["classes"], batch)
    t = np.zeros((batch, cfg["classes"]), np.float32)
    t[np.arange(batch), labels] = 1.0
    return x, t


def forward_backward(o, layers, params, x, target, divisor=None, input_requires_grad=False, buffers=None,
                     training=True, rng=None):
    """One forward + backward pass; returns (loss, grads in parameter order, logits).

    `buffers` (bn_buffers) are updated in place by training-mode batchnorm layers.  `rng` = {"seed", "offset"}
    is the dropout mask stream (the device library's definition, nrs_oracle.c); each dropout layer consumes
    ceil(mask_len / 4) counter blocks and advances the offset.

    Backward visits layers in reverse and ACCUMULATES into zeroed gradients, like
    zero_grad + loss_fn.backward + sync_grads (src/nn/sequential.rs:42-58,
    src/nn/loss.rs:78-107)."""
    acts = [np.ascontiguousarray(x, dtype=np.float32)]
    saved = []
    pi = bi = 0
    for l in layers:
        a = acts[-1]
        if l[0] == "conv":
            w, b = params[pi], params[pi + 1]
            saved.append((pi,))
            pi += 2
            acts.append(o.conv2d_fwd(a, w, b, l[4], l[5]))
        elif l[0] == "linear":
            w, b = params[pi], params[pi + 1]
            saved.append((pi,))
            pi += 2
            acts.append(o.bias_add_fwd(o.matmul_fwd(a, w), b))
        elif l[0] == "relu":
            saved.append(None)
            acts.append(o.relu_fwd(a))
        elif l[0] == "gelu":
            saved.append(None)
            acts.append(o.gelu_fwd(a))
        elif l[0] == "maxpool":
            y, am = o.maxpool_fwd(a, l[1], l[2])
            saved.append(am)
            acts.append(y)
        elif l[0] == "flatten":
            saved.append(None)
            acts.append(a.reshape(a.shape[0], -1))
        elif l[0] == "batchnorm":
            y, xhat, istd, rm, rv = o.batchnorm_fwd(a, params[pi], params[pi + 1], buffers[bi], buffers[bi + 1],
                                                    BN_EPS, BN_MOMENTUM, training)
            buffers[bi][...], buffers[bi + 1][...] = rm, rv
            saved.append((pi, xhat, istd))
            pi += 2
            bi += 2
            acts.append(y)
        elif l[0] in ("dropout", "dropout2d"):
            if not training:
                saved.append(None)
                acts.append(a)
                continue
            hw = a.shape[2] * a.shape[3] if l[0] == "dropout2d" else 1
            mask_len = a.size // hw
            mask = o.dropout_mask(mask_len, l[1], rng["seed"], rng["offset"])
            rng["offset"] += (mask_len + 3) // 4
            saved.append((mask, hw))
            acts.append(o.mask_mul(a, mask, hw))
        else:
            raise ValueError(l)
    logits = acts[-1]
    loss = o.ce_fwd(logits, target, divisor)
    g = o.ce_bwd(logits, target, divisor)
    grads = [np.zeros_like(p) for p in params]
    for li in range(len(layers) - 1, -1, -1):
        l, a_in = layers[li], acts[li]
        first = li == 0 and not input_requires_grad
        if l[0] == "conv":
            pidx = saved[li][0]
            dx, dw, db = o.conv2d_bwd(a_in, params[pidx], g, l[4], l[5], need_dx=not first)
            grads[pidx] += dw
            grads[pidx + 1] += db
            g = dx
        elif l[0] == "linear":
            pidx = saved[li][0]
            _, db = o.bias_add_bwd(g)
            da, dw = o.matmul_bwd(a_in, params[pidx], g)
            grads[pidx] += dw
            grads[pidx + 1] += db
            g = da
        elif l[0] == "relu":
            g = o.relu_bwd(a_in, g)
        elif l[0] == "gelu":
            g = o.gelu_bwd(a_in, g)
        elif l[0] == "maxpool":
            g = o.maxpool_bwd(g, saved[li], a_in.shape)
        elif l[0] == "flatten":
            g = g.reshape(a_in.shape)
        elif l[0] == "batchnorm":
            pidx, xhat, istd = saved[li]
            dx, dg, db = o.batchnorm_bwd(g, xhat, istd, params[pidx], training)
            grads[pidx] += dg
            grads[pidx + 1] += db
            g = dx
        elif l[0] in ("dropout", "dropout2d"):
            if saved[li] is not None:
                g = o.mask_mul(g, saved[li][0], saved[li][1])
    return loss, grads, logits


class OracleAdamW:
    """ADAMW over the flattened parameter list (src/optim/adamw.rs:11-55)."""

    def __init__(self, o, lr, beta1, beta2, eps, wd):
        self.o, self.hp, self.t, self.m, self.v = o, (lr, beta1, beta2, eps, wd), 0, None, None

    def step(self, params, grads):
        if self.m is None:
            self.m = [np.zeros_like(p) for p in params]
            self.v = [np.zeros_like(p) for p in params]
        for p, g, m, v in zip(params, grads, self.m, self.v):
            self.o.adamw_step(p.reshape(-1), g.reshape(-1), m.reshape(-1), v.reshape(-1), *self.hp, self.t)
        self.t += 1


def train_step(o, layers, params, opt, x, target, buffers=None, rng=None):
    """zero_grad -> forward -> loss -> backward -> optimizer.step; returns the loss."""
    loss, grads, _ = forward_backward(o, layers, params, x, target, buffers=buffers, rng=rng)
    opt.step(params, grads)
    return loss
