"""Whole-model CPU oracle: the reference's CPU training step restated over oracle/nrs_oracle.c.

TEST INFRASTRUCTURE ONLY (same rule as nrs_oracle.py).

A model is a list of layer tuples, applied in order, exactly as the reference's
``Sequential`` walks its ``Vec<Box<dyn Module>>`` (src/nn/sequential.rs:22-30):

    ("conv", c_in, c_out, k, stride, pad)   Conv2d          src/nn/conv.rs
    ("relu",) / ("gelu",)                    activations     src/autograd/graph/{relu,gelu}.rs
    ("maxpool", k, stride)                   MaxPool2d       src/nn/maxpool.rs
    ("flatten",)                             Flatten         src/nn/flatten.rs
    ("linear", n_in, n_out)                  Linear          src/nn/linear.rs (matmul + bias add)

Parameters are a flat list [w0, b0, w1, b1, ...] in layer order — the order
``ADAMW::step`` flattens them in (src/optim/adamw.rs:48-54).
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
    return params


def synthetic_batch(cfg, batch: int, seed: int, uniform01: bool = False):
    """Synthetic stand-in for the dataset: N(0,1) (or U[0,1)) inputs, uniform labels as one-hot f32."""
    rng = np.random.default_rng(seed)
    shape = (batch,) + tuple(cfg["in_shape"])
    x = rng.random(shape, dtype=np.float32) if uniform01 else rng.standard_normal(shape).astype(np.float32)
    labels = rng.integers(0, cfg["classes"], batch)
    t = np.zeros((batch, cfg["classes"]), np.float32)
    t[np.arange(batch), labels] = 1.0
    return x, t


def forward_backward(o, layers, params, x, target, divisor=None, input_requires_grad=False):
    """One forward + backward pass; returns (loss, grads in parameter order, logits).

    Backward visits layers in reverse and ACCUMULATES into zeroed gradients, like
    zero_grad + loss_fn.backward + sync_grads (src/nn/sequential.rs:42-58,
    src/nn/loss.rs:78-107)."""
    acts = [np.ascontiguousarray(x, dtype=np.float32)]
    saved = []
    pi = 0
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


def train_step(o, layers, params, opt, x, target):
    """zero_grad -> forward -> loss -> backward -> optimizer.step; returns the loss."""
    loss, grads, _ = forward_backward(o, layers, params, x, target)
    opt.step(params, grads)
    return loss
