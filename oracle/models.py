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

from neuralrs_b200.workloads import (ACT_GELU, ACT_RELU, ADAMW_HP, BN_EPS, BN_MOMENTUM, SMALL_CNN, TRANSFORMER_LM,  # noqa: F401
                                     VGG_CIFAR, VGG_CIFAR_BN, WIDE_MLP, bn_buffers, he_init, synthetic_batch,
                                     synthetic_tokens)


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


def lm_forward_backward(o, layers, params, ids, labels, divisor=None):
    """Forward + backward of a token model (first layer "embedding") through the define-by-run CPU graph
    (oracle/autograd.py), the way the reference composes it: Embedding::forward_batch, PositionalEncoding,
    TransformerBlock::forward per block, Linear on every position, cross-entropy over batch*seq rows
    (src/nn/embedding.rs:60-113, positional.rs:36-47, transformer_block.rs:36-55, linear.rs, loss.rs:78-107).
    labels: int class per position.  Returns (loss, grads in parameter order, logits [batch*seq, classes])."""
    from oracle.autograd import Graph, Node, backward_graph
    g = Graph(o)
    ids = np.asarray(ids, np.int32)
    batch, seq = ids.shape
    nodes = [Node(p) for p in params]
    pi = 0
    h = None
    for l in layers:
        if l[0] == "embedding":
            h = g.embedding(nodes[pi], ids)
            pi += 1
            if l[3] > 0:
                h = g.positional(h, l[3])
        elif l[0] == "transformer_block":
            names = ("w_q", "w_k", "w_v", "w_o", "g1", "b1", "g2", "b2", "ff1_w", "ff1_b", "ff2_w", "ff2_b")
            p = dict(zip(names, nodes[pi:pi + 12]))
            pi += 12
            if l[5] & 2:
                raise NotImplementedError("forward_no_final_norm")
            h = g.transformer_block(h, p, l[2], 1e-5, "gelu" if l[4] == ACT_GELU else "relu", causal=bool(l[5] & 1))
        elif l[0] == "layernorm":
            h = g.layernorm(h, nodes[pi], nodes[pi + 1], 1e-5)
            pi += 2
        elif l[0] == "linear":
            d = h.shape[-1]
            flat = g.reshape(h, (batch * seq, d))
            out = g.add(g.matmul(flat, nodes[pi]), nodes[pi + 1])
            h = g.reshape(out, (batch, seq, l[2]))
            pi += 2
        elif l[0] in ("relu", "gelu"):
            h = g.relu(h) if l[0] == "relu" else g.gelu(h)
        else:
            raise ValueError(l)
    classes = h.shape[-1]
    logits = g.reshape(h, (batch * seq, classes))
    target = np.zeros((batch * seq, classes), np.float32)
    target[np.arange(batch * seq), np.asarray(labels).ravel()] = 1.0
    loss = o.ce_fwd(logits.data, target, divisor)
    logits.grad = o.ce_bwd(logits.data, target, divisor).astype(np.float32)
    backward_graph(logits)
    return loss, [n.grad for n in nodes], logits.data
