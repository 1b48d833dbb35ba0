"""The benchmark configurations as layer lists, their seeded initialisation and synthetic batches.

Pure numpy; shared by bench.py, the smoke test and the parity tests.  A model is a list of layer
tuples in the order the reference's ``Sequential`` walks its modules (src/nn/sequential.rs:22-30):

    ("conv", c_in, c_out, k, stride, pad)   ("relu",)  ("gelu",)  ("maxpool", k, stride)  ("flatten",)
    ("linear", n_in, n_out)   ("batchnorm", c)   ("dropout", p)   ("dropout2d", p)
    ("embedding", vocab, d_model, max_len)                token ids -> rows of the table + sinusoidal positions
    ("transformer_block", d_model, heads, d_ff, act, flags)   act 1 = ReLU (the reference's), 2 = GELU;
                                                              flags bit 0 = causal mask, bit 1 = no final norm
    ("layernorm", features)

Parameters are a flat list in layer order, the order ``ADAMW::step`` flattens them in
(src/optim/adamw.rs:48-54): [w, b] per conv / linear layer, [gamma, beta] per batchnorm / layernorm
layer, [table] per embedding, and per transformer block the reference's parameters() order
(src/nn/transformer_block.rs:58-66): w_q, w_k, w_v, w_o, norm1.gamma, norm1.beta, norm2.gamma,
norm2.beta, ff1.weights, ff1.bias, ff2.weights, ff2.bias.
"""
from __future__ import annotations

import numpy as np

ACT_RELU, ACT_GELU = 1, 2

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

# Transformer language model: batch 32 x 128 tokens, vocabulary 1000, d_model 256, two post-LN blocks with
# 8 heads, GELU feed-forward 256 -> 1024 -> 256 and a causal mask, vocabulary head, next-token cross-entropy.
TRANSFORMER_LM = dict(
    name="transformer_lm", in_shape=(128,), classes=1000, vocab=1000, token_model=True,
    layers=[("embedding", 1000, 256, 128),
            ("transformer_block", 256, 8, 1024, ACT_GELU, 1), ("transformer_block", 256, 8, 1024, ACT_GELU, 1),
            ("linear", 256, 1000)])

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
        elif l[0] in ("batchnorm", "layernorm"):   # gamma = 1, beta = 0 (examples/cifar_cuda.rs:42)
            params.append(np.ones(l[1], np.float32))
            params.append(np.zeros(l[1], np.float32))
        elif l[0] == "embedding":   # the reference leaves the table's initialisation to its user
            params.append((rng.standard_normal((l[1], l[2])) * 0.5).astype(np.float32))
        elif l[0] == "transformer_block":
            d, ff = l[1], l[3]
            for _ in range(4):                                   # w_q, w_k, w_v, w_o: N(0, 1/d)
                params.append((rng.standard_normal((d, d)) / np.sqrt(d)).astype(np.float32))
            params += [np.ones(d, np.float32), np.zeros(d, np.float32), np.ones(d, np.float32), np.zeros(d, np.float32)]
            params.append((rng.standard_normal((d, ff)) / np.sqrt(d)).astype(np.float32))
            params.append(np.zeros(ff, np.float32))
            params.append((rng.standard_normal((ff, d)) / np.sqrt(ff)).astype(np.float32))
            params.append(np.zeros(d, np.float32))
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




def synthetic_tokens(cfg, batch: int, seed: int):
    """Synthetic stand-in for a token corpus: uniform ids [batch, seq] and, as labels, the next token at every
    position (the sequence rolled by one, as a corpus window would give), both int32."""
    rng = np.random.default_rng(seed)
    seq = cfg["in_shape"][0]
    ids = rng.integers(0, cfg["vocab"], (batch, seq)).astype(np.int32)
    labels = np.roll(ids, -1, axis=1).astype(np.int32)
    return ids, np.ascontiguousarray(labels.reshape(-1))
