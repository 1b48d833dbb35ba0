"""Define-by-run CPU graph over the oracle primitives — the reference's CPU autograd
(src/autograd/node.rs, src/autograd/graph/*.rs, src/nn/*.rs) restated so that
branching models (attention, transformer blocks) can be written exactly as the
reference writes them.  TEST INFRASTRUCTURE ONLY (same rule as nrs_oracle.py).

Every op builds a node with parents and a backward closure that ACCUMULATES (+=)
into its parents' gradients; ``backward_graph`` walks the DFS topological order in
reverse (src/autograd/node.rs:113-151).
"""
from __future__ import annotations

import numpy as np


class Node:
    def __init__(self, data, parents=(), backward=None):
        self.data = np.ascontiguousarray(data, dtype=np.float32)
        self.grad = np.zeros_like(self.data)
        self.parents = list(parents)
        self.backward_fn = backward

    @property
    def shape(self):
        return self.data.shape


def backward_graph(root: Node):
    topo, seen = [], set()

    def build(n):
        if id(n) in seen:
            return
        seen.add(id(n))
        for p in n.parents:
            build(p)
        topo.append(n)

    build(root)
    for n in reversed(topo):
        if n.backward_fn is not None:
            n.backward_fn(n.grad)


class Graph:
    """Ops bound to one Oracle instance (f32 or f64 accumulation)."""

    def __init__(self, oracle):
        self.o = oracle

    # ---- graph ops (src/autograd/graph/*.rs)
    def matmul(self, a, b):
        o = self.o

        def bwd(g):
            da, db = o.matmul_bwd(a.data, b.data, g)
            a.grad += da
            b.grad += db
        return Node(o.matmul_fwd(a.data, b.data), (a, b), bwd)

    def bmm(self, a, b):
        o = self.o

        def bwd(g):
            da, db = o.bmm_bwd(a.data, b.data, g)
            a.grad += da
            b.grad += db
        return Node(o.bmm_fwd(a.data, b.data), (a, b), bwd)

    def add(self, a, b):
        o = self.o
        broadcast = a.data.ndim == 2 and b.data.ndim == 1 and a.shape[1] == b.shape[0]
        if broadcast:
            def bwd(g):
                da, db = o.bias_add_bwd(g)
                a.grad += da
                b.grad += db
            return Node(o.bias_add_fwd(a.data, b.data), (a, b), bwd)

        def bwd(g):
            a.grad += g
            b.grad += g.reshape(b.shape)
        return Node(o.add_fwd(a.data.ravel(), b.data.ravel()).reshape(a.shape), (a, b), bwd)

    def relu(self, a):
        o = self.o

        def bwd(g):
            a.grad += o.relu_bwd(a.data, g)
        return Node(o.relu_fwd(a.data), (a,), bwd)

    def gelu(self, a):
        o = self.o

        def bwd(g):
            a.grad += o.gelu_bwd(a.data, g)
        return Node(o.gelu_fwd(a.data), (a,), bwd)

    def reshape(self, a, shape):
        def bwd(g):
            a.grad += g.reshape(a.shape)
        return Node(a.data.reshape(shape), (a,), bwd)

    def softmax(self, a):
        o = self.o
        y = o.softmax_fwd(a.data)

        def bwd(g):
            a.grad += o.softmax_bwd(y, g)
        return Node(y, (a,), bwd)

    def transpose(self, a):
        o = self.o

        def bwd(g):
            a.grad += o.transpose_fwd(g)
        return Node(o.transpose_fwd(a.data), (a,), bwd)

    def scale(self, a, s):
        s = np.float32(s)

        def bwd(g):
            a.grad += g * s
        return Node(a.data * s, (a,), bwd)

    def slice_cols(self, a, c0, c1):
        o = self.o

        def bwd(g):
            a.grad += o.slice_cols_bwd(g, (a.data.size // a.shape[-1], a.shape[-1]), c0, c1).reshape(a.shape)
        return Node(o.slice_cols_fwd(a.data, c0, c1), (a,), bwd)

    def concat_cols(self, parts):
        widths = [p.shape[-1] for p in parts]

        def bwd(g):
            off = 0
            for p, w in zip(parts, widths):
                p.grad += g[..., off:off + w]
                off += w
        return Node(np.concatenate([p.data for p in parts], axis=-1), tuple(parts), bwd)

    def causal_mask(self, a):
        """scores[..., i, j > i] = -1e30 before the softmax.  NOT in the reference (it has no
        mask anywhere); defined here for the benchmark's causal LM configuration."""
        s = a.shape[-1]
        keep = np.tril(np.ones((a.shape[-2], s), dtype=bool))

        def bwd(g):
            a.grad += np.where(keep, g, 0.0).astype(np.float32)
        return Node(np.where(keep, a.data, np.float32(-1e30)), (a,), bwd)

    # ---- nn (src/nn/*.rs)
    def layernorm(self, x, gamma, beta, eps):
        o = self.o
        y, xhat, istd = o.layernorm_fwd(x.data, gamma.data, beta.data, eps)

        def bwd(g):
            dx, dg, db = o.layernorm_bwd(g, xhat, istd, gamma.data)
            x.grad += dx
            gamma.grad += dg
            beta.grad += db
        return Node(y, (x, gamma, beta), bwd)

    def embedding(self, weight, idx):
        """Embedding::forward / forward_batch (src/nn/embedding.rs:19-113); idx int array of any shape."""
        o = self.o
        idx = np.asarray(idx, dtype=np.int32)
        vocab, dim = weight.shape

        def bwd(g):
            weight.grad += o.embedding_bwd(g, idx, vocab)
        return Node(o.embedding_fwd(weight.data, idx).reshape(idx.shape + (dim,)), (weight,), bwd)

    def positional(self, x, max_len=None):
        """PositionalEncoding::forward (src/nn/positional.rs:36-47) on [seq, d]; on [batch, seq, d]
        the table is broadcast over the batch (an extension: the reference only has the 2-D form)."""
        seq, d = x.shape[-2], x.shape[-1]
        pe = self.o.positional_table(max_len or seq, d)[:seq]

        def bwd(g):
            x.grad += g
        return Node((x.data + pe).astype(np.float32), (x,), bwd)

    def attention_batch(self, q, k, v, causal=False):
        """src/nn/attention.rs:26-39: softmax(Q K^T / sqrt(d_head)) V on [batch, seq, d_head]."""
        d = q.shape[2]
        scores = self.scale(self.bmm(q, self.transpose(k)), 1.0 / np.sqrt(np.float32(d)))
        if causal:
            scores = self.causal_mask(scores)
        return self.bmm(self.softmax(scores), v)

    def mha_forward_batch(self, x, w_q, w_k, w_v, w_o, num_heads, causal=False):
        """MultiHeadAttention::forward_batch (src/nn/multihead.rs:67-114); no biases."""
        batch, seq, d = x.shape

        def proj(w):
            return self.reshape(self.matmul(self.reshape(x, (batch * seq, d)), w), (batch, seq, d))
        q, k, v = proj(w_q), proj(w_k), proj(w_v)
        dh = d // num_heads
        heads = []
        for h in range(num_heads):
            heads.append(self.attention_batch(self.slice_cols(q, h * dh, (h + 1) * dh),
                                              self.slice_cols(k, h * dh, (h + 1) * dh),
                                              self.slice_cols(v, h * dh, (h + 1) * dh), causal))
        concat = self.concat_cols(heads)
        return self.reshape(self.matmul(self.reshape(concat, (batch * seq, d)), w_o), (batch, seq, d))

    def transformer_block(self, x, p, num_heads, eps=1e-5, act="relu", causal=False):
        """TransformerBlock::forward (src/nn/transformer_block.rs:36-55): post-LN,
        LN1(x + MHA(x)), LN2(x1 + FF2(act(FF1(x1)))).  p: dict of parameter Nodes."""
        batch, seq, d = x.shape
        attn = self.mha_forward_batch(x, p["w_q"], p["w_k"], p["w_v"], p["w_o"], num_heads, causal)
        x1 = self.layernorm(self.add(x, attn), p["g1"], p["b1"], eps)
        flat = self.reshape(x1, (batch * seq, d))
        h = self.add(self.matmul(flat, p["ff1_w"]), p["ff1_b"])
        h = self.relu(h) if act == "relu" else self.gelu(h)
        ff = self.reshape(self.add(self.matmul(h, p["ff2_w"]), p["ff2_b"]), (batch, seq, d))
        return self.layernorm(self.add(x1, ff), p["g2"], p["b2"], eps)
