"""Pins the oracle's transformer compositions (oracle/autograd.py) on CPU.

The reference pins these with finite-difference gradchecks
(tests/attention_batch_test.rs, multihead_batch_test.rs, transformer_block_test.rs:
loss = sum (i+1)*out_i, central differences) and known answers
(tests/embedding_test.rs, positional_test.rs); the same checks run here, plus an
independent float64 restatement in torch.
"""
import numpy as np
import pytest

from oracle.autograd import Graph, Node, backward_graph
from oracle.nrs_oracle import Oracle


def block_params(rng, d, ff):
    mk = lambda *s: Node((rng.standard_normal(s) * 0.3).astype(np.float32))
    return dict(w_q=mk(d, d), w_k=mk(d, d), w_v=mk(d, d), w_o=mk(d, d),
                g1=Node(1 + 0.1 * rng.standard_normal(d)), b1=Node(0.1 * rng.standard_normal(d)),
                g2=Node(1 + 0.1 * rng.standard_normal(d)), b2=Node(0.1 * rng.standard_normal(d)),
                ff1_w=mk(d, ff), ff1_b=mk(ff), ff2_w=mk(ff, d), ff2_b=mk(d))


def torch_block(x, p, heads, eps, act, causal):
    import torch
    import torch.nn.functional as F
    B, S, D = x.shape
    dh = D // heads
    q, k, v = x @ p["w_q"], x @ p["w_k"], x @ p["w_v"]
    outs = []
    for h in range(heads):
        sl = slice(h * dh, (h + 1) * dh)
        sc = (q[..., sl] @ k[..., sl].transpose(1, 2)) / np.sqrt(np.float32(dh)).astype(np.float64)
        if causal:
            sc = sc.masked_fill(torch.triu(torch.ones(S, S, dtype=torch.bool), 1), -1e30)
        outs.append(torch.softmax(sc, -1) @ v[..., sl])
    attn = torch.cat(outs, -1) @ p["w_o"]
    x1 = F.layer_norm(x + attn, (D,), p["g1"], p["b1"], eps)
    h = x1 @ p["ff1_w"] + p["ff1_b"]
    h = torch.relu(h) if act == "relu" else F.gelu(h, approximate="tanh")
    return F.layer_norm(x1 + h @ p["ff2_w"] + p["ff2_b"], (D,), p["g2"], p["b2"], eps)


@pytest.mark.parametrize("act,causal", [("relu", False), ("gelu", True)])
def test_transformer_block_against_torch_float64(act, causal):
    import torch
    rng = np.random.default_rng(0)
    B, S, D, H, FF = 2, 5, 8, 2, 16
    g = Graph(Oracle("f64"))
    p = block_params(rng, D, FF)
    x = Node(rng.standard_normal((B, S, D)).astype(np.float32))
    out = g.transformer_block(x, p, H, 1e-5, act, causal)
    seed = rng.standard_normal(out.shape).astype(np.float32)
    out.grad = seed.copy()
    backward_graph(out)
    tp = {k: torch.tensor(v.data, dtype=torch.float64, requires_grad=True) for k, v in p.items()}
    tx = torch.tensor(x.data, dtype=torch.float64, requires_grad=True)
    tout = torch_block(tx, tp, H, 1e-5, act, causal)
    tout.backward(torch.tensor(seed, dtype=torch.float64))
    assert np.abs(out.data - tout.detach().numpy()).max() < 1e-5
    assert np.abs(x.grad - tx.grad.numpy()).max() < 1e-4
    for k in p:
        assert np.abs(p[k].grad - tp[k].grad.numpy()).max() < 1e-4, k


def test_block_gradcheck_like_reference():
    # tests/transformer_block_test.rs:63-112: loss = sum (i+1)*out_i, h = 1e-3, tolerance 5e-2
    rng = np.random.default_rng(1)
    B, S, D, H, FF = 1, 3, 4, 2, 8
    g = Graph(Oracle("f64"))
    p = block_params(rng, D, FF)
    xd = rng.standard_normal((B, S, D)).astype(np.float32)

    def loss_of(pp, xv):
        out = g.transformer_block(Node(xv), pp, H)
        return float((out.data.ravel().astype(np.float64) * (np.arange(out.data.size) + 1)).sum()), out

    xn = Node(xd)
    out = g.transformer_block(xn, p, H)
    out.grad = (np.arange(out.data.size) + 1).astype(np.float32).reshape(out.shape)
    backward_graph(out)
    h = 1e-3
    for name, idx in [("w_q", (0, 1)), ("ff1_w", (2, 3)), ("g1", (1,)), ("w_o", (3, 0))]:
        base = p[name].data.copy()
        p[name].data = base.copy(); p[name].data[idx] += h
        lp, _ = loss_of(p, xd)
        p[name].data = base.copy(); p[name].data[idx] -= h
        lm, _ = loss_of(p, xd)
        p[name].data = base
        num = (lp - lm) / (2 * h)
        assert abs(num - p[name].grad[idx]) < 5e-2 * max(1.0, abs(num)), name


def test_embedding_and_positional_known_answers():
    o = Oracle("f32")
    g = Graph(o)
    # tests/embedding_test.rs: rows are gathered, gradients of repeated tokens add up
    w = Node(np.arange(12, dtype=np.float32).reshape(4, 3))
    out = g.embedding(w, [2, 0, 2])
    assert out.data.tolist() == [[6, 7, 8], [0, 1, 2], [6, 7, 8]]
    out.grad = np.ones_like(out.data)
    backward_graph(out)
    assert w.grad.tolist() == [[1, 1, 1], [0, 0, 0], [2, 2, 2], [0, 0, 0]]
    outb = g.embedding(w, [[1, 3], [3, 3]])
    assert outb.shape == (2, 2, 3) and outb.data[1, 0].tolist() == [9, 10, 11]
    # tests/positional_test.rs: pe[0] = [0,1,0,1,...]; pe[pos,0] = sin(pos), pe[pos,1] = cos(pos)
    pe = o.positional_table(16, 8)
    assert np.allclose(pe[0], [0, 1] * 4)
    assert np.allclose(pe[3, 0], np.sin(3.0), atol=1e-6) and np.allclose(pe[3, 1], np.cos(3.0), atol=1e-6)
    assert np.allclose(pe[5, 2], np.sin(5.0 / 10000 ** 0.25), atol=1e-6)
    x = Node(np.zeros((2, 4, 8), np.float32))
    assert np.array_equal(g.positional(x, 16).data[1], pe[:4])
