"""GPU parity of the transformer pieces against the CPU oracle graph (oracle/autograd.py):
embedding, positional encoding, batched attention, multi-head attention, the post-LN
block (reference form: ReLU, no mask; and the LM-benchmark form: GELU + causal mask), and a
small language-model training step built from them.  Shapes follow
tests/cuda_transformer_test.rs (batch 2, seq 4..8, d_model 8..16) plus a larger case."""
import numpy as np
import pytest

from neuralrs_b200 import _lib, cuda
from neuralrs_b200.cuda import Node, backward_graph, graph, loss, nn, optim
from neuralrs_b200.cuda import runtime as gpu
from oracle import autograd as og
from .conftest import rel_l2

pytestmark = pytest.mark.gpu

PARAM_ORDER = ["w_q", "w_k", "w_v", "w_o", "g1", "b1", "g2", "b2", "ff1_w", "ff1_b", "ff2_w", "ff2_b"]


def on_gpu(a):
    n = Node.new(a, list(np.shape(a)))
    gpu.to_cuda(n)
    return n


def make_block_params(rng, d, ff):
    mk = lambda *s: (rng.standard_normal(s) * (1.0 / np.sqrt(s[0]))).astype(np.float32)
    return dict(w_q=mk(d, d), w_k=mk(d, d), w_v=mk(d, d), w_o=mk(d, d),
                g1=(1 + 0.1 * rng.standard_normal(d)).astype(np.float32), b1=(0.1 * rng.standard_normal(d)).astype(np.float32),
                g2=(1 + 0.1 * rng.standard_normal(d)).astype(np.float32), b2=(0.1 * rng.standard_normal(d)).astype(np.float32),
                ff1_w=mk(d, ff), ff1_b=(0.1 * rng.standard_normal(ff)).astype(np.float32),
                ff2_w=mk(ff, d), ff2_b=(0.1 * rng.standard_normal(d)).astype(np.float32))


def gpu_block(p, heads, act, causal):
    n = {k: on_gpu(v) for k, v in p.items()}
    mha = nn.MultiHeadAttention(n["w_q"], n["w_k"], n["w_v"], n["w_o"], p["w_q"].shape[0], heads, causal)
    blk = nn.TransformerBlock(mha, nn.LayerNorm(n["g1"], n["b1"], 1e-5), nn.LayerNorm(n["g2"], n["b2"], 1e-5),
                              nn.Linear(n["ff1_w"], n["ff1_b"]), nn.Linear(n["ff2_w"], n["ff2_b"]),
                              p["w_q"].shape[0], p["ff1_w"].shape[1], _lib.ACT_RELU if act == "relu" else _lib.ACT_GELU)
    return blk, n


def test_embedding_and_positional(gpu_ctx, oracle32):
    g = og.Graph(oracle32)
    rng = np.random.default_rng(0)
    vocab, dim = 50, 16
    w = rng.standard_normal((vocab, dim)).astype(np.float32)
    idx = rng.integers(0, vocab, (3, 7))
    idx[0, :3] = 5                                            # repeated tokens add up in the gradient
    cw = og.Node(w)
    cout = g.positional(g.embedding(cw, idx), 32)
    seed = rng.standard_normal(cout.shape).astype(np.float32)
    cout.grad = seed.copy()
    og.backward_graph(cout)
    gw = on_gpu(w)
    emb = nn.Embedding(gw, vocab, dim)
    pe = nn.PositionalEncoding(dim, 32)
    gout = pe.forward(emb.forward_batch(idx))
    assert gout.shape == [3, 7, dim]
    assert np.abs(gpu.to_host(gout) - cout.data.ravel()).max() < 1e-5
    gpu.set_grad(gout, seed)
    backward_graph(gout)
    assert np.abs(gpu.read_grad(gw) - cw.grad.ravel()).max() < 1e-5
    # 1-D form, as the reference's GPU Embedding::forward / PositionalEncoding::forward ([seq, d])
    g1 = pe.forward(emb.forward(idx[1]))
    assert g1.shape == [7, dim]
    assert np.abs(gpu.to_host(g1) - cout.data[1].ravel()).max() < 1e-5
    with pytest.raises(cuda._lib.NrsError, match="out of vocab range"):
        emb.forward([vocab])
    # the table itself (src/nn/positional.rs:23-33)
    assert np.abs(gpu.to_host(pe.table).reshape(32, dim) - oracle32.positional_table(32, dim)).max() < 1e-6


@pytest.mark.parametrize("causal", [False, True])
def test_attention_batch(gpu_ctx, oracle64, causal):
    # tests/attention_batch_test.rs shapes, plus the LM config's head shape [b*?, 128, 32]
    g = og.Graph(oracle64)
    rng = np.random.default_rng(1)
    for b, s, d in [(2, 4, 8), (3, 128, 32), (2, 20, 48), (2, 160, 16)]:   # the last two: outside the fused kernel's range
        q, k, v = (rng.standard_normal((b, s, d)).astype(np.float32) for _ in range(3))
        cq, ck, cv = og.Node(q), og.Node(k), og.Node(v)
        cout = g.attention_batch(cq, ck, cv, causal)
        seed = rng.standard_normal(cout.shape).astype(np.float32)
        cout.grad = seed.copy()
        og.backward_graph(cout)
        gq, gk, gv = on_gpu(q), on_gpu(k), on_gpu(v)
        gout = nn.attention_batch(gq, gk, gv, causal)
        assert rel_l2(gpu.to_host(gout), cout.data) < 1e-4
        gpu.set_grad(gout, seed)
        backward_graph(gout)
        for gn, cn in ((gq, cq), (gk, ck), (gv, cv)):
            assert rel_l2(gpu.read_grad(gn), cn.grad) < 1e-4


@pytest.mark.parametrize("act,causal", [("relu", False), ("gelu", True)])
@pytest.mark.parametrize("shape", [(2, 4, 8, 2, 16), (4, 32, 64, 8, 256), (2, 8, 128, 2, 64), (2, 130, 32, 4, 32)])  # last two: batched-head path
def test_transformer_block(gpu_ctx, oracle64, act, causal, shape):
    # tests/cuda_transformer_test.rs:19-27 (batch 2, seq 4, d 8, 2 heads, ff 16), bar 3e-3 absolute there
    B, S, D, H, FF = shape
    g = og.Graph(oracle64)
    rng = np.random.default_rng(2)
    p = make_block_params(rng, D, FF)
    x = rng.standard_normal((B, S, D)).astype(np.float32)
    cp = {k: og.Node(v) for k, v in p.items()}
    cx = og.Node(x)
    cout = g.transformer_block(cx, cp, H, 1e-5, act, causal)
    seed = rng.standard_normal(cout.shape).astype(np.float32)
    cout.grad = seed.copy()
    og.backward_graph(cout)
    blk, n = gpu_block(p, H, act, causal)
    gx = on_gpu(x)
    gout = blk.forward(gx)
    assert gout.shape == [B, S, D]
    assert np.abs(gpu.to_host(gout) - cout.data.ravel()).max() < 3e-3
    assert rel_l2(gpu.to_host(gout), cout.data) < 1e-4
    gpu.set_grad(gout, seed)
    backward_graph(gout)
    assert rel_l2(gpu.read_grad(gx), cx.grad) < 1e-4
    for k in PARAM_ORDER:
        assert rel_l2(gpu.read_grad(n[k]), cp[k].grad) < 1e-4, k
    # forward_no_final_norm drops LN2 (src/cuda/nn/transformer_block.rs:45-59)
    g2 = blk.forward_no_final_norm(on_gpu(x))
    assert g2.shape == [B, S, D]


def test_language_model_step(gpu_ctx, oracle64):
    """Embedding + PE + 2 blocks (GELU, causal) + Linear head + CE over [B*S, V] + AdamW:
    the transformer-LM benchmark configuration at reduced size."""
    g = og.Graph(oracle64)
    rng = np.random.default_rng(3)
    B, S, V, D, H, FF = 4, 16, 50, 32, 4, 64
    ids = rng.integers(0, V, (B, S))
    tgt = np.roll(ids, -1, axis=1)
    onehot = np.zeros((B * S, V), np.float32)
    onehot[np.arange(B * S), tgt.ravel()] = 1
    emb_w = (rng.standard_normal((V, D)) * 0.5).astype(np.float32)
    blocks = [make_block_params(rng, D, FF) for _ in range(2)]
    head_w = (rng.standard_normal((D, V)) / np.sqrt(D)).astype(np.float32)
    head_b = np.zeros(V, np.float32)

    # --- oracle
    c_emb, c_hw, c_hb = og.Node(emb_w), og.Node(head_w), og.Node(head_b)
    c_blocks = [{k: og.Node(v) for k, v in bp.items()} for bp in blocks]
    h = g.positional(g.embedding(c_emb, ids), 64)
    for cb in c_blocks:
        h = g.transformer_block(h, cb, H, 1e-5, "gelu", True)
    c_logits = g.add(g.matmul(g.reshape(h, (B * S, D)), c_hw), c_hb)
    c_loss = oracle64.ce_fwd(c_logits.data, onehot)
    c_logits.grad = oracle64.ce_bwd(c_logits.data, onehot)
    og.backward_graph(c_logits)

    # --- GPU, through the mirrored API
    g_emb, g_hw, g_hb = on_gpu(emb_w), on_gpu(head_w), on_gpu(head_b)
    g_blocks = [gpu_block(bp, H, "gelu", True) for bp in blocks]
    pe = nn.PositionalEncoding(D, 64)
    params = [g_emb] + [q for blk, _ in g_blocks for q in blk.parameters()] + [g_hw, g_hb]
    opt = optim.AdamW(1e-3, 0.9, 0.999, 1e-8, 1e-4)
    gpu.zero_grad(params)
    hh = pe.forward(nn.Embedding(g_emb, V, D).forward_batch(ids))
    for blk, _ in g_blocks:
        hh = blk.forward(hh)
    logits = graph.add(graph.matmul(graph.reshape(hh, [B * S, D]), g_hw), g_hb)
    gt = on_gpu(onehot)
    g_loss = loss.cross_entropy(logits, gt)
    loss.cross_entropy_backward(logits, gt)
    backward_graph(logits)
    assert abs(g_loss - c_loss) < 1e-4 * max(1.0, abs(c_loss))
    assert rel_l2(gpu.read_grad(g_emb), c_emb.grad) < 1e-4
    assert rel_l2(gpu.read_grad(g_hw), c_hw.grad) < 1e-4
    for (blk, n), cb in zip(g_blocks, c_blocks):
        for k in PARAM_ORDER:
            assert rel_l2(gpu.read_grad(n[k]), cb[k].grad) < 1e-4, k
    before = gpu.to_host(g_emb).copy()
    opt.step(params)
    assert np.abs(gpu.to_host(g_emb) - before).max() > 0
