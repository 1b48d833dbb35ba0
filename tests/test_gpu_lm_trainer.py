"""The native training step of a token model (nrs_trainer_* with an embedding first layer): one C call per
step — Embedding + positional encoding, post-LN transformer blocks, Linear head on every position,
cross-entropy over batch*seq rows, AdamW — against the CPU oracle's define-by-run composition of the same
reference modules (oracle/models.py: lm_forward_backward).  Tolerance 1e-4 relative per tensor in the
default 3xTF32 mode."""
import numpy as np
import pytest

from neuralrs_b200 import _lib, cuda
from oracle import models
from .conftest import rel_l2

pytestmark = pytest.mark.gpu

HP = models.ADAMW_HP


def make_trainer(cfg, ctx, params, fuse=True):
    tr = cuda.Trainer(cfg["layers"], cfg["in_shape"], cfg["classes"], HP["lr"], HP["beta1"], HP["beta2"], HP["eps"],
                      HP["wd"], fuse=fuse, ctx=ctx)
    tr.set_params(params)
    return tr


def small_lm(act, flags, extra_norm=False):
    V, D, H, FF, S = 50, 32, 4, 64, 16
    layers = [("embedding", V, D, 64), ("transformer_block", D, H, FF, act, flags), ("transformer_block", D, H, FF, act, flags)]
    if extra_norm:
        layers.append(("layernorm", D))
    layers.append(("linear", D, V))
    return dict(name="small_lm", in_shape=(S,), classes=V, vocab=V, layers=layers)


@pytest.mark.parametrize("act,flags,extra_norm,fuse", [(models.ACT_GELU, 1, False, True), (models.ACT_RELU, 0, True, True),
                                                       (models.ACT_GELU, 1, False, False)])
def test_native_lm_step_matches_oracle(gpu_ctx, oracle64, act, flags, extra_norm, fuse):
    cfg = small_lm(act, flags, extra_norm)
    params = models.he_init(cfg["layers"], 11)
    if extra_norm:   # a non-trivial affine so that its gradients are exercised
        params[-4][...] = np.linspace(0.5, 1.5, params[-4].size, dtype=np.float32)
        params[-3][...] = np.linspace(-0.2, 0.2, params[-3].size, dtype=np.float32)
    ids, labels = models.synthetic_tokens(cfg, 4, 12)
    c_loss, c_grads, _ = models.lm_forward_backward(oracle64, cfg["layers"], [p.copy() for p in params], ids, labels)
    tr = make_trainer(cfg, gpu_ctx, params, fuse)
    assert tr.n_params == len(params)
    g_loss = tr.forward_backward_tokens(ids, labels)
    assert abs(g_loss - c_loss) <= 1e-4 * max(1.0, abs(c_loss))
    for i, cg in enumerate(c_grads):
        assert rel_l2(tr.get_grad(i), cg) <= 1e-4, f"parameter {i}"
    # one full step against the oracle's AdamW (src/optim/adamw.rs:23-46)
    opt = models.OracleAdamW(oracle64, HP["lr"], HP["beta1"], HP["beta2"], HP["eps"], HP["wd"])
    ref = [p.copy() for p in params]
    opt.step(ref, c_grads)
    tr.step_tokens(ids, labels)
    for i, rp in enumerate(ref):
        assert np.abs(tr.get_param(i) - rp.ravel()).max() <= 2e-6 + 1e-5 * np.abs(rp).max(), f"parameter {i}"
    tr.close()


def test_token_entry_points_agree_and_reject_misuse(gpu_ctx):
    import ctypes as C
    cfg = small_lm(models.ACT_GELU, 1)
    params = models.he_init(cfg["layers"], 21)
    batches = [models.synthetic_tokens(cfg, 3, 30 + i) for i in range(3)]
    a, b, c = (make_trainer(cfg, gpu_ctx, params) for _ in range(3))
    from .gpu_util import Dev
    la, lb, lc = [], [], []
    for ids, labels in batches:                       # host entry point
        la.append(a.step_tokens(ids, labels))
    for i, (ids, labels) in enumerate(batches):       # double-buffered staging
        if i == 0:
            b._keep = [(np.ascontiguousarray(x), np.ascontiguousarray(y)) for x, y in batches]
            b.stage_next_tokens_ptr(b._keep[0][0].ctypes.data, b._keep[0][1].ctypes.data, 3)
        if i + 1 < len(batches):
            b.stage_next_tokens_ptr(b._keep[i + 1][0].ctypes.data, b._keep[i + 1][1].ctypes.data, 3)
        lb.append(b.step_staged(True))
    for ids, labels in batches:                       # resident inputs
        di, dl = Dev(gpu_ctx, ids), Dev(gpu_ctx, labels)
        lc.append(c.step_tokens_device(di.ptr.value, dl.ptr.value, 3, True))
    assert la == lb == lc
    for i in range(a.n_params):
        assert np.array_equal(a.get_param(i), b.get_param(i)) and np.array_equal(a.get_param(i), c.get_param(i))
    # a float-sample entry point on a token model is refused, and vice versa
    x = np.zeros((3, 16), np.float32)
    t = np.zeros((3 * 16, 50), np.float32)
    with pytest.raises(_lib.NrsError):
        a.step(x, t)
    cnn = cuda.Trainer(models.SMALL_CNN["layers"], models.SMALL_CNN["in_shape"], 10, ctx=gpu_ctx)
    with pytest.raises(_lib.NrsError):
        cnn.step_tokens(batches[0][0], batches[0][1])
    # a token id outside the vocabulary is reported, never dereferenced
    bad = batches[0][0].copy()
    bad[1, 5] = 50
    with pytest.raises(_lib.NrsError) as e:
        a.step_tokens(bad, batches[0][1])
    assert e.value.code == 1 and "outside the vocabulary" in str(e.value)
    a.step_tokens(*batches[0])                        # the context stays usable
    for tr in (a, b, c, cnn):
        tr.close()


def test_embedding_layer_must_come_first_and_shapes_are_checked(gpu_ctx):
    with pytest.raises(_lib.NrsError):
        cuda.Trainer([("linear", 16, 8), ("embedding", 10, 8, 0)], (16,), 8, ctx=gpu_ctx)
    with pytest.raises(_lib.NrsError):     # d_model not divisible by heads
        cuda.Trainer([("embedding", 10, 30, 0), ("transformer_block", 30, 4, 64, 1, 0), ("linear", 30, 10)], (8,), 10, ctx=gpu_ctx)
    with pytest.raises(_lib.NrsError):     # sequence longer than the positional table
        cuda.Trainer([("embedding", 10, 32, 4), ("linear", 32, 10)], (8,), 10, ctx=gpu_ctx)


def test_transformer_lm_full_size(gpu_ctx, oracle64):
    """The language-model configuration at its own size (sequence 128, vocabulary 1000, d_model 256, 8 heads of 32,
    d_ff 1024, two causal GELU blocks): the oracle on a batch of two sequences directly; at batch 32 the step's
    additivity over a split of the batch and bit-for-bit determinism."""
    cfg = models.TRANSFORMER_LM
    params = models.he_init(cfg["layers"], 1238)
    tr = make_trainer(cfg, gpu_ctx, params)
    ids, labels = models.synthetic_tokens(cfg, 32, 1239)
    S = cfg["in_shape"][0]
    # (1) two sequences against the oracle: loss and every parameter gradient
    c_loss, c_grads, _ = models.lm_forward_backward(oracle64, cfg["layers"], [p.copy() for p in params], ids[:2], labels[:2 * S])
    g_loss = tr.forward_backward_tokens(ids[:2], labels[:2 * S])
    assert abs(g_loss - c_loss) <= 1e-4 * max(1.0, abs(c_loss))
    for i, cg in enumerate(c_grads):
        assert rel_l2(tr.get_grad(i), cg) <= 1e-4, f"parameter {i}"
    # (2) batch 32: the mean over the batch is the mean of the halves' means
    full = tr.forward_backward_tokens(ids, labels)
    g_full = [tr.get_grad(i).astype(np.float64) for i in range(tr.n_params)]
    lo = tr.forward_backward_tokens(ids[:16], labels[:16 * S])
    g_lo = [tr.get_grad(i).astype(np.float64) for i in range(tr.n_params)]
    hi = tr.forward_backward_tokens(ids[16:], labels[16 * S:])
    g_hi = [tr.get_grad(i).astype(np.float64) for i in range(tr.n_params)]
    assert abs(full - 0.5 * (lo + hi)) <= 1e-5 * abs(full)
    for i in range(tr.n_params):
        assert rel_l2(g_full[i], 0.5 * (g_lo[i] + g_hi[i])) <= 1e-4, f"parameter {i}"
    # (3) determinism
    again = tr.forward_backward_tokens(ids, labels)
    assert again == full
    for i in range(tr.n_params):
        assert np.array_equal(tr.get_grad(i).astype(np.float64), g_full[i]), f"parameter {i}"
    tr.close()


def test_operator_level_buckets_on_one_rank(gpu_ctx, oracle64):
    """nrs_dp_create / nrs_bucket_register / nrs_backward_graph_dp / nrs_grad_ready / nrs_allreduce_wait with a
    world of one (no communicator): the bookkeeping — flat re-homing of the parameters, bucket planning, readiness
    in any order, zero-fill of a parameter nothing wrote — must leave exactly the gradients backward_graph leaves."""
    from neuralrs_b200.cuda import Node, backward_graph, graph, loss, nn
    from neuralrs_b200.cuda import runtime as gpu
    rng = np.random.default_rng(5)

    def on_gpu(a):
        n = Node.new(a, list(a.shape))
        gpu.to_cuda(n)
        return n
    x = rng.standard_normal((8, 12)).astype(np.float32)
    w1, b1 = rng.standard_normal((12, 20)).astype(np.float32), rng.standard_normal(20).astype(np.float32)
    w2, b2 = rng.standard_normal((20, 5)).astype(np.float32), rng.standard_normal(5).astype(np.float32)
    unused = rng.standard_normal(7).astype(np.float32)
    t = np.eye(5, dtype=np.float32)[rng.integers(0, 5, 8)]

    def run(use_dp, manual):
        gx, gt = on_gpu(x), on_gpu(t)
        gx.requires_grad = False
        ps = [on_gpu(a) for a in (w1, b1, w2, b2, unused)]
        dp = None
        if use_dp:
            dp = cuda.DataParallel(0, 1, None, 8, ctx=gpu_ctx)
            dp.register(ps, 4)                        # tiny buckets: one per tensor
            assert dp.bucket_count == 5
        gpu.zero_grad(ps)
        h = graph.relu(graph.add(graph.matmul(gx, ps[0]), ps[1]))
        logits = graph.add(graph.matmul(h, ps[2]), ps[3])
        loss.cross_entropy_backward(logits, gt)
        if not use_dp:
            backward_graph(logits)
        elif manual:
            dp.begin_step()
            backward_graph(logits)
            for p in (ps[1], ps[3], ps[0], ps[2]):    # any order; `unused` is never reported
                dp.grad_ready(p)
            dp.allreduce_wait()
        else:
            dp.backward_graph(logits)
        if dp:
            dp.host_wait()
        out = [gpu.read_grad(p) for p in ps]
        vals = [gpu.to_host(p) for p in ps]
        if dp:
            dp.close()
        return out, vals
    ref, _ = run(False, False)
    for manual in (False, True):
        got, vals = run(True, manual)
        for g, r in zip(got, ref):
            assert np.array_equal(g, r)
        assert np.all(got[4] == 0)
        for v, a in zip(vals, (w1, b1, w2, b2, unused)):     # flattening kept the values
            assert np.array_equal(v, a.ravel())
