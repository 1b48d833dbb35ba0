"""GPU-vs-CPU twin tests in the shape of the reference's own tests/cuda_*.rs: same
input formulas, same call sequence through the mirrored API, same (absolute)
tolerances; the CPU twin is the oracle."""
import numpy as np
import pytest

from neuralrs_b200 import cuda
from neuralrs_b200.cuda import Node, backward_graph, graph, loss, nn, optim
from neuralrs_b200.cuda import runtime as gpu

pytestmark = pytest.mark.gpu


def seq(n, mod, mul, add):
    return (np.arange(n) % mod * mul + add).astype(np.float32)


def on_gpu(data, shape):
    n = Node.new(data, shape)
    gpu.to_cuda(n)
    return n


def test_cuda_conv2d_forward(gpu_ctx, oracle32):
    # tests/cuda_conv2d_test.rs:15-44
    n, c_in, in_h, in_w, c_out, kh, kw, stride, pad = 2, 3, 8, 8, 4, 3, 3, 1, 1
    x = seq(n * c_in * in_h * in_w, 23, 0.05, -0.5)
    w = seq(c_out * c_in * kh * kw, 13, 0.07, -0.4)
    b = seq(c_out, 5, 0.1, -0.2)
    cpu_out = oracle32.conv2d_fwd(x.reshape(n, c_in, in_h, in_w), w.reshape(c_out, c_in, kh, kw), b, stride, pad)
    gout = nn.conv2d(on_gpu(x, [n, c_in, in_h, in_w]), on_gpu(w, [c_out, c_in, kh, kw]), on_gpu(b, [c_out]), stride, pad)
    assert gout.shape == list(cpu_out.shape)
    assert np.abs(gpu.to_host(gout) - cpu_out.ravel()).max() < 1e-4


def test_cuda_conv2d_backward(gpu_ctx, oracle32):
    # tests/cuda_conv2d_test.rs:46-97
    n, c_in, in_h, in_w, c_out, kh, kw, stride, pad = 2, 3, 7, 7, 5, 3, 3, 1, 1
    x = seq(n * c_in * in_h * in_w, 23, 0.05, -0.5)
    w = seq(c_out * c_in * kh * kw, 13, 0.07, -0.4)
    b = seq(c_out, 5, 0.1, -0.2)
    x4, w4 = x.reshape(n, c_in, in_h, in_w), w.reshape(c_out, c_in, kh, kw)
    out_len = oracle32.conv2d_fwd(x4, w4, b, stride, pad).size
    seed = seq(out_len, 7, 0.2, 0.1)
    c_igrad, c_wgrad, c_bgrad = oracle32.conv2d_bwd(x4, w4, seed.reshape(n, c_out, in_h, in_w), stride, pad)
    gi, gw, gb = on_gpu(x, [n, c_in, in_h, in_w]), on_gpu(w, [c_out, c_in, kh, kw]), on_gpu(b, [c_out])
    gout = nn.conv2d(gi, gw, gb, stride, pad)
    gpu.set_grad(gout, seed)
    backward_graph(gout)
    assert np.abs(gpu.read_grad(gi) - c_igrad.ravel()).max() < 1e-3
    assert np.abs(gpu.read_grad(gw) - c_wgrad.ravel()).max() < 1e-3
    assert np.abs(gpu.read_grad(gb) - c_bgrad.ravel()).max() < 1e-3
    # requires_grad = false skips the input gradient (src/cuda/nn/conv.rs:304)
    gi2 = on_gpu(x, [n, c_in, in_h, in_w])
    gi2.requires_grad = False
    gout2 = nn.conv2d(gi2, gw, gb, stride, pad)
    gpu.set_grad(gout2, seed)
    backward_graph(gout2)
    assert np.all(gpu.read_grad(gi2) == 0)
    assert np.abs(gpu.read_grad(gw) - 2 * c_wgrad.ravel()).max() < 2e-3     # gradients accumulate (+=)


def test_cuda_resident_matmul_backward(gpu_ctx, oracle32):
    # tests/cuda_matmul_resident_test.rs:8-45
    m, k, n = 40, 56, 32
    a, b, seed = seq(m * k, 13, 0.1, -0.6), seq(k * n, 7, 0.2, -0.6), seq(m * n, 5, 0.2, 0.1)
    cc = oracle32.matmul_fwd(a.reshape(m, k), b.reshape(k, n))
    cga, cgb = oracle32.matmul_bwd(a.reshape(m, k), b.reshape(k, n), seed.reshape(m, n))
    ga, gb = on_gpu(a, [m, k]), on_gpu(b, [k, n])
    gc = graph.matmul(ga, gb)
    assert np.abs(gpu.to_host(gc) - cc.ravel()).max() < 1e-3
    gpu.set_grad(gc, seed)
    backward_graph(gc)
    assert np.abs(gpu.read_grad(ga) - cga.ravel()).max() < 1e-3
    assert np.abs(gpu.read_grad(gb) - cgb.ravel()).max() < 1e-3


def _linear_inputs():
    batch, in_f, out_f = 16, 24, 10
    return (batch, in_f, out_f, seq(batch * in_f, 17, 0.1, -0.8), seq(in_f * out_f, 13, 0.05, -0.3),
            seq(out_f, 5, 0.2, -0.4))


def test_cuda_resident_linear_chain(gpu_ctx, oracle32):
    # tests/cuda_linear_test.rs:8-58
    batch, in_f, out_f, x, w, bias = _linear_inputs()
    seed = seq(batch * out_f, 7, 0.2, 0.1)
    z = oracle32.matmul_fwd(x.reshape(batch, in_f), w.reshape(in_f, out_f))
    cy = oracle32.bias_add_fwd(z, bias)
    _, cgb = oracle32.bias_add_bwd(seed.reshape(batch, out_f))
    cgx, cgw = oracle32.matmul_bwd(x.reshape(batch, in_f), w.reshape(in_f, out_f), seed.reshape(batch, out_f))
    gx, gw, gb = on_gpu(x, [batch, in_f]), on_gpu(w, [in_f, out_f]), on_gpu(bias, [out_f])
    gy = graph.add(graph.matmul(gx, gw), gb)
    assert np.abs(gpu.to_host(gy) - cy.ravel()).max() < 1e-3
    gpu.set_grad(gy, seed)
    backward_graph(gy)
    assert np.abs(gpu.read_grad(gx) - cgx.ravel()).max() < 1e-3
    assert np.abs(gpu.read_grad(gw) - cgw.ravel()).max() < 1e-3
    assert np.abs(gpu.read_grad(gb) - cgb.ravel()).max() < 1e-3
    # the struct form and the fused form agree with the chain
    gy2 = nn.Linear(gw, gb).forward(gx)
    assert np.abs(gpu.to_host(gy2) - cy.ravel()).max() < 1e-3
    gy3 = nn.linear_act(gx, gw, gb, 0)
    assert np.abs(gpu.to_host(gy3) - cy.ravel()).max() < 1e-3


def test_cuda_cross_entropy_through_linear(gpu_ctx, oracle32):
    # tests/cuda_ce_test.rs:10-59
    batch, in_f, classes, x, w, bias = _linear_inputs()
    target = np.zeros((batch, classes), np.float32)
    target[np.arange(batch), np.arange(batch) % classes] = 1.0
    logits = oracle32.bias_add_fwd(oracle32.matmul_fwd(x.reshape(batch, in_f), w.reshape(in_f, classes)), bias)
    cpu_loss = oracle32.ce_fwd(logits, target)
    g = oracle32.ce_bwd(logits, target)
    _, cgb = oracle32.bias_add_bwd(g)
    cgx, cgw = oracle32.matmul_bwd(x.reshape(batch, in_f), w.reshape(in_f, classes), g)
    gx, gw, gb, gt = on_gpu(x, [batch, in_f]), on_gpu(w, [in_f, classes]), on_gpu(bias, [classes]), on_gpu(target, [batch, classes])
    glogits = graph.add(graph.matmul(gx, gw), gb)
    gpu_loss = loss.cross_entropy(glogits, gt)
    loss.cross_entropy_backward(glogits, gt)
    backward_graph(glogits)
    assert abs(gpu_loss - cpu_loss) < 1e-3
    assert np.abs(gpu.read_grad(gx) - cgx.ravel()).max() < 1e-3
    assert np.abs(gpu.read_grad(gw) - cgw.ravel()).max() < 1e-3
    assert np.abs(gpu.read_grad(gb) - cgb.ravel()).max() < 1e-3


def test_cuda_adamw_matches_cpu(gpu_ctx, oracle32):
    # tests/cuda_adamw_test.rs:9-39
    n = 256
    init, grad = seq(n, 17, 0.1, -0.8), seq(n, 11, 0.05, -0.25)
    lr, b1, b2, eps, wd, steps = 0.001, 0.9, 0.999, 1e-8, 0.01, 10
    p, m, v = init.copy(), np.zeros(n, np.float32), np.zeros(n, np.float32)
    for t in range(steps):
        oracle32.adamw_step(p, grad, m, v, lr, b1, b2, eps, wd, t)
    gp = on_gpu(init, [n])
    gopt = optim.AdamW(lr, b1, b2, eps, wd)
    for _ in range(steps):
        gpu.set_grad(gp, grad)
        gopt.step([gp])
    assert np.abs(gpu.to_host(gp) - p).max() < 1e-4


def test_cuda_adamw_state_roundtrip(gpu_ctx):
    # tests/cuda_adamw_test.rs:41-83
    n = 64
    init = seq(n, 11, 0.1, -0.5)
    g1, g2, g3 = seq(n, 7, 0.05, 0.01), seq(n, 5, 0.04, -0.08), seq(n, 9, 0.03, 0.02)
    a, b = on_gpu(init, [n]), on_gpu(init, [n])
    oa, ob = optim.AdamW(0.01, 0.9, 0.999, 1e-8, 0.01), optim.AdamW(0.01, 0.9, 0.999, 1e-8, 0.01)
    for g in (g1, g2):
        gpu.set_grad(a, g); oa.step([a])
        gpu.set_grad(b, g); ob.step([b])
    t, moments = ob.export_state()
    assert t == 2 and len(moments) == 2
    ob2 = optim.AdamW(0.01, 0.9, 0.999, 1e-8, 0.01)
    ob2.import_state(t, moments)
    gpu.set_grad(a, g3); oa.step([a])
    gpu.set_grad(b, g3); ob2.step([b])
    assert np.abs(gpu.to_host(a) - gpu.to_host(b)).max() < 1e-6


def test_adamw_flat_and_per_tensor_agree(gpu_ctx):
    rng = np.random.default_rng(0)
    shapes = [(5, 7), (7,), (3, 3, 3, 3), (3,)]
    vals = [rng.normal(size=s).astype(np.float32) for s in shapes]
    grads = [rng.normal(size=s).astype(np.float32) for s in shapes]
    pa = [on_gpu(v, list(v.shape)) for v in vals]
    pb = [on_gpu(v, list(v.shape)) for v in vals]
    gpu.flatten_params(pb)
    oa, ob = optim.AdamW(0.01, 0.9, 0.999, 1e-8, 0.01), optim.AdamW(0.01, 0.9, 0.999, 1e-8, 0.01)
    for _ in range(3):
        for p, g in zip(pa, grads): gpu.set_grad(p, g)
        for p, g in zip(pb, grads): gpu.set_grad(p, g)
        oa.step(pa); ob.step(pb)
    # the flat launch takes the 128-bit path, single tensors may take the scalar tail:
    # same formula, fused-multiply-add contraction may differ by an ulp
    for p, q in zip(pa, pb):
        assert np.abs(gpu.to_host(p) - gpu.to_host(q)).max() <= 1e-6
    ta, ma = oa.export_state()
    tb, mb = ob.export_state()
    assert ta == tb == 3 and len(ma) == len(mb) == 8
    for x, y in zip(ma, mb):
        assert np.abs(x - y).max() <= 1e-6


@pytest.mark.parametrize("cfg", [(2, 3, 8, 8, 2, 2), (2, 3, 7, 7, 3, 1)])
def test_cuda_maxpool(gpu_ctx, oracle32, cfg):
    # tests/cuda_maxpool_test.rs:8-58
    n, c, in_h, in_w, k, stride = cfg
    in_len = n * c * in_h * in_w
    x = ((np.arange(in_len) * 31 + 7) % 97 * 0.05 - 2.0).astype(np.float32)
    cout, am = oracle32.maxpool_fwd(x.reshape(n, c, in_h, in_w), k, stride)
    seed = seq(cout.size, 7, 0.2, 0.1)
    c_igrad = oracle32.maxpool_bwd(seed, am, (n, c, in_h, in_w))
    gi = on_gpu(x, [n, c, in_h, in_w])
    gout = nn.maxpool2d(gi, k, stride)
    assert gout.shape == list(cout.shape)
    assert np.abs(gpu.to_host(gout) - cout.ravel()).max() < 1e-5
    gpu.set_grad(gout, seed)
    backward_graph(gout)
    assert np.abs(gpu.read_grad(gi) - c_igrad.ravel()).max() < 1e-4


def test_cuda_resident_relu_gelu_backward(gpu_ctx, oracle32):
    # tests/cuda_relu_test.rs:8-39 (+ the gelu twin, tests/cuda_activations_test.rs)
    n = 4096
    a, seed = seq(n, 21, 0.1, -1.0), seq(n, 7, 0.3, 0.1)
    for op, fwd, bwd, tol in ((graph.relu, oracle32.relu_fwd, oracle32.relu_bwd, 1e-4),
                              (graph.gelu, oracle32.gelu_fwd, oracle32.gelu_bwd, 1e-4)):
        ga = on_gpu(a, [n])
        gout = op(ga)
        assert np.abs(gpu.to_host(gout) - fwd(a)).max() < tol
        gpu.set_grad(gout, seed)
        backward_graph(gout)
        assert np.abs(gpu.read_grad(ga) - bwd(a, seed)).max() < tol


def test_branching_graph_accumulates(gpu_ctx, oracle32):
    # residual: y = relu(x) + x ; both paths add into x.grad (src/autograd/node.rs:113-126)
    n = 1000
    a, seed = seq(n, 21, 0.1, -1.0), seq(n, 7, 0.3, 0.1)
    ga = on_gpu(a, [n])
    y = graph.add(graph.relu(ga), ga)
    gpu.set_grad(y, seed)
    backward_graph(y)
    assert np.abs(gpu.read_grad(ga) - (oracle32.relu_bwd(a, seed) + seed)).max() < 1e-6


def test_layernorm_softmax_manip_graph(gpu_ctx, oracle64):
    rng = np.random.default_rng(5)
    rows, f = 12, 16
    x, g = rng.normal(size=(rows, f)).astype(np.float32), rng.normal(size=(rows, f)).astype(np.float32)
    gamma, beta = rng.normal(size=f).astype(np.float32), rng.normal(size=f).astype(np.float32)
    yr, xh, ist = oracle64.layernorm_fwd(x, gamma, beta, 1e-5)
    dxr, dgr, dbr = oracle64.layernorm_bwd(g, xh, ist, gamma)
    gx, gg, gb = on_gpu(x, [rows, f]), on_gpu(gamma, [f]), on_gpu(beta, [f])
    y = nn.layernorm(gx, gg, gb, 1e-5)
    assert np.abs(gpu.to_host(y) - yr.ravel()).max() < 1e-4
    gpu.set_grad(y, g)
    backward_graph(y)
    assert np.abs(gpu.read_grad(gx) - dxr.ravel()).max() < 1e-4
    assert np.abs(gpu.read_grad(gg) - dgr).max() < 1e-4
    assert np.abs(gpu.read_grad(gb) - dbr).max() < 1e-4
    # softmax -> slice -> concat -> transpose -> scale, gradients through the chain
    gx2 = on_gpu(x, [rows, f])
    s = graph.softmax(gx2)
    parts = [graph.slice_cols(s, 0, 8), graph.slice_cols(s, 8, 16)]
    cat = graph.concat_cols(parts[::-1])
    out = graph.scale(graph.transpose(graph.reshape(cat, [1, rows, f])), 0.5)
    assert out.shape == [1, f, rows]
    sr = oracle64.softmax_fwd(x)
    ref = 0.5 * np.concatenate([sr[:, 8:], sr[:, :8]], 1).T
    assert np.abs(gpu.to_host(out) - ref.ravel()).max() < 1e-6
    gt = rng.normal(size=(f, rows)).astype(np.float32)
    gpu.set_grad(out, gt)
    backward_graph(out)
    gcat = 0.5 * gt.T
    gs = np.concatenate([gcat[:, 8:], gcat[:, :8]], 1)
    assert np.abs(gpu.read_grad(gx2) - oracle64.softmax_bwd(sr, gs).ravel()).max() < 1e-5


def test_errors_are_reported_not_fatal(gpu_ctx):
    a, b = on_gpu(np.zeros(6), [2, 3]), on_gpu(np.zeros(8), [4, 2])
    with pytest.raises(cuda._lib.NrsError, match="inner dims"):
        graph.matmul(a, b)
    host_only = Node.new(np.zeros(6), [2, 3])
    with pytest.raises(cuda._lib.NrsError, match="not on GPU"):
        graph.relu(host_only)
    # the context is still usable afterwards
    assert np.all(gpu.to_host(graph.relu(a)) == 0)


def test_pool_over_fused_relu_conv_with_second_consumer(gpu_ctx, oracle64):
    """conv+ReLU (folded) feeds a max-pool AND a second consumer.  The pool's backward hands the
    convolution a gradient that already carries the ReLU mask; the other consumer adds an
    unmasked share.  Whatever the visiting order, the sum must end up masked exactly once."""
    rng = np.random.default_rng(12)
    n, ci, h, w, co = 2, 32, 8, 8, 32
    x = rng.normal(size=(n, ci, h, w)).astype(np.float32)
    wt = (rng.normal(size=(co, ci, 3, 3)) * 0.1).astype(np.float32)
    b = (rng.normal(size=co) * 0.1).astype(np.float32)
    gx, gw, gb = on_gpu(x, x.shape), on_gpu(wt, wt.shape), on_gpu(b, b.shape)
    z = oracle64.conv2d_fwd(x, wt, b, 1, 1)
    yr = oracle64.relu_fwd(z)
    _, am = oracle64.maxpool_fwd(yr, 2, 2)
    for pool_first in (True, False):
        y = nn.conv2d_act(gx, gw, gb, 1, 1, 1)
        pooled = nn.maxpool2d(y, 2, 2)
        scaled = graph.scale(y, 0.5)
        parts = [graph.reshape(pooled, [1, len(pooled)]), graph.reshape(scaled, [1, len(scaled)])]
        sp = rng.normal(size=len(pooled)).astype(np.float32)
        ss = rng.normal(size=len(scaled)).astype(np.float32)
        # the branch listed LAST is visited first by the reverse topological walk
        both = graph.concat_cols(parts[::-1] if pool_first else parts)
        seed = np.concatenate([ss, sp] if pool_first else [sp, ss])
        gpu.zero_grad([gx, gw, gb])
        gpu.set_grad(both, seed)
        backward_graph(both)
        dy = oracle64.maxpool_bwd(sp.reshape(n, co, h // 2, w // 2), am, yr.shape) + 0.5 * ss.reshape(yr.shape)
        dxr, dwr, dbr = oracle64.conv2d_bwd(x, wt, oracle64.relu_bwd(z, dy), 1, 1)
        assert np.linalg.norm(gpu.read_grad(gw) - dwr.ravel()) <= 1e-4 * np.linalg.norm(dwr)
        assert np.linalg.norm(gpu.read_grad(gx) - dxr.ravel()) <= 1e-4 * np.linalg.norm(dxr)
        assert np.linalg.norm(gpu.read_grad(gb) - dbr.ravel()) <= 1e-4 * np.linalg.norm(dbr)


def test_conv_over_fused_relu_conv_with_second_consumer(gpu_ctx, oracle64):
    """conv+ReLU (folded) feeds a second convolution AND another consumer.  The second
    convolution's data-gradient kernel applies the first one's ReLU mask in its epilogue and
    leaves the gradient's operand planes; the other consumer adds an unmasked share.  Whatever
    the visiting order, the first convolution must see the masked sum."""
    rng = np.random.default_rng(13)
    n, ci, h, w, c1, c2 = 2, 32, 8, 8, 64, 32
    x = rng.normal(size=(n, ci, h, w)).astype(np.float32)
    w1 = (rng.normal(size=(c1, ci, 3, 3)) * 0.1).astype(np.float32)
    b1 = (rng.normal(size=c1) * 0.1).astype(np.float32)
    w2 = (rng.normal(size=(c2, c1, 3, 3)) * 0.1).astype(np.float32)
    b2 = (rng.normal(size=c2) * 0.1).astype(np.float32)
    gx, gw1, gb1 = on_gpu(x, x.shape), on_gpu(w1, w1.shape), on_gpu(b1, b1.shape)
    gw2, gb2 = on_gpu(w2, w2.shape), on_gpu(b2, b2.shape)
    z1 = oracle64.conv2d_fwd(x, w1, b1, 1, 1)
    y1 = oracle64.relu_fwd(z1)
    for conv_first in (True, False):
        y = nn.conv2d_act(gx, gw1, gb1, 1, 1, 1)
        y2 = nn.conv2d(y, gw2, gb2, 1, 1)
        scaled = graph.scale(y, 0.5)
        parts = [graph.reshape(y2, [1, len(y2)]), graph.reshape(scaled, [1, len(scaled)])]
        s2 = rng.normal(size=len(y2)).astype(np.float32)
        ss = rng.normal(size=len(scaled)).astype(np.float32)
        # the branch listed LAST is visited first by the reverse topological walk
        both = graph.concat_cols(parts[::-1] if conv_first else parts)
        seed = np.concatenate([ss, s2] if conv_first else [s2, ss])
        params = [gx, gw1, gb1, gw2, gb2]
        gpu.zero_grad(params)
        gpu.set_grad(both, seed)
        backward_graph(both)
        dy2 = s2.reshape(n, c2, h, w)
        dy1_from_conv, dw2r, db2r = oracle64.conv2d_bwd(y1, w2, dy2, 1, 1)
        dy1 = dy1_from_conv + 0.5 * ss.reshape(y1.shape)
        dxr, dw1r, db1r = oracle64.conv2d_bwd(x, w1, oracle64.relu_bwd(z1, dy1), 1, 1)
        for got, want in ((gw2, dw2r), (gb2, db2r), (gw1, dw1r), (gb1, db1r), (gx, dxr)):
            assert np.linalg.norm(gpu.read_grad(got) - want.ravel()) <= 1e-4 * np.linalg.norm(want)


@pytest.mark.parametrize("chans", [[32, 64, 64, 32], [3, 32, 64, 32]])   # second: image layer on the FFMA kernels
@pytest.mark.parametrize("n,h,w", [(3, 16, 16), (20, 32, 32)])   # split-K reduce store / direct epilogue
@pytest.mark.parametrize("mode", ["3xtf32", "tf32", "fp32"])
def test_conv_relu_conv_chain_all_modes(gpu_ctx, oracle64, mode, n, h, w, chans):
    """Three stacked conv+ReLU layers (no pooling): every inner gradient reaches its producer
    through the data-gradient epilogue (mask folded, planes emitted) in the tensor-core modes
    and through the separate passes in FP32 mode."""
    from neuralrs_b200 import cuda as api
    modes = {"3xtf32": 0, "tf32": 1, "fp32": 2}
    tol = {"3xtf32": 1e-4, "tf32": 1e-2, "fp32": 1e-4}[mode]
    rng = np.random.default_rng(14)
    x = rng.normal(size=(n, chans[0], h, w)).astype(np.float32)
    ws = [(rng.normal(size=(chans[i + 1], chans[i], 3, 3)) * np.sqrt(2.0 / (9 * chans[i]))).astype(np.float32) for i in range(3)]
    bs = [(rng.normal(size=chans[i + 1]) * 0.1).astype(np.float32) for i in range(3)]
    gpu_ctx.set_math_mode(modes[mode])
    try:
        gx = on_gpu(x, x.shape)
        gws = [on_gpu(a, a.shape) for a in ws]
        gbs = [on_gpu(a, a.shape) for a in bs]
        hcur = gx
        outs = []
        for i in range(3):
            hcur = nn.conv2d_act(hcur, gws[i], gbs[i], 1, 1, 1)
            outs.append(hcur)
        seed = rng.normal(size=len(hcur)).astype(np.float32)
        gpu.zero_grad([gx] + gws + gbs)
        gpu.set_grad(hcur, seed)
        backward_graph(hcur)
        # oracle
        acts, zs = [x], []
        for i in range(3):
            z = oracle64.conv2d_fwd(acts[-1], ws[i], bs[i], 1, 1)
            zs.append(z)
            acts.append(oracle64.relu_fwd(z))
        assert np.linalg.norm(gpu.to_host(hcur) - acts[-1].ravel()) <= tol * np.linalg.norm(acts[-1])
        # A pre-activation within rounding error of zero may fall on the other side of the ReLU on
        # the device; one flipped element moves a gradient by far more than the tolerance.  The
        # backward pass is therefore checked with the ReLU masks the device actually used.
        g = seed.reshape(acts[-1].shape)
        for i in (2, 1, 0):
            mask_src = gpu.to_host(outs[i]).reshape(zs[i].shape)
            assert np.mean((mask_src > 0) != (zs[i] > 0)) < 1e-3
            g, dw, db = oracle64.conv2d_bwd(acts[i], ws[i], oracle64.relu_bwd(mask_src, g), 1, 1)
            assert np.linalg.norm(gpu.read_grad(gws[i]) - dw.ravel()) <= tol * np.linalg.norm(dw), (mode, i)
            assert np.linalg.norm(gpu.read_grad(gbs[i]) - db.ravel()) <= tol * np.linalg.norm(db), (mode, i)
        assert np.linalg.norm(gpu.read_grad(gx) - g.ravel()) <= tol * np.linalg.norm(g)
    finally:
        gpu_ctx.set_math_mode(0)


def test_reuploaded_input_node_restages_its_operand_planes(gpu_ctx, oracle64):
    # One input node, two uploads: the convolution after the second upload must see the new values
    # (the tensor-core path caches re-laid-out operand planes per node), forward and weight gradient.
    rng = np.random.default_rng(77)
    n, ci, h, w, co = 4, 32, 16, 16, 64
    wt = (rng.standard_normal((co, ci, 3, 3)) * 0.1).astype(np.float32)
    b = np.zeros(co, np.float32)
    gw, gb = on_gpu(wt, list(wt.shape)), on_gpu(b, [co])
    xs = [rng.standard_normal((n, ci, h, w)).astype(np.float32) for _ in range(3)]
    seed = rng.standard_normal((n, co, h, w)).astype(np.float32)
    gx = Node.new(xs[0], list(xs[0].shape))
    for step, x in enumerate(xs):
        if step == 2:        # written in place through the device pointer, then declared
            import ctypes as C
            from neuralrs_b200 import _lib
            _lib.check(gpu_ctx.h, _lib.lib().nrs_h2d(gpu_ctx.h, C.c_void_p(gx.data_ptr()), C.c_void_p(x.ctypes.data), x.nbytes))
            gpu_ctx.sync()
            gx.invalidate()
        else:
            gx.set_data(x)
            gpu.to_cuda(gx)
        gpu.zero_grad([gw, gb])
        out = nn.conv2d(gx, gw, gb, 1, 1)
        ref = oracle64.conv2d_fwd(x, wt, b, 1, 1)
        assert np.linalg.norm(gpu.to_host(out) - ref.ravel()) <= 1e-4 * np.linalg.norm(ref), f"forward after upload {step}"
        gpu.set_grad(out, seed)
        backward_graph(out)
        _, dw, _ = oracle64.conv2d_bwd(x, wt, seed, 1, 1)
        assert np.linalg.norm(gpu.read_grad(gw) - dw.ravel()) <= 1e-4 * np.linalg.norm(dw), f"weight gradient after upload {step}"
