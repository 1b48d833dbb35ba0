"""ctypes mirror of the reference's ``neuralrs::cuda`` API over the node-level C ABI.

Names and argument order follow the Rust functions so a test can be read next to
the reference's own (``tests/cuda_*.rs``):

    gi = Node.new(input, [n, c_in, h, w]); runtime.to_cuda(gi)
    gout = nn.conv2d(gi, gw, gb, stride, pad)
    runtime.set_grad(gout, seed); backward_graph(gout)
    g = runtime.read_grad(gi)

All arithmetic happens in libnrs_b200.so on the GPU; this file only marshals
numpy arrays and handles.  Reference: src/cuda/{runtime,graph,nn,loss,optim}.
"""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import _lib
from ._lib import VP, check

_default_ctx = None


class Context:
    """One device context + stream (the reference's global backend, src/cuda/backend.rs:17-32)."""

    def __init__(self, device: int = 0):
        self._l = _lib.lib()
        h = VP()
        st = self._l.nrs_init(device, C.byref(h))
        if st != 0:
            raise _lib.NrsError(st, (self._l.nrs_last_error(None) or b"").decode())
        self.h = h
        self.device = device

    def set_math_mode(self, mode: int):
        check(self.h, self._l.nrs_set_math_mode(self.h, mode))

    def set_stream(self, stream_ptr: int | None):
        check(self.h, self._l.nrs_set_stream(self.h, VP(stream_ptr or 0)))

    def sync(self):
        check(self.h, self._l.nrs_sync(self.h))

    def launch_count(self) -> int:
        return int(self._l.nrs_launch_count(self.h))

    def close(self):
        if self.h:
            self._l.nrs_destroy(self.h)
            self.h = None


def default_context() -> Context:
    global _default_ctx
    if _default_ctx is None:
        _default_ctx = Context(0)
    return _default_ctx


def set_default_context(ctx: Context | None):
    global _default_ctx
    _default_ctx = ctx


def _f32(a) -> np.ndarray:
    return np.ascontiguousarray(np.asarray(a, dtype=np.float32))


def _ptr(a: np.ndarray) -> VP:
    return VP(a.ctypes.data)


class Node:
    """Handle to a graph node (src/autograd/node.rs:38-53)."""

    def __init__(self, handle: VP, ctx: Context):
        self.h = handle
        self.ctx = ctx

    @staticmethod
    def new(data, shape, ctx: Context | None = None) -> "Node":
        ctx = ctx or default_context()
        shape = [int(s) for s in shape]
        arr = _f32(data).reshape(-1)
        if arr.size != int(np.prod(shape, dtype=np.int64)) and arr.size != 0:
            raise ValueError("data does not match shape")
        sh = (C.c_int64 * len(shape))(*shape)
        h = VP()
        check(ctx.h, ctx._l.nrs_node_new(ctx.h, _ptr(arr) if arr.size else None, sh, len(shape), C.byref(h)))
        return Node(h, ctx)

    @property
    def shape(self) -> list[int]:
        l = self.ctx._l
        nd = l.nrs_node_ndim(self.h)
        buf = (C.c_int64 * max(nd, 1))()
        check(self.ctx.h, l.nrs_node_shape(self.h, buf, nd))
        return [int(buf[i]) for i in range(nd)]

    def __len__(self) -> int:
        return int(self.ctx._l.nrs_node_len(self.h))

    @property
    def requires_grad(self):
        raise AttributeError("write-only")

    @requires_grad.setter
    def requires_grad(self, flag: bool):
        check(self.ctx.h, self.ctx._l.nrs_node_set_requires_grad(self.h, int(bool(flag))))

    def set_data(self, data):
        """New host contents for the node (uploaded by the next runtime.to_cuda)."""
        arr = _f32(data).reshape(-1)
        if arr.size != len(self):
            raise ValueError("data does not match the node's length")
        check(self.ctx.h, self.ctx._l.nrs_node_set_data(self.h, _ptr(arr)))

    def invalidate(self):
        """After writing new values through data_ptr(): drops the operand planes cached for the old ones."""
        check(self.ctx.h, self.ctx._l.nrs_node_invalidate(self.h))

    def data_ptr(self) -> int:
        return int(self.ctx._l.nrs_node_data_ptr(self.h) or 0)

    def grad_ptr(self) -> int:
        return int(self.ctx._l.nrs_node_grad_ptr(self.h) or 0)

    def __del__(self):
        try:
            if self.h and self.ctx.h:
                self.ctx._l.nrs_node_release(self.h)
        except Exception:
            pass
        self.h = None


def _out(ctx: Context, st: int, h: VP) -> Node:
    check(ctx.h, st)
    return Node(h, ctx)


def _handles(nodes):
    arr = (VP * len(nodes))(*[n.h for n in nodes])
    return arr


class runtime:
    """src/cuda/runtime.rs:39-124."""

    @staticmethod
    def to_cuda(n: Node):
        check(n.ctx.h, n.ctx._l.nrs_to_cuda(n.h))

    @staticmethod
    def to_host(n: Node) -> np.ndarray:
        out = np.empty(len(n), dtype=np.float32)
        check(n.ctx.h, n.ctx._l.nrs_to_host(n.h, _ptr(out)))
        return out

    @staticmethod
    def set_grad(n: Node, grad):
        g = _f32(grad).reshape(-1)
        if g.size != len(n):
            raise ValueError("gradient size mismatch")
        check(n.ctx.h, n.ctx._l.nrs_set_grad(n.h, _ptr(g)))

    @staticmethod
    def read_grad(n: Node) -> np.ndarray:
        out = np.empty(len(n), dtype=np.float32)
        check(n.ctx.h, n.ctx._l.nrs_read_grad(n.h, _ptr(out)))
        return out

    @staticmethod
    def zero_grad(params):
        if params:
            check(params[0].ctx.h, params[0].ctx._l.nrs_zero_grad(_handles(params), len(params)))

    @staticmethod
    def flatten_params(params):
        check(params[0].ctx.h, params[0].ctx._l.nrs_flatten_params(_handles(params), len(params)))

    @staticmethod
    def synchronize(ctx: Context | None = None):
        (ctx or default_context()).sync()


def _unary(name):
    def f(x: Node) -> Node:
        h = VP()
        return _out(x.ctx, getattr(x.ctx._l, name)(x.h, C.byref(h)), h)
    return staticmethod(f)


def _binary(name):
    def f(a: Node, b: Node) -> Node:
        h = VP()
        return _out(a.ctx, getattr(a.ctx._l, name)(a.h, b.h, C.byref(h)), h)
    return staticmethod(f)


class graph:
    """src/cuda/graph/*.rs."""
    matmul = _binary("nrs_op_matmul")
    add = _binary("nrs_op_add")
    bmm = _binary("nrs_op_bmm")
    relu = _unary("nrs_op_relu")
    gelu = _unary("nrs_op_gelu")
    softmax = _unary("nrs_op_softmax")
    transpose = _unary("nrs_op_transpose")
    causal_mask = _unary("nrs_op_causal_mask")   # extension: the reference has no mask

    @staticmethod
    def reshape(x: Node, shape) -> Node:
        sh = (C.c_int64 * len(shape))(*[int(s) for s in shape])
        h = VP()
        return _out(x.ctx, x.ctx._l.nrs_op_reshape(x.h, sh, len(shape), C.byref(h)), h)

    @staticmethod
    def scale(x: Node, s: float) -> Node:
        h = VP()
        return _out(x.ctx, x.ctx._l.nrs_op_scale(x.h, C.c_float(s), C.byref(h)), h)

    @staticmethod
    def slice_cols(x: Node, c0: int, c1: int) -> Node:
        h = VP()
        return _out(x.ctx, x.ctx._l.nrs_op_slice_cols(x.h, int(c0), int(c1), C.byref(h)), h)

    @staticmethod
    def concat_cols(parts) -> Node:
        h = VP()
        return _out(parts[0].ctx, parts[0].ctx._l.nrs_op_concat_cols(_handles(parts), len(parts), C.byref(h)), h)


class nn:
    """src/cuda/nn/{conv,maxpool,flatten,normalization,linear}.rs."""
    flatten = _unary("nrs_op_flatten")

    @staticmethod
    def conv2d(x: Node, w: Node, b: Node, stride: int, pad: int) -> Node:
        h = VP()
        return _out(x.ctx, x.ctx._l.nrs_op_conv2d(x.h, w.h, b.h, int(stride), int(pad), C.byref(h)), h)

    @staticmethod
    def conv2d_act(x: Node, w: Node, b: Node, stride: int, pad: int, act: int) -> Node:
        h = VP()
        return _out(x.ctx, x.ctx._l.nrs_op_conv2d_act(x.h, w.h, b.h, int(stride), int(pad), int(act), C.byref(h)), h)

    @staticmethod
    def maxpool2d(x: Node, kernel: int, stride: int) -> Node:
        h = VP()
        return _out(x.ctx, x.ctx._l.nrs_op_maxpool2d(x.h, int(kernel), int(stride), C.byref(h)), h)

    @staticmethod
    def layernorm(x: Node, gamma: Node, beta: Node, eps: float) -> Node:
        h = VP()
        return _out(x.ctx, x.ctx._l.nrs_op_layernorm(x.h, gamma.h, beta.h, C.c_float(eps), C.byref(h)), h)

    @staticmethod
    def batchnorm(x: Node, gamma: Node, beta: Node, running_mean: Node, running_var: Node, momentum: float,
                  eps: float, training: bool) -> Node:
        """src/cuda/nn/batchnorm.rs:110-232: x [batch, features]; the running statistics are updated in place."""
        h = VP()
        return _out(x.ctx, x.ctx._l.nrs_op_batchnorm(x.h, gamma.h, beta.h, running_mean.h, running_var.h,
                                                      C.c_float(momentum), C.c_float(eps), int(training), C.byref(h)), h)

    @staticmethod
    def batchnorm2d(x: Node, gamma: Node, beta: Node, running_mean: Node, running_var: Node, momentum: float,
                    eps: float, training: bool) -> Node:
        """src/cuda/nn/batchnorm2d.rs:130-232: x [batch, channels, h, w]."""
        h = VP()
        return _out(x.ctx, x.ctx._l.nrs_op_batchnorm2d(x.h, gamma.h, beta.h, running_mean.h, running_var.h,
                                                        C.c_float(momentum), C.c_float(eps), int(training), C.byref(h)), h)

    @staticmethod
    def batchnorm_act(x: Node, gamma: Node, beta: Node, running_mean: Node, running_var: Node, momentum: float,
                      eps: float, training: bool, act: int) -> Node:
        """batchnorm / batchnorm2d (by rank) with the following ReLU fused (act: _lib.ACT_NONE / ACT_RELU)."""
        h = VP()
        return _out(x.ctx, x.ctx._l.nrs_op_batchnorm_act(x.h, gamma.h, beta.h, running_mean.h, running_var.h,
                                                          C.c_float(momentum), C.c_float(eps), int(training), int(act),
                                                          C.byref(h)), h)

    @staticmethod
    def dropout(x: Node, p: float, training: bool, mask: Node | None = None) -> Node:
        """src/cuda/nn/dropout.rs:31-84.  mask=None draws the mask on the device (context seed and counter)."""
        h = VP()
        return _out(x.ctx, x.ctx._l.nrs_op_dropout(x.h, C.c_float(p), int(training), mask.h if mask else None, C.byref(h)), h)

    @staticmethod
    def dropout2d(x: Node, p: float, training: bool, mask: Node | None = None) -> Node:
        """src/cuda/nn/dropout2d.rs: one mask value per (sample, channel) plane."""
        h = VP()
        return _out(x.ctx, x.ctx._l.nrs_op_dropout2d(x.h, C.c_float(p), int(training), mask.h if mask else None, C.byref(h)), h)

    @staticmethod
    def linear_act(x: Node, w: Node, b: Node, act: int) -> Node:
        h = VP()
        return _out(x.ctx, x.ctx._l.nrs_op_linear_act(x.h, w.h, b.h, int(act), C.byref(h)), h)

    @staticmethod
    def attention_batch(q: Node, k: Node, v: Node, causal: bool = False) -> Node:
        """src/cuda/nn/attention.rs:23-32 (causal is an extension)."""
        h = VP()
        return _out(q.ctx, q.ctx._l.nrs_op_attention_batch(q.h, k.h, v.h, int(causal), C.byref(h)), h)

    class LayerNorm:
        """src/cuda/nn/normalization.rs (struct form)."""

        def __init__(self, gamma: Node, beta: Node, eps: float = 1e-5):
            self.gamma, self.beta, self.eps = gamma, beta, eps

        def forward(self, x: Node) -> Node:
            return nn.layernorm(x, self.gamma, self.beta, self.eps)

    class Embedding:
        """src/cuda/nn/embedding.rs:41-100; forward_batch mirrors src/nn/embedding.rs:60-113."""

        def __init__(self, weight: Node, vocab_size: int, embedding_dim: int):
            self.weight, self.vocab_size, self.embedding_dim = weight, vocab_size, embedding_dim

        def forward(self, indices) -> Node:
            idx = np.ascontiguousarray(indices, dtype=np.int32).reshape(-1)
            h = VP()
            l = self.weight.ctx._l
            return _out(self.weight.ctx, l.nrs_op_embedding(self.weight.h, _ptr(idx), idx.size, C.byref(h)), h)

        def forward_batch(self, batch_indices) -> Node:
            idx = np.ascontiguousarray(batch_indices, dtype=np.int32)
            b, s = idx.shape
            h = VP()
            l = self.weight.ctx._l
            return _out(self.weight.ctx, l.nrs_op_embedding_batch(self.weight.h, _ptr(idx), b, s, C.byref(h)), h)

    class PositionalEncoding:
        """src/cuda/nn/positional.rs:18-44; the table is built once and stays on the device."""

        def __init__(self, d_model: int, max_len: int, ctx: Context | None = None):
            ctx = ctx or default_context()
            h = VP()
            check(ctx.h, ctx._l.nrs_positional_new(ctx.h, int(d_model), int(max_len), C.byref(h)))
            self.table = Node(h, ctx)
            self.d_model, self.max_len = d_model, max_len

        def forward(self, x: Node) -> Node:
            h = VP()
            return _out(x.ctx, x.ctx._l.nrs_op_positional(x.h, self.table.h, C.byref(h)), h)

    class MultiHeadAttention:
        """src/cuda/nn/multihead.rs:20-85 (weights [d,d], no biases)."""

        def __init__(self, w_q, w_k, w_v, w_o, d_model: int, num_heads: int, causal: bool = False):
            self.w_q, self.w_k, self.w_v, self.w_o = w_q, w_k, w_v, w_o
            self.d_model, self.num_heads, self.causal = d_model, num_heads, causal

        def parameters(self):
            return [self.w_q, self.w_k, self.w_v, self.w_o]

        def forward_batch(self, x: Node) -> Node:
            h = VP()
            return _out(x.ctx, x.ctx._l.nrs_op_mha(x.h, self.w_q.h, self.w_k.h, self.w_v.h, self.w_o.h,
                                                  int(self.num_heads), int(self.causal), C.byref(h)), h)

    class TransformerBlock:
        """src/cuda/nn/transformer_block.rs:14-60."""

        def __init__(self, mha, norm1, norm2, ff1, ff2, d_model: int, d_ff: int, act: int = 1):
            self.mha, self.norm1, self.norm2, self.ff1, self.ff2 = mha, norm1, norm2, ff1, ff2
            self.d_model, self.d_ff, self.act = d_model, d_ff, act

        def parameters(self):
            return self.mha.parameters() + [self.norm1.gamma, self.norm1.beta, self.norm2.gamma, self.norm2.beta,
                                            self.ff1.weights, self.ff1.bias, self.ff2.weights, self.ff2.bias]

        def _run(self, x: Node, final_norm: bool) -> Node:
            h = VP()
            return _out(x.ctx, x.ctx._l.nrs_op_transformer_block(
                x.h, _handles(self.parameters()), int(self.mha.num_heads), C.c_float(self.norm1.eps), int(self.act),
                int(self.mha.causal), int(final_norm), C.byref(h)), h)

        def forward(self, x: Node) -> Node:
            return self._run(x, True)

        def forward_no_final_norm(self, x: Node) -> Node:
            return self._run(x, False)

    class Linear:
        """weights [in, out], bias [out]; forward = add(matmul(x, W), b) (src/cuda/nn/linear.rs:11-26)."""

        def __init__(self, weights: Node, bias: Node):
            self.weights, self.bias = weights, bias

        def forward(self, x: Node) -> Node:
            return graph.add(graph.matmul(x, self.weights), self.bias)


class loss:
    """src/cuda/loss/cross_entropy.rs:74-128."""

    @staticmethod
    def cross_entropy(pred: Node, target: Node) -> float:
        out = C.c_float()
        check(pred.ctx.h, pred.ctx._l.nrs_cross_entropy(pred.h, target.h, C.byref(out)))
        return float(out.value)

    @staticmethod
    def cross_entropy_backward(pred: Node, target: Node):
        check(pred.ctx.h, pred.ctx._l.nrs_cross_entropy_backward(pred.h, target.h))


def backward_graph(root: Node):
    """src/autograd/node.rs:113-126."""
    check(root.ctx.h, root.ctx._l.nrs_backward_graph(root.h))


class optim:
    class AdamW:
        """src/cuda/optim/adamw.rs:43-144."""

        def __init__(self, lr, beta1, beta2, epsilon, weight_decay, ctx: Context | None = None):
            self.ctx = ctx or default_context()
            h = VP()
            check(self.ctx.h, self.ctx._l.nrs_adamw_new(self.ctx.h, C.c_float(lr), C.c_float(beta1), C.c_float(beta2),
                                                         C.c_float(epsilon), C.c_float(weight_decay), C.byref(h)))
            self.h = h

        @property
        def t(self) -> int:
            return int(self.ctx._l.nrs_adamw_t(self.h))

        def step(self, params):
            check(self.ctx.h, self.ctx._l.nrs_adamw_step_nodes(self.h, _handles(params), len(params)))

        def export_state(self):
            l = self.ctx._l
            n = l.nrs_adamw_state_count(self.h)
            if n < 0:
                check(self.ctx.h, 4)
            out = []
            for i in range(n):
                a = np.empty(int(l.nrs_adamw_state_len(self.h, i)), dtype=np.float32)
                check(self.ctx.h, l.nrs_adamw_state_get(self.h, i, _ptr(a)))
                out.append(a)
            return self.t, out

        def import_state(self, t: int, moments):
            arrs = [_f32(m).reshape(-1) for m in moments]
            ptrs = (VP * len(arrs))(*[a.ctypes.data for a in arrs])
            lens = (C.c_int64 * len(arrs))(*[a.size for a in arrs])
            check(self.ctx.h, self.ctx._l.nrs_adamw_import_state(self.h, int(t), ptrs, lens, len(arrs)))

        def __del__(self):
            try:
                if self.h and self.ctx.h:
                    self.ctx._l.nrs_adamw_free(self.h)
            except Exception:
                pass
            self.h = None


LAYER_KINDS = {"conv": 0, "relu": 1, "maxpool": 2, "flatten": 3, "linear": 4, "gelu": 5, "batchnorm": 6, "dropout": 7,
               "dropout2d": 8, "embedding": 9, "transformer_block": 10, "layernorm": 11}


class _LayerSpec(C.Structure):
    _fields_ = [("kind", C.c_int), ("a", C.c_int), ("b", C.c_int), ("c", C.c_int), ("d", C.c_int), ("e", C.c_int)]


class Trainer:
    """Native training loop for a sequential model (include/nrs_graph.h, nrs_trainer_*).

    `layers` uses the tuples ("conv", c_in, c_out, k, stride, pad), ("relu",), ("gelu",),
    ("maxpool", k, stride), ("flatten",), ("linear", n_in, n_out), ("batchnorm", channels),
    ("dropout", p), ("dropout2d", p), and for token models ("embedding", vocab, d_model, max_len) as the first
    layer, ("transformer_block", d_model, heads, d_ff, act, flags), ("layernorm", features); see
    neuralrs_b200/workloads.py.
    """

    def __init__(self, layers, in_shape, classes, lr=1e-3, beta1=0.9, beta2=0.999, eps=1e-8, wd=1e-4,
                 fuse=True, ctx: Context | None = None):
        self.ctx = ctx or default_context()
        l = self.ctx._l
        specs = (_LayerSpec * len(layers))()
        for i, ly in enumerate(layers):
            if ly[0] in ("dropout", "dropout2d"):      # the probability crosses as parts per million
                vals = [LAYER_KINDS[ly[0]], int(round(float(ly[1]) * 1e6))]
            else:
                vals = [LAYER_KINDS[ly[0]]] + [int(v) for v in ly[1:]]
            vals += [0] * (6 - len(vals))
            specs[i] = _LayerSpec(*vals)
        shp = (C.c_int64 * len(in_shape))(*[int(s) for s in in_shape])
        h = VP()
        check(self.ctx.h, l.nrs_trainer_create(self.ctx.h, specs, len(layers), shp, len(in_shape), int(classes),
                                               C.c_float(lr), C.c_float(beta1), C.c_float(beta2), C.c_float(eps),
                                               C.c_float(wd), int(bool(fuse)), C.byref(h)))
        self.h = h
        self.in_shape = tuple(int(s) for s in in_shape)
        self.classes = int(classes)

    @property
    def n_params(self) -> int:
        return int(self.ctx._l.nrs_trainer_param_count(self.h))

    def param_len(self, i: int) -> int:
        return int(self.ctx._l.nrs_trainer_param_len(self.h, i))

    def set_params(self, params):
        assert len(params) == self.n_params
        for i, p in enumerate(params):
            a = _f32(p).reshape(-1)
            assert a.size == self.param_len(i)
            check(self.ctx.h, self.ctx._l.nrs_trainer_set_param(self.h, i, _ptr(a)))

    def get_param(self, i: int) -> np.ndarray:
        out = np.empty(self.param_len(i), np.float32)
        check(self.ctx.h, self.ctx._l.nrs_trainer_get_param(self.h, i, _ptr(out)))
        return out

    def get_grad(self, i: int) -> np.ndarray:
        out = np.empty(self.param_len(i), np.float32)
        check(self.ctx.h, self.ctx._l.nrs_trainer_get_grad(self.h, i, _ptr(out)))
        return out

    @property
    def n_buffers(self) -> int:
        return int(self.ctx._l.nrs_trainer_buffer_count(self.h))

    def get_buffer(self, i: int) -> np.ndarray:
        """Running statistics of the batchnorm layers: [mean0, var0, mean1, var1, ...]."""
        out = np.empty(int(self.ctx._l.nrs_trainer_buffer_len(self.h, i)), np.float32)
        check(self.ctx.h, self.ctx._l.nrs_trainer_get_buffer(self.h, i, _ptr(out)))
        return out

    def set_buffer(self, i: int, values):
        a = _f32(values).reshape(-1)
        assert a.size == int(self.ctx._l.nrs_trainer_buffer_len(self.h, i))
        check(self.ctx.h, self.ctx._l.nrs_trainer_set_buffer(self.h, i, _ptr(a)))

    def save_checkpoint(self, path: str, names=None):
        """Parameters, batchnorm running statistics and the AdamW state (optim.t, optim.m.NN, optim.v.NN)."""
        arr = (C.c_char_p * len(names))(*[n.encode() for n in names]) if names else None
        check(self.ctx.h, self.ctx._l.nrs_trainer_save_checkpoint(self.h, arr, str(path).encode()))

    def load_checkpoint(self, path: str, names=None):
        arr = (C.c_char_p * len(names))(*[n.encode() for n in names]) if names else None
        check(self.ctx.h, self.ctx._l.nrs_trainer_load_checkpoint(self.h, arr, str(path).encode()))

    def set_training(self, training: bool):
        check(self.ctx.h, self.ctx._l.nrs_trainer_set_training(self.h, int(bool(training))))

    def _host_call(self, fn, x, target, want_loss):
        x, target = _f32(x), _f32(target)
        batch = x.shape[0]
        loss = C.c_float()
        check(self.ctx.h, fn(self.h, _ptr(x), _ptr(target), batch, C.byref(loss) if want_loss else None))
        return float(loss.value) if want_loss else None

    def forward_backward(self, x, target, want_loss=True):
        return self._host_call(self.ctx._l.nrs_trainer_forward_backward, x, target, want_loss)

    def step(self, x, target, want_loss=True):
        return self._host_call(self.ctx._l.nrs_trainer_step, x, target, want_loss)

    def step_ptr(self, x_host_ptr: int, target_host_ptr: int, batch: int, want_loss=True):
        """Step from raw HOST pointers (e.g. pinned torch tensors)."""
        loss = C.c_float()
        check(self.ctx.h, self.ctx._l.nrs_trainer_step(self.h, VP(x_host_ptr), VP(target_host_ptr), int(batch),
                                                       C.byref(loss) if want_loss else None))
        return float(loss.value) if want_loss else None

    def stage_next_ptr(self, x_host_ptr: int, target_host_ptr: int, batch: int):
        """Starts the asynchronous copy of a batch from (pinned) HOST pointers into the idle staging slot."""
        check(self.ctx.h, self.ctx._l.nrs_trainer_stage_next(self.h, VP(x_host_ptr), VP(target_host_ptr), int(batch)))

    def stage_next(self, x, target):
        """As stage_next_ptr for numpy arrays; the arrays are kept alive until their step has been issued."""
        x, target = _f32(x), _f32(target)
        self._staged = getattr(self, "_staged", []) + [(x, target)]
        self.stage_next_ptr(x.ctypes.data, target.ctypes.data, x.shape[0])

    def stage_next_indexed(self, x, labels):
        """As stage_next with int32 class indices; the step expands them to one-hot rows on the device."""
        x = _f32(x)
        labels = np.ascontiguousarray(labels, np.int32)
        self._staged = getattr(self, "_staged", []) + [(x, labels)]
        check(self.ctx.h, self.ctx._l.nrs_trainer_stage_next_indexed(self.h, VP(x.ctypes.data), VP(labels.ctypes.data),
                                                                      int(x.shape[0])))

    def set_augment(self, max_shift: int, flip: bool = True):
        """On-device flip/shift augmentation of staged batches (max_shift < 0: off)."""
        check(self.ctx.h, self.ctx._l.nrs_trainer_set_augment(self.h, int(max_shift), int(bool(flip))))

    def step_staged(self, want_loss=True):
        """A full training step on the oldest staged batch."""
        loss = C.c_float()
        check(self.ctx.h, self.ctx._l.nrs_trainer_step_staged(self.h, C.byref(loss) if want_loss else None))
        if want_loss and getattr(self, "_staged", None):
            self._staged.pop(0)   # the step has run to completion: its host arrays may go
        return float(loss.value) if want_loss else None

    def step_staged_lagged(self):
        """A full training step on the oldest staged batch; returns the loss of the PREVIOUS lagged step (None on
        the first call).  last_loss() gives the newest one."""
        loss, have = C.c_float(), C.c_int()
        check(self.ctx.h, self.ctx._l.nrs_trainer_step_staged_lagged(self.h, C.byref(loss), C.byref(have)))
        if have.value and len(getattr(self, "_staged", None) or []) > 1:
            self._staged.pop(0)   # the step before this one has run to completion: its host arrays may go
        return float(loss.value) if have.value else None

    def step_device(self, x_dev_ptr: int, target_dev_ptr: int, batch: int, want_loss=False):
        loss = C.c_float()
        check(self.ctx.h, self.ctx._l.nrs_trainer_step_device(self.h, VP(x_dev_ptr), VP(target_dev_ptr), int(batch),
                                                              C.byref(loss) if want_loss else None))
        return float(loss.value) if want_loss else None

    # ---- token models (first layer "embedding"): int32 ids [batch, seq], int32 labels [batch*seq]
    def _token_call(self, fn, ids, labels, want_loss):
        ids = np.ascontiguousarray(ids, np.int32)
        labels = np.ascontiguousarray(labels, np.int32).reshape(-1)
        assert labels.size == ids.size
        loss = C.c_float()
        check(self.ctx.h, fn(self.h, VP(ids.ctypes.data), VP(labels.ctypes.data), int(ids.shape[0]),
                             C.byref(loss) if want_loss else None))
        return float(loss.value) if want_loss else None

    def forward_backward_tokens(self, ids, labels, want_loss=True):
        return self._token_call(self.ctx._l.nrs_trainer_forward_backward_tokens, ids, labels, want_loss)

    def step_tokens(self, ids, labels, want_loss=True):
        return self._token_call(self.ctx._l.nrs_trainer_step_tokens, ids, labels, want_loss)

    def stage_next_tokens_ptr(self, ids_host_ptr: int, labels_host_ptr: int, batch: int):
        check(self.ctx.h, self.ctx._l.nrs_trainer_stage_next_tokens(self.h, VP(ids_host_ptr), VP(labels_host_ptr), int(batch)))

    def step_tokens_device(self, ids_dev_ptr: int, labels_dev_ptr: int, batch: int, want_loss=False):
        loss = C.c_float()
        check(self.ctx.h, self.ctx._l.nrs_trainer_step_tokens_device(self.h, VP(ids_dev_ptr), VP(labels_dev_ptr), int(batch),
                                                                     C.byref(loss) if want_loss else None))
        return float(loss.value) if want_loss else None

    def set_sync_batchnorm(self, on: bool = True):
        check(self.ctx.h, self.ctx._l.nrs_trainer_set_sync_batchnorm(self.h, int(bool(on))))

    def set_dp_timeout_ms(self, ms: float):
        check(self.ctx.h, self.ctx._l.nrs_trainer_set_dp_timeout_ms(self.h, C.c_double(ms)))

    def last_loss(self) -> float:
        loss = C.c_float()
        check(self.ctx.h, self.ctx._l.nrs_trainer_last_loss(self.h, C.byref(loss)))
        return float(loss.value)

    def enable_dp(self, rank: int, world: int, unique_id: bytes | None, global_batch: int, bucket_bytes: int = 0):
        buf = C.create_string_buffer(unique_id, 128) if unique_id is not None else None
        check(self.ctx.h, self.ctx._l.nrs_trainer_enable_dp(self.h, rank, world, buf, int(global_batch),
                                                            C.c_size_t(bucket_bytes)))

    def close(self):
        if self.h and self.ctx.h:
            self.ctx._l.nrs_trainer_free(self.h)
        self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class DataParallel:
    """Operator-level gradient exchange for a loop over nodes (include/nrs_graph.h: nrs_dp_create,
    nrs_bucket_register, nrs_grad_ready, nrs_allreduce_wait, nrs_backward_graph_dp)."""

    def __init__(self, rank: int, world: int, unique_id: bytes | None, global_batch: int, timeout_ms: float = 0.0,
                 ctx: Context | None = None):
        self.ctx = ctx or default_context()
        buf = C.create_string_buffer(unique_id, 128) if unique_id is not None else None
        h = VP()
        check(self.ctx.h, self.ctx._l.nrs_dp_create(self.ctx.h, rank, world, buf, int(global_batch), C.c_double(timeout_ms),
                                                    C.byref(h)))
        self.h = h

    def register(self, params, bucket_bytes: int = 0):
        arr = _handles(params)
        check(self.ctx.h, self.ctx._l.nrs_bucket_register(self.h, arr, len(params), C.c_size_t(bucket_bytes)))

    @property
    def bucket_count(self) -> int:
        return int(self.ctx._l.nrs_dp_bucket_count(self.h))

    def begin_step(self):
        check(self.ctx.h, self.ctx._l.nrs_dp_begin_step(self.h))

    def grad_ready(self, param: Node):
        check(self.ctx.h, self.ctx._l.nrs_grad_ready(self.h, param.h))

    def allreduce_wait(self):
        check(self.ctx.h, self.ctx._l.nrs_allreduce_wait(self.h))

    def backward_graph(self, root: Node):
        check(self.ctx.h, self.ctx._l.nrs_backward_graph_dp(root.h, self.h))

    def host_wait(self):
        check(self.ctx.h, self.ctx._l.nrs_dp_host_wait(self.h))

    def set_timeout_ms(self, ms: float):
        check(self.ctx.h, self.ctx._l.nrs_dp_set_timeout_ms(self.h, C.c_double(ms)))

    def all_reduce_sum(self, dev_ptr: int, count: int):
        check(self.ctx.h, self.ctx._l.nrs_dp_all_reduce_sum(self.h, VP(dev_ptr), C.c_size_t(count)))

    def close(self):
        if self.h and self.ctx.h:
            self.ctx._l.nrs_dp_free(self.h)
        self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def dp_fingerprint(param_lens, bucket_bytes: int, global_batch: int, world: int) -> int:
    arr = (C.c_int64 * len(param_lens))(*[int(v) for v in param_lens])
    return int(_lib.lib().nrs_dp_fingerprint(arr, len(param_lens), C.c_size_t(bucket_bytes), int(global_batch), int(world)))


def dp_check_fingerprints(fingerprints):
    arr = (C.c_uint64 * len(fingerprints))(*[int(v) for v in fingerprints])
    st = _lib.lib().nrs_dp_check_fingerprints(arr, len(fingerprints))
    if st != 0:
        raise _lib.NrsError(st, (_lib.lib().nrs_last_error(None) or b"").decode())


def watchdog_wait(poll, timeout_ms: float, interval_us: float = 200.0) -> float:
    """Runs the library's deadline loop over a Python poll function (0 running, 1 done, negative failed);
    returns the milliseconds waited, raises NrsError (NRS_ERR_TIMEOUT / NRS_ERR_NCCL) otherwise."""
    cb = _lib.POLL_FN(lambda _user: int(poll()))
    waited = C.c_double()
    st = _lib.lib().nrs_watchdog_wait(cb, None, C.c_double(timeout_ms), C.c_double(interval_us), C.byref(waited))
    if st != 0:
        raise _lib.NrsError(st, (_lib.lib().nrs_last_error(None) or b"").decode())
    return float(waited.value)


def dp_unique_id() -> bytes:
    buf = C.create_string_buffer(128)
    st = _lib.lib().nrs_dp_unique_id(buf)
    if st != 0:
        raise _lib.NrsError(st, (_lib.lib().nrs_last_error(None) or b"").decode())
    return buf.raw


def dp_shard_range(global_batch: int, rank: int, world: int) -> tuple[int, int]:
    b, e = C.c_int(), C.c_int()
    st = _lib.lib().nrs_dp_shard_range(global_batch, rank, world, C.byref(b), C.byref(e))
    if st != 0:
        raise _lib.NrsError(st, (_lib.lib().nrs_last_error(None) or b"").decode())
    return b.value, e.value


def dp_plan_buckets(param_lens, bucket_bytes: int) -> list[tuple[int, int]]:
    l = _lib.lib()
    lens = (C.c_int64 * len(param_lens))(*[int(v) for v in param_lens])
    n = l.nrs_dp_plan_buckets(lens, len(param_lens), C.c_size_t(bucket_bytes), None, None, 0)
    if n < 0:
        raise ValueError("bad parameter lengths")
    s, e = (C.c_int64 * max(n, 1))(), (C.c_int64 * max(n, 1))()
    l.nrs_dp_plan_buckets(lens, len(param_lens), C.c_size_t(bucket_bytes), s, e, n)
    return [(int(s[i]), int(e[i])) for i in range(n)]


class serialize:
    """src/serialize.rs `save` / `load` through the library's host-side reader / writer (include/nrs_checkpoint.h)."""

    class _Named(C.Structure):
        _fields_ = [("name", C.c_char_p), ("shape", C.POINTER(C.c_int64)), ("ndim", C.c_int), ("data", C.c_void_p)]

    @staticmethod
    def save(tensors, path: str):
        """tensors: [(name, shape, data)]; '.safetensors' writes safetensors, anything else the positional text format."""
        l = _lib.lib()
        keep, arr = [], (serialize._Named * len(tensors))()
        for i, (name, shape, data) in enumerate(tensors):
            d = _f32(data).reshape(-1)
            if d.size != int(np.prod([int(s) for s in shape], dtype=np.int64)):
                # the C struct carries no length: the shape says how many floats are read (serialize.rs:204 panics here)
                raise ValueError(f"save: tensor shape does not match its data length ({name})")
            sh = (C.c_int64 * len(shape))(*[int(s) for s in shape])
            keep += [d, sh]
            arr[i] = serialize._Named(name.encode(), sh, len(shape), d.ctypes.data)
        _lib.check(None, l.nrs_save(arr, len(tensors), str(path).encode()))

    @staticmethod
    def load(path: str):
        """-> [(name, shape, data)]: sorted by name for safetensors, tensor_{i} / flat length for text."""
        l = _lib.lib()
        h = VP()
        _lib.check(None, l.nrs_load(str(path).encode(), C.byref(h)))
        try:
            out = []
            for i in range(l.nrs_checkpoint_count(h)):
                name = C.string_at(l.nrs_checkpoint_name(h, i)).decode()
                shape = [int(l.nrs_checkpoint_dim(h, i, d)) for d in range(l.nrs_checkpoint_ndim(h, i))]
                n = int(l.nrs_checkpoint_len(h, i))
                data = np.frombuffer(C.string_at(l.nrs_checkpoint_data(h, i), n * 4), np.float32).copy() if n else np.zeros(0, np.float32)
                out.append((name, shape, data))
            return out
        finally:
            l.nrs_checkpoint_free(h)
