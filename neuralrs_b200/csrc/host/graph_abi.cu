// extern "C" wrappers over the C++ graph layer (nrs_graph.h).  Exceptions stop
// here: every wrapper returns a status code and records the message on the
// node's context.
#include <cstring>

#include "host/graph.h"
#include "host/abi_types.h"
#include "nrs_graph.h"
#include "nrs_internal.h"

struct nrs_adamw {
  nrs_ctx* ctx;
  std::unique_ptr<nrs::cuda::AdamW> opt;
  mutable std::vector<std::vector<float>> exported;  // cache for state_len/get
  mutable bool exported_valid = false;
};

namespace {

template <class F>
int guarded(nrs_ctx* ctx, F&& f) {
  try {
    f();
    return NRS_OK;
  } catch (const nrs::Error& e) {
    return nrs_fail(ctx, e.code, "%s", e.what());
  } catch (const std::bad_alloc&) {
    return nrs_fail(ctx, NRS_ERR_ALLOC, "host allocation failed");
  } catch (const std::exception& e) {
    return nrs_fail(ctx, NRS_ERR_ARG, "%s", e.what());
  }
}

nrs_ctx* ctx_of(const nrs_node* n) { return n && n->p ? n->p->ctx : nullptr; }

int wrap(nrs_ctx* ctx, nrs_node** out, const std::function<nrs::NodeP()>& make) {
  if (!out) return nrs_fail(ctx, NRS_ERR_ARG, "null out handle");
  *out = nullptr;
  return guarded(ctx, [&] {
    nrs::NodeP p = make();
    *out = new nrs_node{p};
  });
}

std::vector<nrs::NodeP> gather(nrs_node* const* nodes, int count) {
  if (count < 0 || (count > 0 && !nodes)) throw nrs::Error(NRS_ERR_ARG, "null node list");
  std::vector<nrs::NodeP> v;
  for (int i = 0; i < count; ++i) {
    if (!nodes[i] || !nodes[i]->p) throw nrs::Error(NRS_ERR_ARG, "null node in list");
    v.push_back(nodes[i]->p);
  }
  return v;
}

#define NODE_OK(n) \
  do { if (!(n) || !(n)->p) return nrs_fail(nullptr, NRS_ERR_ARG, "%s: null node", __func__); } while (0)

}  // namespace

extern "C" {

int nrs_node_new(nrs_ctx* ctx, const float* host_data, const int64_t* shape, int ndim, nrs_node** out) {
  NRS_REQUIRE_CTX(ctx);
  NRS_REQUIRE(ctx, ndim >= 0 && (ndim == 0 || shape), NRS_ERR_ARG, "nrs_node_new: bad shape argument");
  for (int i = 0; i < ndim; ++i) NRS_REQUIRE(ctx, shape[i] >= 0, NRS_ERR_SHAPE, "nrs_node_new: negative extent");
  return wrap(ctx, out, [&] {
    std::vector<size_t> s(shape, shape + ndim);
    return nrs::node_new(ctx, host_data, s);
  });
}

int nrs_node_release(nrs_node* n) {
  delete n;
  return NRS_OK;
}

int nrs_node_ndim(const nrs_node* n) { return n && n->p ? (int)n->p->shape.size() : -1; }

int nrs_node_shape(const nrs_node* n, int64_t* shape_out, int capacity) {
  NODE_OK(n);
  const int nd = (int)n->p->shape.size();
  if (!shape_out || capacity < nd) return nrs_fail(ctx_of(n), NRS_ERR_ARG, "nrs_node_shape: buffer too small");
  for (int i = 0; i < nd; ++i) shape_out[i] = (int64_t)n->p->shape[i];
  return NRS_OK;
}

int64_t nrs_node_len(const nrs_node* n) { return n && n->p ? (int64_t)n->p->len() : -1; }

int nrs_node_set_requires_grad(nrs_node* n, int flag) {
  NODE_OK(n);
  n->p->requires_grad = flag != 0;
  return NRS_OK;
}

int nrs_node_set_data(nrs_node* n, const float* host_data) {
  NODE_OK(n);
  if (!host_data && n->p->len()) return nrs_fail(ctx_of(n), NRS_ERR_ARG, "nrs_node_set_data: null data");
  return guarded(ctx_of(n), [&] {
    // a copy still in flight from an earlier to_cuda reads the old host vector
    if (n->p->on_gpu()) nrs::cuda::synchronize(n->p->ctx);
    n->p->host.assign(host_data, host_data + n->p->len());
  });
}

float* nrs_node_data_ptr(nrs_node* n) { return n && n->p ? n->p->data : nullptr; }

int nrs_node_invalidate(nrs_node* n) {
  NODE_OK(n);
  return guarded(ctx_of(n), [&] {
    nrs::Node* r = n->p.get();
    while (r->view_of) r = r->view_of.get();
    nrs::invalidate_operand_caches(r);
    if (r != n->p.get()) nrs::invalidate_operand_caches(n->p.get());
  });
}

float* nrs_node_grad_ptr(nrs_node* n) {
  if (!n || !n->p) return nullptr;
  nrs::Node* r = n->p.get();
  while (r->view_of) r = r->view_of.get();
  return r->grad_valid ? r->grad : nullptr;
}

int nrs_to_cuda(nrs_node* n) {
  NODE_OK(n);
  return guarded(ctx_of(n), [&] { nrs::cuda::to_cuda(n->p); });
}

int nrs_to_host(nrs_node* n, float* host_out) {
  NODE_OK(n);
  if (!host_out && n->p->len()) return nrs_fail(ctx_of(n), NRS_ERR_ARG, "nrs_to_host: null output");
  return guarded(ctx_of(n), [&] {
    auto v = nrs::cuda::to_host(n->p);
    std::memcpy(host_out, v.data(), v.size() * sizeof(float));
  });
}

int nrs_set_grad(nrs_node* n, const float* host_grad) {
  NODE_OK(n);
  if (!host_grad && n->p->len()) return nrs_fail(ctx_of(n), NRS_ERR_ARG, "nrs_set_grad: null gradient");
  return guarded(ctx_of(n), [&] { nrs::cuda::set_grad(n->p, host_grad); });
}

int nrs_read_grad(nrs_node* n, float* host_out) {
  NODE_OK(n);
  if (!host_out && n->p->len()) return nrs_fail(ctx_of(n), NRS_ERR_ARG, "nrs_read_grad: null output");
  return guarded(ctx_of(n), [&] {
    auto v = nrs::cuda::read_grad(n->p);
    std::memcpy(host_out, v.data(), v.size() * sizeof(float));
  });
}

int nrs_node_backward(nrs_node* n) {
  NODE_OK(n);
  return guarded(ctx_of(n), [&] {
    if (n->p->backward_fn) n->p->backward_fn();
  });
}

int nrs_zero_grad(nrs_node* const* params, int count) {
  nrs_ctx* ctx = count > 0 && params && params[0] ? ctx_of(params[0]) : nullptr;
  return guarded(ctx, [&] { nrs::cuda::zero_grad(gather(params, count)); });
}

int nrs_flatten_params(nrs_node* const* params, int count) {
  nrs_ctx* ctx = count > 0 && params && params[0] ? ctx_of(params[0]) : nullptr;
  return guarded(ctx, [&] { nrs::cuda::flatten_params(gather(params, count)); });
}

#define UNARY(name, expr)                                   \
  int name(nrs_node* x, nrs_node** out) {                   \
    NODE_OK(x);                                             \
    return wrap(ctx_of(x), out, [&] { return expr; });      \
  }
#define BINARY(name, expr)                                  \
  int name(nrs_node* a, nrs_node* b, nrs_node** out) {      \
    NODE_OK(a);                                             \
    NODE_OK(b);                                             \
    return wrap(ctx_of(a), out, [&] { return expr; });      \
  }

BINARY(nrs_op_matmul, nrs::cuda::matmul(a->p, b->p))
BINARY(nrs_op_add, nrs::cuda::add(a->p, b->p))
BINARY(nrs_op_bmm, nrs::cuda::bmm(a->p, b->p))
UNARY(nrs_op_relu, nrs::cuda::relu(x->p))
UNARY(nrs_op_gelu, nrs::cuda::gelu(x->p))
UNARY(nrs_op_softmax, nrs::cuda::softmax(x->p))
UNARY(nrs_op_transpose, nrs::cuda::transpose(x->p))
UNARY(nrs_op_flatten, nrs::cuda::flatten(x->p))

int nrs_op_reshape(nrs_node* x, const int64_t* shape, int ndim, nrs_node** out) {
  NODE_OK(x);
  if (ndim < 0 || (ndim > 0 && !shape)) return nrs_fail(ctx_of(x), NRS_ERR_ARG, "nrs_op_reshape: bad shape argument");
  return wrap(ctx_of(x), out, [&] {
    std::vector<size_t> s;
    for (int i = 0; i < ndim; ++i) {
      if (shape[i] < 0) throw nrs::Error(NRS_ERR_SHAPE, "nrs_op_reshape: negative extent");
      s.push_back((size_t)shape[i]);
    }
    return nrs::cuda::reshape(x->p, s);
  });
}

int nrs_op_scale(nrs_node* x, float s, nrs_node** out) {
  NODE_OK(x);
  return wrap(ctx_of(x), out, [&] { return nrs::cuda::scale(x->p, s); });
}

int nrs_op_slice_cols(nrs_node* x, int64_t col_start, int64_t col_end, nrs_node** out) {
  NODE_OK(x);
  if (col_start < 0 || col_end < 0) return nrs_fail(ctx_of(x), NRS_ERR_SHAPE, "nrs_op_slice_cols: negative column");
  return wrap(ctx_of(x), out, [&] { return nrs::cuda::slice_cols(x->p, (size_t)col_start, (size_t)col_end); });
}

int nrs_op_concat_cols(nrs_node* const* parts, int count, nrs_node** out) {
  nrs_ctx* ctx = count > 0 && parts && parts[0] ? ctx_of(parts[0]) : nullptr;
  return wrap(ctx, out, [&] { return nrs::cuda::concat_cols(gather(parts, count)); });
}

int nrs_op_conv2d(nrs_node* input, nrs_node* weight, nrs_node* bias, int64_t stride, int64_t pad, nrs_node** out) {
  return nrs_op_conv2d_act(input, weight, bias, stride, pad, NRS_ACT_NONE, out);
}

int nrs_op_conv2d_act(nrs_node* input, nrs_node* weight, nrs_node* bias, int64_t stride, int64_t pad, int act,
                      nrs_node** out) {
  NODE_OK(input);
  NODE_OK(weight);
  NODE_OK(bias);
  if (stride < 1 || pad < 0) return nrs_fail(ctx_of(input), NRS_ERR_SHAPE, "conv2d: bad stride/pad");
  return wrap(ctx_of(input), out,
              [&] { return nrs::cuda::conv2d_act(input->p, weight->p, bias->p, (size_t)stride, (size_t)pad, act); });
}

int nrs_op_maxpool2d(nrs_node* input, int64_t kernel, int64_t stride, nrs_node** out) {
  NODE_OK(input);
  if (kernel < 1 || stride < 1) return nrs_fail(ctx_of(input), NRS_ERR_SHAPE, "maxpool2d: bad kernel/stride");
  return wrap(ctx_of(input), out, [&] { return nrs::cuda::maxpool2d(input->p, (size_t)kernel, (size_t)stride); });
}

int nrs_op_layernorm(nrs_node* x, nrs_node* gamma, nrs_node* beta, float eps, nrs_node** out) {
  NODE_OK(x);
  NODE_OK(gamma);
  NODE_OK(beta);
  return wrap(ctx_of(x), out, [&] { return nrs::cuda::layernorm(x->p, gamma->p, beta->p, eps); });
}

int nrs_op_batchnorm(nrs_node* x, nrs_node* gamma, nrs_node* beta, nrs_node* running_mean, nrs_node* running_var,
                     float momentum, float eps, int training, nrs_node** out) {
  NODE_OK(x);
  NODE_OK(gamma);
  NODE_OK(beta);
  NODE_OK(running_mean);
  NODE_OK(running_var);
  return wrap(ctx_of(x), out, [&] {
    return nrs::cuda::batchnorm(x->p, gamma->p, beta->p, running_mean->p, running_var->p, momentum, eps, training != 0);
  });
}

int nrs_op_batchnorm2d(nrs_node* x, nrs_node* gamma, nrs_node* beta, nrs_node* running_mean, nrs_node* running_var,
                       float momentum, float eps, int training, nrs_node** out) {
  NODE_OK(x);
  NODE_OK(gamma);
  NODE_OK(beta);
  NODE_OK(running_mean);
  NODE_OK(running_var);
  return wrap(ctx_of(x), out, [&] {
    return nrs::cuda::batchnorm2d(x->p, gamma->p, beta->p, running_mean->p, running_var->p, momentum, eps, training != 0);
  });
}

int nrs_op_batchnorm_act(nrs_node* x, nrs_node* gamma, nrs_node* beta, nrs_node* running_mean, nrs_node* running_var,
                         float momentum, float eps, int training, int act, nrs_node** out) {
  NODE_OK(x);
  NODE_OK(gamma);
  NODE_OK(beta);
  NODE_OK(running_mean);
  NODE_OK(running_var);
  return wrap(ctx_of(x), out, [&] {
    return nrs::cuda::batchnorm_act(x->p, gamma->p, beta->p, running_mean->p, running_var->p, momentum, eps, training != 0, act);
  });
}

int nrs_op_dropout(nrs_node* x, float p, int training, nrs_node* mask, nrs_node** out) {
  NODE_OK(x);
  if (mask) NODE_OK(mask);
  return wrap(ctx_of(x), out, [&] { return nrs::cuda::dropout(x->p, p, training != 0, mask ? mask->p : nullptr); });
}

int nrs_op_dropout2d(nrs_node* x, float p, int training, nrs_node* mask, nrs_node** out) {
  NODE_OK(x);
  if (mask) NODE_OK(mask);
  return wrap(ctx_of(x), out, [&] { return nrs::cuda::dropout2d(x->p, p, training != 0, mask ? mask->p : nullptr); });
}

int nrs_op_linear_act(nrs_node* x, nrs_node* w, nrs_node* b, int act, nrs_node** out) {
  NODE_OK(x);
  NODE_OK(w);
  NODE_OK(b);
  return wrap(ctx_of(x), out, [&] { return nrs::cuda::linear_act(x->p, w->p, b->p, act); });
}

int nrs_op_embedding(nrs_node* weight, const int32_t* indices_host, int64_t count, nrs_node** out) {
  NODE_OK(weight);
  if (count < 0 || weight->p->shape.size() != 2) return nrs_fail(ctx_of(weight), NRS_ERR_SHAPE, "embedding: weight must be [vocab, dim]");
  return wrap(ctx_of(weight), out, [&] {
    nrs::cuda::Embedding e{weight->p, weight->p->shape[0], weight->p->shape[1]};
    return e.forward(indices_host, (size_t)count);
  });
}

int nrs_op_embedding_batch(nrs_node* weight, const int32_t* indices_host, int64_t batch, int64_t seq, nrs_node** out) {
  NODE_OK(weight);
  if (batch < 0 || seq < 0 || weight->p->shape.size() != 2) return nrs_fail(ctx_of(weight), NRS_ERR_SHAPE, "embedding: bad shape");
  return wrap(ctx_of(weight), out, [&] {
    nrs::cuda::Embedding e{weight->p, weight->p->shape[0], weight->p->shape[1]};
    return e.forward_batch(indices_host, (size_t)batch, (size_t)seq);
  });
}

int nrs_positional_new(nrs_ctx* ctx, int64_t d_model, int64_t max_len, nrs_node** table_out) {
  NRS_REQUIRE_CTX(ctx);
  NRS_REQUIRE(ctx, d_model > 0 && max_len > 0, NRS_ERR_SHAPE, "nrs_positional_new: non-positive size");
  return wrap(ctx, table_out, [&] { return nrs::cuda::PositionalEncoding::make(ctx, (size_t)d_model, (size_t)max_len).table; });
}

int nrs_op_positional(nrs_node* x, nrs_node* table, nrs_node** out) {
  NODE_OK(x);
  NODE_OK(table);
  if (table->p->shape.size() != 2) return nrs_fail(ctx_of(x), NRS_ERR_SHAPE, "positional: table must be [max_len, d_model]");
  return wrap(ctx_of(x), out, [&] {
    nrs::cuda::PositionalEncoding pe;
    pe.max_len = table->p->shape[0];
    pe.d_model = table->p->shape[1];
    pe.table = table->p;
    return pe.forward(x->p);
  });
}

UNARY(nrs_op_causal_mask, nrs::cuda::causal_mask(x->p))

int nrs_op_attention_batch(nrs_node* q, nrs_node* k, nrs_node* v, int causal, nrs_node** out) {
  NODE_OK(q);
  NODE_OK(k);
  NODE_OK(v);
  return wrap(ctx_of(q), out, [&] { return nrs::cuda::attention_batch(q->p, k->p, v->p, causal != 0); });
}

int nrs_op_mha(nrs_node* x, nrs_node* w_q, nrs_node* w_k, nrs_node* w_v, nrs_node* w_o, int64_t num_heads,
               int causal, nrs_node** out) {
  NODE_OK(x);
  NODE_OK(w_q);
  NODE_OK(w_k);
  NODE_OK(w_v);
  NODE_OK(w_o);
  if (num_heads < 1 || x->p->shape.size() != 3) return nrs_fail(ctx_of(x), NRS_ERR_SHAPE, "mha: bad heads or input rank");
  return wrap(ctx_of(x), out, [&] {
    nrs::cuda::MultiHeadAttention m{w_q->p, w_k->p, w_v->p, w_o->p, x->p->shape[2], (size_t)num_heads, causal != 0};
    return m.forward_batch(x->p);
  });
}

int nrs_op_transformer_block(nrs_node* x, nrs_node* const* params, int64_t num_heads, float eps, int act,
                             int causal, int final_norm, nrs_node** out) {
  NODE_OK(x);
  if (num_heads < 1 || x->p->shape.size() != 3) return nrs_fail(ctx_of(x), NRS_ERR_SHAPE, "transformer block: bad heads or input rank");
  if (act != NRS_ACT_RELU && act != NRS_ACT_GELU) return nrs_fail(ctx_of(x), NRS_ERR_ARG, "transformer block: act must be ReLU or GELU");
  return wrap(ctx_of(x), out, [&] {
    auto p = gather(params, 12);
    nrs::cuda::TransformerBlock b;
    b.mha = nrs::cuda::MultiHeadAttention{p[0], p[1], p[2], p[3], x->p->shape[2], (size_t)num_heads, causal != 0};
    b.norm1 = nrs::cuda::LayerNorm{p[4], p[5], eps};
    b.norm2 = nrs::cuda::LayerNorm{p[6], p[7], eps};
    b.ff1 = nrs::cuda::Linear{p[8], p[9]};
    b.ff2 = nrs::cuda::Linear{p[10], p[11]};
    b.d_model = x->p->shape[2];
    b.d_ff = p[8]->shape.size() == 2 ? p[8]->shape[1] : 0;
    b.act = act;
    return final_norm ? b.forward(x->p) : b.forward_no_final_norm(x->p);
  });
}

int nrs_cross_entropy(nrs_node* pred, nrs_node* target, float* loss_out) {
  NODE_OK(pred);
  NODE_OK(target);
  if (!loss_out) return nrs_fail(ctx_of(pred), NRS_ERR_ARG, "nrs_cross_entropy: null output");
  return guarded(ctx_of(pred), [&] { *loss_out = nrs::cuda::cross_entropy(pred->p, target->p); });
}

int nrs_cross_entropy_backward(nrs_node* pred, nrs_node* target) {
  NODE_OK(pred);
  NODE_OK(target);
  return guarded(ctx_of(pred), [&] { nrs::cuda::cross_entropy_backward(pred->p, target->p); });
}

int nrs_backward_graph(nrs_node* root) {
  NODE_OK(root);
  return guarded(ctx_of(root), [&] { nrs::backward_graph(root->p); });
}

int nrs_adamw_new(nrs_ctx* ctx, float lr, float beta1, float beta2, float eps, float weight_decay, nrs_adamw** out) {
  NRS_REQUIRE_CTX(ctx);
  NRS_REQUIRE(ctx, out != nullptr, NRS_ERR_ARG, "nrs_adamw_new: null out handle");
  *out = nullptr;
  return guarded(ctx, [&] {
    auto* h = new nrs_adamw();
    h->ctx = ctx;
    h->opt.reset(new nrs::cuda::AdamW(ctx, lr, beta1, beta2, eps, weight_decay));
    *out = h;
  });
}

int nrs_adamw_free(nrs_adamw* opt) {
  delete opt;
  return NRS_OK;
}

int nrs_adamw_step_nodes(nrs_adamw* opt, nrs_node* const* params, int count) {
  if (!opt) return nrs_fail(nullptr, NRS_ERR_ARG, "nrs_adamw_step_nodes: null optimizer");
  opt->exported_valid = false;
  return guarded(opt->ctx, [&] { opt->opt->step(gather(params, count)); });
}

int64_t nrs_adamw_t(const nrs_adamw* opt) { return opt ? (int64_t)opt->opt->t : -1; }

static int refresh_export(const nrs_adamw* opt) {
  if (opt->exported_valid) return NRS_OK;
  return guarded(opt->ctx, [&] {
    opt->exported = opt->opt->export_state(nullptr);
    opt->exported_valid = true;
  });
}

int nrs_adamw_state_count(const nrs_adamw* opt) {
  if (!opt || refresh_export(opt) != NRS_OK) return -1;
  return (int)opt->exported.size();
}

int64_t nrs_adamw_state_len(const nrs_adamw* opt, int i) {
  if (!opt || refresh_export(opt) != NRS_OK || i < 0 || i >= (int)opt->exported.size()) return -1;
  return (int64_t)opt->exported[i].size();
}

int nrs_adamw_state_get(const nrs_adamw* opt, int i, float* host_out) {
  if (!opt) return nrs_fail(nullptr, NRS_ERR_ARG, "nrs_adamw_state_get: null optimizer");
  int st = refresh_export(opt);
  if (st != NRS_OK) return st;
  if (i < 0 || i >= (int)opt->exported.size() || !host_out)
    return nrs_fail(opt->ctx, NRS_ERR_ARG, "nrs_adamw_state_get: bad index or null output");
  std::memcpy(host_out, opt->exported[i].data(), opt->exported[i].size() * sizeof(float));
  return NRS_OK;
}

int nrs_adamw_import_state(nrs_adamw* opt, int64_t t, const float* const* moments, const int64_t* lens, int count) {
  if (!opt) return nrs_fail(nullptr, NRS_ERR_ARG, "nrs_adamw_import_state: null optimizer");
  if (count < 0 || t < 0 || (count > 0 && (!moments || !lens)))
    return nrs_fail(opt->ctx, NRS_ERR_ARG, "nrs_adamw_import_state: bad arguments");
  opt->exported_valid = false;
  return guarded(opt->ctx, [&] {
    std::vector<std::vector<float>> m;
    for (int i = 0; i < count; ++i) {
      if (lens[i] < 0 || (lens[i] > 0 && !moments[i])) throw nrs::Error(NRS_ERR_ARG, "import_state: bad tensor");
      m.emplace_back(moments[i], moments[i] + lens[i]);
    }
    opt->opt->import_state((size_t)t, m);
  });
}

}  // extern "C"
