// Transformer-side operators of the graph layer: embedding, positional encoding,
// batched attention, multi-head attention, the post-LN transformer block.
// They are written the way the reference writes them — compositions of the
// resident graph ops (src/cuda/nn/attention.rs:23-32, multihead.rs:57-85,
// transformer_block.rs:28-60) — plus the embedding gather/scatter kernels and
// the causal mask, which need their own backward closures.
#include <cmath>
#include <cstring>

#include "host/graph.h"

namespace nrs {
namespace cuda {

static void fail(int code, const std::string& m) { throw Error(code, m); }

NodeP causal_mask(const NodeP& scores) {
  if (!scores || !scores->on_gpu()) fail(NRS_ERR_ARG, "cuda causal_mask: input not on GPU");
  const size_t nd = scores->shape.size();
  if (nd < 2 || scores->shape[nd - 1] != scores->shape[nd - 2]) fail(NRS_ERR_SHAPE, "cuda causal_mask: last two dims must be equal");
  nrs_ctx* ctx = scores->ctx;
  const int s = (int)scores->shape[nd - 1];
  const int batch = (int)(scores->len() / ((size_t)s * s));
  NodeP out = make_result(ctx, scores->shape, {scores});
  check(ctx, nrs_causal_mask(ctx, scores->data, out->data, batch, s, 0, 0));
  Node* self = out.get();
  out->backward_fn = [self, scores, batch, s]() {
    if (!scores->requires_grad) return;
    const float* g = grad_view(self);
    GradSlot t = grad_slot(scores);
    check(self->ctx, nrs_causal_mask(self->ctx, g, t.ptr, batch, s, 1, t.accumulate));
  };
  return out;
}

// softmax(q k^T / sqrt(d_head)) v for every head of [batch, seq, heads*d_head] tensors in one kernel
// (shapes inside nrs_attention_supported only).
static NodeP fused_attention(const NodeP& q, const NodeP& k, const NodeP& v, size_t heads, bool causal) {
  nrs_ctx* ctx = q->ctx;
  const size_t batch = q->shape[0], seq = q->shape[1], d = q->shape[2], d_head = d / heads;
  if (k->shape != q->shape || v->shape != q->shape) fail(NRS_ERR_SHAPE, "cuda attention: q, k, v shapes differ");
  NodeP out = make_result(ctx, q->shape, {q, k, v});
  void* probs = nullptr;
  check(ctx, nrs_alloc(ctx, std::max<size_t>(1, batch * heads * seq * seq) * sizeof(float), 0, &probs));
  out->saved.push_back(probs);
  check(ctx, nrs_attention_fwd(ctx, q->data, k->data, v->data, out->data, (float*)probs, (int)batch, (int)seq, (int)heads,
                               (int)d_head, causal ? 1 : 0));
  Node* self = out.get();
  out->backward_fn = [self, q, k, v, probs, batch, seq, heads, d_head]() {
    nrs_ctx* ctx = self->ctx;
    const float* g = grad_view(self);
    // a tensor that needs no gradient still gets a scratch target: the kernel computes all three
    const size_t len = self->len();
    auto target = [&](const NodeP& n, float** scratch) {
      if (n->requires_grad) return grad_slot(n);
      void* p = nullptr;
      check(ctx, nrs_alloc(ctx, std::max<size_t>(1, len) * sizeof(float), 0, &p));
      *scratch = (float*)p;
      return GradSlot{(float*)p, 0};
    };
    float *sq = nullptr, *sk = nullptr, *sv = nullptr;
    GradSlot tq = target(q, &sq), tk = target(k, &sk), tv = target(v, &sv);
    check(ctx, nrs_attention_bwd(ctx, q->data, k->data, v->data, (const float*)probs, g, tq.ptr, tk.ptr, tv.ptr, (int)batch,
                                 (int)seq, (int)heads, (int)d_head, tq.accumulate, tk.accumulate, tv.accumulate));
    for (float* s : {sq, sk, sv})
      if (s) nrs_free(ctx, s);
  };
  return out;
}

NodeP attention_batch(const NodeP& q, const NodeP& k, const NodeP& v, bool causal) {
  if (!q || q->shape.size() != 3) fail(NRS_ERR_SHAPE, "cuda attention_batch: q must be [batch, seq, d_head]");
  if (k && v && k->on_gpu() && v->on_gpu() && q->on_gpu() && nrs_attention_supported((int)q->shape[1], (int)q->shape[2]))
    return fused_attention(q, k, v, 1, causal);
  const float scale_factor = 1.0f / std::sqrt((float)q->shape[2]);
  NodeP scores = scale(bmm(q, transpose(k)), scale_factor);
  if (causal) scores = causal_mask(scores);
  return bmm(softmax(scores), v);
}

NodeP Linear::forward(const NodeP& x) const { return add(matmul(x, weights), bias); }

NodeP LayerNorm::forward(const NodeP& x) const { return layernorm(x, gamma, beta, eps); }

// Gather (+ positional table) from indices already on the device; the node does not own `idx_dev`.
static NodeP embed_resident(const Embedding& e, const int32_t* idx_dev, size_t count, const std::vector<size_t>& out_shape,
                            const NodeP& pos_table, size_t seq) {
  nrs_ctx* ctx = e.weight->ctx;
  const int dim = (int)e.embedding_dim, vocab = (int)e.vocab_size;
  NodeP out = make_result(ctx, out_shape, {e.weight});
  check(ctx, nrs_embedding_pos_fwd(ctx, e.weight->data, idx_dev, pos_table ? pos_table->data : nullptr, out->data, (int)count,
                                   (int)seq, dim, vocab));
  Node* self = out.get();
  const NodeP w = e.weight;
  out->backward_fn = [self, w, idx_dev, count, dim, vocab]() {
    if (!w->requires_grad) return;
    const float* g = grad_view(self);
    GradSlot t = grad_slot(w);
    check(self->ctx, nrs_embedding_bwd(self->ctx, g, idx_dev, t.ptr, (int)count, dim, vocab, t.accumulate));
  };
  return out;
}

static NodeP embed(const Embedding& e, const int32_t* indices, size_t count, const std::vector<size_t>& out_shape) {
  if (!e.weight || !e.weight->on_gpu()) fail(NRS_ERR_ARG, "cuda embedding: weight not on GPU");
  if (!indices && count) fail(NRS_ERR_ARG, "cuda embedding: null indices");
  for (size_t i = 0; i < count; ++i)
    if (indices[i] < 0 || (size_t)indices[i] >= e.vocab_size) fail(NRS_ERR_ARG, "embedding: token index out of vocab range");
  nrs_ctx* ctx = e.weight->ctx;
  void* idx_dev = nullptr;
  check(ctx, nrs_alloc(ctx, (count ? count : 1) * sizeof(int32_t), 0, &idx_dev));
  NodeP out;
  try {
    check(ctx, nrs_h2d(ctx, idx_dev, indices, count * sizeof(int32_t)));
    check(ctx, nrs_sync(ctx));  // the caller's index buffer may go away
    out = embed_resident(e, (const int32_t*)idx_dev, count, out_shape, nullptr, 1);
  } catch (...) {
    nrs_free(ctx, idx_dev);
    throw;
  }
  out->saved.push_back(idx_dev);
  return out;
}

NodeP Embedding::forward_resident(const int32_t* idx_dev, size_t batch, size_t seq, const NodeP& pos_table) const {
  if (!weight || !weight->on_gpu()) fail(NRS_ERR_ARG, "cuda embedding: weight not on GPU");
  if (!idx_dev && batch * seq) fail(NRS_ERR_ARG, "cuda embedding: null indices");
  if (pos_table) {
    if (!pos_table->on_gpu() || pos_table->shape.size() != 2 || pos_table->shape[1] != embedding_dim)
      fail(NRS_ERR_SHAPE, "cuda embedding: positional table must be a resident [max_len, dim] tensor");
    if (seq > pos_table->shape[0]) fail(NRS_ERR_SHAPE, "sequence longer than max_len");
  }
  return embed_resident(*this, idx_dev, batch * seq, {batch, seq, embedding_dim}, pos_table, seq);
}

NodeP Embedding::forward(const int32_t* indices, size_t count) const {
  return embed(*this, indices, count, {count, embedding_dim});
}

NodeP Embedding::forward_batch(const int32_t* indices, size_t batch, size_t seq) const {
  return embed(*this, indices, batch * seq, {batch, seq, embedding_dim});
}

PositionalEncoding PositionalEncoding::make(nrs_ctx* ctx, size_t d_model, size_t max_len) {
  // The table is computed on the host in f32 exactly as the reference does
  // (src/cuda/nn/positional.rs:24-33), once, and stays resident.
  std::vector<float> pe(max_len * d_model);
  for (size_t pos = 0; pos < max_len; ++pos)
    for (size_t i = 0; i < d_model; ++i) {
      const float exponent = (float)(2 * (i / 2)) / (float)d_model;
      const float freq = 1.0f / std::pow(10000.0f, exponent);
      const float angle = (float)pos * freq;
      pe[pos * d_model + i] = (i % 2 == 0) ? std::sin(angle) : std::cos(angle);
    }
  PositionalEncoding p;
  p.d_model = d_model;
  p.max_len = max_len;
  p.table = node_new(ctx, pe.data(), {max_len, d_model});
  p.table->requires_grad = false;
  to_cuda(p.table);
  synchronize(ctx);
  return p;
}

NodeP PositionalEncoding::forward(const NodeP& x) const {
  if (!x || !x->on_gpu()) fail(NRS_ERR_ARG, "cuda positional: input not on GPU");
  const size_t nd = x->shape.size();
  if (nd != 2 && nd != 3) fail(NRS_ERR_SHAPE, "cuda positional: input must be [seq, d] or [batch, seq, d]");
  const size_t seq = x->shape[nd - 2], d = x->shape[nd - 1];
  if (d != d_model) fail(NRS_ERR_SHAPE, "cuda positional: feature size differs from d_model");
  if (seq > max_len) fail(NRS_ERR_SHAPE, "sequence longer than max_len");
  nrs_ctx* ctx = x->ctx;
  const size_t batch = nd == 3 ? x->shape[0] : 1;
  // out[b, i] = x[b, i] + pe[i] over the first seq*d entries of the table: a row-broadcast add.
  NodeP out = make_result(ctx, x->shape, {x});
  check(ctx, nrs_bias_add(ctx, x->data, table->data, out->data, (int)batch, (int)(seq * d)));
  Node* self = out.get();
  const size_t len = x->len();
  out->backward_fn = [self, x, len]() {
    if (!x->requires_grad) return;
    const float* g = grad_view(self);
    GradSlot t = grad_slot(x);
    if (t.accumulate) check(self->ctx, nrs_accumulate(self->ctx, t.ptr, g, len));
    else check(self->ctx, nrs_d2d(self->ctx, t.ptr, g, len * sizeof(float)));
  };
  return out;
}

// [batch, seq, heads*d_head] <-> [batch*heads, seq, d_head]; the backward pass is the opposite permutation.
static NodeP permute_heads(const NodeP& x, size_t batch, size_t seq, size_t heads, size_t d_head, bool to_heads) {
  nrs_ctx* ctx = x->ctx;
  NodeP out = make_result(ctx, to_heads ? std::vector<size_t>{batch * heads, seq, d_head}
                                        : std::vector<size_t>{batch, seq, heads * d_head}, {x});
  check(ctx, nrs_permute_heads(ctx, x->data, out->data, (int)batch, (int)seq, (int)heads, (int)d_head, to_heads ? 1 : 0, 0));
  Node* self = out.get();
  out->backward_fn = [self, x, batch, seq, heads, d_head, to_heads]() {
    if (!x->requires_grad) return;
    const float* g = grad_view(self);
    GradSlot t = grad_slot(x);
    check(self->ctx, nrs_permute_heads(self->ctx, g, t.ptr, (int)batch, (int)seq, (int)heads, (int)d_head, to_heads ? 0 : 1,
                                       t.accumulate));
  };
  return out;
}

NodeP MultiHeadAttention::forward_batch(const NodeP& x) const {
  if (!x || x->shape.size() != 3) fail(NRS_ERR_SHAPE, "cuda mha: input must be [batch, seq, d_model]");
  const size_t batch = x->shape[0], seq = x->shape[1], d = x->shape[2];
  if (d != d_model || num_heads == 0 || d_model % num_heads != 0) fail(NRS_ERR_SHAPE, "cuda mha: d_model / num_heads mismatch");
  auto proj = [&](const NodeP& w) { return reshape(matmul(reshape(x, {batch * seq, d}), w), {batch, seq, d}); };
  NodeP q = proj(w_q), k = proj(w_k), v = proj(w_v);
  // The reference slices the heads out column by column, runs attention_batch per head and
  // concatenates (multihead.rs:94-107).  The same arithmetic in one pass: heads become extra
  // batch entries, attention_batch runs once over [batch*heads, seq, d_head].
  const size_t d_head = d_model / num_heads;
  if (nrs_attention_supported((int)seq, (int)d_head))   // short sequences: the whole core in one kernel, heads in place
    return reshape(matmul(reshape(fused_attention(q, k, v, num_heads, causal), {batch * seq, d}), w_o), {batch, seq, d});
  auto split = [&](const NodeP& t) { return permute_heads(t, batch, seq, num_heads, d_head, true); };
  NodeP attended = attention_batch(split(q), split(k), split(v), causal);
  NodeP concat = permute_heads(attended, batch, seq, num_heads, d_head, false);
  return reshape(matmul(reshape(concat, {batch * seq, d}), w_o), {batch, seq, d});
}

static NodeP block_body(const TransformerBlock& b, const NodeP& x, bool final_norm) {
  if (!x || x->shape.size() != 3) fail(NRS_ERR_SHAPE, "cuda transformer block: input must be [batch, seq, d_model]");
  const size_t batch = x->shape[0], seq = x->shape[1], d = x->shape[2];
  NodeP attn_out = b.mha.forward_batch(x);
  NodeP x1 = b.fused_epilogues ? layernorm_residual(x, attn_out, b.norm1.gamma, b.norm1.beta, b.norm1.eps, true)
                               : b.norm1.forward(add(x, attn_out));
  NodeP flat = reshape(x1, {batch * seq, d});
  NodeP h, ff;
  if (b.fused_epilogues) {
    h = linear_act(flat, b.ff1.weights, b.ff1.bias, b.act);
    ff = linear_act(h, b.ff2.weights, b.ff2.bias, NRS_ACT_NONE);
  } else {
    h = b.ff1.forward(flat);
    h = b.act == NRS_ACT_GELU ? gelu(h) : relu(h);
    ff = b.ff2.forward(h);
  }
  NodeP ff_out = reshape(ff, {batch, seq, d});
  if (final_norm && b.fused_epilogues) return layernorm_residual(x1, ff_out, b.norm2.gamma, b.norm2.beta, b.norm2.eps, true);
  NodeP x2 = add(x1, ff_out);
  return final_norm ? b.norm2.forward(x2) : x2;
}

NodeP TransformerBlock::forward(const NodeP& x) const { return block_body(*this, x, true); }
NodeP TransformerBlock::forward_no_final_norm(const NodeP& x) const { return block_body(*this, x, false); }

}  // namespace cuda
}  // namespace nrs
