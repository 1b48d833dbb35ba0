// Native training loop for sequential models + data-parallel gradient exchange.
//
// One nrs_trainer_step is the reference's user loop (examples/cifar_cuda.rs:
// 267-286): to_cuda(batch) -> zero_grad -> forward -> cross-entropy ->
// backward_graph -> optimizer.step, built from the same graph operators as
// graph.cu.  Parameters, gradients and AdamW moments live in flat blocks, so
// the optimizer is one launch and the data-parallel exchange is one
// ncclAllReduce per bucket, issued on a second stream as soon as backward has
// produced the bucket, overlapping the rest of backward.
//
// The gradient exchange itself lives in dp.cu (DpGroup).
#include <algorithm>
#include <cstring>
#include <unordered_set>

#include "host/graph.h"
#include "host/dp.h"
#include "host/checkpoint.h"
#include "nrs_checkpoint.h"
#include <map>
#include <cstdio>
#include "nrs_graph.h"
#include "nrs_internal.h"

using nrs::NodeP;

struct nrs_trainer {
  nrs_ctx* ctx = nullptr;
  std::vector<nrs_layer_spec> layers;
  std::vector<size_t> in_shape;
  int classes = 0;
  bool fuse = false;
  std::vector<NodeP> params;            // [w0,b0,w1,b1,...]
  std::vector<NodeP> buffers;           // running statistics of the batchnorm layers [mean0,var0,...]
  bool training = true;
  float bn_momentum = 0.9f, bn_eps = 1e-5f;
  std::shared_ptr<nrs::FlatStore> flat;
  std::unique_ptr<nrs::cuda::AdamW> opt;
  float* loss_dev = nullptr;
  // Loss read-back one step behind (nrs_trainer_step_staged_lagged): pinned slots the stream copies each
  // step's loss into, and the events that say a slot is filled.
  float* loss_ring = nullptr;
  cudaEvent_t loss_ready[2] = {nullptr, nullptr};
  bool loss_pending[2] = {false, false};
  int loss_slot = 0;
  // staging for host inputs (grow-only device buffers)
  float* x_dev = nullptr; size_t x_cap = 0;
  float* t_dev = nullptr; size_t t_cap = 0;
  // Double-buffered input staging (nrs_trainer_stage_next / nrs_trainer_step_staged): while the compute
  // stream works on one slot, the copy stream fills the other from host memory.  The slots are plain
  // cudaMalloc blocks, not pool blocks: the pool recycles in compute-stream order, which a second stream
  // writing into a recycled block would violate.
  struct Slot {
    float* x = nullptr; size_t x_cap = 0;
    float* t = nullptr; size_t t_cap = 0;
    float* labels = nullptr; size_t labels_cap = 0;   // int32 class indices (in a float-sized block) when `indexed`
    int batch = 0;
    bool pending = false, used = false, indexed = false;
    cudaEvent_t filled = nullptr, consumed = nullptr;
  };
  Slot slots[2];
  int fill_idx = 0, run_idx = 0;
  cudaStream_t copy_stream = nullptr;
  // On-device augmentation of staged batches (nrs_trainer_set_augment): off when max_shift < 0.
  int aug_shift = -1, aug_flip = 0;
  float* aug_buf = nullptr; size_t aug_cap = 0;
  // Token models (first layer NRS_LAYER_EMBEDDING): the input is int32 ids [batch, seq] and the loss runs
  // over batch * seq rows.
  bool token_input = false;
  size_t rows_per_sample = 1;
  NodeP pos_table;                      // sinusoidal table of the embedding layer (no gradient)
  // data parallel
  int rank = 0, world = 1, global_batch = 0;
  bool sync_batchnorm = false;          // batch statistics over all ranks' shards (nrs_trainer_set_sync_batchnorm)
  double dp_timeout_ms = 300000.0;      // joining the communicator, and every host wait of a step
  std::unique_ptr<nrs::DpGroup> dp;
  ~nrs_trainer() {
    if (ctx && ctx->weight_set.owner == this) nrs_weight_set_clear(ctx);
    dp.reset();
    if (copy_stream) { cudaStreamSynchronize(copy_stream); cudaStreamDestroy(copy_stream); }
    for (Slot& sl : slots) {
      if (sl.filled) cudaEventDestroy(sl.filled);
      if (sl.consumed) cudaEventDestroy(sl.consumed);
      if (sl.x) cudaFree(sl.x);
      if (sl.t) cudaFree(sl.t);
      if (sl.labels) cudaFree(sl.labels);
    }
    if (aug_buf) cudaFree(aug_buf);
    if (loss_ring) {
      if (ctx) cudaStreamSynchronize(ctx->stream);   // a queued loss copy may still target the pinned slots
      cudaFreeHost(loss_ring);
      for (cudaEvent_t e : loss_ready) if (e) cudaEventDestroy(e);
    }
    opt.reset();
    params.clear();
    buffers.clear();
    pos_table.reset();
    flat.reset();
    if (ctx) {
      if (loss_dev) nrs_free(ctx, loss_dev);
      if (x_dev) nrs_free(ctx, x_dev);
      if (t_dev) nrs_free(ctx, t_dev);
    }
  }
};

namespace {

void fail(int code, const std::string& m) { throw nrs::Error(code, m); }

void validate_and_build_params(nrs_trainer* t) {
  // Walk the shapes once to validate the spec and create the parameters.
  std::vector<size_t> shp = t->in_shape;  // per-sample
  for (size_t li = 0; li < t->layers.size(); ++li) {
    const nrs_layer_spec& l = t->layers[li];
    switch (l.kind) {
      case NRS_LAYER_CONV: {
        if (shp.size() != 3) fail(NRS_ERR_SHAPE, "trainer: conv layer needs a [C,H,W] input");
        if (l.a != (int)shp[0]) fail(NRS_ERR_SHAPE, "trainer: conv c_in does not match the incoming channels");
        if (l.b <= 0 || l.c <= 0 || l.d <= 0 || l.e < 0) fail(NRS_ERR_SHAPE, "trainer: bad conv hyper-parameters");
        if ((int)shp[1] + 2 * l.e < l.c || (int)shp[2] + 2 * l.e < l.c) fail(NRS_ERR_SHAPE, "trainer: conv kernel too large");
        t->params.push_back(nrs::node_new(t->ctx, nullptr, {(size_t)l.b, (size_t)l.a, (size_t)l.c, (size_t)l.c}));
        t->params.push_back(nrs::node_new(t->ctx, nullptr, {(size_t)l.b}));
        shp = {(size_t)l.b, (shp[1] + 2 * l.e - l.c) / l.d + 1, (shp[2] + 2 * l.e - l.c) / l.d + 1};
        break;
      }
      case NRS_LAYER_MAXPOOL:
        if (shp.size() != 3) fail(NRS_ERR_SHAPE, "trainer: maxpool needs a [C,H,W] input");
        if (l.a <= 0 || l.b <= 0 || l.a > (int)shp[1] || l.a > (int)shp[2]) fail(NRS_ERR_SHAPE, "trainer: bad maxpool window");
        shp = {shp[0], (shp[1] - l.a) / l.b + 1, (shp[2] - l.a) / l.b + 1};
        break;
      case NRS_LAYER_FLATTEN: {
        size_t n = 1;
        for (size_t d : shp) n *= d;
        shp = {n};
        break;
      }
      case NRS_LAYER_LINEAR:
        // [F] per sample, or [seq, F] per sample of a token model (applied to every position)
        if ((shp.size() != 1 && shp.size() != 2) || (int)shp.back() != l.a || l.b <= 0)
          fail(NRS_ERR_SHAPE, "trainer: linear layer input size mismatch");
        t->params.push_back(nrs::node_new(t->ctx, nullptr, {(size_t)l.a, (size_t)l.b}));
        t->params.push_back(nrs::node_new(t->ctx, nullptr, {(size_t)l.b}));
        shp.back() = (size_t)l.b;
        break;
      case NRS_LAYER_EMBEDDING: {
        if (li != 0) fail(NRS_ERR_ARG, "trainer: an embedding layer must come first (it reads the token ids)");
        if (shp.size() != 1) fail(NRS_ERR_SHAPE, "trainer: a token model's input shape is {seq}");
        if (l.a <= 0 || l.b <= 0 || l.c < 0) fail(NRS_ERR_SHAPE, "trainer: bad embedding hyper-parameters");
        if (l.c > 0 && (size_t)l.c < shp[0]) fail(NRS_ERR_SHAPE, "sequence longer than max_len");
        t->params.push_back(nrs::node_new(t->ctx, nullptr, {(size_t)l.a, (size_t)l.b}));
        if (l.c > 0) t->pos_table = nrs::cuda::PositionalEncoding::make(t->ctx, (size_t)l.b, (size_t)l.c).table;
        t->token_input = true;
        t->rows_per_sample = shp[0];
        shp = {shp[0], (size_t)l.b};
        break;
      }
      case NRS_LAYER_TRANSFORMER_BLOCK: {
        if (shp.size() != 2 || (int)shp[1] != l.a) fail(NRS_ERR_SHAPE, "trainer: transformer block needs a [seq, d_model] input");
        if (l.b <= 0 || l.a % l.b != 0 || l.c <= 0) fail(NRS_ERR_SHAPE, "trainer: d_model must be divisible by num_heads");
        if (l.d != NRS_ACT_RELU && l.d != NRS_ACT_GELU) fail(NRS_ERR_ARG, "trainer: transformer block activation must be ReLU or GELU");
        const size_t d = (size_t)l.a, ff = (size_t)l.c;
        // parameters() order of src/nn/transformer_block.rs:58-66
        for (int k = 0; k < 4; ++k) t->params.push_back(nrs::node_new(t->ctx, nullptr, {d, d}));          // w_q w_k w_v w_o
        for (int k = 0; k < 4; ++k) t->params.push_back(nrs::node_new(t->ctx, nullptr, {d}));             // norm1/2 gamma, beta
        t->params.push_back(nrs::node_new(t->ctx, nullptr, {d, ff}));
        t->params.push_back(nrs::node_new(t->ctx, nullptr, {ff}));
        t->params.push_back(nrs::node_new(t->ctx, nullptr, {ff, d}));
        t->params.push_back(nrs::node_new(t->ctx, nullptr, {d}));
        break;
      }
      case NRS_LAYER_LAYERNORM:
        if (shp.empty() || (int)shp.back() != l.a) fail(NRS_ERR_SHAPE, "trainer: layernorm feature count mismatch");
        t->params.push_back(nrs::node_new(t->ctx, nullptr, {(size_t)l.a}));
        t->params.push_back(nrs::node_new(t->ctx, nullptr, {(size_t)l.a}));
        break;
      case NRS_LAYER_RELU:
      case NRS_LAYER_GELU:
        break;
      case NRS_LAYER_BATCHNORM: {
        if ((shp.size() != 3 && shp.size() != 1) || l.a != (int)shp[0])
          fail(NRS_ERR_SHAPE, "trainer: batchnorm channels do not match the incoming [C,H,W] or [F]");
        t->params.push_back(nrs::node_new(t->ctx, nullptr, {(size_t)l.a}));   // gamma
        t->params.push_back(nrs::node_new(t->ctx, nullptr, {(size_t)l.a}));   // beta
        std::vector<float> zeros((size_t)l.a, 0.0f), ones((size_t)l.a, 1.0f);
        for (const std::vector<float>* init : {&zeros, &ones}) {
          NodeP b = nrs::node_new(t->ctx, init->data(), {(size_t)l.a});
          b->requires_grad = false;
          nrs::cuda::to_cuda(b);
          t->buffers.push_back(b);
        }
        break;
      }
      case NRS_LAYER_DROPOUT:
      case NRS_LAYER_DROPOUT2D:
        if (l.a < 0 || l.a > 1000000) fail(NRS_ERR_ARG, "trainer: dropout probability outside [0, 1000000] ppm");
        if (l.kind == NRS_LAYER_DROPOUT2D && shp.size() != 3) fail(NRS_ERR_SHAPE, "trainer: dropout2d needs a [C,H,W] input");
        break;
      default:
        fail(NRS_ERR_ARG, "trainer: unknown layer kind");
    }
  }
  if (t->token_input ? (shp.size() != 2 || (int)shp[1] != t->classes) : (shp.size() != 1 || (int)shp[0] != t->classes))
    fail(NRS_ERR_SHAPE, "trainer: model output does not match `classes`");
  if (t->params.empty()) fail(NRS_ERR_ARG, "trainer: model has no parameters");
  for (auto& p : t->params) {
    p->host.assign(p->len(), 0.0f);
    nrs::cuda::to_cuda(p);
    p->host.clear();
    p->host.shrink_to_fit();
  }
  t->flat = nrs::cuda::flatten_params(t->params);
}

// x@W + b (+ activation) on the last axis of h: [rows, F], or every position of [batch, seq, F].
NodeP linear_layer(nrs_trainer* t, const NodeP& h, const NodeP& w, const NodeP& b, int act) {
  const bool tokens = h->shape.size() == 3;
  NodeP in = tokens ? nrs::cuda::reshape(h, {h->shape[0] * h->shape[1], h->shape[2]}) : h;
  NodeP out;
  if (t->fuse) {
    out = nrs::cuda::linear_act(in, w, b, act);
  } else {
    out = nrs::cuda::add(nrs::cuda::matmul(in, w), b);
    if (act == NRS_ACT_RELU) out = nrs::cuda::relu(out);
    else if (act == NRS_ACT_GELU) out = nrs::cuda::gelu(out);
  }
  return tokens ? nrs::cuda::reshape(out, {h->shape[0], h->shape[1], out->shape[1]}) : out;
}

NodeP forward(nrs_trainer* t, const NodeP& x, const int32_t* ids_dev, size_t batch) {
  NodeP h = x;
  size_t pi = 0, bi = 0;
  for (size_t li = 0; li < t->layers.size(); ++li) {
    const nrs_layer_spec& l = t->layers[li];
    const bool relu_next = t->fuse && li + 1 < t->layers.size() && t->layers[li + 1].kind == NRS_LAYER_RELU;
    switch (l.kind) {
      case NRS_LAYER_CONV: {
        // The layer list shows what reads this output: if it is a stride-1 convolution, its
        // NHWC operand planes are written by this layer's kernel.
        const size_t nx = li + (relu_next ? 2 : 1);
        const bool conv_reads = nx < t->layers.size() && t->layers[nx].kind == NRS_LAYER_CONV && t->layers[nx].d == 1;
        h = nrs::cuda::conv2d_act(h, t->params[pi], t->params[pi + 1], (size_t)l.d, (size_t)l.e,
                                  relu_next ? NRS_ACT_RELU : NRS_ACT_NONE, conv_reads);
        pi += 2;
        if (relu_next) ++li;
        break;
      }
      case NRS_LAYER_LINEAR: {
        const bool gelu_next = t->fuse && li + 1 < t->layers.size() && t->layers[li + 1].kind == NRS_LAYER_GELU;
        h = linear_layer(t, h, t->params[pi], t->params[pi + 1], relu_next ? NRS_ACT_RELU : gelu_next ? NRS_ACT_GELU : NRS_ACT_NONE);
        if (relu_next || gelu_next) ++li;
        pi += 2;
        break;
      }
      case NRS_LAYER_EMBEDDING: {
        nrs::cuda::Embedding e;
        e.weight = t->params[pi];
        e.vocab_size = (size_t)l.a;
        e.embedding_dim = (size_t)l.b;
        h = e.forward_resident(ids_dev, batch, t->in_shape[0], t->pos_table);
        pi += 1;
        break;
      }
      case NRS_LAYER_TRANSFORMER_BLOCK: {
        nrs::cuda::TransformerBlock b;
        const NodeP* p = &t->params[pi];
        b.mha.w_q = p[0]; b.mha.w_k = p[1]; b.mha.w_v = p[2]; b.mha.w_o = p[3];
        b.mha.d_model = (size_t)l.a; b.mha.num_heads = (size_t)l.b; b.mha.causal = (l.e & 1) != 0;
        b.norm1.gamma = p[4]; b.norm1.beta = p[5]; b.norm2.gamma = p[6]; b.norm2.beta = p[7];
        b.ff1.weights = p[8]; b.ff1.bias = p[9]; b.ff2.weights = p[10]; b.ff2.bias = p[11];
        b.d_model = (size_t)l.a; b.d_ff = (size_t)l.c; b.act = l.d; b.fused_epilogues = t->fuse;
        h = (l.e & 2) ? b.forward_no_final_norm(h) : b.forward(h);
        pi += 12;
        break;
      }
      case NRS_LAYER_LAYERNORM:
        h = nrs::cuda::layernorm(h, t->params[pi], t->params[pi + 1], 1e-5f);
        pi += 2;
        break;
      case NRS_LAYER_RELU: h = nrs::cuda::relu(h); break;
      case NRS_LAYER_GELU: h = nrs::cuda::gelu(h); break;
      case NRS_LAYER_MAXPOOL: {
        const bool conv_reads = li + 1 < t->layers.size() && t->layers[li + 1].kind == NRS_LAYER_CONV && t->layers[li + 1].d == 1;
        h = nrs::cuda::maxpool2d(h, (size_t)l.a, (size_t)l.b, conv_reads);
        break;
      }
      case NRS_LAYER_FLATTEN: h = nrs::cuda::flatten(h); break;
      case NRS_LAYER_BATCHNORM:
        // a ReLU behind the layer rides in its two passes (relu_next is only set when fusing is on)
        h = nrs::cuda::batchnorm_act(h, t->params[pi], t->params[pi + 1], t->buffers[bi], t->buffers[bi + 1],
                                     t->bn_momentum, t->bn_eps, t->training, relu_next ? NRS_ACT_RELU : NRS_ACT_NONE);
        pi += 2;
        bi += 2;
        if (relu_next) ++li;
        break;
      case NRS_LAYER_DROPOUT: h = nrs::cuda::dropout(h, (float)l.a * 1e-6f, t->training); break;
      case NRS_LAYER_DROPOUT2D: h = nrs::cuda::dropout2d(h, (float)l.a * 1e-6f, t->training); break;
    }
  }
  return h;
}

// The model's contraction weights, staged for the tensor-core kernels in one launch per step
// (weight_set.cu) instead of one small launch per layer and pass.
void stage_weights(nrs_trainer* t) {
  nrs_ctx* ctx = t->ctx;
  NrsWeightSet& ws = ctx->weight_set;
  if (ws.owner != t || ws.mode != ctx->math_mode) {
    std::vector<NrsWeightDesc> d;
    auto linear = [&](const NodeP& w) {   // W[in,out]: transposed for x@W, as stored for dz@W^T
      const int in = (int)w->shape[0], out = (int)w->shape[1];
      if (in < 32 || out < 32) return;    // thin products run on the FFMA kernels
      d.push_back(NrsWeightDesc{w->data, NRS_WF_LINEAR_T, out, in, 0, 0, 0});
      d.push_back(NrsWeightDesc{w->data, NRS_WF_LINEAR_ROWS, in, out, 0, 0, 0});
    };
    size_t pi = 0;
    bool first_contraction = true;
    for (const nrs_layer_spec& l : t->layers) {
      switch (l.kind) {
        case NRS_LAYER_CONV:
          if (l.d == 1 && l.a % 32 == 0 && l.b % 32 == 0) {
            const NodeP& w = t->params[pi];
            d.push_back(NrsWeightDesc{w->data, NRS_WF_CONV_FWD, 0, 0, l.b, l.a, l.c * l.c});
            if (!first_contraction) d.push_back(NrsWeightDesc{w->data, NRS_WF_CONV_DGRAD, 0, 0, l.b, l.a, l.c * l.c});
          }
          first_contraction = false;
          pi += 2;
          break;
        case NRS_LAYER_LINEAR:
          linear(t->params[pi]);
          first_contraction = false;
          pi += 2;
          break;
        case NRS_LAYER_BATCHNORM:
        case NRS_LAYER_LAYERNORM: pi += 2; break;
        case NRS_LAYER_EMBEDDING: pi += 1; break;
        case NRS_LAYER_TRANSFORMER_BLOCK:
          for (int k : {0, 1, 2, 3, 8, 10}) linear(t->params[pi + k]);
          first_contraction = false;
          pi += 12;
          break;
        default: break;
      }
    }
    nrs::check(ctx, nrs_weight_set_build(ctx, d.data(), (int)d.size()));
    ws.owner = t;
    ws.mode = ctx->math_mode;
  }
  if (!ws.fresh) nrs::check(ctx, nrs_weight_set_refresh(ctx));
}

// For the duration of a scope, tells the context which samples of the global batch this rank holds, so that
// per-sample random draws (dropout masks, augmentation) are the ones a single process would make for them.
// Applies when the batch is this rank's contiguous share of the global batch (nrs_dp_shard_range).
struct ShardScope {
  nrs_ctx* c;
  ShardScope(nrs_trainer* t, int batch) : c(t->ctx) {
    if (!t->dp || t->world <= 1) return;
    int b0 = 0, b1 = 0;
    if (nrs_dp_shard_range(t->global_batch, t->rank, t->world, &b0, &b1) != NRS_OK || b1 - b0 != batch) return;
    c->shard_begin = b0;
    c->shard_local = batch;
    c->shard_global = t->global_batch;
  }
  ~ShardScope() { c->shard_begin = c->shard_local = c->shard_global = 0; }
};

// Whoever writes a parameter behind the optimizer's back (uploads, checkpoints) calls this.
void weights_changed(nrs_trainer* t) {
  if (t->ctx->weight_set.owner == t) t->ctx->weight_set.fresh = false;
}

// One step's inputs, all on the device: x (float samples) or ids (token models); targets as one-hot rows
// or as int32 class indices (one per loss row).
struct StepInput {
  const float* x = nullptr;
  const int32_t* ids = nullptr;
  const float* target = nullptr;
  const int32_t* labels = nullptr;
  int batch = 0;
};

void run_step(nrs_trainer* t, const StepInput& in, bool optimize) {
  nrs_ctx* ctx = t->ctx;
  const int batch = in.batch;
  if (batch <= 0) fail(NRS_ERR_SHAPE, "trainer: batch must be positive");
  if (t->token_input ? !in.ids : !in.x) fail(NRS_ERR_ARG, t->token_input ? "trainer: this model reads token ids" : "trainer: this model reads float samples");
  const size_t rows = (size_t)batch * t->rows_per_sample;
  if (rows > 2147483647u) fail(NRS_ERR_UNSUPPORTED, "trainer: more than 2^31-1 loss rows");
  // Input nodes wrap the caller's device buffers (not owned).
  auto wrap = [&](const float* dev, std::vector<size_t> shape) {
    auto n = std::make_shared<nrs::Node>();
    n->ctx = ctx;
    n->shape = std::move(shape);
    n->data = const_cast<float*>(dev);
    n->owns_data = false;
    n->requires_grad = false;  // examples/cifar_cuda.rs:270: skips the first conv's data gradient
    return n;
  };
  if (!in.target && !in.labels) fail(NRS_ERR_ARG, "trainer: no targets");
  NodeP x;
  if (!t->token_input) {
    std::vector<size_t> xs{(size_t)batch};
    xs.insert(xs.end(), t->in_shape.begin(), t->in_shape.end());
    x = wrap(in.x, xs);
  }

  nrs::cuda::zero_grad(t->params);
  stage_weights(t);
  // batch-normalisation statistics over the global batch: the layers find the cross-rank sum in the context
  // for the duration of this step (forward and backward)
  struct StatSyncScope {
    nrs_ctx* c;
    explicit StatSyncScope(nrs_ctx* ctx, nrs::DpGroup* g) : c(ctx) {
      if (g) {
        c->stat_sync.user = g;
        c->stat_sync.all_reduce_sum = [](void* user, float* dev, size_t count) -> int {
          nrs::DpGroup* grp = static_cast<nrs::DpGroup*>(user);
          try {
            grp->all_reduce_sum(dev, count);
          } catch (const nrs::Error& e) {
            return nrs_fail(grp->context(), e.code, "%s", e.what());
          }
          return NRS_OK;
        };
      }
    }
    ~StatSyncScope() { c->stat_sync = NrsStatSync(); }
  } stat_sync(ctx, t->sync_batchnorm && t->dp && t->world > 1 && t->training ? t->dp.get() : nullptr);
  ShardScope shard(t, batch);
  NodeP logits = forward(t, x, in.ids, (size_t)batch);
  if (logits->shape.size() == 3) logits = nrs::cuda::reshape(logits, {rows, (size_t)t->classes});
  const bool dp = t->dp && t->world > 1 && optimize;
  const size_t divisor = (t->world > 1 ? (size_t)t->global_batch : (size_t)batch) * t->rows_per_sample;
  if (divisor > 2147483647u) fail(NRS_ERR_UNSUPPORTED, "trainer: more than 2^31-1 loss rows");
  // class indices feed the loss kernel directly: the values of the one-hot rows the reference's
  // cross_entropy takes (src/cuda/loss/cross_entropy.rs:74-98) without the dense tensor
  if (in.target) nrs::cuda::cross_entropy_fused(logits, wrap(in.target, {rows, (size_t)t->classes}), t->loss_dev, (int)divisor);
  else nrs::cuda::cross_entropy_fused_indexed(logits, in.labels, t->loss_dev, (int)divisor);

  if (dp) {
    // Each bucket is all-reduced on the comm stream as soon as backward has produced it, and its
    // parameters are updated there right behind the reduce (DpGroup::after_bucket), so both overlap
    // the rest of backward; the compute stream joins at the end.
    // The weight planes of a bucket are restaged there too, behind its update: the next step finds them ready.
    t->opt->begin_flat_step(t->params);
    ctx->weight_set.refreshed_jobs = 0;
    t->dp->begin_step();
    try {
      nrs::backward_graph_dp(logits, t->dp.get());
      t->dp->finish();
    } catch (...) {
      ctx->weight_set.fresh = false;
      throw;
    }
    t->opt->end_flat_step();
    // every plane was rewritten behind its bucket's update: still fresh; otherwise restage at the next step
    ctx->weight_set.fresh = ctx->weight_set.n_jobs > 0 && ctx->weight_set.refreshed_jobs == ctx->weight_set.n_jobs;
    ctx->weight_set.refreshed_jobs = 0;
  } else {
    nrs::backward_graph(logits);
    if (optimize) {
      t->opt->step(t->params);
      ctx->weight_set.fresh = false;   // the planes describe the weights before this update
    }
  }
}

void stage(nrs_trainer* t, float** buf, size_t* cap, const float* host, size_t floats) {
  if (floats > *cap) {
    if (*buf) nrs_free(t->ctx, *buf);
    void* p = nullptr;
    nrs::check(t->ctx, nrs_alloc(t->ctx, floats * sizeof(float), 0, &p));
    *buf = (float*)p;
    *cap = floats;
  }
  nrs::check(t->ctx, nrs_h2d(t->ctx, *buf, host, floats * sizeof(float)));
}

void cuda_ok(cudaError_t e, const char* what) {
  if (e != cudaSuccess) fail(NRS_ERR_CUDA, std::string("trainer: ") + what + " failed: " + cudaGetErrorString(e));
}

// Grows a staging block.  Growth is rare (the first batch, or a larger one): it waits for everything in
// flight so that nothing still reads the old block.
void grow_slot_block(float** buf, size_t* cap, size_t floats) {
  if (floats <= *cap) return;
  cuda_ok(cudaDeviceSynchronize(), "synchronize before growing a staging block");
  if (*buf) cuda_ok(cudaFree(*buf), "cudaFree of a staging block");
  *buf = nullptr;
  *cap = 0;
  void* p = nullptr;
  if (cudaMalloc(&p, floats * sizeof(float)) != cudaSuccess) {
    cudaGetLastError();
    fail(NRS_ERR_ALLOC, "trainer: out of device memory for an input staging block");
  }
  *buf = (float*)p;
  *cap = floats;
}

// Reads the loss of the step just issued.  Under data parallelism the wait runs through the group's
// deadline loop, so a rank that never arrives surfaces as NRS_ERR_TIMEOUT instead of a hang.
void read_loss(nrs_trainer* t, float* loss_out) {
  if (t->dp && t->world > 1) t->dp->host_wait(t->ctx->stream);
  nrs::check(t->ctx, nrs_d2h(t->ctx, loss_out, t->loss_dev, sizeof(float)));
}

size_t sample_words(const nrs_trainer* t) {   // 4-byte words per sample: floats, or token ids
  size_t per = 1;
  for (size_t d : t->in_shape) per *= d;
  return per;
}

// x_host: float samples, or int32 token ids for a token model (same word size).  Exactly one of
// target_host (one-hot rows) / labels_host (one class index per loss row) is given.
void stage_next(nrs_trainer* t, const void* x_host, const float* target_host, const int32_t* labels_host, int batch) {
  if (batch <= 0) fail(NRS_ERR_SHAPE, "trainer: batch must be positive");
  nrs_trainer::Slot& sl = t->slots[t->fill_idx];
  if (sl.pending) fail(NRS_ERR_ARG, "trainer: both staging slots hold a batch that no step has consumed yet");
  if (!t->copy_stream) cuda_ok(cudaStreamCreateWithFlags(&t->copy_stream, cudaStreamNonBlocking), "copy stream creation");
  if (!sl.filled) {
    cuda_ok(cudaEventCreateWithFlags(&sl.filled, cudaEventDisableTiming), "event creation");
    cuda_ok(cudaEventCreateWithFlags(&sl.consumed, cudaEventDisableTiming), "event creation");
  }
  const size_t per = sample_words(t), rows = (size_t)batch * t->rows_per_sample;
  grow_slot_block(&sl.x, &sl.x_cap, per * batch);
  if (labels_host) grow_slot_block(&sl.labels, &sl.labels_cap, rows);
  else grow_slot_block(&sl.t, &sl.t_cap, (size_t)t->classes * rows);
  // the step that last read this slot must have finished with it
  if (sl.used) cuda_ok(cudaStreamWaitEvent(t->copy_stream, sl.consumed, 0), "wait for the slot's last consumer");
  cuda_ok(cudaMemcpyAsync(sl.x, x_host, per * batch * sizeof(float), cudaMemcpyHostToDevice, t->copy_stream), "input copy");
  if (labels_host) {
    cuda_ok(cudaMemcpyAsync(sl.labels, labels_host, rows * sizeof(int32_t), cudaMemcpyHostToDevice, t->copy_stream), "label copy");
  } else {
    cuda_ok(cudaMemcpyAsync(sl.t, target_host, (size_t)t->classes * rows * sizeof(float), cudaMemcpyHostToDevice, t->copy_stream),
            "target copy");
  }
  sl.indexed = labels_host != nullptr;
  cuda_ok(cudaEventRecord(sl.filled, t->copy_stream), "event record");
  sl.batch = batch;
  sl.pending = true;
  t->fill_idx ^= 1;
}

void step_staged(nrs_trainer* t, float* loss_out) {
  nrs_trainer::Slot& sl = t->slots[t->run_idx];
  if (!sl.pending) fail(NRS_ERR_ARG, "trainer: no staged batch (call nrs_trainer_stage_next first)");
  cuda_ok(cudaStreamWaitEvent(t->ctx->stream, sl.filled, 0), "wait for the staged batch");
  StepInput in;
  in.batch = sl.batch;
  if (sl.indexed) in.labels = reinterpret_cast<const int32_t*>(sl.labels);   // expanded to one-hot rows by the step
  else in.target = sl.t;
  if (t->token_input) {
    in.ids = reinterpret_cast<const int32_t*>(sl.x);
  } else {
    in.x = sl.x;
    if (t->aug_shift >= 0 && t->training && t->in_shape.size() == 3) {
      grow_slot_block(&t->aug_buf, &t->aug_cap, sample_words(t) * sl.batch);
      ShardScope shard(t, sl.batch);
      nrs::check(t->ctx, nrs_augment_flip_shift(t->ctx, sl.x, t->aug_buf, sl.batch, (int)t->in_shape[0], (int)t->in_shape[1],
                                                (int)t->in_shape[2], t->aug_shift, t->aug_flip));
      in.x = t->aug_buf;
    }
  }
  run_step(t, in, true);
  cuda_ok(cudaEventRecord(sl.consumed, t->ctx->stream), "event record");
  sl.pending = false;
  sl.used = true;
  t->run_idx ^= 1;
  if (loss_out) read_loss(t, loss_out);
}

// Issues the staged step, queues an asynchronous copy of its loss into a pinned slot, and hands back the loss of
// the step BEFORE it (which has finished, or nearly): the host is never more than one step behind the device
// and the device never waits for the host to enqueue.
void step_staged_lagged(nrs_trainer* t, float* prev_loss_out, int* have_prev) {
  if (!t->loss_ring) {
    cuda_ok(cudaMallocHost((void**)&t->loss_ring, 2 * sizeof(float)), "pinned loss slots");
    for (int i = 0; i < 2; ++i) cuda_ok(cudaEventCreateWithFlags(&t->loss_ready[i], cudaEventDisableTiming), "event creation");
  }
  step_staged(t, nullptr);
  const int cur = t->loss_slot, prev = cur ^ 1;
  cuda_ok(cudaMemcpyAsync(t->loss_ring + cur, t->loss_dev, sizeof(float), cudaMemcpyDeviceToHost, t->ctx->stream), "loss copy");
  cuda_ok(cudaEventRecord(t->loss_ready[cur], t->ctx->stream), "event record");
  t->loss_pending[cur] = true;
  t->loss_slot = prev;
  if (have_prev) *have_prev = 0;
  if (t->loss_pending[prev]) {
    if (t->dp && t->world > 1) t->dp->host_wait_event(t->loss_ready[prev]);
    else cuda_ok(cudaEventSynchronize(t->loss_ready[prev]), "waiting for the previous step's loss");
    t->loss_pending[prev] = false;
    if (prev_loss_out) *prev_loss_out = t->loss_ring[prev];
    if (have_prev) *have_prev = 1;
  }
}

template <class F>
int guarded(nrs_ctx* ctx, F&& f) {
  try {
    f();
    return NRS_OK;
  } catch (const nrs::Error& e) {
    return nrs_fail(ctx, e.code, "%s", e.what());
  } catch (const std::exception& e) {
    return nrs_fail(ctx, NRS_ERR_ARG, "%s", e.what());
  }
}

// Synchronous step from host buffers: inputs and targets are copied on the compute stream.
int host_step(nrs_trainer* t, const void* x_host, const float* target_host, const int32_t* labels_host, int batch,
              float* loss_out, bool optimize, bool tokens) {
  if (!t) return nrs_fail(nullptr, NRS_ERR_ARG, "trainer: null handle");
  if (!x_host || (!target_host && !labels_host)) return nrs_fail(t->ctx, NRS_ERR_ARG, "trainer: null input");
  return guarded(t->ctx, [&] {
    if (batch <= 0) fail(NRS_ERR_SHAPE, "trainer: batch must be positive");
    if (tokens != t->token_input)
      fail(NRS_ERR_ARG, tokens ? "trainer: this model reads float samples, not token ids" : "trainer: this model reads token ids (use the *_tokens entry points)");
    const size_t rows = (size_t)batch * t->rows_per_sample;
    stage(t, &t->x_dev, &t->x_cap, (const float*)x_host, sample_words(t) * batch);
    StepInput in;
    in.batch = batch;
    if (tokens) in.ids = reinterpret_cast<const int32_t*>(t->x_dev); else in.x = t->x_dev;
    if (labels_host) {
      stage(t, &t->t_dev, &t->t_cap, reinterpret_cast<const float*>(labels_host), rows);
      in.labels = reinterpret_cast<const int32_t*>(t->t_dev);
    } else {
      stage(t, &t->t_dev, &t->t_cap, target_host, (size_t)t->classes * rows);
      in.target = t->t_dev;
    }
    run_step(t, in, optimize);
    if (loss_out) read_loss(t, loss_out);
  });
}

}  // namespace

extern "C" {

int nrs_trainer_create(nrs_ctx* ctx, const nrs_layer_spec* layers, int n_layers, const int64_t* in_shape,
                       int in_ndim, int classes, float lr, float beta1, float beta2, float eps,
                       float weight_decay, int fuse, nrs_trainer** out) {
  NRS_REQUIRE_CTX(ctx);
  NRS_REQUIRE(ctx, out != nullptr, NRS_ERR_ARG, "nrs_trainer_create: null out handle");
  *out = nullptr;
  NRS_REQUIRE(ctx, layers && n_layers > 0 && in_shape && in_ndim > 0 && classes > 0, NRS_ERR_ARG,
              "nrs_trainer_create: bad arguments");
  nrs_trainer* t = new nrs_trainer();
  const int st = guarded(ctx, [&] {
    t->ctx = ctx;
    t->layers.assign(layers, layers + n_layers);
    for (int i = 0; i < in_ndim; ++i) {
      if (in_shape[i] <= 0) fail(NRS_ERR_SHAPE, "nrs_trainer_create: non-positive input extent");
      t->in_shape.push_back((size_t)in_shape[i]);
    }
    t->classes = classes;
    t->fuse = fuse != 0;
    validate_and_build_params(t);
    t->opt.reset(new nrs::cuda::AdamW(ctx, lr, beta1, beta2, eps, weight_decay));
    void* p = nullptr;
    nrs::check(ctx, nrs_alloc(ctx, sizeof(float), 1, &p));
    t->loss_dev = (float*)p;
  });
  if (st != NRS_OK) { delete t; return st; }
  *out = t;
  return NRS_OK;
}

int nrs_trainer_free(nrs_trainer* t) {
  if (t && t->ctx) cudaStreamSynchronize(t->ctx->stream);
  delete t;
  return NRS_OK;
}

int nrs_trainer_param_count(const nrs_trainer* t) { return t ? (int)t->params.size() : -1; }

int nrs_trainer_buffer_count(const nrs_trainer* t) { return t ? (int)t->buffers.size() : -1; }

int64_t nrs_trainer_buffer_len(const nrs_trainer* t, int i) {
  return (t && i >= 0 && i < (int)t->buffers.size()) ? (int64_t)t->buffers[i]->len() : -1;
}

int nrs_trainer_set_buffer(nrs_trainer* t, int i, const float* host) {
  if (!t) return nrs_fail(nullptr, NRS_ERR_ARG, "nrs_trainer_set_buffer: null handle");
  NRS_REQUIRE(t->ctx, host && i >= 0 && i < (int)t->buffers.size(), NRS_ERR_ARG, "nrs_trainer_set_buffer: bad index or null data");
  int st = nrs_h2d(t->ctx, t->buffers[i]->data, host, t->buffers[i]->len() * sizeof(float));
  if (st == NRS_OK) st = nrs_sync(t->ctx);
  return st;
}

int nrs_trainer_get_buffer(nrs_trainer* t, int i, float* host_out) {
  if (!t) return nrs_fail(nullptr, NRS_ERR_ARG, "nrs_trainer_get_buffer: null handle");
  NRS_REQUIRE(t->ctx, host_out && i >= 0 && i < (int)t->buffers.size(), NRS_ERR_ARG, "nrs_trainer_get_buffer: bad index or null output");
  return nrs_d2h(t->ctx, host_out, t->buffers[i]->data, t->buffers[i]->len() * sizeof(float));
}

namespace {

std::string tensor_name(const char* const* names, size_t i, const char* prefix, size_t k) {
  if (names) {
    if (!names[i]) throw nrs::Error(NRS_ERR_ARG, "trainer checkpoint: null name");
    return names[i];
  }
  char buf[32];
  std::snprintf(buf, sizeof buf, "%s.%02zu", prefix, k);
  return buf;
}

std::vector<float> download(nrs_ctx* ctx, const NodeP& n) {
  std::vector<float> h(n->len());
  nrs::check(ctx, nrs_d2h(ctx, h.data(), n->data, h.size() * sizeof(float)));
  return h;
}

void save_checkpoint(nrs_trainer* t, const char* const* names, const char* path) {
  std::vector<nrs::checkpoint::Tensor> out;
  const size_t np = t->params.size();
  for (size_t i = 0; i < np + t->buffers.size(); ++i) {
    const NodeP& n = i < np ? t->params[i] : t->buffers[i - np];
    nrs::checkpoint::Tensor ct;
    ct.name = i < np ? tensor_name(names, i, "param", i) : tensor_name(names, i, "buffer", i - np);
    ct.shape.assign(n->shape.begin(), n->shape.end());
    ct.data = download(t->ctx, n);
    out.push_back(std::move(ct));
  }
  // examples/mnist_cuda_cnn.rs:173-185: optim.t as one f32 (exact below 2^24), then the moments, flat
  size_t steps = 0;
  std::vector<std::vector<float>> moments = t->opt->export_state(&steps);
  out.push_back({"optim.t", {1}, {(float)steps}});
  const size_t half = moments.size() / 2;
  for (size_t i = 0; i < moments.size(); ++i) {
    char buf[32];
    std::snprintf(buf, sizeof buf, i < half ? "optim.m.%02zu" : "optim.v.%02zu", i < half ? i : i - half);
    const int64_t len = (int64_t)moments[i].size();
    out.push_back({buf, {len}, std::move(moments[i])});
  }
  nrs::checkpoint::save(out, path);
}

void load_checkpoint(nrs_trainer* t, const char* const* names, const char* path) {
  std::vector<nrs::checkpoint::Tensor> file = nrs::checkpoint::load(path);
  const std::string p(path);
  const bool named = p.size() >= 12 && p.compare(p.size() - 12, 12, ".safetensors") == 0;
  std::map<std::string, const nrs::checkpoint::Tensor*> by_name;
  for (const auto& ct : file) by_name[ct.name] = &ct;
  const size_t np = t->params.size(), total = np + t->buffers.size();
  auto lookup = [&](size_t i, const std::string& name) -> const nrs::checkpoint::Tensor* {
    if (!named) return i < file.size() ? &file[i] : nullptr;   // the text format is positional
    auto it = by_name.find(name);
    return it == by_name.end() ? nullptr : it->second;
  };
  for (size_t i = 0; i < total; ++i) {
    const NodeP& n = i < np ? t->params[i] : t->buffers[i - np];
    const std::string name = i < np ? tensor_name(names, i, "param", i) : tensor_name(names, i, "buffer", i - np);
    const nrs::checkpoint::Tensor* ct = lookup(i, name);
    if (!ct) throw nrs::Error(NRS_ERR_ARG, "checkpoint is missing tensor `" + name + "`");
    if (ct->data.size() != n->len()) throw nrs::Error(NRS_ERR_SHAPE, "checkpoint tensor `" + name + "` has the wrong size");
    nrs::check(t->ctx, nrs_h2d(t->ctx, n->data, ct->data.data(), ct->data.size() * sizeof(float)));
  }
  nrs::check(t->ctx, nrs_sync(t->ctx));
  // examples/mnist_cuda_cnn.rs:208-218: the optimizer state rides along when "optim.t" is present
  const nrs::checkpoint::Tensor* tt = lookup(total, "optim.t");
  if (!tt || tt->data.size() != 1 || (!named && file.size() != total + 1 + 2 * np)) return;
  std::vector<std::vector<float>> moments;
  for (int pass = 0; pass < 2; ++pass)
    for (size_t i = 0; i < np; ++i) {
      char buf[32];
      std::snprintf(buf, sizeof buf, pass == 0 ? "optim.m.%02zu" : "optim.v.%02zu", i);
      const nrs::checkpoint::Tensor* ct = lookup(total + 1 + (size_t)pass * np + i, buf);
      if (!ct) throw nrs::Error(NRS_ERR_ARG, std::string("checkpoint is missing tensor `") + buf + "`");
      if (ct->data.size() != t->params[i]->len()) throw nrs::Error(NRS_ERR_SHAPE, std::string("checkpoint tensor `") + buf + "` has the wrong size");
      moments.push_back(ct->data);
    }
  t->opt->import_state((size_t)tt->data[0], moments);
}

}  // namespace

int nrs_trainer_save_checkpoint(nrs_trainer* t, const char* const* names, const char* path) {
  if (!t || !path) return nrs_fail(nullptr, NRS_ERR_ARG, "nrs_trainer_save_checkpoint: null handle or path");
  return guarded(t->ctx, [&] { save_checkpoint(t, names, path); });
}

int nrs_trainer_load_checkpoint(nrs_trainer* t, const char* const* names, const char* path) {
  if (!t || !path) return nrs_fail(nullptr, NRS_ERR_ARG, "nrs_trainer_load_checkpoint: null handle or path");
  weights_changed(t);
  return guarded(t->ctx, [&] { load_checkpoint(t, names, path); });
}

int nrs_trainer_set_training(nrs_trainer* t, int training) {
  if (!t) return nrs_fail(nullptr, NRS_ERR_ARG, "nrs_trainer_set_training: null handle");
  t->training = training != 0;
  return NRS_OK;
}

int nrs_trainer_set_batchnorm(nrs_trainer* t, float momentum, float eps) {
  if (!t) return nrs_fail(nullptr, NRS_ERR_ARG, "nrs_trainer_set_batchnorm: null handle");
  NRS_REQUIRE(t->ctx, momentum >= 0.0f && momentum <= 1.0f && eps > 0.0f, NRS_ERR_ARG,
              "nrs_trainer_set_batchnorm: momentum must lie in [0,1] and eps must be positive");
  t->bn_momentum = momentum;
  t->bn_eps = eps;
  return NRS_OK;
}

int64_t nrs_trainer_param_len(const nrs_trainer* t, int i) {
  return (t && i >= 0 && i < (int)t->params.size()) ? (int64_t)t->params[i]->len() : -1;
}

int nrs_trainer_set_param(nrs_trainer* t, int i, const float* host) {
  if (!t) return nrs_fail(nullptr, NRS_ERR_ARG, "nrs_trainer_set_param: null handle");
  NRS_REQUIRE(t->ctx, host && i >= 0 && i < (int)t->params.size(), NRS_ERR_ARG, "nrs_trainer_set_param: bad index or null data");
  weights_changed(t);
  int st = nrs_h2d(t->ctx, t->params[i]->data, host, t->params[i]->len() * sizeof(float));
  if (st == NRS_OK) st = nrs_sync(t->ctx);
  return st;
}

int nrs_trainer_get_param(nrs_trainer* t, int i, float* host_out) {
  if (!t) return nrs_fail(nullptr, NRS_ERR_ARG, "nrs_trainer_get_param: null handle");
  NRS_REQUIRE(t->ctx, host_out && i >= 0 && i < (int)t->params.size(), NRS_ERR_ARG, "nrs_trainer_get_param: bad index or null output");
  return nrs_d2h(t->ctx, host_out, t->params[i]->data, t->params[i]->len() * sizeof(float));
}

int nrs_trainer_get_grad(nrs_trainer* t, int i, float* host_out) {
  if (!t) return nrs_fail(nullptr, NRS_ERR_ARG, "nrs_trainer_get_grad: null handle");
  NRS_REQUIRE(t->ctx, host_out && i >= 0 && i < (int)t->params.size(), NRS_ERR_ARG, "nrs_trainer_get_grad: bad index or null output");
  return guarded(t->ctx, [&] {
    auto v = nrs::cuda::read_grad(t->params[i]);
    std::memcpy(host_out, v.data(), v.size() * sizeof(float));
  });
}

int nrs_trainer_forward_backward(nrs_trainer* t, const float* x_host, const float* target_host, int batch, float* loss_out) {
  return host_step(t, x_host, target_host, nullptr, batch, loss_out, false, false);
}

int nrs_trainer_step(nrs_trainer* t, const float* x_host, const float* target_host, int batch, float* loss_out) {
  return host_step(t, x_host, target_host, nullptr, batch, loss_out, true, false);
}

int nrs_trainer_forward_backward_tokens(nrs_trainer* t, const int32_t* ids_host, const int32_t* labels_host, int batch,
                                        float* loss_out) {
  return host_step(t, ids_host, nullptr, labels_host, batch, loss_out, false, true);
}

int nrs_trainer_step_tokens(nrs_trainer* t, const int32_t* ids_host, const int32_t* labels_host, int batch, float* loss_out) {
  return host_step(t, ids_host, nullptr, labels_host, batch, loss_out, true, true);
}

int nrs_trainer_stage_next_tokens(nrs_trainer* t, const int32_t* ids_host, const int32_t* labels_host, int batch) {
  if (!t) return nrs_fail(nullptr, NRS_ERR_ARG, "nrs_trainer_stage_next_tokens: null handle");
  if (!ids_host || !labels_host) return nrs_fail(t->ctx, NRS_ERR_ARG, "nrs_trainer_stage_next_tokens: null input");
  NRS_REQUIRE(t->ctx, t->token_input, NRS_ERR_ARG, "nrs_trainer_stage_next_tokens: this model reads float samples");
  return guarded(t->ctx, [&] { stage_next(t, ids_host, nullptr, labels_host, batch); });
}

int nrs_trainer_step_tokens_device(nrs_trainer* t, const int32_t* ids_dev, const int32_t* labels_dev, int batch, float* loss_out) {
  if (!t) return nrs_fail(nullptr, NRS_ERR_ARG, "nrs_trainer_step_tokens_device: null handle");
  if (!ids_dev || !labels_dev) return nrs_fail(t->ctx, NRS_ERR_ARG, "nrs_trainer_step_tokens_device: null input");
  NRS_REQUIRE(t->ctx, t->token_input, NRS_ERR_ARG, "nrs_trainer_step_tokens_device: this model reads float samples");
  return guarded(t->ctx, [&] {
    StepInput in;
    in.ids = ids_dev;
    in.labels = labels_dev;
    in.batch = batch;
    run_step(t, in, true);
    if (loss_out) read_loss(t, loss_out);
  });
}

int nrs_trainer_stage_next(nrs_trainer* t, const float* x_host, const float* target_host, int batch) {
  if (!t) return nrs_fail(nullptr, NRS_ERR_ARG, "nrs_trainer_stage_next: null handle");
  if (!x_host || !target_host) return nrs_fail(t->ctx, NRS_ERR_ARG, "nrs_trainer_stage_next: null input");
  NRS_REQUIRE(t->ctx, !t->token_input, NRS_ERR_ARG, "nrs_trainer_stage_next: this model reads token ids");
  return guarded(t->ctx, [&] { stage_next(t, x_host, target_host, nullptr, batch); });
}

int nrs_trainer_stage_next_indexed(nrs_trainer* t, const float* x_host, const int32_t* labels_host, int batch) {
  if (!t) return nrs_fail(nullptr, NRS_ERR_ARG, "nrs_trainer_stage_next_indexed: null handle");
  if (!x_host || !labels_host) return nrs_fail(t->ctx, NRS_ERR_ARG, "nrs_trainer_stage_next_indexed: null input");
  NRS_REQUIRE(t->ctx, !t->token_input, NRS_ERR_ARG, "nrs_trainer_stage_next_indexed: this model reads token ids");
  return guarded(t->ctx, [&] { stage_next(t, x_host, nullptr, labels_host, batch); });
}

int nrs_trainer_set_augment(nrs_trainer* t, int max_shift, int flip) {
  if (!t) return nrs_fail(nullptr, NRS_ERR_ARG, "nrs_trainer_set_augment: null handle");
  NRS_REQUIRE(t->ctx, max_shift < 4096, NRS_ERR_ARG, "nrs_trainer_set_augment: bad shift range %d", max_shift);
  NRS_REQUIRE(t->ctx, max_shift < 0 || t->in_shape.size() == 3, NRS_ERR_SHAPE,
              "nrs_trainer_set_augment: augmentation needs [C,H,W] samples");
  t->aug_shift = max_shift;
  t->aug_flip = flip != 0;
  return NRS_OK;
}

int nrs_trainer_step_staged(nrs_trainer* t, float* loss_out) {
  if (!t) return nrs_fail(nullptr, NRS_ERR_ARG, "nrs_trainer_step_staged: null handle");
  return guarded(t->ctx, [&] { step_staged(t, loss_out); });
}

int nrs_trainer_step_staged_lagged(nrs_trainer* t, float* prev_loss_out, int* have_prev) {
  if (!t) return nrs_fail(nullptr, NRS_ERR_ARG, "nrs_trainer_step_staged_lagged: null handle");
  return guarded(t->ctx, [&] { step_staged_lagged(t, prev_loss_out, have_prev); });
}

int nrs_trainer_step_device(nrs_trainer* t, const float* x_dev, const float* target_dev, int batch, float* loss_out) {
  if (!t) return nrs_fail(nullptr, NRS_ERR_ARG, "nrs_trainer_step_device: null handle");
  if (!x_dev || !target_dev) return nrs_fail(t->ctx, NRS_ERR_ARG, "nrs_trainer_step_device: null input");
  NRS_REQUIRE(t->ctx, !t->token_input, NRS_ERR_ARG, "nrs_trainer_step_device: this model reads token ids");
  return guarded(t->ctx, [&] {
    StepInput in;
    in.x = x_dev;
    in.target = target_dev;
    in.batch = batch;
    run_step(t, in, true);
    if (loss_out) read_loss(t, loss_out);
  });
}

int nrs_trainer_last_loss(nrs_trainer* t, float* loss_out) {
  if (!t) return nrs_fail(nullptr, NRS_ERR_ARG, "nrs_trainer_last_loss: null handle");
  NRS_REQUIRE(t->ctx, loss_out != nullptr, NRS_ERR_ARG, "nrs_trainer_last_loss: null output");
  return guarded(t->ctx, [&] { read_loss(t, loss_out); });
}

int nrs_trainer_enable_dp(nrs_trainer* t, int rank, int world, const void* unique_id, int global_batch,
                          size_t bucket_bytes) {
  if (!t) return nrs_fail(nullptr, NRS_ERR_ARG, "nrs_trainer_enable_dp: null handle");
  nrs_ctx* ctx = t->ctx;
  NRS_REQUIRE(ctx, world >= 1 && rank >= 0 && rank < world, NRS_ERR_ARG, "nrs_trainer_enable_dp: rank %d / world %d", rank, world);
  NRS_REQUIRE(ctx, global_batch > 0, NRS_ERR_ARG, "nrs_trainer_enable_dp: global batch must be positive");
  NRS_REQUIRE(ctx, !t->dp, NRS_ERR_ARG, "nrs_trainer_enable_dp: already enabled");
  NRS_REQUIRE(ctx, world == 1 || unique_id != nullptr, NRS_ERR_ARG, "nrs_trainer_enable_dp: null unique id");
  return guarded(ctx, [&] {
    std::unique_ptr<nrs::DpGroup> g(new nrs::DpGroup(ctx, rank, world, unique_id, global_batch, t->dp_timeout_ms));
    if (world > 1) {
      g->register_params(t->params, bucket_bytes);
      // each bucket's parameters are updated right behind its all-reduce, on the comm stream
      g->after_bucket = [t](const nrs::DpBucket& b) {
        t->opt->step_flat_range(b.begin, b.end);
        if (t->ctx->weight_set.owner == t && t->ctx->weight_set.fresh) {
          const nrs::NodeP& last = t->params[b.last_param];
          nrs::check(t->ctx, nrs_weight_set_refresh_range(t->ctx, t->params[b.first_param]->data, last->data + last->len()));
        }
      };
    }
    // the parameters may have moved into the group's flat block: weight planes are rebuilt at the next step
    if (ctx->weight_set.owner == t) nrs_weight_set_clear(ctx);
    t->dp = std::move(g);
    t->rank = rank;
    t->world = world;
    t->global_batch = global_batch;
  });
}

int nrs_trainer_set_sync_batchnorm(nrs_trainer* t, int on) {
  if (!t) return nrs_fail(nullptr, NRS_ERR_ARG, "nrs_trainer_set_sync_batchnorm: null handle");
  t->sync_batchnorm = on != 0;
  return NRS_OK;
}

int nrs_trainer_set_dp_timeout_ms(nrs_trainer* t, double timeout_ms) {
  if (!t) return nrs_fail(nullptr, NRS_ERR_ARG, "nrs_trainer_set_dp_timeout_ms: null handle");
  NRS_REQUIRE(t->ctx, timeout_ms > 0, NRS_ERR_ARG, "nrs_trainer_set_dp_timeout_ms: the deadline must be positive");
  t->dp_timeout_ms = timeout_ms;
  if (t->dp) t->dp->set_timeout_ms(timeout_ms);
  return NRS_OK;
}

}  // extern "C"
