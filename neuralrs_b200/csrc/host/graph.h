// Host-side mirror of the reference's resident-GPU operator API.
//
// The reference is a Rust crate whose GPU path is a set of free functions over
// `Rc<RefCell<Node>>` (src/cuda/{runtime,graph,nn,loss,optim}); the graph engine
// is shared with the CPU path (src/autograd/node.rs:38-151).  No Rust toolchain
// exists in the build image, so this C++ layer plays the role the Rust side
// would: the same Node (data/grad buffers, parents, backward closure,
// requires_grad), the same function names and argument meaning, the same
// backward_graph ordering and += gradient semantics — all on top of the C ABI
// in nrs.h, and itself exported through the node-level C ABI in nrs_graph.h so
// tests can drive it without a compiler.
#pragma once

#include <functional>
#include <memory>
#include <stdexcept>
#include <string>
#include <vector>

#include "nrs.h"

namespace nrs {

struct Error : std::runtime_error {
  int code;
  Error(int c, const std::string& m) : std::runtime_error(m), code(c) {}
};

// Throws nrs::Error carrying nrs_last_error() when a C-ABI call fails.
void check(nrs_ctx* ctx, int status);

struct FlatStore;

// Node of the define-by-run graph (src/autograd/node.rs:38-53).
struct Node {
  nrs_ctx* ctx = nullptr;
  std::vector<size_t> shape;
  std::vector<float> host;          // `data` before to_cuda()
  float* data = nullptr;            // GpuBuffers.data
  float* grad = nullptr;            // GpuBuffers.grad, allocated on first use
  // false: the gradient is logically all-zero and the first writer overwrites
  // the buffer instead of adding to it (the reference zero-fills at creation
  // and always adds; both give the same values).
  bool grad_valid = false;
  bool requires_grad = true;
  bool owns_data = true, owns_grad = true;
  std::shared_ptr<Node> view_of;     // reshape/flatten alias their parent
  std::shared_ptr<FlatStore> flat;   // keeps a flat parameter block alive
  std::vector<std::shared_ptr<Node>> parents;
  std::function<void()> backward_fn;
  std::vector<void*> saved;          // argmax, xhat, ... freed with the node
  // NHWC operand planes of `data` for the tensor-core convolutions, staged once and shared
  // by the forward pass and the weight gradient (registered with the context while alive).
  float* planes_hi = nullptr;
  float* planes_lo = nullptr;
  // For an image tensor (1 or 3 channels) read by a 3x3 layer: its patch planes, shared by that
  // layer's forward pass and weight gradient (registered with the context while alive).
  float* patches_hi = nullptr;
  float* patches_lo = nullptr;
  // Set on the output of a convolution that folded a ReLU into its epilogue.  A max-pool
  // directly above may then hand back a gradient that already carries the ReLU mask
  // (grad_premasked), together with its NHWC planes (gplanes_*, freed with the node).
  bool relu_folded = false, wants_grad_planes = false, grad_premasked = false;
  float* gplanes_hi = nullptr;
  float* gplanes_lo = nullptr;
  // With a premasked gradient: per-block channel sums of it ([rows][channels]), which the
  // convolution's bias gradient folds instead of summing the whole NCHW gradient again.
  float* gchan_partial = nullptr;
  int gchan_rows = 0;

  size_t len() const;
  bool on_gpu() const { return data != nullptr; }
  ~Node();
};
using NodeP = std::shared_ptr<Node>;

// Contiguous home for a model's parameters: one block each for values and
// gradients, so the optimizer is one launch and a gradient all-reduce is one
// call per bucket.  Tensors are padded to 4 floats (16-byte alignment).
struct FlatStore {
  nrs_ctx* ctx = nullptr;
  float* data = nullptr;
  float* grad = nullptr;
  size_t total = 0;                  // floats, padding included
  std::vector<size_t> offset, length;
  ~FlatStore();
};

NodeP node_new(nrs_ctx* ctx, const float* host, const std::vector<size_t>& shape);
// Drops the operand planes cached for a node's data (call after writing `data` in place).
void invalidate_operand_caches(Node* n);

// Building blocks for operators defined outside graph.cu.
struct GradSlot {
  float* ptr;      // where to write the gradient of a parent
  int accumulate;  // 0: overwrite (first writer), 1: add
};
GradSlot grad_slot(const NodeP& n);   // marks the gradient as written
const float* grad_view(Node* n);      // a node's own incoming gradient (zeros if nothing wrote it)
NodeP make_result(nrs_ctx* ctx, const std::vector<size_t>& shape, std::vector<NodeP> parents);

namespace cuda {

// ---- runtime (src/cuda/runtime.rs:39-124)
void to_cuda(const NodeP& n);
std::vector<float> to_host(const NodeP& n);
void set_grad(const NodeP& n, const float* host);
std::vector<float> read_grad(const NodeP& n);
void zero_grad(const std::vector<NodeP>& params);
void synchronize(nrs_ctx* ctx);
// Re-homes resident parameters into one FlatStore (values are preserved).
std::shared_ptr<FlatStore> flatten_params(const std::vector<NodeP>& params);

// ---- graph ops (src/cuda/graph/*.rs)
NodeP matmul(const NodeP& a, const NodeP& b);
NodeP add(const NodeP& a, const NodeP& b);   // same shape, or [r,c] + [c]
NodeP relu(const NodeP& x);
NodeP gelu(const NodeP& x);
NodeP reshape(const NodeP& x, const std::vector<size_t>& shape);
NodeP softmax(const NodeP& x);
NodeP bmm(const NodeP& a, const NodeP& b);
NodeP transpose(const NodeP& x);
NodeP scale(const NodeP& x, float s);
NodeP slice_cols(const NodeP& x, size_t c0, size_t c1);
NodeP concat_cols(const std::vector<NodeP>& parts);

// ---- nn (src/cuda/nn/*.rs)
NodeP conv2d(const NodeP& x, const NodeP& w, const NodeP& b, size_t stride, size_t pad);
NodeP maxpool2d(const NodeP& x, size_t kernel, size_t stride, bool emit_planes = false);   // hint as in conv2d_act
NodeP flatten(const NodeP& x);
NodeP layernorm(const NodeP& x, const NodeP& gamma, const NodeP& beta, float eps);
// layernorm(add(x, residual), ...) as one operator: the sum is never written, and the backward pass
// hands the input gradient to both addends from one kernel.  Same values as the two-operator form.
// emit_planes: see layernorm_impl (graph.cu): only for callers that know the result's readers are tensor-core
// GEMMs and that `residual` has no other reader.
NodeP layernorm_residual(const NodeP& x, const NodeP& residual, const NodeP& gamma, const NodeP& beta, float eps,
                         bool emit_planes = false);
// batchnorm.rs / batchnorm2d.rs: running_mean / running_var are resident nodes updated in place when training
NodeP batchnorm(const NodeP& x, const NodeP& gamma, const NodeP& beta, const NodeP& running_mean,
                const NodeP& running_var, float momentum, float eps, bool training);
NodeP batchnorm2d(const NodeP& x, const NodeP& gamma, const NodeP& beta, const NodeP& running_mean,
                  const NodeP& running_var, float momentum, float eps, bool training);
// either of the two followed by a fused activation (NRS_ACT_NONE / NRS_ACT_RELU); rank 2 or 4 input
NodeP batchnorm_act(const NodeP& x, const NodeP& gamma, const NodeP& beta, const NodeP& running_mean,
                    const NodeP& running_var, float momentum, float eps, bool training, int act);
// dropout.rs / dropout2d.rs: evaluation returns `x` itself; `mask` == nullptr draws the mask on the device
NodeP dropout(const NodeP& x, float p, bool training, const NodeP& mask = nullptr);
NodeP dropout2d(const NodeP& x, float p, bool training, const NodeP& mask = nullptr);
// Fused variants with no counterpart op in the reference: one kernel for
// x@W + b followed by an activation, and conv + bias + activation.  Backward is
// the composition of the unfused backward passes.
NodeP linear_act(const NodeP& x, const NodeP& w, const NodeP& b, int act);
// emit_planes: the caller knows a tensor-core convolution reads the result next, so the kernel
// also writes the result's NHWC operand planes (a hint; ignored where it does not apply).
NodeP conv2d_act(const NodeP& x, const NodeP& w, const NodeP& b, size_t stride, size_t pad, int act,
                 bool emit_planes = false);

// ---- transformer pieces (src/cuda/nn/{embedding,positional,attention,multihead,
//      normalization,linear,transformer_block}.rs), defined in transformer_graph.cu
// scores[..., i, j > i] = -1e30; no reference counterpart (the reference has no mask).
NodeP causal_mask(const NodeP& scores);
// softmax(Q K^T / sqrt(d_head)) V on [batch, seq, d_head]  (attention.rs:23-32).
NodeP attention_batch(const NodeP& q, const NodeP& k, const NodeP& v, bool causal = false);

struct Linear {                       // linear.rs:11-26
  NodeP weights, bias;
  NodeP forward(const NodeP& x) const;
};
struct LayerNorm {                    // normalization.rs (struct form of layernorm())
  NodeP gamma, beta;
  float eps = 1e-5f;
  NodeP forward(const NodeP& x) const;
};
struct Embedding {                    // embedding.rs:41-100
  NodeP weight;
  size_t vocab_size = 0, embedding_dim = 0;
  // indices: `count` token ids; result is [count, dim] (forward) or [batch, seq, dim] (forward_batch,
  // which the reference has on the CPU only: src/nn/embedding.rs:60-113).
  NodeP forward(const int32_t* indices, size_t count) const;
  NodeP forward_batch(const int32_t* indices, size_t batch, size_t seq) const;
  // The batched form on token ids already resident on the device (the caller keeps `idx_dev` alive
  // until the backward pass has run), optionally with PositionalEncoding::forward folded into the
  // gather (pos_table = PositionalEncoding::table).  Ids are range-checked by the kernel.
  NodeP forward_resident(const int32_t* idx_dev, size_t batch, size_t seq, const NodeP& pos_table = nullptr) const;
};
struct PositionalEncoding {           // positional.rs:18-44; the table is computed once and kept resident
  size_t d_model = 0, max_len = 0;
  NodeP table;                        // [max_len, d_model], no gradient
  static PositionalEncoding make(nrs_ctx* ctx, size_t d_model, size_t max_len);
  // x: [seq, d] as in the reference, or [batch, seq, d] (table broadcast over the batch).
  NodeP forward(const NodeP& x) const;
};
struct MultiHeadAttention {           // multihead.rs:57-85; no biases
  NodeP w_q, w_k, w_v, w_o;
  size_t d_model = 0, num_heads = 1;
  bool causal = false;                // extension
  NodeP forward_batch(const NodeP& x) const;
};
struct TransformerBlock {             // transformer_block.rs:28-60: post-LN, ReLU feed-forward
  MultiHeadAttention mha;
  LayerNorm norm1, norm2;
  Linear ff1, ff2;
  size_t d_model = 0, d_ff = 0;
  int act = NRS_ACT_RELU;             // NRS_ACT_GELU is an extension for the LM benchmark configuration
  bool fused_epilogues = false;       // feed-forward bias (+ activation) in the GEMM epilogue instead of separate passes
  NodeP forward(const NodeP& x) const;
  NodeP forward_no_final_norm(const NodeP& x) const;
};

// ---- loss (src/cuda/loss/cross_entropy.rs:74-128)
float cross_entropy(const NodeP& pred, const NodeP& target);
void cross_entropy_backward(const NodeP& pred, const NodeP& target);
// Both at once; the loss stays on the device (read it later with d2h) and the
// mean is taken over `divisor` rows (the global batch under data parallelism).
void cross_entropy_fused(const NodeP& pred, const NodeP& target, float* loss_dev, int divisor);
// The same for targets given as one int32 class index per row (resident on the device): the values
// of the one-hot form without building or reading the dense target tensor.
void cross_entropy_fused_indexed(const NodeP& pred, const int32_t* labels_dev, float* loss_dev, int divisor);

// ---- optim (src/cuda/optim/adamw.rs:43-144)
struct AdamW {
  float lr, beta1, beta2, epsilon, weight_decay;
  size_t t = 0;
  float grad_scale = 1.0f;           // 1/world for averaged all-reduced gradients
  AdamW(nrs_ctx* ctx, float lr, float b1, float b2, float eps, float wd);
  ~AdamW();
  void step(const std::vector<NodeP>& params);
  // The same update in pieces, for parameters that share one FlatStore: begin_flat_step readies the
  // moments, step_flat_range updates floats [begin, end) of the flat block with the current step's
  // bias corrections (every float exactly once per step, in any order, on the context's current
  // stream), end_flat_step advances t.  The data-parallel trainer updates each gradient bucket as
  // soon as its all-reduce has landed.
  void begin_flat_step(const std::vector<NodeP>& params);
  void step_flat_range(size_t begin, size_t end);
  void end_flat_step();
  // (t, all first moments in parameter order, then all second moments).
  std::vector<std::vector<float>> export_state(size_t* t_out) const;
  void import_state(size_t t, const std::vector<std::vector<float>>& moments);

 private:
  nrs_ctx* ctx_;
  std::vector<float*> m_, v_;        // per-parameter views
  std::vector<size_t> len_;
  float* flat_m_ = nullptr;          // set when the parameters share a FlatStore
  float* flat_v_ = nullptr;
  size_t flat_total_ = 0;
  bool owns_each_ = false;
  std::shared_ptr<FlatStore> stepping_;   // set between begin_flat_step and end_flat_step
  void ensure_state(const std::vector<NodeP>& params);
  void release();
};

}  // namespace cuda

// Topological backward pass (src/autograd/node.rs:113-151).
void backward_graph(const NodeP& root);

}  // namespace nrs
