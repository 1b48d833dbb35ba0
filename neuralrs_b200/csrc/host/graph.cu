// Define-by-run graph over the C ABI: Node, the resident operators with their
// backward closures, backward_graph and AdamW.  See graph.h for what it mirrors.
#include "host/graph.h"
#include "nrs_internal.h"
#include "tc_mainloop.cuh"

#include <cmath>
#include <cstring>
#include <unordered_set>

namespace nrs {

void check(nrs_ctx* ctx, int status) {
  if (status != NRS_OK) throw Error(status, nrs_last_error(ctx));
}

static void fail(int code, const std::string& msg) { throw Error(code, msg); }

static float* dalloc(nrs_ctx* ctx, size_t floats, bool zero = false) {
  void* p = nullptr;
  check(ctx, nrs_alloc(ctx, floats * sizeof(float), zero ? 1 : 0, &p));
  return (float*)p;
}

size_t Node::len() const {
  size_t n = 1;
  for (size_t d : shape) n *= d;
  return n;
}

Node::~Node() {
  if (!ctx) return;
  if (planes_hi) {
    ctx->plane_hints.erase(data);
    nrs_free(ctx, planes_hi);
    if (planes_lo) nrs_free(ctx, planes_lo);
  }
  if (patches_hi) {
    ctx->patch_hints.erase(data);
    nrs_free(ctx, patches_hi);
    if (patches_lo) nrs_free(ctx, patches_lo);
  }
  if (gplanes_hi) {
    ctx->plane_hints.erase(grad);
    nrs_free(ctx, gplanes_hi);
    if (gplanes_lo) nrs_free(ctx, gplanes_lo);
  }
  if (gchan_partial) nrs_free(ctx, gchan_partial);
  if (data && owns_data) nrs_free(ctx, data);
  if (grad && owns_grad) nrs_free(ctx, grad);
  for (void* p : saved) nrs_free(ctx, p);
}

FlatStore::~FlatStore() {
  if (!ctx) return;
  if (data) nrs_free(ctx, data);
  if (grad) nrs_free(ctx, grad);
}

// Operand planes and patch planes are functions of the tensor's contents: whoever rewrites `data`
// in place drops them (and the context's hints), so the next convolution stages fresh ones.
void invalidate_operand_caches(Node* n) {
  nrs_ctx* ctx = n->ctx;
  if (!ctx) return;
  if (n->planes_hi) {
    ctx->plane_hints.erase(n->data);
    nrs_free(ctx, n->planes_hi);
    if (n->planes_lo) nrs_free(ctx, n->planes_lo);
    n->planes_hi = n->planes_lo = nullptr;
  }
  if (n->patches_hi) {
    ctx->patch_hints.erase(n->data);
    nrs_free(ctx, n->patches_hi);
    if (n->patches_lo) nrs_free(ctx, n->patches_lo);
    n->patches_hi = n->patches_lo = nullptr;
  }
}

NodeP node_new(nrs_ctx* ctx, const float* host, const std::vector<size_t>& shape) {
  if (!ctx) fail(NRS_ERR_ARG, "Node::new: null context");
  auto n = std::make_shared<Node>();
  n->ctx = ctx;
  n->shape = shape;
  if (host) n->host.assign(host, host + n->len());
  return n;
}

// The node whose gradient buffer `n` uses (reshape/flatten results alias their input).
static Node* grad_root(Node* n) {
  while (n->view_of) n = n->view_of.get();
  return n;
}

struct GradTarget {
  float* ptr;
  int accumulate;
};
// Where a backward pass writes the gradient of `n`, and whether it must add.
static GradTarget grad_target(const NodeP& n) {
  Node* r = grad_root(n.get());
  if (!r->grad) r->grad = dalloc(r->ctx, r->len());
  if (r->grad_premasked) {
    // A second consumer adds an unmasked share: drop the claim (and the now stale planes); the
    // ReLU mask is a 0/1 factor, so masking the sum later leaves the first share unchanged.
    r->grad_premasked = false;
    if (r->gplanes_hi) { nrs_free(r->ctx, r->gplanes_hi); r->gplanes_hi = nullptr; }
    if (r->gplanes_lo) { nrs_free(r->ctx, r->gplanes_lo); r->gplanes_lo = nullptr; }
    if (r->gchan_partial) { nrs_free(r->ctx, r->gchan_partial); r->gchan_partial = nullptr; r->gchan_rows = 0; }
  }
  GradTarget t{r->grad, r->grad_valid ? 1 : 0};
  r->grad_valid = true;
  return t;
}
// The gradient a node's own backward pass reads (zeros if nothing wrote it).
static const float* grad_in(Node* n) {
  Node* r = grad_root(n);
  if (!r->grad) r->grad = dalloc(r->ctx, r->len());
  if (!r->grad_valid) {
    check(r->ctx, nrs_memset_zero(r->ctx, r->grad, r->len() * sizeof(float)));
    r->grad_valid = true;
  }
  return r->grad;
}

static void require_gpu(const NodeP& n, const char* what) {
  if (!n) fail(NRS_ERR_ARG, std::string(what) + ": null node");
  if (!n->on_gpu()) fail(NRS_ERR_ARG, std::string(what) + ": not on GPU");
}

static NodeP make_out(nrs_ctx* ctx, const std::vector<size_t>& shape, std::vector<NodeP> parents) {
  auto out = std::make_shared<Node>();
  out->ctx = ctx;
  out->shape = shape;
  out->data = dalloc(ctx, out->len());
  out->parents = std::move(parents);
  return out;
}

// Public faces of the helpers above, for operator files outside this one.
GradSlot grad_slot(const NodeP& n) {
  GradTarget t = grad_target(n);
  return GradSlot{t.ptr, t.accumulate};
}
const float* grad_view(Node* n) { return grad_in(n); }
NodeP make_result(nrs_ctx* ctx, const std::vector<size_t>& shape, std::vector<NodeP> parents) {
  return make_out(ctx, shape, std::move(parents));
}

// Stages NHWC planes of an NCHW tensor [n,c,h,w] at `src` into fresh pool blocks and registers
// them with the context under `src`.  Returns false (nothing allocated) when the tensor-core
// convolutions would not take this tensor (FP32 mode, channel count not a multiple of 32).
static bool stage_planes(nrs_ctx* ctx, const float* src, const std::vector<size_t>& shape, float** hi, float** lo) {
  *hi = *lo = nullptr;
  if (ctx->math_mode == NRS_MATH_FP32 || shape.size() != 4 || shape[1] % 32 != 0 || shape[0] == 0) return false;
  if (!tc::tensor_map_encoder()) return false;
  if (ctx->plane_hints.count(src)) return false;   // already there (the tensor feeds two convolutions)
  const bool split = ctx->math_mode == NRS_MATH_3XTF32;
  const size_t n = shape[0], c = shape[1], hw = shape[2] * shape[3];
  *hi = dalloc(ctx, n * c * hw);
  if (split) *lo = dalloc(ctx, n * c * hw);
  check(ctx, nrs_tc_stage(ctx, src, *hi, *lo, (int)hw, (int)c, (int)c, (int)n, c * hw, c * hw, true));
  ctx->plane_hints[src] = NrsPlanes{*hi, *lo, split ? 1 : 0};
  return true;
}

// Row planes of a 2-D tensor [rows][cols] (cols a multiple of 32) for the tensor-core GEMMs: the layout
// is the tensor's own, so the same planes serve it as the A operand of x@W and, read along the rows, as
// an operand of the weight gradient x^T dz.  Stages them into fresh pool blocks and registers them with
// the context under `src`; false (nothing allocated) when a tensor-core GEMM would not read them.
static bool stage_planes_2d(nrs_ctx* ctx, const float* src, size_t rows, size_t cols, float** hi, float** lo) {
  *hi = *lo = nullptr;
  if (ctx->math_mode == NRS_MATH_FP32 || cols % 32 != 0 || rows == 0 || rows > 2147483647u || cols > 2147483647u) return false;
  if (!tc::tensor_map_encoder() || ctx->plane_hints.count(src)) return false;
  const bool split = ctx->math_mode == NRS_MATH_3XTF32;
  *hi = dalloc(ctx, rows * cols);
  if (split) *lo = dalloc(ctx, rows * cols);
  check(ctx, nrs_tc_stage(ctx, src, *hi, *lo, (int)rows, (int)cols, (int)cols, 1, 0, 0, false));
  NrsPlanes pl{*hi, *lo, split ? 1 : 0};
  pl.rows = (int)rows;
  pl.cols = (int)cols;
  ctx->plane_hints[src] = pl;
  return true;
}

// Planes of a backward pass's incoming gradient, staged once for the two products that read it
// (dX = dz W^T and dW = x^T dz) and dropped when the scope ends.
struct GradPlanes {
  nrs_ctx* ctx;
  const float* key = nullptr;
  float *hi = nullptr, *lo = nullptr;
  GradPlanes(nrs_ctx* c, const float* dz, size_t rows, size_t cols, bool wanted) : ctx(c) {
    if (wanted && stage_planes_2d(c, dz, rows, cols, &hi, &lo)) key = dz;
  }
  ~GradPlanes() {
    if (!key) return;
    ctx->plane_hints.erase(key);
    nrs_free(ctx, hi);
    if (lo) nrs_free(ctx, lo);
  }
};

// The forward operand's planes live with its node (both products that read x find them there).
static void cache_planes_2d(const NodeP& x, size_t rows, size_t cols) {
  if (x->planes_hi) return;
  float *hi = nullptr, *lo = nullptr;
  if (stage_planes_2d(x->ctx, x->data, rows, cols, &hi, &lo)) {
    x->planes_hi = hi;
    x->planes_lo = lo;
  }
}

static bool planes_possible(nrs_ctx* ctx) {
  return ctx->math_mode != NRS_MATH_FP32 && tc::tensor_map_encoder();
}

namespace cuda {

// ------------------------------------------------------------------ runtime

void to_cuda(const NodeP& n) {
  if (!n) fail(NRS_ERR_ARG, "to_cuda: null node");
  if (n->host.size() != n->len()) fail(NRS_ERR_SHAPE, "to_cuda: host data does not match the shape");
  if (!n->data) n->data = dalloc(n->ctx, n->len());
  invalidate_operand_caches(n.get());   // planes staged from the previous contents are stale
  check(n->ctx, nrs_h2d(n->ctx, n->data, n->host.data(), n->len() * sizeof(float)));
  // The copy is asynchronous and n->host stays alive with the node.
  Node* r = grad_root(n.get());
  r->grad_valid = false;
}

std::vector<float> to_host(const NodeP& n) {
  require_gpu(n, "to_host: node");
  std::vector<float> out(n->len());
  check(n->ctx, nrs_d2h(n->ctx, out.data(), n->data, out.size() * sizeof(float)));
  return out;
}

void set_grad(const NodeP& n, const float* host) {
  require_gpu(n, "set_grad: node");
  Node* r = grad_root(n.get());
  if (!r->grad) r->grad = dalloc(r->ctx, r->len());
  check(n->ctx, nrs_h2d(n->ctx, r->grad, host, r->len() * sizeof(float)));
  check(n->ctx, nrs_sync(n->ctx));  // the caller's buffer may go away
  r->grad_valid = true;
}

std::vector<float> read_grad(const NodeP& n) {
  require_gpu(n, "read_grad: node");
  Node* r = grad_root(n.get());
  std::vector<float> out(r->len(), 0.0f);
  if (r->grad && r->grad_valid) check(n->ctx, nrs_d2h(n->ctx, out.data(), r->grad, out.size() * sizeof(float)));
  return out;
}

void zero_grad(const std::vector<NodeP>& params) {
  for (const auto& p : params) {
    require_gpu(p, "zero_grad: node");
    grad_root(p.get())->grad_valid = false;  // the next writer overwrites
  }
}

void synchronize(nrs_ctx* ctx) { check(ctx, nrs_sync(ctx)); }

std::shared_ptr<FlatStore> flatten_params(const std::vector<NodeP>& params) {
  if (params.empty()) fail(NRS_ERR_ARG, "flatten_params: no parameters");
  nrs_ctx* ctx = params[0]->ctx;
  auto fs = std::make_shared<FlatStore>();
  fs->ctx = ctx;
  size_t total = 0;
  for (const auto& p : params) {
    require_gpu(p, "flatten_params: parameter");
    if (p->view_of) fail(NRS_ERR_ARG, "flatten_params: a parameter is a view");
    fs->offset.push_back(total);
    fs->length.push_back(p->len());
    total += (p->len() + 3) / 4 * 4;
  }
  fs->total = total;
  fs->data = dalloc(ctx, total, true);
  fs->grad = dalloc(ctx, total, true);
  for (size_t i = 0; i < params.size(); ++i) {
    Node* p = params[i].get();
    check(ctx, nrs_d2d(ctx, fs->data + fs->offset[i], p->data, p->len() * sizeof(float)));
    if (p->grad && p->grad_valid)
      check(ctx, nrs_d2d(ctx, fs->grad + fs->offset[i], p->grad, p->len() * sizeof(float)));
    if (p->owns_data) nrs_free(ctx, p->data);
    if (p->grad && p->owns_grad) nrs_free(ctx, p->grad);
    p->data = fs->data + fs->offset[i];
    p->grad = fs->grad + fs->offset[i];
    p->owns_data = p->owns_grad = false;
    p->grad_valid = true;  // zero-filled (or copied) above
    p->flat = fs;
  }
  return fs;
}

// ---------------------------------------------------------------- graph ops

NodeP matmul(const NodeP& a, const NodeP& b) {
  require_gpu(a, "cuda matmul: lhs");
  require_gpu(b, "cuda matmul: rhs");
  if (a->shape.size() != 2 || b->shape.size() != 2) fail(NRS_ERR_SHAPE, "cuda matmul: operands must be 2-D");
  const int m = (int)a->shape[0], k = (int)a->shape[1], n = (int)b->shape[1];
  if (b->shape[0] != a->shape[1]) fail(NRS_ERR_SHAPE, "cuda matmul: inner dims mismatch");
  nrs_ctx* ctx = a->ctx;
  NodeP out = make_out(ctx, {(size_t)m, (size_t)n}, {a, b});
  const bool tensor_cores = nrs_gemm_on_tensor_cores(ctx, m, n, k);
  if (tensor_cores && b->requires_grad) cache_planes_2d(a, (size_t)m, (size_t)k);   // read again by dB = A^T dC
  check(ctx, nrs_gemm(ctx, 0, 0, m, n, k, a->data, b->data, out->data, nullptr, NRS_ACT_NONE, 0.0f));
  Node* self = out.get();
  out->backward_fn = [self, a, b, m, k, n, tensor_cores]() {
    nrs_ctx* ctx = self->ctx;
    const float* dc = grad_in(self);
    GradPlanes dc_planes(ctx, dc, (size_t)m, (size_t)n, tensor_cores && a->requires_grad && b->requires_grad);
    if (a->requires_grad) {
      GradTarget t = grad_target(a);  // dA (+)= dC . B^T
      check(ctx, nrs_gemm(ctx, 0, 1, m, k, n, dc, b->data, t.ptr, nullptr, NRS_ACT_NONE, t.accumulate ? 1.0f : 0.0f));
    }
    if (b->requires_grad) {
      GradTarget t = grad_target(b);  // dB (+)= A^T . dC: reads nothing dA wrote, so it may start under dA's tail
      NrsIndependentNext overlap(ctx, a->requires_grad);
      check(ctx, nrs_gemm(ctx, 1, 0, k, n, m, a->data, dc, t.ptr, nullptr, NRS_ACT_NONE, t.accumulate ? 1.0f : 0.0f));
    }
  };
  return out;
}

// dst (+)= src, n floats.
static void pass_grad(nrs_ctx* ctx, const NodeP& parent, const float* g, size_t n) {
  if (!parent->requires_grad) return;
  GradTarget t = grad_target(parent);
  if (t.accumulate) check(ctx, nrs_accumulate(ctx, t.ptr, g, n));
  else check(ctx, nrs_d2d(ctx, t.ptr, g, n * sizeof(float)));
}

NodeP add(const NodeP& a, const NodeP& b) {
  require_gpu(a, "cuda add: lhs");
  require_gpu(b, "cuda add: rhs");
  nrs_ctx* ctx = a->ctx;
  const bool broadcast = a->shape.size() == 2 && b->shape.size() == 1 && a->shape[1] == b->shape[0];
  if (!broadcast && a->len() != b->len()) fail(NRS_ERR_SHAPE, "cuda add: shapes differ and are not [r,c]+[c]");
  NodeP out = make_out(ctx, a->shape, {a, b});
  const size_t len = a->len();
  if (broadcast)
    check(ctx, nrs_bias_add(ctx, a->data, b->data, out->data, (int)a->shape[0], (int)a->shape[1]));
  else
    check(ctx, nrs_add(ctx, a->data, b->data, out->data, len));
  Node* self = out.get();
  out->backward_fn = [self, a, b, broadcast, len]() {
    nrs_ctx* ctx = self->ctx;
    const float* g = grad_in(self);
    pass_grad(ctx, a, g, len);
    if (broadcast) {
      if (b->requires_grad) {
        GradTarget t = grad_target(b);
        check(ctx, nrs_sum_axis0(ctx, g, t.ptr, (int)a->shape[0], (int)a->shape[1], t.accumulate));
      }
    } else {
      pass_grad(ctx, b, g, len);
    }
  };
  return out;
}

NodeP relu(const NodeP& x) {
  require_gpu(x, "cuda relu: input");
  nrs_ctx* ctx = x->ctx;
  NodeP out = make_out(ctx, x->shape, {x});
  const size_t len = x->len();
  check(ctx, nrs_relu_fwd(ctx, x->data, out->data, len));
  Node* self = out.get();
  out->backward_fn = [self, x, len]() {
    if (!x->requires_grad) return;
    const float* g = grad_in(self);
    GradTarget t = grad_target(x);
    check(self->ctx, nrs_relu_bwd(self->ctx, x->data, g, t.ptr, len, t.accumulate));
  };
  return out;
}

NodeP gelu(const NodeP& x) {
  require_gpu(x, "cuda gelu: input");
  nrs_ctx* ctx = x->ctx;
  NodeP out = make_out(ctx, x->shape, {x});
  const size_t len = x->len();
  check(ctx, nrs_gelu_fwd(ctx, x->data, out->data, len));
  Node* self = out.get();
  out->backward_fn = [self, x, len]() {
    if (!x->requires_grad) return;
    const float* g = grad_in(self);
    GradTarget t = grad_target(x);
    check(self->ctx, nrs_gelu_bwd(self->ctx, x->data, g, t.ptr, len, t.accumulate));
  };
  return out;
}

// The reference copies on reshape and adds the gradient back
// (src/cuda/graph/reshape.rs:31-72).  Here the result aliases the input's data
// and gradient buffers: same values, no kernels.
NodeP reshape(const NodeP& x, const std::vector<size_t>& shape) {
  require_gpu(x, "cuda reshape: input");
  size_t n = 1;
  for (size_t d : shape) n *= d;
  if (n != x->len()) fail(NRS_ERR_SHAPE, "cuda reshape: element count mismatched");
  auto out = std::make_shared<Node>();
  out->ctx = x->ctx;
  out->shape = shape;
  out->data = x->data;
  out->owns_data = false;
  out->view_of = x;
  out->parents = {x};
  out->requires_grad = x->requires_grad;
  return out;
}

NodeP softmax(const NodeP& x) {
  require_gpu(x, "cuda softmax: input");
  if (x->shape.empty()) fail(NRS_ERR_SHAPE, "cuda softmax: scalar input");
  nrs_ctx* ctx = x->ctx;
  const int width = (int)x->shape.back();
  const int rows = (int)(x->len() / (size_t)width);
  NodeP out = make_out(ctx, x->shape, {x});
  check(ctx, nrs_softmax_fwd(ctx, x->data, out->data, rows, width));
  Node* self = out.get();
  out->backward_fn = [self, x, rows, width]() {
    if (!x->requires_grad) return;
    const float* g = grad_in(self);
    GradTarget t = grad_target(x);
    check(self->ctx, nrs_softmax_bwd(self->ctx, self->data, g, t.ptr, rows, width, t.accumulate));
  };
  return out;
}

NodeP bmm(const NodeP& a, const NodeP& b) {
  require_gpu(a, "cuda bmm: lhs");
  require_gpu(b, "cuda bmm: rhs");
  if (a->shape.size() != 3 || b->shape.size() != 3) fail(NRS_ERR_SHAPE, "cuda bmm: operands must be 3-D");
  if (a->shape[0] != b->shape[0] || a->shape[2] != b->shape[1]) fail(NRS_ERR_SHAPE, "cuda bmm: shape mismatch");
  nrs_ctx* ctx = a->ctx;
  const int batch = (int)a->shape[0], m = (int)a->shape[1], k = (int)a->shape[2], n = (int)b->shape[2];
  NodeP out = make_out(ctx, {(size_t)batch, (size_t)m, (size_t)n}, {a, b});
  check(ctx, nrs_bmm(ctx, 0, 0, batch, m, n, k, a->data, b->data, out->data, 0.0f));
  Node* self = out.get();
  out->backward_fn = [self, a, b, batch, m, k, n]() {
    nrs_ctx* ctx = self->ctx;
    const float* dc = grad_in(self);
    if (a->requires_grad) {
      GradTarget t = grad_target(a);
      check(ctx, nrs_bmm(ctx, 0, 1, batch, m, k, n, dc, b->data, t.ptr, t.accumulate ? 1.0f : 0.0f));
    }
    if (b->requires_grad) {
      GradTarget t = grad_target(b);
      check(ctx, nrs_bmm(ctx, 1, 0, batch, k, n, m, a->data, dc, t.ptr, t.accumulate ? 1.0f : 0.0f));
    }
  };
  return out;
}

NodeP transpose(const NodeP& x) {
  require_gpu(x, "cuda transpose: input");
  if (x->shape.size() < 2) fail(NRS_ERR_SHAPE, "cuda transpose: needs at least 2 dims");
  nrs_ctx* ctx = x->ctx;
  const size_t nd = x->shape.size();
  const int rows = (int)x->shape[nd - 2], cols = (int)x->shape[nd - 1];
  const int batch = (int)(x->len() / ((size_t)rows * cols));
  std::vector<size_t> os = x->shape;
  os[nd - 2] = cols;
  os[nd - 1] = rows;
  NodeP out = make_out(ctx, os, {x});
  check(ctx, nrs_transpose(ctx, x->data, out->data, batch, rows, cols, 0));
  Node* self = out.get();
  out->backward_fn = [self, x, batch, rows, cols]() {
    if (!x->requires_grad) return;
    const float* g = grad_in(self);
    GradTarget t = grad_target(x);
    check(self->ctx, nrs_transpose(self->ctx, g, t.ptr, batch, cols, rows, t.accumulate));
  };
  return out;
}

NodeP scale(const NodeP& x, float s) {
  require_gpu(x, "cuda scale: input");
  nrs_ctx* ctx = x->ctx;
  NodeP out = make_out(ctx, x->shape, {x});
  const size_t len = x->len();
  check(ctx, nrs_scale(ctx, x->data, out->data, len, s, 0));
  Node* self = out.get();
  out->backward_fn = [self, x, len, s]() {
    if (!x->requires_grad) return;
    const float* g = grad_in(self);
    GradTarget t = grad_target(x);
    check(self->ctx, nrs_scale(self->ctx, g, t.ptr, len, s, t.accumulate));
  };
  return out;
}

NodeP slice_cols(const NodeP& x, size_t c0, size_t c1) {
  require_gpu(x, "cuda slice_cols: input");
  if (x->shape.empty()) fail(NRS_ERR_SHAPE, "cuda slice_cols: scalar input");
  const size_t total = x->shape.back();
  if (c0 > c1 || c1 > total) fail(NRS_ERR_SHAPE, "cuda slice_cols: range outside the last dim");
  nrs_ctx* ctx = x->ctx;
  const int rows = (int)(x->len() / total);
  std::vector<size_t> os = x->shape;
  os.back() = c1 - c0;
  NodeP out = make_out(ctx, os, {x});
  check(ctx, nrs_slice_cols_fwd(ctx, x->data, out->data, rows, (int)total, (int)c0, (int)c1));
  Node* self = out.get();
  out->backward_fn = [self, x, rows, total, c0, c1]() {
    if (!x->requires_grad) return;
    const float* g = grad_in(self);
    Node* r = grad_root(x.get());
    // Only a column band is written: the rest of a fresh gradient must read as zero.
    if (!r->grad_valid) (void)grad_in(x.get());
    GradTarget t = grad_target(x);
    check(self->ctx, nrs_slice_cols_bwd(self->ctx, g, t.ptr, rows, (int)total, (int)c0, (int)c1, 1));
  };
  return out;
}

NodeP concat_cols(const std::vector<NodeP>& parts) {
  if (parts.empty()) fail(NRS_ERR_ARG, "cuda concat_cols: no parts");
  for (const auto& p : parts) require_gpu(p, "cuda concat_cols: part");
  nrs_ctx* ctx = parts[0]->ctx;
  std::vector<int> widths;
  size_t total = 0;
  const size_t rows = parts[0]->len() / parts[0]->shape.back();
  for (const auto& p : parts) {
    if (p->len() / p->shape.back() != rows) fail(NRS_ERR_SHAPE, "cuda concat_cols: row counts differ");
    widths.push_back((int)p->shape.back());
    total += p->shape.back();
  }
  std::vector<size_t> os = parts[0]->shape;
  os.back() = total;
  NodeP out = make_out(ctx, os, parts);
  int off = 0;
  for (size_t i = 0; i < parts.size(); ++i) {
    check(ctx, nrs_concat_write(ctx, parts[i]->data, out->data, (int)rows, (int)total, off, widths[i]));
    off += widths[i];
  }
  Node* self = out.get();
  out->backward_fn = [self, parts, widths, rows, total]() {
    const float* g = grad_in(self);
    int off = 0;
    for (size_t i = 0; i < parts.size(); ++i) {
      if (parts[i]->requires_grad) {
        GradTarget t = grad_target(parts[i]);
        check(self->ctx, nrs_concat_read(self->ctx, g, t.ptr, (int)rows, (int)total, off, widths[i], t.accumulate));
      }
      off += widths[i];
    }
  };
  return out;
}

// ----------------------------------------------------------------------- nn

static void conv_backward(Node* self, const NodeP& x, const NodeP& w, const NodeP& b, const float* dy, int n,
                          int ci, int h, int wd, int co, int kh, int kw, int stride, int pad) {
  nrs_ctx* ctx = self->ctx;
  // Each output may be in a different accumulate state, so issue them separately.
  if (x->requires_grad) {
    // x is the output of a convolution with a folded ReLU and this is the first share of its
    // gradient: the data-gradient kernel can apply that ReLU's mask and emit the NHWC planes the
    // producer's own backward pass wants, instead of a separate mask-and-stage pass later.
    Node* xr = x.get();
    const bool fold = xr->relu_folded && !xr->view_of && !xr->grad_valid && !xr->grad_premasked && !xr->gplanes_hi &&
                      planes_possible(ctx);
    GradTarget t = grad_target(x);
    float *ghi = nullptr, *glo = nullptr;
    if (fold) {
      if (xr->wants_grad_planes) {
        ghi = dalloc(ctx, xr->len());
        if (ctx->math_mode == NRS_MATH_3XTF32) glo = dalloc(ctx, xr->len());
      }
      ctx->out_extras[t.ptr] = NrsOutExtras{xr->data, ghi, glo};
      // ... and per-tile channel sums of the masked gradient, for the producer's bias gradient.
      const size_t pixels = (size_t)n * h * wd;
      const int cap = (int)(4 * (pixels / 64 + 2));
      ctx->colsum_requests[t.ptr] = NrsColsumRequest{dalloc(ctx, (size_t)cap * ci), cap, 0};
    }
    try {
      check(ctx, nrs_conv2d_bwd(ctx, x->data, w->data, dy, t.ptr, nullptr, nullptr, n, ci, h, wd, co, kh, kw, stride,
                                pad, t.accumulate));
    } catch (...) {
      // the requests are keyed by a pool address that will be handed out again: never leave them behind
      if (fold) {
        auto it = ctx->colsum_requests.find(t.ptr);
        if (it != ctx->colsum_requests.end()) { nrs_free(ctx, it->second.partial); ctx->colsum_requests.erase(it); }
        ctx->out_extras.erase(t.ptr);
        if (ghi) nrs_free(ctx, ghi);
        if (glo) nrs_free(ctx, glo);
      }
      throw;
    }
    if (fold) {
      NrsColsumRequest sums = ctx->colsum_requests[t.ptr];
      ctx->colsum_requests.erase(t.ptr);
      if (ctx->out_extras.erase(t.ptr)) {   // not honoured (the kernel that ran does not fold)
        if (ghi) nrs_free(ctx, ghi);
        if (glo) nrs_free(ctx, glo);
        sums.rows = 0;
      } else {
        xr->gplanes_hi = ghi;
        xr->gplanes_lo = glo;
        xr->grad_premasked = true;
      }
      if (sums.rows > 0) {
        xr->gchan_partial = sums.partial;
        xr->gchan_rows = sums.rows;
      } else {
        nrs_free(ctx, sums.partial);
      }
    }
  }
  if (w->requires_grad) {   // reads nothing the data gradient wrote: it may start under that kernel's tail
    GradTarget t = grad_target(w);
    NrsIndependentNext overlap(ctx, x->requires_grad);
    check(ctx, nrs_conv2d_bwd(ctx, x->data, w->data, dy, nullptr, t.ptr, nullptr, n, ci, h, wd, co, kh, kw, stride,
                              pad, t.accumulate));
  }
  if (b->requires_grad) {
    GradTarget t = grad_target(b);
    if (self->grad_premasked && self->gchan_partial && self->gchan_rows > 0)   // the producer of dy left channel sums
      check(ctx, nrs_sum_axis0(ctx, self->gchan_partial, t.ptr, self->gchan_rows, co, t.accumulate));
    else
      check(ctx, nrs_conv2d_bwd(ctx, x->data, w->data, dy, nullptr, nullptr, t.ptr, n, ci, h, wd, co, kh, kw, stride,
                                pad, t.accumulate));
  }
}

NodeP conv2d_act(const NodeP& x, const NodeP& w, const NodeP& b, size_t stride, size_t pad, int act, bool emit_planes) {
  require_gpu(x, "cuda conv2d: input");
  require_gpu(w, "cuda conv2d: weight");
  require_gpu(b, "cuda conv2d: bias");
  if (x->shape.size() != 4 || w->shape.size() != 4) fail(NRS_ERR_SHAPE, "cuda conv2d: input and weight must be 4-D");
  if (w->shape[1] != x->shape[1]) fail(NRS_ERR_SHAPE, "cuda conv2d: channel mismatch");
  if (b->len() != w->shape[0]) fail(NRS_ERR_SHAPE, "cuda conv2d: bias length mismatch");
  if (act != NRS_ACT_NONE && act != NRS_ACT_RELU) fail(NRS_ERR_UNSUPPORTED, "cuda conv2d: only ReLU can be fused");
  if (stride == 0) fail(NRS_ERR_SHAPE, "cuda conv2d: stride 0");
  nrs_ctx* ctx = x->ctx;
  const int n = (int)x->shape[0], ci = (int)x->shape[1], h = (int)x->shape[2], wd = (int)x->shape[3];
  const int co = (int)w->shape[0], kh = (int)w->shape[2], kw = (int)w->shape[3];
  if (h + 2 * (int)pad < kh || wd + 2 * (int)pad < kw) fail(NRS_ERR_SHAPE, "cuda conv2d: kernel larger than padded input");
  const int oh = (h + 2 * (int)pad - kh) / (int)stride + 1, ow = (wd + 2 * (int)pad - kw) / (int)stride + 1;
  NodeP out = make_out(ctx, {(size_t)n, (size_t)co, (size_t)oh, (size_t)ow}, {x, w, b});
  // The input's NHWC planes serve this forward pass and, later, the weight gradient.
  if (stride == 1 && !x->planes_hi && co % 32 == 0 && w->requires_grad) {
    float *phi = nullptr, *plo = nullptr;
    if (stage_planes(ctx, x->data, x->shape, &phi, &plo)) { x->planes_hi = phi; x->planes_lo = plo; }
  }
  // Image layer in a TF32 mode: forward and weight gradient both run on the tensor cores over the
  // input's patch planes; make them once.
  if ((ci == 1 || ci == 3) && kh == 3 && kw == 3 && stride == 1 && co % 32 == 0 && !x->patches_hi && planes_possible(ctx) &&
      (size_t)n * oh * ow >= 4096 && !ctx->patch_hints.count(x->data)) {
    const size_t floats = (size_t)n * oh * ow * 32;
    float* phi = dalloc(ctx, floats);
    float* plo = ctx->math_mode == NRS_MATH_3XTF32 ? dalloc(ctx, floats) : nullptr;
    const int st = nrs_smallc_patch_planes(ctx, x->data, phi, plo, n, ci, h, wd, (int)pad);
    if (st == NRS_OK) {
      x->patches_hi = phi;
      x->patches_lo = plo;
      ctx->patch_hints[x->data] = NrsPlanes{phi, plo, (plo ? 1 : 0) | ((int)pad << 8)};
    } else {
      nrs_free(ctx, phi);
      if (plo) nrs_free(ctx, plo);
      if (st != NRS_ERR_UNSUPPORTED) check(ctx, st);
    }
  }
  // The caller knows a tensor-core convolution consumes this output: let the kernel write the
  // output's NHWC planes itself (otherwise the consumer stages them in a pass of its own).
  float *ohi = nullptr, *olo = nullptr;
  if (emit_planes && co % 32 == 0 && planes_possible(ctx)) {
    ohi = dalloc(ctx, out->len());
    if (ctx->math_mode == NRS_MATH_3XTF32) olo = dalloc(ctx, out->len());
    ctx->out_extras[out->data] = NrsOutExtras{nullptr, ohi, olo};
  }
  try {
    check(ctx, nrs_conv2d_fwd(ctx, x->data, w->data, b->data, out->data, n, ci, h, wd, co, kh, kw, (int)stride,
                              (int)pad, act));
  } catch (...) {
    if (ohi) {
      ctx->out_extras.erase(out->data);
      nrs_free(ctx, ohi);
      if (olo) nrs_free(ctx, olo);
    }
    throw;
  }
  if (ohi) {
    if (ctx->out_extras.erase(out->data)) {   // not honoured
      nrs_free(ctx, ohi);
      if (olo) nrs_free(ctx, olo);
    } else {
      out->planes_hi = ohi;
      out->planes_lo = olo;
      ctx->plane_hints[out->data] = NrsPlanes{ohi, olo, olo ? 1 : 0};
    }
  }
  Node* self = out.get();
  const int s = (int)stride, p = (int)pad;
  out->relu_folded = act == NRS_ACT_RELU;
  // (an image layer with 1 or 3 input channels takes dy planes too: its weight gradient runs on the
  // tensor cores over patch planes)
  const bool image_layer = (ci == 1 || ci == 3) && kh == 3 && kw == 3;
  out->wants_grad_planes = act == NRS_ACT_RELU && s == 1 && (ci % 32 == 0 || image_layer) && co % 32 == 0;
  out->backward_fn = [self, x, w, b, n, ci, h, wd, co, kh, kw, s, p, act, image_layer]() {
    nrs_ctx* ctx = self->ctx;
    const float* dy = grad_in(self);
    float* masked = nullptr;
    float *dhi = nullptr, *dlo = nullptr;
    bool staged = false;
    // Do the tensor-core data / weight gradients want NHWC planes of dy?
    const bool want_planes = s == 1 && (ci % 32 == 0 || image_layer) && co % 32 == 0 && planes_possible(ctx);
    if (self->grad_premasked) {
      // The consumer (a max-pool's backward pass or a convolution's data-gradient epilogue) already
      // folded the ReLU mask into this gradient, and may have left its planes.
      if (self->gplanes_hi && want_planes && !ctx->plane_hints.count(dy)) {
        ctx->plane_hints[dy] = NrsPlanes{self->gplanes_hi, self->gplanes_lo, self->gplanes_lo ? 1 : 0};
        staged = true;   // owned by the node, only unregistered below
      }
    } else if (act == NRS_ACT_RELU) {  // y > 0 exactly where the pre-activation was > 0
      masked = dalloc(ctx, self->len());
      if (want_planes) {   // mask and stage in one pass
        const bool split = ctx->math_mode == NRS_MATH_3XTF32;
        dhi = dalloc(ctx, self->len());
        if (split) dlo = dalloc(ctx, self->len());
        check(ctx, nrs_tc_stage_masked(ctx, 0, dy, self->data, nullptr, n, co, (int)self->shape[2], (int)self->shape[3], 1,
                                       masked, dhi, dlo));
        ctx->plane_hints[masked] = NrsPlanes{dhi, dlo, split ? 1 : 0};
        staged = true;
      } else {
        check(ctx, nrs_relu_bwd(ctx, self->data, dy, masked, self->len(), 0));
      }
      dy = masked;
    } else if (want_planes) {
      // dy feeds both the data and the weight gradient: stage its planes once.
      staged = stage_planes(ctx, dy, self->shape, &dhi, &dlo);
    }
    auto cleanup = [&] {
      if (staged) ctx->plane_hints.erase(dy);
      if (dhi) nrs_free(ctx, dhi);
      if (dlo) nrs_free(ctx, dlo);
      if (masked) nrs_free(ctx, masked);
    };
    try {
      conv_backward(self, x, w, b, dy, n, ci, h, wd, co, kh, kw, s, p);
    } catch (...) {
      cleanup();
      throw;
    }
    cleanup();
  };
  return out;
}

NodeP conv2d(const NodeP& x, const NodeP& w, const NodeP& b, size_t stride, size_t pad) {
  return conv2d_act(x, w, b, stride, pad, NRS_ACT_NONE, false);
}

NodeP maxpool2d(const NodeP& x, size_t kernel, size_t stride, bool emit_planes) {
  require_gpu(x, "cuda maxpool: input");
  if (x->shape.size() != 4) fail(NRS_ERR_SHAPE, "cuda maxpool: input must be 4-D");
  nrs_ctx* ctx = x->ctx;
  const int n = (int)x->shape[0], c = (int)x->shape[1], h = (int)x->shape[2], w = (int)x->shape[3];
  const int k = (int)kernel, s = (int)stride;
  if (k < 1 || s < 1 || k > h || k > w) fail(NRS_ERR_SHAPE, "cuda maxpool: window does not fit the input");
  const int oh = (h - k) / s + 1, ow = (w - k) / s + 1;
  NodeP out = make_out(ctx, {(size_t)n, (size_t)c, (size_t)oh, (size_t)ow}, {x});
  void* am = nullptr;
  check(ctx, nrs_alloc(ctx, out->len() * sizeof(int32_t), 0, &am));
  out->saved.push_back(am);
  bool done = false;
  if (emit_planes && k == 2 && s == 2 && c % 32 == 0 && planes_possible(ctx)) {
    // a tensor-core convolution reads the result next: write its operand planes in the same pass
    float* phi = dalloc(ctx, out->len());
    float* plo = ctx->math_mode == NRS_MATH_3XTF32 ? dalloc(ctx, out->len()) : nullptr;
    const int st = nrs_tc_pool2_fwd_planes(ctx, x->data, out->data, (int32_t*)am, phi, plo, n, c, h, w);
    if (st == NRS_OK) {
      out->planes_hi = phi;
      out->planes_lo = plo;
      ctx->plane_hints[out->data] = NrsPlanes{phi, plo, plo ? 1 : 0};
      done = true;
    } else {
      nrs_free(ctx, phi);
      if (plo) nrs_free(ctx, plo);
      if (st != NRS_ERR_UNSUPPORTED) check(ctx, st);
    }
  }
  if (!done) check(ctx, nrs_maxpool_fwd(ctx, x->data, out->data, (int32_t*)am, n, c, h, w, k, s));
  Node* self = out.get();
  out->backward_fn = [self, x, am, n, c, h, w, k, s]() {
    if (!x->requires_grad) return;
    nrs_ctx* ctx = self->ctx;
    const float* g = grad_in(self);
    // Pool over the output of a convolution with a folded ReLU: one pass computes that
    // convolution's masked gradient (and its NHWC planes when its tensor-core backward wants
    // them) instead of pool-backward, ReLU-backward and staging as three passes.
    Node* xr = x.get();
    if (k == s && xr->relu_folded && !xr->view_of && !xr->grad_valid && !xr->grad_premasked) {
      GradTarget t = grad_target(x);   // overwrite mode by construction
      float *phi = nullptr, *plo = nullptr;
      if (xr->wants_grad_planes && planes_possible(ctx) && !xr->gplanes_hi) {
        phi = dalloc(ctx, xr->len());
        if (ctx->math_mode == NRS_MATH_3XTF32) plo = dalloc(ctx, xr->len());
      }
      // self->data (the pooled maximum) is > 0 exactly where the ReLU let the winner through.
      float* partial = k == 2 ? dalloc(ctx, nrs_stage_masked_partial_rows(n, h, w) * (size_t)c) : nullptr;
      int partial_rows = 0;
      check(ctx, nrs_tc_stage_masked(ctx, 1, g, self->data, (const int32_t*)am, n, c, h, w, k, t.ptr, phi, plo, partial,
                                     &partial_rows));
      if (partial && partial_rows == 0) { nrs_free(ctx, partial); partial = nullptr; }
      xr->gplanes_hi = phi;
      xr->gplanes_lo = plo;
      xr->gchan_partial = partial;
      xr->gchan_rows = partial_rows;
      xr->grad_premasked = true;
      return;
    }
    GradTarget t = grad_target(x);
    check(ctx, nrs_maxpool_bwd(ctx, g, (const int32_t*)am, t.ptr, n, c, h, w, k, s, t.accumulate));
  };
  return out;
}

NodeP flatten(const NodeP& x) {
  require_gpu(x, "cuda flatten: input");
  if (x->shape.empty()) fail(NRS_ERR_SHAPE, "cuda flatten: scalar input");
  size_t rest = 1;
  for (size_t i = 1; i < x->shape.size(); ++i) rest *= x->shape[i];
  return reshape(x, {x->shape[0], rest});
}

// LayerNorm of x (residual == nullptr) or of x + residual with the add folded into the same kernels
// (the add + layernorm pairs of src/cuda/nn/transformer_block.rs:33-34,41-42).  One backward launch
// produces the input gradient(s) and, through per-block partial sums, dgamma / dbeta.
// emit_planes: the caller knows that the result feeds tensor-core GEMMs and that the residual addend's only
// reader is this node (the transformer block): the forward kernel then writes the result's TF32 planes itself,
// and the backward kernel those of the addend's gradient, instead of a staging pass per tensor.
static NodeP layernorm_impl(const NodeP& x, const NodeP& residual, const NodeP& gamma, const NodeP& beta, float eps,
                            bool emit_planes = false) {
  require_gpu(x, "cuda layernorm: input");
  require_gpu(gamma, "cuda layernorm: gamma");
  require_gpu(beta, "cuda layernorm: beta");
  if (residual) require_gpu(residual, "cuda layernorm: residual");
  if (x->shape.empty()) fail(NRS_ERR_SHAPE, "cuda layernorm: scalar input");
  if (residual && residual->len() != x->len()) fail(NRS_ERR_SHAPE, "cuda layernorm: residual shape differs from the input's");
  nrs_ctx* ctx = x->ctx;
  const int f = (int)x->shape.back();
  if ((int)gamma->len() != f || (int)beta->len() != f) fail(NRS_ERR_SHAPE, "cuda layernorm: gamma/beta length mismatch");
  const int rows = (int)(x->len() / (size_t)f);
  std::vector<NodeP> parents{x, gamma, beta};
  if (residual) parents.push_back(residual);
  NodeP out = make_out(ctx, x->shape, parents);
  float* xhat = dalloc(ctx, x->len());
  float* istd = dalloc(ctx, (size_t)rows);
  out->saved.push_back(xhat);
  out->saved.push_back(istd);
  const bool planes = emit_planes && planes_possible(ctx) && f % 32 == 0 && rows > 0;
  const bool split = ctx->math_mode == NRS_MATH_3XTF32;
  if (planes && !ctx->plane_hints.count(out->data)) {
    float* hi = dalloc(ctx, x->len());
    float* lo = split ? dalloc(ctx, x->len()) : nullptr;
    int emitted = 0;
    const int st = nrs_layernorm_fwd_planes(ctx, x->data, residual ? residual->data : nullptr, gamma->data, beta->data, out->data,
                                            xhat, istd, rows, f, eps, hi, lo, &emitted);
    if (st == NRS_OK && emitted) {
      out->planes_hi = hi;
      out->planes_lo = lo;
      NrsPlanes pl{hi, lo, split ? 1 : 0};
      pl.rows = rows;
      pl.cols = f;
      ctx->plane_hints[out->data] = pl;
    } else {
      nrs_free(ctx, hi);
      if (lo) nrs_free(ctx, lo);
    }
    check(ctx, st);
  } else if (residual) {
    check(ctx, nrs_layernorm_residual_fwd(ctx, x->data, residual->data, gamma->data, beta->data, out->data, xhat, istd, rows, f, eps));
  } else {
    check(ctx, nrs_layernorm_fwd(ctx, x->data, gamma->data, beta->data, out->data, xhat, istd, rows, f, eps));
  }
  Node* self = out.get();
  out->backward_fn = [self, x, residual, gamma, beta, xhat, istd, rows, f, planes, split]() {
    nrs_ctx* ctx = self->ctx;
    const float* g = grad_in(self);
    float *da = nullptr, *db = nullptr, *dg = nullptr, *dbt = nullptr;
    int acc_a = 0, acc_b = 0, acc_p = 0;
    if (x->requires_grad) {
      GradTarget t = grad_target(x);
      da = t.ptr;
      acc_a = t.accumulate;
    }
    if (residual && residual->requires_grad) {
      if (grad_root(residual.get()) == grad_root(x.get()) && da) {
        // x + x: the one buffer receives the gradient twice
        check(ctx, nrs_layernorm_residual_bwd(ctx, g, xhat, istd, gamma->data, da, nullptr, nullptr, nullptr, rows, f, acc_a, 0, 0));
        acc_a = 1;
      } else {
        GradTarget t = grad_target(residual);
        db = t.ptr;
        acc_b = t.accumulate;
      }
    }
    if (gamma->requires_grad || beta->requires_grad) {
      GradTarget tg = grad_target(gamma), tb = grad_target(beta);
      if (tg.accumulate != tb.accumulate) {  // bring both to "accumulate" state
        if (!tg.accumulate) check(ctx, nrs_memset_zero(ctx, tg.ptr, sizeof(float) * f));
        if (!tb.accumulate) check(ctx, nrs_memset_zero(ctx, tb.ptr, sizeof(float) * f));
        tg.accumulate = tb.accumulate = 1;
      }
      dg = tg.ptr;
      dbt = tb.ptr;
      acc_p = tg.accumulate;
    }
    if (!(da || db || dg)) return;
    Node* rb = db ? grad_root(residual.get()) : nullptr;
    // planes an earlier backward pass over this graph left with the addend describe its old gradient
    auto hint = db ? ctx->plane_hints.find(db) : ctx->plane_hints.end();
    const bool mine = rb && rb->gplanes_hi && hint != ctx->plane_hints.end() && hint->second.hi == rb->gplanes_hi &&
                      (hint->second.split != 0) == split;
    const bool fresh_slot = rb && !rb->gplanes_hi && hint == ctx->plane_hints.end();
    if (planes && da && db && acc_b == 0 && (mine || fresh_slot)) {
      // the addend's gradient is exactly this kernel's result: its planes come out of the same pass
      float* hi = mine ? rb->gplanes_hi : dalloc(ctx, self->len());
      float* lo = mine ? rb->gplanes_lo : (split ? dalloc(ctx, self->len()) : nullptr);
      int emitted = 0;
      const int st = nrs_layernorm_bwd_planes(ctx, g, xhat, istd, gamma->data, da, db, dg, dbt, rows, f, acc_a, acc_b, acc_p, hi, lo,
                                              &emitted);
      if (st == NRS_OK && emitted) {
        if (!mine) {
          rb->gplanes_hi = hi;
          rb->gplanes_lo = lo;
          NrsPlanes pl{hi, lo, split ? 1 : 0};
          pl.rows = rows;
          pl.cols = f;
          ctx->plane_hints[db] = pl;   // dropped with the node (keyed by its gradient buffer)
        }
      } else {
        if (mine) {
          ctx->plane_hints.erase(db);
          rb->gplanes_hi = rb->gplanes_lo = nullptr;
        }
        nrs_free(ctx, hi);
        if (lo) nrs_free(ctx, lo);
      }
      check(ctx, st);
      return;
    }
    if (mine) {   // this pass adds to the gradient (or stages nothing): the old planes must go
      ctx->plane_hints.erase(db);
      nrs_free(ctx, rb->gplanes_hi);
      if (rb->gplanes_lo) nrs_free(ctx, rb->gplanes_lo);
      rb->gplanes_hi = rb->gplanes_lo = nullptr;
    }
    check(ctx, nrs_layernorm_residual_bwd(ctx, g, xhat, istd, gamma->data, da, db, dg, dbt, rows, f, acc_a, acc_b, acc_p));
  };
  return out;
}

NodeP layernorm(const NodeP& x, const NodeP& gamma, const NodeP& beta, float eps) {
  return layernorm_impl(x, nullptr, gamma, beta, eps);
}

NodeP layernorm_residual(const NodeP& x, const NodeP& residual, const NodeP& gamma, const NodeP& beta, float eps,
                         bool emit_planes) {
  if (!residual) fail(NRS_ERR_ARG, "cuda layernorm: null residual");
  return layernorm_impl(x, residual, gamma, beta, eps, emit_planes);
}

// batchnorm (src/cuda/nn/batchnorm.rs:110-232) for [batch, features] and batchnorm2d
// (src/cuda/nn/batchnorm2d.rs:130-232) for [batch, channels, h, w]: the running statistics are resident
// nodes owned by the caller and updated in place in training mode.
NodeP batchnorm_nd(const NodeP& x, const NodeP& gamma, const NodeP& beta, const NodeP& running_mean,
                   const NodeP& running_var, float momentum, float eps, bool training, size_t want_dims,
                   const char* what, int act = NRS_ACT_NONE) {
  const std::string w(what);
  require_gpu(x, (w + ": input").c_str());
  require_gpu(gamma, (w + ": gamma").c_str());
  require_gpu(beta, (w + ": beta").c_str());
  require_gpu(running_mean, (w + ": running_mean").c_str());
  require_gpu(running_var, (w + ": running_var").c_str());
  if (x->shape.size() != want_dims && !(want_dims == 0 && (x->shape.size() == 2 || x->shape.size() == 4)))
    fail(NRS_ERR_SHAPE, (w + ": input has the wrong number of dimensions").c_str());
  if (act != NRS_ACT_NONE && act != NRS_ACT_RELU) fail(NRS_ERR_ARG, (w + ": only a ReLU can be fused").c_str());
  nrs_ctx* ctx = x->ctx;
  const int n = (int)x->shape[0], c = (int)x->shape[1];
  if (n < 1 || c < 1 || x->len() == 0) fail(NRS_ERR_SHAPE, (w + ": empty input").c_str());
  const int hw = (int)(x->len() / ((size_t)n * c));
  if ((int)gamma->len() != c || (int)beta->len() != c || (int)running_mean->len() != c || (int)running_var->len() != c)
    fail(NRS_ERR_SHAPE, (w + ": gamma/beta/running statistics length mismatch").c_str());
  NodeP out = make_out(ctx, x->shape, {x, gamma, beta});
  float* xhat = dalloc(ctx, x->len());
  float* istd = dalloc(ctx, (size_t)c);
  out->saved.push_back(xhat);
  out->saved.push_back(istd);
  check(ctx, nrs_batchnorm_act_fwd(ctx, x->data, gamma->data, beta->data, running_mean->data, running_var->data, out->data,
                                   xhat, istd, n, c, hw, eps, momentum, training ? 1 : 0, act));
  Node* self = out.get();
  out->backward_fn = [self, x, gamma, beta, xhat, istd, n, c, hw, training, act]() {
    nrs_ctx* ctx = self->ctx;
    const float* g = grad_in(self);
    float *dg = nullptr, *db = nullptr;
    int acc_p = 0;
    if (gamma->requires_grad || beta->requires_grad) {
      GradTarget tg = grad_target(gamma), tb = grad_target(beta);
      if (tg.accumulate != tb.accumulate) {  // bring both to "accumulate" state
        if (!tg.accumulate) check(ctx, nrs_memset_zero(ctx, tg.ptr, sizeof(float) * c));
        if (!tb.accumulate) check(ctx, nrs_memset_zero(ctx, tb.ptr, sizeof(float) * c));
        tg.accumulate = tb.accumulate = 1;
      }
      dg = tg.ptr;
      db = tb.ptr;
      acc_p = tg.accumulate;
    }
    float* dx = nullptr;
    int acc_x = 0;
    if (x->requires_grad) {
      GradTarget t = grad_target(x);
      dx = t.ptr;
      acc_x = t.accumulate;
    }
    check(ctx, nrs_batchnorm_act_bwd(ctx, g, xhat, istd, gamma->data, beta->data, dx, dg, db, n, c, hw, training ? 1 : 0,
                                     acc_x, acc_p, act));
  };
  return out;
}

NodeP batchnorm(const NodeP& x, const NodeP& gamma, const NodeP& beta, const NodeP& running_mean,
                const NodeP& running_var, float momentum, float eps, bool training) {
  return batchnorm_nd(x, gamma, beta, running_mean, running_var, momentum, eps, training, 2, "cuda bn");
}

NodeP batchnorm2d(const NodeP& x, const NodeP& gamma, const NodeP& beta, const NodeP& running_mean,
                  const NodeP& running_var, float momentum, float eps, bool training) {
  return batchnorm_nd(x, gamma, beta, running_mean, running_var, momentum, eps, training, 4, "cuda bn2d");
}

// batchnorm / batchnorm2d (by the input's rank) followed by `act` (NRS_ACT_NONE or NRS_ACT_RELU) in the same
// two passes: the conv -> batchnorm2d -> relu unit of examples/cifar_cuda.rs:44-48 without the ReLU's own passes.
NodeP batchnorm_act(const NodeP& x, const NodeP& gamma, const NodeP& beta, const NodeP& running_mean,
                    const NodeP& running_var, float momentum, float eps, bool training, int act) {
  return batchnorm_nd(x, gamma, beta, running_mean, running_var, momentum, eps, training, 0, "cuda bn+act", act);
}

// dropout (src/cuda/nn/dropout.rs:31-84) and dropout2d (src/cuda/nn/dropout2d.rs:37-end): evaluation returns
// the input node itself; training multiplies by a mask of 0 / 1/(1-p) values (one per element, or one per
// (sample, channel) plane) that also routes the gradient.  `mask` == nullptr draws the mask on the device
// from the context's counter-based generator; otherwise the caller's resident mask is used as it is.
NodeP dropout_nd(const NodeP& x, float p, bool training, const NodeP& mask, bool spatial, const char* what) {
  if (!training) return x;
  const std::string w(what);
  require_gpu(x, (w + ": input").c_str());
  if (!(p >= 0.0f && p <= 1.0f)) fail(NRS_ERR_ARG, (w + ": probability outside [0,1]").c_str());
  nrs_ctx* ctx = x->ctx;
  size_t hw = 1;
  if (spatial) {
    if (x->shape.size() != 4) fail(NRS_ERR_SHAPE, (w + ": input must be [batch, channels, h, w]").c_str());
    hw = x->shape[2] * x->shape[3];
  }
  if (x->len() == 0 || hw == 0) fail(NRS_ERR_SHAPE, (w + ": empty input").c_str());
  const size_t mask_len = x->len() / hw;
  const float* mask_ptr = nullptr;
  NodeP out = make_out(ctx, x->shape, {x});
  if (mask) {
    require_gpu(mask, (w + ": mask").c_str());
    if (mask->len() != mask_len) fail(NRS_ERR_SHAPE, (w + ": mask length mismatch").c_str());
    mask_ptr = mask->data;
    out->parents.push_back(mask);   // keeps the caller's mask alive until the backward pass has run
  } else {
    float* m = dalloc(ctx, mask_len);
    out->saved.push_back(m);
    check(ctx, nrs_dropout_mask(ctx, m, mask_len, p));
    mask_ptr = m;
  }
  check(ctx, nrs_mask_mul(ctx, x->data, mask_ptr, out->data, x->len(), (int)hw, 0));
  Node* self = out.get();
  const size_t total = x->len();
  out->backward_fn = [self, x, mask_ptr, total, hw]() {
    if (!x->requires_grad) return;
    nrs_ctx* ctx = self->ctx;
    GradTarget t = grad_target(x);
    check(ctx, nrs_mask_mul(ctx, grad_in(self), mask_ptr, t.ptr, total, (int)hw, t.accumulate));
  };
  return out;
}

NodeP dropout(const NodeP& x, float p, bool training, const NodeP& mask) {
  return dropout_nd(x, p, training, mask, false, "cuda dropout");
}

NodeP dropout2d(const NodeP& x, float p, bool training, const NodeP& mask) {
  return dropout_nd(x, p, training, mask, true, "cuda dropout2d");
}

NodeP linear_act(const NodeP& x, const NodeP& w, const NodeP& b, int act) {
  require_gpu(x, "cuda linear: input");
  require_gpu(w, "cuda linear: weights");
  require_gpu(b, "cuda linear: bias");
  if (x->shape.size() != 2 || w->shape.size() != 2) fail(NRS_ERR_SHAPE, "cuda linear: operands must be 2-D");
  if (w->shape[0] != x->shape[1] || b->len() != w->shape[1]) fail(NRS_ERR_SHAPE, "cuda linear: shape mismatch");
  if (act < NRS_ACT_NONE || act > NRS_ACT_GELU) fail(NRS_ERR_ARG, "cuda linear: unknown activation");
  nrs_ctx* ctx = x->ctx;
  const int m = (int)x->shape[0], k = (int)x->shape[1], n = (int)w->shape[1];
  NodeP out = make_out(ctx, {(size_t)m, (size_t)n}, {x, w, b});
  const bool tensor_cores = nrs_gemm_on_tensor_cores(ctx, m, n, k);
  if (tensor_cores && w->requires_grad) cache_planes_2d(x, (size_t)m, (size_t)k);   // read again by dW = x^T dz
  float* pre = nullptr;  // GELU's derivative needs the pre-activation
  if (act == NRS_ACT_GELU) {
    pre = dalloc(ctx, out->len());
    out->saved.push_back(pre);
    // one kernel writes the pre-activation (GELU's derivative reads it) and the activation
    const int st = nrs_linear_act_pre(ctx, m, n, k, x->data, w->data, b->data, NRS_ACT_GELU, out->data, pre);
    if (st == NRS_ERR_UNSUPPORTED) {
      check(ctx, nrs_gemm(ctx, 0, 0, m, n, k, x->data, w->data, pre, b->data, NRS_ACT_NONE, 0.0f));
      check(ctx, nrs_gelu_fwd(ctx, pre, out->data, out->len()));
    } else {
      check(ctx, st);
    }
  } else {
    check(ctx, nrs_gemm(ctx, 0, 0, m, n, k, x->data, w->data, out->data, b->data, act, 0.0f));
  }
  Node* self = out.get();
  out->backward_fn = [self, x, w, b, pre, act, m, k, n, tensor_cores]() {
    nrs_ctx* ctx = self->ctx;
    const float* dz = grad_in(self);
    float* tmp = nullptr;
    if (act != NRS_ACT_NONE) {
      tmp = dalloc(ctx, self->len());
      if (act == NRS_ACT_RELU) check(ctx, nrs_relu_bwd(ctx, self->data, dz, tmp, self->len(), 0));
      else check(ctx, nrs_gelu_bwd(ctx, pre, dz, tmp, self->len(), 0));
      dz = tmp;
    }
    // dz feeds both dW = x^T dz and dX = dz W^T: its planes are made once
    GradPlanes dz_planes(ctx, dz, (size_t)m, (size_t)n, tensor_cores && w->requires_grad && x->requires_grad);
    if (b->requires_grad) {
      GradTarget t = grad_target(b);
      check(ctx, nrs_sum_axis0(ctx, dz, t.ptr, m, n, t.accumulate));
    }
    if (x->requires_grad) {
      GradTarget t = grad_target(x);
      check(ctx, nrs_gemm(ctx, 0, 1, m, k, n, dz, w->data, t.ptr, nullptr, NRS_ACT_NONE, t.accumulate ? 1.0f : 0.0f));
    }
    if (w->requires_grad) {   // after dX: it reads nothing dX wrote, so it may start under dX's tail
      GradTarget t = grad_target(w);
      NrsIndependentNext overlap(ctx, x->requires_grad);
      check(ctx, nrs_gemm(ctx, 1, 0, k, n, m, x->data, dz, t.ptr, nullptr, NRS_ACT_NONE, t.accumulate ? 1.0f : 0.0f));
    }
    if (tmp) nrs_free(ctx, tmp);
  };
  return out;
}

// --------------------------------------------------------------------- loss

static void batch_classes(const NodeP& n, int* batch, int* classes) {
  if (n->shape.size() == 2) { *batch = (int)n->shape[0]; *classes = (int)n->shape[1]; }
  else { *batch = 1; *classes = (int)n->shape[0]; }  // src/cuda/loss/cross_entropy.rs:62-67
}

float cross_entropy(const NodeP& pred, const NodeP& target) {
  require_gpu(pred, "cuda ce: logits");
  require_gpu(target, "cuda ce: target");
  if (pred->len() != target->len()) fail(NRS_ERR_SHAPE, "cuda ce: logits and target sizes differ");
  nrs_ctx* ctx = pred->ctx;
  int batch, classes;
  batch_classes(pred, &batch, &classes);
  float* loss_dev = dalloc(ctx, 1);
  float loss = 0.0f;
  int st = nrs_ce_fwd(ctx, pred->data, target->data, loss_dev, nullptr, batch, classes, batch);
  if (st == NRS_OK) st = nrs_d2h(ctx, &loss, loss_dev, sizeof(float));
  nrs_free(ctx, loss_dev);
  check(ctx, st);
  return loss;
}

void cross_entropy_backward(const NodeP& pred, const NodeP& target) {
  require_gpu(pred, "cuda ce: logits");
  require_gpu(target, "cuda ce: target");
  if (pred->len() != target->len()) fail(NRS_ERR_SHAPE, "cuda ce: logits and target sizes differ");
  nrs_ctx* ctx = pred->ctx;
  int batch, classes;
  batch_classes(pred, &batch, &classes);
  Node* r = grad_root(pred.get());
  if (!r->grad) r->grad = dalloc(ctx, r->len());
  check(ctx, nrs_ce_bwd(ctx, pred->data, target->data, r->grad, batch, classes, batch));
  r->grad_valid = true;  // overwritten, as the reference does
}

void cross_entropy_fused(const NodeP& pred, const NodeP& target, float* loss_dev, int divisor) {
  require_gpu(pred, "cuda ce: logits");
  require_gpu(target, "cuda ce: target");
  if (pred->len() != target->len()) fail(NRS_ERR_SHAPE, "cuda ce: logits and target sizes differ");
  nrs_ctx* ctx = pred->ctx;
  int batch, classes;
  batch_classes(pred, &batch, &classes);
  Node* r = grad_root(pred.get());
  if (!r->grad) r->grad = dalloc(ctx, r->len());
  check(ctx, nrs_ce_fwd_bwd(ctx, pred->data, target->data, loss_dev, r->grad, batch, classes, divisor));
  r->grad_valid = true;
}

void cross_entropy_fused_indexed(const NodeP& pred, const int32_t* labels_dev, float* loss_dev, int divisor) {
  require_gpu(pred, "cuda ce: logits");
  if (!labels_dev) fail(NRS_ERR_ARG, "cuda ce: null labels");
  if (pred->shape.size() != 2) fail(NRS_ERR_SHAPE, "cuda ce: logits must be [rows, classes]");
  nrs_ctx* ctx = pred->ctx;
  Node* r = grad_root(pred.get());
  if (!r->grad) r->grad = dalloc(ctx, r->len());
  check(ctx, nrs_ce_fwd_bwd_indexed(ctx, pred->data, labels_dev, loss_dev, r->grad, (int)pred->shape[0], (int)pred->shape[1], divisor));
  r->grad_valid = true;
}

// -------------------------------------------------------------------- optim

// f32 integer power by repeated squaring — what Rust's f32::powi lowers to.
static float powi_f32(float a, int b) {
  float r = 1.0f;
  while (true) {
    if (b & 1) r *= a;
    b /= 2;
    if (b == 0) break;
    a *= a;
  }
  return r;
}

AdamW::AdamW(nrs_ctx* ctx, float lr_, float b1, float b2, float eps, float wd)
    : lr(lr_), beta1(b1), beta2(b2), epsilon(eps), weight_decay(wd), ctx_(ctx) {
  if (!ctx) fail(NRS_ERR_ARG, "AdamW::new: null context");
}

void AdamW::release() {
  if (owns_each_) {
    for (float* p : m_) nrs_free(ctx_, p);
    for (float* p : v_) nrs_free(ctx_, p);
  }
  if (flat_m_) nrs_free(ctx_, flat_m_);
  if (flat_v_) nrs_free(ctx_, flat_v_);
  m_.clear(); v_.clear(); len_.clear();
  flat_m_ = flat_v_ = nullptr;
  flat_total_ = 0;
  owns_each_ = false;
}

AdamW::~AdamW() { release(); }

// True when the parameters are exactly the tensors of one FlatStore, in order.
static std::shared_ptr<FlatStore> common_flat(const std::vector<NodeP>& params) {
  if (params.empty() || !params[0]->flat) return nullptr;
  auto fs = params[0]->flat;
  if (fs->offset.size() != params.size()) return nullptr;
  for (size_t i = 0; i < params.size(); ++i)
    if (params[i]->flat != fs || params[i]->data != fs->data + fs->offset[i]) return nullptr;
  return fs;
}

void AdamW::ensure_state(const std::vector<NodeP>& params) {
  const bool imported = !m_.empty() && !flat_m_ && owns_each_;
  if (!m_.empty() && !imported) return;
  auto fs = common_flat(params);
  if (imported) {
    // State came from import_state as per-parameter vectors; when the parameters
    // live in one flat block, move the moments into matching flat blocks.
    if (m_.size() != params.size()) fail(NRS_ERR_SHAPE, "adamw: parameter count changed between steps");
    for (size_t i = 0; i < params.size(); ++i)
      if (len_[i] != params[i]->len()) fail(NRS_ERR_SHAPE, "adamw: imported moment size does not match its parameter");
    if (!fs) return;
    float* fm = dalloc(ctx_, fs->total, true);
    float* fv = dalloc(ctx_, fs->total, true);
    for (size_t i = 0; i < params.size(); ++i) {
      check(ctx_, nrs_d2d(ctx_, fm + fs->offset[i], m_[i], len_[i] * sizeof(float)));
      check(ctx_, nrs_d2d(ctx_, fv + fs->offset[i], v_[i], len_[i] * sizeof(float)));
      nrs_free(ctx_, m_[i]);
      nrs_free(ctx_, v_[i]);
      m_[i] = fm + fs->offset[i];
      v_[i] = fv + fs->offset[i];
    }
    flat_m_ = fm; flat_v_ = fv; flat_total_ = fs->total;
    owns_each_ = false;
    return;
  }
  // First step: zero moments matched to the parameters (adamw.rs:68-74).
  if (fs) {
    flat_m_ = dalloc(ctx_, fs->total, true);
    flat_v_ = dalloc(ctx_, fs->total, true);
    flat_total_ = fs->total;
    for (size_t i = 0; i < params.size(); ++i) {
      m_.push_back(flat_m_ + fs->offset[i]);
      v_.push_back(flat_v_ + fs->offset[i]);
      len_.push_back(params[i]->len());
    }
  } else {
    owns_each_ = true;
    for (const auto& p : params) {
      m_.push_back(dalloc(ctx_, p->len(), true));
      v_.push_back(dalloc(ctx_, p->len(), true));
      len_.push_back(p->len());
    }
  }
}

void AdamW::step(const std::vector<NodeP>& params) {
  for (const auto& p : params) require_gpu(p, "adamw: param");
  ensure_state(params);
  if (params.size() != m_.size()) fail(NRS_ERR_SHAPE, "adamw: parameter count changed between steps");
  const float bc1 = 1.0f - powi_f32(beta1, (int)t + 1);
  const float bc2 = 1.0f - powi_f32(beta2, (int)t + 1);
  for (const auto& p : params) (void)grad_in(p.get());  // unwritten gradients read as zero
  auto fs = flat_m_ ? common_flat(params) : nullptr;
  if (fs && fs->total == flat_total_) {
    check(ctx_, nrs_adamw_step(ctx_, fs->data, fs->grad, flat_m_, flat_v_, fs->total, lr, beta1, beta2, epsilon,
                               weight_decay, bc1, bc2, grad_scale));
  } else {
    for (size_t i = 0; i < params.size(); ++i) {
      if (params[i]->len() != len_[i]) fail(NRS_ERR_SHAPE, "adamw: parameter size changed between steps");
      check(ctx_, nrs_adamw_step(ctx_, params[i]->data, grad_root(params[i].get())->grad, m_[i], v_[i], len_[i], lr,
                                 beta1, beta2, epsilon, weight_decay, bc1, bc2, grad_scale));
    }
  }
  t += 1;
}

void AdamW::begin_flat_step(const std::vector<NodeP>& params) {
  for (const auto& p : params) require_gpu(p, "adamw: param");
  ensure_state(params);
  auto fs = flat_m_ ? common_flat(params) : nullptr;
  if (!fs || fs->total != flat_total_) fail(NRS_ERR_ARG, "adamw: a flat step needs parameters that share one flat block");
  stepping_ = fs;
}

void AdamW::step_flat_range(size_t begin, size_t end) {
  if (!stepping_) fail(NRS_ERR_ARG, "adamw: step_flat_range outside begin_flat_step / end_flat_step");
  if (begin > end || end > flat_total_) fail(NRS_ERR_ARG, "adamw: range outside the flat block");
  if (begin == end) return;
  const float bc1 = 1.0f - powi_f32(beta1, (int)t + 1);
  const float bc2 = 1.0f - powi_f32(beta2, (int)t + 1);
  check(ctx_, nrs_adamw_step(ctx_, stepping_->data + begin, stepping_->grad + begin, flat_m_ + begin, flat_v_ + begin,
                             end - begin, lr, beta1, beta2, epsilon, weight_decay, bc1, bc2, grad_scale));
}

void AdamW::end_flat_step() {
  if (!stepping_) fail(NRS_ERR_ARG, "adamw: end_flat_step without begin_flat_step");
  stepping_.reset();
  t += 1;
}

std::vector<std::vector<float>> AdamW::export_state(size_t* t_out) const {
  if (t_out) *t_out = t;
  std::vector<std::vector<float>> out;
  for (int pass = 0; pass < 2; ++pass)
    for (size_t i = 0; i < m_.size(); ++i) {
      std::vector<float> h(len_[i]);
      check(ctx_, nrs_d2h(ctx_, h.data(), pass == 0 ? m_[i] : v_[i], h.size() * sizeof(float)));
      out.push_back(std::move(h));
    }
  return out;
}

void AdamW::import_state(size_t t_in, const std::vector<std::vector<float>>& moments) {
  if (moments.size() % 2 != 0) fail(NRS_ERR_ARG, "adamw: moments must be all m's then all v's");
  release();
  const size_t half = moments.size() / 2;
  owns_each_ = true;
  for (size_t i = 0; i < half; ++i) {
    if (moments[i].size() != moments[half + i].size()) fail(NRS_ERR_SHAPE, "adamw: m/v size mismatch");
    float* m = dalloc(ctx_, moments[i].size());
    float* v = dalloc(ctx_, moments[i].size());
    m_.push_back(m);
    v_.push_back(v);
    len_.push_back(moments[i].size());
    check(ctx_, nrs_h2d(ctx_, m, moments[i].data(), moments[i].size() * sizeof(float)));
    check(ctx_, nrs_h2d(ctx_, v, moments[half + i].data(), moments[i].size() * sizeof(float)));
  }
  check(ctx_, nrs_sync(ctx_));
  t = t_in;
}

}  // namespace cuda

// ---------------------------------------------------------------- backward

static void build_topo(const NodeP& n, std::unordered_set<const Node*>& seen, std::vector<NodeP>& topo) {
  // Iterative DFS (post-order) so deep chains cannot overflow the stack.
  struct Frame { NodeP node; size_t next; };
  std::vector<Frame> stack;
  if (!seen.insert(n.get()).second) return;
  stack.push_back({n, 0});
  while (!stack.empty()) {
    Frame& f = stack.back();
    if (f.next < f.node->parents.size()) {
      const NodeP& p = f.node->parents[f.next++];
      if (seen.insert(p.get()).second) stack.push_back({p, 0});
    } else {
      topo.push_back(f.node);
      stack.pop_back();
    }
  }
}

void backward_graph(const NodeP& root) {
  if (!root) fail(NRS_ERR_ARG, "backward_graph: null root");
  std::vector<NodeP> topo;
  std::unordered_set<const Node*> seen;
  build_topo(root, seen, topo);
  for (auto it = topo.rbegin(); it != topo.rend(); ++it)
    if ((*it)->backward_fn) (*it)->backward_fn();
}

}  // namespace nrs
