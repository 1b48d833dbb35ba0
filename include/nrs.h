/*
 * nrs.h — C ABI of libnrs_b200.so, a Blackwell (sm_100a) backend for the
 * resident-GPU training path of NeuralRs (JackpotMachine777/neuralrs v0.3.0).
 *
 * The reference drives its GPU path from Rust through the cudarc crate: one
 * NVRTC-compiled CUDA-C kernel string per operator, launched by name
 * (src/cuda/backend.rs:39-42, src/cuda/runtime.rs:24-34).  This header is the
 * set of entry points a Rust `extern "C"` block would bind instead.  Each
 * declaration names the reference interface it stands in for.
 *
 * Conventions
 *  - Every pointer named x, w, y, dy, ... is a DEVICE pointer to f32 unless the
 *    comment says "host".  Tensors are dense, row-major, in the reference's own
 *    layouts (images NCHW, conv weights [c_out,c_in,kh,kw], Linear weights
 *    [in,out]).
 *  - Every call returns an int status (NRS_OK == 0).  The reference panics via
 *    `.expect(...)` (e.g. src/cuda/runtime.rs:43-45); a binding turns a non-zero
 *    status into the same panic, with the text from nrs_last_error().
 *  - All work is enqueued on the context's stream; calls return without
 *    waiting unless they say otherwise.  A context is bound to one device and is
 *    not thread-safe, like the reference's single global backend
 *    (src/cuda/backend.rs:17).
 *  - There is no CPU fallback: every entry point fails with NRS_ERR_CUDA when no
 *    usable device is present.
 *  - Backward entry points take `accumulate`: 0 overwrites the destination
 *    gradient, non-zero adds to it.  The reference always adds into the parent's
 *    gradient (src/cuda/runtime.rs:14-18, 67-83); overwrite mode lets the first
 *    writer skip the zero-fill plus the extra read-modify-write pass.
 */
#ifndef NRS_H
#define NRS_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct nrs_ctx nrs_ctx;

enum nrs_status {
  NRS_OK = 0,
  NRS_ERR_ARG = 1,         /* null pointer, negative size, bad enum          */
  NRS_ERR_SHAPE = 2,       /* dimensions inconsistent with each other        */
  NRS_ERR_ALLOC = 3,       /* device or host allocation failed               */
  NRS_ERR_CUDA = 4,        /* a CUDA runtime/driver call failed              */
  NRS_ERR_NCCL = 5,        /* an NCCL call failed or NCCL cannot be loaded   */
  NRS_ERR_TIMEOUT = 6,     /* a bounded wait ran out                         */
  NRS_ERR_UNSUPPORTED = 7  /* valid request this build has no kernel for     */
};

/* Contraction precision.  3xTF32 (default): each f32 operand is split into a
 * TF32 high part and a TF32 residual and three tensor-core products are summed
 * in f32 (error ~1e-6 relative).  TF32: one product (error ~1e-3).  FP32: the
 * CUDA-core FFMA kernels only. */
enum nrs_math_mode { NRS_MATH_3XTF32 = 0, NRS_MATH_TF32 = 1, NRS_MATH_FP32 = 2 };

/* Activation fused into a contraction's epilogue. */
enum nrs_act { NRS_ACT_NONE = 0, NRS_ACT_RELU = 1, NRS_ACT_GELU = 2 };

/* ------------------------------------------------------------- lifecycle -- */

/* Create a context on `device` with its own non-blocking stream.
 * Stands in for the lazily initialised global backend: CudaContext::new(0) +
 * default_stream (src/cuda/backend.rs:19-32). */
int nrs_init(int device, nrs_ctx** out);
int nrs_destroy(nrs_ctx* ctx);
/* Text of the last failure on this context (never NULL).  With ctx == NULL:
 * the last failure of a call that had no context (e.g. nrs_init). */
const char* nrs_last_error(const nrs_ctx* ctx);
/* Run this context's work on a caller-owned cudaStream_t (e.g. the stream a
 * host framework is using).  NULL restores the context's own stream. */
int nrs_set_stream(nrs_ctx* ctx, void* cuda_stream);
void* nrs_get_stream(nrs_ctx* ctx);
int nrs_set_math_mode(nrs_ctx* ctx, int mode);
int nrs_get_math_mode(const nrs_ctx* ctx);
/* Number of kernels this library has launched on this context so far. */
uint64_t nrs_launch_count(const nrs_ctx* ctx);
/* 1 if the tensor-core (tcgen05) kernels were compiled into this build. */
int nrs_has_tensor_core_path(void);

/* Device timing per kernel family, off by default.  While enabled, the library
 * brackets every launch of the listed families with CUDA events on the
 * context's stream; nrs_profile_get waits for the stream and returns the
 * summed device time, the summed algorithmic work (FLOP for contractions,
 * bytes for AdamW) and the number of bracketed calls since the last reset.
 * The reference has no profiling hooks (it prints wall-clock times,
 * examples/cifar_cuda.rs:265,284). */
enum nrs_prof_kind {
  NRS_PROF_CONV_FWD = 0, NRS_PROF_CONV_DGRAD = 1, NRS_PROF_CONV_WGRAD = 2,
  NRS_PROF_GEMM = 3, NRS_PROF_ADAMW = 4, NRS_PROF_BATCHNORM = 5 /* work = algorithmic bytes */, NRS_PROF_KINDS = 6
};
/* Self-test of the time-out path (no reference counterpart).  Every device-side wait of the
 * tensor-core kernels is bounded: on expiry the kernel records a code, and the next nrs_sync /
 * nrs_d2h returns NRS_ERR_TIMEOUT while the context stays usable.  This entry point launches a
 * one-thread kernel that waits `limit_clocks` SM clocks on a barrier nobody completes, so that path
 * can be exercised without a fault or a hang. */
int nrs_selftest_bounded_wait(nrs_ctx* ctx, int64_t limit_clocks);
/* Host-only self-test (no reference counterpart, needs no GPU): the library remembers per device
 * ordinal which kernels already had their dynamic shared-memory limit raised, so that contexts on
 * several GPUs of one process each get theirs.  Returns 0 when that bookkeeping behaves. */
int nrs_selftest_smem_attr_bookkeeping(void);

/* Measures the tensor pipe's dense-TF32 rate on this device (no reference counterpart): every SM
 * issues tcgen05.mma.kind::tf32 (128 x 256 x 8) back to back on operands resident in shared memory
 * for a few milliseconds; the result is what the contraction kernels' tensor-core roofline is
 * quoted against.  Waits for the stream. */
int nrs_measure_tf32_umma_peak(nrs_ctx* ctx, double* tflops_out);

int nrs_profile_enable(nrs_ctx* ctx, int on);
int nrs_profile_reset(nrs_ctx* ctx);
int nrs_profile_get(nrs_ctx* ctx, int kind, double* ms_out, double* work_out, uint64_t* calls_out);

/* ---------------------------------------------------------------- memory -- */
/* stream.alloc_zeros / clone_htod / clone_dtoh / memset_zeros / synchronize
 * (src/cuda/runtime.rs:39-51, 55-62, 108-124).  nrs_alloc draws from a
 * size-bucketed pool owned by the context, so steady-state training steps call
 * no cudaMalloc; memory is zero-filled like alloc_zeros only when `zero`. */
int nrs_alloc(nrs_ctx* ctx, size_t bytes, int zero, void** dptr);
int nrs_free(nrs_ctx* ctx, void* dptr);
int nrs_memset_zero(nrs_ctx* ctx, void* dptr, size_t bytes);
int nrs_h2d(nrs_ctx* ctx, void* dst_dev, const void* src_host, size_t bytes);
int nrs_d2h(nrs_ctx* ctx, void* dst_host, const void* src_dev, size_t bytes); /* waits */
int nrs_d2d(nrs_ctx* ctx, void* dst_dev, const void* src_dev, size_t bytes);
int nrs_sync(nrs_ctx* ctx);

/* ---------------------------------------------------------- contractions -- */

/* C[m,n] = act(op(A).op(B) + bias[n]) + beta*C, all row-major.
 * trans_a == 0: A is [m,k]; else A is stored [k,m].
 * trans_b == 0: B is [k,n]; else B is stored [n,k].
 * bias may be NULL.  beta is 0 or 1.
 * Replaces mm("matmul_nn"|"matmul_nt"|"matmul_tn") and the bias_add pass
 * (src/cuda/graph/matmul.rs:269-293, 343-348; src/cuda/graph/add.rs:26-30). */
int nrs_gemm(nrs_ctx* ctx, int trans_a, int trans_b, int m, int n, int k,
             const float* a, const float* b, float* c, const float* bias, int act, float beta);

/* Batched C[b] = op(A[b]).op(B[b]) + beta*C[b]; operands densely stacked.
 * Replaces bmm_forward / bmm_grad_a / bmm_grad_b (src/cuda/graph/bmm.rs:12-56). */
int nrs_bmm(nrs_ctx* ctx, int trans_a, int trans_b, int batch, int m, int n, int k,
            const float* a, const float* b, float* c, float beta);

/* y[N,Co,oh,ow] = act(conv(x[N,Ci,H,W], w[Co,Ci,kh,kw]) + b[Co]); zero padding,
 * cross-correlation, oh=(H+2p-kh)/s+1.  Replaces conv2d_im2col + matmul_nn +
 * conv2d_col2out (src/cuda/nn/conv.rs:244-279). */
int nrs_conv2d_fwd(nrs_ctx* ctx, const float* x, const float* w, const float* b, float* y,
                   int n, int ci, int h, int wd, int co, int kh, int kw, int stride, int pad,
                   int act);
/* Gradients of nrs_conv2d_fwd (act == NONE) given dy[N,Co,oh,ow]:
 *   dx[N,Ci,H,W] (skipped when NULL, as for requires_grad == false,
 *   src/cuda/nn/conv.rs:304), dw[Co,Ci,kh,kw], db[Co]; any may be NULL.
 * The weight gradient is a split-K contraction reduced in a fixed order, so it
 * is run-to-run deterministic (the reference's atomicAdd split-K is not,
 * src/cuda/graph/matmul.rs:207-261).
 * Replaces out2mm + matmul_tn + col2im + im2col + matmul_nt_splitk + bias_grad
 * + 3x accumulate (src/cuda/nn/conv.rs:298-324). */
int nrs_conv2d_bwd(nrs_ctx* ctx, const float* x, const float* w, const float* dy,
                   float* dx, float* dw, float* db,
                   int n, int ci, int h, int wd, int co, int kh, int kw, int stride, int pad,
                   int accumulate);

/* Operand caching for callers that drive the convolutions operator by operator.  The tensor-core
 * kernels read an activation as channels-last TF32 planes; nrs_conv2d_fwd / _bwd make them from the
 * NCHW tensor on every call.  A caller that knows a tensor is read more than once (x by the forward
 * pass and by the weight gradient; dy by both gradients) has them made once:
 * nrs_planes_cache(t, [n,c,h,w]) stages the planes of t's CURRENT contents into memory the library
 * owns and every later convolution call that is given t uses them; nrs_planes_drop(t) forgets them
 * (required before t's contents change or its memory is freed; dropping an unknown pointer is not an
 * error).  No-ops (NRS_OK) in FP32 mode and for channel counts the tensor-core path does not take.
 * The node-level graph and the trainer do this by themselves.  No reference counterpart: its
 * im2col + GEMM reads f32 tensors directly (src/cuda/nn/conv.rs:244-324). */
int nrs_planes_cache(nrs_ctx* ctx, const float* t, int n, int c, int h, int w);
int nrs_planes_drop(nrs_ctx* ctx, const float* t);

/* ------------------------------------------------------------ elementwise -- */

/* out = a + b (src/cuda/graph/add.rs:20-24); out[r,c] = a[r,c] + bias[c]
 * (:26-30); acc += src (src/cuda/runtime.rs:14-18). */
int nrs_add(nrs_ctx* ctx, const float* a, const float* b, float* out, size_t n);
int nrs_bias_add(nrs_ctx* ctx, const float* a, const float* bias, float* out, int rows, int cols);
int nrs_accumulate(nrs_ctx* ctx, float* acc, const float* src, size_t n);
/* out[c] (+)= sum_r g[r,c]  — sum_axis0 (src/cuda/reduce.rs:13-20). */
int nrs_sum_axis0(nrs_ctx* ctx, const float* g, float* out, int rows, int cols, int accumulate);
/* Same result as nrs_sum_axis0, for callers that must not allocate device memory
 * (inside a stream capture, in a real-time loop, or under a host framework that
 * owns all device memory).  It has no counterpart in the reference.  The split
 * partial sums go to a fixed 1 MiB array built into the library instead of the
 * context's cudaMalloc'ed workspace, so the call never reaches cudaMalloc/cudaFree.
 * Limits and caveats: cols <= 8192 (larger is refused with NRS_ERR_UNSUPPORTED);
 * the first call on a device looks up the array's device address
 * (cudaGetSymbolAddress) — make that first call before any stream capture; all
 * calls on a device share the one array, so two calls that overlap on the GPU
 * (different streams) race — serialise them. */
int nrs_sum_axis0_static(nrs_ctx* ctx, const float* g, float* out, int rows, int cols, int accumulate);
/* out[c] (+)= sum_{n,p} g[n,c,p] — conv2d_bias_grad (src/cuda/nn/conv.rs:78-90). */
int nrs_channel_sum(nrs_ctx* ctx, const float* g, float* out, int n, int c, int plane, int accumulate);
/* vrelu / relu_grad (src/cuda/graph/relu.rs:17-27): y=max(0,x); dx (+)= g*[x>0]. */
int nrs_relu_fwd(nrs_ctx* ctx, const float* x, float* y, size_t n);
int nrs_relu_bwd(nrs_ctx* ctx, const float* x, const float* g, float* dx, size_t n, int accumulate);
/* vgelu / gelu_grad (src/cuda/graph/gelu.rs:12-32), tanh approximation. */
int nrs_gelu_fwd(nrs_ctx* ctx, const float* x, float* y, size_t n);
int nrs_gelu_bwd(nrs_ctx* ctx, const float* x, const float* g, float* dx, size_t n, int accumulate);
/* vscale / scale_grad (src/cuda/graph/scale.rs:11-19): y = x*s ; dx (+)= g*s. */
int nrs_scale(nrs_ctx* ctx, const float* x, float* y, size_t n, float s, int accumulate);
/* transpose2d (src/cuda/graph/transpose.rs:12-23): batched swap of the last two dims;
 * y[b,j,i] (+)= x[b,i,j]. */
int nrs_transpose(nrs_ctx* ctx, const float* x, float* y, int batch, int rows, int cols, int accumulate);
/* slice_fwd / slice_bwd (src/cuda/graph/slice_cols.rs:12-29):
 * fwd: y[r,c] = x[r,c0+c] for c in [0,c1-c0); bwd: dx[r,c0+c] (+)= g[r,c]. */
int nrs_slice_cols_fwd(nrs_ctx* ctx, const float* x, float* y, int rows, int total, int c0, int c1);
int nrs_slice_cols_bwd(nrs_ctx* ctx, const float* g, float* dx, int rows, int total, int c0, int c1, int accumulate);
/* concat_write / concat_read (src/cuda/graph/concat_cols.rs:12-29). */
int nrs_concat_write(nrs_ctx* ctx, const float* part, float* out, int rows, int total, int off, int pw);
int nrs_concat_read(nrs_ctx* ctx, const float* g, float* dpart, int rows, int total, int off, int pw, int accumulate);

/* ---------------------------------------------------------------- pooling -- */

/* maxpool_forward / maxpool_backward (src/cuda/nn/maxpool.rs:19-55): k x k
 * windows, stride s, no padding, first maximum wins; argmax[N,C,oh,ow] holds
 * the flat input index (int32) and may be NULL in the forward call.
 * Backward: dx (+)= scatter of g through argmax.  With accumulate == 0 dx is
 * fully overwritten (non-winners get 0).  For k == s the backward is a
 * gather (no atomics, deterministic); otherwise dx is zeroed/kept and an
 * atomicAdd scatter runs, as in the reference. */
int nrs_maxpool_fwd(nrs_ctx* ctx, const float* x, float* y, int32_t* argmax,
                    int n, int c, int h, int w, int k, int stride);
int nrs_maxpool_bwd(nrs_ctx* ctx, const float* g, const int32_t* argmax, float* dx,
                    int n, int c, int h, int w, int k, int stride, int accumulate);

/* --------------------------------------------------- layernorm / softmax -- */

/* ln_forward (src/cuda/nn/normalization.rs:14-41): per row of `f` features,
 * biased variance, eps inside the sqrt; saves xhat[rows,f] and istd[rows]. */
int nrs_layernorm_fwd(nrs_ctx* ctx, const float* x, const float* gamma, const float* beta,
                      float* y, float* xhat, float* istd, int rows, int f, float eps);
/* ln_dx + ln_reduce (src/cuda/nn/normalization.rs:43-78): dx (+)=, dgamma (+)=,
 * dbeta (+)=; dx may be NULL. */
int nrs_layernorm_bwd(nrs_ctx* ctx, const float* g, const float* xhat, const float* istd,
                      const float* gamma, float* dx, float* dgamma, float* dbeta,
                      int rows, int f, int accumulate_dx, int accumulate_params);
/* The residual add that precedes a LayerNorm in the transformer block
 * (add + layernorm, src/cuda/nn/transformer_block.rs:33-34,41-42) folded into the same two
 * kernels: forward normalises a + b without writing the sum; backward hands the one input
 * gradient to both addends (da and db, each written or added to; either may be NULL). */
int nrs_layernorm_residual_fwd(nrs_ctx* ctx, const float* a, const float* b, const float* gamma, const float* beta,
                               float* y, float* xhat, float* istd, int rows, int f, float eps);
int nrs_layernorm_residual_bwd(nrs_ctx* ctx, const float* g, const float* xhat, const float* istd, const float* gamma,
                               float* da, float* db, float* dgamma, float* dbeta, int rows, int f, int accumulate_da,
                               int accumulate_db, int accumulate_params);
/* softmax_forward / softmax_backward (src/cuda/graph/softmax.rs:12-35).  The
 * backward takes the forward OUTPUT y: dx (+)= y*(g - sum(y*g)). */
int nrs_softmax_fwd(nrs_ctx* ctx, const float* x, float* y, int rows, int width);
int nrs_softmax_bwd(nrs_ctx* ctx, const float* y, const float* g, float* dx, int rows, int width, int accumulate);

/* ------------------------------------------------ batchnorm / dropout -- */

/* bn2d_stats + bn2d_normalize (src/cuda/nn/batchnorm2d.rs:22-75) and, with hw == 1,
 * bn_stats + bn_normalize (src/cuda/nn/batchnorm.rs:20-63): x is [n, c, hw],
 * statistics pool over n and hw per channel.  training != 0: batch mean and biased
 * variance; running = momentum*running + (1-momentum)*batch (updated in place).
 * training == 0: the running statistics normalise.  Saves xhat[n,c,hw] (may be
 * NULL when no backward follows) and istd[c] = 1/sqrt(var + eps). */
int nrs_batchnorm_fwd(nrs_ctx* ctx, const float* x, const float* gamma, const float* beta,
                      float* running_mean, float* running_var, float* y, float* xhat, float* istd,
                      int n, int c, int hw, float eps, float momentum, int training);
/* bn2d_reduce + bn2d_dx (src/cuda/nn/batchnorm2d.rs:77-117; batchnorm.rs:65-108):
 * dgamma (+)= sum g*xhat, dbeta (+)= sum g, dx (+)= istd*(g*gamma - gamma*dbeta/N -
 * xhat*gamma*dgamma/N) in training, g*gamma*istd in evaluation.  dx may be NULL;
 * dgamma and dbeta are given together or not at all. */
int nrs_batchnorm_bwd(nrs_ctx* ctx, const float* g, const float* xhat, const float* istd,
                      const float* gamma, float* dx, float* dgamma, float* dbeta,
                      int n, int c, int hw, int training, int accumulate_dx, int accumulate_params);
/* The same two passes with the ReLU that follows the layer in the reference's
 * models (examples/cifar_cuda.rs:44-48: conv -> batchnorm2d -> relu) folded in:
 * act = NRS_ACT_RELU writes y = max(0, gamma*xhat + beta), and the backward pass
 * masks the incoming gradient where that output was not positive (relu_backward,
 * src/cuda/graph/relu.rs:28-45: strict >) before the BatchNorm arithmetic.  The
 * mask is recomputed from xhat, gamma and beta with the forward pass's own
 * expression, so no activation or mask tensor is stored or read.  act =
 * NRS_ACT_NONE is nrs_batchnorm_fwd / _bwd. */
int nrs_batchnorm_act_fwd(nrs_ctx* ctx, const float* x, const float* gamma, const float* beta,
                          float* running_mean, float* running_var, float* y, float* xhat, float* istd,
                          int n, int c, int hw, float eps, float momentum, int training, int act);
int nrs_batchnorm_act_bwd(nrs_ctx* ctx, const float* g, const float* xhat, const float* istd,
                          const float* gamma, const float* beta, float* dx, float* dgamma, float* dbeta,
                          int n, int c, int hw, int training, int accumulate_dx, int accumulate_params, int act);
/* mask_mul (src/cuda/nn/dropout.rs:17-22) with hw == 1 and mask_mul_channels
 * (src/cuda/nn/dropout2d.rs:18-27) with hw = h*w: out (+)= a * mask[i / hw].  The
 * same call routes the gradient in the backward pass. */
int nrs_mask_mul(nrs_ctx* ctx, const float* a, const float* mask, float* out, size_t total, int hw, int accumulate);
/* The mask the reference draws on the host (dropout.rs:45-48: 0 with probability
 * p, else 1/(1-p)), generated on the device instead: Philox-4x32-10 keyed by the
 * context's seed; element i is word i%4 of counter block (offset + i/4),
 * u = (word >> 8) * 2^-24, mask = u < p ? 0 : 1/(1-p).  Each call consumes
 * ceil(count/4) counter blocks.  nrs_rng_seed sets the seed and rewinds the
 * offset to 0; nrs_rng_offset reads the next unused block. */
int nrs_dropout_mask(nrs_ctx* ctx, float* mask, size_t count, float p);
int nrs_rng_seed(nrs_ctx* ctx, uint64_t seed);
int nrs_rng_offset(nrs_ctx* ctx, uint64_t* offset);

/* ------------------------------------------------------- input pipeline -- */

/* `augment` of examples/cifar_cuda.rs:146-169 on a resident batch x[n,c,h,w] -> y:
 * per image a horizontal flip (probability 1/2, when flip != 0) and a shift by
 * (dx, dy) in [-max_shift, max_shift] with zero fill: y[ch,yy,xx] = x[ch, yy-dy,
 * flip ? w-1-(xx-dx) : xx-dx].  Draws: Philox block (offset + image) of the
 * context's stream (nrs_rng_seed): flip = top bit of word 0, dx = floor(u(word 1)
 * * (2*max_shift+1)) - max_shift, dy likewise from word 2.  Consumes n blocks.
 * x and y must not alias. */
int nrs_augment_flip_shift(nrs_ctx* ctx, const float* x, float* y, int n, int c, int h, int w, int max_shift, int flip);
/* One-hot f32 target rows from int32 class indices (what the reference's loaders
 * hand to cross_entropy): out[b, k] = (labels[b] == k).  An index outside
 * [0, classes) gives an all-zero row. */
int nrs_onehot(nrs_ctx* ctx, const int32_t* labels, float* out, int batch, int classes);

/* ------------------------------------------------------------ transformer -- */

/* embed_forward / embed_backward (src/cuda/nn/embedding.rs:13-30): row gather
 * out[t,:] = weight[idx[t],:] for `tokens` int32 device indices, and the
 * scatter-add of the gradient back into dweight[vocab,dim] (+)=.  The backward
 * walks tokens in order per vocabulary row: deterministic, unlike the
 * reference's atomicAdd.  The reference asserts on the host that indices lie in
 * [0, vocab) (embedding.rs:55-57); these indices live on the device, so the kernel
 * checks instead: an index outside the range is not dereferenced, its output row
 * is zeros, and the next nrs_sync / nrs_d2h returns NRS_ERR_ARG. */
int nrs_embedding_fwd(nrs_ctx* ctx, const float* weight, const int32_t* idx, float* out, int tokens, int dim, int vocab);
/* The same gather with PositionalEncoding::forward (src/cuda/nn/positional.rs:36-44) folded in:
 * out[t, :] = weight[idx[t], :] + pos_table[t % seq, :] for tokens laid out [batch, seq]. */
int nrs_embedding_pos_fwd(nrs_ctx* ctx, const float* weight, const int32_t* idx, const float* pos_table, float* out,
                          int tokens, int seq, int dim, int vocab);
int nrs_embedding_bwd(nrs_ctx* ctx, const float* g, const int32_t* idx, float* dweight, int tokens, int dim,
                      int vocab, int accumulate);
/* Causal mask over [batch, s, s] attention scores.  No reference counterpart (the
 * reference has no mask).  backward == 0: y = (j > i) ? -1e30 : x;
 * backward != 0: y (+)= (j > i) ? 0 : x. */
int nrs_causal_mask(nrs_ctx* ctx, const float* x, float* y, int batch, int s, int backward, int accumulate);
/* Fused attention core for short sequences (nrs_attention_supported: seq <= 128, d_head <= 32).
 * q, k, v, out, dout, dq, dk, dv: [batch, seq, heads*d_head] (head h = columns [h*d_head, (h+1)*d_head));
 * probs: [batch*heads, seq, seq], written by the forward pass and read by the backward pass.
 *   out = softmax(q k^T / sqrt(d_head), masked above the diagonal when causal) v     per (batch, head)
 * i.e. src/cuda/nn/attention.rs:23-32 applied to every head of src/cuda/nn/multihead.rs:57-85 at once,
 * without the slice / transpose / scale / concat passes.  The backward pass writes (acc_* == 0) or
 * adds to (acc_* != 0) dq, dk, dv.  Deterministic. */
int nrs_attention_supported(int seq, int d_head);
int nrs_attention_fwd(nrs_ctx* ctx, const float* q, const float* k, const float* v, float* out, float* probs, int batch,
                      int seq, int heads, int d_head, int causal);
int nrs_attention_bwd(nrs_ctx* ctx, const float* q, const float* k, const float* v, const float* probs, const float* dout,
                      float* dq, float* dk, float* dv, int batch, int seq, int heads, int d_head, int acc_q, int acc_k,
                      int acc_v);
/* Head split / merge for multi-head attention: to_heads != 0 maps x[batch, s, heads*d_head] to
 * y[batch*heads, s, d_head] (head h = column slice [h*d_head, (h+1)*d_head), exactly the slices
 * src/nn/multihead.rs:94-107 takes one by one); to_heads == 0 is the inverse, i.e. the
 * reference's concat_cols of the per-head results.  y (+)= when accumulate. */
int nrs_permute_heads(nrs_ctx* ctx, const float* x, float* y, int batch, int s, int heads, int d_head, int to_heads,
                      int accumulate);

/* ------------------------------------------------------------------- loss -- */

/* ce_forward (src/cuda/loss/cross_entropy.rs:18-36, 74-98): writes
 * loss_dev[0] = sum_b(-sum_c t*log_softmax(x)) / divisor on the device (no
 * host round trip).  row_loss[batch] is optional scratch-free output of the
 * per-row terms.  The reference divides by the row count; data-parallel shards
 * pass the global batch. */
int nrs_ce_fwd(nrs_ctx* ctx, const float* logits, const float* target, float* loss_dev,
               float* row_loss, int batch, int classes, int divisor);
/* ce_backward (src/cuda/loss/cross_entropy.rs:38-57, 107-128): overwrites
 * grad = (softmax(x) - t) / divisor. */
int nrs_ce_bwd(nrs_ctx* ctx, const float* logits, const float* target, float* grad,
               int batch, int classes, int divisor);
/* Both in one pass over the logits. */
int nrs_ce_fwd_bwd(nrs_ctx* ctx, const float* logits, const float* target, float* loss_dev,
                   float* grad, int batch, int classes, int divisor);

/* nrs_ce_fwd_bwd for targets given as one int32 class index per row instead of one-hot rows
 * (the same values as running it on nrs_onehot's output: an index outside [0, classes) is an
 * all-zero target row); the dense target tensor is neither built nor read. */
int nrs_ce_fwd_bwd_indexed(nrs_ctx* ctx, const float* logits, const int32_t* labels, float* loss_dev, float* grad,
                           int batch, int classes, int divisor);

/* -------------------------------------------------------------- optimizer -- */

/* One AdamW update over flat vectors of n elements, as the `adamw` kernel
 * (src/cuda/optim/adamw.rs:19-35) but one launch for the whole model:
 *   m = b1*m + (1-b1)*g ; v = b2*v + (1-b2)*g*g ;
 *   p = p - lr*(m/bc1)/(sqrt(v/bc2)+eps) - lr*wd*p        (pre-update p)
 * with g = grad_scale*grad.  bc1 = 1-b1^(t+1), bc2 = 1-b2^(t+1) are computed by
 * the caller exactly as the reference does on the host (:77-78). */
int nrs_adamw_step(nrs_ctx* ctx, float* p, const float* grad, float* m, float* v, size_t n,
                   float lr, float beta1, float beta2, float eps, float wd,
                   float bc1, float bc2, float grad_scale);

#ifdef __cplusplus
}
#endif
#endif /* NRS_H */
