/*
 * nrs_graph.h — node-level C ABI of libnrs_b200.so.
 *
 * The reference's GPU path is used through Rust functions over graph nodes
 * (`Rc<RefCell<Node>>`): cuda::runtime, cuda::graph, cuda::nn, cuda::loss,
 * cuda::optim.  This header exports the same operations over opaque node
 * handles so a caller without a C++ compiler (a Rust shim, a ctypes test) can
 * run a reference-style program: build nodes, move them to the GPU, call
 * operators that return new nodes, seed a gradient, run backward_graph, step an
 * optimizer.  Each entry names the reference function it mirrors.
 *
 * Status codes, error text and stream semantics are those of nrs.h.  Handles
 * are reference counted: every `*_out` handle must be passed to
 * nrs_node_release once (releasing a node does not free tensors that other
 * live nodes still use as parents).
 */
#ifndef NRS_GRAPH_H
#define NRS_GRAPH_H

#include "nrs.h"

#ifdef __cplusplus
extern "C" {
#endif

typedef struct nrs_node nrs_node;
typedef struct nrs_adamw nrs_adamw;
typedef struct nrs_trainer nrs_trainer;

/* Node::new(data, shape) — src/autograd/node.rs:60-74.  host_data: host f32,
 * may be NULL for a node that only receives device data later. */
int nrs_node_new(nrs_ctx* ctx, const float* host_data, const int64_t* shape, int ndim, nrs_node** out);
int nrs_node_release(nrs_node* n);
int nrs_node_ndim(const nrs_node* n);
int nrs_node_shape(const nrs_node* n, int64_t* shape_out, int capacity);
int64_t nrs_node_len(const nrs_node* n);
/* Node.requires_grad — src/autograd/node.rs:33-36,45. */
int nrs_node_set_requires_grad(nrs_node* n, int flag);
/* Replaces the node's HOST data (what the reference does by assigning `node.borrow_mut().data`);
 * the next nrs_to_cuda uploads it into the node's existing device buffer. */
int nrs_node_set_data(nrs_node* n, const float* host_data);
/* Device pointers of a resident node (NULL when absent).  The library caches re-laid-out copies
 * of a tensor that a convolution has read (its tensor-core operand planes); a caller that writes
 * new values through nrs_node_data_ptr must call nrs_node_invalidate afterwards, or use a fresh
 * node.  nrs_to_cuda invalidates by itself. */
float* nrs_node_data_ptr(nrs_node* n);
float* nrs_node_grad_ptr(nrs_node* n);
int nrs_node_invalidate(nrs_node* n);

/* cuda::runtime — src/cuda/runtime.rs:39-124. */
int nrs_to_cuda(nrs_node* n);
int nrs_to_host(nrs_node* n, float* host_out);
int nrs_set_grad(nrs_node* n, const float* host_grad);
int nrs_read_grad(nrs_node* n, float* host_out);
int nrs_zero_grad(nrs_node* const* params, int count);
/* Moves resident parameters into one contiguous block (values kept) so the
 * optimizer runs as one launch.  No reference counterpart. */
int nrs_flatten_params(nrs_node* const* params, int count);

/* cuda::graph — src/cuda/graph/{matmul,add,relu,gelu,reshape,softmax,bmm,
 * transpose,scale,slice_cols,concat_cols}.rs */
int nrs_op_matmul(nrs_node* a, nrs_node* b, nrs_node** out);
int nrs_op_add(nrs_node* a, nrs_node* b, nrs_node** out);
int nrs_op_relu(nrs_node* x, nrs_node** out);
int nrs_op_gelu(nrs_node* x, nrs_node** out);
int nrs_op_reshape(nrs_node* x, const int64_t* shape, int ndim, nrs_node** out);
int nrs_op_softmax(nrs_node* x, nrs_node** out);
int nrs_op_bmm(nrs_node* a, nrs_node* b, nrs_node** out);
int nrs_op_transpose(nrs_node* x, nrs_node** out);
int nrs_op_scale(nrs_node* x, float s, nrs_node** out);
int nrs_op_slice_cols(nrs_node* x, int64_t col_start, int64_t col_end, nrs_node** out);
int nrs_op_concat_cols(nrs_node* const* parts, int count, nrs_node** out);

/* cuda::nn — src/cuda/nn/{conv,maxpool,flatten,normalization,linear}.rs */
int nrs_op_conv2d(nrs_node* input, nrs_node* weight, nrs_node* bias, int64_t stride, int64_t pad, nrs_node** out);
int nrs_op_maxpool2d(nrs_node* input, int64_t kernel, int64_t stride, nrs_node** out);
int nrs_op_flatten(nrs_node* x, nrs_node** out);
int nrs_op_layernorm(nrs_node* x, nrs_node* gamma, nrs_node* beta, float eps, nrs_node** out);
/* batchnorm (src/cuda/nn/batchnorm.rs:110-232, x [batch, features]) and batchnorm2d
 * (src/cuda/nn/batchnorm2d.rs:130-232, x [batch, channels, h, w]).  running_mean and
 * running_var are resident nodes of length channels; training != 0 updates them in
 * place (running = momentum*running + (1-momentum)*batch). */
int nrs_op_batchnorm(nrs_node* x, nrs_node* gamma, nrs_node* beta, nrs_node* running_mean, nrs_node* running_var,
                     float momentum, float eps, int training, nrs_node** out);
int nrs_op_batchnorm2d(nrs_node* x, nrs_node* gamma, nrs_node* beta, nrs_node* running_mean, nrs_node* running_var,
                       float momentum, float eps, int training, nrs_node** out);
/* Either of the two (chosen by the input's rank, 2 or 4) with the activation that
 * follows it fused (enum nrs_act: NONE or RELU), like nrs_op_conv2d_act. */
int nrs_op_batchnorm_act(nrs_node* x, nrs_node* gamma, nrs_node* beta, nrs_node* running_mean, nrs_node* running_var,
                         float momentum, float eps, int training, int act, nrs_node** out);
/* dropout (src/cuda/nn/dropout.rs:31-84) and dropout2d (src/cuda/nn/dropout2d.rs:37-).
 * training == 0 hands back the input node itself (one more reference on it).  `mask`
 * NULL draws the mask on the device (nrs_dropout_mask: the context's seed and
 * counter); a resident mask node (one value per element, or per (sample, channel)
 * plane for dropout2d; values 0 or 1/(1-p)) is used as given, which is how a caller
 * replays masks drawn elsewhere. */
int nrs_op_dropout(nrs_node* x, float p, int training, nrs_node* mask, nrs_node** out);
int nrs_op_dropout2d(nrs_node* x, float p, int training, nrs_node* mask, nrs_node** out);
/* Fused x@W+b -> activation and conv+bias -> activation (enum nrs_act). */
int nrs_op_linear_act(nrs_node* x, nrs_node* w, nrs_node* b, int act, nrs_node** out);
int nrs_op_conv2d_act(nrs_node* input, nrs_node* weight, nrs_node* bias, int64_t stride, int64_t pad, int act,
                      nrs_node** out);

/* Transformer pieces — src/cuda/nn/{embedding,positional,attention,multihead,
 * transformer_block}.rs.
 * Embedding::forward(indices) -> [count, dim]; the batched form -> [batch, seq, dim]
 * (the reference has it on the CPU only, src/nn/embedding.rs:60-113).  `indices`
 * is a HOST array of token ids, checked against the weight's row count. */
int nrs_op_embedding(nrs_node* weight, const int32_t* indices_host, int64_t count, nrs_node** out);
int nrs_op_embedding_batch(nrs_node* weight, const int32_t* indices_host, int64_t batch, int64_t seq, nrs_node** out);
/* PositionalEncoding::new(d_model, max_len): the resident sinusoidal table, and
 * forward(x) = x + table[:seq] for x [seq, d] or [batch, seq, d]. */
int nrs_positional_new(nrs_ctx* ctx, int64_t d_model, int64_t max_len, nrs_node** table_out);
int nrs_op_positional(nrs_node* x, nrs_node* table, nrs_node** out);
/* attention_batch(q, k, v) on [batch, seq, d_head]; causal != 0 masks j > i
 * (an extension: the reference has no mask). */
int nrs_op_causal_mask(nrs_node* scores, nrs_node** out);
int nrs_op_attention_batch(nrs_node* q, nrs_node* k, nrs_node* v, int causal, nrs_node** out);
/* MultiHeadAttention::forward_batch(x) with weights [d,d] and no biases. */
int nrs_op_mha(nrs_node* x, nrs_node* w_q, nrs_node* w_k, nrs_node* w_v, nrs_node* w_o, int64_t num_heads,
               int causal, nrs_node** out);
/* TransformerBlock::forward / forward_no_final_norm.  params: 12 nodes in the
 * order w_q, w_k, w_v, w_o, norm1.gamma, norm1.beta, norm2.gamma, norm2.beta,
 * ff1.weights, ff1.bias, ff2.weights, ff2.bias (the reference's parameters()
 * order, src/nn/transformer_block.rs:58-66).  act: NRS_ACT_RELU as the reference,
 * or NRS_ACT_GELU. */
int nrs_op_transformer_block(nrs_node* x, nrs_node* const* params, int64_t num_heads, float eps, int act,
                             int causal, int final_norm, nrs_node** out);

/* cuda::loss — src/cuda/loss/cross_entropy.rs:74-128. */
int nrs_cross_entropy(nrs_node* pred, nrs_node* target, float* loss_out);
int nrs_cross_entropy_backward(nrs_node* pred, nrs_node* target);

/* autograd::node::backward_graph — src/autograd/node.rs:113-126. */
int nrs_backward_graph(nrs_node* root);
/* One node's own backward closure (what backward_graph calls for it, src/autograd/node.rs:121-124):
 * lets a caller that keeps the reference's graph walk on its side of the boundary (a Rust
 * `Node` whose backward_fn is this call) drive the same closures in its own topological order.
 * A node without a closure (a leaf, a reshape) is a no-op. */
int nrs_node_backward(nrs_node* n);

/* cuda::optim::AdamW — src/cuda/optim/adamw.rs:54-143. */
int nrs_adamw_new(nrs_ctx* ctx, float lr, float beta1, float beta2, float eps, float weight_decay, nrs_adamw** out);
int nrs_adamw_free(nrs_adamw* opt);
int nrs_adamw_step_nodes(nrs_adamw* opt, nrs_node* const* params, int count);
int64_t nrs_adamw_t(const nrs_adamw* opt);
/* export_state: number of moment tensors (2 x parameters, 0 before the first
 * step), the length of tensor i, and a copy of tensor i to the host. */
int nrs_adamw_state_count(const nrs_adamw* opt);
int64_t nrs_adamw_state_len(const nrs_adamw* opt, int i);
int nrs_adamw_state_get(const nrs_adamw* opt, int i, float* host_out);
/* import_state(t, moments): `lens[i]` floats at `moments[i]`, all m's then all v's. */
int nrs_adamw_import_state(nrs_adamw* opt, int64_t t, const float* const* moments, const int64_t* lens, int count);

/* ------------------------------------------------------------- trainer -- */
/* The reference leaves the training loop to user code: to_cuda(batch),
 * zero_grad, forward, cross_entropy(+_backward), backward_graph, optimizer.step
 * (examples/cifar_cuda.rs:267-286, examples/mnist_cuda_cnn.rs:254-275).  The
 * trainer runs that same loop natively for a sequential model, so a whole step
 * is one call (no per-operator crossing of the language boundary), and adds
 * what the reference does not have: data-parallel gradient all-reduce. */
enum nrs_layer_kind {
  NRS_LAYER_CONV = 0,     /* a=c_in b=c_out c=kernel d=stride e=pad              */
  NRS_LAYER_RELU = 1,
  NRS_LAYER_MAXPOOL = 2,  /* a=kernel b=stride                                   */
  NRS_LAYER_FLATTEN = 3,
  NRS_LAYER_LINEAR = 4,   /* a=in b=out                                          */
  NRS_LAYER_GELU = 5,
  NRS_LAYER_BATCHNORM = 6, /* a=channels (features after flatten): BatchNorm2d on [C,H,W], BatchNorm on [F];
                              momentum 0.9, eps 1e-5 unless nrs_trainer_set_batchnorm says otherwise */
  NRS_LAYER_DROPOUT = 7,   /* a=drop probability in parts per million (500000 = 0.5) */
  NRS_LAYER_DROPOUT2D = 8, /* a=as above; whole (sample, channel) planes             */
  /* Token models.  An embedding layer must be the first layer: the model then reads int32 token ids
   * [batch, seq] (in_shape = {seq}) through the *_tokens entry points, activations are [batch, seq, d],
   * a linear layer acts on every position, and the loss runs over batch*seq rows. */
  NRS_LAYER_EMBEDDING = 9, /* a=vocab b=d_model c=max_len: Embedding::forward_batch (src/nn/embedding.rs:60-113)
                              followed, when c > 0, by PositionalEncoding::new(d_model, max_len).forward
                              (src/cuda/nn/positional.rs:18-44), both in one gather kernel               */
  NRS_LAYER_TRANSFORMER_BLOCK = 10, /* a=d_model b=num_heads c=d_ff d=activation (NRS_ACT_RELU as
                              src/cuda/nn/transformer_block.rs:28-60, or NRS_ACT_GELU) e=flags: bit 0 causal
                              attention mask, bit 1 forward_no_final_norm.  Adds the block's 12 parameters in
                              the reference's parameters() order (see nrs_op_transformer_block)             */
  NRS_LAYER_LAYERNORM = 11 /* a=features; eps 1e-5; adds [gamma, beta]                */
};
typedef struct nrs_layer_spec { int kind, a, b, c, d, e; } nrs_layer_spec;

/* in_shape: per-sample input shape (e.g. {3,32,32}).  fuse != 0 folds a ReLU
 * that follows a conv/linear layer into that layer's kernel.  Parameters are
 * created zero-filled in layer order [w0,b0,w1,b1,...] inside one flat block
 * (a batchnorm layer adds [gamma,beta]); fill them with nrs_trainer_set_param.
 * The running statistics of batchnorm layers are buffers [mean0,var0,mean1,...],
 * created at 0 / 1, updated by training-mode steps, never touched by the
 * optimizer (examples/cifar_cuda.rs:44-66 keeps them out of `trainable`). */
int nrs_trainer_create(nrs_ctx* ctx, const nrs_layer_spec* layers, int n_layers, const int64_t* in_shape,
                       int in_ndim, int classes, float lr, float beta1, float beta2, float eps,
                       float weight_decay, int fuse, nrs_trainer** out);
int nrs_trainer_free(nrs_trainer* t);
int nrs_trainer_param_count(const nrs_trainer* t);
int64_t nrs_trainer_param_len(const nrs_trainer* t, int i);
int nrs_trainer_set_param(nrs_trainer* t, int i, const float* host);
int nrs_trainer_get_param(nrs_trainer* t, int i, float* host_out);
int nrs_trainer_get_grad(nrs_trainer* t, int i, float* host_out);
int nrs_trainer_buffer_count(const nrs_trainer* t);
int64_t nrs_trainer_buffer_len(const nrs_trainer* t, int i);
int nrs_trainer_set_buffer(nrs_trainer* t, int i, const float* host);
int nrs_trainer_get_buffer(nrs_trainer* t, int i, float* host_out);
/* Training (default) or evaluation mode of the batchnorm and dropout layers
 * (`training` of src/cuda/nn/batchnorm2d.rs:139 and dropout.rs:31). */
int nrs_trainer_set_training(nrs_trainer* t, int training);
int nrs_trainer_set_batchnorm(nrs_trainer* t, float momentum, float eps);
/* zero_grad + forward + cross-entropy + backward (no optimizer step).
 * x_host [batch, in_shape...] and target_host [batch, classes] (one-hot f32) are
 * HOST buffers copied to the device inside the call; loss_out (host) may be
 * NULL, otherwise the call waits for the loss. */
int nrs_trainer_forward_backward(nrs_trainer* t, const float* x_host, const float* target_host, int batch,
                                 float* loss_out);
/* A full training step: the above plus the gradient all-reduce (when data
 * parallel) and one fused AdamW update. */
int nrs_trainer_step(nrs_trainer* t, const float* x_host, const float* target_host, int batch, float* loss_out);
/* The same step with its input copy taken off the critical path (the reference
 * uploads synchronously at the top of every step, src/cuda/runtime.rs:43).
 * nrs_trainer_stage_next starts an asynchronous copy of a batch from host memory
 * (pinned, for the copy to overlap) into the idle one of two device slots on a
 * copy stream and returns at once; nrs_trainer_step_staged runs a full training
 * step on the oldest staged batch as soon as its copy has landed.  Staging batch
 * i+1 before stepping batch i overlaps the copy with the step; at most two
 * batches can be staged and unconsumed (a third is refused with NRS_ERR_ARG).
 * The host buffers must stay valid and unchanged until the step that consumes
 * them has been issued and the stream synchronised (loss_out != NULL does that). */
int nrs_trainer_stage_next(nrs_trainer* t, const float* x_host, const float* target_host, int batch);
int nrs_trainer_step_staged(nrs_trainer* t, float* loss_out);
/* The same step with the loss read one step behind: the step is issued, an asynchronous copy of ITS loss
 * into a pinned slot is queued behind it, and the call returns the loss of the PREVIOUS lagged step
 * (*have_prev = 0 on the first call, when there is none) after waiting for that earlier copy only.  The
 * host thus stays one step ahead of the device, which never idles while the next step is being enqueued
 * (a read-back of the step just issued drains the stream first: a fifth of the step at small batches).
 * Every step's loss is still read, in order; nrs_trainer_last_loss returns the newest one (and is where
 * a device-side error of a lagged step is reported).  Under data parallelism the wait runs through the
 * group's deadline.  The reference reads its loss synchronously every step
 * (src/cuda/loss/cross_entropy.rs:96-97). */
int nrs_trainer_step_staged_lagged(nrs_trainer* t, float* prev_loss_out, int* have_prev);
/* As nrs_trainer_stage_next with int32 class indices instead of one-hot rows
 * (batch * 4 bytes over the bus instead of batch * classes * 4); the loss kernel
 * reads them directly (nrs_ce_fwd_bwd_indexed). */
int nrs_trainer_stage_next_indexed(nrs_trainer* t, const float* x_host, const int32_t* labels_host, int batch);
/* On-device augmentation of staged [C,H,W] batches in training mode
 * (nrs_augment_flip_shift: shift by up to max_shift pixels, horizontal flip when
 * flip != 0; examples/cifar_cuda.rs:146-169 does this on the host before the
 * upload).  max_shift < 0 switches it off (the default). */
int nrs_trainer_set_augment(nrs_trainer* t, int max_shift, int flip);
/* Same step on inputs already resident on the device. */
int nrs_trainer_step_device(nrs_trainer* t, const float* x_dev, const float* target_dev, int batch,
                            float* loss_out);
/* The same entry points for a token model (first layer NRS_LAYER_EMBEDDING): ids is int32
 * [batch, seq]; labels is int32 [batch*seq], the class of every position (for a language model
 * the next token): the loss kernel reads the indices directly and gives the values of
 * cross_entropy on the matching one-hot rows (src/cuda/loss/cross_entropy.rs:74-98).  The loss is the mean over batch*seq rows.  An id outside
 * the vocabulary is not dereferenced; the next call that waits returns NRS_ERR_ARG. */
int nrs_trainer_forward_backward_tokens(nrs_trainer* t, const int32_t* ids_host, const int32_t* labels_host, int batch,
                                        float* loss_out);
int nrs_trainer_step_tokens(nrs_trainer* t, const int32_t* ids_host, const int32_t* labels_host, int batch, float* loss_out);
int nrs_trainer_stage_next_tokens(nrs_trainer* t, const int32_t* ids_host, const int32_t* labels_host, int batch);
int nrs_trainer_step_tokens_device(nrs_trainer* t, const int32_t* ids_dev, const int32_t* labels_dev, int batch,
                                   float* loss_out);
/* Loss of the most recent step (waits for it).  With data parallelism enabled every loss this
 * library reports (here and through loss_out) is THIS RANK'S SHARE of the global mean: the sum
 * over its shard divided by the global batch; the shares of all ranks add up to the loss a single
 * GPU would report for the whole batch. */
int nrs_trainer_last_loss(nrs_trainer* t, float* loss_out);

/* Data parallelism (no reference counterpart: the reference is single-GPU).
 * Rank 0 makes an id with nrs_dp_unique_id (128 bytes, host) and the launcher
 * broadcasts it; every rank then calls nrs_trainer_enable_dp.  Each rank feeds
 * its shard of `global_batch`; the loss/gradient are divided by global_batch so
 * the all-reduced SUM equals the single-GPU full-batch gradient.  Gradients
 * are reduced in flat buckets of about bucket_bytes on a second stream as soon
 * as backward has produced them, and each bucket's parameters are updated on that
 * stream right behind its reduce.  Every rank must describe the same model, bucket
 * size and global batch: nrs_trainer_enable_dp compares a fingerprint of them across
 * the ranks and fails with NRS_ERR_SHAPE before any gradient is exchanged.
 * Deadlines: joining the communicator and every host-side wait of a step (a call with
 * loss_out != NULL, nrs_trainer_last_loss) give up after the time-out (300 s unless
 * nrs_trainer_set_dp_timeout_ms says otherwise): the communicator is aborted, the
 * call returns NRS_ERR_TIMEOUT (or NRS_ERR_NCCL for an error NCCL reported), and the
 * trainer refuses further data-parallel steps. */
int nrs_dp_unique_id(void* id_out_128_bytes);
int nrs_trainer_enable_dp(nrs_trainer* t, int rank, int world, const void* unique_id_128_bytes,
                          int global_batch, size_t bucket_bytes);
int nrs_trainer_set_dp_timeout_ms(nrs_trainer* t, double timeout_ms);
/* Batch normalisation under data parallelism.  Off (default): every rank normalises with the mean
 * and variance of its own shard, as the reference would on one GPU with that batch
 * (src/cuda/nn/batchnorm2d.rs:22-59), so an N-GPU step is NOT the single-GPU full-batch step.
 * On: the per-channel sums of the forward pass (taken around the running mean, which all ranks share)
 * and of the backward pass are added up across the ranks together with the element counts (one small
 * all-reduce per layer and direction, in order on the compute stream), so every rank normalises with
 * the statistics of the GLOBAL batch, the running statistics stay identical on all ranks, and the
 * N-GPU step equals the single-GPU step on the full batch up to summation order.  Training mode only;
 * every rank must set the same value.  No reference counterpart (it is single-GPU). */
int nrs_trainer_set_sync_batchnorm(nrs_trainer* t, int on);
/* Random draws under data parallelism need no call: when a rank's batch is its contiguous share of the
 * global batch (nrs_dp_shard_range), its dropout masks and augmentation draws are the ones its samples
 * have in the global batch's counter stream, so N ranks reproduce a single process's draws. */

/* The same exchange for a caller's own loop over nodes (examples/cifar_cuda.rs:267-286 run on
 * several GPUs), without the trainer:
 *     nrs_dp_create(...);  nrs_bucket_register(dp, params, n, bucket_bytes);      once
 *     per step: forward, cross-entropy backward, then EITHER
 *         nrs_backward_graph_dp(logits, dp)       backward_graph that reports each parameter as soon
 *                                                 as the last node reading it has run, and waits
 *       OR nrs_dp_begin_step; the caller's own backward calls with nrs_grad_ready(dp, param) after
 *         each parameter's gradient is complete; nrs_allreduce_wait(dp)
 *     then the optimizer step (nrs_adamw_step_nodes) on the summed gradients.
 * nrs_bucket_register moves the parameters into one flat block (as nrs_flatten_params) and plans
 * buckets from the last parameter to the first.  A bucket is all-reduced (sum) on the group's own
 * stream once it and every bucket before it are complete, so every rank issues the same sequence
 * whatever order its gradients arrive in.  nrs_allreduce_wait sends what is left (a parameter that
 * received no gradient goes out as zeros) and makes the context's stream wait for the exchange; it
 * does not block the host.  nrs_dp_host_wait blocks the host until the context's stream is idle,
 * under the group's deadline (see above).  Each rank's cross-entropy must divide by the GLOBAL batch
 * (nrs_ce_fwd_bwd's divisor) for the summed gradient to be the full-batch one. */
typedef struct nrs_dp nrs_dp;
int nrs_dp_create(nrs_ctx* ctx, int rank, int world, const void* unique_id_128_bytes, int global_batch,
                  double timeout_ms, nrs_dp** out);
int nrs_dp_free(nrs_dp* dp);
int nrs_bucket_register(nrs_dp* dp, nrs_node* const* params, int count, size_t bucket_bytes);
int nrs_dp_bucket_count(const nrs_dp* dp);
int nrs_dp_begin_step(nrs_dp* dp);
int nrs_grad_ready(nrs_dp* dp, nrs_node* param);
int nrs_allreduce_wait(nrs_dp* dp);
int nrs_backward_graph_dp(nrs_node* root, nrs_dp* dp);
int nrs_dp_host_wait(nrs_dp* dp);
int nrs_dp_set_timeout_ms(nrs_dp* dp, double timeout_ms);
/* Sum of `count` floats at values_dev over all ranks, in place, on the context's stream (the loss
 * shares, a metric). */
int nrs_dp_all_reduce_sum(nrs_dp* dp, float* values_dev, size_t count);
/* Host-only helpers (usable without a GPU): sample range of a rank, and the
 * bucket boundaries (in floats, from the END of the flat gradient, the order
 * backward produces them) for given parameter lengths.  Returns the bucket
 * count; starts_out/ends_out may be NULL to only count. */
int nrs_dp_shard_range(int global_batch, int rank, int world, int* begin_out, int* end_out);
int nrs_dp_plan_buckets(const int64_t* param_lens, int n_params, size_t bucket_bytes,
                        int64_t* starts_out, int64_t* ends_out, int capacity);
/* Host-only: the 64-bit fingerprint of what all ranks must agree on (parameter lengths in order,
 * bucket size, global batch, world size), and the comparison of the ranks' fingerprints
 * (NRS_ERR_SHAPE naming the first rank that differs from rank 0).  nrs_bucket_register and
 * nrs_trainer_enable_dp run this check over the communicator; a launcher can run it earlier over
 * its own channel. */
uint64_t nrs_dp_fingerprint(const int64_t* param_lens, int n_params, size_t bucket_bytes, int global_batch, int world);
int nrs_dp_check_fingerprints(const uint64_t* fingerprints, int world);
/* Host-only: the deadline loop the data-parallel waits run on, over a caller's poll function
 * (0 = still running, 1 = finished, negative = failed; called at least once, then every
 * interval_us).  Returns NRS_OK, NRS_ERR_TIMEOUT after timeout_ms, or NRS_ERR_NCCL when poll
 * reported a failure; waited_ms_out (optional) receives the time spent. */
typedef int (*nrs_poll_fn)(void* user);
int nrs_watchdog_wait(nrs_poll_fn poll, void* user, double timeout_ms, double interval_us, double* waited_ms_out);

#ifdef __cplusplus
}
#endif
#endif /* NRS_GRAPH_H */
