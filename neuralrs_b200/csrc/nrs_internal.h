// Internal declarations shared by the translation units of libnrs_b200.so.
#pragma once

#include <cuda_runtime.h>

#include <cstdarg>
#include <cstdint>
#include <cstdio>
#include <map>
#include <string>
#include <utility>
#include <vector>

#include "nrs.h"

// Size-bucketed device memory pool.  Blocks are handed back to a free list
// keyed by their rounded size instead of being cudaFree'd, so a training loop
// whose shapes repeat stops calling cudaMalloc after its first step.  All work
// runs on one stream, so reuse right after release is ordered correctly.
struct NrsPool {
  std::multimap<size_t, void*> free_blocks;   // rounded size -> block
  std::map<void*, size_t> live;               // block -> rounded size
  size_t bytes_reserved = 0;
  static size_t round_up(size_t bytes) {
    const size_t g = bytes <= (1u << 20) ? 512 : (size_t)1 << 16;
    return (bytes + g - 1) / g * g;
  }
};

struct NrsProfRecord {
  int kind;
  double work;
  cudaEvent_t start, stop;
};

// NHWC planes of an NCHW activation, staged ahead of time by a caller that knows
// the tensor will feed several tensor-core convolutions (forward and weight gradient,
// or data and weight gradient).  lo is null unless `split` (3xTF32).
struct NrsPlanes {
  float* hi;
  float* lo;
  int split;
  // Set for the planes of a 2-D tensor [rows][cols] (cols a multiple of 32) staged for a GEMM; zero for
  // image planes, whose NHWC order is not the tensor's own row-major order.
  int rows = 0, cols = 0;
};

// Extra work a convolution kernel can fold into the epilogue that writes `out` (keyed by the
// output pointer in nrs_ctx::out_extras).  A kernel that honours the request erases the entry;
// an entry still present after the call means the caller has to do the work itself.
struct NrsOutExtras {
  const float* relu_mask_src;   // NCHW tensor of out's shape: out = relu_mask_src > 0 ? out : 0 (or null)
  float* hi;                    // NHWC TF32 planes of the (masked) result, or null
  float* lo;                    // residual plane (3xTF32), or null
};

// Request for per-tile channel sums of a convolution kernel's (masked) output, keyed by the output
// pointer in nrs_ctx::colsum_requests: the bias gradient of the layer below is then a fold of
// [rows][channels] partial sums instead of a pass over the whole gradient.  A kernel that honours
// it sets `rows` (> 0); the caller removes the entry either way.
struct NrsColsumRequest {
  float* partial;   // [cap_rows][channels]
  int cap_rows;
  int rows;         // out: rows written, 0 = not honoured
};

// Weight operand planes staged ahead of the contractions by a caller that knows its weights (the
// trainer): see weight_set.cu.  Forms: convolution forward [co][tap*ci + ci] and data gradient
// [ci][tap*co + co]; Linear W[in,out] transposed to [out][in] (B operand of x@W) and as stored
// [in][out] (B operand of dz@W^T), rows padded to a multiple of 32 floats.
enum NrsWeightForm { NRS_WF_CONV_FWD = 0, NRS_WF_CONV_DGRAD = 1, NRS_WF_LINEAR_T = 2, NRS_WF_LINEAR_ROWS = 3 };
struct NrsWeightDesc {
  const float* w;
  int form;
  int rows, K;        // linear forms: the DESTINATION's row count and reduction length
  int co, ci, taps;   // convolution forms
};
struct NrsWeightPlanes {
  float* hi;
  float* lo;          // null unless 3xTF32
  int rows, K, co, ci, taps;
};
struct NrsWeightSet {
  void* storage = nullptr;
  void* jobs_dev = nullptr;
  int n_jobs = 0;
  unsigned blocks = 0;
  bool split = false;
  bool fresh = false;   // staged since the weights last changed (the owner clears it when it updates them)
  const void* owner = nullptr;   // whoever built the set (a trainer); a different owner rebuilds it
  int mode = -1;                 // math mode it was built for
  std::map<std::pair<const void*, int>, NrsWeightPlanes> planes;
  // per job, in launch order: the weight it reads and its first block (the last entry of job_first is `blocks`)
  std::vector<const float*> job_src;
  std::vector<unsigned> job_first;
  int refreshed_jobs = 0;   // jobs restaged range by range since the last full refresh / reset (refresh_range)
};

// Cross-rank sum of a few per-channel statistics (batch normalisation under data parallelism): set by
// whoever owns a communicator (the trainer); null = statistics are per process.  Sums `count` floats at
// `dev` over all ranks in place, in order on the context's stream; every rank must make the same calls.
struct NrsStatSync {
  int (*all_reduce_sum)(void* user, float* dev, size_t count) = nullptr;
  void* user = nullptr;
};

struct nrs_ctx {
  int device = 0;
  cudaStream_t own_stream = nullptr;
  cudaStream_t stream = nullptr;
  int math_mode = NRS_MATH_3XTF32;
  int sm_count = 148;
  uint64_t launches = 0;
  std::string err;
  NrsPool pool;
  // Grow-only scratch for split-K partial sums and operand staging.
  void* workspace = nullptr;
  size_t workspace_bytes = 0;
  // Named grow-only scratch blocks (operand staging for the tensor-core kernels).
  void* ws_slot[8] = {nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr};
  size_t ws_slot_bytes[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  // Device word the tensor-core kernels set when a bounded wait runs out; read at sync points.
  int* err_flag = nullptr;
  unsigned* fold_ticket = nullptr;   // arrival counter of kernels whose last block folds the blocks' partial sums
  // Planes registered for a source tensor (keyed by its device pointer); the conv kernels
  // use them instead of staging again.  Whoever registers keeps both alive and unregisters.
  std::map<const void*, NrsPlanes> plane_hints;
  std::map<const void*, NrsPlanes> owned_planes;   // nrs_planes_cache: planes the context itself allocated
  std::map<const void*, NrsOutExtras> out_extras;
  std::map<const void*, NrsColsumRequest> colsum_requests;
  // Patch planes ([pixels][32], see conv_smallc.cu) of an image tensor, keyed by its device pointer:
  // the host graph makes them once per step for the image layer's forward pass and weight gradient
  // (`split`: bit 0 = residual plane present, bits 8.. = the padding they were made for).
  std::map<const void*, NrsPlanes> patch_hints;
  NrsWeightSet weight_set;
  // Set by a caller that has just issued a kernel whose output the NEXT tensor-core weight-gradient launch
  // does not read (see NRS_PDL_PROLOGUE): that launch may overlap it.  Consumed by the launch.
  bool independent_next = false;
  NrsStatSync stat_sync;
  // Counter-based generator state of the dropout masks (dropout.cu): seed, and the next unused counter block.
  uint64_t rng_seed = 0, rng_offset = 0;
  // A process that works on samples [shard_begin, shard_begin + shard_local) of a batch of shard_global
  // (data parallelism; set by the trainer for the duration of a step, 0 = off): per-sample random draws
  // (dropout masks, augmentation) then take the counters those samples have in the GLOBAL batch's stream
  // and the stream advances by the global batch's amount, so N processes draw what one process would.
  int shard_begin = 0, shard_local = 0, shard_global = 0;
  // Optional per-family device timing (nrs_profile_*).
  bool profiling = false;
  std::vector<NrsProfRecord> prof_records;
  std::vector<cudaEvent_t> prof_free_events;
};

// Marks, for the duration of a scope, that the kernel launched last wrote nothing the next tensor-core
// weight-gradient launch reads (nrs_ctx::independent_next).
struct NrsIndependentNext {
  nrs_ctx* c;
  NrsIndependentNext(nrs_ctx* ctx, bool on) : c(ctx) { c->independent_next = on; }
  ~NrsIndependentNext() { c->independent_next = false; }
  NrsIndependentNext(const NrsIndependentNext&) = delete;
  NrsIndependentNext& operator=(const NrsIndependentNext&) = delete;
};

// Brackets the launches issued during its lifetime with two events when
// profiling is on; free otherwise.
struct NrsProfScope {
  nrs_ctx* ctx;
  bool active = false;
  NrsProfRecord rec{};
  NrsProfScope(nrs_ctx* c, int kind, double work);
  ~NrsProfScope();
};

int nrs_fail(nrs_ctx* ctx, int code, const char* fmt, ...);
int nrs_workspace(nrs_ctx* ctx, size_t bytes, void** out);
// (the weight-gradient kernels keep their split partials in a slot of their own: they may run while the
// data gradient's K-split is still being folded out of NRS_WS_PARTIAL)
enum { NRS_WS_A_HI = 0, NRS_WS_A_LO = 1, NRS_WS_B_HI = 2, NRS_WS_B_LO = 3, NRS_WS_PARTIAL = 4, NRS_WS_WGRAD_PARTIAL = 5, NRS_WS_COUNT = 8 };
int nrs_ws_slot(nrs_ctx* ctx, int slot, size_t bytes, void** out);
int nrs_err_flag(nrs_ctx* ctx, int** out);
// Zero-initialised device counters (kNrsFoldTickets of them) for "the last block to arrive folds the partials"
// reductions; the folding block resets its counter, so consecutive launches on the context's stream can share
// them.  Slot 0 serves kernels with one counter, slots 1.. kernels with a counter per column block.
constexpr int kNrsFoldTickets = 4096;
int nrs_fold_ticket(nrs_ctx* ctx, unsigned** out);
// LayerNorm with the TF32 planes of its result written by the kernel (norm_softmax.cu).
extern "C" int nrs_layernorm_fwd_planes(nrs_ctx* ctx, const float* a, const float* b, const float* gamma, const float* beta,
                                        float* y, float* xhat, float* istd, int rows, int f, float eps, float* y_hi, float* y_lo,
                                        int* emitted);
extern "C" int nrs_layernorm_bwd_planes(nrs_ctx* ctx, const float* g, const float* xhat, const float* istd, const float* gamma,
                                        float* da, float* db, float* dgamma, float* dbeta, int rows, int f, int accumulate_da,
                                        int accumulate_db, int accumulate_params, float* d_hi, float* d_lo, int* emitted);
// TF32 planes of a batch of [rows][K] matrices (tc_stage.cu); see tc_mainloop.cuh for the layouts.
int nrs_tc_stage(nrs_ctx* ctx, const float* src, float* hi, float* lo, int rows, int K, int ldk, int batch,
                 size_t src_bstride, size_t dst_bstride, bool src_k_by_rows);
// Counter window of a per-sample draw of `count` elements (count = samples * per-sample) in blocks of four:
// first block to use and by how many blocks the stream advances.  Falls back to the plain stream (this
// process's own draws) when no shard is set, the call is not per-sample, or the shard does not start on a
// block boundary.
inline void nrs_rng_window(const nrs_ctx* ctx, size_t count, uint64_t* first_block, uint64_t* advance) {
  *first_block = ctx->rng_offset;
  *advance = (count + 3) / 4;
  if (ctx->shard_global <= 0 || ctx->shard_local <= 0 || count % (size_t)ctx->shard_local != 0) return;
  const size_t per = count / (size_t)ctx->shard_local, before = (size_t)ctx->shard_begin * per;
  if (before % 4 != 0) return;
  *first_block = ctx->rng_offset + before / 4;
  *advance = ((size_t)ctx->shard_global * per + 3) / 4;
}

inline const NrsPlanes* nrs_planes_find(nrs_ctx* ctx, const void* src, bool split) {
  auto it = ctx->plane_hints.find(src);
  if (it == ctx->plane_hints.end() || (it->second.split != 0) != split) return nullptr;
  return &it->second;
}
// Reads and clears the device error word (the stream must be idle); NRS_ERR_TIMEOUT if a kernel gave up a wait.
int nrs_check_device_error(nrs_ctx* ctx);

// Batched weight staging (weight_set.cu).  build: allocates planes for the described weights in the
// context's current math mode (nothing in FP32 mode) and replaces any earlier set; refresh: one launch
// that stages them all from the weights' current values; find: the planes of (w, form) when the set is
// fresh and was built for the current mode, else null.
int nrs_weight_set_build(nrs_ctx* ctx, const NrsWeightDesc* descs, int count);
int nrs_weight_set_refresh(nrs_ctx* ctx);
// Restages only the weights stored in [lo, hi) (a bucket of parameters that has just been updated), on the
// context's current stream; counts the jobs done in refreshed_jobs.  The caller decides when the set as a
// whole is fresh again.
int nrs_weight_set_refresh_range(nrs_ctx* ctx, const float* lo, const float* hi);
void nrs_weight_set_clear(nrs_ctx* ctx);
inline const NrsWeightPlanes* nrs_weight_planes_find(nrs_ctx* ctx, const void* w, int form) {
  const NrsWeightSet& ws = ctx->weight_set;
  if (!ws.fresh || ws.n_jobs == 0 || ws.split != (ctx->math_mode == NRS_MATH_3XTF32) || ctx->math_mode == NRS_MATH_FP32) return nullptr;
  auto it = ws.planes.find(std::make_pair(w, form));
  return it == ws.planes.end() ? nullptr : &it->second;
}

#define NRS_REQUIRE_CTX(ctx) \
  do { if (!(ctx)) return nrs_fail(nullptr, NRS_ERR_ARG, "%s: null context", __func__); } while (0)
#define NRS_REQUIRE(ctx, cond, code, ...) \
  do { if (!(cond)) return nrs_fail((ctx), (code), __VA_ARGS__); } while (0)
#define NRS_CUDA(ctx, call)                                                              \
  do {                                                                                   \
    cudaError_t e__ = (call);                                                            \
    if (e__ != cudaSuccess)                                                              \
      return nrs_fail((ctx), NRS_ERR_CUDA, "%s: %s failed: %s", __func__, #call,         \
                      cudaGetErrorString(e__));                                          \
  } while (0)
// After a kernel launch: count it and surface launch-configuration errors.
#define NRS_LAUNCHED(ctx)                                                                \
  do {                                                                                   \
    (ctx)->launches++;                                                                   \
    cudaError_t e__ = cudaGetLastError();                                                \
    if (e__ != cudaSuccess)                                                              \
      return nrs_fail((ctx), NRS_ERR_CUDA, "%s: kernel launch failed: %s", __func__,     \
                      cudaGetErrorString(e__));                                          \
  } while (0)

// cudaFuncAttributeMaxDynamicSharedMemorySize belongs to a (kernel, device) pair, and one process may hold
// contexts on several devices.  Each launcher keeps one NrsSmemAttr per kernel instantiation: the largest
// value already set on every device ordinal.
constexpr int kNrsMaxDevices = 64;
struct NrsSmemAttr {
  size_t bytes[kNrsMaxDevices] = {};
};
// True when `bytes` of dynamic shared memory on `device` still has to be requested (values that fit the
// 48 KB default never do); records the request.
inline bool nrs_smem_attr_update(NrsSmemAttr& a, int device, size_t bytes) {
  if (bytes <= 48 * 1024) return false;
  if (device < 0 || device >= kNrsMaxDevices) return true;   // not tracked: always set
  if (bytes <= a.bytes[device]) return false;
  a.bytes[device] = bytes;
  return true;
}
#define NRS_ENSURE_SMEM(ctx, attr, kernel, bytes)                                                          \
  do {                                                                                                     \
    if (nrs_smem_attr_update((attr), (ctx)->device, (size_t)(bytes)))                                      \
      NRS_CUDA((ctx), cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)(bytes))); \
  } while (0)

// Programmatic dependent launch.  A kernel launched through nrs_pdl_launch may be scheduled while
// the kernel before it in the stream is still running (as SMs free up in its last wave), so that its
// launch latency and prologue overlap with that kernel's tail; it must execute NRS_PDL_WAIT() before
// its first global-memory access — the wait returns once the preceding kernel has completed and its
// writes are visible.  NRS_PDL_TRIGGER() lets the NEXT kernel start the same way; every CTA of a grid
// has to issue it (or exit) before that happens, so only a grid's last wave is ever shared.
#define NRS_PDL_WAIT() asm volatile("griddepcontrol.wait;" ::: "memory")
#define NRS_PDL_TRIGGER() asm volatile("griddepcontrol.launch_dependents;" ::: "memory")
// Order: every kernel WAITS first and only then triggers.  That keeps one property a few kernels rely on:
// when kernel N+1 has been launched, every CTA of kernel N has passed its wait, so kernel N-1 and all
// before it have completed.  A kernel that does not depend on its immediate predecessor (a weight
// gradient issued right after the data gradient of the same layer: both read the same inputs) may then
// skip the wait at its start, begin on the SMs its predecessor's last wave leaves idle, and wait just
// before it exits instead, so that kernels after it still see everything before them complete.  Such a
// kernel triggers at once: its successor's own wait returns only when this kernel has completed, late wait
// included, so the successor still sees everything before it.  Two such kernels are never adjacent: the
// callers mark a launch independent only right after issuing the data gradient it may overlap.
#define NRS_PDL_PROLOGUE() \
  do { NRS_PDL_WAIT(); NRS_PDL_TRIGGER(); } while (0)

template <class... P, class... A>
inline cudaError_t nrs_pdl_launch(void (*kernel)(P...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, A&&... args) {
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr{};
  attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr.val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = &attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<P>(args)...);
}
// kernel<<<grid, block, smem, stream>>>(args...) as a programmatic dependent launch.  The kernel
// expression goes in parentheses when its template arguments contain commas.
#define NRS_PDL_LAUNCH(kernel, grid, block, smem, stream, ...) \
  (void)nrs_pdl_launch(kernel, dim3(grid), dim3(block), (size_t)(smem), stream, __VA_ARGS__)

// Split reduces of the weight-gradient kernels: threads per block, and how many of them share one output
// (each summing every lanes-th split) for a given number of splits.
constexpr int kReduceThreads = 256;
static inline int reduce_lanes(int splits) { return splits >= 32 ? 8 : splits >= 16 ? 4 : splits >= 8 ? 2 : 1; }

static inline unsigned nrs_blocks(size_t work, unsigned per_block) {
  return (unsigned)((work + per_block - 1) / per_block);
}

// Tensor-core contraction entry points (tc_gemm.cu / tc_conv.cu).  Each returns
// NRS_ERR_UNSUPPORTED (without setting an error text) when the shape is outside
// what the tcgen05 kernels cover, and the caller then runs the FFMA kernels.
// pre_out (optional, [batch][m][n]): the value before the activation, written by the same epilogue.
int nrs_tc_gemm(nrs_ctx* ctx, int trans_a, int trans_b, int batch, int m, int n, int k,
                const float* a, const float* b, float* c, const float* bias, int act, float beta, float* pre_out = nullptr);
// c = act(a[m,k] . w[k,n] + bias) and pre = a . w + bias from one tensor-core kernel; NRS_ERR_UNSUPPORTED (no
// error text) when the product would not run there.
int nrs_linear_act_pre(nrs_ctx* ctx, int m, int n, int k, const float* a, const float* w, const float* bias, int act, float* c,
                       float* pre);
int nrs_tc_conv_fwd(nrs_ctx* ctx, const float* x, const float* w, const float* b, float* y, int n, int ci, int h,
                    int wd, int co, int kh, int kw, int stride, int pad, int act);
int nrs_tc_conv_dgrad(nrs_ctx* ctx, const float* w, const float* dy, float* dx, int n, int ci, int h, int wd, int co,
                      int kh, int kw, int stride, int pad, int accumulate);
int nrs_tc_conv_wgrad(nrs_ctx* ctx, const float* x, const float* dy, float* dw, int n, int ci, int h, int wd, int co,
                      int kh, int kw, int stride, int pad, int accumulate);
bool nrs_gemm_on_tensor_cores(const nrs_ctx* ctx, int m, int n, int k);
// C[m,n] (+)= A^T B, A stored [k][m], B stored [k][n], on the weight-gradient kernel (no transposes).
int nrs_tc_gemm_tn(nrs_ctx* ctx, int m, int n, int k, const float* a, const float* b, float* c, int accumulate);
// Row-streaming variant for 3x3 / stride 1 / pad 1 (tc_wgrad_rows.cu); tried first.
int nrs_tc_conv_wgrad_rows(nrs_ctx* ctx, const float* x, const float* dy, float* dw, int n, int ci, int h, int wd, int co,
                           int kh, int kw, int stride, int pad, int accumulate);
// Fused attention core on the tensor cores (attention_tc.cu); NRS_ERR_UNSUPPORTED (no error text) outside its range.
int nrs_tc_attention_fwd(nrs_ctx* ctx, const float* q, const float* k, const float* v, float* out, float* probs, int batch,
                         int seq, int heads, int d_head, int causal);
int nrs_tc_attention_bwd(nrs_ctx* ctx, const float* q, const float* k, const float* v, const float* probs, const float* dout,
                         float* dq, float* dk, float* dv, int batch, int seq, int heads, int d_head, int acc_q, int acc_k,
                         int acc_v);
// Patch planes of x[n,ci,h,w] for a 3x3 / pad `pad` image layer (ci = 1 or 3): hi/lo [n*oh*ow][32].
int nrs_smallc_patch_planes(nrs_ctx* ctx, const float* x, float* hi, float* lo, int n, int ci, int h, int wd, int pad);
// Direct FFMA kernels for 3x3 stride-1 layers over 1 or 3 input channels (conv_smallc.cu).
int nrs_smallc_conv_fwd(nrs_ctx* ctx, const float* x, const float* w, const float* b, float* y, int n, int ci, int h,
                        int wd, int co, int kh, int kw, int stride, int pad, int act);
int nrs_smallc_conv_wgrad(nrs_ctx* ctx, const float* x, const float* dy, float* dw, int n, int ci, int h, int wd, int co,
                          int kh, int kw, int stride, int pad, int accumulate);
