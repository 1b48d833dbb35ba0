// Batch normalisation over [n, c, hw] (hw == 1 is the [batch, features] layer), forward and backward.
// Reference: bn2d_stats / bn2d_normalize / bn2d_reduce / bn2d_dx (src/cuda/nn/batchnorm2d.rs:22-128) and their
// 2-D twins bn_stats / bn_normalize / bn_reduce / bn_dx (src/cuda/nn/batchnorm.rs:20-108); CPU semantics
// src/nn/batchnorm2d.rs:28-164, src/nn/batchnorm.rs:28-150.
//
// The reference walks a channel with one thread (two serial passes for the statistics).  Here every
// per-channel reduction is a pair of sums spread over (channel, sample-split) blocks and folded in a fixed
// order, so results are bit-reproducible and the pass runs at HBM speed:
//   forward   S = sum(x - K), Q = sum((x - K)^2) with the pivot K = the channel's first element, which keeps
//             Q/N - (S/N)^2 free of the cancellation a raw sum of squares has when |mean| >> std;
//   backward  S = sum(g) = dbeta, Q = sum(g * xhat) = dgamma.
// x is read twice in the forward pass (statistics, normalise) and g / xhat twice in the backward pass.
#include "nrs_internal.h"

namespace {

constexpr int kThreads = 256;

__device__ __forceinline__ bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

__device__ __forceinline__ float wsum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// The two values an element contributes.  FWD: a = x, b unused, k = pivot.  BWD: a = g, b = xhat.
template <bool FWD>
__device__ __forceinline__ void contribute(float a, float b, float k, float& s, float& q) {
  if (FWD) {
    const float d = a - k;
    s += d;
    q += d * d;
  } else {
    s += a;
    q += a * b;
  }
}

// Planes layout (hw >= 2): one block per (channel, sample split), 128-bit loads when the plane allows.
// partial[split][ch] = (S, Q).
// RELU (backward only): the layer's output went through a ReLU fused into the normalise pass; the incoming
// gradient is masked where that output was not positive, the output being recomputed from xhat with the very
// expression of the forward pass (fmaf(gamma, xhat, beta)), so the mask is the forward one bit for bit.
template <bool FWD, bool RELU>
__global__ void __launch_bounds__(kThreads)
bn_pair_planes_kernel(const float* __restrict__ a, const float* __restrict__ b, float2* __restrict__ partial, int n,
                      int c, int hw, int splits, const float* __restrict__ gamma, const float* __restrict__ beta,
                      const float* __restrict__ pivot) {
  NRS_PDL_PROLOGUE();
  __shared__ float2 sm[kThreads / 32];
  const int ch = blockIdx.x, split = blockIdx.y;
  const int lane = threadIdx.x & 31, wrp = threadIdx.x >> 5;
  const int n_per = (n + splits - 1) / splits;
  const int n0 = split * n_per, n1 = min(n, n0 + n_per);
  const float k = FWD ? (pivot ? pivot[ch] : a[(size_t)ch * hw]) : 0.0f;
  const float ga = RELU ? gamma[ch] : 0.0f, be = RELU ? beta[ch] : 0.0f;
  const bool vec = (hw & 3) == 0 && aligned16(a) && (FWD || aligned16(b));
  // The block's threads walk the split's (image, element) pairs as one flat index, so that planes shorter
  // than a warp's reach (8x8, 4x4 feature maps) still keep every lane loading.
  float s = 0.0f, q = 0.0f, s1 = 0.0f, q1 = 0.0f;
  const int per = vec ? hw / 4 : hw;                       // items per plane
  const int items = max(n1 - n0, 0) * per;               // n * hw < 2^31 is checked on the host
  for (int j = threadIdx.x; j < items; j += kThreads) {
    const int di = j / per, i = j - di * per;
    const size_t base = ((size_t)(n0 + di) * c + ch) * hw;
    if (vec) {
      float4 va = reinterpret_cast<const float4*>(a + base)[i];
      float4 vb = make_float4(0.f, 0.f, 0.f, 0.f);
      if (!FWD) vb = reinterpret_cast<const float4*>(b + base)[i];
      if (RELU) {
        va.x = fmaf(ga, vb.x, be) > 0.0f ? va.x : 0.0f;
        va.y = fmaf(ga, vb.y, be) > 0.0f ? va.y : 0.0f;
        va.z = fmaf(ga, vb.z, be) > 0.0f ? va.z : 0.0f;
        va.w = fmaf(ga, vb.w, be) > 0.0f ? va.w : 0.0f;
      }
      contribute<FWD>(va.x, vb.x, k, s, q);
      contribute<FWD>(va.y, vb.y, k, s1, q1);
      contribute<FWD>(va.z, vb.z, k, s, q);
      contribute<FWD>(va.w, vb.w, k, s1, q1);
    } else {
      const float vb = FWD ? 0.0f : b[base + i];
      float va = a[base + i];
      if (RELU) va = fmaf(ga, vb, be) > 0.0f ? va : 0.0f;
      contribute<FWD>(va, vb, k, s, q);
    }
  }
  s += s1;
  q += q1;
  s = wsum(s);
  q = wsum(q);
  if (lane == 0) sm[wrp] = make_float2(s, q);
  __syncthreads();
  if (threadIdx.x == 0) {
    float2 t = sm[0];
#pragma unroll
    for (int i = 1; i < kThreads / 32; ++i) { t.x += sm[i].x; t.y += sm[i].y; }
    partial[(size_t)split * c + ch] = t;
  }
}

// Columns layout (hw == 1): a block owns 32 features and a slice of the rows; its 8 warps stride the rows
// reading 128-byte row segments.
template <bool FWD, bool RELU>
__global__ void __launch_bounds__(kThreads)
bn_pair_cols_kernel(const float* __restrict__ a, const float* __restrict__ b, float2* __restrict__ partial, int rows,
                    int cols, int splits, const float* __restrict__ gamma, const float* __restrict__ beta,
                    const float* __restrict__ pivot) {
  NRS_PDL_PROLOGUE();
  __shared__ float2 sm[kThreads / 32][33];
  const int lane = threadIdx.x & 31, wrp = threadIdx.x >> 5;
  const int col = blockIdx.x * 32 + lane, split = blockIdx.y;
  const int rows_per = (rows + splits - 1) / splits;
  const int r0 = split * rows_per, r1 = min(rows, r0 + rows_per);
  float s = 0.0f, q = 0.0f;
  if (col < cols) {
    const float k = FWD ? (pivot ? pivot[col] : a[col]) : 0.0f;
    const float ga = RELU ? gamma[col] : 0.0f, be = RELU ? beta[col] : 0.0f;
    for (int r = r0 + wrp; r < r1; r += kThreads / 32) {
      const size_t i = (size_t)r * cols + col;
      const float vb = FWD ? 0.0f : b[i];
      float va = a[i];
      if (RELU) va = fmaf(ga, vb, be) > 0.0f ? va : 0.0f;
      contribute<FWD>(va, vb, k, s, q);
    }
  }
  sm[wrp][lane] = make_float2(s, q);
  __syncthreads();
  if (wrp == 0 && col < cols) {
    float2 t = sm[0][lane];
#pragma unroll
    for (int i = 1; i < kThreads / 32; ++i) { t.x += sm[i][lane].x; t.y += sm[i][lane].y; }
    partial[(size_t)split * cols + col] = t;
  }
}

// One thread per channel folds the splits in order and finishes the statistics: mean, biased variance,
// running statistics (running = momentum * running + (1 - momentum) * batch value, batchnorm2d.rs:52-53),
// 1/sqrt(var + eps).  In evaluation mode the running statistics are used as they are (batchnorm2d.rs:57-60).
// `pivot` / `count_dev` (both or neither): the sums were taken around pivot[ch] (the running mean, read here
// before it is updated) over *count_dev elements — statistics summed over several processes.
__global__ void bn_stats_finish_kernel(const float2* __restrict__ partial, const float* __restrict__ x, float* mean,
                                       float* istd, float* running_mean, float* running_var, int c, int hw,
                                       int splits, float count, float eps, float momentum, int training,
                                       const float* __restrict__ pivot, const float* __restrict__ count_dev) {
  NRS_PDL_PROLOGUE();
  const int ch = blockIdx.x * blockDim.x + threadIdx.x;
  if (ch >= c) return;
  if (!training) {
    mean[ch] = running_mean[ch];
    istd[ch] = 1.0f / sqrtf(running_var[ch] + eps);
    return;
  }
  float s = 0.0f, q = 0.0f;
  for (int z = 0; z < splits; ++z) {
    const float2 t = partial[(size_t)z * c + ch];
    s += t.x;
    q += t.y;
  }
  const float k = pivot ? pivot[ch] : x[(size_t)ch * hw];
  if (count_dev) count = *count_dev;
  const float d = s / count;
  const float m = k + d;
  const float v = fmaxf(q / count - d * d, 0.0f);
  running_mean[ch] = momentum * running_mean[ch] + (1.0f - momentum) * m;
  running_var[ch] = momentum * running_var[ch] + (1.0f - momentum) * v;
  mean[ch] = m;
  istd[ch] = 1.0f / sqrtf(v + eps);
}

// Folds the backward sums; sums[ch] = (dbeta, dgamma) of this call feeds the dx kernel, and the parameter
// gradients receive them (+)=.
__global__ void bn_grad_finish_kernel(const float2* __restrict__ partial, float2* __restrict__ sums, float* dgamma,
                                      float* dbeta, int c, int splits, int accumulate) {
  NRS_PDL_PROLOGUE();
  const int ch = blockIdx.x * blockDim.x + threadIdx.x;
  if (ch >= c) return;
  float s = 0.0f, q = 0.0f;
  for (int z = 0; z < splits; ++z) {
    const float2 t = partial[(size_t)z * c + ch];
    s += t.x;
    q += t.y;
  }
  sums[ch] = make_float2(s, q);
  if (dgamma) dgamma[ch] = accumulate ? dgamma[ch] + q : q;
  if (dbeta) dbeta[ch] = accumulate ? dbeta[ch] + s : s;
}

// y = gamma * xhat + beta, xhat = (x - mean) * istd (bn2d_normalize, batchnorm2d.rs:62-75).
template <bool VEC, bool RELU>
__global__ void __launch_bounds__(kThreads)
bn_normalize_kernel(const float* __restrict__ x, const float* __restrict__ mean, const float* __restrict__ istd,
                    const float* __restrict__ gamma, const float* __restrict__ beta, float* __restrict__ y,
                    float* __restrict__ xhat, size_t total, int c, int hw) {
  NRS_PDL_PROLOGUE();
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  const size_t tid = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (VEC) {   // hw % 4 == 0: the four elements of a vector share their channel
    for (size_t i = tid; i < total / 4; i += stride) {
      const int ch = (int)((i * 4 / hw) % c);
      const float m = mean[ch], is = istd[ch], ga = gamma[ch], be = beta[ch];
      const float4 v = reinterpret_cast<const float4*>(x)[i];
      const float4 h = make_float4((v.x - m) * is, (v.y - m) * is, (v.z - m) * is, (v.w - m) * is);
      if (xhat) reinterpret_cast<float4*>(xhat)[i] = h;
      float4 o = make_float4(fmaf(ga, h.x, be), fmaf(ga, h.y, be), fmaf(ga, h.z, be), fmaf(ga, h.w, be));
      if (RELU) o = make_float4(fmaxf(o.x, 0.0f), fmaxf(o.y, 0.0f), fmaxf(o.z, 0.0f), fmaxf(o.w, 0.0f));
      reinterpret_cast<float4*>(y)[i] = o;
    }
  } else {
    for (size_t i = tid; i < total; i += stride) {
      const int ch = (int)((i / hw) % c);
      const float h = (x[i] - mean[ch]) * istd[ch];
      if (xhat) xhat[i] = h;
      const float o = fmaf(gamma[ch], h, beta[ch]);
      y[i] = RELU ? fmaxf(o, 0.0f) : o;
    }
  }
}

// bn2d_dx (batchnorm2d.rs:96-117): training dx = istd * (g*gamma - gamma*dbeta/N - xhat*gamma*dgamma/N);
// evaluation dx = g * gamma * istd.
template <bool VEC, bool RELU>
__global__ void __launch_bounds__(kThreads)
bn_dx_kernel(const float* __restrict__ g, const float* __restrict__ xhat, const float* __restrict__ istd,
             const float* __restrict__ gamma, const float* __restrict__ beta, const float2* __restrict__ sums, float* dx,
             size_t total, int c, int hw, float count, int training, int accumulate, const float* __restrict__ count_dev) {
  NRS_PDL_PROLOGUE();
  if (count_dev) count = *count_dev;   // elements per channel over all processes
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  const size_t tid = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (VEC) {
    for (size_t i = tid; i < total / 4; i += stride) {
      const int ch = (int)((i * 4 / hw) % c);
      const float ga = gamma[ch], is = istd[ch];
      float4 vg = reinterpret_cast<const float4*>(g)[i];
      float4 vh = make_float4(0.f, 0.f, 0.f, 0.f);
      if (training || RELU) vh = reinterpret_cast<const float4*>(xhat)[i];
      if (RELU) {
        const float be = beta[ch];
        vg.x = fmaf(ga, vh.x, be) > 0.0f ? vg.x : 0.0f;
        vg.y = fmaf(ga, vh.y, be) > 0.0f ? vg.y : 0.0f;
        vg.z = fmaf(ga, vh.z, be) > 0.0f ? vg.z : 0.0f;
        vg.w = fmaf(ga, vh.w, be) > 0.0f ? vg.w : 0.0f;
      }
      float4 r;
      if (training) {
        const float2 sm = sums[ch];
        const float m1 = ga * sm.x / count, m2 = ga * sm.y / count;
        r = make_float4(is * (vg.x * ga - m1 - vh.x * m2), is * (vg.y * ga - m1 - vh.y * m2),
                        is * (vg.z * ga - m1 - vh.z * m2), is * (vg.w * ga - m1 - vh.w * m2));
      } else {
        r = make_float4(vg.x * ga * is, vg.y * ga * is, vg.z * ga * is, vg.w * ga * is);
      }
      float4* dst = reinterpret_cast<float4*>(dx) + i;
      if (accumulate) {
        const float4 o = *dst;
        r = make_float4(o.x + r.x, o.y + r.y, o.z + r.z, o.w + r.w);
      }
      *dst = r;
    }
  } else {
    for (size_t i = tid; i < total; i += stride) {
      const int ch = (int)((i / hw) % c);
      const float ga = gamma[ch], is = istd[ch];
      float gi = g[i];
      if (RELU) gi = fmaf(ga, xhat[i], beta[ch]) > 0.0f ? gi : 0.0f;
      float r;
      if (training) {
        const float2 sm = sums[ch];
        r = is * (gi * ga - ga * sm.x / count - xhat[i] * (ga * sm.y / count));
      } else {
        r = gi * ga * is;
      }
      dx[i] = accumulate ? dx[i] + r : r;
    }
  }
}

// Statistics shared by several processes: the splits of this process folded in order into out[ch], the
// element count behind them (one slot), ready for one cross-rank sum of 2c + 1 floats.
__global__ void bn_fold_for_sync_kernel(const float2* __restrict__ partial, float2* __restrict__ out, float* count_slot,
                                        int c, int splits, float local_count) {
  NRS_PDL_PROLOGUE();
  const int ch = blockIdx.x * blockDim.x + threadIdx.x;
  if (ch == 0) *count_slot = local_count;
  if (ch >= c) return;
  float s = 0.0f, q = 0.0f;
  for (int z = 0; z < splits; ++z) {
    const float2 t = partial[(size_t)z * c + ch];
    s += t.x;
    q += t.y;
  }
  out[ch] = make_float2(s, q);
}
__global__ void bn_set_count_kernel(float* count_slot, float local_count) {
  NRS_PDL_PROLOGUE();
  if (blockIdx.x == 0 && threadIdx.x == 0) *count_slot = local_count;
}

// How many sample splits the per-channel reductions use: enough blocks to fill the device a few times over,
// no fewer than 8 images (planes) or 64 rows (columns) per block.
int plan_splits(const nrs_ctx* ctx, int n, int c, int hw) {
  const int blocks_c = hw == 1 ? (c + 31) / 32 : c;
  const int min_per = hw == 1 ? 64 : 8;
  int splits = (4 * ctx->sm_count + blocks_c - 1) / blocks_c;
  if (splits > n / min_per) splits = n / min_per;
  if (splits < 1) splits = 1;
  if (splits > 65535) splits = 65535;
  return splits;
}

template <bool FWD, bool RELU>
int launch_pair(nrs_ctx* ctx, const float* a, const float* b, float2* partial, int n, int c, int hw, int splits,
                const float* gamma, const float* beta, const float* pivot = nullptr) {
  if (hw == 1) {
    NRS_PDL_LAUNCH((bn_pair_cols_kernel<FWD, RELU>), dim3((c + 31) / 32, splits), kThreads, 0, ctx->stream, a, b, partial, n, c,
                   splits, gamma, beta, pivot);
  } else {
    NRS_PDL_LAUNCH((bn_pair_planes_kernel<FWD, RELU>), dim3(c, splits), kThreads, 0, ctx->stream, a, b, partial, n, c, hw,
                   splits, gamma, beta, pivot);
  }
  NRS_LAUNCHED(ctx);
  return NRS_OK;
}

unsigned ew_blocks(const nrs_ctx* ctx, size_t work_items) {
  const size_t want = (work_items + kThreads - 1) / kThreads;
  const size_t cap = (size_t)ctx->sm_count * 16;
  return (unsigned)(want < 1 ? 1 : (want > cap ? cap : want));
}

bool check_dims(int n, int c, int hw) {
  return n >= 1 && c >= 1 && hw >= 1 && (size_t)n * c * hw <= (size_t)1 << 40 && (size_t)c * hw <= 0x7fffffffu &&
         (size_t)n * hw <= 0x7fffffffu;
}

}  // namespace

namespace {

int bn_forward(nrs_ctx* ctx, const char* who, const float* x, const float* gamma, const float* beta, float* running_mean,
               float* running_var, float* y, float* xhat, float* istd, int n, int c, int hw, float eps, float momentum,
               int training, bool relu) {
  NRS_REQUIRE_CTX(ctx);
  NRS_REQUIRE(ctx, check_dims(n, c, hw), NRS_ERR_SHAPE, "%s: bad shape [%d,%d,%d]", who, n, c, hw);
  NRS_REQUIRE(ctx, x && gamma && beta && running_mean && running_var && y && istd, NRS_ERR_ARG, "%s: null tensor", who);
  NrsProfScope prof(ctx, NRS_PROF_BATCHNORM, 12.0 * (double)n * c * hw);   // x in; y, xhat out
  const int splits = training ? plan_splits(ctx, n, c, hw) : 1;
  // statistics over every process's shard: sums around a pivot all ranks share (the running mean), folded,
  // summed across ranks together with the element count, then finished as usual
  const bool shared = training && ctx->stat_sync.all_reduce_sum != nullptr;
  void* ws = nullptr;
  const int st = nrs_workspace(ctx, ((size_t)splits * c * 2 + c + (size_t)c * 2 + 4) * sizeof(float), &ws);
  if (st != NRS_OK) return st;
  float2* partial = (float2*)ws;
  float* mean = (float*)(partial + (size_t)splits * c);
  float2* summed = (float2*)(mean + c + (c & 1));   // 8-byte aligned; [c] pairs + the count
  float* count_slot = (float*)(summed + c);
  if (training) {
    const int sp = launch_pair<true, false>(ctx, x, nullptr, partial, n, c, hw, splits, nullptr, nullptr,
                                            shared ? running_mean : nullptr);
    if (sp != NRS_OK) return sp;
  }
  if (shared) {
    NRS_PDL_LAUNCH(bn_fold_for_sync_kernel, nrs_blocks(c, 128), 128, 0, ctx->stream, (const float2*)partial, summed, count_slot, c,
                   splits, (float)((double)n * hw));
    NRS_LAUNCHED(ctx);
    const int sr = ctx->stat_sync.all_reduce_sum(ctx->stat_sync.user, (float*)summed, (size_t)c * 2 + 1);
    if (sr != NRS_OK) return sr;
    NRS_PDL_LAUNCH(bn_stats_finish_kernel, nrs_blocks(c, 128), 128, 0, ctx->stream, (const float2*)summed, x, mean, istd,
                   running_mean, running_var, c, hw, 1, 0.0f, eps, momentum, training, (const float*)running_mean,
                   (const float*)count_slot);
  } else {
    NRS_PDL_LAUNCH(bn_stats_finish_kernel, nrs_blocks(c, 128), 128, 0, ctx->stream, (const float2*)partial, x, mean, istd,
                   running_mean, running_var, c, hw, splits, (float)((double)n * hw), eps, momentum, training,
                   (const float*)nullptr, (const float*)nullptr);
  }
  NRS_LAUNCHED(ctx);
  const size_t total = (size_t)n * c * hw;
  const bool vec = (hw & 3) == 0 && ((uintptr_t)x & 15) == 0 && ((uintptr_t)y & 15) == 0 && ((uintptr_t)xhat & 15) == 0;
  const unsigned blocks = ew_blocks(ctx, vec ? total / 4 : total);
#define NRS_BN_NORM(V, R)                                                                                          \
  NRS_PDL_LAUNCH((bn_normalize_kernel<V, R>), blocks, kThreads, 0, ctx->stream, x, (const float*)mean, (const float*)istd, \
                 gamma, beta, y, xhat, total, c, hw)
  if (vec) { if (relu) NRS_BN_NORM(true, true); else NRS_BN_NORM(true, false); }
  else { if (relu) NRS_BN_NORM(false, true); else NRS_BN_NORM(false, false); }
#undef NRS_BN_NORM
  NRS_LAUNCHED(ctx);
  return NRS_OK;
}

int bn_backward(nrs_ctx* ctx, const char* who, const float* g, const float* xhat, const float* istd, const float* gamma,
                const float* beta, float* dx, float* dgamma, float* dbeta, int n, int c, int hw, int training,
                int accumulate_dx, int accumulate_params, bool relu) {
  NRS_REQUIRE_CTX(ctx);
  NRS_REQUIRE(ctx, check_dims(n, c, hw), NRS_ERR_SHAPE, "%s: bad shape [%d,%d,%d]", who, n, c, hw);
  NRS_REQUIRE(ctx, (dgamma == nullptr) == (dbeta == nullptr), NRS_ERR_ARG, "%s: dgamma and dbeta must be given together", who);
  NRS_REQUIRE(ctx, g && xhat && istd && gamma && (!relu || beta), NRS_ERR_ARG, "%s: null tensor", who);
  if (!dx && !dgamma) return NRS_OK;
  NrsProfScope prof(ctx, NRS_PROF_BATCHNORM, 12.0 * (double)n * c * hw);   // g, xhat in; dx out
  const bool need_sums = dgamma || training;
  const int splits = need_sums ? plan_splits(ctx, n, c, hw) : 1;
  void* ws = nullptr;
  const int st = nrs_workspace(ctx, ((size_t)splits * c * 2 + (size_t)c * 2 + 4) * sizeof(float), &ws);
  if (st != NRS_OK) return st;
  float2* partial = (float2*)ws;
  float2* sums = partial + (size_t)splits * c;
  float* count_slot = (float*)(sums + c);
  // with shared statistics dx needs the sums over every process's shard; the parameter gradients keep this
  // process's own sums (they are summed across ranks with all other gradients)
  const bool shared = training && dx && ctx->stat_sync.all_reduce_sum != nullptr;
  if (need_sums) {
    const int sp = relu ? launch_pair<false, true>(ctx, g, xhat, partial, n, c, hw, splits, gamma, beta)
                        : launch_pair<false, false>(ctx, g, xhat, partial, n, c, hw, splits, nullptr, nullptr);
    if (sp != NRS_OK) return sp;
    NRS_PDL_LAUNCH(bn_grad_finish_kernel, nrs_blocks(c, 128), 128, 0, ctx->stream, (const float2*)partial, sums, dgamma, dbeta,
                   c, splits, accumulate_params);
    NRS_LAUNCHED(ctx);
  }
  if (!dx) return NRS_OK;
  if (shared) {
    NRS_PDL_LAUNCH(bn_set_count_kernel, 1, 32, 0, ctx->stream, count_slot, (float)((double)n * hw));
    NRS_LAUNCHED(ctx);
    const int sr = ctx->stat_sync.all_reduce_sum(ctx->stat_sync.user, (float*)sums, (size_t)c * 2 + 1);
    if (sr != NRS_OK) return sr;
  }
  const size_t total = (size_t)n * c * hw;
  const float count = (float)((double)n * hw);
  const bool vec = (hw & 3) == 0 && ((uintptr_t)g & 15) == 0 && ((uintptr_t)xhat & 15) == 0 && ((uintptr_t)dx & 15) == 0;
  const unsigned blocks = ew_blocks(ctx, vec ? total / 4 : total);
#define NRS_BN_DX(V, R)                                                                                              \
  NRS_PDL_LAUNCH((bn_dx_kernel<V, R>), blocks, kThreads, 0, ctx->stream, g, xhat, istd, gamma, beta, (const float2*)sums, dx, \
                 total, c, hw, count, training, accumulate_dx, shared ? (const float*)count_slot : (const float*)nullptr)
  if (vec) { if (relu) NRS_BN_DX(true, true); else NRS_BN_DX(true, false); }
  else { if (relu) NRS_BN_DX(false, true); else NRS_BN_DX(false, false); }
#undef NRS_BN_DX
  NRS_LAUNCHED(ctx);
  return NRS_OK;
}

bool act_ok(int act) { return act == NRS_ACT_NONE || act == NRS_ACT_RELU; }

}  // namespace

int nrs_batchnorm_fwd(nrs_ctx* ctx, const float* x, const float* gamma, const float* beta, float* running_mean,
                      float* running_var, float* y, float* xhat, float* istd, int n, int c, int hw, float eps,
                      float momentum, int training) {
  return bn_forward(ctx, "nrs_batchnorm_fwd", x, gamma, beta, running_mean, running_var, y, xhat, istd, n, c, hw, eps,
                    momentum, training, false);
}

int nrs_batchnorm_bwd(nrs_ctx* ctx, const float* g, const float* xhat, const float* istd, const float* gamma, float* dx,
                      float* dgamma, float* dbeta, int n, int c, int hw, int training, int accumulate_dx,
                      int accumulate_params) {
  return bn_backward(ctx, "nrs_batchnorm_bwd", g, xhat, istd, gamma, nullptr, dx, dgamma, dbeta, n, c, hw, training,
                     accumulate_dx, accumulate_params, false);
}

int nrs_batchnorm_act_fwd(nrs_ctx* ctx, const float* x, const float* gamma, const float* beta, float* running_mean,
                          float* running_var, float* y, float* xhat, float* istd, int n, int c, int hw, float eps,
                          float momentum, int training, int act) {
  NRS_REQUIRE_CTX(ctx);
  NRS_REQUIRE(ctx, act_ok(act), NRS_ERR_ARG, "nrs_batchnorm_act_fwd: activation %d is not NONE or RELU", act);
  NRS_REQUIRE(ctx, act == NRS_ACT_NONE || xhat, NRS_ERR_ARG, "nrs_batchnorm_act_fwd: a fused ReLU needs xhat saved");
  return bn_forward(ctx, "nrs_batchnorm_act_fwd", x, gamma, beta, running_mean, running_var, y, xhat, istd, n, c, hw, eps,
                    momentum, training, act == NRS_ACT_RELU);
}

int nrs_batchnorm_act_bwd(nrs_ctx* ctx, const float* g, const float* xhat, const float* istd, const float* gamma,
                          const float* beta, float* dx, float* dgamma, float* dbeta, int n, int c, int hw, int training,
                          int accumulate_dx, int accumulate_params, int act) {
  NRS_REQUIRE_CTX(ctx);
  NRS_REQUIRE(ctx, act_ok(act), NRS_ERR_ARG, "nrs_batchnorm_act_bwd: activation %d is not NONE or RELU", act);
  return bn_backward(ctx, "nrs_batchnorm_act_bwd", g, xhat, istd, gamma, beta, dx, dgamma, dbeta, n, c, hw, training,
                     accumulate_dx, accumulate_params, act == NRS_ACT_RELU);
}
