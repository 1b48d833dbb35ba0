// Cross-entropy on raw logits with dense one-hot (f32) targets.
// Reference: ce_forward / ce_backward (src/cuda/loss/cross_entropy.rs:18-57),
// host side :74-128; CPU semantics src/nn/loss.rs:50-107.  The reference runs
// one thread per row and sums the per-row losses on the host after a blocking
// device-to-host copy; here a warp owns a row (shuffle reductions, the row is
// re-read from L1), forward and backward share one pass, and the batch mean is
// reduced on the device in a fixed order.
#include "nrs_internal.h"

namespace {

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// One warp per row.  row_loss (optional) gets -sum_c t*(x - lse); grad (optional)
// gets (softmax - t) * inv_div.  Scalar path (any width / alignment).
__global__ void __launch_bounds__(256)
ce_rows_kernel(const float* __restrict__ logits, const float* __restrict__ target, const int32_t* __restrict__ labels,
               float* __restrict__ row_loss, float* __restrict__ grad, int batch, int classes, float inv_div) {
  NRS_PDL_PROLOGUE();
  const int lane = threadIdx.x & 31;
  const int warps_per_block = blockDim.x >> 5;
  for (int b = blockIdx.x * warps_per_block + (threadIdx.x >> 5); b < batch; b += gridDim.x * warps_per_block) {
    const float* row = logits + (size_t)b * classes;
    const float* trow = target ? target + (size_t)b * classes : nullptr;
    const int label = labels ? labels[b] : -1;
    float mx = -INFINITY;
    for (int c = lane; c < classes; c += 32) mx = fmaxf(mx, row[c]);
    mx = warp_max(mx);
    float se = 0.0f;
    for (int c = lane; c < classes; c += 32) se += expf(row[c] - mx);
    se = warp_sum(se);
    const float lse = logf(se) + mx;
    float loss = 0.0f;
    for (int c = lane; c < classes; c += 32) {
      const float xv = row[c], tv = trow ? trow[c] : (c == label ? 1.0f : 0.0f);
      loss += -tv * (xv - lse);
      if (grad) grad[(size_t)b * classes + c] = (expf(xv - mx) / se - tv) * inv_div;
    }
    if (row_loss) {
      loss = warp_sum(loss);
      if (lane == 0) row_loss[b] = loss;
    }
  }
}

// The same with the row held in registers: logits (and the one-hot row) are read once with 128-bit
// loads (lane l takes float4s l, l+32, ...: 512 contiguous bytes per load instruction), every
// exponential is evaluated once, the gradient is written once.  Rows of up to 1024 classes whose
// width is a multiple of four.  With `labels` (int32 class per row) the dense one-hot tensor is not read.
// Registers hold two rows only, which is what bounds the rows in flight per SM (three blocks per SM): the
// target row, and the logits row that is overwritten by its exponentials once sum(t*x) and sum(t) have been
// taken (the row loss is lse*sum(t) - sum(t*x)).
template <int VPL>
__global__ void __launch_bounds__(256, 3)
ce_rows_vec_kernel(const float* __restrict__ logits, const float* __restrict__ target, const int32_t* __restrict__ labels,
                   float* __restrict__ row_loss, float* __restrict__ grad, int batch, int classes, float inv_div,
                   float* block_partial, unsigned* ticket, float* loss_dev) {
  NRS_PDL_PROLOGUE();
  const int lane = threadIdx.x & 31;
  const int warps_per_block = blockDim.x >> 5;
  const int c4 = classes >> 2;
  float warp_loss = 0.0f;   // this warp's rows, in the order it takes them
  for (int b = blockIdx.x * warps_per_block + (threadIdx.x >> 5); b < batch; b += gridDim.x * warps_per_block) {
    const size_t base = (size_t)b * classes;
    float4 x[VPL], t[VPL];
    float mx = -INFINITY;
    const int label = labels ? labels[b] : -1;
    // the row this warp takes next is pulled into L2 while this one is worked on: a warp is a serial chain
    // (loads, two reductions, stores), and this takes the DRAM round trip out of the next link
    {
      const int nb = b + gridDim.x * warps_per_block;
      if (nb < batch) {
        const char* nx = reinterpret_cast<const char*>(logits + (size_t)nb * classes);
        for (int off = lane * 128; off < classes * 4; off += 32 * 128) {
          asm volatile("prefetch.global.L2 [%0];" ::"l"(nx + off));
          if (target) asm volatile("prefetch.global.L2 [%0];" ::"l"(reinterpret_cast<const char*>(target + (size_t)nb * classes) + off));
        }
      }
    }
    // every load of the row (logits and one-hot row) is in flight before the first reduction waits
#pragma unroll
    for (int k = 0; k < VPL; ++k) {
      const int c = lane + 32 * k;
      if (c < c4) {
        x[k] = __ldcs(reinterpret_cast<const float4*>(logits + base) + c);
        if (target) {
          t[k] = __ldcs(reinterpret_cast<const float4*>(target + base) + c);
        } else {
          const int d = label - 4 * c;     // position of the label inside this float4, if any
          t[k] = make_float4(d == 0 ? 1.0f : 0.0f, d == 1 ? 1.0f : 0.0f, d == 2 ? 1.0f : 0.0f, d == 3 ? 1.0f : 0.0f);
        }
      }
    }
    float stx = 0.0f, st = 0.0f;   // sum(t*x), sum(t) of this lane's elements
#pragma unroll
    for (int k = 0; k < VPL; ++k)
      if (lane + 32 * k < c4) {
        mx = fmaxf(mx, fmaxf(fmaxf(x[k].x, x[k].y), fmaxf(x[k].z, x[k].w)));
        stx += (t[k].x * x[k].x + t[k].y * x[k].y) + (t[k].z * x[k].z + t[k].w * x[k].w);
        st += (t[k].x + t[k].y) + (t[k].z + t[k].w);
      }
    mx = warp_max(mx);
    float se = 0.0f;
#pragma unroll
    for (int k = 0; k < VPL; ++k)
      if (lane + 32 * k < c4) {
        x[k] = make_float4(expf(x[k].x - mx), expf(x[k].y - mx), expf(x[k].z - mx), expf(x[k].w - mx));
        se += (x[k].x + x[k].y) + (x[k].z + x[k].w);
      }
    se = warp_sum(se);          // three independent butterflies: their shuffles interleave
    stx = warp_sum(stx);
    st = warp_sum(st);
    const float lse = logf(se) + mx;
    const float inv_se = 1.0f / se;
    if (grad) {
#pragma unroll
      for (int k = 0; k < VPL; ++k) {
        const int c = lane + 32 * k;
        if (c < c4)
          __stcs(reinterpret_cast<float4*>(grad + base) + c,
                 make_float4((x[k].x * inv_se - t[k].x) * inv_div, (x[k].y * inv_se - t[k].y) * inv_div,
                             (x[k].z * inv_se - t[k].z) * inv_div, (x[k].w * inv_se - t[k].w) * inv_div));
      }
    }
    const float rl = lse * st - stx;
    if (row_loss && lane == 0) row_loss[b] = rl;
    warp_loss += rl;
  }
  if (!loss_dev) return;
  // Batch mean without a second launch: warps -> block (warp order) -> block_partial[block]; the block that
  // arrives last folds the partials in block order (lane l takes l, l+32, ..., then a butterfly), so the order
  // of the additions is fixed whichever block that is.
  __shared__ float wsum[32];
  __shared__ bool last;
  if (lane == 0) wsum[threadIdx.x >> 5] = warp_loss;
  __syncthreads();
  if (threadIdx.x == 0) {
    float s = 0.0f;
    for (int w = 0; w < warps_per_block; ++w) s += wsum[w];
    block_partial[blockIdx.x] = s;
    __threadfence();
    last = atomicAdd(ticket, 1u) == gridDim.x - 1;
  }
  __syncthreads();
  if (!last || threadIdx.x >= 32) return;
  __threadfence();
  float s = 0.0f;
  for (unsigned i = lane; i < gridDim.x; i += 32) s += __ldcg(block_partial + i);
  s = warp_sum(s);
  if (lane == 0) {
    loss_dev[0] = s * inv_div;
    *ticket = 0;
  }
}

// loss_dev[0] = (sum_b row_loss[b]) * inv_div, one block, fixed summation tree.
__global__ void __launch_bounds__(1024)
ce_mean_kernel(const float* __restrict__ row_loss, float* __restrict__ loss_dev, int batch, float inv_div) {
  NRS_PDL_PROLOGUE();
  __shared__ float sm[32];
  float s = 0.0f;
  int i = threadIdx.x;
  const int step = blockDim.x;
  for (; i + 7 * step < batch; i += 8 * step) {   // eight loads in flight; the additions keep the order of i
    float v[8];
#pragma unroll
    for (int u = 0; u < 8; ++u) v[u] = row_loss[i + u * step];
#pragma unroll
    for (int u = 0; u < 8; ++u) s += v[u];
  }
  for (; i < batch; i += step) s += row_loss[i];
  s = warp_sum(s);
  if ((threadIdx.x & 31) == 0) sm[threadIdx.x >> 5] = s;
  __syncthreads();
  if (threadIdx.x < 32) {
    float t = threadIdx.x < (blockDim.x >> 5) ? sm[threadIdx.x] : 0.0f;
    t = warp_sum(t);
    if (threadIdx.x == 0) loss_dev[0] = t * inv_div;
  }
}

int run_ce(nrs_ctx* ctx, const char* who, const float* logits, const float* target, const int32_t* labels, float* loss_dev,
           float* row_loss, float* grad, int batch, int classes, int divisor) {
  NRS_REQUIRE(ctx, batch >= 0 && classes > 0, NRS_ERR_SHAPE, "%s: bad shape [%d,%d]", who, batch, classes);
  NRS_REQUIRE(ctx, divisor > 0, NRS_ERR_ARG, "%s: divisor must be positive", who);
  if (batch == 0) {
    if (loss_dev) NRS_CUDA(ctx, cudaMemsetAsync(loss_dev, 0, sizeof(float), ctx->stream));
    return NRS_OK;
  }
  NRS_REQUIRE(ctx, logits && (target || labels), NRS_ERR_ARG, "%s: null tensor", who);
  const float inv_div = 1.0f / (float)divisor;
  int blocks = (batch + 7) / 8;
  if (blocks > ctx->sm_count * 8) blocks = ctx->sm_count * 8;
  // wide rows: one resident wave (three blocks of 80 registers per SM) of warps that walk several rows each,
  // prefetching the next
  if (classes > 512 && blocks > ctx->sm_count * 3) blocks = ctx->sm_count * 3;
  const bool vec = classes % 4 == 0 && classes <= 1024 &&
                   ((reinterpret_cast<uintptr_t>(logits) | reinterpret_cast<uintptr_t>(target) | reinterpret_cast<uintptr_t>(grad)) & 15) == 0;
  // the vector kernels fold the batch mean themselves (per-block partial sums, last block folds); the scalar
  // kernel leaves per-row losses to a second launch
  float* rl = row_loss;
  float* partial = nullptr;
  unsigned* ticket = nullptr;
  if (loss_dev) {
    void* ws = nullptr;
    int st = nrs_workspace(ctx, (size_t)(vec ? blocks : (rl ? 0 : batch)) * sizeof(float) + 16, &ws);
    if (st == NRS_OK && vec) st = nrs_fold_ticket(ctx, &ticket);
    if (st != NRS_OK) return st;
    if (vec) partial = (float*)ws;
    else if (!rl) rl = (float*)ws;
  }
  if (vec && classes <= 128) {
    NRS_PDL_LAUNCH(ce_rows_vec_kernel<1>, blocks, 256, 0, ctx->stream, logits, target, labels, row_loss, grad, batch, classes, inv_div,
                   partial, ticket, loss_dev);
  } else if (vec && classes <= 512) {
    NRS_PDL_LAUNCH(ce_rows_vec_kernel<4>, blocks, 256, 0, ctx->stream, logits, target, labels, row_loss, grad, batch, classes, inv_div,
                   partial, ticket, loss_dev);
  } else if (vec) {
    NRS_PDL_LAUNCH(ce_rows_vec_kernel<8>, blocks, 256, 0, ctx->stream, logits, target, labels, row_loss, grad, batch, classes, inv_div,
                   partial, ticket, loss_dev);
  } else {
    NRS_PDL_LAUNCH(ce_rows_kernel, blocks, 256, 0, ctx->stream, logits, target, labels, rl, grad, batch, classes, inv_div);
  }
  NRS_LAUNCHED(ctx);
  if (loss_dev && !vec) {
    NRS_PDL_LAUNCH(ce_mean_kernel, 1, 1024, 0, ctx->stream, rl, loss_dev, batch, inv_div);
    NRS_LAUNCHED(ctx);
  }
  return NRS_OK;
}

}  // namespace

extern "C" {

int nrs_ce_fwd(nrs_ctx* ctx, const float* logits, const float* target, float* loss_dev, float* row_loss,
               int batch, int classes, int divisor) {
  NRS_REQUIRE_CTX(ctx);
  NRS_REQUIRE(ctx, loss_dev || row_loss, NRS_ERR_ARG, "nrs_ce_fwd: no output requested");
  return run_ce(ctx, "nrs_ce_fwd", logits, target, nullptr, loss_dev, row_loss, nullptr, batch, classes, divisor);
}

int nrs_ce_bwd(nrs_ctx* ctx, const float* logits, const float* target, float* grad, int batch, int classes,
               int divisor) {
  NRS_REQUIRE_CTX(ctx);
  NRS_REQUIRE(ctx, grad || batch == 0, NRS_ERR_ARG, "nrs_ce_bwd: null grad");
  return run_ce(ctx, "nrs_ce_bwd", logits, target, nullptr, nullptr, nullptr, grad, batch, classes, divisor);
}

int nrs_ce_fwd_bwd(nrs_ctx* ctx, const float* logits, const float* target, float* loss_dev, float* grad,
                   int batch, int classes, int divisor) {
  NRS_REQUIRE_CTX(ctx);
  NRS_REQUIRE(ctx, loss_dev && (grad || batch == 0), NRS_ERR_ARG, "nrs_ce_fwd_bwd: null output");
  return run_ce(ctx, "nrs_ce_fwd_bwd", logits, target, nullptr, loss_dev, nullptr, grad, batch, classes, divisor);
}

int nrs_ce_fwd_bwd_indexed(nrs_ctx* ctx, const float* logits, const int32_t* labels, float* loss_dev, float* grad,
                           int batch, int classes, int divisor) {
  NRS_REQUIRE_CTX(ctx);
  NRS_REQUIRE(ctx, loss_dev && (grad || batch == 0), NRS_ERR_ARG, "nrs_ce_fwd_bwd_indexed: null output");
  NRS_REQUIRE(ctx, labels || batch == 0, NRS_ERR_ARG, "nrs_ce_fwd_bwd_indexed: null labels");
  return run_ce(ctx, "nrs_ce_fwd_bwd_indexed", logits, nullptr, labels, loss_dev, nullptr, grad, batch, classes, divisor);
}

}  // extern "C"
