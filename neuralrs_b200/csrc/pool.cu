// Max pooling forward / backward.
// Reference: maxpool_forward / maxpool_backward (src/cuda/nn/maxpool.rs:19-55);
// CPU semantics src/nn/maxpool.rs:32-62 — strict '>' so the first maximum in
// row-major window order wins, argmax is the flat input index.
#include "nrs_internal.h"

namespace {

// 2x2 stride-2 windows: one thread per output pair-row reads two float2.
__global__ void __launch_bounds__(256)
maxpool2x2_fwd_kernel(const float* __restrict__ x, float* __restrict__ y, int32_t* __restrict__ argmax,
                      size_t planes, int h, int w, int oh, int ow) {
  NRS_PDL_PROLOGUE();
  const size_t total = planes * oh * ow;
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  const bool vec = (w & 1) == 0 && ((reinterpret_cast<uintptr_t>(x) & 7) == 0);
  for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += stride) {
    const int ox = (int)(idx % ow);
    const size_t t = idx / ow;
    const int oy = (int)(t % oh);
    const size_t pl = t / oh;
    const size_t first = (pl * h + 2 * oy) * w + 2 * ox;
    float v00, v01, v10, v11;
    if (vec) {
      const float2 r0 = *reinterpret_cast<const float2*>(x + first);
      const float2 r1 = *reinterpret_cast<const float2*>(x + first + w);
      v00 = r0.x; v01 = r0.y; v10 = r1.x; v11 = r1.y;
    } else {
      v00 = x[first]; v01 = x[first + 1]; v10 = x[first + w]; v11 = x[first + w + 1];
    }
    float best = v00; size_t bi = first;
    if (v01 > best) { best = v01; bi = first + 1; }
    if (v10 > best) { best = v10; bi = first + w; }
    if (v11 > best) { best = v11; bi = first + w + 1; }
    y[idx] = best;
    if (argmax) argmax[idx] = (int32_t)bi;
  }
}

__global__ void __launch_bounds__(256)
maxpool_fwd_kernel(const float* __restrict__ x, float* __restrict__ y, int32_t* __restrict__ argmax,
                   size_t planes, int h, int w, int k, int s, int oh, int ow) {
  NRS_PDL_PROLOGUE();
  const size_t total = planes * oh * ow;
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += stride) {
    const int ox = (int)(idx % ow);
    const size_t t = idx / ow;
    const int oy = (int)(t % oh);
    const size_t pl = t / oh;
    const size_t first = (pl * h + (size_t)oy * s) * w + (size_t)ox * s;
    float best = x[first];
    size_t bi = first;
    for (int i = 0; i < k; ++i)
      for (int j = 0; j < k; ++j) {
        const size_t in = first + (size_t)i * w + j;
        const float v = x[in];
        if (v > best) { best = v; bi = in; }
      }
    y[idx] = best;
    if (argmax) argmax[idx] = (int32_t)bi;
  }
}

// k == stride: windows do not overlap, so every input element has at most one
// window; dx is a pure gather through argmax (no atomics, deterministic).
__global__ void __launch_bounds__(256)
maxpool_bwd_gather_kernel(const float* __restrict__ g, const int32_t* __restrict__ argmax, float* dx,
                          size_t planes, int h, int w, int k, int oh, int ow, int accumulate) {
  NRS_PDL_PROLOGUE();
  const size_t total = planes * h * w;
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += stride) {
    const int ix = (int)(idx % w);
    const size_t t = idx / w;
    const int iy = (int)(t % h);
    const size_t pl = t / h;
    const int oy = iy / k, ox = ix / k;
    float v = 0.0f;
    if (oy < oh && ox < ow) {
      const size_t o = (pl * oh + oy) * ow + ox;
      if ((size_t)argmax[o] == idx) v = g[o];
    }
    dx[idx] = accumulate ? dx[idx] + v : v;
  }
}

__global__ void __launch_bounds__(256)
maxpool_bwd_scatter_kernel(const float* __restrict__ g, const int32_t* __restrict__ argmax, float* dx, size_t total) {
  NRS_PDL_PROLOGUE();
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += stride)
    atomicAdd(&dx[argmax[idx]], g[idx]);
}

unsigned grid_for(const nrs_ctx* ctx, size_t work) {
  size_t blocks = (work + 255) / 256;
  const size_t cap = (size_t)ctx->sm_count * 16;
  return (unsigned)(blocks > cap ? cap : (blocks ? blocks : 1));
}

int check_pool(nrs_ctx* ctx, const char* who, int n, int c, int h, int w, int k, int stride) {
  NRS_REQUIRE(ctx, n >= 0 && c >= 0 && h > 0 && w > 0, NRS_ERR_SHAPE, "%s: bad tensor dims", who);
  NRS_REQUIRE(ctx, k >= 1 && stride >= 1 && k <= h && k <= w, NRS_ERR_SHAPE,
              "%s: window %d / stride %d does not fit %dx%d", who, k, stride, h, w);
  NRS_REQUIRE(ctx, (size_t)n * c * h * w < ((size_t)1 << 31), NRS_ERR_UNSUPPORTED,
              "%s: input has 2^31 or more elements (argmax is int32)", who);
  return NRS_OK;
}

}  // namespace

extern "C" {

int nrs_maxpool_fwd(nrs_ctx* ctx, const float* x, float* y, int32_t* argmax, int n, int c, int h, int w,
                    int k, int stride) {
  NRS_REQUIRE_CTX(ctx);
  int st = check_pool(ctx, "nrs_maxpool_fwd", n, c, h, w, k, stride);
  if (st != NRS_OK) return st;
  const int oh = (h - k) / stride + 1, ow = (w - k) / stride + 1;
  const size_t planes = (size_t)n * c, total = planes * oh * ow;
  if (total == 0) return NRS_OK;
  NRS_REQUIRE(ctx, x && y, NRS_ERR_ARG, "nrs_maxpool_fwd: null tensor");
  if (k == 2 && stride == 2)
    NRS_PDL_LAUNCH(maxpool2x2_fwd_kernel, grid_for(ctx, total), 256, 0, ctx->stream, x, y, argmax, planes, h, w, oh, ow);
  else
    NRS_PDL_LAUNCH(maxpool_fwd_kernel, grid_for(ctx, total), 256, 0, ctx->stream, x, y, argmax, planes, h, w, k, stride, oh, ow);
  NRS_LAUNCHED(ctx);
  return NRS_OK;
}

int nrs_maxpool_bwd(nrs_ctx* ctx, const float* g, const int32_t* argmax, float* dx, int n, int c, int h,
                    int w, int k, int stride, int accumulate) {
  NRS_REQUIRE_CTX(ctx);
  int st = check_pool(ctx, "nrs_maxpool_bwd", n, c, h, w, k, stride);
  if (st != NRS_OK) return st;
  const int oh = (h - k) / stride + 1, ow = (w - k) / stride + 1;
  const size_t planes = (size_t)n * c, in_total = planes * h * w, out_total = planes * oh * ow;
  if (in_total == 0) return NRS_OK;
  NRS_REQUIRE(ctx, g && argmax && dx, NRS_ERR_ARG, "nrs_maxpool_bwd: null tensor");
  if (k == stride) {
    NRS_PDL_LAUNCH(maxpool_bwd_gather_kernel, grid_for(ctx, in_total), 256, 0, ctx->stream, g, argmax, dx, planes, h, w, k,
                                                                                oh, ow, accumulate);
    NRS_LAUNCHED(ctx);
  } else {
    if (!accumulate) NRS_CUDA(ctx, cudaMemsetAsync(dx, 0, in_total * sizeof(float), ctx->stream));
    NRS_PDL_LAUNCH(maxpool_bwd_scatter_kernel, grid_for(ctx, out_total), 256, 0, ctx->stream, g, argmax, dx, out_total);
    NRS_LAUNCHED(ctx);
  }
  return NRS_OK;
}

}  // extern "C"
