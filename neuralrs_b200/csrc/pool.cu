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

// 2x2 stride-2 windows on rows whose length is a multiple of four: one thread takes two neighbouring
// windows, i.e. one float4 from each of the two input rows, and writes a float2 of maxima and an int2 of
// argmax indices: every access of a warp is one contiguous 128-bit-per-lane segment.
__global__ void __launch_bounds__(256)
maxpool2x2_fwd_vec_kernel(const float* __restrict__ x, float* __restrict__ y, int32_t* __restrict__ argmax,
                          size_t planes, int h, int w, int oh, int ow) {
  NRS_PDL_PROLOGUE();
  const int owp = ow >> 1;
  const size_t total = planes * oh * owp;
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += stride) {
    const int oxp = (int)(idx % owp);
    const size_t t = idx / owp;
    const int oy = (int)(t % oh);
    const size_t pl = t / oh;
    const size_t first = (pl * h + 2 * oy) * w + 4 * oxp;
    const float4 r0 = __ldcs(reinterpret_cast<const float4*>(x + first));
    const float4 r1 = __ldcs(reinterpret_cast<const float4*>(x + first + w));
    float b0 = r0.x; size_t i0 = first;
    if (r0.y > b0) { b0 = r0.y; i0 = first + 1; }
    if (r1.x > b0) { b0 = r1.x; i0 = first + w; }
    if (r1.y > b0) { b0 = r1.y; i0 = first + w + 1; }
    float b1 = r0.z; size_t i1 = first + 2;
    if (r0.w > b1) { b1 = r0.w; i1 = first + 3; }
    if (r1.z > b1) { b1 = r1.z; i1 = first + w + 2; }
    if (r1.w > b1) { b1 = r1.w; i1 = first + w + 3; }
    const size_t o = (pl * oh + oy) * ow + 2 * oxp;
    *reinterpret_cast<float2*>(y + o) = make_float2(b0, b1);
    if (argmax) *reinterpret_cast<int2*>(argmax + o) = make_int2((int)i0, (int)i1);
  }
}

// Its backward pass: the thread that owns two neighbouring windows reads their float2 gradient and int2
// argmax and writes both rows of the two windows (one float4 each): the winners get the gradient, the
// rest zeros.  dx is written (or read-modified-written) exactly once, fully coalesced.
__global__ void __launch_bounds__(256)
maxpool2x2_bwd_vec_kernel(const float* __restrict__ g, const int32_t* __restrict__ argmax, float* dx, size_t planes,
                          int h, int w, int oh, int ow, int accumulate) {
  NRS_PDL_PROLOGUE();
  const int owp = ow >> 1;
  const size_t total = planes * oh * owp;
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += stride) {
    const int oxp = (int)(idx % owp);
    const size_t t = idx / owp;
    const int oy = (int)(t % oh);
    const size_t pl = t / oh;
    const size_t first = (pl * h + 2 * oy) * w + 4 * oxp;
    const size_t o = (pl * oh + oy) * ow + 2 * oxp;
    const float2 gv = __ldcs(reinterpret_cast<const float2*>(g + o));
    const int2 am = __ldcs(reinterpret_cast<const int2*>(argmax + o));
    const int a0 = am.x - (int)first, a1 = am.y - (int)first;        // 0, 1, w, w+1  /  2, 3, w+2, w+3
    float4 r0 = make_float4(a0 == 0 ? gv.x : 0.0f, a0 == 1 ? gv.x : 0.0f, a1 == 2 ? gv.y : 0.0f, a1 == 3 ? gv.y : 0.0f);
    float4 r1 = make_float4(a0 == w ? gv.x : 0.0f, a0 == w + 1 ? gv.x : 0.0f, a1 == w + 2 ? gv.y : 0.0f, a1 == w + 3 ? gv.y : 0.0f);
    float4* d0 = reinterpret_cast<float4*>(dx + first);
    float4* d1 = reinterpret_cast<float4*>(dx + first + w);
    if (accumulate) {
      const float4 o0 = *d0, o1 = *d1;
      r0.x += o0.x; r0.y += o0.y; r0.z += o0.z; r0.w += o0.w;
      r1.x += o1.x; r1.y += o1.y; r1.z += o1.z; r1.w += o1.w;
    }
    *d0 = r0;
    *d1 = r1;
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
  const bool vec2 = k == 2 && stride == 2 && w % 4 == 0 && h % 2 == 0 &&
                    ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(y) | reinterpret_cast<uintptr_t>(argmax)) & 15) == 0;
  if (vec2)
    NRS_PDL_LAUNCH(maxpool2x2_fwd_vec_kernel, grid_for(ctx, total / 2), 256, 0, ctx->stream, x, y, argmax, planes, h, w, oh, ow);
  else if (k == 2 && stride == 2)
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
  const bool vec2 = k == 2 && stride == 2 && w % 4 == 0 && h % 2 == 0 &&
                    ((reinterpret_cast<uintptr_t>(g) | reinterpret_cast<uintptr_t>(dx) | reinterpret_cast<uintptr_t>(argmax)) & 15) == 0;
  if (vec2) {
    // every input element lies in exactly one window (h and w even): the windows' owners write all of dx
    NRS_PDL_LAUNCH(maxpool2x2_bwd_vec_kernel, grid_for(ctx, out_total / 2), 256, 0, ctx->stream, g, argmax, dx, planes, h, w, oh,
                   ow, accumulate);
    NRS_LAUNCHED(ctx);
  } else if (k == stride) {
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
