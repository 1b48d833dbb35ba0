// LayerNorm and row softmax, forward and backward.  One warp per row with
// shuffle reductions (the reference runs one thread per row); the parameter
// gradients of LayerNorm are column sums reduced in two fixed-order stages.
// Reference: ln_forward / ln_reduce / ln_dx (src/cuda/nn/normalization.rs:14-78),
// softmax_forward / softmax_backward (src/cuda/graph/softmax.rs:12-35); CPU
// semantics src/nn/normalization.rs:38-103, src/autograd/graph/softmax.rs:23-60.
#include "nrs_internal.h"

namespace {

__device__ __forceinline__ float wsum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float wmax(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

__global__ void __launch_bounds__(256)
ln_fwd_kernel(const float* __restrict__ x, const float* __restrict__ gamma, const float* __restrict__ beta,
              float* __restrict__ y, float* __restrict__ xhat, float* __restrict__ istd_out, int rows, int f,
              float eps) {
  NRS_PDL_PROLOGUE();
  const int lane = threadIdx.x & 31, wpb = blockDim.x >> 5;
  for (int r = blockIdx.x * wpb + (threadIdx.x >> 5); r < rows; r += gridDim.x * wpb) {
    const float* row = x + (size_t)r * f;
    float s = 0.0f;
    for (int i = lane; i < f; i += 32) s += row[i];
    const float mean = wsum(s) / (float)f;
    float vs = 0.0f;
    for (int i = lane; i < f; i += 32) { const float d = row[i] - mean; vs += d * d; }
    const float var = wsum(vs) / (float)f;
    const float istd = 1.0f / sqrtf(var + eps);
    if (lane == 0 && istd_out) istd_out[r] = istd;
    for (int i = lane; i < f; i += 32) {
      const float xn = (row[i] - mean) * istd;
      if (xhat) xhat[(size_t)r * f + i] = xn;
      y[(size_t)r * f + i] = gamma[i] * xn + beta[i];
    }
  }
}

__global__ void __launch_bounds__(256)
ln_dx_kernel(const float* __restrict__ g, const float* __restrict__ xhat, const float* __restrict__ istd,
             const float* __restrict__ gamma, float* dx, int rows, int f, int accumulate) {
  NRS_PDL_PROLOGUE();
  const int lane = threadIdx.x & 31, wpb = blockDim.x >> 5;
  const float nf = (float)f;
  for (int r = blockIdx.x * wpb + (threadIdx.x >> 5); r < rows; r += gridDim.x * wpb) {
    const size_t st = (size_t)r * f;
    float s1 = 0.0f, s2 = 0.0f;
    for (int i = lane; i < f; i += 32) {
      const float dxh = g[st + i] * gamma[i];
      s1 += dxh;
      s2 += dxh * xhat[st + i];
    }
    s1 = wsum(s1);
    s2 = wsum(s2);
    const float is = istd[r];
    for (int i = lane; i < f; i += 32) {
      const float dxh = g[st + i] * gamma[i];
      const float v = is * (dxh - s1 / nf - xhat[st + i] * s2 / nf);
      dx[st + i] = accumulate ? dx[st + i] + v : v;
    }
  }
}

// dgamma[c] = sum_r g*xhat, dbeta[c] = sum_r g over a row split; 32 columns per block.
__global__ void __launch_bounds__(256)
ln_param_kernel(const float* __restrict__ g, const float* __restrict__ xhat, float* __restrict__ partial,
                int rows, int f, int splits) {
  NRS_PDL_PROLOGUE();
  __shared__ float sg[8][33], sb[8][33];
  const int lane = threadIdx.x & 31, wrp = threadIdx.x >> 5;
  const int c = blockIdx.x * 32 + lane, split = blockIdx.y;
  const int rows_per = (rows + splits - 1) / splits;
  const int r0 = split * rows_per, r1 = min(rows, r0 + rows_per);
  float dg = 0.0f, db = 0.0f;
  if (c < f)
    for (int r = r0 + wrp; r < r1; r += 8) {
      const float gv = g[(size_t)r * f + c];
      dg += gv * xhat[(size_t)r * f + c];
      db += gv;
    }
  sg[wrp][lane] = dg;
  sb[wrp][lane] = db;
  __syncthreads();
  if (wrp == 0 && c < f) {
    float tg = 0.0f, tb = 0.0f;
#pragma unroll
    for (int i = 0; i < 8; ++i) { tg += sg[i][lane]; tb += sb[i][lane]; }
    partial[((size_t)split * 2 + 0) * f + c] = tg;
    partial[((size_t)split * 2 + 1) * f + c] = tb;
  }
}
__global__ void ln_param_fold_kernel(const float* __restrict__ partial, float* dgamma, float* dbeta, int f,
                                     int splits, int accumulate) {
  NRS_PDL_PROLOGUE();
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= f) return;
  float tg = 0.0f, tb = 0.0f;
  for (int s = 0; s < splits; ++s) {
    tg += partial[((size_t)s * 2 + 0) * f + c];
    tb += partial[((size_t)s * 2 + 1) * f + c];
  }
  dgamma[c] = accumulate ? dgamma[c] + tg : tg;
  dbeta[c] = accumulate ? dbeta[c] + tb : tb;
}

__global__ void __launch_bounds__(256)
softmax_fwd_kernel(const float* __restrict__ x, float* __restrict__ y, int rows, int width) {
  NRS_PDL_PROLOGUE();
  const int lane = threadIdx.x & 31, wpb = blockDim.x >> 5;
  for (int r = blockIdx.x * wpb + (threadIdx.x >> 5); r < rows; r += gridDim.x * wpb) {
    const float* row = x + (size_t)r * width;
    float mx = -INFINITY;
    for (int i = lane; i < width; i += 32) mx = fmaxf(mx, row[i]);
    mx = wmax(mx);
    float s = 0.0f;
    for (int i = lane; i < width; i += 32) s += expf(row[i] - mx);
    s = wsum(s);
    for (int i = lane; i < width; i += 32) y[(size_t)r * width + i] = expf(row[i] - mx) / s;
  }
}

__global__ void __launch_bounds__(256)
softmax_bwd_kernel(const float* __restrict__ y, const float* __restrict__ g, float* dx, int rows, int width,
                   int accumulate) {
  NRS_PDL_PROLOGUE();
  const int lane = threadIdx.x & 31, wpb = blockDim.x >> 5;
  for (int r = blockIdx.x * wpb + (threadIdx.x >> 5); r < rows; r += gridDim.x * wpb) {
    const size_t st = (size_t)r * width;
    float dot = 0.0f;
    for (int i = lane; i < width; i += 32) dot += y[st + i] * g[st + i];
    dot = wsum(dot);
    for (int i = lane; i < width; i += 32) {
      const float v = y[st + i] * (g[st + i] - dot);
      dx[st + i] = accumulate ? dx[st + i] + v : v;
    }
  }
}

int row_grid(const nrs_ctx* ctx, int rows) {
  int blocks = (rows + 7) / 8;
  if (blocks > ctx->sm_count * 8) blocks = ctx->sm_count * 8;
  return blocks < 1 ? 1 : blocks;
}

}  // namespace

extern "C" {

int nrs_layernorm_fwd(nrs_ctx* ctx, const float* x, const float* gamma, const float* beta, float* y,
                      float* xhat, float* istd, int rows, int f, float eps) {
  NRS_REQUIRE_CTX(ctx);
  NRS_REQUIRE(ctx, rows >= 0 && f > 0, NRS_ERR_SHAPE, "nrs_layernorm_fwd: bad shape [%d,%d]", rows, f);
  if (rows == 0) return NRS_OK;
  NRS_REQUIRE(ctx, x && gamma && beta && y, NRS_ERR_ARG, "nrs_layernorm_fwd: null tensor");
  NRS_PDL_LAUNCH(ln_fwd_kernel, row_grid(ctx, rows), 256, 0, ctx->stream, x, gamma, beta, y, xhat, istd, rows, f, eps);
  NRS_LAUNCHED(ctx);
  return NRS_OK;
}

int nrs_layernorm_bwd(nrs_ctx* ctx, const float* g, const float* xhat, const float* istd, const float* gamma,
                      float* dx, float* dgamma, float* dbeta, int rows, int f, int accumulate_dx,
                      int accumulate_params) {
  NRS_REQUIRE_CTX(ctx);
  NRS_REQUIRE(ctx, rows >= 0 && f > 0, NRS_ERR_SHAPE, "nrs_layernorm_bwd: bad shape [%d,%d]", rows, f);
  NRS_REQUIRE(ctx, (dgamma == nullptr) == (dbeta == nullptr), NRS_ERR_ARG,
              "nrs_layernorm_bwd: dgamma and dbeta must be given together");
  if (rows == 0) {
    if (dgamma && !accumulate_params) {
      NRS_CUDA(ctx, cudaMemsetAsync(dgamma, 0, sizeof(float) * f, ctx->stream));
      NRS_CUDA(ctx, cudaMemsetAsync(dbeta, 0, sizeof(float) * f, ctx->stream));
    }
    return NRS_OK;
  }
  NRS_REQUIRE(ctx, g && xhat && istd && gamma, NRS_ERR_ARG, "nrs_layernorm_bwd: null tensor");
  if (dx) {
    NRS_PDL_LAUNCH(ln_dx_kernel, row_grid(ctx, rows), 256, 0, ctx->stream, g, xhat, istd, gamma, dx, rows, f, accumulate_dx);
    NRS_LAUNCHED(ctx);
  }
  if (dgamma) {
    const int col_blocks = (f + 31) / 32;
    int splits = (2 * ctx->sm_count + col_blocks - 1) / col_blocks;
    if (splits > rows / 32) splits = rows / 32;
    if (splits < 1) splits = 1;
    if (splits > 65535) splits = 65535;
    void* ws = nullptr;
    const int st = nrs_workspace(ctx, (size_t)splits * 2 * f * sizeof(float), &ws);
    if (st != NRS_OK) return st;
    NRS_PDL_LAUNCH(ln_param_kernel, dim3(col_blocks, splits), 256, 0, ctx->stream, g, xhat, (float*)ws, rows, f, splits);
    NRS_LAUNCHED(ctx);
    NRS_PDL_LAUNCH(ln_param_fold_kernel, nrs_blocks(f, 256), 256, 0, ctx->stream, (const float*)ws, dgamma, dbeta, f, splits,
                                                                      accumulate_params);
    NRS_LAUNCHED(ctx);
  }
  return NRS_OK;
}

int nrs_softmax_fwd(nrs_ctx* ctx, const float* x, float* y, int rows, int width) {
  NRS_REQUIRE_CTX(ctx);
  NRS_REQUIRE(ctx, rows >= 0 && width > 0, NRS_ERR_SHAPE, "nrs_softmax_fwd: bad shape [%d,%d]", rows, width);
  if (rows == 0) return NRS_OK;
  NRS_REQUIRE(ctx, x && y, NRS_ERR_ARG, "nrs_softmax_fwd: null tensor");
  NRS_PDL_LAUNCH(softmax_fwd_kernel, row_grid(ctx, rows), 256, 0, ctx->stream, x, y, rows, width);
  NRS_LAUNCHED(ctx);
  return NRS_OK;
}

int nrs_softmax_bwd(nrs_ctx* ctx, const float* y, const float* g, float* dx, int rows, int width, int accumulate) {
  NRS_REQUIRE_CTX(ctx);
  NRS_REQUIRE(ctx, rows >= 0 && width > 0, NRS_ERR_SHAPE, "nrs_softmax_bwd: bad shape [%d,%d]", rows, width);
  if (rows == 0) return NRS_OK;
  NRS_REQUIRE(ctx, y && g && dx, NRS_ERR_ARG, "nrs_softmax_bwd: null tensor");
  NRS_PDL_LAUNCH(softmax_bwd_kernel, row_grid(ctx, rows), 256, 0, ctx->stream, y, g, dx, rows, width, accumulate);
  NRS_LAUNCHED(ctx);
  return NRS_OK;
}

}  // extern "C"
