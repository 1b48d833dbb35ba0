// Direct convolution kernels for layers with very few input channels (the image
// layer of a CNN: c_in = 1 or 3, 3x3, stride 1).  With K = c_in*kh*kw = 9 or 27 the
// contraction is too short for a tensor-core K-block and a 128x128 implicit-GEMM
// tile is mostly padding, so these layers get their own FFMA kernels:
//   forward        TF32 modes: the same patch planes as the weight gradient, run through the
//                  tensor-core convolution kernel as a 1x1 layer (its epilogue adds the bias,
//                  the ReLU and the output's planes).  FP32 mode, FFMA:
//                  one thread per output pixel holds the K-element input patch in
//                  registers and sweeps the output channels against weights kept
//                  in shared memory (128-bit broadcast loads); stores are full
//                  128-byte lines per channel; on request the result is also
//                  written as NHWC TF32 planes for the tensor-core layer behind it
//   weight grad    TF32 modes: the patches are written out as [pixels][32] operand planes
//                  and the tensor-core weight-gradient kernel treats them as a 32-channel
//                  1x1 layer.  FP32 mode, FFMA:
//                  dW[co][k] = sum_p dy[p][co] * patch[p][k]: blocks stream pixel
//                  tiles through shared memory, each thread accumulates a 3 x 8
//                  (k x co) register tile; per-block partials are summed in a
//                  fixed order by a second kernel (deterministic)
// Exact f32.  Reference counterparts: conv2d_im2col + matmul_nn + col2out and
// im2col + matmul_nt_splitk (src/cuda/nn/conv.rs:244-320).
#include "igemm_problems.cuh"
#include "nrs_internal.h"
#include "tc_common.cuh"

namespace {

constexpr int kTileLd = 36;   // floats per pixel row of the plane-emission tile (16-byte aligned, spreads banks)

// EMIT: also write the result as NHWC TF32 planes (hi, and lo when non-null) for a tensor-core
// convolution that reads it next.  Each warp (32 consecutive pixels) passes 32 channels at a
// time through a shared-memory tile so that every plane store covers four full 128-byte lines.
template <int CI, int KS, bool EMIT>
__global__ void __launch_bounds__(256)
smallc_fwd_kernel(const float* __restrict__ x, const float* __restrict__ w, const float* __restrict__ b,
                  float* __restrict__ y, int n, int h, int wd, int co, int pad, int oh, int ow, int act,
                  float* __restrict__ hi, float* __restrict__ lo) {
  constexpr int K = CI * KS * KS;
  constexpr int K4 = (K + 3) / 4 * 4;
  extern __shared__ __align__(16) float smem_f[];
  float* w_s = smem_f;               // [co][K4]
  float* b_s = smem_f + (size_t)co * K4;
  // [warp][32 pixels][kTileLd], 16-byte aligned behind the bias
  float* tile = smem_f + (((size_t)co * K4 + co + 3) / 4 * 4) + (size_t)(threadIdx.x >> 5) * 32 * kTileLd;
  for (int i = threadIdx.x; i < co * K4; i += blockDim.x) {
    const int c = i / K4, k = i - c * K4;
    w_s[i] = k < K ? w[(size_t)c * K + k] : 0.0f;
  }
  for (int i = threadIdx.x; i < co; i += blockDim.x) b_s[i] = b ? b[i] : 0.0f;
  __syncthreads();
  const int lane = threadIdx.x & 31;
  const size_t plane = (size_t)oh * ow;
  const size_t total = (size_t)n * plane;
  // warp-uniform trip count: `base` is the warp's first pixel
  for (size_t base = (size_t)blockIdx.x * blockDim.x + (threadIdx.x - lane); base < total; base += (size_t)gridDim.x * blockDim.x) {
    const size_t p = base + lane;
    const bool live = p < total;
    const size_t img = live ? p / plane : 0;
    const int pix = live ? (int)(p - img * plane) : 0;
    const int oy = pix / ow, ox = pix - oy * ow;
    float patch[K4];
#pragma unroll
    for (int k = 0; k < K4; ++k) {
      float v = 0.0f;
      if (k < K && live) {
        const int c = k / (KS * KS), t = k - c * KS * KS, i = t / KS, j = t - i * KS;
        const int iy = oy + i - pad, ix = ox + j - pad;
        if ((unsigned)iy < (unsigned)h && (unsigned)ix < (unsigned)wd)
          v = x[((img * CI + c) * h + iy) * wd + ix];
      }
      patch[k] = v;
    }
    float* dst = y + img * co * plane + pix;
    for (int c0 = 0; c0 < co; c0 += 32) {
      const int cn = min(32, co - c0);
      for (int cc = 0; cc < cn; ++cc) {
        const int c = c0 + cc;
        float acc = b_s[c];
        const float4* wr = reinterpret_cast<const float4*>(w_s + (size_t)c * K4);
#pragma unroll
        for (int k4 = 0; k4 < K4 / 4; ++k4) {
          const float4 wv = wr[k4];
          acc = fmaf(patch[4 * k4 + 0], wv.x, acc);
          acc = fmaf(patch[4 * k4 + 1], wv.y, acc);
          acc = fmaf(patch[4 * k4 + 2], wv.z, acc);
          acc = fmaf(patch[4 * k4 + 3], wv.w, acc);
        }
        acc = nrs_apply_act(acc, act);
        if (live) dst[(size_t)c * plane] = acc;
        if (EMIT) tile[lane * kTileLd + cc] = acc;
      }
      if (EMIT) {   // co is a multiple of 32 on this path
        __syncwarp();
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const int pr = i * 4 + (lane >> 3), chunk = (lane & 7) * 4;
          const float4 v = *reinterpret_cast<const float4*>(tile + pr * kTileLd + chunk);
          if (base + pr < total) {
            const size_t o = (base + pr) * co + c0 + chunk;
            const float4 hv = make_float4(tc::tf32_rn(v.x), tc::tf32_rn(v.y), tc::tf32_rn(v.z), tc::tf32_rn(v.w));
            *reinterpret_cast<float4*>(hi + o) = hv;
            if (lo) *reinterpret_cast<float4*>(lo + o) = make_float4(v.x - hv.x, v.y - hv.y, v.z - hv.z, v.w - hv.w);
          }
        }
        __syncwarp();
      }
    }
  }
}

// Patch planes for the tensor-core weight gradient of an image layer: row p of the
// [pixels][32] matrix holds the K = CI*KS*KS input values under output pixel p (zeros
// beyond K and outside the image), as a TF32 high plane and, when lo != null, a residual
// plane.  Seen as an NHWC tensor with 32 channels, the layer's weight gradient is then a
// 1x1 convolution's: dW[co][k] = sum_p dy[p][co] * patch[p][k].
template <int CI, int KS>
__global__ void __launch_bounds__(256)
smallc_patch_planes_kernel(const float* __restrict__ x, float* __restrict__ hi, float* __restrict__ lo, int n, int h,
                           int wd, int pad, int oh, int ow) {
  NRS_PDL_PROLOGUE();
  constexpr int K = CI * KS * KS;
  static_assert(K <= 32, "patch must fit one 32-channel block");
  __shared__ __align__(16) float tiles[8][32 * kTileLd];
  float* tile = tiles[threadIdx.x >> 5];
  const int lane = threadIdx.x & 31;
  const size_t plane = (size_t)oh * ow;
  const size_t total = (size_t)n * plane;
  for (size_t base = (size_t)blockIdx.x * blockDim.x + (threadIdx.x - lane); base < total; base += (size_t)gridDim.x * blockDim.x) {
    const size_t p = base + lane;
    const bool live = p < total;
    const size_t img = live ? p / plane : 0;
    const int pix = live ? (int)(p - img * plane) : 0;
    const int oy = pix / ow, ox = pix - oy * ow;
#pragma unroll
    for (int k = 0; k < 32; ++k) {
      float v = 0.0f;
      if (k < K && live) {
        const int c = k / (KS * KS), t = k - c * KS * KS, i = t / KS, j = t - i * KS;
        const int iy = oy + i - pad, ix = ox + j - pad;
        if ((unsigned)iy < (unsigned)h && (unsigned)ix < (unsigned)wd) v = x[((img * CI + c) * h + iy) * wd + ix];
      }
      tile[lane * kTileLd + k] = v;
    }
    __syncwarp();
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int pr = i * 4 + (lane >> 3), chunk = (lane & 7) * 4;
      const float4 v = *reinterpret_cast<const float4*>(tile + pr * kTileLd + chunk);
      if (base + pr < total) {
        const size_t o = (base + pr) * 32 + chunk;
        const float4 hv = make_float4(tc::tf32_rn(v.x), tc::tf32_rn(v.y), tc::tf32_rn(v.z), tc::tf32_rn(v.w));
        *reinterpret_cast<float4*>(hi + o) = hv;
        if (lo) *reinterpret_cast<float4*>(lo + o) = make_float4(v.x - hv.x, v.y - hv.y, v.z - hv.z, v.w - hv.w);
      }
    }
    __syncwarp();
  }
}

// dw[co][k] (+)= wide[co][k] for k < K (wide rows are 32 long).
__global__ void __launch_bounds__(256)
smallc_narrow_kernel(const float* __restrict__ wide, float* __restrict__ dw, int co, int K, int accumulate) {
  NRS_PDL_PROLOGUE();
  const int idx = blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= co * K) return;
  const int c = idx / K, k = idx - c * K;
  const float v = wide[c * 32 + k];
  dw[idx] = accumulate ? dw[idx] + v : v;
}

constexpr int TP = 128;   // pixels per shared-memory tile (weight gradient)

template <int CI, int KS>
__global__ void __launch_bounds__(256)
smallc_wgrad_kernel(const float* __restrict__ x, const float* __restrict__ dy, float* __restrict__ partial, int n, int h,
                    int wd, int co, int pad, int oh, int ow, int tiles_per_img, int total_tiles, int ns) {
  constexpr int K = CI * KS * KS;
  constexpr int KG = K / 3;            // thread owns 3 consecutive k
  extern __shared__ __align__(16) float smem_f[];
  float* dy_s = smem_f;                               // [co][TP+1]
  float* pa_s = smem_f + (size_t)co * (TP + 1);       // [K][TP+1]
  const int cob = co / 8;
  const int t = threadIdx.x;
  const bool active = t < ns * KG * cob;
  const int kg = t % KG, cb = (t / KG) % cob, s = t / (KG * cob);
  float acc[3][8];
#pragma unroll
  for (int a = 0; a < 3; ++a)
#pragma unroll
    for (int c = 0; c < 8; ++c) acc[a][c] = 0.0f;
  const int plane = oh * ow;
  for (int tile = blockIdx.x; tile < total_tiles; tile += gridDim.x) {
    const int img = tile / tiles_per_img, p0 = (tile - img * tiles_per_img) * TP;
    const int tp = min(TP, plane - p0);
    __syncthreads();   // previous tile fully consumed
    for (int i = t; i < co * TP; i += blockDim.x) {
      const int c = i / TP, p = i - c * TP;
      dy_s[c * (TP + 1) + p] = p < tp ? dy[((size_t)img * co + c) * plane + p0 + p] : 0.0f;
    }
    for (int i = t; i < K * TP; i += blockDim.x) {
      const int k = i / TP, p = i - k * TP;
      float v = 0.0f;
      if (p < tp) {
        const int pix = p0 + p, oy = pix / ow, ox = pix - oy * ow;
        const int c = k / (KS * KS), tt = k - c * KS * KS, ii = tt / KS, jj = tt - ii * KS;
        const int iy = oy + ii - pad, ix = ox + jj - pad;
        if ((unsigned)iy < (unsigned)h && (unsigned)ix < (unsigned)wd)
          v = x[(((size_t)img * CI + c) * h + iy) * wd + ix];
      }
      pa_s[k * (TP + 1) + p] = v;
    }
    __syncthreads();
    if (active) {
      for (int p = s; p < tp; p += ns) {
        float a[3], d[8];
#pragma unroll
        for (int q = 0; q < 3; ++q) a[q] = pa_s[(3 * kg + q) * (TP + 1) + p];
#pragma unroll
        for (int c = 0; c < 8; ++c) d[c] = dy_s[(8 * cb + c) * (TP + 1) + p];
#pragma unroll
        for (int q = 0; q < 3; ++q)
#pragma unroll
          for (int c = 0; c < 8; ++c) acc[q][c] = fmaf(a[q], d[c], acc[q][c]);
      }
    }
  }
  if (active) {
    float* dst = partial + ((size_t)blockIdx.x * ns + s) * co * K;
#pragma unroll
    for (int q = 0; q < 3; ++q)
#pragma unroll
      for (int c = 0; c < 8; ++c) dst[(size_t)(8 * cb + c) * K + 3 * kg + q] = acc[q][c];
  }
}

__global__ void smallc_wgrad_reduce_kernel(const float* __restrict__ partial, float* dw, int parts, int len, int accumulate) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= len) return;
  float s = 0.0f;
  for (int z = 0; z < parts; ++z) s += partial[(size_t)z * len + i];
  dw[i] = accumulate ? dw[i] + s : s;
}

template <int CI, int KS, bool EMIT>
int run_fwd(nrs_ctx* ctx, const float* x, const float* w, const float* b, float* y, int n, int h, int wd, int co,
            int pad, int oh, int ow, int act, float* hi, float* lo) {
  constexpr int K4 = (CI * KS * KS + 3) / 4 * 4;
  size_t smem = (((size_t)co * K4 + co + 3) / 4 * 4) * sizeof(float);
  if (EMIT) smem += (size_t)8 * 32 * kTileLd * sizeof(float);
  static NrsSmemAttr attr;
  NRS_ENSURE_SMEM(ctx, attr, (smallc_fwd_kernel<CI, KS, EMIT>), smem);
  const size_t total = (size_t)n * oh * ow;
  size_t blocks = (total + 255) / 256;
  const size_t cap = (size_t)ctx->sm_count * 8;
  if (blocks > cap) blocks = cap;
  smallc_fwd_kernel<CI, KS, EMIT><<<(unsigned)blocks, 256, smem, ctx->stream>>>(x, w, b, y, n, h, wd, co, pad, oh, ow, act, hi, lo);
  NRS_LAUNCHED(ctx);
  return NRS_OK;
}

template <int CI, int KS>
int run_wgrad(nrs_ctx* ctx, const float* x, const float* dy, float* dw, int n, int h, int wd, int co, int pad, int oh,
              int ow, int accumulate) {
  constexpr int K = CI * KS * KS, KG = K / 3;
  const int cob = co / 8;
  int ns = 256 / (KG * cob);
  if (ns < 1) return NRS_ERR_UNSUPPORTED;
  if (ns > 8) ns = 8;
  const size_t smem = ((size_t)co + K) * (TP + 1) * sizeof(float);
  if (smem > 200 * 1024) return NRS_ERR_UNSUPPORTED;
  static NrsSmemAttr attr;
  NRS_ENSURE_SMEM(ctx, attr, (smallc_wgrad_kernel<CI, KS>), smem);
  const int plane = oh * ow;
  const int tiles_per_img = (plane + TP - 1) / TP;
  const long total_tiles = (long)tiles_per_img * n;
  if (total_tiles > 2147483647L) return NRS_ERR_UNSUPPORTED;
  int blocks = ctx->sm_count * 4;
  if (blocks > total_tiles) blocks = (int)total_tiles;
  void* ws = nullptr;
  const int st = nrs_workspace(ctx, (size_t)blocks * ns * co * K * sizeof(float), &ws);
  if (st != NRS_OK) return st;
  smallc_wgrad_kernel<CI, KS><<<blocks, 256, smem, ctx->stream>>>(x, dy, (float*)ws, n, h, wd, co, pad, oh, ow,
                                                                  tiles_per_img, (int)total_tiles, ns);
  NRS_LAUNCHED(ctx);
  smallc_wgrad_reduce_kernel<<<nrs_blocks((size_t)co * K, 256), 256, 0, ctx->stream>>>((const float*)ws, dw, blocks * ns,
                                                                                      co * K, accumulate);
  NRS_LAUNCHED(ctx);
  return NRS_OK;
}

// wide[co][32] = w[co][K] padded with zeros (the 32-"channel" 1x1 weights of the patch formulation).
__global__ void __launch_bounds__(256)
smallc_widen_kernel(const float* __restrict__ w, float* __restrict__ wide, int co, int K) {
  NRS_PDL_PROLOGUE();
  const int idx = blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= co * 32) return;
  const int c = idx >> 5, k = idx & 31;
  wide[idx] = k < K ? w[c * K + k] : 0.0f;
}

template <int CI, int KS>
int launch_patches(nrs_ctx* ctx, const float* x, float* hi, float* lo, int n, int h, int wd, int pad, int oh, int ow) {
  const size_t pixels = (size_t)n * oh * ow;
  size_t blocks = (pixels + 255) / 256;
  const size_t cap = (size_t)ctx->sm_count * 16;
  if (blocks > cap) blocks = cap;
  NRS_PDL_LAUNCH((smallc_patch_planes_kernel<CI, KS>), (unsigned)blocks, 256, 0, ctx->stream, x, hi, lo, n, h, wd, pad, oh, ow);
  NRS_LAUNCHED(ctx);
  return NRS_OK;
}

// The patch planes of x: the caller's registered ones, or fresh ones in pool blocks (*owned).
template <int CI, int KS>
int get_patches(nrs_ctx* ctx, const float* x, int n, int h, int wd, int pad, int oh, int ow, float** hi, float** lo, bool* owned) {
  const bool split = ctx->math_mode == NRS_MATH_3XTF32;
  *owned = false;
  auto it = ctx->patch_hints.find(x);
  // (`split` of a patch hint: bit 0 = residual plane present, bits 8.. = the padding it was made for)
  if (it != ctx->patch_hints.end() && ((it->second.split & 1) != 0) == split && (it->second.split >> 8) == pad) {
    *hi = it->second.hi;
    *lo = it->second.lo;
    return NRS_OK;
  }
  const size_t pixels = (size_t)n * oh * ow;
  void *phi = nullptr, *plo = nullptr;
  int st = nrs_alloc(ctx, pixels * 32 * sizeof(float), 0, &phi);
  if (st == NRS_OK && split) st = nrs_alloc(ctx, pixels * 32 * sizeof(float), 0, &plo);
  if (st == NRS_OK) st = launch_patches<CI, KS>(ctx, x, (float*)phi, (float*)plo, n, h, wd, pad, oh, ow);
  if (st != NRS_OK) {
    if (phi) nrs_free(ctx, phi);
    if (plo) nrs_free(ctx, plo);
    return st;
  }
  *hi = (float*)phi;
  *lo = (float*)plo;
  *owned = true;
  return NRS_OK;
}

// Tensor-core route (TF32 modes): with the input written out as patch planes the layer is a 1x1
// convolution over 32 "channels", and the general tensor-core kernels run it.
template <int CI, int KS>
int run_wgrad_tc(nrs_ctx* ctx, const float* x, const float* dy, float* dw, int n, int h, int wd, int co, int pad, int oh,
                 int ow, int accumulate) {
  constexpr int K = CI * KS * KS;
  const bool split = ctx->math_mode == NRS_MATH_3XTF32;
  float *phi = nullptr, *plo = nullptr;
  bool owned = false;
  int st = get_patches<CI, KS>(ctx, x, n, h, wd, pad, oh, ow, &phi, &plo, &owned);
  if (st != NRS_OK) return st;
  void* wide = nullptr;
  st = nrs_alloc(ctx, (size_t)co * 32 * sizeof(float), 0, &wide);
  if (st == NRS_OK) {
    ctx->plane_hints[phi] = NrsPlanes{phi, plo, split ? 1 : 0};
    ctx->independent_next = false;   // phi was written by the kernel just launched
    st = nrs_tc_conv_wgrad(ctx, phi, dy, (float*)wide, n, 32, oh, ow, co, 1, 1, 1, 0, 0);
    ctx->plane_hints.erase(phi);
  }
  if (st == NRS_OK) {
    NRS_PDL_LAUNCH(smallc_narrow_kernel, nrs_blocks((size_t)co * K, 256), 256, 0, ctx->stream, (const float*)wide, dw, co, K, accumulate);
    ctx->launches++;
    if (cudaGetLastError() != cudaSuccess) st = NRS_ERR_CUDA;
  }
  if (owned) {
    nrs_free(ctx, phi);
    if (plo) nrs_free(ctx, plo);
  }
  if (wide) nrs_free(ctx, wide);
  return st;
}

template <int CI, int KS>
int run_fwd_tc(nrs_ctx* ctx, const float* x, const float* w, const float* b, float* y, int n, int h, int wd, int co, int pad,
               int oh, int ow, int act) {
  constexpr int K = CI * KS * KS;
  const bool split = ctx->math_mode == NRS_MATH_3XTF32;
  float *phi = nullptr, *plo = nullptr;
  bool owned = false;
  int st = get_patches<CI, KS>(ctx, x, n, h, wd, pad, oh, ow, &phi, &plo, &owned);
  if (st != NRS_OK) return st;
  void* wide = nullptr;
  st = nrs_alloc(ctx, (size_t)co * 32 * sizeof(float), 0, &wide);
  if (st == NRS_OK) {
    NRS_PDL_LAUNCH(smallc_widen_kernel, nrs_blocks((size_t)co * 32, 256), 256, 0, ctx->stream, w, (float*)wide, co, K);
    ctx->launches++;
    if (cudaGetLastError() != cudaSuccess) st = NRS_ERR_CUDA;
  }
  if (st == NRS_OK) {
    ctx->plane_hints[phi] = NrsPlanes{phi, plo, split ? 1 : 0};
    st = nrs_tc_conv_fwd(ctx, phi, (const float*)wide, b, y, n, 32, oh, ow, co, 1, 1, 1, 0, act);
    ctx->plane_hints.erase(phi);
  }
  if (owned) {
    nrs_free(ctx, phi);
    if (plo) nrs_free(ctx, plo);
  }
  if (wide) nrs_free(ctx, wide);
  return st;
}

bool eligible(int ci, int kh, int kw, int stride, int co) {
  return stride == 1 && kh == 3 && kw == 3 && (ci == 1 || ci == 3) && co >= 8 && co % 8 == 0 && co <= 256;
}

}  // namespace

// NRS_ERR_UNSUPPORTED when the layer is not a 3x3 stride-1 convolution over 1 or 3 channels.
int nrs_smallc_conv_fwd(nrs_ctx* ctx, const float* x, const float* w, const float* b, float* y, int n, int ci, int h,
                        int wd, int co, int kh, int kw, int stride, int pad, int act) {
  if (!eligible(ci, kh, kw, stride, co)) return NRS_ERR_UNSUPPORTED;
  const int oh = h + 2 * pad - 2, ow = wd + 2 * pad - 2;
  if (ctx->math_mode != NRS_MATH_FP32 && co % 32 == 0 && (long)n * oh * ow >= 4096) {
    const int st = ci == 1 ? run_fwd_tc<1, 3>(ctx, x, w, b, y, n, h, wd, co, pad, oh, ow, act)
                           : run_fwd_tc<3, 3>(ctx, x, w, b, y, n, h, wd, co, pad, oh, ow, act);
    if (st != NRS_ERR_UNSUPPORTED) return st;
  }
  // Planes of the result requested by the caller (a tensor-core convolution reads it next)?
  float *hi = nullptr, *lo = nullptr;
  auto extras = ctx->out_extras.find(y);
  if (extras != ctx->out_extras.end() && !extras->second.relu_mask_src && extras->second.hi && co % 32 == 0) {
    hi = extras->second.hi;
    lo = extras->second.lo;
    ctx->out_extras.erase(extras);   // honoured
  }
  if (hi) {
    if (ci == 1) return run_fwd<1, 3, true>(ctx, x, w, b, y, n, h, wd, co, pad, oh, ow, act, hi, lo);
    return run_fwd<3, 3, true>(ctx, x, w, b, y, n, h, wd, co, pad, oh, ow, act, hi, lo);
  }
  if (ci == 1) return run_fwd<1, 3, false>(ctx, x, w, b, y, n, h, wd, co, pad, oh, ow, act, nullptr, nullptr);
  return run_fwd<3, 3, false>(ctx, x, w, b, y, n, h, wd, co, pad, oh, ow, act, nullptr, nullptr);
}

int nrs_smallc_patch_planes(nrs_ctx* ctx, const float* x, float* hi, float* lo, int n, int ci, int h, int wd, int pad) {
  const int oh = h + 2 * pad - 2, ow = wd + 2 * pad - 2;
  if ((ci != 1 && ci != 3) || oh < 1 || ow < 1 || n < 1) return NRS_ERR_UNSUPPORTED;
  return ci == 1 ? launch_patches<1, 3>(ctx, x, hi, lo, n, h, wd, pad, oh, ow) : launch_patches<3, 3>(ctx, x, hi, lo, n, h, wd, pad, oh, ow);
}

int nrs_smallc_conv_wgrad(nrs_ctx* ctx, const float* x, const float* dy, float* dw, int n, int ci, int h, int wd, int co,
                          int kh, int kw, int stride, int pad, int accumulate) {
  if (!eligible(ci, kh, kw, stride, co) || co > 128) return NRS_ERR_UNSUPPORTED;
  const int oh = h + 2 * pad - 2, ow = wd + 2 * pad - 2;
  if (ctx->math_mode != NRS_MATH_FP32 && co % 32 == 0 && (long)n * oh * ow >= 4096) {
    const int st = ci == 1 ? run_wgrad_tc<1, 3>(ctx, x, dy, dw, n, h, wd, co, pad, oh, ow, accumulate)
                           : run_wgrad_tc<3, 3>(ctx, x, dy, dw, n, h, wd, co, pad, oh, ow, accumulate);
    if (st != NRS_ERR_UNSUPPORTED) return st;
  }
  if (ci == 1) return run_wgrad<1, 3>(ctx, x, dy, dw, n, h, wd, co, pad, oh, ow, accumulate);
  return run_wgrad<3, 3>(ctx, x, dy, dw, n, h, wd, co, pad, oh, ow, accumulate);
}
