// LayerNorm and row softmax, forward and backward.
//
// One warp owns a row and keeps it in registers: rows whose width is a multiple of four (up to
// 1024 floats) are read ONCE with 128-bit loads — lane l takes the float4s l, l+32, l+64, ... so every
// load instruction of the warp covers 512 contiguous bytes — reduced with shuffles, and written once.
// Other widths run scalar loops with the same arithmetic.  The LayerNorm backward pass produces the
// input gradient (optionally into two destinations: the fused residual add) and the parameter
// gradients from one read of g and xhat: every warp keeps column partials of dgamma / dbeta in
// registers over the rows it visits, the block folds its warps in warp order through shared memory,
// and a second small kernel folds the blocks in block order — fixed order, no atomics, bit-reproducible.
// (The reference runs one thread per row and three kernels.)
// Reference: ln_forward / ln_reduce / ln_dx (src/cuda/nn/normalization.rs:14-78),
// softmax_forward / softmax_backward (src/cuda/graph/softmax.rs:12-35); CPU
// semantics src/nn/normalization.rs:38-103, src/autograd/graph/softmax.rs:23-60.
#include "nrs_internal.h"
#include "tc_common.cuh"

namespace {

// The TF32 operand planes of a value that the next tensor-core GEMM will read (rows x f, the tensor's own
// layout): written by the producing kernel so that no separate staging pass reads the tensor again.
__device__ __forceinline__ void put_planes(float* hi, float* lo, size_t at, float4 v) {
  const float4 h = make_float4(tc::tf32_rn(v.x), tc::tf32_rn(v.y), tc::tf32_rn(v.z), tc::tf32_rn(v.w));
  *reinterpret_cast<float4*>(hi + at) = h;
  if (lo) *reinterpret_cast<float4*>(lo + at) = make_float4(v.x - h.x, v.y - h.y, v.z - h.z, v.w - h.w);
}

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

constexpr int kMaxVpl = 8;                 // float4s per lane: rows of up to 32 * 4 * 8 = 1024 floats
constexpr int kRowThreads = 256;

__device__ __forceinline__ float4 ld4(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ void st4(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
// streaming variants for tensors that are read or written exactly once
__device__ __forceinline__ float4 ld4_stream(const float* p) { return __ldcs(reinterpret_cast<const float4*>(p)); }
__device__ __forceinline__ void st4_stream(float* p, float4 v) { __stcs(reinterpret_cast<float4*>(p), v); }

// ------------------------------------------------------------------ LayerNorm forward
// x = a (+ b when given: the residual add folded in); y = gamma * xhat + beta.
// EMIT: also write the TF32 planes of y (a separate instantiation, so that the plain kernel keeps its registers).
template <int VPL, bool EMIT>
__global__ void __launch_bounds__(kRowThreads)
ln_fwd_vec_kernel(const float* __restrict__ a, const float* __restrict__ b, const float* __restrict__ gamma,
                  const float* __restrict__ beta, float* __restrict__ y, float* __restrict__ xhat,
                  float* __restrict__ istd_out, int rows, int f, float eps, float* __restrict__ y_hi,
                  float* __restrict__ y_lo) {
  NRS_PDL_PROLOGUE();
  const int lane = threadIdx.x & 31, wpb = blockDim.x >> 5;
  const int f4 = f >> 2;
  const float inv_f = 1.0f / (float)f;
  for (int r = blockIdx.x * wpb + (threadIdx.x >> 5); r < rows; r += gridDim.x * wpb) {
    const size_t base = (size_t)r * f;
    float4 v[VPL];
    float s = 0.0f;
#pragma unroll
    for (int k = 0; k < VPL; ++k) {
      const int c = lane + 32 * k;
      v[k] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
      if (c < f4) {
        v[k] = ld4_stream(a + base + 4 * c);
        if (b) {
          const float4 w = ld4_stream(b + base + 4 * c);
          v[k].x += w.x; v[k].y += w.y; v[k].z += w.z; v[k].w += w.w;
        }
        s += (v[k].x + v[k].y) + (v[k].z + v[k].w);
      }
    }
    const float mean = wsum(s) * inv_f;
    float vs = 0.0f;
#pragma unroll
    for (int k = 0; k < VPL; ++k)
      if (lane + 32 * k < f4) {
        const float dx = v[k].x - mean, dy = v[k].y - mean, dz = v[k].z - mean, dw = v[k].w - mean;
        vs += (dx * dx + dy * dy) + (dz * dz + dw * dw);
      }
    const float istd = 1.0f / sqrtf(wsum(vs) * inv_f + eps);
    if (lane == 0 && istd_out) istd_out[r] = istd;
#pragma unroll
    for (int k = 0; k < VPL; ++k) {
      const int c = lane + 32 * k;
      if (c < f4) {
        const float4 gm = ld4(gamma + 4 * c), bt = ld4(beta + 4 * c);
        float4 xn;
        xn.x = (v[k].x - mean) * istd; xn.y = (v[k].y - mean) * istd;
        xn.z = (v[k].z - mean) * istd; xn.w = (v[k].w - mean) * istd;
        if (xhat) st4_stream(xhat + base + 4 * c, xn);
        const float4 out = make_float4(gm.x * xn.x + bt.x, gm.y * xn.y + bt.y, gm.z * xn.z + bt.z, gm.w * xn.w + bt.w);
        st4_stream(y + base + 4 * c, out);
        if (EMIT) put_planes(y_hi, y_lo, base + 4 * c, out);
      }
    }
  }
}

__global__ void __launch_bounds__(kRowThreads)
ln_fwd_kernel(const float* __restrict__ a, const float* __restrict__ b, const float* __restrict__ gamma,
              const float* __restrict__ beta, float* __restrict__ y, float* __restrict__ xhat,
              float* __restrict__ istd_out, int rows, int f, float eps) {
  NRS_PDL_PROLOGUE();
  const int lane = threadIdx.x & 31, wpb = blockDim.x >> 5;
  for (int r = blockIdx.x * wpb + (threadIdx.x >> 5); r < rows; r += gridDim.x * wpb) {
    const float* ra = a + (size_t)r * f;
    const float* rb = b ? b + (size_t)r * f : nullptr;
    float s = 0.0f;
    for (int i = lane; i < f; i += 32) s += rb ? ra[i] + rb[i] : ra[i];
    const float mean = wsum(s) / (float)f;
    float vs = 0.0f;
    for (int i = lane; i < f; i += 32) { const float d = (rb ? ra[i] + rb[i] : ra[i]) - mean; vs += d * d; }
    const float var = wsum(vs) / (float)f;
    const float istd = 1.0f / sqrtf(var + eps);
    if (lane == 0 && istd_out) istd_out[r] = istd;
    for (int i = lane; i < f; i += 32) {
      const float xn = ((rb ? ra[i] + rb[i] : ra[i]) - mean) * istd;
      if (xhat) xhat[(size_t)r * f + i] = xn;
      y[(size_t)r * f + i] = gamma[i] * xn + beta[i];
    }
  }
}

// ------------------------------------------------------------------ LayerNorm backward
// dx (+)= istd * (g*gamma - mean(g*gamma) - xhat * mean(g*gamma*xhat)), optionally also into dx2 (the
// second addend of a fused residual add receives the same gradient); per-block column partials of
// dgamma = sum_r g*xhat and dbeta = sum_r g into partial[block][2][f] when `partial` is given.
template <int VPL, bool EMIT>
__global__ void __launch_bounds__(kRowThreads)
ln_bwd_vec_kernel(const float* __restrict__ g, const float* __restrict__ xhat, const float* __restrict__ istd,
                  const float* __restrict__ gamma, float* dx, float* dx2, float* __restrict__ partial, int rows, int f,
                  int acc1, int acc2, float* __restrict__ d_hi, float* __restrict__ d_lo) {
  NRS_PDL_PROLOGUE();
  extern __shared__ float ln_smem[];          // [warps][2][f] when partial != nullptr
  const int lane = threadIdx.x & 31, wrp = threadIdx.x >> 5, wpb = blockDim.x >> 5;
  const int f4 = f >> 2;
  const float inv_f = 1.0f / (float)f;
  float4 gm[VPL], pg[VPL], pb[VPL];
#pragma unroll
  for (int k = 0; k < VPL; ++k) {
    const int c = lane + 32 * k;
    gm[k] = c < f4 ? ld4(gamma + 4 * c) : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    pg[k] = pb[k] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
  }
  for (int r = blockIdx.x * wpb + wrp; r < rows; r += gridDim.x * wpb) {
    const size_t base = (size_t)r * f;
    float4 gv[VPL], xh[VPL];
    float s1 = 0.0f, s2 = 0.0f;
#pragma unroll
    for (int k = 0; k < VPL; ++k) {
      const int c = lane + 32 * k;
      gv[k] = xh[k] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
      if (c < f4) {
        gv[k] = ld4_stream(g + base + 4 * c);
        xh[k] = ld4_stream(xhat + base + 4 * c);
        if (partial) {
          pg[k].x += gv[k].x * xh[k].x; pg[k].y += gv[k].y * xh[k].y; pg[k].z += gv[k].z * xh[k].z; pg[k].w += gv[k].w * xh[k].w;
          pb[k].x += gv[k].x; pb[k].y += gv[k].y; pb[k].z += gv[k].z; pb[k].w += gv[k].w;
        }
        gv[k].x *= gm[k].x; gv[k].y *= gm[k].y; gv[k].z *= gm[k].z; gv[k].w *= gm[k].w;    // dxhat
        s1 += (gv[k].x + gv[k].y) + (gv[k].z + gv[k].w);
        s2 += (gv[k].x * xh[k].x + gv[k].y * xh[k].y) + (gv[k].z * xh[k].z + gv[k].w * xh[k].w);
      }
    }
    if (dx) {
      s1 = wsum(s1) * inv_f;
      s2 = wsum(s2) * inv_f;
      const float is = istd[r];
#pragma unroll
      for (int k = 0; k < VPL; ++k) {
        const int c = lane + 32 * k;
        if (c < f4) {
          float4 o;
          o.x = is * (gv[k].x - s1 - xh[k].x * s2); o.y = is * (gv[k].y - s1 - xh[k].y * s2);
          o.z = is * (gv[k].z - s1 - xh[k].z * s2); o.w = is * (gv[k].w - s1 - xh[k].w * s2);
          if (EMIT) put_planes(d_hi, d_lo, base + 4 * c, o);   // planes of the gradient itself (before any accumulation)
          float4 w = o;
          if (acc1) { const float4 old = ld4(dx + base + 4 * c); w.x += old.x; w.y += old.y; w.z += old.z; w.w += old.w; }
          st4(dx + base + 4 * c, w);
          if (dx2) {
            if (acc2) { const float4 old = ld4(dx2 + base + 4 * c); o.x += old.x; o.y += old.y; o.z += old.z; o.w += old.w; }
            st4(dx2 + base + 4 * c, o);
          }
        }
      }
    }
  }
  if (partial) {
    float* mine = ln_smem + (size_t)wrp * 2 * f;
#pragma unroll
    for (int k = 0; k < VPL; ++k) {
      const int c = lane + 32 * k;
      if (c < f4) { st4(mine + 4 * c, pg[k]); st4(mine + f + 4 * c, pb[k]); }
    }
    __syncthreads();
    float* out = partial + (size_t)blockIdx.x * 2 * f;
    for (int i = threadIdx.x; i < 2 * f; i += blockDim.x) {
      float t = 0.0f;
      for (int w = 0; w < wpb; ++w) t += ln_smem[(size_t)w * 2 * f + i];     // warp order
      out[i] = t;
    }
  }
}

__global__ void __launch_bounds__(kRowThreads)
ln_dx_kernel(const float* __restrict__ g, const float* __restrict__ xhat, const float* __restrict__ istd,
             const float* __restrict__ gamma, float* dx, float* dx2, int rows, int f, int acc1, int acc2) {
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
      dx[st + i] = acc1 ? dx[st + i] + v : v;
      if (dx2) dx2[st + i] = acc2 ? dx2[st + i] + v : v;
    }
  }
}

// Scalar path of the parameter gradients: dgamma[c] = sum_r g*xhat, dbeta[c] = sum_r g over a row split;
// 32 columns per block.
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
// partial[part][2][f] folded over the parts: a block owns 32 of the 2f columns; its eight warps each
// sum every eighth part (128-byte row segments, coalesced), and the eight sums are combined in warp
// order — a fixed order of additions whatever the launch shape.
__global__ void __launch_bounds__(256)
ln_param_fold_kernel(const float* __restrict__ partial, float* dgamma, float* dbeta, int f, int parts, int accumulate) {
  NRS_PDL_PROLOGUE();
  __shared__ float sm[8][33];
  const int lane = threadIdx.x & 31, wrp = threadIdx.x >> 5;
  const int c = blockIdx.x * 32 + lane;          // column of the [2f]-wide partial rows
  float t = 0.0f;
  if (c < 2 * f) {
    // four loads in flight per thread; the additions keep the order s = wrp, wrp + 8, ...
    const size_t step = (size_t)8 * 2 * f;
    const float* src = partial + (size_t)wrp * 2 * f + c;
    int s = wrp;
    for (; s + 24 < parts; s += 32, src += 4 * step) {
      const float v0 = src[0], v1 = src[step], v2 = src[2 * step], v3 = src[3 * step];
      t += v0; t += v1; t += v2; t += v3;
    }
    for (; s < parts; s += 8, src += step) t += *src;
  }
  sm[wrp][lane] = t;
  __syncthreads();
  if (wrp != 0 || c >= 2 * f) return;
  float sum = 0.0f;
#pragma unroll
  for (int w = 0; w < 8; ++w) sum += sm[w][lane];
  float* dst = c < f ? dgamma + c : dbeta + (c - f);
  *dst = accumulate ? *dst + sum : sum;
}

// ------------------------------------------------------------------ softmax
template <int VPL>
__global__ void __launch_bounds__(kRowThreads)
softmax_fwd_vec_kernel(const float* __restrict__ x, float* __restrict__ y, int rows, int width) {
  NRS_PDL_PROLOGUE();
  const int lane = threadIdx.x & 31, wpb = blockDim.x >> 5;
  const int w4 = width >> 2;
  for (int r = blockIdx.x * wpb + (threadIdx.x >> 5); r < rows; r += gridDim.x * wpb) {
    const size_t base = (size_t)r * width;
    float4 v[VPL];
    float mx = -INFINITY;
#pragma unroll
    for (int k = 0; k < VPL; ++k) {
      const int c = lane + 32 * k;
      if (c < w4) {
        v[k] = ld4_stream(x + base + 4 * c);
        mx = fmaxf(mx, fmaxf(fmaxf(v[k].x, v[k].y), fmaxf(v[k].z, v[k].w)));
      }
    }
    mx = wmax(mx);
    float s = 0.0f;
#pragma unroll
    for (int k = 0; k < VPL; ++k)
      if (lane + 32 * k < w4) {
        v[k].x = expf(v[k].x - mx); v[k].y = expf(v[k].y - mx); v[k].z = expf(v[k].z - mx); v[k].w = expf(v[k].w - mx);
        s += (v[k].x + v[k].y) + (v[k].z + v[k].w);
      }
    s = wsum(s);
#pragma unroll
    for (int k = 0; k < VPL; ++k) {
      const int c = lane + 32 * k;
      if (c < w4) st4_stream(y + base + 4 * c, make_float4(v[k].x / s, v[k].y / s, v[k].z / s, v[k].w / s));
    }
  }
}

__global__ void __launch_bounds__(kRowThreads)
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

template <int VPL>
__global__ void __launch_bounds__(kRowThreads)
softmax_bwd_vec_kernel(const float* __restrict__ y, const float* __restrict__ g, float* dx, int rows, int width,
                       int accumulate) {
  NRS_PDL_PROLOGUE();
  const int lane = threadIdx.x & 31, wpb = blockDim.x >> 5;
  const int w4 = width >> 2;
  for (int r = blockIdx.x * wpb + (threadIdx.x >> 5); r < rows; r += gridDim.x * wpb) {
    const size_t base = (size_t)r * width;
    float4 yv[VPL], gv[VPL];
    float dot = 0.0f;
#pragma unroll
    for (int k = 0; k < VPL; ++k) {
      const int c = lane + 32 * k;
      if (c < w4) {
        yv[k] = ld4_stream(y + base + 4 * c);
        gv[k] = ld4_stream(g + base + 4 * c);
        dot += (yv[k].x * gv[k].x + yv[k].y * gv[k].y) + (yv[k].z * gv[k].z + yv[k].w * gv[k].w);
      }
    }
    dot = wsum(dot);
#pragma unroll
    for (int k = 0; k < VPL; ++k) {
      const int c = lane + 32 * k;
      if (c < w4) {
        float4 o = make_float4(yv[k].x * (gv[k].x - dot), yv[k].y * (gv[k].y - dot), yv[k].z * (gv[k].z - dot),
                               yv[k].w * (gv[k].w - dot));
        if (accumulate) { const float4 old = ld4(dx + base + 4 * c); o.x += old.x; o.y += old.y; o.z += old.z; o.w += old.w; }
        st4(dx + base + 4 * c, o);
      }
    }
  }
}

__global__ void __launch_bounds__(kRowThreads)
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

int row_grid(const nrs_ctx* ctx, int rows, int warps_per_block = 8) {
  int blocks = (rows + warps_per_block - 1) / warps_per_block;
  if (blocks > ctx->sm_count * 8) blocks = ctx->sm_count * 8;
  return blocks < 1 ? 1 : blocks;
}

// float4s per lane for a row of `width` floats, or 0 when the vector path does not apply.
int vec_vpl(int width, std::initializer_list<const void*> ptrs) {
  if (width % 4 != 0 || width > 32 * 4 * kMaxVpl) return 0;
  for (const void* p : ptrs)
    if (reinterpret_cast<uintptr_t>(p) & 15) return 0;
  const int f4 = width / 4;
  return f4 <= 32 ? 1 : f4 <= 64 ? 2 : f4 <= 128 ? 4 : 8;
}

#define NRS_DISPATCH_VPL(vpl, CALL) \
  do {                              \
    switch (vpl) {                  \
      case 1: { constexpr int V = 1; CALL; } break; \
      case 2: { constexpr int V = 2; CALL; } break; \
      case 4: { constexpr int V = 4; CALL; } break; \
      default: { constexpr int V = 8; CALL; } break; \
    }                               \
  } while (0)

int layernorm_fwd(nrs_ctx* ctx, const char* who, const float* a, const float* b, const float* gamma, const float* beta,
                  float* y, float* xhat, float* istd, int rows, int f, float eps, float* y_hi = nullptr, float* y_lo = nullptr,
                  int* emitted = nullptr) {
  if (emitted) *emitted = 0;
  NRS_REQUIRE(ctx, rows >= 0 && f > 0, NRS_ERR_SHAPE, "%s: bad shape [%d,%d]", who, rows, f);
  if (rows == 0) return NRS_OK;
  NRS_REQUIRE(ctx, a && gamma && beta && y, NRS_ERR_ARG, "%s: null tensor", who);
  const int vpl = vec_vpl(f, {a, b, gamma, beta, y, xhat, y_hi, y_lo});
  if (vpl) {
    if (y_hi)
      NRS_DISPATCH_VPL(vpl, NRS_PDL_LAUNCH((ln_fwd_vec_kernel<V, true>), row_grid(ctx, rows), kRowThreads, 0, ctx->stream, a, b, gamma,
                                           beta, y, xhat, istd, rows, f, eps, y_hi, y_lo));
    else
      NRS_DISPATCH_VPL(vpl, NRS_PDL_LAUNCH((ln_fwd_vec_kernel<V, false>), row_grid(ctx, rows), kRowThreads, 0, ctx->stream, a, b, gamma,
                                           beta, y, xhat, istd, rows, f, eps, y_hi, y_lo));
    if (emitted && y_hi) *emitted = 1;
  } else {
    NRS_PDL_LAUNCH(ln_fwd_kernel, row_grid(ctx, rows), kRowThreads, 0, ctx->stream, a, b, gamma, beta, y, xhat, istd, rows, f, eps);
  }
  NRS_LAUNCHED(ctx);
  return NRS_OK;
}

int layernorm_bwd(nrs_ctx* ctx, const char* who, const float* g, const float* xhat, const float* istd, const float* gamma,
                  float* dx, float* dx2, float* dgamma, float* dbeta, int rows, int f, int acc1, int acc2, int accumulate_params,
                  float* d_hi = nullptr, float* d_lo = nullptr, int* emitted = nullptr) {
  if (emitted) *emitted = 0;
  NRS_REQUIRE(ctx, rows >= 0 && f > 0, NRS_ERR_SHAPE, "%s: bad shape [%d,%d]", who, rows, f);
  NRS_REQUIRE(ctx, (dgamma == nullptr) == (dbeta == nullptr), NRS_ERR_ARG, "%s: dgamma and dbeta must be given together", who);
  NRS_REQUIRE(ctx, dx || !dx2, NRS_ERR_ARG, "%s: a second input gradient without the first", who);
  if (rows == 0) {
    if (dgamma && !accumulate_params) {
      NRS_CUDA(ctx, cudaMemsetAsync(dgamma, 0, sizeof(float) * f, ctx->stream));
      NRS_CUDA(ctx, cudaMemsetAsync(dbeta, 0, sizeof(float) * f, ctx->stream));
    }
    return NRS_OK;
  }
  NRS_REQUIRE(ctx, g && xhat && istd && gamma, NRS_ERR_ARG, "%s: null tensor", who);
  if (!dx && !dgamma) return NRS_OK;
  const int vpl = vec_vpl(f, {g, xhat, gamma, dx, dx2, d_hi, d_lo});
  if (vpl) {
    // one pass over g and xhat for everything; the block size keeps the per-warp column partials within 32 KB
    int warps = 8;
    while (dgamma && warps > 1 && (size_t)warps * 2 * f * sizeof(float) > 32 * 1024) warps >>= 1;
    int blocks = row_grid(ctx, rows, warps);
    if (dgamma && blocks > 4 * ctx->sm_count) blocks = 4 * ctx->sm_count;   // one resident wave of longer-lived blocks: fewer partial rows to fold
    float* partial = nullptr;
    if (dgamma) {
      void* ws = nullptr;
      const int st = nrs_workspace(ctx, (size_t)blocks * 2 * f * sizeof(float), &ws);
      if (st != NRS_OK) return st;
      partial = (float*)ws;
    }
    const size_t smem = dgamma ? (size_t)warps * 2 * f * sizeof(float) : 0;
    if (dx && d_hi)
      NRS_DISPATCH_VPL(vpl, NRS_PDL_LAUNCH((ln_bwd_vec_kernel<V, true>), blocks, warps * 32, smem, ctx->stream, g, xhat, istd, gamma, dx,
                                           dx2, partial, rows, f, acc1, acc2, d_hi, d_lo));
    else
      NRS_DISPATCH_VPL(vpl, NRS_PDL_LAUNCH((ln_bwd_vec_kernel<V, false>), blocks, warps * 32, smem, ctx->stream, g, xhat, istd, gamma, dx,
                                           dx2, partial, rows, f, acc1, acc2, (float*)nullptr, (float*)nullptr));
    if (emitted && dx && d_hi) *emitted = 1;
    NRS_LAUNCHED(ctx);
    if (dgamma) {
      NRS_PDL_LAUNCH(ln_param_fold_kernel, nrs_blocks(2 * (size_t)f, 32), 256, 0, ctx->stream, (const float*)partial, dgamma, dbeta, f,
                     blocks, accumulate_params);
      NRS_LAUNCHED(ctx);
    }
    return NRS_OK;
  }
  if (dx) {
    NRS_PDL_LAUNCH(ln_dx_kernel, row_grid(ctx, rows), kRowThreads, 0, ctx->stream, g, xhat, istd, gamma, dx, dx2, rows, f, acc1, acc2);
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
    NRS_PDL_LAUNCH(ln_param_fold_kernel, nrs_blocks(2 * (size_t)f, 32), 256, 0, ctx->stream, (const float*)ws, dgamma, dbeta, f, splits,
                   accumulate_params);
    NRS_LAUNCHED(ctx);
  }
  return NRS_OK;
}

}  // namespace

extern "C" {

int nrs_layernorm_fwd(nrs_ctx* ctx, const float* x, const float* gamma, const float* beta, float* y,
                      float* xhat, float* istd, int rows, int f, float eps) {
  NRS_REQUIRE_CTX(ctx);
  return layernorm_fwd(ctx, "nrs_layernorm_fwd", x, nullptr, gamma, beta, y, xhat, istd, rows, f, eps);
}

int nrs_layernorm_residual_fwd(nrs_ctx* ctx, const float* a, const float* b, const float* gamma, const float* beta, float* y,
                               float* xhat, float* istd, int rows, int f, float eps) {
  NRS_REQUIRE_CTX(ctx);
  NRS_REQUIRE(ctx, b != nullptr || rows == 0, NRS_ERR_ARG, "nrs_layernorm_residual_fwd: null second addend");
  return layernorm_fwd(ctx, "nrs_layernorm_residual_fwd", a, b, gamma, beta, y, xhat, istd, rows, f, eps);
}

int nrs_layernorm_bwd(nrs_ctx* ctx, const float* g, const float* xhat, const float* istd, const float* gamma,
                      float* dx, float* dgamma, float* dbeta, int rows, int f, int accumulate_dx,
                      int accumulate_params) {
  NRS_REQUIRE_CTX(ctx);
  return layernorm_bwd(ctx, "nrs_layernorm_bwd", g, xhat, istd, gamma, dx, nullptr, dgamma, dbeta, rows, f, accumulate_dx, 0,
                       accumulate_params);
}

int nrs_layernorm_residual_bwd(nrs_ctx* ctx, const float* g, const float* xhat, const float* istd, const float* gamma,
                               float* da, float* db, float* dgamma, float* dbeta, int rows, int f, int accumulate_da,
                               int accumulate_db, int accumulate_params) {
  NRS_REQUIRE_CTX(ctx);
  // the gradient of a + b is the same for both addends; either may be absent
  float* first = da ? da : db;
  float* second = da ? db : nullptr;
  const int acc_first = da ? accumulate_da : accumulate_db;
  return layernorm_bwd(ctx, "nrs_layernorm_residual_bwd", g, xhat, istd, gamma, first, second, dgamma, dbeta, rows, f, acc_first,
                       accumulate_db, accumulate_params);
}

// The same two operators with the TF32 planes of their result written by the kernel itself (y forward; the
// input gradient backward): *emitted = 1 when the planes were written (vector path), 0 when the caller has
// to stage them itself.  Internal: the graph's fused transformer block calls them.
int nrs_layernorm_fwd_planes(nrs_ctx* ctx, const float* a, const float* b, const float* gamma, const float* beta, float* y,
                             float* xhat, float* istd, int rows, int f, float eps, float* y_hi, float* y_lo, int* emitted) {
  NRS_REQUIRE_CTX(ctx);
  return layernorm_fwd(ctx, "nrs_layernorm_fwd_planes", a, b, gamma, beta, y, xhat, istd, rows, f, eps, y_hi, y_lo, emitted);
}

int nrs_layernorm_bwd_planes(nrs_ctx* ctx, const float* g, const float* xhat, const float* istd, const float* gamma, float* da,
                             float* db, float* dgamma, float* dbeta, int rows, int f, int accumulate_da, int accumulate_db,
                             int accumulate_params, float* d_hi, float* d_lo, int* emitted) {
  NRS_REQUIRE_CTX(ctx);
  float* first = da ? da : db;
  float* second = da ? db : nullptr;
  const int acc_first = da ? accumulate_da : accumulate_db;
  return layernorm_bwd(ctx, "nrs_layernorm_bwd_planes", g, xhat, istd, gamma, first, second, dgamma, dbeta, rows, f, acc_first,
                       accumulate_db, accumulate_params, d_hi, d_lo, emitted);
}

int nrs_softmax_fwd(nrs_ctx* ctx, const float* x, float* y, int rows, int width) {
  NRS_REQUIRE_CTX(ctx);
  NRS_REQUIRE(ctx, rows >= 0 && width > 0, NRS_ERR_SHAPE, "nrs_softmax_fwd: bad shape [%d,%d]", rows, width);
  if (rows == 0) return NRS_OK;
  NRS_REQUIRE(ctx, x && y, NRS_ERR_ARG, "nrs_softmax_fwd: null tensor");
  const int vpl = vec_vpl(width, {x, y});
  if (vpl) {
    NRS_DISPATCH_VPL(vpl, NRS_PDL_LAUNCH(softmax_fwd_vec_kernel<V>, row_grid(ctx, rows), kRowThreads, 0, ctx->stream, x, y, rows, width));
  } else {
    NRS_PDL_LAUNCH(softmax_fwd_kernel, row_grid(ctx, rows), kRowThreads, 0, ctx->stream, x, y, rows, width);
  }
  NRS_LAUNCHED(ctx);
  return NRS_OK;
}

int nrs_softmax_bwd(nrs_ctx* ctx, const float* y, const float* g, float* dx, int rows, int width, int accumulate) {
  NRS_REQUIRE_CTX(ctx);
  NRS_REQUIRE(ctx, rows >= 0 && width > 0, NRS_ERR_SHAPE, "nrs_softmax_bwd: bad shape [%d,%d]", rows, width);
  if (rows == 0) return NRS_OK;
  NRS_REQUIRE(ctx, y && g && dx, NRS_ERR_ARG, "nrs_softmax_bwd: null tensor");
  const int vpl = vec_vpl(width, {y, g, dx});
  if (vpl) {
    NRS_DISPATCH_VPL(vpl, NRS_PDL_LAUNCH(softmax_bwd_vec_kernel<V>, row_grid(ctx, rows), kRowThreads, 0, ctx->stream, y, g, dx, rows,
                                         width, accumulate));
  } else {
    NRS_PDL_LAUNCH(softmax_bwd_kernel, row_grid(ctx, rows), kRowThreads, 0, ctx->stream, y, g, dx, rows, width, accumulate);
  }
  NRS_LAUNCHED(ctx);
  return NRS_OK;
}

}  // extern "C"
