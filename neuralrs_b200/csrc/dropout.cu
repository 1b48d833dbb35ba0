// Dropout and spatial dropout: the mask multiply of the reference (mask_mul, src/cuda/nn/dropout.rs:17-22;
// mask_mul_channels, src/cuda/nn/dropout2d.rs:18-27) and a device-side mask generator.
//
// The reference draws the mask on the host with the thread-local generator of the `rand` crate and uploads it
// (dropout.rs:45-48): a value per element, 0 with probability p, else 1/(1-p).  Uploading a mask per layer per
// step would put the host on the training path, so the mask is made on the device from a counter-based
// generator (Philox-4x32-10, Salmon et al., "Parallel random numbers: as easy as 1, 2, 3", SC'11): element i of
// a call is word i%4 of the block at counter (offset + i/4) under the context's 64-bit seed, u = (word >> 8) *
// 2^-24 in [0,1), mask = u < p ? 0 : 1/(1-p).  The same seed and offset give the same mask on any launch
// shape; a caller that wants the reference's own masks passes them to nrs_mask_mul instead.
#include "nrs_internal.h"
#include "philox.cuh"

namespace {

constexpr int kThreads = 256;

__device__ __forceinline__ float mask_value(uint32_t word, float p, float scale) {
  return nrs_rng::uniform01(word) < p ? 0.0f : scale;
}

__global__ void __launch_bounds__(kThreads)
dropout_mask_kernel(float* __restrict__ mask, size_t count, float p, float scale, uint64_t seed, uint64_t offset) {
  NRS_PDL_PROLOGUE();
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  const size_t blocks = (count + 3) / 4;
  const bool vec = (reinterpret_cast<uintptr_t>(mask) & 15) == 0;
  for (size_t b = (size_t)blockIdx.x * blockDim.x + threadIdx.x; b < blocks; b += stride) {
    uint32_t ctr[4];
    nrs_rng::block(seed, offset + b, ctr);
    const float4 v = make_float4(mask_value(ctr[0], p, scale), mask_value(ctr[1], p, scale),
                                 mask_value(ctr[2], p, scale), mask_value(ctr[3], p, scale));
    const size_t i = b * 4;
    if (vec && i + 4 <= count) {
      reinterpret_cast<float4*>(mask)[b] = v;
    } else {
      const float e[4] = {v.x, v.y, v.z, v.w};
      for (int j = 0; j < 4 && i + j < count; ++j) mask[i + j] = e[j];
    }
  }
}

// out (+)= a * mask[i / hw]; hw == 1 is the per-element mask.
template <bool VEC>
__global__ void __launch_bounds__(kThreads)
mask_mul_kernel(const float* __restrict__ a, const float* __restrict__ mask, float* out, size_t total, int hw,
                int accumulate) {
  NRS_PDL_PROLOGUE();
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  const size_t tid = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (VEC) {   // hw == 1 (a mask vector per data vector) or hw % 4 == 0 (one mask value per data vector)
    for (size_t i = tid; i < total / 4; i += stride) {
      const float4 v = reinterpret_cast<const float4*>(a)[i];
      float4 m;
      if (hw == 1) {
        m = reinterpret_cast<const float4*>(mask)[i];
      } else {
        const float s = mask[i * 4 / hw];
        m = make_float4(s, s, s, s);
      }
      float4 r = make_float4(v.x * m.x, v.y * m.y, v.z * m.z, v.w * m.w);
      float4* dst = reinterpret_cast<float4*>(out) + i;
      if (accumulate) {
        const float4 o = *dst;
        r = make_float4(o.x + r.x, o.y + r.y, o.z + r.z, o.w + r.w);
      }
      *dst = r;
    }
    if (tid < (total & 3)) {   // tail of a per-element mask whose length is not a multiple of four
      const size_t i = (total & ~(size_t)3) + tid;
      const float r = a[i] * mask[i / hw];
      out[i] = accumulate ? out[i] + r : r;
    }
  } else {
    for (size_t i = tid; i < total; i += stride) {
      const float r = a[i] * mask[i / hw];
      out[i] = accumulate ? out[i] + r : r;
    }
  }
}

unsigned ew_blocks(const nrs_ctx* ctx, size_t work_items) {
  const size_t want = (work_items + kThreads - 1) / kThreads;
  const size_t cap = (size_t)ctx->sm_count * 16;
  return (unsigned)(want < 1 ? 1 : (want > cap ? cap : want));
}

}  // namespace

int nrs_rng_seed(nrs_ctx* ctx, uint64_t seed) {
  NRS_REQUIRE_CTX(ctx);
  ctx->rng_seed = seed;
  ctx->rng_offset = 0;
  return NRS_OK;
}

int nrs_rng_offset(nrs_ctx* ctx, uint64_t* offset) {
  NRS_REQUIRE_CTX(ctx);
  NRS_REQUIRE(ctx, offset, NRS_ERR_ARG, "nrs_rng_offset: null output");
  *offset = ctx->rng_offset;
  return NRS_OK;
}

int nrs_dropout_mask(nrs_ctx* ctx, float* mask, size_t count, float p) {
  NRS_REQUIRE_CTX(ctx);
  NRS_REQUIRE(ctx, p >= 0.0f && p <= 1.0f, NRS_ERR_ARG, "nrs_dropout_mask: probability %g outside [0,1]", (double)p);
  if (count == 0) return NRS_OK;
  NRS_REQUIRE(ctx, mask, NRS_ERR_ARG, "nrs_dropout_mask: null mask");
  const size_t blocks = (count + 3) / 4;
  // p == 1 drops everything (u < 1 always holds), so the infinite scale is never used: the reference's
  // 1/(1-p) is kept as it is (dropout.rs:38).
  const float scale = 1.0f / (1.0f - p);
  uint64_t first = 0, advance = 0;
  nrs_rng_window(ctx, count, &first, &advance);   // a data-parallel shard draws its samples' part of the global mask
  NRS_PDL_LAUNCH(dropout_mask_kernel, ew_blocks(ctx, blocks), kThreads, 0, ctx->stream, mask, count, p, scale, ctx->rng_seed,
                 first);
  NRS_LAUNCHED(ctx);
  ctx->rng_offset += advance;
  return NRS_OK;
}

int nrs_mask_mul(nrs_ctx* ctx, const float* a, const float* mask, float* out, size_t total, int hw, int accumulate) {
  NRS_REQUIRE_CTX(ctx);
  NRS_REQUIRE(ctx, hw >= 1, NRS_ERR_SHAPE, "nrs_mask_mul: bad plane size %d", hw);
  if (total == 0) return NRS_OK;
  NRS_REQUIRE(ctx, a && mask && out, NRS_ERR_ARG, "nrs_mask_mul: null tensor");
  NRS_REQUIRE(ctx, total % (size_t)hw == 0, NRS_ERR_SHAPE, "nrs_mask_mul: %zu elements are not whole planes of %d", total, hw);
  const bool al = (((uintptr_t)a | (uintptr_t)out) & 15) == 0;
  const bool vec = al && ((hw == 1 && ((uintptr_t)mask & 15) == 0) || (hw & 3) == 0);
  if (vec) {
    NRS_PDL_LAUNCH(mask_mul_kernel<true>, ew_blocks(ctx, total / 4 + 1), kThreads, 0, ctx->stream, a, mask, out, total, hw, accumulate);
  } else {
    NRS_PDL_LAUNCH(mask_mul_kernel<false>, ew_blocks(ctx, total), kThreads, 0, ctx->stream, a, mask, out, total, hw, accumulate);
  }
  NRS_LAUNCHED(ctx);
  return NRS_OK;
}
