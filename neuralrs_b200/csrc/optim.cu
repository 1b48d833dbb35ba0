// Fused multi-tensor AdamW: one launch over the model's flat parameter,
// gradient and moment vectors.  HBM-bound: 16 B read + 12 B written per
// parameter, moved as 128-bit accesses.
// Reference: `adamw` kernel, one launch per parameter tensor
// (src/cuda/optim/adamw.rs:19-35, host loop :84-107); CPU semantics
// src/optim/adamw.rs:23-46 (decoupled decay on the pre-update parameter).
#include "nrs_internal.h"

namespace {

struct AdamWArgs {
  float lr, b1, b2, eps, wd, bc1, bc2, gscale;
};

__device__ __forceinline__ void adamw_one(float& p, float g, float& m, float& v, const AdamWArgs& a) {
  g *= a.gscale;
  m = a.b1 * m + (1.0f - a.b1) * g;
  v = a.b2 * v + (1.0f - a.b2) * g * g;
  const float m_hat = m / a.bc1;
  const float v_hat = v / a.bc2;
  p = p - a.lr * m_hat / (sqrtf(v_hat) + a.eps) - a.lr * a.wd * p;
}

__global__ void __launch_bounds__(256)
adamw_kernel(float* __restrict__ p, const float* __restrict__ g, float* __restrict__ m, float* __restrict__ v,
             size_t n, AdamWArgs a) {
  NRS_PDL_PROLOGUE();
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  const size_t tid = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  const bool vec = ((reinterpret_cast<uintptr_t>(p) | reinterpret_cast<uintptr_t>(g) |
                     reinterpret_cast<uintptr_t>(m) | reinterpret_cast<uintptr_t>(v)) & 15) == 0;
  const size_t n4 = vec ? n / 4 : 0;
  for (size_t i = tid; i < n4; i += stride) {
    float4 pp = reinterpret_cast<float4*>(p)[i];
    const float4 gg = reinterpret_cast<const float4*>(g)[i];
    float4 mm = reinterpret_cast<float4*>(m)[i];
    float4 vv = reinterpret_cast<float4*>(v)[i];
    adamw_one(pp.x, gg.x, mm.x, vv.x, a);
    adamw_one(pp.y, gg.y, mm.y, vv.y, a);
    adamw_one(pp.z, gg.z, mm.z, vv.z, a);
    adamw_one(pp.w, gg.w, mm.w, vv.w, a);
    reinterpret_cast<float4*>(p)[i] = pp;
    reinterpret_cast<float4*>(m)[i] = mm;
    reinterpret_cast<float4*>(v)[i] = vv;
  }
  for (size_t i = n4 * 4 + tid; i < n; i += stride) adamw_one(p[i], g[i], m[i], v[i], a);
}

}  // namespace

extern "C" int nrs_adamw_step(nrs_ctx* ctx, float* p, const float* grad, float* m, float* v, size_t n,
                              float lr, float beta1, float beta2, float eps, float wd, float bc1, float bc2,
                              float grad_scale) {
  NRS_REQUIRE_CTX(ctx);
  if (n == 0) return NRS_OK;
  NRS_REQUIRE(ctx, p && grad && m && v, NRS_ERR_ARG, "nrs_adamw_step: null vector");
  NRS_REQUIRE(ctx, bc1 != 0.0f && bc2 != 0.0f, NRS_ERR_ARG, "nrs_adamw_step: zero bias correction");
  size_t blocks = (n / 4 + 255) / 256 + 1;
  const size_t cap = (size_t)ctx->sm_count * 16;
  if (blocks > cap) blocks = cap;
  NrsProfScope prof(ctx, NRS_PROF_ADAMW, 28.0 * (double)n);
  const AdamWArgs a{lr, beta1, beta2, eps, wd, bc1, bc2, grad_scale};
  NRS_PDL_LAUNCH(adamw_kernel, (unsigned)blocks, 256, 0, ctx->stream, p, grad, m, v, n, a);
  NRS_LAUNCHED(ctx);
  return NRS_OK;
}
