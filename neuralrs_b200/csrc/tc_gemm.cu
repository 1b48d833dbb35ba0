// Dense / batched GEMM on the 5th-generation tensor cores (tcgen05), TF32 and
// 3xTF32:  C[b][m,n] = act(op(A[b]) . op(B[b]) + bias[n]) + beta * C.
//
// The main loop is tc_mainloop.cuh (TMA -> 128B-swizzled smem ring -> tcgen05.mma
// kind::tf32 -> TMEM -> tcgen05.ld epilogue); this file supplies the GEMM policy
// (dense K-major row slices, row-major store with bias/activation/accumulate) and
// operand preparation.  Both operands are consumed K-major: an operand stored
// the other way round is transposed by the staging pass, which for 3xTF32 also
// writes the high/residual planes.  Plain TF32 reads untransposed, 16-byte
// aligned operands in place.
//
// Reference counterparts: matmul_nn / matmul_nt / matmul_tn, 64x64x16 FFMA tiles
// (src/cuda/graph/matmul.rs:44-198); bmm kernels (src/cuda/graph/bmm.rs:12-56).
#include "tc_mainloop.cuh"

namespace {

struct GemmPolicy {
  float* C;
  const float* bias;
  int act;
  float beta;
  int M, N;
  size_t batch_stride;
  bool vec_ok;
  float* pre;   // optional second output: the value before the activation (what GELU's derivative needs)
  static constexpr bool kCanEmit = false;

  __device__ __forceinline__ uint32_t a_slice_bytes() const { return tc::BM * tc::BK * 4; }
  __device__ __forceinline__ void load_a(void* dst, const CUtensorMap* tm, uint64_t* bar, int kb, int tile_m, int batch) const {
    tc::tma_load_3d(dst, tm, bar, kb * tc::BK, tile_m * tc::BM, batch);
  }
  __device__ __forceinline__ void store(int tile_m, int batch, int row, int n, float v) const {
    const int m = tile_m * tc::BM + row;
    if (m >= M || n >= N) return;
    float* dst = C + (size_t)batch * batch_stride + (size_t)m * N + n;
    if (bias) v += bias[n];
    if (pre) pre[(size_t)batch * batch_stride + (size_t)m * N + n] = v;
    v = nrs_apply_act(v, act);
    if (beta != 0.0f) v += beta * *dst;
    *dst = v;
  }
  // 32 consecutive columns [nb, nb+32) of one accumulator row.
  __device__ __forceinline__ void epilogue(int tile_m, int batch, int row, int nb, int ncols, const uint32_t (&r)[32]) const {
    const int m = tile_m * tc::BM + row;
    if (m >= M || nb >= N) return;
    float* crow = C + (size_t)batch * batch_stride + (size_t)m * N;
    if (vec_ok && ncols == 32 && nb + 32 <= N) {
#pragma unroll
      for (int j = 0; j < 32; j += 4) {
        float4 v = make_float4(__uint_as_float(r[j]), __uint_as_float(r[j + 1]), __uint_as_float(r[j + 2]),
                               __uint_as_float(r[j + 3]));
        if (bias) {
          const float4 bv = *reinterpret_cast<const float4*>(bias + nb + j);
          v.x += bv.x; v.y += bv.y; v.z += bv.z; v.w += bv.w;
        }
        if (pre) *reinterpret_cast<float4*>(pre + (size_t)batch * batch_stride + (size_t)m * N + nb + j) = v;
        v.x = nrs_apply_act(v.x, act); v.y = nrs_apply_act(v.y, act);
        v.z = nrs_apply_act(v.z, act); v.w = nrs_apply_act(v.w, act);
        float4* dst = reinterpret_cast<float4*>(crow + nb + j);
        if (beta != 0.0f) {
          const float4 o = *dst;
          v.x += beta * o.x; v.y += beta * o.y; v.z += beta * o.z; v.w += beta * o.w;
        }
        *dst = v;
      }
    } else {
#pragma unroll
      for (int j = 0; j < 32; ++j) {
        const int n = nb + j;
        if (j < ncols && n < N) {
          float v = __uint_as_float(r[j]);
          if (bias) v += bias[n];
          if (pre) pre[(size_t)batch * batch_stride + (size_t)m * N + n] = v;
          v = nrs_apply_act(v, act);
          if (beta != 0.0f) v += beta * crow[n];
          crow[n] = v;
        }
      }
    }
  }
};

struct Operand {
  const float* hi;
  const float* lo;
  int ld;          // leading dimension in floats
  int kdim;        // K extent given to the tensor map (TMA zero-fills beyond it)
  size_t bstride;  // floats between batches
};

// Brings one operand into K-major planes.  stored_kmajor: memory is [rows][K]; else [K][rows].
int prepare_operand(nrs_ctx* ctx, const float* src, int rows, int K, int batch, bool stored_kmajor, bool split,
                    int ws_hi, int ws_lo, Operand* out, bool is_weight) {
  if (batch == 1) {
    const int ldk = (K + 31) / 32 * 32;
    // a weight staged ahead with the rest of the model's (weight_set.cu) ...
    if (is_weight) {
      const NrsWeightPlanes* wp = nrs_weight_planes_find(ctx, src, stored_kmajor ? NRS_WF_LINEAR_ROWS : NRS_WF_LINEAR_T);
      if (wp && wp->rows == rows && wp->K == K) {
        *out = Operand{wp->hi, wp->lo, ldk, ldk, (size_t)rows * ldk};
        return NRS_OK;
      }
    }
    // ... or an activation whose [rows][K] planes its producer or an earlier consumer left with the context
    if (stored_kmajor && K == ldk) {
      const NrsPlanes* ready = nrs_planes_find(ctx, src, split);
      if (ready && ready->rows == rows && ready->cols == K) {
        *out = Operand{ready->hi, ready->lo, ldk, ldk, (size_t)rows * ldk};
        return NRS_OK;
      }
    }
  }
  const bool direct = !split && stored_kmajor && (K % 4 == 0) && ((reinterpret_cast<uintptr_t>(src) & 15) == 0);
  if (direct) {
    *out = Operand{src, nullptr, K, K, (size_t)rows * K};
    return NRS_OK;
  }
  const int ldk = (K + 31) / 32 * 32;
  const size_t plane = (size_t)rows * ldk;
  void *phi = nullptr, *plo = nullptr;
  int st = nrs_ws_slot(ctx, ws_hi, plane * batch * sizeof(float), &phi);
  if (st != NRS_OK) return st;
  if (split) {
    st = nrs_ws_slot(ctx, ws_lo, plane * batch * sizeof(float), &plo);
    if (st != NRS_OK) return st;
  }
  st = nrs_tc_stage(ctx, src, (float*)phi, (float*)plo, rows, K, ldk, batch, (size_t)rows * K, plane, !stored_kmajor);
  if (st != NRS_OK) return st;
  *out = Operand{(const float*)phi, (const float*)plo, ldk, ldk, plane};
  return NRS_OK;
}

bool make_operand_map(CUtensorMap* tm, const float* base, const Operand& op, int rows, int batch, int box_rows) {
  const uint64_t dim[3] = {(uint64_t)op.kdim, (uint64_t)rows, (uint64_t)batch};
  const uint64_t str[2] = {(uint64_t)op.ld * 4, (uint64_t)op.bstride * 4};
  const uint32_t box[3] = {(uint32_t)tc::BK, (uint32_t)box_rows, 1};
  return tc::encode_tmap_f32(tm, base, 3, dim, str, box);
}

template <int BN, int NPLANES>
int run(nrs_ctx* ctx, const Operand& A, const Operand& B, int batch, int m, int n, int k, const GemmPolicy& pol) {
  CUtensorMap ta_hi, ta_lo, tb_hi, tb_lo;
  bool ok = make_operand_map(&ta_hi, A.hi, A, m, batch, tc::BM) && make_operand_map(&tb_hi, B.hi, B, n, batch, BN);
  if (NPLANES == 2) ok = ok && make_operand_map(&ta_lo, A.lo, A, m, batch, tc::BM) && make_operand_map(&tb_lo, B.lo, B, n, batch, BN);
  else { ta_lo = ta_hi; tb_lo = tb_hi; }
  NRS_REQUIRE(ctx, ok, NRS_ERR_CUDA, "tc_gemm: cuTensorMapEncodeTiled failed (m=%d n=%d k=%d)", m, n, k);
  return tc::launch<BN, NPLANES, GemmPolicy>(ctx, ta_hi, ta_lo, tb_hi, tb_lo, pol, (m + tc::BM - 1) / tc::BM, n, batch,
                                             (k + tc::BK - 1) / tc::BK);
}

}  // namespace

namespace {
// Waits on an mbarrier nobody ever arrives on, with the kernels' own bounded-wait primitive and a
// short limit, and reports the expiry the way they do.
__global__ void bounded_wait_probe_kernel(long long limit_clocks, int* __restrict__ err_flag) {
  __shared__ uint64_t bar;
  if (threadIdx.x == 0) {
    tc::mbar_init(&bar, 1);
    tc::fence_barrier_init();
    if (!tc::mbar_wait_limit(&bar, 0, limit_clocks)) atomicExch(err_flag, tc::kErrMmaWait);
  }
}
}  // namespace

extern "C" int nrs_selftest_bounded_wait(nrs_ctx* ctx, int64_t limit_clocks) {
  NRS_REQUIRE_CTX(ctx);
  NRS_REQUIRE(ctx, limit_clocks > 0 && limit_clocks <= 100000000, NRS_ERR_ARG,
              "nrs_selftest_bounded_wait: limit must be in (0, 1e8] clocks");
  int* err = nullptr;
  const int st = nrs_err_flag(ctx, &err);
  if (st != NRS_OK) return st;
  bounded_wait_probe_kernel<<<1, 32, 0, ctx->stream>>>((long long)limit_clocks, err);
  NRS_LAUNCHED(ctx);
  return NRS_OK;
}

namespace {
// Back-to-back tcgen05.mma.kind::tf32 (M = 128, N = 256, K = 8) on operands that never leave shared
// memory: the tensor pipe's own rate, with no TMA traffic and no epilogue.  One issuing thread per CTA,
// one CTA per SM; every wait is bounded.
__global__ void __launch_bounds__(128, 1) umma_rate_kernel(int iters, int* __restrict__ err_flag) {
  extern __shared__ uint8_t umma_rate_smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(umma_rate_smem_raw) + 1023) & ~(uintptr_t)1023);
  __shared__ uint64_t bar;
  __shared__ uint32_t tmem_slot;
  for (int i = threadIdx.x; i < 48 * 1024 / 4; i += blockDim.x) reinterpret_cast<float*>(smem)[i] = 1.0f;
  if (threadIdx.x == 0) { tc::mbar_init(&bar, 1); tc::fence_barrier_init(); }
  if (threadIdx.x < 32) { tc::tmem_alloc(&tmem_slot, 512); tc::tmem_relinquish(); }
  tc::fence_proxy_async();
  tc::tc_fence_before_sync();
  __syncthreads();
  tc::tc_fence_after_sync();
  const uint32_t tmem = tmem_slot;
  if (threadIdx.x == 0) {
    const uint32_t idesc = tc::make_idesc_tf32(128, 256, false, false);
    const uint32_t a = tc::smem_u32(smem), b = a + 16384;     // A: 128 rows x 128 B; B: 256 rows x 128 B
    for (int i = 0; i < iters; ++i) {
      const uint32_t koff = (uint32_t)(i & 3) * 32u;            // the four K-steps of a 32-element K block
      tc::umma_tf32(tmem + ((i & 1) ? 256u : 0u), tc::make_smem_desc_sw128(a + koff, 16, 1024),
                    tc::make_smem_desc_sw128(b + koff, 16, 1024), idesc, 1);
    }
    tc::umma_commit(&bar);
    if (!tc::mbar_wait(&bar, 0)) atomicExch(err_flag, tc::kErrMmaWait);
  }
  tc::tc_fence_before_sync();
  __syncthreads();
  if (threadIdx.x < 32) { tc::tc_fence_after_sync(); tc::tmem_dealloc(tmem, 512); }
}
}  // namespace

extern "C" int nrs_measure_tf32_umma_peak(nrs_ctx* ctx, double* tflops_out) {
  NRS_REQUIRE_CTX(ctx);
  NRS_REQUIRE(ctx, tflops_out != nullptr, NRS_ERR_ARG, "nrs_measure_tf32_umma_peak: null output");
  *tflops_out = 0.0;
  int* err = nullptr;
  int st = nrs_err_flag(ctx, &err);
  if (st != NRS_OK) return st;
  constexpr int kSmem = 64 * 1024, kIters = 40000;          // ~2.6 ms at 128 clocks per UMMA
  static NrsSmemAttr attr;
  NRS_ENSURE_SMEM(ctx, attr, umma_rate_kernel, kSmem);
  cudaEvent_t e0 = nullptr, e1 = nullptr;
  NRS_CUDA(ctx, cudaEventCreate(&e0));
  NRS_CUDA(ctx, cudaEventCreate(&e1));
  float best_ms = 0.0f;
  for (int rep = 0; rep < 4; ++rep) {                        // the first launch warms up
    cudaEventRecord(e0, ctx->stream);
    umma_rate_kernel<<<ctx->sm_count, 128, kSmem, ctx->stream>>>(kIters, err);
    ctx->launches++;
    cudaEventRecord(e1, ctx->stream);
    if (cudaEventSynchronize(e1) != cudaSuccess) break;
    float ms = 0.0f;
    cudaEventElapsedTime(&ms, e0, e1);
    if (rep > 0 && (best_ms == 0.0f || ms < best_ms)) best_ms = ms;
  }
  cudaEventDestroy(e0);
  cudaEventDestroy(e1);
  NRS_CUDA(ctx, cudaGetLastError());
  st = nrs_check_device_error(ctx);
  if (st != NRS_OK) return st;
  if (best_ms > 0.0f) *tflops_out = 2.0 * 128 * 256 * 8 * (double)kIters * ctx->sm_count / (best_ms * 1e-3) / 1e12;
  return NRS_OK;
}

int nrs_tc_gemm(nrs_ctx* ctx, int trans_a, int trans_b, int batch, int m, int n, int k, const float* a, const float* b,
                float* c, const float* bias, int act, float beta, float* pre_out) {
  if (!tc::tensor_map_encoder()) return NRS_ERR_UNSUPPORTED;
  // Small or skinny problems stay on the FFMA kernel: a 128-row tile would be mostly padding.
  if (m < 64 || n < 32 || k < 32) return NRS_ERR_UNSUPPORTED;
  if (batch > 65535) return NRS_ERR_UNSUPPORTED;
  // Batched operands read in place need 16-byte aligned batch strides.
  const bool split = ctx->math_mode == NRS_MATH_3XTF32;
  Operand A, B;
  int st = prepare_operand(ctx, a, m, k, batch, /*stored_kmajor=*/!trans_a, split, NRS_WS_A_HI, NRS_WS_A_LO, &A, false);
  if (st != NRS_OK) return st;
  st = prepare_operand(ctx, b, n, k, batch, /*stored_kmajor=*/trans_b != 0, split, NRS_WS_B_HI, NRS_WS_B_LO, &B, true);
  if (st != NRS_OK) return st;
  if (batch > 1 && ((A.bstride % 4) || (B.bstride % 4))) return NRS_ERR_UNSUPPORTED;
  GemmPolicy pol{c, bias, act, beta, m, n, (size_t)m * n, false, pre_out};
  pol.vec_ok = (n % 4 == 0) && ((reinterpret_cast<uintptr_t>(c) & 15) == 0) && (((size_t)m * n) % 4 == 0) &&
               ((reinterpret_cast<uintptr_t>(bias) & 15) == 0) && ((reinterpret_cast<uintptr_t>(pre_out) & 15) == 0);
  // Tile width: 128 columns is the efficient shape, but a product with few tiles leaves most SMs idle and
  // a K-split needs a second pass, so narrower tiles are taken until about two thirds of the SMs have one.
  const long tiles_m = (m + tc::BM - 1) / tc::BM;
  auto tiles = [&](int bn) { return tiles_m * ((n + bn - 1) / bn) * batch; };
  const long want = (long)ctx->sm_count * 2 / 3;
  int bn = n <= 32 ? 32 : n <= 64 ? 64 : 128;
  if (bn == 128 && tiles(128) < want) bn = 64;
  if (bn == 64 && n > 32 && tiles(64) < want) bn = 32;
#define NRS_RUN_GEMM(BN_) (split ? run<BN_, 2>(ctx, A, B, batch, m, n, k, pol) : run<BN_, 1>(ctx, A, B, batch, m, n, k, pol))
  if (bn == 128) return NRS_RUN_GEMM(128);
  if (bn == 64) return NRS_RUN_GEMM(64);
  return NRS_RUN_GEMM(32);
#undef NRS_RUN_GEMM
}

extern "C" int nrs_has_tensor_core_path(void) { return 1; }
