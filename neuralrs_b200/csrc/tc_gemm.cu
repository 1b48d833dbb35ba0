// Dense / batched GEMM on the 5th-generation tensor cores (tcgen05), TF32 and
// 3xTF32.
//
//   C[b][m,n] = act(op(A[b]) . op(B[b]) + bias[n]) + beta * C
//
// Kernel shape: one CTA per 128 x BN output tile, 6 warps with fixed roles —
//   warp 0     TMA producer: cp.async.bulk.tensor tiles of 128 B (32 x f32) K-slices
//              into a 128-byte-swizzled shared-memory ring, one mbarrier per stage
//   warp 1     allocates TMEM, then one thread issues tcgen05.mma kind::tf32
//              (M=128, N=BN, K=8) against shared-memory descriptors; the f32
//              accumulator lives in TMEM; tcgen05.commit releases ring slots
//   warps 2-5  epilogue: tcgen05.ld the accumulator (one TMEM lane = one output
//              row per thread), add bias, apply the activation, store
// Both operands are consumed K-major.  3xTF32: each operand is staged once into
// a TF32 high plane (round-to-nearest) and an f32 residual plane, and each
// K-slice issues hi*hi + hi*lo + lo*hi into the same accumulator.  Operands that
// are stored MN-major (transposed) are transposed by the same staging pass.
// Plain TF32 reads untransposed operands in place.
//
// Every mbarrier wait is bounded (tc::kWaitClocks); on expiry the kernel writes
// an error code, drains and frees its TMEM instead of hanging.
//
// Reference counterparts: matmul_nn / matmul_nt / matmul_tn, 64x64x16 FFMA tiles
// (src/cuda/graph/matmul.rs:44-198); bmm kernels (src/cuda/graph/bmm.rs:12-56).
#include "igemm_problems.cuh"
#include "nrs_internal.h"
#include "tc_common.cuh"

namespace {

constexpr int BM = 128, BK = 32;  // BK f32 = 128 bytes = one swizzle row
constexpr int kThreads = 192;

struct GemmEpilogue {
  float* C;
  const float* bias;
  int act;
  float beta;
  int M, N;
  size_t batch_stride;
};

template <int BN, int NPLANES>
struct SmemLayout {
  static constexpr int kATile = BM * BK * 4;   // 16 KB
  static constexpr int kBTile = BN * BK * 4;
  static constexpr int kStage = NPLANES * (kATile + kBTile);
  static constexpr int kStages = (200 * 1024) / kStage >= 6 ? 6 : (200 * 1024) / kStage;
  static constexpr int kBytes = kStages * kStage + 1024 /*align*/ + 256 /*barriers*/;
};

template <int BN, int NPLANES>
__global__ void __launch_bounds__(kThreads, 1)
tc_gemm_kernel(const __grid_constant__ CUtensorMap tm_a_hi, const __grid_constant__ CUtensorMap tm_a_lo,
               const __grid_constant__ CUtensorMap tm_b_hi, const __grid_constant__ CUtensorMap tm_b_lo,
               const GemmEpilogue ep, const int num_kblocks, int* __restrict__ err_flag) {
  using L = SmemLayout<BN, NPLANES>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + L::kStages * L::kStage);
  uint64_t* empty_bar = full_bar + L::kStages;
  uint64_t* accum_bar = empty_bar + L::kStages;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(accum_bar + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int m0 = blockIdx.x * BM, n0 = blockIdx.y * BN, batch = blockIdx.z;

  if (warp == 0 && lane == 0) {
    tc::prefetch_tmap(&tm_a_hi);
    tc::prefetch_tmap(&tm_b_hi);
    if (NPLANES == 2) { tc::prefetch_tmap(&tm_a_lo); tc::prefetch_tmap(&tm_b_lo); }
    for (int s = 0; s < L::kStages; ++s) { tc::mbar_init(&full_bar[s], 1); tc::mbar_init(&empty_bar[s], 1); }
    tc::mbar_init(accum_bar, 1);
    tc::fence_barrier_init();
  }
  if (warp == 1) {
    tc::tmem_alloc(tmem_slot, BN);   // BN f32 columns x 128 lanes
    tc::tmem_relinquish();
  }
  tc::tc_fence_before_sync();
  __syncthreads();
  tc::tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      // ---------------- TMA producer
      int issued = 0;
      bool ok = true;
      for (int kb = 0; kb < num_kblocks && ok; ++kb, ++issued) {
        const int s = kb % L::kStages;
        const uint32_t ph = (uint32_t)(kb / L::kStages) & 1u;
        if (!tc::mbar_wait(&empty_bar[s], ph ^ 1u)) { atomicExch(err_flag, tc::kErrProducerWait); ok = false; break; }
        uint8_t* st = smem + s * L::kStage;
        tc::mbar_expect_tx(&full_bar[s], (uint32_t)L::kStage);
        tc::tma_load_3d(st, &tm_a_hi, &full_bar[s], kb * BK, m0, batch);
        tc::tma_load_3d(st + L::kATile, &tm_b_hi, &full_bar[s], kb * BK, n0, batch);
        if (NPLANES == 2) {
          tc::tma_load_3d(st + L::kATile + L::kBTile, &tm_a_lo, &full_bar[s], kb * BK, m0, batch);
          tc::tma_load_3d(st + 2 * L::kATile + L::kBTile, &tm_b_lo, &full_bar[s], kb * BK, n0, batch);
        }
      }
      if (!ok) {
        // Loads already issued still land in this CTA's shared memory: wait for them
        // (bounded) before the CTA may retire.
        for (int kb = (issued > L::kStages ? issued - L::kStages : 0); kb < issued; ++kb) {
          const int s = kb % L::kStages;
          if (!tc::mbar_wait(&full_bar[s], (uint32_t)(kb / L::kStages) & 1u)) { atomicExch(err_flag, tc::kErrDrainWait); break; }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      // ---------------- UMMA issuer
      constexpr uint32_t idesc = tc::make_idesc_tf32(BM, BN, false, false);
      bool ok = true;
      for (int kb = 0; kb < num_kblocks; ++kb) {
        const int s = kb % L::kStages;
        const uint32_t ph = (uint32_t)(kb / L::kStages) & 1u;
        if (!tc::mbar_wait(&full_bar[s], ph)) { atomicExch(err_flag, tc::kErrMmaWait); ok = false; break; }
        tc::tc_fence_after_sync();
        const uint32_t a_hi = tc::smem_u32(smem + s * L::kStage);
        const uint32_t b_hi = a_hi + L::kATile;
        const uint32_t a_lo = b_hi + L::kBTile;
        const uint32_t b_lo = a_lo + L::kATile;
#pragma unroll
        for (int k = 0; k < BK / 8; ++k) {
          const uint32_t koff = k * 32;  // 8 f32 along K inside the 128-byte swizzle row
          const uint64_t da_hi = tc::make_smem_desc_sw128(a_hi + koff, 16, 1024);
          const uint64_t db_hi = tc::make_smem_desc_sw128(b_hi + koff, 16, 1024);
          if (NPLANES == 2) {
            const uint64_t da_lo = tc::make_smem_desc_sw128(a_lo + koff, 16, 1024);
            const uint64_t db_lo = tc::make_smem_desc_sw128(b_lo + koff, 16, 1024);
            tc::umma_tf32(tmem_base, da_lo, db_hi, idesc, (kb | k) != 0);
            tc::umma_tf32(tmem_base, da_hi, db_lo, idesc, 1);
            tc::umma_tf32(tmem_base, da_hi, db_hi, idesc, 1);
          } else {
            tc::umma_tf32(tmem_base, da_hi, db_hi, idesc, (kb | k) != 0);
          }
        }
        tc::umma_commit(&empty_bar[s]);  // slot reusable once these UMMAs have read it
      }
      if (ok) tc::umma_commit(accum_bar);
    }
  } else {
    // ---------------- epilogue: 4 warps, warp w owns TMEM lanes [32*(w%4), +32)
    const int q = warp & 3;
    const bool ok = tc::mbar_wait(accum_bar, 0);
    if (!ok && lane == 0) atomicExch(err_flag, tc::kErrEpilogueWait);
    if (ok) {
      tc::tc_fence_after_sync();
      const int row = m0 + q * 32 + lane;
      float* crow = ep.C + (size_t)batch * ep.batch_stride + (size_t)row * ep.N;
      const bool vec_ok = (ep.N & 3) == 0 && ((reinterpret_cast<uintptr_t>(ep.C) & 15) == 0) &&
                          ((ep.batch_stride & 3) == 0) && ((reinterpret_cast<uintptr_t>(ep.bias) & 15) == 0);
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t r[32];
        tc::tmem_ld_32x32(tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(c * 32), r);
        tc::tmem_ld_wait();
        const int nb = n0 + c * 32;
        if (row < ep.M && nb < ep.N) {
          if (vec_ok && nb + 32 <= ep.N) {
#pragma unroll
            for (int j = 0; j < 32; j += 4) {
              float4 v = make_float4(__uint_as_float(r[j]), __uint_as_float(r[j + 1]), __uint_as_float(r[j + 2]),
                                     __uint_as_float(r[j + 3]));
              if (ep.bias) {
                const float4 bv = *reinterpret_cast<const float4*>(ep.bias + nb + j);
                v.x += bv.x; v.y += bv.y; v.z += bv.z; v.w += bv.w;
              }
              v.x = nrs_apply_act(v.x, ep.act); v.y = nrs_apply_act(v.y, ep.act);
              v.z = nrs_apply_act(v.z, ep.act); v.w = nrs_apply_act(v.w, ep.act);
              float4* dst = reinterpret_cast<float4*>(crow + nb + j);
              if (ep.beta != 0.0f) {
                const float4 o = *dst;
                v.x += ep.beta * o.x; v.y += ep.beta * o.y; v.z += ep.beta * o.z; v.w += ep.beta * o.w;
              }
              *dst = v;
            }
          } else {
#pragma unroll
            for (int j = 0; j < 32; ++j) {
              const int n = nb + j;
              if (n < ep.N) {
                float v = __uint_as_float(r[j]);
                if (ep.bias) v += ep.bias[n];
                v = nrs_apply_act(v, ep.act);
                if (ep.beta != 0.0f) v += ep.beta * crow[n];
                crow[n] = v;
              }
            }
          }
        }
      }
    }
  }

  tc::tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc::tc_fence_after_sync();
    tc::tmem_dealloc(tmem_base, BN);
  }
}

// ------------------------------------------------------------------ staging
// dst planes are [rows][ldk] with ldk a multiple of 32, zero beyond K.
// SPLIT: hi = round-to-nearest TF32, lo = x - hi (exact in f32).  !SPLIT: hi = x.
template <bool SPLIT>
__global__ void __launch_bounds__(256)
stage_rows_kernel(const float* __restrict__ src, float* __restrict__ hi, float* __restrict__ lo, int rows, int K,
                  int ldk, size_t src_bstride, size_t dst_bstride) {
  const int b = blockIdx.y;
  src += b * src_bstride;
  hi += b * dst_bstride;
  if (SPLIT) lo += b * dst_bstride;
  const size_t total4 = (size_t)rows * (ldk / 4);
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total4; i += stride) {
    const size_t r = i / (ldk / 4);
    const int k = (int)(i - r * (ldk / 4)) * 4;
    float v[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) v[j] = (k + j < K) ? src[r * K + k + j] : 0.0f;
    float4 h, l;
    if (SPLIT) {
      h = make_float4(tc::tf32_rn(v[0]), tc::tf32_rn(v[1]), tc::tf32_rn(v[2]), tc::tf32_rn(v[3]));
      l = make_float4(v[0] - h.x, v[1] - h.y, v[2] - h.z, v[3] - h.w);
      *reinterpret_cast<float4*>(lo + r * ldk + k) = l;
    } else {
      h = make_float4(v[0], v[1], v[2], v[3]);
    }
    *reinterpret_cast<float4*>(hi + r * ldk + k) = h;
  }
}

// Source is stored [K][rows] (rows contiguous); output [rows][ldk].  32x32 tiles through
// shared memory keep both sides coalesced; the zero padding up to ldk is written too.
template <bool SPLIT>
__global__ void __launch_bounds__(256)
stage_transpose_kernel(const float* __restrict__ src, float* __restrict__ hi, float* __restrict__ lo, int rows, int K,
                       int ldk, size_t src_bstride, size_t dst_bstride) {
  __shared__ float tile[32][33];
  const int b = blockIdx.z;
  src += b * src_bstride;
  hi += b * dst_bstride;
  if (SPLIT) lo += b * dst_bstride;
  const int r0 = blockIdx.x * 32, k0 = blockIdx.y * 32;
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  for (int i = ty; i < 32; i += 8) {
    const int k = k0 + i, r = r0 + tx;
    tile[i][tx] = (k < K && r < rows) ? src[(size_t)k * rows + r] : 0.0f;
  }
  __syncthreads();
  for (int i = ty; i < 32; i += 8) {
    const int r = r0 + i, k = k0 + tx;  // k < ldk always (ldk is a multiple of 32)
    if (r < rows) {
      const float v = tile[tx][i];
      if (SPLIT) {
        const float h = tc::tf32_rn(v);
        hi[(size_t)r * ldk + k] = h;
        lo[(size_t)r * ldk + k] = v - h;
      } else {
        hi[(size_t)r * ldk + k] = v;
      }
    }
  }
}

struct Operand {
  const float* hi;
  const float* lo;
  int ld;        // leading dimension in floats (K extent seen by TMA = kdim)
  int kdim;      // K extent given to the tensor map (zero-filled beyond)
  size_t bstride;
};

// Prepares one operand as K-major planes.  `stored_kmajor`: memory is [rows][K]; otherwise [K][rows].
int prepare_operand(nrs_ctx* ctx, const float* src, int rows, int K, int batch, bool stored_kmajor, bool split,
                    int ws_hi, int ws_lo, Operand* out) {
  const bool direct = !split && stored_kmajor && (K % 4 == 0) && ((reinterpret_cast<uintptr_t>(src) & 15) == 0) &&
                      (batch == 1 || ((size_t)rows * K) % 4 == 0);
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
  if (stored_kmajor) {
    size_t blocks = (plane / 4 + 255) / 256;
    const size_t cap = (size_t)ctx->sm_count * 16;
    if (blocks > cap) blocks = cap;
    if (blocks < 1) blocks = 1;
    dim3 grid((unsigned)blocks, (unsigned)batch);
    if (split)
      stage_rows_kernel<true><<<grid, 256, 0, ctx->stream>>>(src, (float*)phi, (float*)plo, rows, K, ldk, (size_t)rows * K, plane);
    else
      stage_rows_kernel<false><<<grid, 256, 0, ctx->stream>>>(src, (float*)phi, nullptr, rows, K, ldk, (size_t)rows * K, plane);
  } else {
    dim3 grid((unsigned)((rows + 31) / 32), (unsigned)(ldk / 32), (unsigned)batch);
    if (grid.y > 65535 || grid.z > 65535) return NRS_ERR_UNSUPPORTED;
    if (split)
      stage_transpose_kernel<true><<<grid, 256, 0, ctx->stream>>>(src, (float*)phi, (float*)plo, rows, K, ldk, (size_t)rows * K, plane);
    else
      stage_transpose_kernel<false><<<grid, 256, 0, ctx->stream>>>(src, (float*)phi, nullptr, rows, K, ldk, (size_t)rows * K, plane);
  }
  NRS_LAUNCHED(ctx);
  *out = Operand{(const float*)phi, (const float*)plo, ldk, ldk, plane};
  return NRS_OK;
}

bool make_operand_map(CUtensorMap* tm, const float* base, const Operand& op, int rows, int batch, int box_rows) {
  const uint64_t dim[3] = {(uint64_t)op.kdim, (uint64_t)rows, (uint64_t)batch};
  const uint64_t str[2] = {(uint64_t)op.ld * 4, (uint64_t)op.bstride * 4};
  const uint32_t box[3] = {(uint32_t)BK, (uint32_t)box_rows, 1};
  return tc::encode_tmap_f32(tm, base, 3, dim, str, box);
}

template <int BN, int NPLANES>
int launch_gemm(nrs_ctx* ctx, const Operand& A, const Operand& B, int batch, int m, int n, int k, const GemmEpilogue& ep) {
  using L = SmemLayout<BN, NPLANES>;
  static bool attr_set = false;
  if (!attr_set) {
    NRS_CUDA(ctx, cudaFuncSetAttribute(tc_gemm_kernel<BN, NPLANES>, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kBytes));
    attr_set = true;
  }
  CUtensorMap ta_hi, ta_lo, tb_hi, tb_lo;
  bool ok = make_operand_map(&ta_hi, A.hi, A, m, batch, BM) && make_operand_map(&tb_hi, B.hi, B, n, batch, BN);
  if (NPLANES == 2) ok = ok && make_operand_map(&ta_lo, A.lo, A, m, batch, BM) && make_operand_map(&tb_lo, B.lo, B, n, batch, BN);
  else { ta_lo = ta_hi; tb_lo = tb_hi; }
  NRS_REQUIRE(ctx, ok, NRS_ERR_CUDA, "tc_gemm: cuTensorMapEncodeTiled failed (m=%d n=%d k=%d)", m, n, k);
  int* err = nullptr;
  int st = nrs_err_flag(ctx, &err);
  if (st != NRS_OK) return st;
  dim3 grid((unsigned)((m + BM - 1) / BM), (unsigned)((n + BN - 1) / BN), (unsigned)batch);
  const int num_kblocks = (k + BK - 1) / BK;
  tc_gemm_kernel<BN, NPLANES><<<grid, kThreads, L::kBytes, ctx->stream>>>(ta_hi, ta_lo, tb_hi, tb_lo, ep, num_kblocks, err);
  NRS_LAUNCHED(ctx);
  return NRS_OK;
}

}  // namespace

int nrs_tc_gemm(nrs_ctx* ctx, int trans_a, int trans_b, int batch, int m, int n, int k, const float* a, const float* b,
                float* c, const float* bias, int act, float beta) {
  if (!tc::tensor_map_encoder()) return NRS_ERR_UNSUPPORTED;
  // Small or skinny problems stay on the FFMA kernel: a 128-row tile would be mostly padding.
  if (m < 64 || n < 64 || k < 32) return NRS_ERR_UNSUPPORTED;
  if ((long)((m + BM - 1) / BM) > 2147483647L || (n + 127) / 128 > 65535 || batch > 65535) return NRS_ERR_UNSUPPORTED;
  const bool split = ctx->math_mode == NRS_MATH_3XTF32;
  Operand A, B;
  int st = prepare_operand(ctx, a, m, k, batch, /*stored_kmajor=*/!trans_a, split, NRS_WS_A_HI, NRS_WS_A_LO, &A);
  if (st != NRS_OK) return st;
  st = prepare_operand(ctx, b, n, k, batch, /*stored_kmajor=*/trans_b != 0, split, NRS_WS_B_HI, NRS_WS_B_LO, &B);
  if (st != NRS_OK) return st;
  GemmEpilogue ep{c, bias, act, beta, m, n, (size_t)m * n};
  if (split) return launch_gemm<128, 2>(ctx, A, B, batch, m, n, k, ep);
  return launch_gemm<128, 1>(ctx, A, B, batch, m, n, k, ep);
}

extern "C" int nrs_has_tensor_core_path(void) { return 1; }
