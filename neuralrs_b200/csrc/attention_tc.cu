// Fused multi-head attention core on the tensor cores (tcgen05, TF32 / 3xTF32) for short sequences:
// seq <= 128, d_head <= 32 and a multiple of 8.  One CTA of 128 threads per (batch, head):
//
//   forward   S = Q K^T         one 128 x 128 x d_head UMMA chain into tensor memory
//             P = softmax(S * scale, masked above the diagonal when causal)
//                               thread i owns query row i: tcgen05.ld brings its 128 scores into registers,
//                               the row is normalised there and written ONCE — as TF32 planes into shared
//                               memory (the A operand of the next product) and, from those planes, as exact
//                               f32 rows to global memory for the backward pass
//             O = P V           128 x d_head x 128 UMMA chain, written into the head's column slice
//   backward  dP = dO V^T, dV = P^T dO, dS = P o (dP - rowsum(dP o P)) * scale, dQ = dS K, dK = dS^T Q
//                               five UMMA chains; the 128 x 128 operands (P^T, dS, dS^T) take turns in
//                               one shared-memory buffer, dP and the three gradients sit in tensor memory
//
// Operands are staged from the projections' own [batch, seq, heads*d_head] layout by the CTA itself
// (plain 128-bit loads, split into a TF32 high plane rounded to nearest and an f32 residual, stored in
// the 128-byte-swizzled K-major layout the UMMA descriptors name); 3xTF32 issues lo*hi + hi*lo + hi*hi
// per product.  Every barrier wait is bounded.  Same values, within 3xTF32 rounding, as the exact-f32
// kernels of attention.cu, which stay for FP32 mode and other head sizes.
//
// Replaces, per head, slice_cols x3 -> transpose -> bmm -> scale -> softmax -> bmm -> concat_cols
// of src/cuda/nn/multihead.rs:57-85 and src/cuda/nn/attention.rs:23-32.
#include "nrs_internal.h"
#include "tc_common.cuh"

namespace {

constexpr int kS = 128;                 // rows / keys of the tile (sequences are zero-padded to it)
constexpr int kThreads = 128;
constexpr uint32_t kTileBytes = 128 * 128;   // one K-major tile: 128 rows x 32 floats

// Byte offset of the 16-byte chunk `c` (0..7) of row `r` in a 128-byte-swizzled K-major tile.
__device__ __forceinline__ uint32_t sw_off(int r, int c) {
  return (uint32_t)((r >> 3) * 1024 + (r & 7) * 128 + ((c ^ (r & 7)) << 4));
}

__device__ __forceinline__ void split4(const float4 v, float4* hi, float4* lo) {
  *hi = make_float4(tc::tf32_rn(v.x), tc::tf32_rn(v.y), tc::tf32_rn(v.z), tc::tf32_rn(v.w));
  *lo = make_float4(v.x - hi->x, v.y - hi->y, v.z - hi->z, v.w - hi->w);
}

// Thread r's row of a [seq][d_head] slice: src[r * ld + (0..32)), zeros beyond d_head and for r >= live.  All
// eight 128-bit loads are issued before anything waits on them (the CTA has only four warps to hide latency).
struct RowRegs {
  float4 c[8];
};
__device__ __forceinline__ RowRegs load_row(const float* __restrict__ src, size_t ld, int live, int dh) {
  RowRegs v;
  const int r = threadIdx.x;
#pragma unroll
  for (int c = 0; c < 8; ++c) {
    v.c[c] = make_float4(0.f, 0.f, 0.f, 0.f);
    if (r < live && 4 * c < dh) v.c[c] = *reinterpret_cast<const float4*>(src + (size_t)r * ld + 4 * c);
  }
  return v;
}
__device__ __forceinline__ void prefetch_row(const float* __restrict__ src, size_t ld, int live) {
  if ((int)threadIdx.x < live) asm volatile("prefetch.global.L2 [%0];" ::"l"(src + (size_t)threadIdx.x * ld));
}

// The row as row r of a K-major A / B tile [128][32] (hi/lo planes, 128-byte swizzle).
__device__ __forceinline__ void store_row_tile(uint8_t* hi, uint8_t* lo, const RowRegs& v) {
  const int r = threadIdx.x;
#pragma unroll
  for (int c = 0; c < 8; ++c) {
    float4 h, l;
    split4(v.c[c], &h, &l);
    const uint32_t off = sw_off(r, c);
    *reinterpret_cast<float4*>(hi + off) = h;
    *reinterpret_cast<float4*>(lo + off) = l;
  }
}

// The row as COLUMN r of the transposed operand [n_rows = d][K = 128] in four K blocks of 32: element
// (d, r) = row[d].  For a fixed d a warp writes 32 consecutive floats of row d: conflict-free.
__device__ __forceinline__ void store_col_tile(uint8_t* hi, uint8_t* lo, const RowRegs& v, int n_rows) {
  const int r = threadIdx.x;
  const uint32_t blk_bytes = (uint32_t)n_rows * 128u;
  const int blk = r >> 5, kk = r & 31;
#pragma unroll
  for (int c = 0; c < 8; ++c) {
    if (4 * c >= n_rows) break;
    const float e[4] = {v.c[c].x, v.c[c].y, v.c[c].z, v.c[c].w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int d = 4 * c + j;
      const float h = tc::tf32_rn(e[j]);
      const uint32_t off = (uint32_t)blk * blk_bytes + sw_off(d, kk >> 2) + (uint32_t)(kk & 3) * 4u;
      *reinterpret_cast<float*>(hi + off) = h;
      *reinterpret_cast<float*>(lo + off) = e[j] - h;
    }
  }
}

// Row r of a 128 x 128 matrix held in registers (p[0..128)) as an A operand: four K blocks of [128][32].
__device__ __forceinline__ void stage_row_regs(uint8_t* hi, uint8_t* lo, int r, const float (&p)[kS]) {
#pragma unroll
  for (int kb = 0; kb < 4; ++kb)
#pragma unroll
    for (int c = 0; c < 8; ++c) {
      float4 h, l;
      split4(make_float4(p[kb * 32 + 4 * c], p[kb * 32 + 4 * c + 1], p[kb * 32 + 4 * c + 2], p[kb * 32 + 4 * c + 3]), &h, &l);
      const uint32_t off = (uint32_t)kb * kTileBytes + sw_off(r, c);
      *reinterpret_cast<float4*>(hi + off) = h;
      *reinterpret_cast<float4*>(lo + off) = l;
    }
}

// The transpose of that matrix as an A operand: element (row j, column r) = p[j] for this thread's r.  For a
// fixed j the 32 threads of a warp write 32 consecutive floats of row j: conflict-free.
__device__ __forceinline__ void stage_col_regs(uint8_t* hi, uint8_t* lo, int r, const float (&p)[kS]) {
  const int kb = r >> 5, kk = r & 31;
#pragma unroll
  for (int j = 0; j < kS; ++j) {
    const float h = tc::tf32_rn(p[j]);
    const uint32_t off = (uint32_t)kb * kTileBytes + sw_off(j, kk >> 2) + (uint32_t)(kk & 3) * 4u;
    *reinterpret_cast<float*>(hi + off) = h;
    *reinterpret_cast<float*>(lo + off) = p[j] - h;
  }
}

// D[tmem] (+)= A . B^T over `ksteps` K steps of 8 starting at the operands' base addresses (one K block of
// 32 per 128-byte row).  SPLIT: lo*hi + hi*lo + hi*hi.
template <bool SPLIT>
__device__ __forceinline__ void issue_block(uint32_t tmem_d, uint32_t a_hi, uint32_t a_lo, uint32_t b_hi, uint32_t b_lo,
                                            uint32_t idesc, int ksteps, bool first) {
  for (int k = 0; k < ksteps; ++k) {
    const uint32_t koff = (uint32_t)k * 32u;
    const uint64_t dah = tc::make_smem_desc_sw128(a_hi + koff, 16, 1024), dbh = tc::make_smem_desc_sw128(b_hi + koff, 16, 1024);
    if (SPLIT) {
      const uint64_t dal = tc::make_smem_desc_sw128(a_lo + koff, 16, 1024), dbl = tc::make_smem_desc_sw128(b_lo + koff, 16, 1024);
      tc::umma_tf32(tmem_d, dal, dbh, idesc, (first && k == 0) ? 0u : 1u);
      tc::umma_tf32(tmem_d, dah, dbl, idesc, 1u);
      tc::umma_tf32(tmem_d, dah, dbh, idesc, 1u);
    } else {
      tc::umma_tf32(tmem_d, dah, dbh, idesc, (first && k == 0) ? 0u : 1u);
    }
  }
}

// Everything written to shared memory by this CTA's threads becomes visible to the tensor core, and the
// CTA meets: the issuing thread may start the next UMMA chain afterwards.
__device__ __forceinline__ void publish_smem() {
  tc::fence_proxy_async();
  tc::tc_fence_before_sync();
  __syncthreads();
  tc::tc_fence_after_sync();
}

__device__ __forceinline__ void load_row128(uint32_t taddr, float (&v)[kS]) {
#pragma unroll
  for (int c = 0; c < 4; ++c) {
    uint32_t r[32];
    tc::tmem_ld_32x32(taddr + (uint32_t)(c * 32), r);
    tc::tmem_ld_wait();
#pragma unroll
    for (int j = 0; j < 32; ++j) v[c * 32 + j] = __uint_as_float(r[j]);
  }
}

// ------------------------------------------------------------------------------------------- forward
// Shared memory: [0, 128 KB) Q hi/lo + K hi/lo (4 x 16 KB), later P hi (64 KB) + P lo (64 KB);
//                [128 KB, +32 KB) V^T hi/lo (2 x 4 blocks x n_pv x 128 B); then barriers.
template <bool SPLIT>
__global__ void __launch_bounds__(kThreads, 1)
attn_fwd_tc_kernel(const float* __restrict__ q, const float* __restrict__ k, const float* __restrict__ v, float* __restrict__ out,
                   float* __restrict__ probs, int S, int H, int dh, int causal, float scale, int* __restrict__ err_flag) {
  extern __shared__ uint8_t attn_smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(attn_smem_raw) + 1023) & ~(uintptr_t)1023);
  uint8_t* q_hi = smem;
  uint8_t* q_lo = smem + kTileBytes;
  uint8_t* k_hi = smem + 2 * kTileBytes;
  uint8_t* k_lo = smem + 3 * kTileBytes;
  uint8_t* p_hi = smem;                       // over Q / K once S has been computed
  uint8_t* p_lo = smem + 4 * kTileBytes;
  uint8_t* vt_hi = smem + 8 * kTileBytes;
  uint8_t* vt_lo = vt_hi + kTileBytes;
  uint64_t* bar = reinterpret_cast<uint64_t*>(vt_lo + kTileBytes);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bar + 2);

  const int tid = threadIdx.x, warp = tid >> 5;
  const int bh = blockIdx.x, b = bh / H, hd = bh - b * H;
  const size_t D = (size_t)H * dh;
  const size_t base = (size_t)b * S * D + (size_t)hd * dh;
  const int n_pv = (dh + 15) & ~15;           // UMMA N of the second product
  if (tid == 0) {
    tc::mbar_init(&bar[0], 1);
    tc::mbar_init(&bar[1], 1);
    tc::fence_barrier_init();
  }
  if (warp == 0) {
    tc::tmem_alloc(tmem_slot, 256);
    tc::tmem_relinquish();
  }
  NRS_PDL_WAIT();
  NRS_PDL_TRIGGER();
  {
    const RowRegs rq = load_row(q + base, D, S, dh), rk = load_row(k + base, D, S, dh), rv = load_row(v + base, D, S, dh);
    store_row_tile(q_hi, q_lo, rq);
    store_row_tile(k_hi, k_lo, rk);
    store_col_tile(vt_hi, vt_lo, rv, n_pv);
  }
  publish_smem();
  const uint32_t tmem = *tmem_slot;
  const uint32_t lane_base = (uint32_t)(warp * 32) << 16;
  bool ok = true;

  if (tid == 0) {   // S = Q K^T
    issue_block<SPLIT>(tmem, tc::smem_u32(q_hi), tc::smem_u32(q_lo), tc::smem_u32(k_hi), tc::smem_u32(k_lo),
                       tc::make_idesc_tf32(128, 128, false, false), dh / 8, true);
    tc::umma_commit(&bar[0]);
  }
  ok = __syncthreads_and(tc::mbar_wait(&bar[0], 0)) != 0;      // the same verdict in every thread
  tc::tc_fence_after_sync();
  float p[kS];
  if (ok) {
    load_row128(tmem + lane_base, p);
    const int i = tid;
    float mx = -3.0e38f;
#pragma unroll
    for (int j = 0; j < kS; ++j) {
      float s = p[j] * scale;
      if (causal && j > i) s = -1e30f;
      if (j >= S) s = -3.0e38f;                // keys beyond the sequence take no part
      p[j] = s;
      mx = fmaxf(mx, s);
    }
    float sum = 0.0f;
#pragma unroll
    for (int j = 0; j < kS; ++j) {
      const float e = j < S ? expf(p[j] - mx) : 0.0f;
      p[j] = e;
      sum += e;
    }
    const float inv = i < S ? 1.0f / sum : 0.0f;
#pragma unroll
    for (int j = 0; j < kS; ++j) p[j] *= inv;
    stage_row_regs(p_hi, p_lo, i, p);          // Q and K are no longer read: the UMMA chain has completed
  }
  publish_smem();
  if (tid == 0 && ok) {   // O = P V
    const uint32_t idesc = tc::make_idesc_tf32(128, n_pv, false, false);
    const uint32_t blk = (uint32_t)n_pv * 128u;
    for (int kb = 0; kb < 4; ++kb)
      issue_block<SPLIT>(tmem + 128u, tc::smem_u32(p_hi) + kb * kTileBytes, tc::smem_u32(p_lo) + kb * kTileBytes,
                         tc::smem_u32(vt_hi) + kb * blk, tc::smem_u32(vt_lo) + kb * blk, idesc, 4, kb == 0);
    tc::umma_commit(&bar[1]);
  }
  // the probabilities, exact (hi + lo), as coalesced rows: a warp writes 512 contiguous bytes per row
  if (ok) {
    const int lane = tid & 31;
    float* prow = probs + (size_t)bh * S * S;
    for (int r = warp; r < S; r += 4) {
      const uint32_t off = (uint32_t)(lane >> 3) * kTileBytes + sw_off(r, lane & 7);
      const float4 h = *reinterpret_cast<const float4*>(p_hi + off), l = *reinterpret_cast<const float4*>(p_lo + off);
      const float e[4] = {h.x + l.x, h.y + l.y, h.z + l.z, h.w + l.w};
      if (S % 4 == 0) {
        if (4 * lane < S) *reinterpret_cast<float4*>(prow + (size_t)r * S + 4 * lane) = make_float4(e[0], e[1], e[2], e[3]);
      } else {
#pragma unroll
        for (int j = 0; j < 4; ++j)
          if (4 * lane + j < S) prow[(size_t)r * S + 4 * lane + j] = e[j];
      }
    }
  }
  if (ok) ok = __syncthreads_and(tc::mbar_wait(&bar[1], 0)) != 0;
  tc::tc_fence_after_sync();
  if (ok) {
    uint32_t r[32];
    tc::tmem_ld_32x32(tmem + lane_base + 128u, r);     // every lane of the warp takes part
    tc::tmem_ld_wait();
    if (tid < S) {
      float* dst = out + base + (size_t)tid * D;
#pragma unroll
      for (int d = 0; d < 32; d += 4)
        if (d < dh)
          *reinterpret_cast<float4*>(dst + d) =
              make_float4(__uint_as_float(r[d]), __uint_as_float(r[d + 1]), __uint_as_float(r[d + 2]), __uint_as_float(r[d + 3]));
    }
  }
  if (!ok && tid == 0) atomicExch(err_flag, tc::kErrEpilogueWait);
  tc::tc_fence_before_sync();
  __syncthreads();
  if (warp == 0) {
    tc::tc_fence_after_sync();
    tc::tmem_dealloc(tmem, 256);
  }
}

// ------------------------------------------------------------------------------------------- backward
// Shared memory: BIG (128 KB: hi 64 KB + lo 64 KB) holds P^T, then dS, then dS^T; three 32 KB operand slots
// X1 (dO rows, later K^T), X2 (V rows, later Q^T), X3 (dO^T).  Tensor memory: dP at columns [0, 128),
// dV at 128, dQ at 160, dK at 192.
template <bool SPLIT>
__global__ void __launch_bounds__(kThreads, 1)
attn_bwd_tc_kernel(const float* __restrict__ q, const float* __restrict__ k, const float* __restrict__ v,
                   const float* __restrict__ probs, const float* __restrict__ dout, float* dq, float* dk, float* dv, int S, int H,
                   int dh, float scale, int acc_q, int acc_k, int acc_v, int* __restrict__ err_flag) {
  extern __shared__ uint8_t attn_smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(attn_smem_raw) + 1023) & ~(uintptr_t)1023);
  uint8_t* big_hi = smem;
  uint8_t* big_lo = smem + 4 * kTileBytes;
  uint8_t* x1_hi = smem + 8 * kTileBytes;
  uint8_t* x1_lo = x1_hi + kTileBytes;
  uint8_t* x2_hi = x1_lo + kTileBytes;
  uint8_t* x2_lo = x2_hi + kTileBytes;
  uint8_t* x3_hi = x2_lo + kTileBytes;
  uint8_t* x3_lo = x3_hi + kTileBytes;
  uint64_t* bar = reinterpret_cast<uint64_t*>(x3_lo + kTileBytes);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bar + 4);

  const int tid = threadIdx.x, warp = tid >> 5;
  const int bh = blockIdx.x, b = bh / H, hd = bh - b * H;
  const size_t D = (size_t)H * dh;
  const size_t base = (size_t)b * S * D + (size_t)hd * dh;
  const int n_d = (dh + 15) & ~15;            // UMMA N of the three d_head-wide products
  const uint32_t blk = (uint32_t)n_d * 128u;  // one K block of a transposed operand
  if (tid == 0) {
    for (int i = 0; i < 4; ++i) tc::mbar_init(&bar[i], 1);
    tc::fence_barrier_init();
  }
  if (warp == 0) {
    tc::tmem_alloc(tmem_slot, 256);
    tc::tmem_relinquish();
  }
  NRS_PDL_WAIT();
  NRS_PDL_TRIGGER();
  prefetch_row(k + base, D, S);               // read two and three phases from now
  prefetch_row(q + base, D, S);
  {
    const RowRegs rdo = load_row(dout + base, D, S, dh), rv = load_row(v + base, D, S, dh);
    store_row_tile(x1_hi, x1_lo, rdo);
    store_row_tile(x2_hi, x2_lo, rv);
    store_col_tile(x3_hi, x3_lo, rdo, n_d);
  }
  float p[kS];
  {
    const float* prow = probs + ((size_t)bh * S + tid) * S;
    const bool vec = S % 4 == 0;
#pragma unroll
    for (int j = 0; j < kS; j += 4) {
      float4 t4 = make_float4(0.f, 0.f, 0.f, 0.f);
      if (tid < S) {
        if (vec) {
          if (j < S) t4 = *reinterpret_cast<const float4*>(prow + j);
        } else {
          if (j + 0 < S) t4.x = prow[j + 0];
          if (j + 1 < S) t4.y = prow[j + 1];
          if (j + 2 < S) t4.z = prow[j + 2];
          if (j + 3 < S) t4.w = prow[j + 3];
        }
      }
      p[j] = t4.x; p[j + 1] = t4.y; p[j + 2] = t4.z; p[j + 3] = t4.w;
    }
  }
  stage_col_regs(big_hi, big_lo, tid, p);     // P^T
  publish_smem();
  const uint32_t tmem = *tmem_slot;
  const uint32_t lane_base = (uint32_t)(warp * 32) << 16;
  const uint32_t idesc_d = tc::make_idesc_tf32(128, n_d, false, false);

  if (tid == 0) {
    // dP = dO V^T
    issue_block<SPLIT>(tmem, tc::smem_u32(x1_hi), tc::smem_u32(x1_lo), tc::smem_u32(x2_hi), tc::smem_u32(x2_lo),
                       tc::make_idesc_tf32(128, 128, false, false), dh / 8, true);
    tc::umma_commit(&bar[0]);
    // dV = P^T dO
    for (int kb = 0; kb < 4; ++kb)
      issue_block<SPLIT>(tmem + 128u, tc::smem_u32(big_hi) + kb * kTileBytes, tc::smem_u32(big_lo) + kb * kTileBytes,
                         tc::smem_u32(x3_hi) + kb * blk, tc::smem_u32(x3_lo) + kb * blk, idesc_d, 4, kb == 0);
    tc::umma_commit(&bar[1]);
  }
  bool ok = __syncthreads_and(tc::mbar_wait(&bar[0], 0)) != 0;
  tc::tc_fence_after_sync();
  if (ok) {
    // dS = P o (dP - sum_j dP_j P_j) * scale, two passes over the dP row in tensor memory
    float dot = 0.0f;
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      uint32_t r[32];
      tc::tmem_ld_32x32(tmem + lane_base + (uint32_t)(c * 32), r);
      tc::tmem_ld_wait();
#pragma unroll
      for (int j = 0; j < 32; ++j) dot = fmaf(__uint_as_float(r[j]), p[c * 32 + j], dot);
    }
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      uint32_t r[32];
      tc::tmem_ld_32x32(tmem + lane_base + (uint32_t)(c * 32), r);
      tc::tmem_ld_wait();
#pragma unroll
      for (int j = 0; j < 32; ++j) p[c * 32 + j] = p[c * 32 + j] * (__uint_as_float(r[j]) - dot) * scale;
    }
    ok = tc::mbar_wait(&bar[1], 0);           // dV done: P^T, dO^T, dO and V are no longer read
  }
  ok = __syncthreads_and(ok) != 0;
  tc::tc_fence_after_sync();
  if (ok) {
    stage_row_regs(big_hi, big_lo, tid, p);   // dS
    store_col_tile(x1_hi, x1_lo, load_row(k + base, D, S, dh), n_d);   // K^T
  }
  publish_smem();
  if (tid == 0 && ok) {   // dQ = dS K
    for (int kb = 0; kb < 4; ++kb)
      issue_block<SPLIT>(tmem + 160u, tc::smem_u32(big_hi) + kb * kTileBytes, tc::smem_u32(big_lo) + kb * kTileBytes,
                         tc::smem_u32(x1_hi) + kb * blk, tc::smem_u32(x1_lo) + kb * blk, idesc_d, 4, kb == 0);
    tc::umma_commit(&bar[2]);
  }
  // dV rows while dQ runs: row = key
  auto write_rows = [&](uint32_t col, float* dst_base, int accumulate) {
    uint32_t r[32];
    tc::tmem_ld_32x32(tmem + lane_base + col, r);
    tc::tmem_ld_wait();
    if (tid < S) {
      float* dst = dst_base + base + (size_t)tid * D;
#pragma unroll
      for (int d = 0; d < 32; d += 4)
        if (d < dh) {
          float4 o = make_float4(__uint_as_float(r[d]), __uint_as_float(r[d + 1]), __uint_as_float(r[d + 2]), __uint_as_float(r[d + 3]));
          if (accumulate) {
            const float4 old = *reinterpret_cast<const float4*>(dst + d);
            o.x += old.x; o.y += old.y; o.z += old.z; o.w += old.w;
          }
          *reinterpret_cast<float4*>(dst + d) = o;
        }
    }
  };
  if (ok) write_rows(128u, dv, acc_v);
  if (ok) ok = tc::mbar_wait(&bar[2], 0);     // dQ done: dS and K^T are no longer read
  ok = __syncthreads_and(ok) != 0;
  tc::tc_fence_after_sync();
  if (ok) {
    stage_col_regs(big_hi, big_lo, tid, p);   // dS^T
    store_col_tile(x2_hi, x2_lo, load_row(q + base, D, S, dh), n_d);   // Q^T
  }
  publish_smem();
  if (tid == 0 && ok) {   // dK = dS^T Q
    for (int kb = 0; kb < 4; ++kb)
      issue_block<SPLIT>(tmem + 192u, tc::smem_u32(big_hi) + kb * kTileBytes, tc::smem_u32(big_lo) + kb * kTileBytes,
                         tc::smem_u32(x2_hi) + kb * blk, tc::smem_u32(x2_lo) + kb * blk, idesc_d, 4, kb == 0);
    tc::umma_commit(&bar[3]);
  }
  if (ok) write_rows(160u, dq, acc_q);
  if (ok) ok = tc::mbar_wait(&bar[3], 0);
  ok = __syncthreads_and(ok) != 0;
  tc::tc_fence_after_sync();
  if (ok) write_rows(192u, dk, acc_k);
  if (!ok && tid == 0) atomicExch(err_flag, tc::kErrEpilogueWait);
  tc::tc_fence_before_sync();
  __syncthreads();
  if (warp == 0) {
    tc::tc_fence_after_sync();
    tc::tmem_dealloc(tmem, 256);
  }
}

constexpr size_t kFwdSmem = 10 * kTileBytes + 64 + 1024;
constexpr size_t kBwdSmem = 14 * kTileBytes + 64 + 1024;
static_assert(kBwdSmem <= 227 * 1024, "shared memory budget of the backward kernel");

}  // namespace

// softmax(q k^T / sqrt(d_head)) v for all heads on the tensor cores; NRS_ERR_UNSUPPORTED (no error text) outside
// seq <= 128, d_head in {8, 16, 24, 32}, 16-byte aligned head slices, a TF32 math mode.
int nrs_tc_attention_fwd(nrs_ctx* ctx, const float* q, const float* k, const float* v, float* out, float* probs, int batch,
                         int seq, int heads, int d_head, int causal) {
  if (ctx->math_mode == NRS_MATH_FP32) return NRS_ERR_UNSUPPORTED;
  if (seq < 1 || seq > kS || d_head < 8 || d_head > 32 || d_head % 8 != 0) return NRS_ERR_UNSUPPORTED;
  if (((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k) | reinterpret_cast<uintptr_t>(v) |
        reinterpret_cast<uintptr_t>(out) | reinterpret_cast<uintptr_t>(probs)) & 15) != 0)
    return NRS_ERR_UNSUPPORTED;
  int* err = nullptr;
  const int st = nrs_err_flag(ctx, &err);
  if (st != NRS_OK) return st;
  const float scale = 1.0f / sqrtf((float)d_head);
  const unsigned grid = (unsigned)(batch * heads);
  if (ctx->math_mode == NRS_MATH_3XTF32) {
    static NrsSmemAttr attr;
    NRS_ENSURE_SMEM(ctx, attr, attn_fwd_tc_kernel<true>, kFwdSmem);
    NRS_PDL_LAUNCH(attn_fwd_tc_kernel<true>, grid, kThreads, kFwdSmem, ctx->stream, q, k, v, out, probs, seq, heads, d_head, causal, scale, err);
  } else {
    static NrsSmemAttr attr;
    NRS_ENSURE_SMEM(ctx, attr, attn_fwd_tc_kernel<false>, kFwdSmem);
    NRS_PDL_LAUNCH(attn_fwd_tc_kernel<false>, grid, kThreads, kFwdSmem, ctx->stream, q, k, v, out, probs, seq, heads, d_head, causal, scale, err);
  }
  NRS_LAUNCHED(ctx);
  return NRS_OK;
}

// Gradients of the above: dq, dk, dv written (acc_* == 0) or added to.  Same conditions.
int nrs_tc_attention_bwd(nrs_ctx* ctx, const float* q, const float* k, const float* v, const float* probs, const float* dout,
                         float* dq, float* dk, float* dv, int batch, int seq, int heads, int d_head, int acc_q, int acc_k,
                         int acc_v) {
  if (ctx->math_mode == NRS_MATH_FP32) return NRS_ERR_UNSUPPORTED;
  if (seq < 1 || seq > kS || d_head < 8 || d_head > 32 || d_head % 8 != 0) return NRS_ERR_UNSUPPORTED;
  if (((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k) | reinterpret_cast<uintptr_t>(v) |
        reinterpret_cast<uintptr_t>(probs) | reinterpret_cast<uintptr_t>(dout) | reinterpret_cast<uintptr_t>(dq) |
        reinterpret_cast<uintptr_t>(dk) | reinterpret_cast<uintptr_t>(dv)) & 15) != 0)
    return NRS_ERR_UNSUPPORTED;
  int* err = nullptr;
  const int st = nrs_err_flag(ctx, &err);
  if (st != NRS_OK) return st;
  const float scale = 1.0f / sqrtf((float)d_head);
  const unsigned grid = (unsigned)(batch * heads);
  if (ctx->math_mode == NRS_MATH_3XTF32) {
    static NrsSmemAttr attr;
    NRS_ENSURE_SMEM(ctx, attr, attn_bwd_tc_kernel<true>, kBwdSmem);
    NRS_PDL_LAUNCH(attn_bwd_tc_kernel<true>, grid, kThreads, kBwdSmem, ctx->stream, q, k, v, probs, dout, dq, dk, dv, seq, heads, d_head,
                   scale, acc_q, acc_k, acc_v, err);
  } else {
    static NrsSmemAttr attr;
    NRS_ENSURE_SMEM(ctx, attr, attn_bwd_tc_kernel<false>, kBwdSmem);
    NRS_PDL_LAUNCH(attn_bwd_tc_kernel<false>, grid, kThreads, kBwdSmem, ctx->stream, q, k, v, probs, dout, dq, dk, dv, seq, heads, d_head,
                   scale, acc_q, acc_k, acc_v, err);
  }
  NRS_LAUNCHED(ctx);
  return NRS_OK;
}
