// Fused multi-head attention core for short sequences (seq <= 128, d_head <= 32):
//   out[b, i, h*dh + d] = sum_j softmax_j(q_i . k_j / sqrt(dh)  [masked j > i])  v[b, j, h*dh + d]
// on the projections' own [batch, seq, heads*d_head] layout — one CTA per (batch, head) reads its
// column slice of Q, K, V in place, keeps K and V in shared memory and the score row in registers,
// writes the probabilities once (the backward pass needs them) and the mixed values straight into
// the head's column slice of the output.  The backward kernel does the five products of the
// reference's composition (dV = P^T dO, dP = dO V^T, softmax backward, dQ = dS K, dK = dS^T Q) in
// one CTA with every sum in a fixed order.  Exact f32 FFMA: the whole core is 0.5 GFLOP per pass in
// the transformer-LM configuration, so launch count, not arithmetic, is what it saves.
//
// Replaces, per head, slice_cols x3 -> transpose -> bmm -> scale -> softmax -> bmm -> concat_cols
// of src/cuda/nn/multihead.rs:57-85 and src/cuda/nn/attention.rs:23-32 (same arithmetic, the
// causal mask being the extension described with nrs_causal_mask).
#include "nrs_internal.h"

namespace {

constexpr int kMaxSeq = 128, kMaxDh = 32, kLs = kMaxSeq + 1;
constexpr int kLd = kMaxDh + 4;   // row pitch of the [seq][d_head] tiles: 16-byte aligned rows, read as float4

// acc += a[0..31] . row[0..31] (entries beyond d_head are zero in both)
__device__ __forceinline__ float dot32(const float (&a)[kMaxDh], const float* row) {
  float acc = 0.0f;
#pragma unroll
  for (int g = 0; g < kMaxDh / 4; ++g) {
    const float4 r = *reinterpret_cast<const float4*>(row + 4 * g);
    acc = fmaf(a[4 * g], r.x, acc); acc = fmaf(a[4 * g + 1], r.y, acc);
    acc = fmaf(a[4 * g + 2], r.z, acc); acc = fmaf(a[4 * g + 3], r.w, acc);
  }
  return acc;
}
// a[0..31] += s * row[0..31]
__device__ __forceinline__ void axpy32(float (&a)[kMaxDh], float s_, const float* row) {
#pragma unroll
  for (int g = 0; g < kMaxDh / 4; ++g) {
    const float4 r = *reinterpret_cast<const float4*>(row + 4 * g);
    a[4 * g] = fmaf(s_, r.x, a[4 * g]); a[4 * g + 1] = fmaf(s_, r.y, a[4 * g + 1]);
    a[4 * g + 2] = fmaf(s_, r.z, a[4 * g + 2]); a[4 * g + 3] = fmaf(s_, r.w, a[4 * g + 3]);
  }
}

__global__ void __launch_bounds__(256)
attn_fwd_kernel(const float* __restrict__ q, const float* __restrict__ k, const float* __restrict__ v,
                float* __restrict__ out, float* __restrict__ probs, int S, int H, int dh, int causal, float scale) {
  NRS_PDL_PROLOGUE();
  __shared__ __align__(16) float Ks[kMaxSeq * kLd];
  __shared__ __align__(16) float Vs[kMaxSeq * kLd];
  const int tid = threadIdx.x;
  const int bh = blockIdx.x, b = bh / H, hd = bh - b * H;
  const size_t D = (size_t)H * dh;
  const size_t base = (size_t)b * S * D + (size_t)hd * dh;   // element (i, d) of this head at base + i*D + d
  for (int idx = tid; idx < S * kMaxDh; idx += blockDim.x) {   // columns beyond d_head are zero
    const int i = idx / kMaxDh, d = idx - i * kMaxDh;
    Ks[i * kLd + d] = d < dh ? k[base + (size_t)i * D + d] : 0.0f;
    Vs[i * kLd + d] = d < dh ? v[base + (size_t)i * D + d] : 0.0f;
  }
  __syncthreads();
  const int i = tid >> 1, half = tid & 1, j0 = half * 64;   // two threads per query row, 64 keys each
  const bool row_live = i < S;
  float qr[kMaxDh];
#pragma unroll
  for (int d = 0; d < kMaxDh; ++d) qr[d] = (row_live && d < dh) ? q[base + (size_t)i * D + d] : 0.0f;
  float s[64];
  float mx = -3.0e38f;
#pragma unroll
  for (int jj = 0; jj < 64; ++jj) {
    const int j = j0 + jj;
    float acc = -3.0e38f;   // keys beyond the sequence take no part
    if (row_live && j < S) {
      acc = dot32(qr, Ks + j * kLd) * scale;
      if (causal && j > i) acc = -1e30f;
      mx = fmaxf(mx, acc);
    }
    s[jj] = acc;
  }
  mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
  float sum = 0.0f;
#pragma unroll
  for (int jj = 0; jj < 64; ++jj) {
    const float e = (row_live && j0 + jj < S) ? expf(s[jj] - mx) : 0.0f;
    s[jj] = e;
    sum += e;
  }
  sum += __shfl_xor_sync(0xffffffffu, sum, 1);
  const float inv = row_live ? 1.0f / sum : 0.0f;
  float o[kMaxDh];
#pragma unroll
  for (int d = 0; d < kMaxDh; ++d) o[d] = 0.0f;
#pragma unroll
  for (int jj = 0; jj < 64; ++jj) {
    const int j = j0 + jj;
    const float p = s[jj] * inv;
    s[jj] = p;
    if (row_live && j < S) axpy32(o, p, Vs + j * kLd);
  }
#pragma unroll
  for (int d = 0; d < kMaxDh; ++d) o[d] += __shfl_xor_sync(0xffffffffu, o[d], 1);
  if (row_live) {
#pragma unroll
    for (int d = 0; d < kMaxDh; ++d)
      if ((d >> 4) == half && d < dh) out[base + (size_t)i * D + d] = o[d];   // each thread of the pair writes 16 columns
  }
  // The probabilities (saved for the backward pass) leave through shared memory, 32 key columns at a time, so
  // that a warp writes one 128-byte row segment per store; written from the registers directly, the 32 lanes
  // of a store would hit 32 different rows.  The K tile is no longer needed and holds the staging rows.
  float* stage = Ks;
#pragma unroll
  for (int chunk = 0; chunk < 4; ++chunk) {
    __syncthreads();   // the K tile (first round) / the previous chunk has been consumed by every thread
    if (half == (chunk >> 1) && row_live) {
#pragma unroll
      for (int c = 0; c < 32; ++c) stage[i * kLd + c] = s[(chunk & 1) * 32 + c];
    }
    __syncthreads();
    for (int e = tid; e < kMaxSeq * 32; e += 256) {
      const int r = e >> 5, c = e & 31, j = chunk * 32 + c;
      if (r < S && j < S) probs[((size_t)bh * S + r) * S + j] = stage[r * kLd + c];
    }
  }
}

__global__ void __launch_bounds__(256)
attn_bwd_kernel(const float* __restrict__ q, const float* __restrict__ k, const float* __restrict__ v,
                const float* __restrict__ probs, const float* __restrict__ dout, float* dq, float* dk, float* dv, int S,
                int H, int dh, float scale, int acc_q, int acc_k, int acc_v) {
  NRS_PDL_PROLOGUE();
  extern __shared__ __align__(16) float sm[];
  float* Qs = sm;                       // [S][kLd]
  float* Ks = Qs + kMaxSeq * kLd;
  float* Vs = Ks + kMaxSeq * kLd;
  float* Os = Vs + kMaxSeq * kLd;       // dO
  float* Ps = Os + kMaxSeq * kLd;       // [S][kLs] probabilities
  float* Ds = Ps + kMaxSeq * kLs;       // [S][kLs] dS
  const int tid = threadIdx.x;
  const int bh = blockIdx.x, b = bh / H, hd = bh - b * H;
  const size_t D = (size_t)H * dh;
  const size_t base = (size_t)b * S * D + (size_t)hd * dh;
  for (int idx = tid; idx < S * kMaxDh; idx += blockDim.x) {   // columns beyond d_head are zero
    const int i = idx / kMaxDh, d = idx - i * kMaxDh;
    const size_t g = base + (size_t)i * D + d;
    const bool in = d < dh;
    Qs[i * kLd + d] = in ? q[g] : 0.0f;
    Ks[i * kLd + d] = in ? k[g] : 0.0f;
    Vs[i * kLd + d] = in ? v[g] : 0.0f;
    Os[i * kLd + d] = in ? dout[g] : 0.0f;
  }
  for (int idx = tid; idx < S * S; idx += blockDim.x) {
    const int i = idx / S, j = idx - i * S;
    Ps[i * kLs + j] = probs[(size_t)bh * S * S + idx];
  }
  __syncthreads();
  const int i = tid >> 1, half = tid & 1, j0 = half * 64;
  const bool row_live = i < S;
  // dP = dO V^T, delta_i = sum_j P dP, dS = P (dP - delta) * scale
  {
    float dor[kMaxDh];
#pragma unroll
    for (int d = 0; d < kMaxDh; ++d) dor[d] = (row_live && d < dh) ? Os[i * kLd + d] : 0.0f;
    float t[64];
    float dsum = 0.0f;
#pragma unroll
    for (int jj = 0; jj < 64; ++jj) {
      const int j = j0 + jj;
      float dp = 0.0f;
      if (row_live && j < S) {
        dp = dot32(dor, Vs + j * kLd);
        dsum = fmaf(Ps[i * kLs + j], dp, dsum);
      }
      t[jj] = dp;
    }
    dsum += __shfl_xor_sync(0xffffffffu, dsum, 1);
#pragma unroll
    for (int jj = 0; jj < 64; ++jj) {
      const int j = j0 + jj;
      if (row_live && j < S) Ds[i * kLs + j] = Ps[i * kLs + j] * (t[jj] - dsum) * scale;
    }
  }
  __syncthreads();
  // dQ[i] = sum_j dS[i][j] K[j]
  {
    float a[kMaxDh];
#pragma unroll
    for (int d = 0; d < kMaxDh; ++d) a[d] = 0.0f;
    if (row_live)
      for (int jj = 0; jj < 64; ++jj) {
        const int j = j0 + jj;
        if (j >= S) break;
        axpy32(a, Ds[i * kLs + j], Ks + j * kLd);
      }
#pragma unroll
    for (int d = 0; d < kMaxDh; ++d) a[d] += __shfl_xor_sync(0xffffffffu, a[d], 1);
    if (row_live) {
#pragma unroll
      for (int d = 0; d < kMaxDh; ++d)
        if ((d >> 4) == half && d < dh) {
          float* dst = dq + base + (size_t)i * D + d;
          *dst = acc_q ? *dst + a[d] : a[d];
        }
    }
  }
  // dK[j] = sum_i dS[i][j] Q[i],  dV[j] = sum_i P[i][j] dO[i]: thread (j, half) owns 16 columns of d
  {
    const int j = i, d0 = half * 16;
    float ak[16], av[16];
#pragma unroll
    for (int dd = 0; dd < 16; ++dd) { ak[dd] = 0.0f; av[dd] = 0.0f; }
    if (j < S)
      for (int r = 0; r < S; ++r) {
        const float ds = Ds[r * kLs + j], p = Ps[r * kLs + j];
#pragma unroll
        for (int g = 0; g < 4; ++g) {
          const float4 qv = *reinterpret_cast<const float4*>(Qs + r * kLd + d0 + 4 * g);
          const float4 ov = *reinterpret_cast<const float4*>(Os + r * kLd + d0 + 4 * g);
          ak[4 * g] = fmaf(ds, qv.x, ak[4 * g]); ak[4 * g + 1] = fmaf(ds, qv.y, ak[4 * g + 1]);
          ak[4 * g + 2] = fmaf(ds, qv.z, ak[4 * g + 2]); ak[4 * g + 3] = fmaf(ds, qv.w, ak[4 * g + 3]);
          av[4 * g] = fmaf(p, ov.x, av[4 * g]); av[4 * g + 1] = fmaf(p, ov.y, av[4 * g + 1]);
          av[4 * g + 2] = fmaf(p, ov.z, av[4 * g + 2]); av[4 * g + 3] = fmaf(p, ov.w, av[4 * g + 3]);
        }
      }
    if (j < S) {
#pragma unroll
      for (int dd = 0; dd < 16; ++dd)
        if (d0 + dd < dh) {
          const size_t g = base + (size_t)j * D + d0 + dd;
          dk[g] = acc_k ? dk[g] + ak[dd] : ak[dd];
          dv[g] = acc_v ? dv[g] + av[dd] : av[dd];
        }
    }
  }
}

constexpr size_t kBwdSmem = (size_t)(4 * kMaxSeq * kLd + 2 * kMaxSeq * kLs) * sizeof(float);

}  // namespace

extern "C" {

int nrs_attention_supported(int seq, int d_head) { return seq >= 1 && seq <= kMaxSeq && d_head >= 1 && d_head <= kMaxDh; }

int nrs_attention_fwd(nrs_ctx* ctx, const float* q, const float* k, const float* v, float* out, float* probs, int batch,
                      int seq, int heads, int d_head, int causal) {
  NRS_REQUIRE_CTX(ctx);
  NRS_REQUIRE(ctx, batch >= 0 && heads >= 1, NRS_ERR_SHAPE, "nrs_attention_fwd: bad batch / heads");
  NRS_REQUIRE(ctx, nrs_attention_supported(seq, d_head), NRS_ERR_UNSUPPORTED,
              "nrs_attention_fwd: seq %d / d_head %d outside the fused kernel's range (%d / %d)", seq, d_head, kMaxSeq, kMaxDh);
  if (batch == 0) return NRS_OK;
  NRS_REQUIRE(ctx, q && k && v && out && probs, NRS_ERR_ARG, "nrs_attention_fwd: null tensor");
  NRS_REQUIRE(ctx, (long)batch * heads <= 2147483647L, NRS_ERR_UNSUPPORTED, "nrs_attention_fwd: too many (batch, head) pairs");
  {
    const int st = nrs_tc_attention_fwd(ctx, q, k, v, out, probs, batch, seq, heads, d_head, causal);   // tensor cores in the TF32 modes
    if (st != NRS_ERR_UNSUPPORTED) return st;
  }
  NRS_PDL_LAUNCH(attn_fwd_kernel, (unsigned)(batch * heads), 256, 0, ctx->stream, q, k, v, out, probs, seq, heads, d_head, causal,
                                                                      1.0f / sqrtf((float)d_head));
  NRS_LAUNCHED(ctx);
  return NRS_OK;
}

int nrs_attention_bwd(nrs_ctx* ctx, const float* q, const float* k, const float* v, const float* probs, const float* dout,
                      float* dq, float* dk, float* dv, int batch, int seq, int heads, int d_head, int acc_q, int acc_k,
                      int acc_v) {
  NRS_REQUIRE_CTX(ctx);
  NRS_REQUIRE(ctx, batch >= 0 && heads >= 1, NRS_ERR_SHAPE, "nrs_attention_bwd: bad batch / heads");
  NRS_REQUIRE(ctx, nrs_attention_supported(seq, d_head), NRS_ERR_UNSUPPORTED,
              "nrs_attention_bwd: seq %d / d_head %d outside the fused kernel's range (%d / %d)", seq, d_head, kMaxSeq, kMaxDh);
  if (batch == 0) return NRS_OK;
  NRS_REQUIRE(ctx, q && k && v && probs && dout && dq && dk && dv, NRS_ERR_ARG, "nrs_attention_bwd: null tensor");
  {
    const int st = nrs_tc_attention_bwd(ctx, q, k, v, probs, dout, dq, dk, dv, batch, seq, heads, d_head, acc_q, acc_k, acc_v);
    if (st != NRS_ERR_UNSUPPORTED) return st;
  }
  static NrsSmemAttr attr;
  NRS_ENSURE_SMEM(ctx, attr, attn_bwd_kernel, kBwdSmem);
  NRS_PDL_LAUNCH(attn_bwd_kernel, (unsigned)(batch * heads), 256, kBwdSmem, ctx->stream, q, k, v, probs, dout, dq, dk, dv, seq, heads, d_head,
                                                                               1.0f / sqrtf((float)d_head), acc_q, acc_k, acc_v);
  NRS_LAUNCHED(ctx);
  return NRS_OK;
}

}  // extern "C"
