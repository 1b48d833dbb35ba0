// CUDA-core (FFMA) implicit-GEMM kernel and the contraction entry points.
//
// One 128x128x8 register-blocked kernel (256 threads, 8x8 outputs per thread,
// double-buffered shared tiles) computes every contraction as
// C(m,n) = sum_k A(m,k) B(k,n) over the index functions in igemm_problems.cuh:
// dense/batched GEMM in all transpositions and convolution forward, data
// gradient and weight gradient read straight from the NCHW tensors.  It is the
// exact-f32 path: NRS_MATH_FP32 always runs it, and the tensor-core modes run
// it for shapes the tcgen05 kernels do not cover (tiny channel counts, strides,
// ragged tiles).  Long-K problems (weight gradients) are split along K into a
// workspace and reduced in a fixed order, so results are run-to-run
// deterministic.
//
// Reference counterparts: matmul_nn/nt/tn + matmul_nt_splitk
// (src/cuda/graph/matmul.rs:44-261), bmm kernels (src/cuda/graph/bmm.rs:12-56),
// conv2d im2col/col2out/out2mm/col2im (src/cuda/nn/conv.rs:27-149).
#include "igemm_problems.cuh"
#include "nrs_internal.h"
#include "tc_common.cuh"

namespace {

constexpr int BM = 128, BN = 128, BK = 8, NTHREADS = 256, PADM = 4;

// Which tile element a thread fetches.  Operands contiguous along the tile's
// long side (m or n) are read by consecutive threads along that side; operands
// contiguous along k are read 8-wide along k.
template <bool ContigMN>
struct LoadMap {
  // ContigMN: thread owns one row/col (tid%128) and 4 k's (tid/128 + 2*i).
  // else    : thread owns one k (tid%8) and 4 rows/cols (tid/8 + 32*i).
  static __device__ __forceinline__ int mn(int tid, int i) { return ContigMN ? (tid & 127) : ((tid >> 3) + 32 * i); }
  static __device__ __forceinline__ int k(int tid, int i) { return ContigMN ? ((tid >> 7) + 2 * i) : (tid & 7); }
  static constexpr int kCtx = ContigMN ? 1 : 4;
};

template <class P>
__global__ void __launch_bounds__(NTHREADS)
igemm_kernel(const P p, const int splits, const int k_per_split, float* __restrict__ partial) {
  NRS_PDL_PROLOGUE();
  __shared__ __align__(16) float As[2][BK][BM + PADM];
  __shared__ __align__(16) float Bs[2][BK][BN + PADM];
  using LA = LoadMap<P::kAContigM>;
  using LB = LoadMap<P::kBContigN>;

  const int tid = threadIdx.x;
  const int m0 = blockIdx.x * BM, n0 = blockIdx.y * BN;
  const int batch = blockIdx.z / splits, split = blockIdx.z - batch * splits;
  const int k_begin = split * k_per_split;
  const int k_end = min(p.K, k_begin + k_per_split);

  typename P::ARow arow[LA::kCtx];
  typename P::BCol bcol[LB::kCtx];
  bool aval[LA::kCtx], bval[LB::kCtx];
#pragma unroll
  for (int i = 0; i < LA::kCtx; ++i) {
    const int m = m0 + LA::mn(tid, i);
    aval[i] = m < p.M;
    arow[i] = p.a_row(batch, aval[i] ? m : 0);
  }
#pragma unroll
  for (int i = 0; i < LB::kCtx; ++i) {
    const int n = n0 + LB::mn(tid, i);
    bval[i] = n < p.N;
    bcol[i] = p.b_col(batch, bval[i] ? n : 0);
  }

  float ra[4], rb[4];
  auto fetch = [&](int kt) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int ka = kt + LA::k(tid, i);
      const int ia = LA::kCtx == 1 ? 0 : i;
      ra[i] = (aval[ia] && ka < k_end) ? p.a_load(arow[ia], ka) : 0.0f;
      const int kb = kt + LB::k(tid, i);
      const int ib = LB::kCtx == 1 ? 0 : i;
      rb[i] = (bval[ib] && kb < k_end) ? p.b_load(bcol[ib], kb) : 0.0f;
    }
  };
  auto stash = [&](int buf) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      As[buf][LA::k(tid, i)][LA::mn(tid, i)] = ra[i];
      Bs[buf][LB::k(tid, i)][LB::mn(tid, i)] = rb[i];
    }
  };

  // Output micro-tile: rows {4*tm..+3, 64+4*tm..+3}, cols likewise with tn.
  const int tm = P::kStoreContigM ? (tid & 15) : (tid >> 4);
  const int tn = P::kStoreContigM ? (tid >> 4) : (tid & 15);
  float acc[8][8];
#pragma unroll
  for (int i = 0; i < 8; ++i)
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[i][j] = 0.0f;

  if (k_begin < k_end) {
    fetch(k_begin);
    stash(0);
    __syncthreads();
    int buf = 0;
    for (int kt = k_begin; kt < k_end; kt += BK) {
      const bool more = kt + BK < k_end;
      if (more) fetch(kt + BK);
#pragma unroll
      for (int kk = 0; kk < BK; ++kk) {
        const float4 a0 = *reinterpret_cast<const float4*>(&As[buf][kk][4 * tm]);
        const float4 a1 = *reinterpret_cast<const float4*>(&As[buf][kk][64 + 4 * tm]);
        const float4 b0 = *reinterpret_cast<const float4*>(&Bs[buf][kk][4 * tn]);
        const float4 b1 = *reinterpret_cast<const float4*>(&Bs[buf][kk][64 + 4 * tn]);
        const float av[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
        const float bv[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
#pragma unroll
        for (int i = 0; i < 8; ++i)
#pragma unroll
          for (int j = 0; j < 8; ++j) acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
      }
      if (more) {
        stash(buf ^ 1);
        __syncthreads();
        buf ^= 1;
      }
    }
  }

#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int m = m0 + (i < 4 ? 4 * tm + i : 64 + 4 * tm + i - 4);
    if (m >= p.M) continue;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int n = n0 + (j < 4 ? 4 * tn + j : 64 + 4 * tn + j - 4);
      if (n >= p.N) continue;
      if (splits > 1)
        partial[(((size_t)split * p.batches + batch) * p.M + m) * p.N + n] = acc[i][j];
      else
        p.store(batch, m, n, acc[i][j]);
    }
  }
}

// Sums the split-K partials in split order and applies the problem's epilogue.
template <class P>
__global__ void __launch_bounds__(256)
igemm_splitk_reduce(const P p, const int splits, const float* __restrict__ partial) {
  NRS_PDL_PROLOGUE();
  const size_t per = (size_t)p.batches * p.M * p.N;
  const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= per) return;
  float s = 0.0f;
  for (int z = 0; z < splits; ++z) s += partial[(size_t)z * per + idx];
  const int n = (int)(idx % p.N);
  const size_t bm = idx / p.N;
  const int m = (int)(bm % p.M);
  const int b = (int)(bm / p.M);
  p.store(b, m, n, s);
}

template <class P>
int run_igemm(nrs_ctx* ctx, const P& p, const char* who) {
  if (p.M <= 0 || p.N <= 0 || p.batches <= 0) return NRS_OK;
  const int tiles_m = (p.M + BM - 1) / BM, tiles_n = (p.N + BN - 1) / BN;
  const long tiles = (long)tiles_m * tiles_n * p.batches;
  NRS_REQUIRE(ctx, tiles_n <= 65535 && (long)p.batches * 1 <= 65535, NRS_ERR_UNSUPPORTED,
              "%s: grid too large (n tiles %d, batches %d)", who, tiles_n, p.batches);
  int splits = 1;
  const int k_tiles = (p.K + BK - 1) / BK;
  if (tiles < ctx->sm_count && k_tiles >= 64) {
    splits = (int)((2L * ctx->sm_count + tiles - 1) / tiles);
    const int max_splits = k_tiles / 16 > 0 ? k_tiles / 16 : 1;
    if (splits > max_splits) splits = max_splits;
    if ((long)splits * p.batches > 65535) splits = 65535 / p.batches;
    if (splits < 1) splits = 1;
  }
  int k_per_split = ((k_tiles + splits - 1) / splits) * BK;
  if (k_per_split <= 0) k_per_split = BK;
  splits = p.K > 0 ? (p.K + k_per_split - 1) / k_per_split : 1;
  float* partial = nullptr;
  if (splits > 1) {
    void* ws = nullptr;
    int st = nrs_workspace(ctx, (size_t)splits * p.batches * p.M * p.N * sizeof(float), &ws);
    if (st != NRS_OK) return st;
    partial = (float*)ws;
  }
  dim3 grid((unsigned)tiles_m, (unsigned)tiles_n, (unsigned)(p.batches * splits));
  NRS_PDL_LAUNCH((igemm_kernel<P>), grid, NTHREADS, 0, ctx->stream, p, splits, k_per_split, partial);
  NRS_LAUNCHED(ctx);
  if (splits > 1) {
    const size_t per = (size_t)p.batches * p.M * p.N;
    NRS_PDL_LAUNCH((igemm_splitk_reduce<P>), nrs_blocks(per, 256), 256, 0, ctx->stream, p, splits, partial);
    NRS_LAUNCHED(ctx);
  }
  return NRS_OK;
}

template <bool TA, bool TB>
int run_gemm_t(nrs_ctx* ctx, int batch, int m, int n, int k, const float* a, const float* b, float* c,
               const float* bias, int act, float beta, const char* who) {
  NrsGemmProb<TA, TB> p;
  p.M = m; p.N = n; p.K = k; p.batches = batch;
  p.A = a; p.B = b; p.C = c; p.bias = bias; p.act = act; p.beta = beta;
  p.strideA = (size_t)m * k; p.strideB = (size_t)k * n; p.strideC = (size_t)m * n;
  return run_igemm(ctx, p, who);
}

int simt_gemm(nrs_ctx* ctx, int ta, int tb, int batch, int m, int n, int k, const float* a, const float* b,
              float* c, const float* bias, int act, float beta, const char* who) {
  if (!ta && !tb) return run_gemm_t<false, false>(ctx, batch, m, n, k, a, b, c, bias, act, beta, who);
  if (!ta && tb) return run_gemm_t<false, true>(ctx, batch, m, n, k, a, b, c, bias, act, beta, who);
  if (ta && !tb) return run_gemm_t<true, false>(ctx, batch, m, n, k, a, b, c, bias, act, beta, who);
  return run_gemm_t<true, true>(ctx, batch, m, n, k, a, b, c, bias, act, beta, who);
}

// Thin products (a classifier head: n or k of a dozen).  A 128 x 128 tile would be nine tenths
// padding and the whole product is a few MFLOP, so what matters is not paying for a tile
// pipeline.  Exact f32; every sum has a fixed order (deterministic).
constexpr int kThinN = 16;

// k <= 16: one thread per output element.
template <bool TA, bool TB>
__global__ void __launch_bounds__(256)
thin_k_kernel(const float* __restrict__ a, const float* __restrict__ b, float* c, const float* __restrict__ bias, int m,
              int n, int k, int act, float beta) {
  NRS_PDL_PROLOGUE();
  const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (size_t)m * n) return;
  const int col = (int)(idx % n);
  const int row = (int)(idx / n);
  const float* ap = TA ? a + row : a + (size_t)row * k;
  const float* bp = TB ? b + (size_t)col * k : b + col;
  const size_t as = TA ? (size_t)m : 1, bs = TB ? 1 : (size_t)n;
  float acc = 0.0f;
  for (int kk = 0; kk < k; ++kk) acc = fmaf(ap[kk * as], bp[kk * bs], acc);
  if (bias) acc += bias[col];
  acc = nrs_apply_act(acc, act);
  if (beta != 0.0f) acc += beta * c[idx];
  c[idx] = acc;
}

// n <= 16, A row-major [m][k]: one warp per output row, lanes stride over k (coalesced reads of
// the A row), each lane keeps n partial sums, butterfly reduction at the end.  B (k x n, a few KB) is
// copied to shared memory first when it fits: the n strided reads per k step then cost no L1 round trips.
constexpr int kThinBFloats = 10240;
template <bool TB>
__global__ void __launch_bounds__(256)
thin_n_rows_kernel(const float* __restrict__ a, const float* __restrict__ bg, float* c, const float* __restrict__ bias, int m,
                   int n, int k, int act, float beta) {
  NRS_PDL_PROLOGUE();
  __shared__ float sb[kThinBFloats];
  const float* b = bg;
  if (k * n <= kThinBFloats) {
    for (int i = threadIdx.x; i < k * n; i += blockDim.x) sb[i] = bg[i];
    __syncthreads();
    b = sb;
  }
  const int lane = threadIdx.x & 31;
  const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= m) return;
  float acc[kThinN];
#pragma unroll
  for (int j = 0; j < kThinN; ++j) acc[j] = 0.0f;
  const float* ar = a + (size_t)row * k;
#pragma unroll 4
  for (int kk = lane; kk < k; kk += 32) {
    const float av = ar[kk];
#pragma unroll
    for (int j = 0; j < kThinN; ++j)
      if (j < n) acc[j] = fmaf(av, TB ? b[(size_t)j * k + kk] : b[(size_t)kk * n + j], acc[j]);
  }
#pragma unroll
  for (int j = 0; j < kThinN; ++j)
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) acc[j] += __shfl_xor_sync(0xffffffffu, acc[j], d);
  if (lane < n) {
    float v = 0.0f;
#pragma unroll
    for (int j = 0; j < kThinN; ++j)
      if (j == lane) v = acc[j];
    if (bias) v += bias[lane];
    v = nrs_apply_act(v, act);
    float* dst = c + (size_t)row * n + lane;
    if (beta != 0.0f) v += beta * *dst;
    *dst = v;
  }
}

// n <= 16, A stored [k][m] (a weight gradient X^T . dY): a block owns 8 output rows; a warp is
// 4 k-groups x 8 rows (32-byte segments of A[kk][row0..row0+7]), so the block's 8 warps split k 32
// ways, and the 32 partial sums of an output are added in k-group order through shared memory.
constexpr int kThinColRows = 8, kThinColSplit = 32;
template <bool TB>
__global__ void __launch_bounds__(256)
thin_n_cols_kernel(const float* __restrict__ a, const float* __restrict__ b, float* c, const float* __restrict__ bias, int m,
                   int n, int k, int act, float beta) {
  NRS_PDL_PROLOGUE();
  __shared__ float part[kThinColSplit][kThinN][kThinColRows + 1];
  const int lane = threadIdx.x & 31;
  const int r8 = lane & 7, kg = (threadIdx.x >> 5) * 4 + (lane >> 3);
  const int row = blockIdx.x * kThinColRows + r8;
  float acc[kThinN];
#pragma unroll
  for (int j = 0; j < kThinN; ++j) acc[j] = 0.0f;
  const int per = (k + kThinColSplit - 1) / kThinColSplit, k0 = kg * per, k1 = min(k, k0 + per);
  if (row < m)
#pragma unroll 8
    for (int kk = k0; kk < k1; ++kk) {   // unrolled so that several rows of A and B are in flight
      const float av = a[(size_t)kk * m + row];
#pragma unroll
      for (int j = 0; j < kThinN; ++j)
        if (j < n) acc[j] = fmaf(av, TB ? b[(size_t)j * k + kk] : b[(size_t)kk * n + j], acc[j]);
    }
#pragma unroll
  for (int j = 0; j < kThinN; ++j) part[kg][j][r8] = acc[j];
  __syncthreads();
  // thread -> (row r, column j) of the block's 8 x n outputs
  for (int o = threadIdx.x; o < kThinColRows * n; o += blockDim.x) {
    const int r = o / n, j = o - r * n;
    if (blockIdx.x * kThinColRows + r >= m) continue;
    float v = 0.0f;
#pragma unroll
    for (int w = 0; w < kThinColSplit; ++w) v += part[w][j][r];
    if (bias) v += bias[j];
    v = nrs_apply_act(v, act);
    float* dst = c + (size_t)(blockIdx.x * kThinColRows + r) * n + j;
    if (beta != 0.0f) v += beta * *dst;
    *dst = v;
  }
}

bool thin_gemm_applies(int m, int n, int k) {
  return (n <= kThinN || k <= 16) && (double)m * n * k <= 6.4e7 && (long)m * n >= 1024;
}

int thin_gemm(nrs_ctx* ctx, int ta, int tb, int m, int n, int k, const float* a, const float* b, float* c,
              const float* bias, int act, float beta) {
  if (k <= 16) {
    const unsigned blocks = nrs_blocks((size_t)m * n, 256);
    if (!ta && !tb) NRS_PDL_LAUNCH((thin_k_kernel<false, false>), blocks, 256, 0, ctx->stream, a, b, c, bias, m, n, k, act, beta);
    else if (!ta && tb) NRS_PDL_LAUNCH((thin_k_kernel<false, true>), blocks, 256, 0, ctx->stream, a, b, c, bias, m, n, k, act, beta);
    else if (ta && !tb) NRS_PDL_LAUNCH((thin_k_kernel<true, false>), blocks, 256, 0, ctx->stream, a, b, c, bias, m, n, k, act, beta);
    else NRS_PDL_LAUNCH((thin_k_kernel<true, true>), blocks, 256, 0, ctx->stream, a, b, c, bias, m, n, k, act, beta);
  } else if (!ta) {
    const unsigned blocks = nrs_blocks((size_t)m, 8);
    if (tb) NRS_PDL_LAUNCH((thin_n_rows_kernel<true>), blocks, 256, 0, ctx->stream, a, b, c, bias, m, n, k, act, beta);
    else NRS_PDL_LAUNCH((thin_n_rows_kernel<false>), blocks, 256, 0, ctx->stream, a, b, c, bias, m, n, k, act, beta);
  } else {
    const unsigned blocks = nrs_blocks((size_t)m, kThinColRows);
    if (tb) NRS_PDL_LAUNCH((thin_n_cols_kernel<true>), blocks, 256, 0, ctx->stream, a, b, c, bias, m, n, k, act, beta);
    else NRS_PDL_LAUNCH((thin_n_cols_kernel<false>), blocks, 256, 0, ctx->stream, a, b, c, bias, m, n, k, act, beta);
  }
  NRS_LAUNCHED(ctx);
  return NRS_OK;
}

int check_conv_dims(nrs_ctx* ctx, const char* who, int n, int ci, int h, int wd, int co, int kh, int kw,
                    int stride, int pad) {
  NRS_REQUIRE(ctx, n >= 0 && ci > 0 && h > 0 && wd > 0 && co > 0 && kh > 0 && kw > 0, NRS_ERR_SHAPE,
              "%s: non-positive dimension (n=%d ci=%d h=%d w=%d co=%d kh=%d kw=%d)", who, n, ci, h, wd, co, kh, kw);
  NRS_REQUIRE(ctx, stride >= 1 && pad >= 0, NRS_ERR_SHAPE, "%s: stride %d / pad %d invalid", who, stride, pad);
  NRS_REQUIRE(ctx, h + 2 * pad >= kh && wd + 2 * pad >= kw, NRS_ERR_SHAPE,
              "%s: kernel %dx%d larger than padded input %dx%d", who, kh, kw, h + 2 * pad, wd + 2 * pad);
  const long oh = (h + 2 * pad - kh) / stride + 1, ow = (wd + 2 * pad - kw) / stride + 1;
  const long lim = (1L << 31) - 1;
  NRS_REQUIRE(ctx, (long)n * oh * ow <= lim && (long)n * h * wd <= lim && (long)ci * kh * kw <= lim &&
                       (long)co * kh * kw <= lim,
              NRS_ERR_UNSUPPORTED, "%s: a contraction extent exceeds 2^31-1", who);
  return NRS_OK;
}

}  // namespace

// True when nrs_gemm would run an [m,k] x [k,n] product (any transposes) on the tensor-core kernels.
bool nrs_gemm_on_tensor_cores(const nrs_ctx* ctx, int m, int n, int k) {
  return ctx->math_mode != NRS_MATH_FP32 && k >= 32 && m >= 64 && n >= 32 && !thin_gemm_applies(m, n, k) &&
         tc::tensor_map_encoder() != nullptr;
}

int nrs_linear_act_pre(nrs_ctx* ctx, int m, int n, int k, const float* a, const float* w, const float* bias, int act, float* c,
                       float* pre) {
  if (!nrs_gemm_on_tensor_cores(ctx, m, n, k)) return NRS_ERR_UNSUPPORTED;
  NrsProfScope prof(ctx, NRS_PROF_GEMM, 2.0 * m * n * k);
  return nrs_tc_gemm(ctx, 0, 0, 1, m, n, k, a, w, c, bias, act, 0.0f, pre);
}

extern "C" {

int nrs_gemm(nrs_ctx* ctx, int trans_a, int trans_b, int m, int n, int k, const float* a, const float* b,
             float* c, const float* bias, int act, float beta) {
  NRS_REQUIRE_CTX(ctx);
  NRS_REQUIRE(ctx, m >= 0 && n >= 0 && k >= 0, NRS_ERR_SHAPE, "nrs_gemm: negative dimension (%d,%d,%d)", m, n, k);
  NRS_REQUIRE(ctx, act >= NRS_ACT_NONE && act <= NRS_ACT_GELU, NRS_ERR_ARG, "nrs_gemm: unknown activation %d", act);
  NRS_REQUIRE(ctx, beta == 0.0f || beta == 1.0f, NRS_ERR_ARG, "nrs_gemm: beta must be 0 or 1");
  if (m == 0 || n == 0) return NRS_OK;
  NRS_REQUIRE(ctx, c && (k == 0 || (a && b)), NRS_ERR_ARG, "nrs_gemm: null operand");
  NrsProfScope prof(ctx, NRS_PROF_GEMM, 2.0 * m * n * k);
  if (k > 0 && thin_gemm_applies(m, n, k)) return thin_gemm(ctx, trans_a, trans_b, m, n, k, a, b, c, bias, act, beta);
  if (ctx->math_mode != NRS_MATH_FP32 && k > 0) {
    if (trans_a && !trans_b && !bias && act == NRS_ACT_NONE && m >= 64) {   // A^T B: both operands read as stored
      const int st = nrs_tc_gemm_tn(ctx, m, n, k, a, b, c, beta != 0.0f);
      if (st != NRS_ERR_UNSUPPORTED) return st;
    }
    const int st = nrs_tc_gemm(ctx, trans_a, trans_b, 1, m, n, k, a, b, c, bias, act, beta);
    if (st != NRS_ERR_UNSUPPORTED) return st;
  }
  return simt_gemm(ctx, trans_a, trans_b, 1, m, n, k, a, b, c, bias, act, beta, "nrs_gemm");
}

int nrs_bmm(nrs_ctx* ctx, int trans_a, int trans_b, int batch, int m, int n, int k, const float* a,
            const float* b, float* c, float beta) {
  NRS_REQUIRE_CTX(ctx);
  NRS_REQUIRE(ctx, batch >= 0 && m >= 0 && n >= 0 && k >= 0, NRS_ERR_SHAPE, "nrs_bmm: negative dimension");
  NRS_REQUIRE(ctx, beta == 0.0f || beta == 1.0f, NRS_ERR_ARG, "nrs_bmm: beta must be 0 or 1");
  if (batch == 0 || m == 0 || n == 0) return NRS_OK;
  NRS_REQUIRE(ctx, c && (k == 0 || (a && b)), NRS_ERR_ARG, "nrs_bmm: null operand");
  NrsProfScope prof(ctx, NRS_PROF_GEMM, 2.0 * batch * m * n * k);
  if (ctx->math_mode != NRS_MATH_FP32 && k > 0) {
    const int st = nrs_tc_gemm(ctx, trans_a, trans_b, batch, m, n, k, a, b, c, nullptr, NRS_ACT_NONE, beta);
    if (st != NRS_ERR_UNSUPPORTED) return st;
  }
  return simt_gemm(ctx, trans_a, trans_b, batch, m, n, k, a, b, c, nullptr, NRS_ACT_NONE, beta, "nrs_bmm");
}

int nrs_conv2d_fwd(nrs_ctx* ctx, const float* x, const float* w, const float* b, float* y, int n, int ci,
                   int h, int wd, int co, int kh, int kw, int stride, int pad, int act) {
  NRS_REQUIRE_CTX(ctx);
  int st = check_conv_dims(ctx, "nrs_conv2d_fwd", n, ci, h, wd, co, kh, kw, stride, pad);
  if (st != NRS_OK) return st;
  NRS_REQUIRE(ctx, act >= NRS_ACT_NONE && act <= NRS_ACT_GELU, NRS_ERR_ARG, "nrs_conv2d_fwd: unknown activation %d", act);
  if (n == 0) return NRS_OK;
  NRS_REQUIRE(ctx, x && w && y, NRS_ERR_ARG, "nrs_conv2d_fwd: null tensor");
  NrsProfScope prof(ctx, NRS_PROF_CONV_FWD,
                    2.0 * n * co * ((h + 2 * pad - kh) / stride + 1) * ((wd + 2 * pad - kw) / stride + 1) * ci * kh * kw);
  st = nrs_smallc_conv_fwd(ctx, x, w, b, y, n, ci, h, wd, co, kh, kw, stride, pad, act);
  if (st != NRS_ERR_UNSUPPORTED) return st;
  if (ctx->math_mode != NRS_MATH_FP32) {
    st = nrs_tc_conv_fwd(ctx, x, w, b, y, n, ci, h, wd, co, kh, kw, stride, pad, act);
    if (st != NRS_ERR_UNSUPPORTED) return st;
  }
  NrsConvFpropProb p;
  p.g = NrsConvGeom(n, ci, h, wd, co, kh, kw, stride, pad);
  p.M = n * p.g.oh * p.g.ow; p.N = co; p.K = ci * kh * kw; p.batches = 1;
  p.x = x; p.wgt = w; p.bias = b; p.y = y; p.act = act;
  return run_igemm(ctx, p, "nrs_conv2d_fwd");
}

int nrs_conv2d_bwd(nrs_ctx* ctx, const float* x, const float* w, const float* dy, float* dx, float* dw,
                   float* db, int n, int ci, int h, int wd, int co, int kh, int kw, int stride, int pad,
                   int accumulate) {
  NRS_REQUIRE_CTX(ctx);
  int st = check_conv_dims(ctx, "nrs_conv2d_bwd", n, ci, h, wd, co, kh, kw, stride, pad);
  if (st != NRS_OK) return st;
  const NrsConvGeom g(n, ci, h, wd, co, kh, kw, stride, pad);
  // a caller that issued the data gradient of this layer just before asking for the weight gradient alone
  // says so through the context; a call that computes both knows it by itself
  bool wgrad_may_overlap = ctx->independent_next && !dx;
  ctx->independent_next = false;
  if (n == 0) {  // an empty batch contributes zero gradients
    if (!accumulate) {
      if (dw) NRS_CUDA(ctx, cudaMemsetAsync(dw, 0, sizeof(float) * co * ci * kh * kw, ctx->stream));
      if (db) NRS_CUDA(ctx, cudaMemsetAsync(db, 0, sizeof(float) * co, ctx->stream));
    }
    return NRS_OK;
  }
  NRS_REQUIRE(ctx, dy != nullptr, NRS_ERR_ARG, "nrs_conv2d_bwd: null dy");
  NRS_REQUIRE(ctx, !dx || w, NRS_ERR_ARG, "nrs_conv2d_bwd: dx requested without w");
  NRS_REQUIRE(ctx, !dw || x, NRS_ERR_ARG, "nrs_conv2d_bwd: dw requested without x");
  const double conv_flop = 2.0 * n * co * g.oh * g.ow * ci * kh * kw;
  // When both gradients are asked for, the data gradient's NHWC planes of dy (staged into the context's
  // operand scratch) serve the weight gradient too: registered for the rest of this call.
  const bool split3 = ctx->math_mode == NRS_MATH_3XTF32;
  const bool dy_had_planes = ctx->math_mode != NRS_MATH_FP32 && nrs_planes_find(ctx, dy, split3) != nullptr;
  bool dy_planes_lent = false;
  struct Unlend {
    nrs_ctx* c; const void* k; bool* on;
    ~Unlend() { if (*on) c->plane_hints.erase(k); }
  } unlend{ctx, dy, &dy_planes_lent};
  if (dx) {
    NrsProfScope prof(ctx, NRS_PROF_CONV_DGRAD, conv_flop);
    st = ctx->math_mode != NRS_MATH_FP32
             ? nrs_tc_conv_dgrad(ctx, w, dy, dx, n, ci, h, wd, co, kh, kw, stride, pad, accumulate)
             : NRS_ERR_UNSUPPORTED;
    if (st != NRS_OK && st != NRS_ERR_UNSUPPORTED) return st;
    if (st == NRS_OK && dw && !dy_had_planes && ctx->ws_slot[NRS_WS_A_HI] && (!split3 || ctx->ws_slot[NRS_WS_A_LO])) {
      ctx->plane_hints[dy] = NrsPlanes{(float*)ctx->ws_slot[NRS_WS_A_HI], split3 ? (float*)ctx->ws_slot[NRS_WS_A_LO] : nullptr, split3 ? 1 : 0};
      dy_planes_lent = true;
    }
    if (st == NRS_ERR_UNSUPPORTED) {
    NrsConvDgradProb p;
    p.g = g; p.M = n * h * wd; p.N = ci; p.K = co * kh * kw; p.batches = 1;
    p.dy = dy; p.wgt = w; p.dx = dx; p.accumulate = accumulate;
    st = run_igemm(ctx, p, "nrs_conv2d_bwd(dx)");
    if (st != NRS_OK) return st;
    }
    wgrad_may_overlap = true;   // x and dy (and any planes of them) were complete before the kernel(s) above
  }
  if (dw) {
    NrsProfScope prof(ctx, NRS_PROF_CONV_WGRAD, conv_flop);
    NrsIndependentNext overlap(ctx, wgrad_may_overlap);
    st = nrs_smallc_conv_wgrad(ctx, x, dy, dw, n, ci, h, wd, co, kh, kw, stride, pad, accumulate);
    if (st == NRS_ERR_UNSUPPORTED && ctx->math_mode != NRS_MATH_FP32)
      st = nrs_tc_conv_wgrad_rows(ctx, x, dy, dw, n, ci, h, wd, co, kh, kw, stride, pad, accumulate);
    if (st == NRS_ERR_UNSUPPORTED && ctx->math_mode != NRS_MATH_FP32)
      st = nrs_tc_conv_wgrad(ctx, x, dy, dw, n, ci, h, wd, co, kh, kw, stride, pad, accumulate);
    if (st != NRS_OK && st != NRS_ERR_UNSUPPORTED) return st;
    if (st == NRS_ERR_UNSUPPORTED) {
    NrsConvWgradProb p;
    p.g = g; p.M = co; p.N = ci * kh * kw; p.K = n * g.oh * g.ow; p.batches = 1;
    p.dy = dy; p.x = x; p.dw = dw; p.accumulate = accumulate;
    st = run_igemm(ctx, p, "nrs_conv2d_bwd(dw)");
    if (st != NRS_OK) return st;
    }
  }
  if (db) {
    st = nrs_channel_sum(ctx, dy, db, n, co, g.oh * g.ow, accumulate);
    if (st != NRS_OK) return st;
  }
  return NRS_OK;
}

int nrs_planes_drop(nrs_ctx* ctx, const float* t) {
  NRS_REQUIRE_CTX(ctx);
  auto it = ctx->owned_planes.find(t);
  if (it == ctx->owned_planes.end()) return NRS_OK;
  auto hint = ctx->plane_hints.find(t);
  if (hint != ctx->plane_hints.end() && hint->second.hi == it->second.hi) ctx->plane_hints.erase(hint);
  nrs_free(ctx, it->second.hi);
  if (it->second.lo) nrs_free(ctx, it->second.lo);
  ctx->owned_planes.erase(it);
  return NRS_OK;
}

int nrs_planes_cache(nrs_ctx* ctx, const float* t, int n, int c, int h, int w) {
  NRS_REQUIRE_CTX(ctx);
  NRS_REQUIRE(ctx, t != nullptr, NRS_ERR_ARG, "nrs_planes_cache: null tensor");
  NRS_REQUIRE(ctx, n >= 0 && c > 0 && h > 0 && w > 0, NRS_ERR_SHAPE, "nrs_planes_cache: bad shape [%d,%d,%d,%d]", n, c, h, w);
  int st = nrs_planes_drop(ctx, t);   // the contents may have changed since an earlier call
  if (st != NRS_OK) return st;
  if (ctx->math_mode == NRS_MATH_FP32 || c % 32 != 0 || n == 0 || !tc::tensor_map_encoder()) return NRS_OK;
  if (ctx->plane_hints.count(t)) return NRS_OK;   // someone else (the node graph) already keeps planes of it
  const bool split = ctx->math_mode == NRS_MATH_3XTF32;
  const size_t hw = (size_t)h * w, floats = (size_t)n * c * hw;
  void *hi = nullptr, *lo = nullptr;
  st = nrs_alloc(ctx, floats * sizeof(float), 0, &hi);
  if (st == NRS_OK && split) st = nrs_alloc(ctx, floats * sizeof(float), 0, &lo);
  if (st == NRS_OK) st = nrs_tc_stage(ctx, t, (float*)hi, (float*)lo, (int)hw, c, c, n, (size_t)c * hw, (size_t)c * hw, true);
  if (st != NRS_OK) {
    if (hi) nrs_free(ctx, hi);
    if (lo) nrs_free(ctx, lo);
    return st;
  }
  const NrsPlanes pl{(float*)hi, (float*)lo, split ? 1 : 0};
  ctx->owned_planes[t] = pl;
  ctx->plane_hints[t] = pl;
  return NRS_OK;
}

}  // extern "C"
