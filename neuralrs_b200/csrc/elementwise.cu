// Memory-bound elementwise, broadcast, reduction and data-movement kernels.
// All are HBM-bound: 128-bit loads/stores where the pointers allow it, grids
// sized from the SM count, warp-shuffle reductions.
//
// Reference counterparts (one scalar thread per element each):
// vadd/bias_add (src/cuda/graph/add.rs:19-30), accumulate (src/cuda/runtime.rs:
// 14-18), sum_axis0 (src/cuda/reduce.rs:13-20), conv2d_bias_grad
// (src/cuda/nn/conv.rs:78-90), vrelu/relu_grad (src/cuda/graph/relu.rs:17-27),
// vgelu/gelu_grad (src/cuda/graph/gelu.rs:12-32), vscale (src/cuda/graph/
// scale.rs:11-19), transpose2d (src/cuda/graph/transpose.rs:12-23), slice_*
// (src/cuda/graph/slice_cols.rs:12-29), concat_* (src/cuda/graph/concat_cols.rs:
// 12-29).
#include "igemm_problems.cuh"
#include "nrs_internal.h"

namespace {

constexpr int EW_THREADS = 256;

__device__ __forceinline__ bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

// out[i] = f(i, a[i], b[i], out_old[i]) over n elements; float4 body + scalar tail.
// F is a functor: float operator()(float a, float b, float old) const.
template <class F, bool HasB, bool ReadOut>
__global__ void __launch_bounds__(EW_THREADS)
ew_kernel(const float* a, const float* b, float* out, size_t n, F f) {
  NRS_PDL_PROLOGUE();
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  const size_t tid = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  const bool vec = aligned16(a) && aligned16(out) && (!HasB || aligned16(b));
  const size_t n4 = vec ? n / 4 : 0;
  for (size_t i = tid; i < n4; i += stride) {
    const float4 va = reinterpret_cast<const float4*>(a)[i];
    float4 vb = make_float4(0, 0, 0, 0), vo = make_float4(0, 0, 0, 0);
    if (HasB) vb = reinterpret_cast<const float4*>(b)[i];
    if (ReadOut) vo = reinterpret_cast<const float4*>(out)[i];
    float4 r;
    r.x = f(va.x, vb.x, vo.x); r.y = f(va.y, vb.y, vo.y);
    r.z = f(va.z, vb.z, vo.z); r.w = f(va.w, vb.w, vo.w);
    reinterpret_cast<float4*>(out)[i] = r;
  }
  for (size_t i = n4 * 4 + tid; i < n; i += stride)
    out[i] = f(a[i], HasB ? b[i] : 0.0f, ReadOut ? out[i] : 0.0f);
}

template <class F, bool HasB, bool ReadOut>
int launch_ew(nrs_ctx* ctx, const float* a, const float* b, float* out, size_t n, F f) {
  if (n == 0) return NRS_OK;
  size_t blocks = (n / 4 + EW_THREADS - 1) / EW_THREADS + 1;
  const size_t cap = (size_t)ctx->sm_count * 16;
  if (blocks > cap) blocks = cap;
  NRS_PDL_LAUNCH((ew_kernel<F, HasB, ReadOut>), (unsigned)blocks, EW_THREADS, 0, ctx->stream, a, b, out, n, f);
  NRS_LAUNCHED(ctx);
  return NRS_OK;
}

struct FAdd { __device__ float operator()(float a, float b, float) const { return a + b; } };
struct FAcc { __device__ float operator()(float a, float, float o) const { return o + a; } };
struct FRelu { __device__ float operator()(float a, float, float) const { return a > 0.0f ? a : 0.0f; } };
struct FGelu { __device__ float operator()(float a, float, float) const { return nrs_gelu_f(a); } };
template <bool Acc>
struct FReluBwd {  // a = x, b = g
  __device__ float operator()(float x, float g, float o) const { return (Acc ? o : 0.0f) + (x > 0.0f ? g : 0.0f); }
};
template <bool Acc>
struct FGeluBwd {
  __device__ float operator()(float xi, float g, float o) const {
    const float c = 0.7978845608f;
    const float inner = c * (xi + 0.044715f * xi * xi * xi);
    const float t = tanhf(inner);
    const float dinner = c * (1.0f + 3.0f * 0.044715f * xi * xi);
    const float dgelu = 0.5f * (1.0f + t) + 0.5f * xi * (1.0f - t * t) * dinner;
    return (Acc ? o : 0.0f) + g * dgelu;
  }
};
template <bool Acc>
struct FScale {
  float s;
  __device__ float operator()(float a, float, float o) const { return (Acc ? o : 0.0f) + a * s; }
};

__global__ void __launch_bounds__(EW_THREADS)
bias_add_kernel(const float* __restrict__ a, const float* __restrict__ bias, float* __restrict__ out,
                int rows, int cols) {
  NRS_PDL_PROLOGUE();
  const size_t n = (size_t)rows * cols;
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  const size_t tid = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if ((cols & 3) == 0 && aligned16(a) && aligned16(out) && aligned16(bias)) {
    const int c4 = cols >> 2;
    for (size_t i = tid; i < n / 4; i += stride) {
      const float4 va = reinterpret_cast<const float4*>(a)[i];
      const float4 vb = reinterpret_cast<const float4*>(bias)[i % c4];
      reinterpret_cast<float4*>(out)[i] = make_float4(va.x + vb.x, va.y + vb.y, va.z + vb.z, va.w + vb.w);
    }
  } else {
    for (size_t i = tid; i < n; i += stride) out[i] = a[i] + bias[i % cols];
  }
}

// out[c] (+)= sum_r g[r,c].  A block owns 32 columns; its 8 warps stride the
// rows reading 128-byte row segments, then combine through shared memory.  When
// rows are many and columns few, several blocks share a column group and write
// partial sums that a second pass folds in a fixed order (no atomics).
__global__ void __launch_bounds__(256)
colsum_kernel(const float* __restrict__ g, float* __restrict__ out, int rows, int cols, int row_splits,
              int accumulate, float* partial, unsigned* tickets) {
  NRS_PDL_PROLOGUE();
  __shared__ float sm[8][33];
  const int lane = threadIdx.x & 31, wrp = threadIdx.x >> 5;
  const int c = blockIdx.x * 32 + lane;
  const int split = blockIdx.y;
  const int rows_per = (rows + row_splits - 1) / row_splits;
  const int r0 = split * rows_per, r1 = min(rows, r0 + rows_per);
  float s = 0.0f;
  if (c < cols)
    for (int r = r0 + wrp; r < r1; r += 8) s += g[(size_t)r * cols + c];
  sm[wrp][lane] = s;
  __syncthreads();
  if (wrp == 0 && c < cols) {
    float t = 0.0f;
#pragma unroll
    for (int i = 0; i < 8; ++i) t += sm[i][lane];
    if (row_splits > 1) partial[(size_t)split * cols + c] = t;
    else out[c] = accumulate ? out[c] + t : t;
  }
  if (row_splits == 1 || !tickets) return;
  // With a ticket per column block the second pass is folded in: the block of a column group that finishes
  // last adds the group's partial rows in split order (a fixed order whichever block that is).
  __shared__ bool last;
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) last = atomicAdd(&tickets[blockIdx.x], 1u) == gridDim.y - 1;
  __syncthreads();
  if (!last) return;
  __threadfence();
  if (wrp == 0 && c < cols) {
    float t = 0.0f;
#pragma unroll 4
    for (int s = 0; s < row_splits; ++s) t += __ldcg(partial + (size_t)s * cols + c);
    out[c] = accumulate ? out[c] + t : t;
  }
  if (threadIdx.x == 0) tickets[blockIdx.x] = 0;
}
__global__ void colsum_fold_kernel(const float* __restrict__ partial, float* __restrict__ out, int cols,
                                   int row_splits, int accumulate) {
  NRS_PDL_PROLOGUE();
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= cols) return;
  float t = 0.0f;
  for (int s = 0; s < row_splits; ++s) t += partial[(size_t)s * cols + c];
  out[c] = accumulate ? out[c] + t : t;
}

// out[c] (+)= sum over n and the `plane` contiguous elements of channel c.
// One block per (channel, sample-split).  Each warp walks its own images (8 in
// flight per block, 128-bit loads along the plane); warp sums are folded in a
// fixed order, so the result is run-to-run deterministic.
__global__ void __launch_bounds__(256)
chansum_kernel(const float* __restrict__ g, float* __restrict__ out, int n, int c, int plane, int splits,
               int accumulate, float* __restrict__ partial) {
  NRS_PDL_PROLOGUE();
  __shared__ float sm[8];
  const int ch = blockIdx.x, split = blockIdx.y;
  const int lane = threadIdx.x & 31, wrp = threadIdx.x >> 5;
  const int n_per = (n + splits - 1) / splits;
  const int n0 = split * n_per, n1 = min(n, n0 + n_per);
  float s = 0.0f;
  const bool vec = (plane & 3) == 0 && aligned16(g);
  for (int img = n0 + wrp; img < n1; img += 8) {
    const float* base = g + ((size_t)img * c + ch) * plane;
    if (vec) {
      float4 a0 = make_float4(0.f, 0.f, 0.f, 0.f), a1 = a0;
      int i = lane;
      for (; i + 32 < plane / 4; i += 64) {
        const float4 v0 = reinterpret_cast<const float4*>(base)[i];
        const float4 v1 = reinterpret_cast<const float4*>(base)[i + 32];
        a0.x += v0.x; a0.y += v0.y; a0.z += v0.z; a0.w += v0.w;
        a1.x += v1.x; a1.y += v1.y; a1.z += v1.z; a1.w += v1.w;
      }
      for (; i < plane / 4; i += 32) {
        const float4 v0 = reinterpret_cast<const float4*>(base)[i];
        a0.x += v0.x; a0.y += v0.y; a0.z += v0.z; a0.w += v0.w;
      }
      s += ((a0.x + a0.y) + (a0.z + a0.w)) + ((a1.x + a1.y) + (a1.z + a1.w));
    } else {
      for (int i = lane; i < plane; i += 32) s += base[i];
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
  if (lane == 0) sm[wrp] = s;
  __syncthreads();
  if (threadIdx.x == 0) {
    float t = 0.0f;
#pragma unroll
    for (int i = 0; i < 8; ++i) t += sm[i];
    if (splits > 1) partial[(size_t)split * c + ch] = t;
    else out[ch] = accumulate ? out[ch] + t : t;
  }
}

// Batched transpose through a padded 32x32 shared tile: coalesced both ways.
__global__ void __launch_bounds__(256)
transpose_kernel(const float* __restrict__ x, float* __restrict__ y, int rows, int cols, int accumulate) {
  NRS_PDL_PROLOGUE();
  __shared__ float tile[32][33];
  const size_t off = (size_t)blockIdx.z * rows * cols;
  const int c0 = blockIdx.x * 32, r0 = blockIdx.y * 32;
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  for (int i = ty; i < 32; i += 8) {
    const int r = r0 + i, c = c0 + tx;
    if (r < rows && c < cols) tile[i][tx] = x[off + (size_t)r * cols + c];
  }
  __syncthreads();
  for (int i = ty; i < 32; i += 8) {
    const int c = c0 + i, r = r0 + tx;  // output is [cols, rows]
    if (r < rows && c < cols) {
      float* dst = y + off + (size_t)c * rows + r;
      *dst = accumulate ? *dst + tile[tx][i] : tile[tx][i];
    }
  }
}

// dst[r, dc0 + c] (=|+=) src[r, sc0 + c] for c < width: covers slice fwd/bwd and
// concat write/read (a strided 2-D block copy).
__global__ void __launch_bounds__(EW_THREADS)
block_copy_kernel(const float* __restrict__ src, float* __restrict__ dst, int rows, int width, int src_ld,
                  int sc0, int dst_ld, int dc0, int accumulate) {
  NRS_PDL_PROLOGUE();
  const size_t n = (size_t)rows * width;
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
    const size_t r = i / width;
    const int c = (int)(i - r * width);
    float* d = dst + r * dst_ld + dc0 + c;
    const float v = src[r * src_ld + sc0 + c];
    *d = accumulate ? *d + v : v;
  }
}

int launch_block_copy(nrs_ctx* ctx, const float* src, float* dst, int rows, int width, int src_ld, int sc0,
                      int dst_ld, int dc0, int accumulate) {
  const size_t n = (size_t)rows * width;
  if (n == 0) return NRS_OK;
  size_t blocks = (n + EW_THREADS - 1) / EW_THREADS;
  const size_t cap = (size_t)ctx->sm_count * 16;
  if (blocks > cap) blocks = cap;
  NRS_PDL_LAUNCH(block_copy_kernel, (unsigned)blocks, EW_THREADS, 0, ctx->stream, src, dst, rows, width, src_ld, sc0,
                                                                      dst_ld, dc0, accumulate);
  NRS_LAUNCHED(ctx);
  return NRS_OK;
}

}  // namespace

extern "C" {

int nrs_add(nrs_ctx* ctx, const float* a, const float* b, float* out, size_t n) {
  NRS_REQUIRE_CTX(ctx);
  NRS_REQUIRE(ctx, n == 0 || (a && b && out), NRS_ERR_ARG, "nrs_add: null tensor");
  return launch_ew<FAdd, true, false>(ctx, a, b, out, n, FAdd());
}

int nrs_bias_add(nrs_ctx* ctx, const float* a, const float* bias, float* out, int rows, int cols) {
  NRS_REQUIRE_CTX(ctx);
  NRS_REQUIRE(ctx, rows >= 0 && cols >= 0, NRS_ERR_SHAPE, "nrs_bias_add: negative dimension");
  const size_t n = (size_t)rows * cols;
  if (n == 0) return NRS_OK;
  NRS_REQUIRE(ctx, a && bias && out, NRS_ERR_ARG, "nrs_bias_add: null tensor");
  size_t blocks = (n / 4 + EW_THREADS - 1) / EW_THREADS + 1;
  const size_t cap = (size_t)ctx->sm_count * 16;
  if (blocks > cap) blocks = cap;
  NRS_PDL_LAUNCH(bias_add_kernel, (unsigned)blocks, EW_THREADS, 0, ctx->stream, a, bias, out, rows, cols);
  NRS_LAUNCHED(ctx);
  return NRS_OK;
}

int nrs_accumulate(nrs_ctx* ctx, float* acc, const float* src, size_t n) {
  NRS_REQUIRE_CTX(ctx);
  NRS_REQUIRE(ctx, n == 0 || (acc && src), NRS_ERR_ARG, "nrs_accumulate: null tensor");
  return launch_ew<FAcc, false, true>(ctx, src, nullptr, acc, n, FAcc());
}

int nrs_sum_axis0(nrs_ctx* ctx, const float* g, float* out, int rows, int cols, int accumulate) {
  NRS_REQUIRE_CTX(ctx);
  NRS_REQUIRE(ctx, rows >= 0 && cols >= 0, NRS_ERR_SHAPE, "nrs_sum_axis0: negative dimension");
  if (cols == 0) return NRS_OK;
  NRS_REQUIRE(ctx, out && (rows == 0 || g), NRS_ERR_ARG, "nrs_sum_axis0: null tensor");
  const int col_blocks = (cols + 31) / 32;
  int splits = 1;
  if (col_blocks < 2 * ctx->sm_count && rows >= 256) {
    splits = (2 * ctx->sm_count + col_blocks - 1) / col_blocks;
    if (splits > rows / 64) splits = rows / 64;
    if (splits < 1) splits = 1;
    if (splits > 65535) splits = 65535;
  }
  float* partial = nullptr;
  if (splits > 1) {
    void* ws = nullptr;
    const int st = nrs_workspace(ctx, (size_t)splits * cols * sizeof(float), &ws);
    if (st != NRS_OK) return st;
    partial = (float*)ws;
  }
  unsigned* tickets = nullptr;
  if (splits > 1 && col_blocks + 1 <= kNrsFoldTickets) {
    const int st = nrs_fold_ticket(ctx, &tickets);
    if (st != NRS_OK) return st;
    tickets += 1;   // slot 0 belongs to the single-counter users
  }
  NRS_PDL_LAUNCH(colsum_kernel, dim3(col_blocks, splits), 256, 0, ctx->stream, g, out, rows, cols, splits, accumulate, partial,
                 tickets);
  NRS_LAUNCHED(ctx);
  if (splits > 1 && !tickets) {
    NRS_PDL_LAUNCH(colsum_fold_kernel, nrs_blocks(cols, 256), 256, 0, ctx->stream, partial, out, cols, splits, accumulate);
    NRS_LAUNCHED(ctx);
  }
  return NRS_OK;
}

int nrs_channel_sum(nrs_ctx* ctx, const float* g, float* out, int n, int c, int plane, int accumulate) {
  NRS_REQUIRE_CTX(ctx);
  NRS_REQUIRE(ctx, n >= 0 && c >= 0 && plane >= 0, NRS_ERR_SHAPE, "nrs_channel_sum: negative dimension");
  if (c == 0) return NRS_OK;
  NRS_REQUIRE(ctx, out && (n == 0 || plane == 0 || g), NRS_ERR_ARG, "nrs_channel_sum: null tensor");
  int splits = 1;
  if (c < 16 * ctx->sm_count && n >= 16) {
    splits = (16 * ctx->sm_count + c - 1) / c;
    if (splits > n / 8) splits = n / 8;
    if (splits < 1) splits = 1;
    if (splits > 65535) splits = 65535;
  }
  float* partial = nullptr;
  if (splits > 1) {
    void* ws = nullptr;
    const int st = nrs_workspace(ctx, (size_t)splits * c * sizeof(float), &ws);
    if (st != NRS_OK) return st;
    partial = (float*)ws;
  }
  NRS_PDL_LAUNCH(chansum_kernel, dim3(c, splits), 256, 0, ctx->stream, g, out, n, c, plane, splits, accumulate, partial);
  NRS_LAUNCHED(ctx);
  if (splits > 1) {
    NRS_PDL_LAUNCH(colsum_fold_kernel, nrs_blocks(c, 256), 256, 0, ctx->stream, partial, out, c, splits, accumulate);
    NRS_LAUNCHED(ctx);
  }
  return NRS_OK;
}

int nrs_relu_fwd(nrs_ctx* ctx, const float* x, float* y, size_t n) {
  NRS_REQUIRE_CTX(ctx);
  NRS_REQUIRE(ctx, n == 0 || (x && y), NRS_ERR_ARG, "nrs_relu_fwd: null tensor");
  return launch_ew<FRelu, false, false>(ctx, x, nullptr, y, n, FRelu());
}

int nrs_relu_bwd(nrs_ctx* ctx, const float* x, const float* g, float* dx, size_t n, int accumulate) {
  NRS_REQUIRE_CTX(ctx);
  NRS_REQUIRE(ctx, n == 0 || (x && g && dx), NRS_ERR_ARG, "nrs_relu_bwd: null tensor");
  if (accumulate) return launch_ew<FReluBwd<true>, true, true>(ctx, x, g, dx, n, FReluBwd<true>());
  return launch_ew<FReluBwd<false>, true, false>(ctx, x, g, dx, n, FReluBwd<false>());
}

int nrs_gelu_fwd(nrs_ctx* ctx, const float* x, float* y, size_t n) {
  NRS_REQUIRE_CTX(ctx);
  NRS_REQUIRE(ctx, n == 0 || (x && y), NRS_ERR_ARG, "nrs_gelu_fwd: null tensor");
  return launch_ew<FGelu, false, false>(ctx, x, nullptr, y, n, FGelu());
}

int nrs_gelu_bwd(nrs_ctx* ctx, const float* x, const float* g, float* dx, size_t n, int accumulate) {
  NRS_REQUIRE_CTX(ctx);
  NRS_REQUIRE(ctx, n == 0 || (x && g && dx), NRS_ERR_ARG, "nrs_gelu_bwd: null tensor");
  if (accumulate) return launch_ew<FGeluBwd<true>, true, true>(ctx, x, g, dx, n, FGeluBwd<true>());
  return launch_ew<FGeluBwd<false>, true, false>(ctx, x, g, dx, n, FGeluBwd<false>());
}

int nrs_scale(nrs_ctx* ctx, const float* x, float* y, size_t n, float s, int accumulate) {
  NRS_REQUIRE_CTX(ctx);
  NRS_REQUIRE(ctx, n == 0 || (x && y), NRS_ERR_ARG, "nrs_scale: null tensor");
  if (accumulate) return launch_ew<FScale<true>, false, true>(ctx, x, nullptr, y, n, FScale<true>{s});
  return launch_ew<FScale<false>, false, false>(ctx, x, nullptr, y, n, FScale<false>{s});
}

int nrs_transpose(nrs_ctx* ctx, const float* x, float* y, int batch, int rows, int cols, int accumulate) {
  NRS_REQUIRE_CTX(ctx);
  NRS_REQUIRE(ctx, batch >= 0 && rows >= 0 && cols >= 0, NRS_ERR_SHAPE, "nrs_transpose: negative dimension");
  if ((size_t)batch * rows * cols == 0) return NRS_OK;
  NRS_REQUIRE(ctx, x && y, NRS_ERR_ARG, "nrs_transpose: null tensor");
  NRS_REQUIRE(ctx, batch <= 65535 && (rows + 31) / 32 <= 65535, NRS_ERR_UNSUPPORTED, "nrs_transpose: grid too large");
  dim3 grid((cols + 31) / 32, (rows + 31) / 32, batch);
  NRS_PDL_LAUNCH(transpose_kernel, grid, 256, 0, ctx->stream, x, y, rows, cols, accumulate);
  NRS_LAUNCHED(ctx);
  return NRS_OK;
}

int nrs_slice_cols_fwd(nrs_ctx* ctx, const float* x, float* y, int rows, int total, int c0, int c1) {
  NRS_REQUIRE_CTX(ctx);
  NRS_REQUIRE(ctx, rows >= 0 && 0 <= c0 && c0 <= c1 && c1 <= total, NRS_ERR_SHAPE,
              "nrs_slice_cols_fwd: bad range [%d,%d) of %d", c0, c1, total);
  NRS_REQUIRE(ctx, (size_t)rows * (c1 - c0) == 0 || (x && y), NRS_ERR_ARG, "nrs_slice_cols_fwd: null tensor");
  return launch_block_copy(ctx, x, y, rows, c1 - c0, total, c0, c1 - c0, 0, 0);
}

int nrs_slice_cols_bwd(nrs_ctx* ctx, const float* g, float* dx, int rows, int total, int c0, int c1, int accumulate) {
  NRS_REQUIRE_CTX(ctx);
  NRS_REQUIRE(ctx, rows >= 0 && 0 <= c0 && c0 <= c1 && c1 <= total, NRS_ERR_SHAPE,
              "nrs_slice_cols_bwd: bad range [%d,%d) of %d", c0, c1, total);
  NRS_REQUIRE(ctx, (size_t)rows * (c1 - c0) == 0 || (g && dx), NRS_ERR_ARG, "nrs_slice_cols_bwd: null tensor");
  return launch_block_copy(ctx, g, dx, rows, c1 - c0, c1 - c0, 0, total, c0, accumulate);
}

int nrs_concat_write(nrs_ctx* ctx, const float* part, float* out, int rows, int total, int off, int pw) {
  NRS_REQUIRE_CTX(ctx);
  NRS_REQUIRE(ctx, rows >= 0 && off >= 0 && pw >= 0 && off + pw <= total, NRS_ERR_SHAPE,
              "nrs_concat_write: part [%d,%d) outside %d columns", off, off + pw, total);
  NRS_REQUIRE(ctx, (size_t)rows * pw == 0 || (part && out), NRS_ERR_ARG, "nrs_concat_write: null tensor");
  return launch_block_copy(ctx, part, out, rows, pw, pw, 0, total, off, 0);
}

int nrs_concat_read(nrs_ctx* ctx, const float* g, float* dpart, int rows, int total, int off, int pw, int accumulate) {
  NRS_REQUIRE_CTX(ctx);
  NRS_REQUIRE(ctx, rows >= 0 && off >= 0 && pw >= 0 && off + pw <= total, NRS_ERR_SHAPE,
              "nrs_concat_read: part [%d,%d) outside %d columns", off, off + pw, total);
  NRS_REQUIRE(ctx, (size_t)rows * pw == 0 || (g && dpart), NRS_ERR_ARG, "nrs_concat_read: null tensor");
  return launch_block_copy(ctx, g, dpart, rows, pw, total, off, pw, 0, accumulate);
}

}  // extern "C"

// ---------------------------------------------------------------------------
// Column sum that allocates nothing.
//
// nrs_sum_axis0 keeps its split partial sums in a workspace the context grows with
// cudaMalloc on demand.  Some callers cannot tolerate that: code running while a
// CUDA graph is being captured, a real-time loop that must not hit the driver's
// allocator, or a host framework that owns all device memory and forbids foreign
// allocations.  For them the same two kernels run against a fixed scratch array
// that lives in the library image itself.  Every GPU that loads the library holds
// these kStaticSplits x kStaticMaxCols floats (1 MiB) until the process exits.
namespace {
constexpr int kStaticMaxCols = 8192;
constexpr int kStaticSplits = 32;
constexpr int kStaticMaxDevices = 64;
static __device__ __align__(256) float g_colsum_static_scratch[kStaticSplits * kStaticMaxCols];
// Device address of the array above, per device ordinal.  The symbol's name is only a
// host-side handle; kernels must be given the address cudaGetSymbolAddress reports.
static float* g_colsum_static_addr[kStaticMaxDevices] = {nullptr};
}  // namespace

extern "C" int nrs_sum_axis0_static(nrs_ctx* ctx, const float* g, float* out, int rows, int cols, int accumulate) {
  NRS_REQUIRE_CTX(ctx);
  NRS_REQUIRE(ctx, rows >= 0 && cols >= 0, NRS_ERR_SHAPE, "nrs_sum_axis0_static: negative dimension");
  NRS_REQUIRE(ctx, cols <= kStaticMaxCols, NRS_ERR_UNSUPPORTED,
              "nrs_sum_axis0_static: %d columns exceed the built-in scratch (max %d); use nrs_sum_axis0", cols,
              kStaticMaxCols);
  if (cols == 0) return NRS_OK;
  NRS_REQUIRE(ctx, out && (rows == 0 || g), NRS_ERR_ARG, "nrs_sum_axis0_static: null tensor");
  NRS_REQUIRE(ctx, ctx->device >= 0 && ctx->device < kStaticMaxDevices, NRS_ERR_UNSUPPORTED,
              "nrs_sum_axis0_static: device ordinal %d not supported", ctx->device);
  float* scratch = g_colsum_static_addr[ctx->device];
  if (!scratch) {
    // One-time set-up for this device, with that device current.
    int current = -1;
    NRS_CUDA(ctx, cudaGetDevice(&current));
    if (current != ctx->device) NRS_CUDA(ctx, cudaSetDevice(ctx->device));
    void* p = nullptr;
    const cudaError_t e = cudaGetSymbolAddress(&p, g_colsum_static_scratch);
    if (current != ctx->device) (void)cudaSetDevice(current);
    if (e != cudaSuccess || !p) {
      (void)cudaGetLastError();
      return nrs_fail(ctx, NRS_ERR_CUDA, "nrs_sum_axis0_static: cudaGetSymbolAddress failed: %s", cudaGetErrorString(e));
    }
    scratch = static_cast<float*>(p);
    g_colsum_static_addr[ctx->device] = scratch;
  }
  const int col_blocks = (cols + 31) / 32;
  int splits = 1;
  if (col_blocks < 2 * ctx->sm_count && rows >= 256) {
    splits = (2 * ctx->sm_count + col_blocks - 1) / col_blocks;
    if (splits > rows / 64) splits = rows / 64;
    if (splits > kStaticSplits) splits = kStaticSplits;
    if (splits < 1) splits = 1;
  }
  // Every partial the fold reads is written by the first kernel, so stale contents of the
  // shared scratch never need clearing.
  NRS_PDL_LAUNCH(colsum_kernel, dim3(col_blocks, splits), 256, 0, ctx->stream, g, out, rows, cols, splits, accumulate, scratch,
                 (unsigned*)nullptr);
  NRS_LAUNCHED(ctx);
  if (splits > 1) {
    NRS_PDL_LAUNCH(colsum_fold_kernel, nrs_blocks(cols, 256), 256, 0, ctx->stream, scratch, out, cols, splits, accumulate);
    NRS_LAUNCHED(ctx);
  }
  return NRS_OK;
}
