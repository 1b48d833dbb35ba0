// Embedding gather / scatter-add and the causal score mask.
// Reference: embed_forward / embed_backward (src/cuda/nn/embedding.rs:13-30; CPU
// semantics src/nn/embedding.rs:19-113).  The reference's backward is a per-element
// atomicAdd scatter (sum order varies run to run); here every vocabulary row is
// owned by one block that walks the tokens in order, so the weight gradient is
// deterministic and needs no atomics.  The causal mask has no reference
// counterpart (the reference has no mask): scores[i, j > i] are set to -1e30
// before the softmax, and their gradient is dropped.
#include "nrs_internal.h"

namespace {

// out[t, :] = w[idx[t], :] (+ pos[t % seq, :] when a positional table is given).  An index outside
// [0, vocab) is never dereferenced: its row reads as zeros and the context's error word is set.
constexpr int kErrBadIndex = 5;
__global__ void __launch_bounds__(256)
embed_fwd_kernel(const float* __restrict__ w, const int32_t* __restrict__ idx, const float* __restrict__ pos,
                 float* __restrict__ out, int tokens, int seq, int dim, int vocab, int* err) {
  NRS_PDL_PROLOGUE();
  const size_t total = (size_t)tokens * dim;
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  const bool vec = (dim & 3) == 0 &&
                   ((reinterpret_cast<uintptr_t>(w) | reinterpret_cast<uintptr_t>(out) | reinterpret_cast<uintptr_t>(pos)) & 15) == 0;
  if (vec) {
    const int d4 = dim >> 2;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total / 4; i += stride) {
      const size_t t = i / d4;
      const int c = (int)(i - t * d4);
      const int row = idx[t];
      float4 v = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
      if (row >= 0 && row < vocab) v = reinterpret_cast<const float4*>(w + (size_t)row * dim)[c];
      else if (c == 0) atomicExch(err, kErrBadIndex);
      if (pos) {
        const float4 p = reinterpret_cast<const float4*>(pos + (t % (size_t)seq) * dim)[c];
        v.x += p.x; v.y += p.y; v.z += p.z; v.w += p.w;
      }
      reinterpret_cast<float4*>(out)[i] = v;
    }
  } else {
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
      const size_t t = i / dim;
      const int c = (int)(i - t * dim);
      const int row = idx[t];
      float v = 0.0f;
      if (row >= 0 && row < vocab) v = w[(size_t)row * dim + c];
      else if (c == 0) atomicExch(err, kErrBadIndex);
      if (pos) v += pos[(t % (size_t)seq) * dim + c];
      out[i] = v;
    }
  }
}

// One block per vocabulary row.  The token indices are scanned 256 at a time: every thread tests one
// token, the matches are compacted IN TOKEN ORDER (warp ballots + a prefix over the warp counts) into a
// shared list, and then thread d adds the matching gradient rows in that order — the same order of
// additions as a serial walk over the tokens, so the result is deterministic and independent of the
// launch shape, at a cost of tokens/256 scan steps per block instead of `tokens` per thread.
__global__ void __launch_bounds__(256)
embed_bwd_kernel(const float* __restrict__ g, const int32_t* __restrict__ idx, float* dw, int tokens, int dim,
                 int accumulate) {
  NRS_PDL_PROLOGUE();
  constexpr int kChunk = 1024;             // tokens whose matches are listed before they are summed
  __shared__ int32_t s_match[kChunk];
  __shared__ int s_warp[2][8];             // per-warp match counts, double-buffered across scan steps
  const int row = blockIdx.x;
  const int lane = threadIdx.x & 31, wrp = threadIdx.x >> 5;
  int step = 0;
  for (int d0 = 0; d0 < dim; d0 += 4 * 256) {             // four features per thread per pass
    float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
    for (int t0 = 0; t0 < tokens; t0 += kChunk) {
      const int nt = min(kChunk, tokens - t0);
      __syncthreads();                                    // the previous chunk's list has been consumed
      int n_match = 0;                                    // kept by every thread; the same in all of them
      for (int sub = 0; sub < nt; sub += 256, ++step) {
        const int t = t0 + sub + threadIdx.x;
        const bool hit = (sub + (int)threadIdx.x) < nt && idx[t] == row;
        const unsigned ballot = __ballot_sync(0xffffffffu, hit);
        if (lane == 0) s_warp[step & 1][wrp] = __popc(ballot);
        __syncthreads();   // one barrier per step: the next step writes the other buffer, and a warp can only
                           // reach the step after that once every warp has passed the next barrier
        int before = n_match, total = 0;
#pragma unroll
        for (int w2 = 0; w2 < 8; ++w2) {
          const int cnt = s_warp[step & 1][w2];
          if (w2 < wrp) before += cnt;
          total += cnt;
        }
        if (hit) s_match[before + __popc(ballot & ((1u << lane) - 1u))] = t;
        n_match += total;
      }
      __syncthreads();                                    // the list is complete
      for (int m = 0; m < n_match; ++m) {
        const float* src = g + (size_t)s_match[m] * dim + d0 + threadIdx.x;
#pragma unroll
        for (int k = 0; k < 4; ++k)
          if (d0 + (int)threadIdx.x + k * 256 < dim) acc[k] += src[k * 256];
      }
    }
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const int d = d0 + threadIdx.x + k * 256;
      if (d < dim) {
        float* dst = dw + (size_t)row * dim + d;
        *dst = accumulate ? *dst + acc[k] : acc[k];
      }
    }
  }
}

// x, y: [batch, s, s].  forward: y = (j > i) ? -1e30 : x.  backward: y (+)= (j > i) ? 0 : x.
__global__ void __launch_bounds__(256)
causal_mask_kernel(const float* __restrict__ x, float* y, size_t total, int s, int backward, int accumulate) {
  NRS_PDL_PROLOGUE();
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += stride) {
    const int j = (int)(idx % s);
    const int i = (int)((idx / s) % s);
    float v = x[idx];
    if (j > i) v = backward ? 0.0f : -1e30f;
    y[idx] = accumulate ? y[idx] + v : v;
  }
}

unsigned grid_for(const nrs_ctx* ctx, size_t work) {
  size_t blocks = (work + 255) / 256;
  const size_t cap = (size_t)ctx->sm_count * 16;
  return (unsigned)(blocks > cap ? cap : (blocks ? blocks : 1));
}

// to_heads: y[((b*H + h)*S + s)*dh + e] = x[((b*S + s)*H + h)*dh + e]; otherwise the inverse.
__global__ void __launch_bounds__(256)
permute_heads_kernel(const float* __restrict__ x, float* y, size_t total, int S, int H, int dh, int to_heads,
                     int accumulate) {
  NRS_PDL_PROLOGUE();
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += stride) {
    // idx walks the [b][s][h][e] order
    const int e = (int)(idx % dh);
    size_t t = idx / dh;
    const int h = (int)(t % H);
    t /= H;
    const int s = (int)(t % S);
    const size_t b = t / S;
    const size_t head_major = ((b * H + h) * S + s) * dh + e;
    const size_t src = to_heads ? idx : head_major, dst = to_heads ? head_major : idx;
    const float v = x[src];
    y[dst] = accumulate ? y[dst] + v : v;
  }
}

}  // namespace

extern "C" {

int nrs_embedding_pos_fwd(nrs_ctx* ctx, const float* weight, const int32_t* idx, const float* pos_table, float* out,
                          int tokens, int seq, int dim, int vocab) {
  NRS_REQUIRE_CTX(ctx);
  NRS_REQUIRE(ctx, tokens >= 0 && dim > 0 && vocab > 0, NRS_ERR_SHAPE, "nrs_embedding_fwd: bad shape [%d,%d], vocabulary %d", tokens,
              dim, vocab);
  NRS_REQUIRE(ctx, !pos_table || seq > 0, NRS_ERR_SHAPE, "nrs_embedding_pos_fwd: sequence length must be positive");
  if (tokens == 0) return NRS_OK;
  NRS_REQUIRE(ctx, weight && idx && out, NRS_ERR_ARG, "nrs_embedding_fwd: null tensor");
  int* err = nullptr;
  const int st = nrs_err_flag(ctx, &err);
  if (st != NRS_OK) return st;
  NRS_PDL_LAUNCH(embed_fwd_kernel, grid_for(ctx, (size_t)tokens * dim / 4 + 1), 256, 0, ctx->stream, weight, idx, pos_table, out,
                 tokens, pos_table ? seq : 1, dim, vocab, err);
  NRS_LAUNCHED(ctx);
  return NRS_OK;
}

int nrs_embedding_fwd(nrs_ctx* ctx, const float* weight, const int32_t* idx, float* out, int tokens, int dim, int vocab) {
  return nrs_embedding_pos_fwd(ctx, weight, idx, nullptr, out, tokens, 1, dim, vocab);
}

int nrs_embedding_bwd(nrs_ctx* ctx, const float* g, const int32_t* idx, float* dweight, int tokens, int dim,
                      int vocab, int accumulate) {
  NRS_REQUIRE_CTX(ctx);
  NRS_REQUIRE(ctx, tokens >= 0 && dim > 0 && vocab > 0, NRS_ERR_SHAPE, "nrs_embedding_bwd: bad shape");
  NRS_REQUIRE(ctx, dweight && (tokens == 0 || (g && idx)), NRS_ERR_ARG, "nrs_embedding_bwd: null tensor");
  NRS_PDL_LAUNCH(embed_bwd_kernel, vocab, 256, 0, ctx->stream, g, idx, dweight, tokens, dim, accumulate);
  NRS_LAUNCHED(ctx);
  return NRS_OK;
}

int nrs_causal_mask(nrs_ctx* ctx, const float* x, float* y, int batch, int s, int backward, int accumulate) {
  NRS_REQUIRE_CTX(ctx);
  NRS_REQUIRE(ctx, batch >= 0 && s >= 0, NRS_ERR_SHAPE, "nrs_causal_mask: negative dimension");
  const size_t total = (size_t)batch * s * s;
  if (total == 0) return NRS_OK;
  NRS_REQUIRE(ctx, x && y, NRS_ERR_ARG, "nrs_causal_mask: null tensor");
  NRS_PDL_LAUNCH(causal_mask_kernel, grid_for(ctx, total), 256, 0, ctx->stream, x, y, total, s, backward, accumulate);
  NRS_LAUNCHED(ctx);
  return NRS_OK;
}

int nrs_permute_heads(nrs_ctx* ctx, const float* x, float* y, int batch, int s, int heads, int d_head, int to_heads,
                      int accumulate) {
  NRS_REQUIRE_CTX(ctx);
  NRS_REQUIRE(ctx, batch >= 0 && s >= 0 && heads > 0 && d_head > 0, NRS_ERR_SHAPE, "nrs_permute_heads: bad shape");
  const size_t total = (size_t)batch * s * heads * d_head;
  if (total == 0) return NRS_OK;
  NRS_REQUIRE(ctx, x && y, NRS_ERR_ARG, "nrs_permute_heads: null tensor");
  NRS_PDL_LAUNCH(permute_heads_kernel, grid_for(ctx, total), 256, 0, ctx->stream, x, y, total, s, heads, d_head, to_heads, accumulate);
  NRS_LAUNCHED(ctx);
  return NRS_OK;
}

}  // extern "C"
