// Operand staging for the tensor-core kernels: one memory-bound pass that brings an
// operand into the K-major, 32-float-aligned form TMA wants and, for 3xTF32,
// splits it into a TF32 high plane (round-to-nearest) and an f32 residual plane
// (x - hi, exact).  Without the split the single plane is still rounded to nearest
// TF32: the tensor core truncates its inputs, and truncation's systematic bias
// compounds through a deep network where rounding's does not.  Transposed sources ([K][rows], e.g. NCHW images seen as
// [C][H*W]) go through 32x32 shared-memory tiles so both sides stay coalesced.
#include "tc_mainloop.cuh"

namespace {

template <bool SPLIT>
__global__ void __launch_bounds__(256)
stage_rows_kernel(const float* __restrict__ src, float* __restrict__ hi, float* __restrict__ lo, int rows, int K,
                  int ldk, size_t src_bstride, size_t dst_bstride) {
  NRS_PDL_PROLOGUE();
  const int b = blockIdx.y;
  src += b * src_bstride;
  hi += b * dst_bstride;
  if (SPLIT) lo += b * dst_bstride;
  const int q = ldk / 4;
  const size_t total4 = (size_t)rows * q;
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  const bool vec = (K & 3) == 0 && ((reinterpret_cast<uintptr_t>(src) & 15) == 0);
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total4; i += stride) {
    const size_t r = i / q;
    const int k = (int)(i - r * q) * 4;
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
    if (vec) {
      if (k < K) v = *reinterpret_cast<const float4*>(src + r * K + k);
    } else {
      if (k + 0 < K) v.x = src[r * K + k + 0];
      if (k + 1 < K) v.y = src[r * K + k + 1];
      if (k + 2 < K) v.z = src[r * K + k + 2];
      if (k + 3 < K) v.w = src[r * K + k + 3];
    }
    if (SPLIT) {
      const float4 h = make_float4(tc::tf32_rn(v.x), tc::tf32_rn(v.y), tc::tf32_rn(v.z), tc::tf32_rn(v.w));
      *reinterpret_cast<float4*>(lo + r * ldk + k) = make_float4(v.x - h.x, v.y - h.y, v.z - h.z, v.w - h.w);
      *reinterpret_cast<float4*>(hi + r * ldk + k) = h;
    } else {
      *reinterpret_cast<float4*>(hi + r * ldk + k) =
          make_float4(tc::tf32_rn(v.x), tc::tf32_rn(v.y), tc::tf32_rn(v.z), tc::tf32_rn(v.w));
    }
  }
}

template <bool SPLIT>
__global__ void __launch_bounds__(256)
stage_transpose_kernel(const float* __restrict__ src, float* __restrict__ hi, float* __restrict__ lo, int rows, int K,
                       int ldk, size_t src_bstride, size_t dst_bstride) {
  NRS_PDL_PROLOGUE();
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
    const int r = r0 + i, k = k0 + tx;  // k < ldk always: ldk is a multiple of 32
    if (r < rows) {
      const float v = tile[tx][i];
      if (SPLIT) {
        const float h = tc::tf32_rn(v);
        hi[(size_t)r * ldk + k] = h;
        lo[(size_t)r * ldk + k] = v - h;
      } else {
        hi[(size_t)r * ldk + k] = tc::tf32_rn(v);
      }
    }
  }
}

template <bool SPLIT>
__global__ void __launch_bounds__(256)
stage_conv_weight_kernel(const float* __restrict__ w, float* __restrict__ hi, float* __restrict__ lo, int co_n, int ci_n,
                         int kh, int kw, int for_dgrad) {
  NRS_PDL_PROLOGUE();
  const size_t total = (size_t)co_n * ci_n * kh * kw;
  const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= total) return;
  // idx enumerates the OUTPUT so writes are coalesced.
  const int taps = kh * kw;
  int co, ci, t;
  if (!for_dgrad) {            // out[co][t*ci_n + ci]
    ci = (int)(idx % ci_n);
    t = (int)((idx / ci_n) % taps);
    co = (int)(idx / ((size_t)ci_n * taps));
  } else {                     // out[ci][t*co_n + co]
    co = (int)(idx % co_n);
    t = (int)((idx / co_n) % taps);
    ci = (int)(idx / ((size_t)co_n * taps));
  }
  const float v = w[((size_t)co * ci_n + ci) * taps + t];
  if (SPLIT) {
    const float h = tc::tf32_rn(v);
    hi[idx] = h;
    lo[idx] = v - h;
  } else {
    hi[idx] = tc::tf32_rn(v);
  }
}

// Gradient staging fused with the masks that precede a convolution's backward pass.
//   MODE 0  v = (y > 0) ? dy : 0                          (ReLU folded into the conv: y is its output)
//   MODE 1  v = (argmax[o] == idx && y[o] > 0) ? g[o] : 0  (k x k / stride k max-pool on top of that;
//           y is the POOLED output here: the window's maximum is > 0 exactly where the winner
//           passed the ReLU, so the full-resolution activation is not read at all)
// One pass reads the NCHW sources through 32 channel x 32 pixel tiles and writes the
// masked gradient in NCHW (optional) and as NHWC TF32 planes (optional).
template <bool SPLIT, int MODE>
__global__ void __launch_bounds__(256)
stage_masked_kernel(const float* __restrict__ g, const float* __restrict__ y, const int32_t* __restrict__ argmax,
                    float* __restrict__ nchw_out, float* __restrict__ hi, float* __restrict__ lo, int c_n, int h,
                    int w, int k, int oh, int ow) {
  NRS_PDL_PROLOGUE();
  __shared__ float tile[32][33];
  const int img = blockIdx.z, hw = h * w;
  const int p0 = blockIdx.x * 32, c0 = blockIdx.y * 32;
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  for (int i = ty; i < 32; i += 8) {
    const int c = c0 + i, px = p0 + tx;
    float v = 0.0f;
    if (c < c_n && px < hw) {
      const size_t idx = ((size_t)img * c_n + c) * hw + px;
      if (MODE == 0) {
        v = y[idx] > 0.0f ? g[idx] : 0.0f;
      } else {
        const int yy = px / w, xx = px - yy * w;
        const int oy = yy / k, ox = xx / k;
        if (oy < oh && ox < ow) {
          const size_t o = (((size_t)img * c_n + c) * oh + oy) * ow + ox;
          if ((size_t)argmax[o] == idx && y[o] > 0.0f) v = g[o];
        }
      }
      if (nchw_out) nchw_out[idx] = v;
    }
    tile[i][tx] = v;
  }
  if (!hi) return;
  __syncthreads();
  for (int i = ty; i < 32; i += 8) {
    const int px = p0 + i, c = c0 + tx;
    if (px < hw && c < c_n) {
      const float v = tile[tx][i];
      const size_t o = ((size_t)img * hw + px) * c_n + c;
      const float hv = tc::tf32_rn(v);
      hi[o] = hv;
      if (SPLIT) lo[o] = v - hv;
    }
  }
}


// MODE 1 for 2x2 / stride-2 pooling over even-sized images, organised around the POOLED
// elements (a quarter of the output): a block takes 32 channels x 32 consecutive pooled
// positions (counted across images), reads g, the pooled output and argmax once, coalesced,
// and produces the 2x2 windows: NCHW as float2 row segments, NHWC planes one full 128-byte
// line (32 channels of a pixel) per warp store, through a shared-memory tile.
template <bool SPLIT>
__global__ void __launch_bounds__(256)
pool2_bwd_planes_kernel(const float* __restrict__ g, const float* __restrict__ pooled, const int32_t* __restrict__ argmax,
                        float* __restrict__ nchw_out, float* __restrict__ hi, float* __restrict__ lo,
                        float* __restrict__ chan_partial /*[gridDim.x][c_n] per-block channel sums, or null*/, int n_img,
                        int c_n, int h, int w) {
  NRS_PDL_PROLOGUE();
  __shared__ float tile[32][129];   // [channel][q*32 + position], q = 2*dy + dx inside the window
  __shared__ long long pix_base[32]; // linear index of each position's top-left pixel, -1 beyond the end
  const int oh = h >> 1, ow = w >> 1, ohw = oh * ow, hw = h * w;
  const long total_pos = (long)n_img * ohw;
  const long gp0 = (long)blockIdx.x * 32;
  const int c0 = blockIdx.y * 32;
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  {
    const long gp = gp0 + tx;
    const bool live = gp < total_pos;
    const int img = live ? (int)(gp / ohw) : 0;
    const int po = live ? (int)(gp - (long)img * ohw) : 0;
    const int oy = po / ow, ox = po - oy * ow;
    if (ty == 0) pix_base[tx] = live ? (long long)img * hw + (long long)(2 * oy) * w + 2 * ox : -1;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int cl = ty + 8 * i, c = c0 + cl;
      float v0 = 0.0f, v1 = 0.0f, v2 = 0.0f, v3 = 0.0f, gv = 0.0f;
      if (live && c < c_n) {
        const size_t chan = (size_t)img * c_n + c;
        const size_t o = chan * ohw + po;
        gv = pooled[o] > 0.0f ? g[o] : 0.0f;
        const int local = (int)((size_t)argmax[o] - chan * hw);   // winner inside the channel plane
        const int wy = local / w, wx = local - wy * w;
        const int q = ((wy - 2 * oy) << 1) | (wx - 2 * ox);
        v0 = q == 0 ? gv : 0.0f; v1 = q == 1 ? gv : 0.0f; v2 = q == 2 ? gv : 0.0f; v3 = q == 3 ? gv : 0.0f;
        if (nchw_out) {
          float* dst = nchw_out + chan * hw + (size_t)(2 * oy) * w + 2 * ox;
          *reinterpret_cast<float2*>(dst) = make_float2(v0, v1);
          *reinterpret_cast<float2*>(dst + w) = make_float2(v2, v3);
        }
      }
      tile[cl][tx] = v0; tile[cl][32 + tx] = v1; tile[cl][64 + tx] = v2; tile[cl][96 + tx] = v3;
      if (chan_partial) {   // the window's four outputs sum to gv: fixed-order butterfly over the 32 positions
        float sum = gv;
#pragma unroll
        for (int d = 16; d > 0; d >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, d);
        if (tx == 0 && c < c_n) chan_partial[(size_t)blockIdx.x * c_n + c] = sum;
      }
    }
  }
  if (!hi) return;
  __syncthreads();
  // warp ty writes pixels k = ty, ty+8, ...: lane = channel
  const int c = c0 + tx;
  if (c >= c_n) return;
#pragma unroll 4
  for (int k = ty; k < 128; k += 8) {
    const int q = k >> 5, pl = k & 31;
    const long long base = pix_base[pl];
    if (base < 0) continue;
    const size_t pixel = (size_t)base + (size_t)(q >> 1) * w + (q & 1);
    const float v = tile[tx][k];
    const float hv = tc::tf32_rn(v);
    hi[pixel * c_n + c] = hv;
    if (SPLIT) lo[pixel * c_n + c] = v - hv;
  }
}


// 2x2 / stride-2 max-pool forward over even-sized images that also writes the pooled output's
// NHWC planes (the next convolution's operand).  Same tiling as pool2_bwd_planes_kernel: 32
// channels x 32 consecutive pooled positions per block; the first maximum in row-major window
// order wins and argmax is the flat input index, as in maxpool2x2_fwd_kernel.
template <bool SPLIT>
__global__ void __launch_bounds__(256)
pool2_fwd_planes_kernel(const float* __restrict__ x, float* __restrict__ y, int32_t* __restrict__ argmax,
                        float* __restrict__ hi, float* __restrict__ lo, int n_img, int c_n, int h, int w) {
  NRS_PDL_PROLOGUE();
  __shared__ float tile[32][33];
  const int oh = h >> 1, ow = w >> 1, ohw = oh * ow, hw = h * w;
  const long total_pos = (long)n_img * ohw;
  const long gp0 = (long)blockIdx.x * 32;
  const int c0 = blockIdx.y * 32;
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  {
    const long gp = gp0 + tx;
    const bool live = gp < total_pos;
    const int img = live ? (int)(gp / ohw) : 0;
    const int po = live ? (int)(gp - (long)img * ohw) : 0;
    const int oy = po / ow, ox = po - oy * ow;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int cl = ty + 8 * i, c = c0 + cl;
      float best = 0.0f;
      if (live && c < c_n) {
        const size_t chan = (size_t)img * c_n + c;
        const size_t first = chan * hw + (size_t)(2 * oy) * w + 2 * ox;
        const float2 r0 = *reinterpret_cast<const float2*>(x + first);
        const float2 r1 = *reinterpret_cast<const float2*>(x + first + w);
        best = r0.x;
        size_t bi = first;
        if (r0.y > best) { best = r0.y; bi = first + 1; }
        if (r1.x > best) { best = r1.x; bi = first + w; }
        if (r1.y > best) { best = r1.y; bi = first + w + 1; }
        y[chan * ohw + po] = best;
        if (argmax) argmax[chan * ohw + po] = (int32_t)bi;
      }
      tile[cl][tx] = best;
    }
  }
  __syncthreads();
  const int c = c0 + tx;   // lane = channel: one full 128-byte line per warp store
  if (c >= c_n) return;
#pragma unroll
  for (int k = ty; k < 32; k += 8) {
    const long gp = gp0 + k;
    if (gp >= total_pos) continue;
    const float v = tile[tx][k];
    const float hv = tc::tf32_rn(v);
    hi[(size_t)gp * c_n + c] = hv;
    if (SPLIT) lo[(size_t)gp * c_n + c] = v - hv;
  }
}

}  // namespace

int nrs_tc_pool2_fwd_planes(nrs_ctx* ctx, const float* x, float* y, int32_t* argmax, float* hi, float* lo, int n, int c,
                            int h, int w) {
  if (n <= 0 || c <= 0) return NRS_OK;
  if (h % 2 != 0 || w % 2 != 0 || !hi || (reinterpret_cast<uintptr_t>(x) & 7) != 0) return NRS_ERR_UNSUPPORTED;
  const long blocks = ((long)n * (h / 2) * (w / 2) + 31) / 32;
  if (blocks > 2147483647L || (c + 31) / 32 > 65535) return NRS_ERR_UNSUPPORTED;
  dim3 grid((unsigned)blocks, (unsigned)((c + 31) / 32));
  if (lo) NRS_PDL_LAUNCH((pool2_fwd_planes_kernel<true>), grid, 256, 0, ctx->stream, x, y, argmax, hi, lo, n, c, h, w);
  else NRS_PDL_LAUNCH((pool2_fwd_planes_kernel<false>), grid, 256, 0, ctx->stream, x, y, argmax, hi, nullptr, n, c, h, w);
  NRS_LAUNCHED(ctx);
  return NRS_OK;
}

int nrs_tc_stage_masked(nrs_ctx* ctx, int mode, const float* g, const float* y, const int32_t* argmax, int n, int c,
                        int h, int w, int k, float* nchw_out, float* hi, float* lo, float* chan_partial,
                        int* chan_partial_rows) {
  if (chan_partial_rows) *chan_partial_rows = 0;
  if (n <= 0 || c <= 0) return NRS_OK;
  const int oh = mode == 1 ? h / k : h, ow = mode == 1 ? w / k : w;
  dim3 grid((unsigned)((h * w + 31) / 32), (unsigned)((c + 31) / 32), (unsigned)n);
  if (grid.y > 65535 || grid.z > 65535) return NRS_ERR_UNSUPPORTED;
  const bool split = lo != nullptr;
  if (mode == 1 && k == 2 && h % 2 == 0 && w % 2 == 0 && (long)n * (h / 2) * (w / 2) / 32 < 2147483647L) {
    dim3 pgrid((unsigned)(((long)n * (h / 2) * (w / 2) + 31) / 32), (unsigned)((c + 31) / 32));
    if (split) NRS_PDL_LAUNCH((pool2_bwd_planes_kernel<true>), pgrid, 256, 0, ctx->stream, g, y, argmax, nchw_out, hi, lo, chan_partial, n, c, h, w);
    else NRS_PDL_LAUNCH((pool2_bwd_planes_kernel<false>), pgrid, 256, 0, ctx->stream, g, y, argmax, nchw_out, hi, lo, chan_partial, n, c, h, w);
    NRS_LAUNCHED(ctx);
    if (chan_partial && chan_partial_rows) *chan_partial_rows = (int)pgrid.x;
    return NRS_OK;
  }
  if (mode == 0) {
    if (split) NRS_PDL_LAUNCH((stage_masked_kernel<true, 0>), grid, 256, 0, ctx->stream, g, y, argmax, nchw_out, hi, lo, c, h, w, k, oh, ow);
    else NRS_PDL_LAUNCH((stage_masked_kernel<false, 0>), grid, 256, 0, ctx->stream, g, y, argmax, nchw_out, hi, lo, c, h, w, k, oh, ow);
  } else {
    if (split) NRS_PDL_LAUNCH((stage_masked_kernel<true, 1>), grid, 256, 0, ctx->stream, g, y, argmax, nchw_out, hi, lo, c, h, w, k, oh, ow);
    else NRS_PDL_LAUNCH((stage_masked_kernel<false, 1>), grid, 256, 0, ctx->stream, g, y, argmax, nchw_out, hi, lo, c, h, w, k, oh, ow);
  }
  NRS_LAUNCHED(ctx);
  return NRS_OK;
}

int nrs_tc_stage(nrs_ctx* ctx, const float* src, float* hi, float* lo, int rows, int K, int ldk, int batch,
                 size_t src_bstride, size_t dst_bstride, bool src_k_by_rows) {
  if (rows <= 0 || K <= 0 || batch <= 0) return NRS_OK;
  if (!src_k_by_rows) {
    size_t blocks = ((size_t)rows * (ldk / 4) + 255) / 256;
    const size_t cap = (size_t)ctx->sm_count * 16;
    if (blocks > cap) blocks = cap;
    if (batch > 65535) return NRS_ERR_UNSUPPORTED;
    dim3 grid((unsigned)blocks, (unsigned)batch);
    if (lo) NRS_PDL_LAUNCH((stage_rows_kernel<true>), grid, 256, 0, ctx->stream, src, hi, lo, rows, K, ldk, src_bstride, dst_bstride);
    else NRS_PDL_LAUNCH((stage_rows_kernel<false>), grid, 256, 0, ctx->stream, src, hi, nullptr, rows, K, ldk, src_bstride, dst_bstride);
  } else {
    dim3 grid((unsigned)((rows + 31) / 32), (unsigned)(ldk / 32), (unsigned)batch);
    if (grid.y > 65535 || grid.z > 65535) return NRS_ERR_UNSUPPORTED;
    if (lo) NRS_PDL_LAUNCH((stage_transpose_kernel<true>), grid, 256, 0, ctx->stream, src, hi, lo, rows, K, ldk, src_bstride, dst_bstride);
    else NRS_PDL_LAUNCH((stage_transpose_kernel<false>), grid, 256, 0, ctx->stream, src, hi, nullptr, rows, K, ldk, src_bstride, dst_bstride);
  }
  NRS_LAUNCHED(ctx);
  return NRS_OK;
}

int nrs_tc_stage_conv_weight(nrs_ctx* ctx, const float* w, float* hi, float* lo, int co, int ci, int kh, int kw,
                             int for_dgrad) {
  const size_t total = (size_t)co * ci * kh * kw;
  if (total == 0) return NRS_OK;
  if (lo) NRS_PDL_LAUNCH((stage_conv_weight_kernel<true>), nrs_blocks(total, 256), 256, 0, ctx->stream, w, hi, lo, co, ci, kh, kw, for_dgrad);
  else NRS_PDL_LAUNCH((stage_conv_weight_kernel<false>), nrs_blocks(total, 256), 256, 0, ctx->stream, w, hi, nullptr, co, ci, kh, kw, for_dgrad);
  NRS_LAUNCHED(ctx);
  return NRS_OK;
}
