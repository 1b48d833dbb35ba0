// Convolution forward and data gradient as implicit GEMM on tcgen05 (TF32 / 3xTF32).
//
// No im2col matrix exists anywhere.  The activation is staged once as NHWC
// (channels innermost) planes; output pixels are GEMM rows (a tile is Wt x Ht x Nt
// = up to 128 pixels of Nt images), output channels are GEMM columns, and the
// reduction runs over (tap, 32-channel block).  For every tap the A slice is ONE
// 4-D TMA box {32 channels, Wt, Ht, Nt} whose spatial origin is shifted by the
// tap offset; rows or columns that fall outside the image are zero-filled by TMA,
// which is exactly the zero padding.  (The shift lands on the W/H coordinates;
// the innermost, 16-byte-aligned coordinate is the channel block.)  The B slice
// is a plain 2-D box of the re-laid-out weights [out_ch][(tap, in_ch)].
//
//   forward        y[n,co,oy,ox]  = act(b[co] + sum x[n,ci,oy+i-p,ox+j-p] w[co,ci,i,j])
//   data gradient  dx[n,ci,y,x] (+)= sum dy[n,co,y-i+p,x-j+p] w[co,ci,i,j]
// are the same kernel with the tap sign flipped and the roles of the channel
// counts exchanged.  The epilogue writes NCHW directly: for a fixed channel the 32
// lanes of a warp hold 32 consecutive pixels, so every store is a full 128-byte line.
//
// Stride-1 convolutions with channel counts that are multiples of 32 run here;
// everything else (first layers with 1 or 3 channels, strides) runs on the FFMA
// implicit-GEMM kernel.
//
// Reference counterparts: conv2d_im2col + matmul_nn + conv2d_col2out (forward),
// conv2d_out2mm + matmul_tn + conv2d_col2im (data gradient) — src/cuda/nn/conv.rs:27-149,
// 244-312.
#include "tc_mainloop.cuh"

namespace {

struct ConvPolicy {
  int Wt, Ht, Nt, tiles_y;
  int out_h, out_w, n_img, n_ch_out;
  int cblocks, kw_taps;
  int sgn, base_y, base_x;
  float* out;
  const float* bias;
  int act, accumulate;
  uint32_t slice_bytes;
  // optional: ReLU mask taken from an NCHW tensor of the output's shape, and NHWC TF32 planes of
  // the result for the next tensor-core kernel
  const float* mask_src;
  float* out_hi;
  float* out_lo;
  // optional: [tiles_m * 4][n_ch_out] sums of the finished values over each epilogue warp's 32 rows
  float* colsum_partial;

  __device__ __forceinline__ uint32_t a_slice_bytes() const { return slice_bytes; }
  __device__ __forceinline__ void load_a(void* dst, const CUtensorMap* tm, uint64_t* bar, int kb, int tile_m, int) const {
    const int tap = kb / cblocks, cb = kb - tap * cblocks;
    const int i = tap / kw_taps, j = tap - i * kw_taps;
    const int n0 = (tile_m / tiles_y) * Nt, y0 = (tile_m % tiles_y) * Ht;
    tc::tma_load_4d(dst, tm, bar, cb * 32, sgn * j + base_x, y0 + sgn * i + base_y, n0);
  }
  // NCHW offset of channel 0 of the pixel behind accumulator row `row`, and the pixel's linear index.
  __device__ __forceinline__ bool locate(int tile_m, int row, size_t* nchw_off, size_t* pixel) const {
    if (row >= Wt * Ht * Nt) return false;
    const int xt = row % Wt, t = row / Wt;
    const int yt = t % Ht, nt = t / Ht;
    const int n = (tile_m / tiles_y) * Nt + nt, y = (tile_m % tiles_y) * Ht + yt;
    if (n >= n_img || y >= out_h) return false;
    *nchw_off = (size_t)n * n_ch_out * out_h * out_w + (size_t)y * out_w + xt;
    *pixel = ((size_t)n * out_h + y) * out_w + xt;
    return true;
  }
  __device__ __forceinline__ void store(int tile_m, int, int row, int ch, float v) const {
    size_t off, pixel;
    if (ch >= n_ch_out || !locate(tile_m, row, &off, &pixel)) return;
    off += (size_t)ch * out_h * out_w;
    if (bias) v += bias[ch];
    v = nrs_apply_act(v, act);
    if (accumulate) v += out[off];
    if (mask_src && !(mask_src[off] > 0.0f)) v = 0.0f;
    out[off] = v;
    if (out_hi) {
      const float hv = tc::tf32_rn(v);
      out_hi[pixel * n_ch_out + ch] = hv;
      if (out_lo) out_lo[pixel * n_ch_out + ch] = v - hv;
    }
  }
  static constexpr bool kCanEmit = true;
  __device__ __forceinline__ float* colsum_row(int tile_m, int q) const {
    return colsum_partial ? colsum_partial + ((size_t)tile_m * 4 + q) * n_ch_out : nullptr;
  }
  // TMA-store origin (x, y, image) of tile_m's pixel box in the NHWC planes.
  __device__ __forceinline__ void out_origin(int tile_m, int* x0, int* y0, int* n0) const {
    *x0 = 0;
    *y0 = (tile_m % tiles_y) * Ht;
    *n0 = (tile_m / tiles_y) * Nt;
  }
  // One accumulator row, 32 consecutive channels [nb, nb+32): bias, activation, accumulate, mask,
  // NCHW store; the finished values come back in v (zeros for rows outside the tensor) so the
  // caller can emit them as planes.  Loads are issued in batches ahead of the stores.
  __device__ __forceinline__ void epilogue(int tile_m, int, int row, int nb, int, const uint32_t (&r)[32], float (&v)[32]) const {
    size_t off, pixel;
    const bool live = nb < n_ch_out && locate(tile_m, row, &off, &pixel);   // channel counts are multiples of 32
    if (!live) {
#pragma unroll
      for (int j = 0; j < 32; ++j) v[j] = 0.0f;
      return;
    }
    const size_t plane = (size_t)out_h * out_w;
    float* dst = out + off + (size_t)nb * plane;
#pragma unroll
    for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]);
    if (bias) {
#pragma unroll
      for (int j = 0; j < 32; ++j) v[j] += __ldg(bias + nb + j);
    }
    if (act != NRS_ACT_NONE) {
#pragma unroll
      for (int j = 0; j < 32; ++j) v[j] = nrs_apply_act(v[j], act);
    }
    if (accumulate) {
      float o[32];
#pragma unroll
      for (int j = 0; j < 32; ++j) o[j] = dst[(size_t)j * plane];
#pragma unroll
      for (int j = 0; j < 32; ++j) v[j] += o[j];
    }
    if (mask_src) {
      const float* m = mask_src + off + (size_t)nb * plane;
      float mv[32];
#pragma unroll
      for (int j = 0; j < 32; ++j) mv[j] = __ldg(m + (size_t)j * plane);
#pragma unroll
      for (int j = 0; j < 32; ++j) v[j] = mv[j] > 0.0f ? v[j] : 0.0f;
    }
#pragma unroll
    for (int j = 0; j < 32; ++j) dst[(size_t)j * plane] = v[j];
  }
};

struct ConvPlan {
  // activation read by the A operand: [n_img][a_h][a_w][a_ch] NHWC planes, staged from NCHW `act_src`
  const float* act_src;
  int n_img, a_ch, a_h, a_w;
  // weights and which re-layout
  const float* w;
  int co, ci, kh, kw, for_dgrad;
  // output NCHW [n_img][n_ch_out][out_h][out_w]
  float* out;
  int n_ch_out, out_h, out_w;
  int sgn, base;
  const float* bias;
  int act, accumulate;
};

template <int BN, int NPLANES>
int run_conv(nrs_ctx* ctx, const ConvPlan& p, const float* a_hi, const float* a_lo, const float* w_hi, const float* w_lo,
             const ConvPolicy& pol, int tiles_m, int* splits_out) {
  const int taps = p.kh * p.kw;
  const int kdim = taps * p.a_ch;
  CUtensorMap ta_hi, ta_lo, tb_hi, tb_lo;
  const uint64_t adim[4] = {(uint64_t)p.a_ch, (uint64_t)p.a_w, (uint64_t)p.a_h, (uint64_t)p.n_img};
  const uint64_t astr[3] = {(uint64_t)p.a_ch * 4, (uint64_t)p.a_w * p.a_ch * 4, (uint64_t)p.a_h * p.a_w * p.a_ch * 4};
  const uint32_t abox[4] = {32, (uint32_t)pol.Wt, (uint32_t)pol.Ht, (uint32_t)pol.Nt};
  const uint64_t bdim[3] = {(uint64_t)kdim, (uint64_t)p.n_ch_out, 1};
  const uint64_t bstr[2] = {(uint64_t)kdim * 4, (uint64_t)kdim * p.n_ch_out * 4};
  const uint32_t bbox[3] = {32, (uint32_t)BN, 1};
  bool ok = tc::encode_tmap_f32(&ta_hi, a_hi, 4, adim, astr, abox) && tc::encode_tmap_f32(&tb_hi, w_hi, 3, bdim, bstr, bbox);
  if (NPLANES == 2) ok = ok && tc::encode_tmap_f32(&ta_lo, a_lo, 4, adim, astr, abox) && tc::encode_tmap_f32(&tb_lo, w_lo, 3, bdim, bstr, bbox);
  else { ta_lo = ta_hi; tb_lo = tb_hi; }
  // Output planes (optional): the same box geometry as an activation load, in output space.
  CUtensorMap to_hi, to_lo;
  if (pol.out_hi) {
    const uint64_t odim[4] = {(uint64_t)p.n_ch_out, (uint64_t)p.out_w, (uint64_t)p.out_h, (uint64_t)p.n_img};
    const uint64_t ostr[3] = {(uint64_t)p.n_ch_out * 4, (uint64_t)p.out_w * p.n_ch_out * 4, (uint64_t)p.out_h * p.out_w * p.n_ch_out * 4};
    ok = ok && tc::encode_tmap_f32(&to_hi, pol.out_hi, 4, odim, ostr, abox);
    if (pol.out_lo) ok = ok && tc::encode_tmap_f32(&to_lo, pol.out_lo, 4, odim, ostr, abox);
  }
  NRS_REQUIRE(ctx, ok, NRS_ERR_CUDA, "tc_conv: cuTensorMapEncodeTiled failed");
  return tc::launch<BN, NPLANES, ConvPolicy>(ctx, ta_hi, ta_lo, tb_hi, tb_lo, pol, tiles_m, p.n_ch_out, 1, taps * (p.a_ch / 32),
                                             pol.out_hi ? &to_hi : nullptr, pol.out_lo ? &to_lo : nullptr, splits_out);
}

int conv_common(nrs_ctx* ctx, const ConvPlan& p) {
  if (!tc::tensor_map_encoder()) return NRS_ERR_UNSUPPORTED;
  if (p.a_ch % 32 != 0 || p.n_ch_out % 32 != 0 || p.out_w > 128 || p.out_w < 1) return NRS_ERR_UNSUPPORTED;
  if (p.a_w > 256 * 1024 || p.n_img < 1) return NRS_ERR_UNSUPPORTED;
  const bool split = ctx->math_mode == NRS_MATH_3XTF32;

  // tile geometry in output space
  ConvPolicy pol{};
  pol.Wt = p.out_w;
  pol.Ht = 128 / pol.Wt;
  if (pol.Ht > p.out_h) pol.Ht = p.out_h;
  pol.Nt = 1;
  if (pol.Ht == p.out_h) {
    pol.Nt = 128 / (pol.Wt * pol.Ht);
    if (pol.Nt > p.n_img) pol.Nt = p.n_img;
    if (pol.Nt < 1) pol.Nt = 1;
  }
  // keep every TMA box inside the tensor's extents (only the origin may leave it)
  if (pol.Wt > p.a_w || pol.Ht > p.a_h || pol.Nt > p.n_img) return NRS_ERR_UNSUPPORTED;
  pol.tiles_y = (p.out_h + pol.Ht - 1) / pol.Ht;
  const long tiles_m = (long)((p.n_img + pol.Nt - 1) / pol.Nt) * pol.tiles_y;
  if (tiles_m > 2147483647L) return NRS_ERR_UNSUPPORTED;
  pol.out_h = p.out_h; pol.out_w = p.out_w; pol.n_img = p.n_img; pol.n_ch_out = p.n_ch_out;
  pol.cblocks = p.a_ch / 32; pol.kw_taps = p.kw;
  pol.sgn = p.sgn; pol.base_y = p.base; pol.base_x = p.base;
  pol.out = p.out; pol.bias = p.bias; pol.act = p.act; pol.accumulate = p.accumulate;
  pol.slice_bytes = (uint32_t)(pol.Wt * pol.Ht * pol.Nt) * 128u;
  auto extras = ctx->out_extras.find(p.out);
  if (extras != ctx->out_extras.end()) {
    const NrsOutExtras& e = extras->second;
    if (e.relu_mask_src && p.accumulate) return NRS_ERR_UNSUPPORTED;   // the mask would hit the old content too
    if (e.lo && !split) return NRS_ERR_UNSUPPORTED;
    pol.mask_src = e.relu_mask_src; pol.out_hi = e.hi; pol.out_lo = e.lo;
  }
  auto colsum = ctx->colsum_requests.find(p.out);
  if (colsum != ctx->colsum_requests.end() && !p.accumulate && tiles_m * 4 <= colsum->second.cap_rows)
    pol.colsum_partial = colsum->second.partial;

  // stage the activation: per image [C][H*W] -> [H*W][C] planes
  const size_t a_plane = (size_t)p.n_img * p.a_h * p.a_w * p.a_ch;
  const size_t w_plane = (size_t)p.co * p.ci * p.kh * p.kw;
  void *a_hi = nullptr, *a_lo = nullptr, *w_hi = nullptr, *w_lo = nullptr;
  int st = NRS_OK;
  const NrsPlanes* ready = nrs_planes_find(ctx, p.act_src, split);
  if (ready) {
    a_hi = ready->hi;
    a_lo = ready->lo;
  } else {
    st = nrs_ws_slot(ctx, NRS_WS_A_HI, a_plane * sizeof(float), &a_hi);
    if (st == NRS_OK && split) st = nrs_ws_slot(ctx, NRS_WS_A_LO, a_plane * sizeof(float), &a_lo);
    if (st != NRS_OK) return st;
    const size_t img = (size_t)p.a_h * p.a_w * p.a_ch;
    st = nrs_tc_stage(ctx, p.act_src, (float*)a_hi, (float*)a_lo, p.a_h * p.a_w, p.a_ch, p.a_ch, p.n_img, img, img, true);
    if (st != NRS_OK) return st;
  }
  const NrsWeightPlanes* wp = nrs_weight_planes_find(ctx, p.w, p.for_dgrad ? NRS_WF_CONV_DGRAD : NRS_WF_CONV_FWD);
  if (wp && wp->co == p.co && wp->ci == p.ci && wp->taps == p.kh * p.kw) {   // staged ahead with the rest of the model's weights
    w_hi = wp->hi;
    w_lo = wp->lo;
  } else {
    st = nrs_ws_slot(ctx, NRS_WS_B_HI, w_plane * sizeof(float), &w_hi);
    if (st == NRS_OK && split) st = nrs_ws_slot(ctx, NRS_WS_B_LO, w_plane * sizeof(float), &w_lo);
    if (st != NRS_OK) return st;
    st = nrs_tc_stage_conv_weight(ctx, p.w, (float*)w_hi, (float*)w_lo, p.co, p.ci, p.kh, p.kw, p.for_dgrad);
    if (st != NRS_OK) return st;
  }

  int bn = p.n_ch_out % 128 == 0 ? 128 : (p.n_ch_out % 64 == 0 ? 64 : 32);
  // Few tiles (small batches): 64-column tiles before a K-split, whose second pass costs more than the narrower
  // tile loses and cannot produce the per-tile channel sums — taken while 128-wide tiles would leave more than a
  // third of the SMs without one.
  if (bn == 128 && (long)tiles_m * (p.n_ch_out / 128) * 3 < 2L * ctx->sm_count) bn = 64;
  if (extras != ctx->out_extras.end()) ctx->out_extras.erase(extras);   // honoured from here on
  int splits = 0;
#define NRS_RUN(BN_)                                                                                                     \
  st = split ? run_conv<BN_, 2>(ctx, p, (const float*)a_hi, (const float*)a_lo, (const float*)w_hi, (const float*)w_lo, pol, (int)tiles_m, &splits) \
             : run_conv<BN_, 1>(ctx, p, (const float*)a_hi, nullptr, (const float*)w_hi, nullptr, pol, (int)tiles_m, &splits)
  if (bn == 128) { NRS_RUN(128); }
  else if (bn == 64) { NRS_RUN(64); }
  else { NRS_RUN(32); }
#undef NRS_RUN
  // channel sums come from the direct epilogue only (a K-split stores through the reduce kernel)
  if (st == NRS_OK && pol.colsum_partial && splits == 1) colsum->second.rows = (int)tiles_m * 4;
  return st;
}

}  // namespace

// y = act(conv(x, w) + b); NRS_ERR_UNSUPPORTED when the shape is outside this kernel's range.
int nrs_tc_conv_fwd(nrs_ctx* ctx, const float* x, const float* w, const float* b, float* y, int n, int ci, int h,
                    int wd, int co, int kh, int kw, int stride, int pad, int act) {
  if (stride != 1) return NRS_ERR_UNSUPPORTED;
  ConvPlan p{};
  p.act_src = x; p.n_img = n; p.a_ch = ci; p.a_h = h; p.a_w = wd;
  p.w = w; p.co = co; p.ci = ci; p.kh = kh; p.kw = kw; p.for_dgrad = 0;
  p.out = y; p.n_ch_out = co; p.out_h = h + 2 * pad - kh + 1; p.out_w = wd + 2 * pad - kw + 1;
  p.sgn = 1; p.base = -pad;
  p.bias = b; p.act = act; p.accumulate = 0;
  return conv_common(ctx, p);
}

// dx (+)= conv_transpose(dy, w)
int nrs_tc_conv_dgrad(nrs_ctx* ctx, const float* w, const float* dy, float* dx, int n, int ci, int h, int wd, int co,
                      int kh, int kw, int stride, int pad, int accumulate) {
  if (stride != 1) return NRS_ERR_UNSUPPORTED;
  ConvPlan p{};
  p.act_src = dy; p.n_img = n; p.a_ch = co; p.a_h = h + 2 * pad - kh + 1; p.a_w = wd + 2 * pad - kw + 1;
  p.w = w; p.co = co; p.ci = ci; p.kh = kh; p.kw = kw; p.for_dgrad = 1;
  p.out = dx; p.n_ch_out = ci; p.out_h = h; p.out_w = wd;
  p.sgn = -1; p.base = pad;
  p.bias = nullptr; p.act = NRS_ACT_NONE; p.accumulate = accumulate;
  return conv_common(ctx, p);
}
