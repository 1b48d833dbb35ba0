// Problem descriptions for the CUDA-core implicit-GEMM kernel (simt_igemm.cu).
//
// Every contraction on the training path is written as C(m,n) = sum_k A(m,k)*B(k,n)
// where A and B are *functions* of the indices that read the caller's tensors in
// place (no im2col matrix, no transposed copies).  A problem type provides
//   ARow a_row(batch, m)            decode everything that depends on m only
//   float a_load(const ARow&, k)    fetch A(m,k), 0 outside the tensor
//   BCol b_col(batch, n), b_load    the same for B
//   void store(batch, m, n, v)      epilogue (bias, activation, accumulate)
// and says along which index each operand is contiguous in memory so the tile
// loader can keep global loads coalesced.
//
// The functions are __host__ __device__ so the index arithmetic can be unit
// tested on a CPU, without a GPU.
#pragma once

#include <cstddef>
#include <cstdint>

#if defined(__CUDACC__)
#define NRS_HD __host__ __device__ __forceinline__
#else
#define NRS_HD inline
#endif

// Division by a runtime constant via multiply-high; valid for 0 <= x < 2^31.
struct NrsFastDiv {
  uint32_t d = 1, mul = 0, shr = 0;
  NrsFastDiv() = default;
  explicit NrsFastDiv(int denom) : d((uint32_t)denom) {
    if (denom != 1) {
      uint32_t lg = 0;
      while ((1u << lg) < (uint32_t)denom) ++lg;
      const uint32_t p = 31 + lg;
      mul = (uint32_t)((((uint64_t)1 << p) + (uint64_t)denom - 1) / (uint64_t)denom);
      shr = p - 32;
    }
  }
  NRS_HD uint32_t div(uint32_t x) const {
#if defined(__CUDA_ARCH__)
    return d != 1 ? __umulhi(x, mul) >> shr : x;
#else
    return d != 1 ? (uint32_t)(((uint64_t)x * mul) >> 32) >> shr : x;
#endif
  }
  NRS_HD void divmod(uint32_t x, uint32_t& q, uint32_t& r) const { q = div(x); r = x - q * d; }
};

NRS_HD float nrs_gelu_f(float xi) {
  const float inner = 0.7978845608f * (xi + 0.044715f * xi * xi * xi);
  return 0.5f * xi * (1.0f + tanhf(inner));
}
NRS_HD float nrs_apply_act(float v, int act) {
  if (act == 1) return v > 0.0f ? v : 0.0f;
  if (act == 2) return nrs_gelu_f(v);
  return v;
}

// ---------------------------------------------------------------- dense GEMM
// C[b][m,n] = act(op(A[b]) op(B[b]) + bias[n]) + beta*C, row-major.
template <bool TA, bool TB>
struct NrsGemmProb {
  static constexpr bool kAContigM = TA;    // A stored [k,m] when transposed
  static constexpr bool kBContigN = !TB;   // B stored [k,n] unless transposed
  static constexpr bool kStoreContigM = false;
  int M, N, K, batches;
  const float* A; const float* B; float* C; const float* bias;
  int act; float beta;
  size_t strideA, strideB, strideC;
  struct ARow { const float* p; };
  struct BCol { const float* p; };
  NRS_HD ARow a_row(int b, int m) const { return {A + b * strideA + (TA ? (size_t)m : (size_t)m * K)}; }
  NRS_HD float a_load(const ARow& r, int k) const { return TA ? r.p[(size_t)k * M] : r.p[k]; }
  NRS_HD BCol b_col(int b, int n) const { return {B + b * strideB + (TB ? (size_t)n * K : (size_t)n)}; }
  NRS_HD float b_load(const BCol& c, int k) const { return TB ? c.p[k] : c.p[(size_t)k * N]; }
  NRS_HD void store(int b, int m, int n, float v) const {
    float* dst = C + b * strideC + (size_t)m * N + n;
    if (bias) v += bias[n];
    v = nrs_apply_act(v, act);
    if (beta != 0.0f) v += beta * *dst;
    *dst = v;
  }
};

// ------------------------------------------------------------- conv geometry
struct NrsConvGeom {
  int n, ci, h, w, co, kh, kw, stride, pad, oh, ow;
  NrsFastDiv div_khkw, div_kw, div_ohow, div_ow, div_hw, div_w;
  NrsConvGeom() = default;
  NrsConvGeom(int n_, int ci_, int h_, int w_, int co_, int kh_, int kw_, int s_, int p_)
      : n(n_), ci(ci_), h(h_), w(w_), co(co_), kh(kh_), kw(kw_), stride(s_), pad(p_) {
    oh = (h + 2 * pad - kh) / stride + 1;
    ow = (w + 2 * pad - kw) / stride + 1;
    div_khkw = NrsFastDiv(kh * kw); div_kw = NrsFastDiv(kw);
    div_ohow = NrsFastDiv(oh * ow); div_ow = NrsFastDiv(ow);
    div_hw = NrsFastDiv(h * w);     div_w = NrsFastDiv(w);
  }
};

// Forward: y[n,co,oy,ox] = act(sum_{ci,i,j} x[n,ci,oy*s+i-p,ox*s+j-p] w[co,ci,i,j] + b[co])
// m = (n,oy,ox), nn = co, k = (ci,i,j).
struct NrsConvFpropProb {
  static constexpr bool kAContigM = true;
  static constexpr bool kBContigN = false;
  static constexpr bool kStoreContigM = true;
  int M, N, K, batches;
  NrsConvGeom g;
  const float* x; const float* wgt; const float* bias; float* y; int act;
  struct ARow { const float* p; int iy0, ix0; };
  struct BCol { const float* p; };
  NRS_HD ARow a_row(int, int m) const {
    uint32_t img, pix, oy, ox;
    g.div_ohow.divmod((uint32_t)m, img, pix);
    g.div_ow.divmod(pix, oy, ox);
    return {x + (size_t)img * g.ci * g.h * g.w, (int)oy * g.stride - g.pad, (int)ox * g.stride - g.pad};
  }
  NRS_HD float a_load(const ARow& r, int k) const {
    uint32_t c, t, i, j;
    g.div_khkw.divmod((uint32_t)k, c, t);
    g.div_kw.divmod(t, i, j);
    const int iy = r.iy0 + (int)i, ix = r.ix0 + (int)j;
    if ((unsigned)iy >= (unsigned)g.h || (unsigned)ix >= (unsigned)g.w) return 0.0f;
    return r.p[((size_t)c * g.h + iy) * g.w + ix];
  }
  NRS_HD BCol b_col(int, int n) const { return {wgt + (size_t)n * K}; }
  NRS_HD float b_load(const BCol& c, int k) const { return c.p[k]; }
  NRS_HD void store(int, int m, int n, float v) const {
    uint32_t img, pix;
    g.div_ohow.divmod((uint32_t)m, img, pix);
    if (bias) v += bias[n];
    y[((size_t)img * g.co + n) * (size_t)(g.oh * g.ow) + pix] = nrs_apply_act(v, act);
  }
};

// Data gradient: dx[n,ci,y,x] (+)= sum_{co,i,j} dy[n,co,(y+p-i)/s,(x+p-j)/s] w[co,ci,i,j]
// (terms whose division is inexact or out of range vanish).
// m = (n,y,x), nn = ci, k = (co,i,j).
struct NrsConvDgradProb {
  static constexpr bool kAContigM = true;
  static constexpr bool kBContigN = false;
  static constexpr bool kStoreContigM = true;
  int M, N, K, batches;
  NrsConvGeom g;
  const float* dy; const float* wgt; float* dx; int accumulate;
  struct ARow { const float* p; int yp, xp; };
  struct BCol { const float* p; };
  NRS_HD ARow a_row(int, int m) const {
    uint32_t img, pix, yy, xx;
    g.div_hw.divmod((uint32_t)m, img, pix);
    g.div_w.divmod(pix, yy, xx);
    return {dy + (size_t)img * g.co * g.oh * g.ow, (int)yy + g.pad, (int)xx + g.pad};
  }
  NRS_HD float a_load(const ARow& r, int k) const {
    uint32_t c, t, i, j;
    g.div_khkw.divmod((uint32_t)k, c, t);
    g.div_kw.divmod(t, i, j);
    int oy = r.yp - (int)i, ox = r.xp - (int)j;
    if (oy < 0 || ox < 0) return 0.0f;
    if (g.stride != 1) {
      if (oy % g.stride || ox % g.stride) return 0.0f;
      oy /= g.stride; ox /= g.stride;
    }
    if (oy >= g.oh || ox >= g.ow) return 0.0f;
    return r.p[((size_t)c * g.oh + oy) * g.ow + ox];
  }
  NRS_HD BCol b_col(int, int n) const { return {wgt + (size_t)n * g.kh * g.kw}; }
  NRS_HD float b_load(const BCol& c, int k) const {
    uint32_t oc, t;
    g.div_khkw.divmod((uint32_t)k, oc, t);
    return c.p[(size_t)oc * g.ci * g.kh * g.kw + t];
  }
  NRS_HD void store(int, int m, int n, float v) const {
    uint32_t img, pix;
    g.div_hw.divmod((uint32_t)m, img, pix);
    float* dst = dx + ((size_t)img * g.ci + n) * (size_t)(g.h * g.w) + pix;
    *dst = accumulate ? *dst + v : v;
  }
};

// Weight gradient: dw[co,ci,i,j] (+)= sum_{n,oy,ox} dy[n,co,oy,ox] x[n,ci,oy*s+i-p,ox*s+j-p]
// m = co, nn = (ci,i,j), k = (n,oy,ox)  — a long-K problem, run split-K.
struct NrsConvWgradProb {
  static constexpr bool kAContigM = false;
  static constexpr bool kBContigN = false;
  static constexpr bool kStoreContigM = false;
  int M, N, K, batches;
  NrsConvGeom g;
  const float* dy; const float* x; float* dw; int accumulate;
  struct ARow { const float* p; };
  struct BCol { const float* p; int dyo, dxo; };
  NRS_HD ARow a_row(int, int m) const { return {dy + (size_t)m * g.oh * g.ow}; }
  NRS_HD float a_load(const ARow& r, int k) const {
    uint32_t img, pix;
    g.div_ohow.divmod((uint32_t)k, img, pix);
    return r.p[(size_t)img * g.co * g.oh * g.ow + pix];
  }
  NRS_HD BCol b_col(int, int n) const {
    uint32_t c, t, i, j;
    g.div_khkw.divmod((uint32_t)n, c, t);
    g.div_kw.divmod(t, i, j);
    return {x + (size_t)c * g.h * g.w, (int)i - g.pad, (int)j - g.pad};
  }
  NRS_HD float b_load(const BCol& c, int k) const {
    uint32_t img, pix, oy, ox;
    g.div_ohow.divmod((uint32_t)k, img, pix);
    g.div_ow.divmod(pix, oy, ox);
    const int iy = (int)oy * g.stride + c.dyo, ix = (int)ox * g.stride + c.dxo;
    if ((unsigned)iy >= (unsigned)g.h || (unsigned)ix >= (unsigned)g.w) return 0.0f;
    return c.p[((size_t)img * g.ci * g.h + iy) * g.w + ix];
  }
  NRS_HD void store(int, int m, int n, float v) const {
    float* dst = dw + (size_t)m * N + n;
    *dst = accumulate ? *dst + v : v;
  }
};
