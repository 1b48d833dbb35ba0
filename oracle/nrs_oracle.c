/*
 * CPU oracle for the NeuralRs resident-GPU training path.
 *
 * TEST INFRASTRUCTURE ONLY.  This file restates, in plain C, the CPU
 * algorithms of the reference crate (JackpotMachine777/neuralrs v0.3.0) for the
 * operators on the training hot path.  It is the checker the CUDA library is
 * compared against; nothing in the shipped library links, loads or calls it.
 *
 * Every function names the reference file:line it follows.  The reference is a
 * Rust crate and no Rust toolchain exists in the build image, so the reference
 * itself cannot be compiled; parity is pinned instead on the known-answer
 * vectors of the reference's own tests (tests/nn_conv_test.rs,
 * tests/nn_conv_padding_test.rs, tests/nn_maxpool_test.rs, ...), which
 * tests/test_oracle_golden.py replays against this file.
 *
 * The file is compiled twice into one shared object:
 *   -DNRS_ACC=float   -> symbols ending in _f32: accumulates in f32 in the
 *                        reference's own loop order (bit-faithful where the
 *                        reference is serial; the reference's Rayon folds are
 *                        themselves order-nondeterministic).
 *   -DNRS_ACC=double  -> symbols ending in _f64: same loops, sums carried in
 *                        f64.  This is the "true value" used to check the
 *                        <=1e-4 relative-error bar.
 * Build with -ffp-contract=off (Rust never contracts a*b+c into an FMA).
 */
#include <math.h>
#include <stddef.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#ifndef NRS_ACC
#define NRS_ACC float
#endif
#ifndef NRS_SUFFIX
#define NRS_SUFFIX _f32
#endif
#define NRS_CAT2(a, b) a##b
#define NRS_CAT(a, b) NRS_CAT2(a, b)
#define FN(name) NRS_CAT(name, NRS_SUFFIX)

typedef NRS_ACC acc_t;

/* ------------------------------------------------------------------ conv2d */

/* Conv2d forward.  src/nn/conv.rs:33-97: zero-pad copy, then a direct
 * cross-correlation; loop order (ic, i, j); the bias is added after the sum
 * (:87-92).  Parallel over (sample, out-channel) maps as the Rayon
 * par_chunks_mut(out_h*out_w) does (:72-75).  out_h=(H+2p-kh)/s+1 (:64-65). */
void FN(nrs_oracle_conv2d_fwd)(const float* x, const float* w, const float* b, float* y,
                               int n, int ci, int h, int wd, int co, int kh, int kw,
                               int stride, int pad) {
  const int ph = h + 2 * pad, pw = wd + 2 * pad;
  const int oh = (ph - kh) / stride + 1, ow = (pw - kw) / stride + 1;
  float* data = (float*)calloc((size_t)n * ci * ph * pw, sizeof(float));
  for (int ni = 0; ni < n; ++ni)
    for (int ic = 0; ic < ci; ++ic)
      for (int yy = 0; yy < h; ++yy)
        memcpy(&data[(((size_t)ni * ci + ic) * ph + (yy + pad)) * pw + pad],
               &x[(((size_t)ni * ci + ic) * h + yy) * wd], sizeof(float) * wd);
#pragma omp parallel for schedule(static)
  for (int map = 0; map < n * co; ++map) {
    const int ni = map / co, oc = map % co;
    float* out_map = y + (size_t)map * oh * ow;
    for (int oy = 0; oy < oh; ++oy)
      for (int ox = 0; ox < ow; ++ox) {
        acc_t sum = 0;
        for (int ic = 0; ic < ci; ++ic)
          for (int i = 0; i < kh; ++i)
            for (int j = 0; j < kw; ++j) {
              const int iy = oy * stride + i, ix = ox * stride + j;
              const size_t in_idx = (((size_t)ni * ci + ic) * ph + iy) * pw + ix;
              const size_t w_idx = (((size_t)oc * ci + ic) * kh + i) * kw + j;
              sum += (acc_t)(data[in_idx] * w[w_idx]);
            }
        sum += (acc_t)b[oc];
        out_map[oy * ow + ox] = (float)sum;
      }
  }
  free(data);
}

/* Conv2d backward.  src/nn/conv.rs:110-200.  Weight/bias gradients: a fold
 * over (sample, out-channel) units (:114-150), serial order inside a unit; the
 * reference's Rayon reduce order across units is unspecified, here units are
 * summed in index order.  Input gradient: scatter into a padded buffer per
 * sample (:152-179), then the un-pad copy accumulates (+=) into the input
 * grad (:181-193).  dw/db/dx all ACCUMULATE into what the caller passes
 * (:195-198); dx may be NULL (the GPU twin skips it when requires_grad is
 * false, src/cuda/nn/conv.rs:304). */
void FN(nrs_oracle_conv2d_bwd)(const float* x, const float* w, const float* dy,
                               float* dx, float* dw, float* db,
                               int n, int ci, int h, int wd, int co, int kh, int kw,
                               int stride, int pad) {
  const int ph = h + 2 * pad, pw = wd + 2 * pad;
  const int oh = (ph - kh) / stride + 1, ow = (pw - kw) / stride + 1;
  const size_t w_len = (size_t)co * ci * kh * kw;
  float* data = (float*)calloc((size_t)n * ci * ph * pw, sizeof(float));
  for (int ni = 0; ni < n; ++ni)
    for (int ic = 0; ic < ci; ++ic)
      for (int yy = 0; yy < h; ++yy)
        memcpy(&data[(((size_t)ni * ci + ic) * ph + (yy + pad)) * pw + pad],
               &x[(((size_t)ni * ci + ic) * h + yy) * wd], sizeof(float) * wd);

  /* weight + bias gradient: each out-channel's slice of dw depends only on
   * units (ni, oc) with that oc, so parallelise over oc and walk ni in order. */
  acc_t* wg = (acc_t*)calloc(w_len, sizeof(acc_t));
  acc_t* bg = (acc_t*)calloc((size_t)co, sizeof(acc_t));
#pragma omp parallel for schedule(static)
  for (int oc = 0; oc < co; ++oc)
    for (int ni = 0; ni < n; ++ni)
      for (int oy = 0; oy < oh; ++oy)
        for (int ox = 0; ox < ow; ++ox) {
          const float g = dy[(((size_t)ni * co + oc) * oh + oy) * ow + ox];
          bg[oc] += (acc_t)g;
          for (int ic = 0; ic < ci; ++ic)
            for (int i = 0; i < kh; ++i)
              for (int j = 0; j < kw; ++j) {
                const int iy = oy * stride + i, ix = ox * stride + j;
                const size_t in_idx = (((size_t)ni * ci + ic) * ph + iy) * pw + ix;
                const size_t w_idx = (((size_t)oc * ci + ic) * kh + i) * kw + j;
                wg[w_idx] += (acc_t)(g * data[in_idx]);
              }
        }
  for (size_t k = 0; k < w_len; ++k) dw[k] += (float)wg[k];
  for (int k = 0; k < co; ++k) db[k] += (float)bg[k];
  free(wg);
  free(bg);

  if (dx) {
    const size_t in_block = (size_t)ci * ph * pw;
#pragma omp parallel for schedule(static)
    for (int ni = 0; ni < n; ++ni) {
      acc_t* chunk = (acc_t*)calloc(in_block, sizeof(acc_t));
      for (int oc = 0; oc < co; ++oc)
        for (int oy = 0; oy < oh; ++oy)
          for (int ox = 0; ox < ow; ++ox) {
            const float g = dy[(((size_t)ni * co + oc) * oh + oy) * ow + ox];
            for (int ic = 0; ic < ci; ++ic)
              for (int i = 0; i < kh; ++i)
                for (int j = 0; j < kw; ++j) {
                  const int iy = oy * stride + i, ix = ox * stride + j;
                  const size_t in_local = ((size_t)ic * ph + iy) * pw + ix;
                  const size_t w_idx = (((size_t)oc * ci + ic) * kh + i) * kw + j;
                  chunk[in_local] += (acc_t)(g * w[w_idx]);
                }
          }
      for (int ic = 0; ic < ci; ++ic)
        for (int yy = 0; yy < h; ++yy)
          for (int xx = 0; xx < wd; ++xx)
            dx[(((size_t)ni * ci + ic) * h + yy) * wd + xx] +=
                (float)chunk[((size_t)ic * ph + (yy + pad)) * pw + (xx + pad)];
      free(chunk);
    }
  }
  free(data);
}

/* ------------------------------------------------------------------ matmul */

/* [m,k] x [k,n] -> [m,n].  src/autograd/graph/matmul.rs:17-24 (i, j, t loop,
 * data[i*n+j] accumulated in place, i.e. in f32 in the reference). */
void FN(nrs_oracle_matmul_fwd)(const float* a, const float* b, float* c, int m, int k, int n) {
#pragma omp parallel for schedule(static)
  for (int i = 0; i < m; ++i)
    for (int j = 0; j < n; ++j) {
      acc_t s = 0;
      for (int t = 0; t < k; ++t) s += (acc_t)(a[(size_t)i * k + t] * b[(size_t)t * n + j]);
      c[(size_t)i * n + j] = (float)s;
    }
}

/* dA += dC.B^T ; dB += A^T.dC.  src/autograd/graph/matmul.rs:42-62. */
void FN(nrs_oracle_matmul_bwd)(const float* a, const float* b, const float* dc,
                               float* da, float* db, int m, int k, int n) {
  if (da) {
#pragma omp parallel for schedule(static)
    for (int i = 0; i < m; ++i)
      for (int t = 0; t < k; ++t) {
        acc_t g = 0;
        for (int j = 0; j < n; ++j) g += (acc_t)(dc[(size_t)i * n + j] * b[(size_t)t * n + j]);
        da[(size_t)i * k + t] += (float)g;
      }
  }
  if (db) {
#pragma omp parallel for schedule(static)
    for (int t = 0; t < k; ++t)
      for (int j = 0; j < n; ++j) {
        acc_t g = 0;
        for (int i = 0; i < m; ++i) g += (acc_t)(a[(size_t)i * k + t] * dc[(size_t)i * n + j]);
        db[(size_t)t * n + j] += (float)g;
      }
  }
}

/* Batched matmul [b,m,k]x[b,k,n].  src/autograd/graph/bmm.rs:13-96. */
void FN(nrs_oracle_bmm_fwd)(const float* a, const float* b, float* c, int batch, int m, int k, int n) {
  for (int bi = 0; bi < batch; ++bi)
    FN(nrs_oracle_matmul_fwd)(a + (size_t)bi * m * k, b + (size_t)bi * k * n,
                              c + (size_t)bi * m * n, m, k, n);
}
void FN(nrs_oracle_bmm_bwd)(const float* a, const float* b, const float* dc, float* da, float* db,
                            int batch, int m, int k, int n) {
  for (int bi = 0; bi < batch; ++bi)
    FN(nrs_oracle_matmul_bwd)(a + (size_t)bi * m * k, b + (size_t)bi * k * n,
                              dc + (size_t)bi * m * n, da ? da + (size_t)bi * m * k : NULL,
                              db ? db + (size_t)bi * k * n : NULL, m, k, n);
}

/* -------------------------------------------------------------- add / bias */

/* Same-shape add and [rows,cols]+[cols] broadcast.  src/autograd/graph/add.rs:
 * 21-36 (forward), :52-70 (backward: passthrough; bias gets the column sum,
 * rows walked in order). */
void FN(nrs_oracle_add_fwd)(const float* a, const float* b, float* out, size_t n) {
  for (size_t i = 0; i < n; ++i) out[i] = a[i] + b[i];
}
void FN(nrs_oracle_bias_add_fwd)(const float* a, const float* bias, float* out, int rows, int cols) {
  for (int r = 0; r < rows; ++r)
    for (int c = 0; c < cols; ++c) out[(size_t)r * cols + c] = a[(size_t)r * cols + c] + bias[c];
}
void FN(nrs_oracle_bias_add_bwd)(const float* g, float* da, float* dbias, int rows, int cols) {
  if (da)
    for (size_t i = 0; i < (size_t)rows * cols; ++i) da[i] += g[i];
  for (int c = 0; c < cols; ++c) {
    acc_t s = 0;
    for (int r = 0; r < rows; ++r) s += (acc_t)g[(size_t)r * cols + c];
    dbias[c] += (float)s;
  }
}

/* ------------------------------------------------------------- activations */

/* ReLU: x>0 ? x : 0, derivative 0 at x<=0.  src/autograd/graph/relu.rs:15-19,
 * :33-41; the gradient accumulates into the parent (:43-45). */
void FN(nrs_oracle_relu_fwd)(const float* x, float* y, size_t n) {
  for (size_t i = 0; i < n; ++i) y[i] = x[i] > 0.0f ? x[i] : 0.0f;
}
void FN(nrs_oracle_relu_bwd)(const float* x, const float* g, float* dx, size_t n) {
  for (size_t i = 0; i < n; ++i) dx[i] += x[i] > 0.0f ? g[i] : 0.0f;
}

/* GELU, tanh approximation, constants 0.7978845608 and 0.044715, all in f32.
 * src/autograd/graph/gelu.rs:10-23 (forward), :36-56 (derivative). */
void FN(nrs_oracle_gelu_fwd)(const float* x, float* y, size_t n) {
  const float c = 0.7978845608f;
  for (size_t i = 0; i < n; ++i) {
    const float xi = x[i];
    const float inner = c * (xi + 0.044715f * xi * xi * xi);
    y[i] = 0.5f * xi * (1.0f + tanhf(inner));
  }
}
void FN(nrs_oracle_gelu_bwd)(const float* x, const float* g, float* dx, size_t n) {
  const float c = 0.7978845608f;
  for (size_t i = 0; i < n; ++i) {
    const float xi = x[i];
    const float inner = c * (xi + 0.044715f * xi * xi * xi);
    const float t = tanhf(inner);
    const float dinner = c * (1.0f + 3.0f * 0.044715f * xi * xi);
    const float dgelu = 0.5f * (1.0f + t) + 0.5f * xi * (1.0f - t * t) * dinner;
    dx[i] += dgelu * g[i];
  }
}

/* ----------------------------------------------------------------- maxpool */

/* k x k window, stride s, no padding; strict '>' so the first maximum in
 * row-major window order wins; argmax is the flat input index.
 * src/nn/maxpool.rs:32-62 (forward), :74-79 (backward scatter-add). */
void FN(nrs_oracle_maxpool_fwd)(const float* x, float* y, int32_t* argmax,
                                int n, int c, int h, int w, int k, int stride) {
  const int oh = (h - k) / stride + 1, ow = (w - k) / stride + 1;
  for (int ni = 0; ni < n; ++ni)
    for (int ch = 0; ch < c; ++ch)
      for (int oy = 0; oy < oh; ++oy)
        for (int ox = 0; ox < ow; ++ox) {
          float best = -INFINITY;
          size_t best_idx = 0;
          for (int i = 0; i < k; ++i)
            for (int j = 0; j < k; ++j) {
              const int iy = oy * stride + i, ix = ox * stride + j;
              const size_t in_idx = (((size_t)ni * c + ch) * h + iy) * w + ix;
              if (x[in_idx] > best) { best = x[in_idx]; best_idx = in_idx; }
            }
          const size_t out_idx = (((size_t)ni * c + ch) * oh + oy) * ow + ox;
          y[out_idx] = best;
          if (argmax) argmax[out_idx] = (int32_t)best_idx;
        }
}
void FN(nrs_oracle_maxpool_bwd)(const float* g, const int32_t* argmax, float* dx, size_t out_len) {
  for (size_t o = 0; o < out_len; ++o) dx[argmax[o]] += g[o];
}

/* ----------------------------------------------------------- cross-entropy */

/* Mean over the batch of -sum_c t*log_softmax(x), max-subtracted.
 * src/nn/loss.rs:50-76.  `divisor` is the batch the mean is taken over: the
 * reference always uses the row count (:75); data-parallel shards pass the
 * global batch so that summed shard losses equal the full-batch loss. */
float FN(nrs_oracle_ce_fwd)(const float* logits, const float* target, int batch, int classes, int divisor) {
  acc_t total = 0;
  for (int b = 0; b < batch; ++b) {
    const float* row = logits + (size_t)b * classes;
    float mx = -INFINITY;
    for (int c = 0; c < classes; ++c) mx = fmaxf(mx, row[c]);
    acc_t sum_exp = 0;
    for (int c = 0; c < classes; ++c) sum_exp += (acc_t)expf(row[c] - mx);
    const float lse = logf((float)sum_exp) + mx;
    for (int c = 0; c < classes; ++c) {
      const float ls = row[c] - lse;
      total += (acc_t)(-target[(size_t)b * classes + c] * ls);
    }
  }
  return (float)(total / (acc_t)divisor);
}
/* grad = (softmax - t)/batch, OVERWRITING the logits' grad.  src/nn/loss.rs:
 * 78-104 (pred.grad = grad, :105). */
void FN(nrs_oracle_ce_bwd)(const float* logits, const float* target, float* grad,
                           int batch, int classes, int divisor) {
  for (int b = 0; b < batch; ++b) {
    const float* row = logits + (size_t)b * classes;
    float mx = -INFINITY;
    for (int c = 0; c < classes; ++c) mx = fmaxf(mx, row[c]);
    acc_t sum = 0;
    for (int c = 0; c < classes; ++c) sum += (acc_t)expf(row[c] - mx);
    for (int c = 0; c < classes; ++c) {
      const float sm = (float)((acc_t)expf(row[c] - mx) / sum);
      grad[(size_t)b * classes + c] = (sm - target[(size_t)b * classes + c]) / (float)divisor;
    }
  }
}

/* ------------------------------------------------------------------- AdamW */

/* f32 integer power by repeated squaring, as Rust's f32::powi lowers to
 * (llvm.powi / compiler-rt __powisf2). */
static float nrs_powi_f32(float a, int b) {
  const int recip = b < 0;
  float r = 1.0f;
  while (1) {
    if (b & 1) r *= a;
    b /= 2;
    if (b == 0) break;
    a *= a;
  }
  return recip ? 1.0f / r : r;
}

/* One AdamW step over one flat parameter vector; `t` is the 0-based step
 * counter BEFORE the step (bias correction uses t+1).  Decoupled decay uses the
 * pre-update parameter.  src/optim/adamw.rs:23-46.  All arithmetic in f32 in
 * both builds (there is no long sum to carry in f64). */
void FN(nrs_oracle_adamw_step)(float* p, const float* g, float* m, float* v, size_t n,
                               float lr, float beta1, float beta2, float eps, float wd, int t) {
  const float bc1 = 1.0f - nrs_powi_f32(beta1, t + 1);
  const float bc2 = 1.0f - nrs_powi_f32(beta2, t + 1);
  for (size_t i = 0; i < n; ++i) {
    m[i] = beta1 * m[i] + (1.0f - beta1) * g[i];
    v[i] = beta2 * v[i] + (1.0f - beta2) * g[i] * g[i];
    const float m_hat = m[i] / bc1;
    const float v_hat = v[i] / bc2;
    p[i] = p[i] - lr * m_hat / (sqrtf(v_hat) + eps) - lr * wd * p[i];
  }
}

/* --------------------------------------------------------------- LayerNorm */

/* Per row over the last dim: mean, biased variance, istd=1/sqrt(var+eps),
 * xhat=(x-mean)*istd, y=gamma*xhat+beta.  src/nn/normalization.rs:38-52.
 * Saves xhat and istd for backward like the reference does. */
void FN(nrs_oracle_layernorm_fwd)(const float* x, const float* gamma, const float* beta, float* y,
                                  float* xhat, float* istd_out, int rows, int f, float eps) {
  for (int r = 0; r < rows; ++r) {
    const float* row = x + (size_t)r * f;
    acc_t s = 0;
    for (int i = 0; i < f; ++i) s += (acc_t)row[i];
    const float mean = (float)(s / (acc_t)f);
    acc_t vs = 0;
    for (int i = 0; i < f; ++i) { const float d = row[i] - mean; vs += (acc_t)(d * d); }
    const float var = (float)(vs / (acc_t)f);
    const float istd = 1.0f / sqrtf(var + eps);
    if (istd_out) istd_out[r] = istd;
    for (int i = 0; i < f; ++i) {
      const float xn = (row[i] - mean) * istd;
      if (xhat) xhat[(size_t)r * f + i] = xn;
      y[(size_t)r * f + i] = gamma[i] * xn + beta[i];
    }
  }
}
/* dx += istd*(dxhat - sum1/F - xhat*sum2/F), dgamma += sum_r g*xhat,
 * dbeta += sum_r g.  src/nn/normalization.rs:66-103. */
void FN(nrs_oracle_layernorm_bwd)(const float* g, const float* xhat, const float* istd,
                                  const float* gamma, float* dx, float* dgamma, float* dbeta,
                                  int rows, int f) {
  acc_t* dg = (acc_t*)calloc((size_t)f, sizeof(acc_t));
  acc_t* dbt = (acc_t*)calloc((size_t)f, sizeof(acc_t));
  const float nf = (float)f;
  for (int r = 0; r < rows; ++r) {
    const size_t st = (size_t)r * f;
    acc_t sum1 = 0, sum2 = 0;
    for (int i = 0; i < f; ++i) {
      const float dxhat = g[st + i] * gamma[i];
      sum1 += (acc_t)dxhat;
      sum2 += (acc_t)(dxhat * xhat[st + i]);
    }
    const float s1 = (float)sum1, s2 = (float)sum2;
    for (int i = 0; i < f; ++i) {
      const float dxhat = g[st + i] * gamma[i];
      if (dx) dx[st + i] += istd[r] * (dxhat - s1 / nf - xhat[st + i] * s2 / nf);
      dg[i] += (acc_t)(g[st + i] * xhat[st + i]);
      dbt[i] += (acc_t)g[st + i];
    }
  }
  for (int i = 0; i < f; ++i) { dgamma[i] += (float)dg[i]; dbeta[i] += (float)dbt[i]; }
  free(dg);
  free(dbt);
}

/* ----------------------------------------------------------------- softmax */

/* Row softmax over the last dim with max subtraction; backward
 * dx += s*(g - sum(s*g)).  src/autograd/graph/softmax.rs:23-35, :49-60. */
void FN(nrs_oracle_softmax_fwd)(const float* x, float* y, int rows, int width) {
  for (int r = 0; r < rows; ++r) {
    const float* row = x + (size_t)r * width;
    float mx = -INFINITY;
    for (int i = 0; i < width; ++i) mx = fmaxf(mx, row[i]);
    acc_t sum = 0;
    for (int i = 0; i < width; ++i) sum += (acc_t)expf(row[i] - mx);
    for (int i = 0; i < width; ++i) y[(size_t)r * width + i] = (float)((acc_t)expf(row[i] - mx) / sum);
  }
}
void FN(nrs_oracle_softmax_bwd)(const float* y, const float* g, float* dx, int rows, int width) {
  for (int r = 0; r < rows; ++r) {
    const size_t st = (size_t)r * width;
    acc_t dot = 0;
    for (int i = 0; i < width; ++i) dot += (acc_t)(y[st + i] * g[st + i]);
    const float d = (float)dot;
    for (int i = 0; i < width; ++i) dx[st + i] += y[st + i] * (g[st + i] - d);
  }
}

/* ------------------------------------------------------------ manipulation */

/* Batched transpose of the last two dims.  src/autograd/graph/transpose.rs:
 * 21-28; backward is the transpose of the gradient, accumulated (:45-52). */
void FN(nrs_oracle_transpose_fwd)(const float* x, float* y, int batch, int rows, int cols) {
  for (int b = 0; b < batch; ++b) {
    const size_t off = (size_t)b * rows * cols;
    for (int i = 0; i < rows; ++i)
      for (int j = 0; j < cols; ++j) y[off + (size_t)j * rows + i] = x[off + (size_t)i * cols + j];
  }
}
void FN(nrs_oracle_transpose_bwd)(const float* g, float* dx, int batch, int rows, int cols) {
  for (int b = 0; b < batch; ++b) {
    const size_t off = (size_t)b * rows * cols;
    for (int i = 0; i < rows; ++i)
      for (int j = 0; j < cols; ++j) dx[off + (size_t)i * cols + j] += g[off + (size_t)j * rows + i];
  }
}
/* x*s ; dx += g*s.  src/autograd/graph/scale.rs:11-16, :29-35. */
void FN(nrs_oracle_scale_fwd)(const float* x, float* y, size_t n, float s) {
  for (size_t i = 0; i < n; ++i) y[i] = x[i] * s;
}
void FN(nrs_oracle_scale_bwd)(const float* g, float* dx, size_t n, float s) {
  for (size_t i = 0; i < n; ++i) dx[i] += g[i] * s;
}
/* Column slice [c0,c1) of a [rows,total] matrix.  src/autograd/graph/
 * slice_cols.rs:20-25, :39-45. */
void FN(nrs_oracle_slice_cols_fwd)(const float* x, float* y, int rows, int total, int c0, int c1) {
  const int sw = c1 - c0;
  for (int r = 0; r < rows; ++r)
    for (int c = 0; c < sw; ++c) y[(size_t)r * sw + c] = x[(size_t)r * total + c0 + c];
}
void FN(nrs_oracle_slice_cols_bwd)(const float* g, float* dx, int rows, int total, int c0, int c1) {
  const int sw = c1 - c0;
  for (int r = 0; r < rows; ++r)
    for (int c = 0; c < sw; ++c) dx[(size_t)r * total + c0 + c] += g[(size_t)r * sw + c];
}
/* Write one part into / read one part out of a column concatenation.
 * src/autograd/graph/concat_cols.rs:22-33, :47-57. */
void FN(nrs_oracle_concat_write)(const float* part, float* out, int rows, int total, int off, int pw) {
  for (int r = 0; r < rows; ++r)
    for (int c = 0; c < pw; ++c) out[(size_t)r * total + off + c] = part[(size_t)r * pw + c];
}
void FN(nrs_oracle_concat_read)(const float* g, float* dpart, int rows, int total, int off, int pw) {
  for (int r = 0; r < rows; ++r)
    for (int c = 0; c < pw; ++c) dpart[(size_t)r * pw + c] += g[(size_t)r * total + off + c];
}

/* --------------------------------------------------------------- embedding */

/* Row gather out[t,:] = weight[idx[t],:]; backward scatter-add in token order.
 * src/nn/embedding.rs:19-30 (forward), :47-55 (backward); the batched form
 * (:60-113) is the same over batch*seq tokens. */
void FN(nrs_oracle_embedding_fwd)(const float* weight, const int32_t* idx, float* out, int tokens, int dim) {
  for (int t = 0; t < tokens; ++t)
    memcpy(out + (size_t)t * dim, weight + (size_t)idx[t] * dim, sizeof(float) * dim);
}
void FN(nrs_oracle_embedding_bwd)(const float* g, const int32_t* idx, float* dweight, int tokens, int dim, int vocab) {
  acc_t* acc = (acc_t*)calloc((size_t)vocab * dim, sizeof(acc_t));
  for (int t = 0; t < tokens; ++t)
    for (int d = 0; d < dim; ++d) acc[(size_t)idx[t] * dim + d] += (acc_t)g[(size_t)t * dim + d];
  for (size_t i = 0; i < (size_t)vocab * dim; ++i) dweight[i] += (float)acc[i];
  free(acc);
}

/* Sinusoidal table pe[pos,i]: exponent = 2*(i/2)/d, freq = 1/10000^exponent,
 * angle = pos*freq, even i -> sin, odd i -> cos, all in f32.
 * src/nn/positional.rs:20-33. */
void FN(nrs_oracle_positional_table)(float* pe, int max_len, int d_model) {
  for (int pos = 0; pos < max_len; ++pos)
    for (int i = 0; i < d_model; ++i) {
      const float exponent = (float)(2 * (i / 2)) / (float)d_model;
      const float freq = 1.0f / powf(10000.0f, exponent);
      const float angle = (float)pos * freq;
      pe[(size_t)pos * d_model + i] = (i % 2 == 0) ? sinf(angle) : cosf(angle);
    }
}

/* --------------------------------------------------------------- BatchNorm */

/* x is [n, c, hw]; hw == 1 is BatchNorm over [batch, features]
 * (src/nn/batchnorm.rs:28-84), hw = h*w is BatchNorm2d (src/nn/batchnorm2d.rs:28-101).
 * Training: per channel, mean then the biased variance of (x - mean) in a second
 * pass (:47-64), running = momentum*running + (1-momentum)*batch value (:66-67),
 * istd = 1/sqrt(var + eps) (:69).  Evaluation: the running statistics (:83-86).
 * xhat = (x - mean)*istd, y = gamma*xhat + beta (:72-78). */
void FN(nrs_oracle_batchnorm_fwd)(const float* x, const float* gamma, const float* beta, float* running_mean,
                                  float* running_var, float* y, float* xhat, float* istd_out, int n, int c,
                                  int hw, float eps, float momentum, int training) {
  const float count = (float)(n * hw);
  for (int ch = 0; ch < c; ++ch) {
    float mean, var;
    if (training) {
      acc_t s = 0;
      for (int ni = 0; ni < n; ++ni) {
        const size_t base = ((size_t)ni * c + ch) * hw;
        for (int p = 0; p < hw; ++p) s += (acc_t)x[base + p];
      }
      mean = (float)(s / (acc_t)count);
      acc_t vs = 0;
      for (int ni = 0; ni < n; ++ni) {
        const size_t base = ((size_t)ni * c + ch) * hw;
        for (int p = 0; p < hw; ++p) { const float d = x[base + p] - mean; vs += (acc_t)(d * d); }
      }
      var = (float)(vs / (acc_t)count);
      running_mean[ch] = momentum * running_mean[ch] + (1.0f - momentum) * mean;
      running_var[ch] = momentum * running_var[ch] + (1.0f - momentum) * var;
    } else {
      mean = running_mean[ch];
      var = running_var[ch];
    }
    const float istd = 1.0f / sqrtf(var + eps);
    istd_out[ch] = istd;
    for (int ni = 0; ni < n; ++ni) {
      const size_t base = ((size_t)ni * c + ch) * hw;
      for (int p = 0; p < hw; ++p) {
        const float xn = (x[base + p] - mean) * istd;
        if (xhat) xhat[base + p] = xn;
        y[base + p] = gamma[ch] * xn + beta[ch];
      }
    }
  }
}
/* src/nn/batchnorm2d.rs:112-163 (batchnorm.rs:97-139): training
 * dx += istd*(dxhat - sum1/N - xhat*sum2/N) with dxhat = g*gamma, sum1 = sum dxhat,
 * sum2 = sum dxhat*xhat; evaluation dx += g*gamma*istd; dgamma += sum g*xhat,
 * dbeta += sum g in both modes. */
void FN(nrs_oracle_batchnorm_bwd)(const float* g, const float* xhat, const float* istd, const float* gamma,
                                  float* dx, float* dgamma, float* dbeta, int n, int c, int hw, int training) {
  const float cnt = (float)(n * hw);
  for (int ch = 0; ch < c; ++ch) {
    acc_t sum1 = 0, sum2 = 0, dg = 0, db = 0;
    for (int ni = 0; ni < n; ++ni) {
      const size_t base = ((size_t)ni * c + ch) * hw;
      for (int p = 0; p < hw; ++p) {
        const float dxhat = g[base + p] * gamma[ch];
        sum1 += (acc_t)dxhat;
        sum2 += (acc_t)(dxhat * xhat[base + p]);
        dg += (acc_t)(g[base + p] * xhat[base + p]);
        db += (acc_t)g[base + p];
      }
    }
    const float s1 = (float)sum1, s2 = (float)sum2;
    if (dx) {
      for (int ni = 0; ni < n; ++ni) {
        const size_t base = ((size_t)ni * c + ch) * hw;
        for (int p = 0; p < hw; ++p) {
          const float dxhat = g[base + p] * gamma[ch];
          if (training) dx[base + p] += istd[ch] * (dxhat - s1 / cnt - xhat[base + p] * s2 / cnt);
          else dx[base + p] += g[base + p] * gamma[ch] * istd[ch];
        }
      }
    }
    if (dgamma) dgamma[ch] += (float)dg;
    if (dbeta) dbeta[ch] += (float)db;
  }
}

/* ----------------------------------------------------------------- Dropout */

/* out (+)= a * mask[i / hw].  hw == 1: Dropout forward `in*scale or 0` and backward
 * `grad*mask` (src/nn/dropout.rs:29-50); hw = h*w: Dropout2d, one mask value per
 * (sample, channel) plane (src/nn/dropout2d.rs, src/cuda/nn/dropout2d.rs:18-27). */
void FN(nrs_oracle_mask_mul)(const float* a, const float* mask, float* out, size_t total, int hw, int accumulate) {
  for (size_t i = 0; i < total; ++i) {
    const float r = a[i] * mask[i / (size_t)hw];
    out[i] = accumulate ? out[i] + r : r;
  }
}

/* Philox-4x32-10 (Salmon, Moraes, Dror, Shaw: "Parallel random numbers: as easy as
 * 1, 2, 3", SC'11): ten rounds of two 32x32->64 multiplies with the key bumped by
 * the Weyl constants between rounds. */
void FN(nrs_oracle_philox4x32_10)(const uint32_t ctr_in[4], const uint32_t key[2], uint32_t out[4]) {
  uint32_t c0 = ctr_in[0], c1 = ctr_in[1], c2 = ctr_in[2], c3 = ctr_in[3], k0 = key[0], k1 = key[1];
  for (int r = 0; r < 10; ++r) {
    const uint64_t p0 = (uint64_t)0xD2511F53u * c0;
    const uint64_t p1 = (uint64_t)0xCD9E8D57u * c2;
    const uint32_t n0 = (uint32_t)(p1 >> 32) ^ c1 ^ k0, n1 = (uint32_t)p1;
    const uint32_t n2 = (uint32_t)(p0 >> 32) ^ c3 ^ k1, n3 = (uint32_t)p0;
    c0 = n0; c1 = n1; c2 = n2; c3 = n3;
    k0 += 0x9E3779B9u;
    k1 += 0xBB67AE85u;
  }
  out[0] = c0; out[1] = c1; out[2] = c2; out[3] = c3;
}
/* The mask of Dropout / Dropout2d: 0 with probability p, else 1/(1-p)
 * (src/nn/dropout.rs:26-37, src/cuda/nn/dropout.rs:38-48).  The reference draws u from
 * the `rand` crate's thread-local generator, which cannot be reproduced; the
 * device library specifies its own stream instead and this restates it: element i
 * is word i%4 of the Philox block at counter (offset + i/4, 0) under the 64-bit
 * seed, u = (word >> 8) * 2^-24. */
void FN(nrs_oracle_dropout_mask)(float* mask, size_t count, float p, uint64_t seed, uint64_t offset) {
  const float scale = 1.0f / (1.0f - p);
  const uint32_t key[2] = {(uint32_t)seed, (uint32_t)(seed >> 32)};
  for (size_t b = 0; b * 4 < count; ++b) {
    const uint64_t at = offset + b;
    const uint32_t ctr[4] = {(uint32_t)at, (uint32_t)(at >> 32), 0u, 0u};
    uint32_t w[4];
    FN(nrs_oracle_philox4x32_10)(ctr, key, w);
    for (int j = 0; j < 4 && b * 4 + j < count; ++j) {
      const float u = (float)(w[j] >> 8) * (1.0f / 16777216.0f);
      mask[b * 4 + j] = u < p ? 0.0f : scale;
    }
  }
}

/* ---------------------------------------------------------- input pipeline */

/* `augment` of examples/cifar_cuda.rs:148-169 for one image [c,h,w] with the draws
 * given: out[ch,y,x] = img[ch, y-dy, flip ? w-1-(x-dx) : x-dx] inside the image,
 * zero outside. */
void FN(nrs_oracle_augment_image)(const float* img, float* out, int c, int h, int w, int flip, int dx, int dy) {
  for (int ch = 0; ch < c; ++ch)
    for (int y = 0; y < h; ++y)
      for (int x = 0; x < w; ++x) {
        const int sx = x - dx, sy = y - dy;
        float v = 0.0f;
        if (sx >= 0 && sx < w && sy >= 0 && sy < h) v = img[((size_t)ch * h + sy) * w + (flip ? w - 1 - sx : sx)];
        out[((size_t)ch * h + y) * w + x] = v;
      }
}
/* The draws of the device library's augmentation stream for image `index` of a
 * call that starts at `offset`: flip = top bit of word 0, dx / dy = floor(u * (2s+1)) - s
 * from words 1 / 2 (the reference draws `(random::<f32>() * 9.0) as i32 - 4`, :151-152). */
void FN(nrs_oracle_augment_draw)(uint64_t seed, uint64_t offset, uint64_t index, int max_shift, int* flip, int* dx, int* dy) {
  const uint64_t at = offset + index;
  const uint32_t ctr[4] = {(uint32_t)at, (uint32_t)(at >> 32), 0u, 0u};
  const uint32_t key[2] = {(uint32_t)seed, (uint32_t)(seed >> 32)};
  uint32_t w[4];
  FN(nrs_oracle_philox4x32_10)(ctr, key, w);
  *flip = (int)(w[0] >> 31);
  const float u1 = (float)(w[1] >> 8) * (1.0f / 16777216.0f), u2 = (float)(w[2] >> 8) * (1.0f / 16777216.0f);
  *dx = (int)(u1 * (float)(2 * max_shift + 1)) - max_shift;
  *dy = (int)(u2 * (float)(2 * max_shift + 1)) - max_shift;
}

/* ------------------------------------------------------------------------------------------------
 * Compiled once (the f32 pass): thread control for the timed baselines, and the reference's FAST
 * CPU kernels — forward only, as in the reference — restated for the "upper bound of the CPU path"
 * baseline.  They are not used as the parity checker (the naive loops above are).
 * ---------------------------------------------------------------------------------------------- */
#ifdef NRS_ONCE
#ifdef _OPENMP
#include <omp.h>
#endif
#if defined(__AVX2__) && defined(__FMA__)
#include <immintrin.h>
#endif

/* Number of host cores OpenMP sees, and the thread count the parallel loops will use.  Launchers
 * (torchrun) export OMP_NUM_THREADS=1; the timed baselines override that with every core. */
int nrs_oracle_host_cores(void) {
#ifdef _OPENMP
  return omp_get_num_procs();
#else
  return 1;
#endif
}
int nrs_oracle_get_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}
void nrs_oracle_set_threads(int n) {
#ifdef _OPENMP
  if (n > 0) omp_set_num_threads(n);
#else
  (void)n;
#endif
}

/* dot_simd (src/ops/simd.rs:7-37): eight FMA lanes over the 8-element chunks, the lanes summed in
 * index order, then the scalar tail. */
static float nrs_dot_simd(const float* a, const float* b, size_t n) {
  const size_t chunks = n / 8;
#if defined(__AVX2__) && defined(__FMA__)
  __m256 acc = _mm256_setzero_ps();
  for (size_t i = 0; i < chunks; ++i)
    acc = _mm256_fmadd_ps(_mm256_loadu_ps(a + i * 8), _mm256_loadu_ps(b + i * 8), acc);
  float tmp[8];
  _mm256_storeu_ps(tmp, acc);
#else
  float tmp[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  for (size_t i = 0; i < chunks; ++i)
    for (int l = 0; l < 8; ++l) tmp[l] = fmaf(a[i * 8 + l], b[i * 8 + l], tmp[l]);
#endif
  float sum = tmp[0] + tmp[1] + tmp[2] + tmp[3] + tmp[4] + tmp[5] + tmp[6] + tmp[7];
  for (size_t i = chunks * 8; i < n; ++i) sum += a[i] * b[i];
  return sum;
}

/* matmul_simd (src/ops/simd.rs:42-77): B transposed once, every output row a parallel unit
 * (par_chunks_mut(n)), each element one dot_simd. */
void nrs_oracle_matmul_simd(const float* a, const float* b, float* c, int m, int k, int n) {
  float* bt = (float*)malloc(sizeof(float) * (size_t)n * k);
  for (int row = 0; row < k; ++row)
    for (int col = 0; col < n; ++col) bt[(size_t)col * k + row] = b[(size_t)row * n + col];
#pragma omp parallel for schedule(static)
  for (int i = 0; i < m; ++i)
    for (int j = 0; j < n; ++j) c[(size_t)i * n + j] = nrs_dot_simd(a + (size_t)i * k, bt + (size_t)j * k, (size_t)k);
  free(bt);
}

/* conv2d_im2col (src/ops/im2col.rs:8-98): unroll every sample's patches into a [ci*kh*kw, oh*ow]
 * column matrix (serial, as in the reference), then per sample weight[co, ci*kh*kw] x columns
 * through `matmul` (matmul_simd on x86-64), the bias added in the copy-out. */
void nrs_oracle_conv2d_im2col(const float* x, const float* w, const float* bias, float* y, int n, int ci, int h, int wd,
                              int co, int kh, int kw, int stride, int pad) {
  const int oh = (h + 2 * pad - kh) / stride + 1, ow = (wd + 2 * pad - kw) / stride + 1;
  const size_t col_h = (size_t)ci * kh * kw, col_w = (size_t)oh * ow;
  float* col = (float*)calloc((size_t)n * col_h * col_w, sizeof(float));
  for (int ni = 0; ni < n; ++ni)
    for (int ic = 0; ic < ci; ++ic)
      for (int i = 0; i < kh; ++i)
        for (int j = 0; j < kw; ++j) {
          const size_t row = ((size_t)ic * kh + i) * kw + j;
          for (int oy = 0; oy < oh; ++oy)
            for (int ox = 0; ox < ow; ++ox) {
              const int iy = oy * stride + i, ix = ox * stride + j;
              float v = 0.0f;
              if (!(iy < pad || ix < pad || iy >= pad + h || ix >= pad + wd))
                v = x[(((size_t)ni * ci + ic) * h + (iy - pad)) * wd + (ix - pad)];
              col[((size_t)ni * col_h + row) * col_w + ((size_t)oy * ow + ox)] = v;
            }
        }
  float* res = (float*)malloc(sizeof(float) * (size_t)co * col_w);
  for (int ni = 0; ni < n; ++ni) {
    nrs_oracle_matmul_simd(w, col + (size_t)ni * col_h * col_w, res, co, (int)col_h, (int)col_w);
    for (int oc = 0; oc < co; ++oc)
      for (size_t p = 0; p < col_w; ++p) y[((size_t)ni * co + oc) * col_w + p] = res[(size_t)oc * col_w + p] + bias[oc];
  }
  free(res);
  free(col);
}
#endif /* NRS_ONCE */
