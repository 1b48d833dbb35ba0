// Batched staging of a model's weights for the tensor-core kernels.
//
// Every contraction reads its weight operand as K-major TF32 planes (a high plane rounded to nearest
// and, for 3xTF32, an f32 residual plane), re-laid out per use: convolution forward and data gradient
// want two different tap-major layouts, x@W wants W transposed, dz@W^T wants W as stored.  Staged per
// call that is one small launch per layer and pass; a training loop knows all its weights in advance,
// so they are staged here in ONE launch per step from a job table resident on the device, and the
// contraction entry points pick the planes up by (weight pointer, form).  The reference has no
// counterpart (its GEMMs read f32 weights directly, src/cuda/graph/matmul.rs:44-261).
#include "tc_mainloop.cuh"

namespace {

struct WeightJob {
  const float* src;
  float* hi;
  float* lo;
  int form;              // NrsWeightForm
  int rows, K, ldk;      // linear forms: destination [rows][ldk], zeros beyond K
  int co, ci, taps;      // convolution forms
  unsigned first_block;  // this job's first block in the launch
};

__device__ __forceinline__ void put(float* hi, float* lo, size_t i, float v) {
  const float h = tc::tf32_rn(v);
  hi[i] = h;
  if (lo) lo[i] = v - h;
}

__global__ void __launch_bounds__(256)
weight_stage_batch_kernel(const WeightJob* __restrict__ jobs, int n_jobs, unsigned block_offset) {
  NRS_PDL_PROLOGUE();
  __shared__ float tile[32][33];
  // the job this block belongs to: the last one whose first_block <= its index in the full launch
  const unsigned bid = blockIdx.x + block_offset;
  int lo_j = 0, hi_j = n_jobs - 1;
  while (lo_j < hi_j) {
    const int mid = (lo_j + hi_j + 1) >> 1;
    if (jobs[mid].first_block <= bid) lo_j = mid; else hi_j = mid - 1;
  }
  const WeightJob j = jobs[lo_j];
  const unsigned blk = bid - j.first_block;
  if (j.form == NRS_WF_LINEAR_ROWS) {
    // dst[r][k] = src[r*K + k], four consecutive k per thread
    const int q = j.ldk / 4;
    const size_t i = (size_t)blk * 256 + threadIdx.x;
    if (i >= (size_t)j.rows * q) return;
    const size_t r = i / q;
    const int k = (int)(i - r * q) * 4;
#pragma unroll
    for (int e = 0; e < 4; ++e) put(j.hi, j.lo, r * j.ldk + k + e, k + e < j.K ? j.src[r * j.K + k + e] : 0.0f);
  } else if (j.form == NRS_WF_LINEAR_T) {
    // dst[r][k] = src[k*rows + r] through a 32x32 tile
    const int tiles_r = (j.rows + 31) / 32;
    const int r0 = (int)(blk % tiles_r) * 32, k0 = (int)(blk / tiles_r) * 32;
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
    for (int i = ty; i < 32; i += 8) {
      const int k = k0 + i, r = r0 + tx;
      tile[i][tx] = (k < j.K && r < j.rows) ? j.src[(size_t)k * j.rows + r] : 0.0f;
    }
    __syncthreads();
    for (int i = ty; i < 32; i += 8) {
      const int r = r0 + i;
      if (r < j.rows) put(j.hi, j.lo, (size_t)r * j.ldk + k0 + tx, tile[tx][i]);
    }
  } else {
    // convolution weights w[co][ci][tap]: forward out[co][tap*ci_n + ci], data gradient out[ci][tap*co_n + co]
    const size_t total = (size_t)j.co * j.ci * j.taps;
    const size_t idx = (size_t)blk * 256 + threadIdx.x;
    if (idx >= total) return;
    int co, ci, t;
    if (j.form == NRS_WF_CONV_FWD) {
      ci = (int)(idx % j.ci);
      t = (int)((idx / j.ci) % j.taps);
      co = (int)(idx / ((size_t)j.ci * j.taps));
    } else {
      co = (int)(idx % j.co);
      t = (int)((idx / j.co) % j.taps);
      ci = (int)(idx / ((size_t)j.co * j.taps));
    }
    put(j.hi, j.lo, idx, j.src[((size_t)co * j.ci + ci) * j.taps + t]);
  }
}

size_t plane_floats(const NrsWeightDesc& d) {
  if (d.form == NRS_WF_LINEAR_ROWS || d.form == NRS_WF_LINEAR_T) return (size_t)d.rows * ((d.K + 31) / 32 * 32);
  return (size_t)d.co * d.ci * d.taps;
}

}  // namespace

void nrs_weight_set_clear(nrs_ctx* ctx) {
  NrsWeightSet& ws = ctx->weight_set;
  if (ws.storage || ws.jobs_dev) cudaStreamSynchronize(ctx->stream);
  if (ws.storage) cudaFree(ws.storage);
  if (ws.jobs_dev) cudaFree(ws.jobs_dev);
  ws = NrsWeightSet();
}

int nrs_weight_set_build(nrs_ctx* ctx, const NrsWeightDesc* descs, int count) {
  nrs_weight_set_clear(ctx);
  if (count <= 0 || ctx->math_mode == NRS_MATH_FP32) return NRS_OK;
  NrsWeightSet& ws = ctx->weight_set;
  const bool split = ctx->math_mode == NRS_MATH_3XTF32;
  size_t total = 0;
  for (int i = 0; i < count; ++i) total += (plane_floats(descs[i]) + 63) / 64 * 64 * (split ? 2 : 1);
  cudaError_t e = cudaMalloc(&ws.storage, total * sizeof(float));
  if (e != cudaSuccess) {
    (void)cudaGetLastError();
    ws.storage = nullptr;
    return nrs_fail(ctx, NRS_ERR_ALLOC, "weight planes: cudaMalloc(%zu) failed: %s", total * sizeof(float), cudaGetErrorString(e));
  }
  std::vector<WeightJob> jobs;
  float* cursor = (float*)ws.storage;
  unsigned block = 0;
  for (int i = 0; i < count; ++i) {
    const NrsWeightDesc& d = descs[i];
    const size_t n = (plane_floats(d) + 63) / 64 * 64;
    WeightJob j{};
    j.src = d.w;
    j.hi = cursor;
    cursor += n;
    j.lo = split ? cursor : nullptr;
    if (split) cursor += n;
    j.form = d.form;
    j.rows = d.rows; j.K = d.K; j.ldk = (d.K + 31) / 32 * 32;
    j.co = d.co; j.ci = d.ci; j.taps = d.taps;
    j.first_block = block;
    if (d.form == NRS_WF_LINEAR_ROWS) block += (unsigned)(((size_t)d.rows * (j.ldk / 4) + 255) / 256);
    else if (d.form == NRS_WF_LINEAR_T) block += (unsigned)(((d.rows + 31) / 32) * (j.ldk / 32));
    else block += (unsigned)(((size_t)d.co * d.ci * d.taps + 255) / 256);
    jobs.push_back(j);
    ws.job_src.push_back(d.w);
    ws.job_first.push_back(j.first_block);
    ws.planes[std::make_pair((const void*)d.w, d.form)] = NrsWeightPlanes{j.hi, j.lo, d.rows, d.K, d.co, d.ci, d.taps};
  }
  e = cudaMalloc(&ws.jobs_dev, jobs.size() * sizeof(WeightJob));
  if (e == cudaSuccess) e = cudaMemcpyAsync(ws.jobs_dev, jobs.data(), jobs.size() * sizeof(WeightJob), cudaMemcpyHostToDevice, ctx->stream);
  if (e == cudaSuccess) e = cudaStreamSynchronize(ctx->stream);   // `jobs` is a local
  if (e != cudaSuccess) {
    (void)cudaGetLastError();
    nrs_weight_set_clear(ctx);
    return nrs_fail(ctx, NRS_ERR_ALLOC, "weight planes: job table upload failed: %s", cudaGetErrorString(e));
  }
  ws.n_jobs = (int)jobs.size();
  ws.blocks = block;
  ws.job_first.push_back(block);
  ws.split = split;
  ws.fresh = false;
  return NRS_OK;
}

int nrs_weight_set_refresh(nrs_ctx* ctx) {
  NrsWeightSet& ws = ctx->weight_set;
  if (ws.n_jobs == 0) return NRS_OK;
  NRS_PDL_LAUNCH(weight_stage_batch_kernel, ws.blocks, 256, 0, ctx->stream, (const WeightJob*)ws.jobs_dev, ws.n_jobs, 0u);
  NRS_LAUNCHED(ctx);
  ws.fresh = true;
  ws.refreshed_jobs = 0;
  return NRS_OK;
}

int nrs_weight_set_refresh_range(nrs_ctx* ctx, const float* lo, const float* hi) {
  NrsWeightSet& ws = ctx->weight_set;
  // one launch per run of consecutive jobs whose weight lies in the range (jobs follow the layer order, so
  // a bucket of adjacent parameters is one run)
  int j = 0;
  while (j < ws.n_jobs) {
    if (ws.job_src[j] < lo || ws.job_src[j] >= hi) { ++j; continue; }
    int e = j;
    while (e < ws.n_jobs && ws.job_src[e] >= lo && ws.job_src[e] < hi) ++e;
    const unsigned first = ws.job_first[j], count = ws.job_first[e] - first;
    if (count > 0) {
      NRS_PDL_LAUNCH(weight_stage_batch_kernel, count, 256, 0, ctx->stream, (const WeightJob*)ws.jobs_dev, ws.n_jobs, first);
      NRS_LAUNCHED(ctx);
    }
    ws.refreshed_jobs += e - j;
    j = e;
  }
  return NRS_OK;
}
