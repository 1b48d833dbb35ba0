// Input pipeline kernels: the augmentation and label expansion that the reference's training examples do on
// the host before every upload (examples/cifar_cuda.rs:146-169 `augment`, and the one-hot target rows the
// loaders build, src/data/cifar.rs), done on the device after the raw batch has landed so that the host only
// hands over bytes.
//
// Random draws come from the context's counter-based stream (dropout.cu): image i of a call uses the
// Philox-4x32-10 block at counter (offset + i); flip = top bit of word 0, dx = floor(u(word 1) * (2s+1)) - s,
// dy likewise from word 2, with u(w) = (w >> 8) * 2^-24 — the reference's `(random::<f32>() * 9.0) as i32 - 4`
// for s = 4.  A call consumes n blocks.
#include "nrs_internal.h"
#include "philox.cuh"

namespace {

constexpr int kThreads = 256;

__device__ __forceinline__ int draw_shift(uint32_t word, int max_shift) {
  return (int)(nrs_rng::uniform01(word) * (float)(2 * max_shift + 1)) - max_shift;
}

// One block per (image, channel) plane; the plane's draw is recomputed by every block of the image (ten
// rounds of two multiplies: cheaper than a round trip through memory).
__global__ void __launch_bounds__(kThreads)
augment_kernel(const float* __restrict__ x, float* __restrict__ y, int c, int h, int w, int max_shift, int do_flip,
               uint64_t seed, uint64_t offset) {
  NRS_PDL_PROLOGUE();
  const int img = blockIdx.x / c;
  uint32_t ctr[4];
  nrs_rng::block(seed, offset + (uint64_t)img, ctr);
  const bool flip = do_flip && (ctr[0] >> 31);
  const int dx = draw_shift(ctr[1], max_shift), dy = draw_shift(ctr[2], max_shift);
  const float* src = x + (size_t)blockIdx.x * h * w;
  float* dst = y + (size_t)blockIdx.x * h * w;
  for (int i = threadIdx.x; i < h * w; i += kThreads) {
    const int yy = i / w, xx = i - yy * w;
    const int sx = xx - dx, sy = yy - dy;
    float v = 0.0f;
    if (sx >= 0 && sx < w && sy >= 0 && sy < h) v = src[sy * w + (flip ? w - 1 - sx : sx)];
    dst[i] = v;
  }
}

__global__ void __launch_bounds__(kThreads)
onehot_kernel(const int32_t* __restrict__ labels, float* __restrict__ out, int batch, int classes) {
  NRS_PDL_PROLOGUE();
  const size_t total = (size_t)batch * classes;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const int b = (int)(i / classes), k = (int)(i - (size_t)b * classes);
    out[i] = labels[b] == k ? 1.0f : 0.0f;
  }
}

}  // namespace

int nrs_augment_flip_shift(nrs_ctx* ctx, const float* x, float* y, int n, int c, int h, int w, int max_shift, int flip) {
  NRS_REQUIRE_CTX(ctx);
  NRS_REQUIRE(ctx, n >= 0 && c >= 1 && h >= 1 && w >= 1 && (size_t)n * c < 0x7fffffffu && (size_t)h * w < 0x7fffffffu,
              NRS_ERR_SHAPE, "nrs_augment_flip_shift: bad shape [%d,%d,%d,%d]", n, c, h, w);
  NRS_REQUIRE(ctx, max_shift >= 0 && max_shift < 4096, NRS_ERR_ARG, "nrs_augment_flip_shift: bad shift range %d", max_shift);
  if (n == 0) return NRS_OK;
  NRS_REQUIRE(ctx, x && y && x != y, NRS_ERR_ARG, "nrs_augment_flip_shift: null tensor, or input and output are the same");
  // one block of the stream per image; a data-parallel shard takes the blocks its images have in the global batch
  uint64_t first = ctx->rng_offset, advance = (uint64_t)n;
  if (ctx->shard_global > 0 && n == ctx->shard_local) {
    first += (uint64_t)ctx->shard_begin;
    advance = (uint64_t)ctx->shard_global;
  }
  NRS_PDL_LAUNCH(augment_kernel, (unsigned)(n * c), kThreads, 0, ctx->stream, x, y, c, h, w, max_shift, flip, ctx->rng_seed,
                 first);
  NRS_LAUNCHED(ctx);
  ctx->rng_offset += advance;
  return NRS_OK;
}

int nrs_onehot(nrs_ctx* ctx, const int32_t* labels, float* out, int batch, int classes) {
  NRS_REQUIRE_CTX(ctx);
  NRS_REQUIRE(ctx, batch >= 0 && classes >= 1, NRS_ERR_SHAPE, "nrs_onehot: bad shape [%d,%d]", batch, classes);
  if (batch == 0) return NRS_OK;
  NRS_REQUIRE(ctx, labels && out, NRS_ERR_ARG, "nrs_onehot: null tensor");
  const size_t total = (size_t)batch * classes;
  size_t blocks = (total + kThreads - 1) / kThreads;
  const size_t cap = (size_t)ctx->sm_count * 8;
  if (blocks > cap) blocks = cap;
  // A label outside [0, classes) yields an all-zero row, as a one-hot built by comparison does; the row is
  // not an error of the kernel (the reference's loaders index `row[label] = 1.0` and would panic instead).
  NRS_PDL_LAUNCH(onehot_kernel, (unsigned)blocks, kThreads, 0, ctx->stream, labels, out, batch, classes);
  NRS_LAUNCHED(ctx);
  return NRS_OK;
}
