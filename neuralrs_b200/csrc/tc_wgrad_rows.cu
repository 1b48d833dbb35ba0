// Weight gradient of 3x3 / stride 1 / pad 1 convolutions on tcgen05 (TF32 / 3xTF32),
// streaming image rows so that each row of x is fetched once for all three vertical taps.
//
//   dw[co,ci,i,j] (+)= sum over (n,y,x) of dy[n,co,y,x] * x[n,ci,y+i-1,x+j-1]
//
// The general kernel (tc_wgrad.cu) loads one shifted x box per tap, so x crosses
// L2 -> shared memory nine times and dy once per tap group; at 2.5 KB per pixel and
// CTA it is bound by L2 bandwidth, not by the tensor pipe.  Here a CTA owns
//   128 output channels x one horizontal tap j x a chunk of <= 128 input channels
// and walks a range of image rows.  Step t brings in ONE new row of x (shifted by j
// through the TMA box origin, zero fill = padding) and one row of dy; the dy row
// y meets the x rows y-1, y, y+1, which are the last three rows brought in.  The
// three vertical taps are separate column ranges of the TMEM accumulator
// (128 x 3*chunk f32).  Per pixel the CTA loads 128 + chunk values instead of
// 128 + 3*chunk, and vertical taps that fall off the image are skipped instead
// of multiplied by zeros.  With 64 output channels or fewer the 128 accumulator
// rows would be half empty, so a CTA takes TWO horizontal taps: the upper rows get a
// second copy of the dy row fetched one pixel to the right, which turns the same x
// operand into the neighbouring tap (sum_p dy[p+1] x[p] = sum_p dy[p] x[p-1]); two
// kinds of CTA then cover the three taps instead of three.
//
// Shared memory: a ring of dy rows and rings of x rows (one per plane), each with its
// own full/empty mbarriers.  The dy row of step t is consumed at step t and goes back
// to the producer when that step's UMMAs have retired (tcgen05.commit); the x row of
// step t is read at steps t, t+1, t+2 and goes back after step t+2.  Operands are MN-major in the
// 128-byte / 32-byte-atom swizzle exactly as in tc_wgrad.cu: [32-channel block]
// [pixel][128 B], K-step = 8 pixels = 1024 B, SBO = 512 B, LBO = block stride.
// Vertical taps whose x rows sit in consecutive slots are issued as one UMMA of
// up to 256 columns (their blocks are then LBO apart throughout).
//
// Rows are split across CTAs (no accumulation chain longer than tc::kMaxChainK
// pixels in 3xTF32 mode); partial tiles are summed in a fixed order by a second
// kernel, which also scatters into [co][ci][3][3].
//
// Replaces conv2d_im2col + conv2d_out2mm + matmul_nt_splitk (src/cuda/nn/conv.rs:
// 298-320) for the shapes it covers; everything else takes tc_wgrad.cu.
#include "tc_mainloop.cuh"

namespace {

constexpr int kRowThreads = 192;
constexpr int kTaps = 3;          // vertical taps per CTA

struct RowParams {
  int W, H, n_img;                // image geometry (dy and x have the same: pad 1, 3x3)
  int co, ci;
  int chunk, n_chunks;            // input channels per CTA (multiple of 32, <= 128) and how many chunks
  int a_blocks;                   // 32-channel blocks of dy one box brings (min(4, co/32))
  int pack;                       // co <= 64: accumulator rows [0,h) and [h,2h), h = 32*a_blocks, hold two
                                  // horizontal taps (the second from a copy of the dy row shifted one pixel)
  int jtypes;                     // CTA kinds along the horizontal taps: 3, or 2 when packed
  int m_blocks;                   // ceil(co / 128)
  int rows_total;                 // n_img * H
  int rows_per_split;
  int SA, SX;                     // ring depths: dy rows, x rows
  int max_run;                    // vertical taps one UMMA may cover (256 / chunk, at most 3)
  float* partial;                 // [split][cta][128][3*chunk]
  int independent;                // reads nothing the kernel launched just before it wrote (NRS_PDL_PROLOGUE)
};

// Is vertical tap i (x row = y + i - 1) inside the image for some row of [r0, r1)?
__device__ __forceinline__ bool tap_ever_valid(int i, int r0, int r1, int H) {
  if (i == 1) return true;
  for (int r = r0; r < r1; ++r) {
    const int y = r % H + i - 1;
    if (y >= 0 && y < H) return true;
  }
  return false;
}

// All UMMAs of one run of vertical taps over one image row (KS K-steps of 8 pixels).  The
// descriptors differ from step to step only in their 14-bit start-address field, so they are
// built once (`dc`: every other field) and advanced by adding (bytes >> 4).
template <int NPLANES, int KS>
__device__ __forceinline__ void issue_row(uint32_t d, uint64_t dc, uint32_t a_hi16, uint32_t a_lo16, uint32_t b_hi16,
                                          uint32_t b_lo16, uint32_t idesc, uint32_t acc_first) {
#pragma unroll
  for (int k = 0; k < KS; ++k) {
    const uint32_t ko = (uint32_t)k * 64u;   // 1024 B per K-step
    const uint32_t acc0 = k > 0 ? 1u : acc_first;
    if (NPLANES == 2) {
      tc::umma_tf32(d, dc + a_lo16 + ko, dc + b_hi16 + ko, idesc, acc0);
      tc::umma_tf32(d, dc + a_hi16 + ko, dc + b_lo16 + ko, idesc, 1);
      tc::umma_tf32(d, dc + a_hi16 + ko, dc + b_hi16 + ko, idesc, 1);
    } else {
      tc::umma_tf32(d, dc + a_hi16 + ko, dc + b_hi16 + ko, idesc, acc0);
    }
  }
}

template <int NPLANES, int KS>
__global__ void __launch_bounds__(kRowThreads, 1)
tc_wgrad_rows_kernel(const __grid_constant__ CUtensorMap tm_dy_hi, const __grid_constant__ CUtensorMap tm_dy_lo,
                     const __grid_constant__ CUtensorMap tm_x_hi, const __grid_constant__ CUtensorMap tm_x_lo,
                     const RowParams p, int* __restrict__ err_flag) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  constexpr uint32_t blk = (uint32_t)KS * 8u * 128u;         // one 32-channel block of one row (W = 8*KS pixels)
  const uint32_t a_box = (uint32_t)p.a_blocks * blk;         // one TMA box of dy
  const uint32_t a_plane = (p.pack ? 2u : 1u) * a_box;       // dy row, one plane (packed: plain + shifted copy)
  const uint32_t a_slot = NPLANES * a_plane;
  const uint32_t x_slot = (uint32_t)(p.chunk / 32) * blk;    // x row, one plane
  const uint32_t x_ring = (uint32_t)p.SX * x_slot;
  uint8_t* a_base = smem;                                    // [slot][plane][block][pixel][128 B]
  uint8_t* x_base = smem + (size_t)p.SA * a_slot;            // [plane][slot][block][pixel][128 B]
  // The UMMA reads 4 blocks of dy whatever a_blocks is: keep that inside the allocation.
  uint64_t* full_a = reinterpret_cast<uint64_t*>(x_base + (size_t)NPLANES * x_ring + 4 * blk);
  uint64_t* empty_a = full_a + p.SA;
  uint64_t* full_x = empty_a + p.SA;
  uint64_t* empty_x = full_x + p.SX;
  uint64_t* accum_bar = empty_x + p.SX;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(accum_bar + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // blockIdx.x = (m block, horizontal tap kind, channel chunk).  Unpacked: kind = tap j, x shifted by
  // j - 1.  Packed: kind 0 shifts x by 0 and holds taps j = 1 (plain dy rows) and j = 0 (dy shifted one
  // pixel: sum_p dy[p+1] x[p] = sum_p dy[p] x[p-1]); kind 1 shifts x by +1 and holds j = 2 alone.
  const int cc = blockIdx.x % p.n_chunks;
  const int jk = (blockIdx.x / p.n_chunks) % p.jtypes;
  const int mb = blockIdx.x / (p.n_chunks * p.jtypes);
  const int x_shift = p.pack ? jk : jk - 1;
  const bool two_taps = p.pack && jk == 0;
  const int split = blockIdx.y;
  const int r0 = split * p.rows_per_split;
  const int r1 = min(p.rows_total, r0 + p.rows_per_split);
  const int nsteps = (r1 - r0) + 2;                          // two leading steps bring x rows only
  const uint32_t tmem_cols = kTaps * p.chunk <= 128 ? 128u : (kTaps * p.chunk <= 256 ? 256u : 512u);

  if (warp == 0 && lane == 0) {
    tc::prefetch_tmap(&tm_dy_hi);
    tc::prefetch_tmap(&tm_x_hi);
    if (NPLANES == 2) { tc::prefetch_tmap(&tm_dy_lo); tc::prefetch_tmap(&tm_x_lo); }
    for (int s = 0; s < p.SA; ++s) { tc::mbar_init(&full_a[s], 1); tc::mbar_init(&empty_a[s], 1); }
    for (int s = 0; s < p.SX; ++s) { tc::mbar_init(&full_x[s], 1); tc::mbar_init(&empty_x[s], 1); }
    tc::mbar_init(accum_bar, 1);
    tc::fence_barrier_init();
  }
  if (warp == 1) {
    tc::tmem_alloc(tmem_slot, tmem_cols);
    tc::tmem_relinquish();
  }
  tc::tc_fence_before_sync();
  __syncthreads();
  tc::tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  if (!p.independent) NRS_PDL_WAIT();   // set-up above may overlap the previous kernel's tail; its results are needed from here
  NRS_PDL_TRIGGER();

  if (warp == 0) {
    if (lane == 0) {
      // ---------------- TMA producer.  Step t: x row r0-1+t (if it exists) and dy row r0+t-2 (t >= 2).
      int sx = 0, sa = 0;
      uint32_t phx = 0, pha = 0;
      int xr = r0 - 1, xy = 0, xn = 0;          // x row, and its (row in image, image)
      if (xr >= 0) { xn = xr / p.H; xy = xr - xn * p.H; } else { xy = -1; }
      int dn = r0 / p.H, dyy = r0 - dn * p.H;   // dy row of step 2
      bool ok = true;
      int t = 0;
      for (; t < nsteps; ++t) {
        if (!tc::mbar_wait(&empty_x[sx], phx ^ 1u)) { atomicExch(err_flag, tc::kErrProducerWait); ok = false; break; }
        const bool has_x = xr >= 0 && xr < p.rows_total;
        if (has_x) {
          tc::mbar_expect_tx(&full_x[sx], NPLANES * x_slot);
          tc::tma_load_5d(x_base + (size_t)sx * x_slot, &tm_x_hi, &full_x[sx], 0, x_shift, xy, xn, cc * (p.chunk / 32));
          if (NPLANES == 2)
            tc::tma_load_5d(x_base + x_ring + (size_t)sx * x_slot, &tm_x_lo, &full_x[sx], 0, x_shift, xy, xn, cc * (p.chunk / 32));
        } else {
          tc::mbar_arrive(&full_x[sx]);
        }
        if (t >= 2) {
          if (!tc::mbar_wait(&empty_a[sa], pha ^ 1u)) { atomicExch(err_flag, tc::kErrProducerWait); ok = false; ++t; break; }
          tc::mbar_expect_tx(&full_a[sa], NPLANES * (two_taps ? 2u : 1u) * a_box);
          uint8_t* a_dst = a_base + (size_t)sa * a_slot;
          tc::tma_load_5d(a_dst, &tm_dy_hi, &full_a[sa], 0, 0, dyy, dn, mb * 4);
          if (two_taps) tc::tma_load_5d(a_dst + a_box, &tm_dy_hi, &full_a[sa], 0, 1, dyy, dn, mb * 4);
          if (NPLANES == 2) {
            tc::tma_load_5d(a_dst + a_plane, &tm_dy_lo, &full_a[sa], 0, 0, dyy, dn, mb * 4);
            if (two_taps) tc::tma_load_5d(a_dst + a_plane + a_box, &tm_dy_lo, &full_a[sa], 0, 1, dyy, dn, mb * 4);
          }
          if (++sa == p.SA) { sa = 0; pha ^= 1u; }
          if (++dyy == p.H) { dyy = 0; ++dn; }
        }
        if (++sx == p.SX) { sx = 0; phx ^= 1u; }
        ++xr;
        if (++xy == p.H) { xy = 0; ++xn; }
      }
      if (!ok) {
        // Loads already issued still land in this CTA's shared memory: wait for them (bounded)
        // before the CTA may retire.  Walk the last ring's worth of steps.
        for (int u = (t > p.SX ? t - p.SX : 0); u < t; ++u)
          if (!tc::mbar_wait(&full_x[u % p.SX], (uint32_t)(u / p.SX) & 1u)) { atomicExch(err_flag, tc::kErrDrainWait); break; }
        for (int u = (t - 2 > p.SA ? t - 2 - p.SA : 0); u < t - 2; ++u)
          if (!tc::mbar_wait(&full_a[u % p.SA], (uint32_t)(u / p.SA) & 1u)) { atomicExch(err_flag, tc::kErrDrainWait); break; }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      // ---------------- UMMA issuer
      bool ok = true;
      uint32_t started = 0;   // bit i: vertical tap i's accumulator columns hold a sum already
      const uint64_t dc = tc::make_smem_desc_sw128_32b(0, blk, 512);
      const uint32_t a_base16 = tc::smem_u32(a_base) >> 4, x_base16 = tc::smem_u32(x_base) >> 4;
      const uint32_t a_slot16 = a_slot >> 4, a_plane16 = a_plane >> 4, x_slot16 = x_slot >> 4, x_ring16 = x_ring >> 4;
      // instruction descriptor of a run of `len` taps: N = len * chunk sits in bits [17,23) as N >> 3
      const uint32_t idesc_n0 = tc::make_idesc_tf32(128, 0, true, true);
      const uint32_t idesc_per_tap = (uint32_t)(p.chunk >> 3) << 17;
      int sx = 0, sa = 0;
      uint32_t phx = 0, pha = 0;
      int y = r0 % p.H;
      for (int t = 0; t < nsteps; ++t) {
        if (!tc::mbar_wait(&full_x[sx], phx)) { atomicExch(err_flag, tc::kErrMmaWait); ok = false; break; }
        if (t >= 2) {
          if (!tc::mbar_wait(&full_a[sa], pha)) { atomicExch(err_flag, tc::kErrMmaWait); ok = false; break; }
          const uint32_t a_hi16 = a_base16 + (uint32_t)sa * a_slot16;
          const uint32_t a_lo16 = a_hi16 + a_plane16;
          int sx0 = sx - 2;                     // slot of the x row brought in at step t-2
          if (sx0 < 0) sx0 += p.SX;
          // vertical tap i reads the x row brought in at step t-2+i
          int i = y == 0 ? 1 : 0;
          const int i_end = y == p.H - 1 ? 2 : 3;
          while (i < i_end) {
            int s0 = sx0 + i;
            if (s0 >= p.SX) s0 -= p.SX;
            int len = 1;
            while (len < p.max_run && i + len < i_end && s0 + len < p.SX &&
                   ((started >> (i + len)) & 1u) == ((started >> i) & 1u))
              ++len;
            const uint32_t b_hi16 = x_base16 + (uint32_t)s0 * x_slot16;
            issue_row<NPLANES, KS>(tmem_base + (uint32_t)(i * p.chunk), dc, a_hi16, a_lo16, b_hi16, b_hi16 + x_ring16,
                                   idesc_n0 + (uint32_t)len * idesc_per_tap, (started >> i) & 1u);
            started |= ((1u << len) - 1u) << i;
            i += len;
          }
          tc::umma_commit(&empty_a[sa]);    // this dy row is done with
          tc::umma_commit(&empty_x[sx0]);   // and so is the x row of step t-2
          if (++sa == p.SA) { sa = 0; pha ^= 1u; }
          if (++y == p.H) y = 0;
        }
        if (++sx == p.SX) { sx = 0; phx ^= 1u; }
      }
      if (ok) tc::umma_commit(accum_bar);
    }
  } else {
    // ---------------- epilogue: raw partial tile to the workspace (zeros for taps that never ran)
    const int q = warp & 3;
    const bool ok = tc::mbar_wait(accum_bar, 0);
    if (!ok && lane == 0) atomicExch(err_flag, tc::kErrEpilogueWait);
    if (ok) {
      tc::tc_fence_after_sync();
      const int row = q * 32 + lane;
      const int cols = kTaps * p.chunk;
      float* dst = p.partial + (((size_t)split * gridDim.x + blockIdx.x) * 128 + row) * cols;
      // packed: rows [0,h) are tap j = 1 or 2, rows [h,2h) tap j = 0 (kind 0 only)
      const int half = 32 * p.a_blocks;
      const bool row_live = p.pack ? (row < half || (two_taps && row < 2 * half)) : (mb * 128 + row < p.co);
      uint32_t valid = 0;
      for (int i = 0; i < kTaps; ++i) valid |= tap_ever_valid(i, r0, r1, p.H) ? (1u << i) : 0u;
#pragma unroll 1
      for (int c = 0; c < cols / 32; ++c) {
        uint32_t r[32];
        tc::tmem_ld_32x32(tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(c * 32), r);
        tc::tmem_ld_wait();
        const bool live = (valid >> ((c * 32) / p.chunk)) & 1u;
        if (row_live) {
#pragma unroll
          for (int e = 0; e < 32; e += 4)
            *reinterpret_cast<float4*>(dst + c * 32 + e) =
                live ? make_float4(__uint_as_float(r[e]), __uint_as_float(r[e + 1]), __uint_as_float(r[e + 2]), __uint_as_float(r[e + 3]))
                     : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        }
      }
    }
  }

  if (p.independent) NRS_PDL_WAIT();   // nothing after this kernel may run ahead of its predecessor
  tc::tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc::tc_fence_after_sync();
    tc::tmem_dealloc(tmem_base, tmem_cols);
  }
}

// dw[co][ci][i][j] (+)= sum over splits of the partial accumulators.  A block is
// (kReduceThreads / lanes) outputs x `lanes` split lanes: lane y sums splits y, y+lanes, ... and the lanes are
// combined in lane order through shared memory: a fixed order of additions (bit-reproducible) without one
// serial load chain per output.
__global__ void __launch_bounds__(kReduceThreads)
tc_wgrad_rows_reduce_kernel(const RowParams p, int splits, int ctas, int lanes, float* __restrict__ dw, int accumulate) {
  NRS_PDL_PROLOGUE();
  __shared__ float4 lane_sum[kReduceThreads];
  const int per_block = kReduceThreads / lanes;   // output quads of this block
  const int lane = threadIdx.x / per_block, slot = threadIdx.x - lane * per_block;
  const int cq = p.ci / 4;                        // a thread owns four consecutive input channels (ci % 32 == 0)
  const size_t total = (size_t)p.co * 9 * cq;
  const size_t idx = (size_t)blockIdx.x * per_block + slot;
  const bool live = idx < total;
  // idx enumerates (co, j, i, ci/4): consecutive threads read consecutive 128-bit groups of partial columns
  const int ci = (int)(idx % cq) * 4;
  const int i = (int)((idx / cq) % 3);
  const int j = (int)((idx / ((size_t)cq * 3)) % 3);
  const int co = (int)(idx / ((size_t)cq * 9));
  int mb = co / 128, row = co - mb * 128, jk = j;
  if (p.pack) {   // tap 1 -> kind 0 rows [0,h); tap 0 -> kind 0 rows [h,2h); tap 2 -> kind 1 rows [0,h)
    mb = 0;
    jk = j == 2 ? 1 : 0;
    row = co + (j == 0 ? 32 * p.a_blocks : 0);
  }
  const int cc = ci / p.chunk, c = ci - cc * p.chunk;
  const int cta = (mb * p.jtypes + jk) * p.n_chunks + cc;
  const size_t cols = (size_t)kTaps * p.chunk;
  const size_t off = ((size_t)cta * 128 + row) * cols + (size_t)i * p.chunk + c;
  const size_t split_stride = (size_t)ctas * 128 * cols;
  float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
  if (live) {
#pragma unroll 4
    for (int z = lane; z < splits; z += lanes) {
      const float4 v = *reinterpret_cast<const float4*>(p.partial + (size_t)z * split_stride + off);
      s.x += v.x; s.y += v.y; s.z += v.z; s.w += v.w;
    }
  }
  lane_sum[threadIdx.x] = s;
  __syncthreads();
  if (lane != 0 || !live) return;
  for (int l = 1; l < lanes; ++l) {
    const float4 v = lane_sum[l * per_block + slot];
    s.x += v.x; s.y += v.y; s.z += v.z; s.w += v.w;
  }
  float* dst = dw + (((size_t)co * p.ci + ci) * 3 + i) * 3 + j;
  const float r[4] = {s.x, s.y, s.z, s.w};
#pragma unroll
  for (int k = 0; k < 4; ++k) dst[(size_t)k * 9] = accumulate ? dst[(size_t)k * 9] + r[k] : r[k];
}

template <int NPLANES, int KS>
int launch_rows(nrs_ctx* ctx, const CUtensorMap* maps, const RowParams& p, int ctas, int splits, size_t smem_bytes) {
  static NrsSmemAttr attr;
  NRS_ENSURE_SMEM(ctx, attr, (tc_wgrad_rows_kernel<NPLANES, KS>), smem_bytes);
  int* err = nullptr;
  const int st = nrs_err_flag(ctx, &err);
  if (st != NRS_OK) return st;
  dim3 grid((unsigned)ctas, (unsigned)splits);
  NRS_PDL_LAUNCH((tc_wgrad_rows_kernel<NPLANES, KS>), grid, kRowThreads, smem_bytes, ctx->stream, maps[0], maps[1], maps[2],
                 maps[3], p, err);
  NRS_LAUNCHED(ctx);
  return NRS_OK;
}

}  // namespace

// NRS_ERR_UNSUPPORTED (no error text) for anything but 3x3 / stride 1 / pad 1 with channel counts
// that are multiples of 32 and image rows of 16, 32 or 64 pixels.
int nrs_tc_conv_wgrad_rows(nrs_ctx* ctx, const float* x, const float* dy, float* dw, int n, int ci, int h, int wd, int co,
                           int kh, int kw, int stride, int pad, int accumulate) {
  if (!tc::tensor_map_encoder()) return NRS_ERR_UNSUPPORTED;
  if (kh != 3 || kw != 3 || stride != 1 || pad != 1 || ci % 32 != 0 || co % 32 != 0 || n < 1) return NRS_ERR_UNSUPPORTED;
  // Rows of 16, 32 or 64 pixels; narrower images amortise the per-row bookkeeping of the single
  // issuing thread poorly and do better on the general kernel's multi-row pixel tiles.
  if ((wd != 16 && wd != 32 && wd != 64) || h < 1 || (long)n * h > 2000000000L) return NRS_ERR_UNSUPPORTED;
  const bool split3 = ctx->math_mode == NRS_MATH_3XTF32;
  const int planes = split3 ? 2 : 1;

  RowParams p{};
  p.W = wd; p.H = h; p.n_img = n; p.co = co; p.ci = ci;
  p.chunk = ci % 128 == 0 ? 128 : (ci <= 128 ? ci : (ci % 96 == 0 ? 96 : (ci % 64 == 0 ? 64 : 32)));
  p.n_chunks = ci / p.chunk;
  p.a_blocks = co / 32 < 4 ? co / 32 : 4;
  p.pack = co <= 64 ? 1 : 0;
  p.jtypes = p.pack ? 2 : 3;
  p.m_blocks = (co + 127) / 128;
  p.rows_total = n * h;
  p.max_run = 256 / p.chunk < kTaps ? 256 / p.chunk : kTaps;

  // ring depths: a dy row lives one step, an x row three; d rows of prefetch on top of that
  const size_t blk = (size_t)wd * 128;
  const size_t a_slot = (size_t)planes * (p.pack ? 2 : 1) * p.a_blocks * blk, x_slot = (size_t)planes * (p.chunk / 32) * blk;
  const long budget = 200 * 1024;
  long d = (budget - 3 * (long)x_slot - (long)a_slot) / (long)(x_slot + a_slot);
  if (d > 8) d = 8;
  if (d < 1) return NRS_ERR_UNSUPPORTED;
  p.SA = 1 + (int)d;
  p.SX = 3 + (int)d;
  const size_t smem_bytes = p.SA * a_slot + p.SX * x_slot + 4 * blk + (size_t)(2 * (p.SA + p.SX) + 1) * 8 + 16 + 1024;
  if (smem_bytes > 227 * 1024) return NRS_ERR_UNSUPPORTED;

  // row split: fill the GPU, bound the accumulation chain in 3xTF32 mode, amortise the partial tile
  const int ctas = p.m_blocks * p.jtypes * p.n_chunks;
  const int max_rows = split3 ? tc::kMaxChainK / wd : 1 << 30;
  int min_rows = (512 + wd - 1) / wd;
  if (min_rows > max_rows) min_rows = max_rows;
  const int rps = tc::plan_units_per_cta(ctx->sm_count, ctas, p.rows_total, min_rows, max_rows, 2 + 256 / wd);
  p.rows_per_split = rps;
  const int splits = (p.rows_total + rps - 1) / rps;
  if (splits > 65535) return NRS_ERR_UNSUPPORTED;

  // workspaces: NHWC planes of dy and x (or the caller's registered planes), and the partial tiles
  const size_t dy_plane = (size_t)n * h * wd * co, x_plane = (size_t)n * h * wd * ci;
  const size_t partial_floats = (size_t)splits * ctas * 128 * kTaps * p.chunk;
  void *dy_hi = nullptr, *dy_lo = nullptr, *x_hi = nullptr, *x_lo = nullptr, *part = nullptr;
  bool may_overlap = ctx->independent_next;   // withdrawn below if this call stages an operand itself
  int st = nrs_ws_slot(ctx, NRS_WS_WGRAD_PARTIAL, partial_floats * sizeof(float), &part);
  if (st != NRS_OK) return st;
  p.partial = (float*)part;
  const size_t dy_img = (size_t)h * wd * co, x_img = (size_t)h * wd * ci;
  if (const NrsPlanes* ready = nrs_planes_find(ctx, dy, split3)) {
    dy_hi = ready->hi;
    dy_lo = ready->lo;
  } else {
    may_overlap = false;
    st = nrs_ws_slot(ctx, NRS_WS_A_HI, dy_plane * sizeof(float), &dy_hi);
    if (st == NRS_OK && split3) st = nrs_ws_slot(ctx, NRS_WS_A_LO, dy_plane * sizeof(float), &dy_lo);
    if (st == NRS_OK) st = nrs_tc_stage(ctx, dy, (float*)dy_hi, (float*)dy_lo, h * wd, co, co, n, dy_img, dy_img, true);
    if (st != NRS_OK) return st;
  }
  if (const NrsPlanes* ready = nrs_planes_find(ctx, x, split3)) {
    x_hi = ready->hi;
    x_lo = ready->lo;
  } else {
    may_overlap = false;
    st = nrs_ws_slot(ctx, NRS_WS_B_HI, x_plane * sizeof(float), &x_hi);
    if (st == NRS_OK && split3) st = nrs_ws_slot(ctx, NRS_WS_B_LO, x_plane * sizeof(float), &x_lo);
    if (st == NRS_OK) st = nrs_tc_stage(ctx, x, (float*)x_hi, (float*)x_lo, h * wd, ci, ci, n, x_img, x_img, true);
    if (st != NRS_OK) return st;
  }

  // planes viewed as [channel block][n][h][w][32 channels]; a box is one image row of some blocks
  CUtensorMap maps[4];
  const uint64_t ddim[5] = {32, (uint64_t)wd, (uint64_t)h, (uint64_t)n, (uint64_t)(co / 32)};
  const uint64_t dstr[4] = {(uint64_t)co * 4, (uint64_t)wd * co * 4, (uint64_t)h * wd * co * 4, 128};
  const uint64_t xdim[5] = {32, (uint64_t)wd, (uint64_t)h, (uint64_t)n, (uint64_t)(ci / 32)};
  const uint64_t xstr[4] = {(uint64_t)ci * 4, (uint64_t)wd * ci * 4, (uint64_t)h * wd * ci * 4, 128};
  const uint32_t dbox[5] = {32, (uint32_t)wd, 1, 1, (uint32_t)p.a_blocks};
  const uint32_t xbox[5] = {32, (uint32_t)wd, 1, 1, (uint32_t)(p.chunk / 32)};
  bool ok = tc::encode_tmap_f32(&maps[0], dy_hi, 5, ddim, dstr, dbox, true) && tc::encode_tmap_f32(&maps[2], x_hi, 5, xdim, xstr, xbox, true);
  if (split3) ok = ok && tc::encode_tmap_f32(&maps[1], dy_lo, 5, ddim, dstr, dbox, true) && tc::encode_tmap_f32(&maps[3], x_lo, 5, xdim, xstr, xbox, true);
  else { maps[1] = maps[0]; maps[3] = maps[2]; }
  NRS_REQUIRE(ctx, ok, NRS_ERR_CUDA, "tc_wgrad_rows: cuTensorMapEncodeTiled failed");
  p.independent = may_overlap ? 1 : 0;

  switch (wd / 8) {
    case 2: st = split3 ? launch_rows<2, 2>(ctx, maps, p, ctas, splits, smem_bytes) : launch_rows<1, 2>(ctx, maps, p, ctas, splits, smem_bytes); break;
    case 4: st = split3 ? launch_rows<2, 4>(ctx, maps, p, ctas, splits, smem_bytes) : launch_rows<1, 4>(ctx, maps, p, ctas, splits, smem_bytes); break;
    default: st = split3 ? launch_rows<2, 8>(ctx, maps, p, ctas, splits, smem_bytes) : launch_rows<1, 8>(ctx, maps, p, ctas, splits, smem_bytes); break;
  }
  if (st != NRS_OK) return st;
  const size_t total = (size_t)co * ci * 9;
  const int lanes = reduce_lanes(splits);
  NRS_PDL_LAUNCH(tc_wgrad_rows_reduce_kernel, nrs_blocks(total / 4, kReduceThreads / lanes), kReduceThreads, 0, ctx->stream, p, splits,
                 ctas, lanes, dw, accumulate);
  NRS_LAUNCHED(ctx);
  return NRS_OK;
}
