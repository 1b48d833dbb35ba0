// Convolution weight gradient as implicit GEMM on tcgen05 (TF32 / 3xTF32).
//
//   dw[co,ci,i,j] (+)= sum over (n,oy,ox) of dy[n,co,oy,ox] * x[n,ci,oy+i-p,ox+j-p]
//
// GEMM view: rows = 128 output channels, columns = (tap, ci) for a group of taps
// (up to 256 columns), reduction over output pixels.  Both operands come from
// the NHWC planes the forward / data-gradient kernels also use, so along the
// reduction (pixels) they are MN-major: a TMA box {32 channels, Wt, Ht, Nt}
// lands in shared memory as [pixel][32 channels = 128 B].  For 32-bit operands
// kind::tf32 takes MN-major data only in the 128-byte swizzle with 32-byte atoms
// (4 pixels x 128 B per swizzle group), which TMA produces with
// CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B.  A K-step of 8 pixels is two groups (SBO =
// 512 B apart); 32-channel blocks sit LBO bytes apart.  The x operand of
// tap (i,j) is the same box shifted by (i-p, j-p) with TMA zero fill as padding.
//
// The reduction is long (batch x H x W pixels) and the output tiny, so pixels
// are split across CTAs; each CTA writes its partial tile and a second kernel
// sums the partials in a fixed order (deterministic, unlike the reference's
// atomicAdd split-K, src/cuda/graph/matmul.rs:207-261) and scatters into the
// [co][ci][kh][kw] layout.  In 3xTF32 mode no CTA accumulates more than
// tc::kMaxChainK pixels (the tensor core's f32 accumulation error grows with the
// chain length).
//
// Replaces conv2d_im2col + conv2d_out2mm + matmul_nt_splitk (src/cuda/nn/conv.rs:
// 298-320).
#include "tc_mainloop.cuh"

namespace {

constexpr int kWgThreads = 192;
constexpr int kMaxN = 256;        // widest UMMA
constexpr int kABlocks = 4;       // 4 x 32 output channels = 128 rows

struct WgradParams {
  int Wt, Ht, Nt, tiles_y, tiles_x;  // pixel tile (box) geometry in dy space
  int kp;                         // pixels per tile = Wt*Ht*Nt (multiple of 8)
  int n_tiles;                    // pixel tiles in all
  int tiles_per_split;
  int co, ci, kh, kw, pad;
  int taps_per_group, n_groups;   // taps handled by one CTA
  int cblocks;                    // ci / 32
  int a_box_blocks;               // 32-channel blocks of dy one box brings (min(4, co/32))
  int m_blocks;                   // ceil(co / 128)
  float* partial;                 // [split][m_block][group][col_block][128][group_cols]
  int group_cols;                 // taps_per_group * ci (1x1 with more than 256 input channels: 256)
  int col_blocks;                 // 1x1 only: column blocks of 256 input channels, each its own CTA
  int independent;                // reads nothing the kernel launched just before it wrote (NRS_PDL_PROLOGUE)
  float* direct;                  // 1x1, one split, no accumulation: the tile is the result; written straight to dw[co][ci]
};

template <int NPLANES, int STAGES>
__global__ void __launch_bounds__(kWgThreads, 1)
tc_wgrad_kernel(const __grid_constant__ CUtensorMap tm_dy_hi, const __grid_constant__ CUtensorMap tm_dy_lo,
                const __grid_constant__ CUtensorMap tm_x_hi, const __grid_constant__ CUtensorMap tm_x_lo,
                const WgradParams p, const int n_cols /*UMMA N, multiple of 16*/, int* __restrict__ err_flag) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  const uint32_t blk_bytes = (uint32_t)p.kp * 128u;               // one 32-channel block of one plane
  const uint32_t a_bytes = kABlocks * blk_bytes;                   // per plane
  const uint32_t b_bytes = (uint32_t)(p.group_cols / 32) * blk_bytes;
  const uint32_t stage_bytes = NPLANES * (a_bytes + b_bytes);
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + STAGES * stage_bytes);
  uint64_t* empty_bar = full_bar + STAGES;
  uint64_t* accum_bar = empty_bar + STAGES;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(accum_bar + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int cbk = blockIdx.x % p.col_blocks;
  const int mg = blockIdx.x / p.col_blocks;
  const int mb = mg / p.n_groups, grp = mg - mb * p.n_groups;
  const int split = blockIdx.y;
  // 32-channel blocks of x this CTA's columns cover (a column block of a wide 1x1 layer may be ragged)
  const int cblocks = p.col_blocks > 1 ? min(8, p.cblocks - cbk * 8) : p.cblocks;
  const int t_begin = split * p.tiles_per_split;
  const int t_end = min(p.n_tiles, t_begin + p.tiles_per_split);
  const int ntiles = t_end - t_begin;
  const int tap0 = grp * p.taps_per_group;
  const int ntaps = min(p.taps_per_group, p.kh * p.kw - tap0);

  if (warp == 0 && lane == 0) {
    tc::prefetch_tmap(&tm_dy_hi);
    tc::prefetch_tmap(&tm_x_hi);
    if (NPLANES == 2) { tc::prefetch_tmap(&tm_dy_lo); tc::prefetch_tmap(&tm_x_lo); }
    for (int s = 0; s < STAGES; ++s) { tc::mbar_init(&full_bar[s], 1); tc::mbar_init(&empty_bar[s], 1); }
    tc::mbar_init(accum_bar, 1);
    tc::fence_barrier_init();
  }
  if (warp == 1) {
    tc::tmem_alloc(tmem_slot, kMaxN);
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
      // ---------------- TMA producer: one pixel tile per ring slot
      // One 5-D box per operand plane brings all 32-channel blocks of a pixel tile at once
      // (the channel-block index is the outermost box dimension), so a tile costs
      // planes x (1 + taps) TMA instructions instead of one per block.
      // (a ragged last column block still receives a full box: TMA zero-fills the blocks beyond the tensor)
      const uint32_t tx = NPLANES * (uint32_t)(p.a_box_blocks + ntaps * (p.col_blocks > 1 ? 8 : p.cblocks)) * blk_bytes;
      int tap_i[9], tap_j[9];
      for (int t = 0; t < ntaps && t < 9; ++t) { tap_i[t] = (tap0 + t) / p.kw; tap_j[t] = (tap0 + t) - tap_i[t] * p.kw; }
      int issued = 0;
      bool ok = true;
      for (int it = 0; it < ntiles; ++it, ++issued) {
        const int s = it % STAGES;
        const uint32_t ph = (uint32_t)(it / STAGES) & 1u;
        if (!tc::mbar_wait(&empty_bar[s], ph ^ 1u)) { atomicExch(err_flag, tc::kErrProducerWait); ok = false; break; }
        const int pt = t_begin + it;
        const int xt = pt % p.tiles_x, rest = pt / p.tiles_x;
        const int n0 = (rest / p.tiles_y) * p.Nt, y0 = (rest % p.tiles_y) * p.Ht, x0 = xt * p.Wt;
        uint8_t* st = smem + (size_t)s * stage_bytes;
        tc::mbar_expect_tx(&full_bar[s], tx);
#pragma unroll 1
        for (int pl = 0; pl < NPLANES; ++pl) {
          const CUtensorMap* tdy = pl == 0 ? &tm_dy_hi : &tm_dy_lo;
          const CUtensorMap* txm = pl == 0 ? &tm_x_hi : &tm_x_lo;
          uint8_t* a_dst = st + pl * (a_bytes + b_bytes);
          uint8_t* b_dst = a_dst + a_bytes;
          tc::tma_load_5d(a_dst, tdy, &full_bar[s], 0, x0, y0, n0, mb * kABlocks);
          for (int t = 0; t < ntaps; ++t)
            tc::tma_load_5d(b_dst + (size_t)t * p.cblocks * blk_bytes, txm, &full_bar[s], 0, x0 + tap_j[t] - p.pad,
                            y0 + tap_i[t] - p.pad, n0, cbk * 8);
        }
      }
      if (!ok) {
        for (int it = (issued > STAGES ? issued - STAGES : 0); it < issued; ++it) {
          const int s = it % STAGES;
          if (!tc::mbar_wait(&full_bar[s], (uint32_t)(it / STAGES) & 1u)) { atomicExch(err_flag, tc::kErrDrainWait); break; }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      // ---------------- UMMA issuer: both operands MN-major, K-step = 8 pixels = one 1024 B atom
      const uint32_t idesc = tc::make_idesc_tf32(128, n_cols, true, true);
      bool ok = true;
      const int ksteps = p.kp / 8;
      for (int it = 0; it < ntiles; ++it) {
        const int s = it % STAGES;
        const uint32_t ph = (uint32_t)(it / STAGES) & 1u;
        if (!tc::mbar_wait(&full_bar[s], ph)) { atomicExch(err_flag, tc::kErrMmaWait); ok = false; break; }
        const uint32_t a_hi = tc::smem_u32(smem + (size_t)s * stage_bytes);
        const uint32_t b_hi = a_hi + a_bytes;
        const uint32_t a_lo = b_hi + b_bytes;
        const uint32_t b_lo = a_lo + a_bytes;
#pragma unroll 1
        for (int k = 0; k < ksteps; ++k) {
          const uint32_t koff = (uint32_t)k * 1024u;
          const uint64_t da_hi = tc::make_smem_desc_sw128_32b(a_hi + koff, blk_bytes, 512);
          const uint64_t db_hi = tc::make_smem_desc_sw128_32b(b_hi + koff, blk_bytes, 512);
          if (NPLANES == 2) {
            const uint64_t da_lo = tc::make_smem_desc_sw128_32b(a_lo + koff, blk_bytes, 512);
            const uint64_t db_lo = tc::make_smem_desc_sw128_32b(b_lo + koff, blk_bytes, 512);
            tc::umma_tf32(tmem_base, da_lo, db_hi, idesc, (it | k) != 0);
            tc::umma_tf32(tmem_base, da_hi, db_lo, idesc, 1);
            tc::umma_tf32(tmem_base, da_hi, db_hi, idesc, 1);
          } else {
            tc::umma_tf32(tmem_base, da_hi, db_hi, idesc, (it | k) != 0);
          }
        }
        tc::umma_commit(&empty_bar[s]);
      }
      if (ok) tc::umma_commit(accum_bar);
    }
  } else {
    // ---------------- epilogue: raw partial tile to the workspace
    const int q = warp & 3;
    const bool ok = tc::mbar_wait(accum_bar, 0);
    if (!ok && lane == 0) atomicExch(err_flag, tc::kErrEpilogueWait);
    if (ok) {
      tc::tc_fence_after_sync();
      const int row = q * 32 + lane;
      const int live_cols = p.col_blocks > 1 ? cblocks * 32 : ntaps * p.ci;
      float* dst = p.direct ? p.direct + (size_t)(mb * 128 + row) * p.ci + (size_t)cbk * 256
                            : p.partial + (((((size_t)split * p.m_blocks + mb) * p.n_groups + grp) * p.col_blocks + cbk) * 128 + row) *
                                              p.group_cols;
      const bool row_live = mb * 128 + row < p.co;
#pragma unroll 1
      for (int c = 0; c < (live_cols + 31) / 32; ++c) {
        uint32_t r[32];
        tc::tmem_ld_32x32(tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(c * 32), r);
        tc::tmem_ld_wait();
        if (row_live) {
#pragma unroll
          for (int j = 0; j < 32; j += 4)
            if (c * 32 + j < live_cols)
              *reinterpret_cast<float4*>(dst + c * 32 + j) =
                  make_float4(__uint_as_float(r[j]), __uint_as_float(r[j + 1]), __uint_as_float(r[j + 2]), __uint_as_float(r[j + 3]));
        }
      }
    }
  }

  if (p.independent) NRS_PDL_WAIT();   // nothing after this kernel may run ahead of its predecessor
  tc::tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc::tc_fence_after_sync();
    tc::tmem_dealloc(tmem_base, kMaxN);
  }
}

// dw[co][ci][tap] (+)= sum over splits of partial[split][mb][grp][row][t*ci + c].  A block is
// (kReduceThreads / lanes) outputs x `lanes` split lanes: lane y sums splits y, y+lanes, ... and the lanes are
// combined in lane order through shared memory, so the order of the additions is fixed (bit-reproducible)
// while the loads of one output are spread over `lanes` threads instead of one serial chain.
__global__ void __launch_bounds__(kReduceThreads)
tc_wgrad_reduce_kernel(const WgradParams p, int splits, int lanes, float* __restrict__ dw, int accumulate) {
  NRS_PDL_PROLOGUE();
  __shared__ float4 lane_sum[kReduceThreads];
  const int per_block = kReduceThreads / lanes;   // output quads of this block
  const int lane = threadIdx.x / per_block, slot = threadIdx.x - lane * per_block;
  const int taps = p.kh * p.kw;
  const int cq = p.ci / 4;                        // a thread owns four consecutive input channels (ci % 32 == 0)
  const size_t total = (size_t)p.co * cq * taps;
  const size_t idx = (size_t)blockIdx.x * per_block + slot;
  const bool live = idx < total;
  // idx enumerates (co, tap, ci/4) so that reads of the partials are coalesced 128-bit loads along ci
  const int c = (int)(idx % cq) * 4;
  const int tap = (int)((idx / cq) % taps);
  const int co = (int)(idx / ((size_t)cq * taps));
  const int mb = co / 128, row = co - mb * 128;
  const int grp = tap / p.taps_per_group, t = tap - grp * p.taps_per_group;
  const size_t tile = (size_t)128 * p.group_cols;
  const int cbk = p.col_blocks > 1 ? c / 256 : 0;
  const size_t col = p.col_blocks > 1 ? (size_t)(c - cbk * 256) : (size_t)t * p.ci + c;
  const size_t off = ((((size_t)mb * p.n_groups + grp) * p.col_blocks + cbk) * 128 + row) * p.group_cols + col;
  const size_t split_stride = (size_t)p.m_blocks * p.n_groups * p.col_blocks * tile;
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
  float* dst = dw + ((size_t)co * p.ci + c) * taps + tap;
  const float r[4] = {s.x, s.y, s.z, s.w};
#pragma unroll
  for (int k = 0; k < 4; ++k) dst[(size_t)k * taps] = accumulate ? dst[(size_t)k * taps] + r[k] : r[k];
}

}  // namespace

namespace {

template <int NPLANES, int STAGES>
int launch_wgrad(nrs_ctx* ctx, const CUtensorMap* maps, const WgradParams& p, int splits, size_t smem_bytes) {
  static NrsSmemAttr attr;
  NRS_ENSURE_SMEM(ctx, attr, (tc_wgrad_kernel<NPLANES, STAGES>), smem_bytes);
  int* err = nullptr;
  const int st = nrs_err_flag(ctx, &err);
  if (st != NRS_OK) return st;
  dim3 grid((unsigned)(p.m_blocks * p.n_groups * p.col_blocks), (unsigned)splits);
  NRS_PDL_LAUNCH((tc_wgrad_kernel<NPLANES, STAGES>), grid, kWgThreads, smem_bytes, ctx->stream, maps[0], maps[1], maps[2],
                 maps[3], p, p.group_cols, err);
  NRS_LAUNCHED(ctx);
  return NRS_OK;
}

}  // namespace

int nrs_tc_conv_wgrad(nrs_ctx* ctx, const float* x, const float* dy, float* dw, int n, int ci, int h, int wd, int co,
                      int kh, int kw, int stride, int pad, int accumulate) {
  if (!tc::tensor_map_encoder()) return NRS_ERR_UNSUPPORTED;
  if (stride != 1 || ci % 32 != 0 || co % 32 != 0 || n < 1) return NRS_ERR_UNSUPPORTED;
  if (ci > kMaxN && !(kh == 1 && kw == 1)) return NRS_ERR_UNSUPPORTED;   // wide layers: 1x1 only (column blocks)
  const int oh = h + 2 * pad - kh + 1, ow = wd + 2 * pad - kw + 1;
  if (ow > wd || oh > h || ow < 1 || oh < 1 || ow > 64) return NRS_ERR_UNSUPPORTED;
  const bool split3 = ctx->math_mode == NRS_MATH_3XTF32;
  const int planes = split3 ? 2 : 1;

  // Pixel tile = one TMA box {32 channels, Wt, Ht, Nt} of about 32 pixels.  (Measured: 16-pixel
  // tiles with a deeper ring are slower — the single producer thread becomes TMA-issue bound.)
  const int target = 32;
  WgradParams p{};
  p.Wt = ow;
  if (ow > target && ow % target == 0) p.Wt = target;
  p.tiles_x = ow / p.Wt;
  p.Ht = target / p.Wt > 1 ? target / p.Wt : 1;
  if (p.Ht > oh) p.Ht = oh;
  while ((p.Wt * p.Ht) % 8 != 0 && p.Ht < oh) ++p.Ht;
  p.Nt = 1;
  if (p.Ht == oh && p.Wt * p.Ht < target) {
    p.Nt = target / (p.Wt * p.Ht);
    if (p.Nt > n) p.Nt = n;
  }
  p.kp = p.Wt * p.Ht * p.Nt;
  if (p.kp % 8 != 0 || p.kp > 64) return NRS_ERR_UNSUPPORTED;
  p.tiles_y = (oh + p.Ht - 1) / p.Ht;
  p.n_tiles = ((n + p.Nt - 1) / p.Nt) * p.tiles_y * p.tiles_x;
  p.co = co; p.ci = ci; p.kh = kh; p.kw = kw; p.pad = pad;
  p.cblocks = ci / 32;
  p.m_blocks = (co + 127) / 128;
  const int taps = kh * kw;
  int tpg = ci <= kMaxN ? kMaxN / ci : 1;
  if (tpg > taps) tpg = taps;
  p.n_groups = (taps + tpg - 1) / tpg;
  p.taps_per_group = (taps + p.n_groups - 1) / p.n_groups;
  p.group_cols = p.taps_per_group * ci;
  p.col_blocks = 1;
  if (ci > kMaxN) {                 // 1x1: the input channels are cut into column blocks of 256, one CTA each
    p.col_blocks = (ci + kMaxN - 1) / kMaxN;
    p.n_groups = 1;
    p.taps_per_group = 1;
    p.group_cols = kMaxN;
  }

  // ring depth from the shared-memory budget
  const size_t stage_bytes = (size_t)planes * (kABlocks + p.group_cols / 32) * p.kp * 128;
  int stages = (int)((200 * 1024) / stage_bytes);
  if (stages < 2) return NRS_ERR_UNSUPPORTED;
  if (stages > 6) stages = 6;
  const size_t smem_bytes = stages * stage_bytes + 1024 + 256;

  // pixel split: fill the GPU, and bound the accumulation chain in 3xTF32 mode
  const int ctas_per_split = p.m_blocks * p.n_groups * p.col_blocks;
  const int max_tiles = split3 ? tc::kMaxChainK / p.kp : 1 << 30;
  int min_tiles = 512 / p.kp;   // amortise the prologue and the partial-tile store
  // ... unless that leaves most of the GPU idle (a short reduction with a small output: Linear layers)
  while (min_tiles > 4 && (long)(p.n_tiles / min_tiles) * ctas_per_split < ctx->sm_count / 2) min_tiles /= 2;
  if (min_tiles > max_tiles) min_tiles = max_tiles;
  const int tps = tc::plan_units_per_cta(ctx->sm_count, ctas_per_split, p.n_tiles, min_tiles, max_tiles, 8);
  p.tiles_per_split = tps;
  const int splits = (p.n_tiles + tps - 1) / tps;
  if (splits > 65535) return NRS_ERR_UNSUPPORTED;

  // workspaces: NHWC planes of dy and x, and the partial tiles
  const size_t dy_plane = (size_t)n * oh * ow * co, x_plane = (size_t)n * h * wd * ci;
  const size_t partial_floats = (size_t)splits * p.m_blocks * p.n_groups * p.col_blocks * 128 * p.group_cols;
  void *dy_hi = nullptr, *dy_lo = nullptr, *x_hi = nullptr, *x_lo = nullptr, *part = nullptr;
  bool may_overlap = ctx->independent_next;   // withdrawn below if this call stages an operand itself
  int st = nrs_ws_slot(ctx, NRS_WS_WGRAD_PARTIAL, partial_floats * sizeof(float), &part);
  if (st != NRS_OK) return st;
  p.partial = (float*)part;
  const size_t dy_img = (size_t)oh * ow * co, x_img = (size_t)h * wd * ci;
  if (const NrsPlanes* ready = nrs_planes_find(ctx, dy, split3)) {
    dy_hi = ready->hi;
    dy_lo = ready->lo;
  } else {
    may_overlap = false;
    st = nrs_ws_slot(ctx, NRS_WS_A_HI, dy_plane * sizeof(float), &dy_hi);
    if (st == NRS_OK && split3) st = nrs_ws_slot(ctx, NRS_WS_A_LO, dy_plane * sizeof(float), &dy_lo);
    if (st == NRS_OK)   // a [n, c, 1, 1] tensor is already pixel-major: split only
      st = oh * ow == 1 ? nrs_tc_stage(ctx, dy, (float*)dy_hi, (float*)dy_lo, n, co, co, 1, 0, 0, false)
                        : nrs_tc_stage(ctx, dy, (float*)dy_hi, (float*)dy_lo, oh * ow, co, co, n, dy_img, dy_img, true);
    if (st != NRS_OK) return st;
  }
  if (const NrsPlanes* ready = nrs_planes_find(ctx, x, split3)) {
    x_hi = ready->hi;
    x_lo = ready->lo;
  } else {
    may_overlap = false;
    st = nrs_ws_slot(ctx, NRS_WS_B_HI, x_plane * sizeof(float), &x_hi);
    if (st == NRS_OK && split3) st = nrs_ws_slot(ctx, NRS_WS_B_LO, x_plane * sizeof(float), &x_lo);
    if (st == NRS_OK)
      st = h * wd == 1 ? nrs_tc_stage(ctx, x, (float*)x_hi, (float*)x_lo, n, ci, ci, 1, 0, 0, false)
                       : nrs_tc_stage(ctx, x, (float*)x_hi, (float*)x_lo, h * wd, ci, ci, n, x_img, x_img, true);
    if (st != NRS_OK) return st;
  }

  CUtensorMap maps[4];
  p.a_box_blocks = co / 32 < kABlocks ? co / 32 : kABlocks;
  // planes viewed as [channel block][n][h][w][32 channels]: the block index is the outermost dimension
  const uint64_t ddim[5] = {32, (uint64_t)ow, (uint64_t)oh, (uint64_t)n, (uint64_t)(co / 32)};
  const uint64_t dstr[4] = {(uint64_t)co * 4, (uint64_t)ow * co * 4, (uint64_t)oh * ow * co * 4, 128};
  const uint64_t xdim[5] = {32, (uint64_t)wd, (uint64_t)h, (uint64_t)n, (uint64_t)(ci / 32)};
  const uint64_t xstr[4] = {(uint64_t)ci * 4, (uint64_t)wd * ci * 4, (uint64_t)h * wd * ci * 4, 128};
  const uint32_t dbox[5] = {32, (uint32_t)p.Wt, (uint32_t)p.Ht, (uint32_t)p.Nt, (uint32_t)p.a_box_blocks};
  const uint32_t xbox[5] = {32, (uint32_t)p.Wt, (uint32_t)p.Ht, (uint32_t)p.Nt, (uint32_t)(p.col_blocks > 1 ? 8 : p.cblocks)};
  bool ok = tc::encode_tmap_f32(&maps[0], dy_hi, 5, ddim, dstr, dbox, true) && tc::encode_tmap_f32(&maps[2], x_hi, 5, xdim, xstr, xbox, true);
  if (split3) ok = ok && tc::encode_tmap_f32(&maps[1], dy_lo, 5, ddim, dstr, dbox, true) && tc::encode_tmap_f32(&maps[3], x_lo, 5, xdim, xstr, xbox, true);
  else { maps[1] = maps[0]; maps[3] = maps[2]; }
  NRS_REQUIRE(ctx, ok, NRS_ERR_CUDA, "tc_wgrad: cuTensorMapEncodeTiled failed");
  p.independent = may_overlap ? 1 : 0;
  // a single split of a 1x1 "convolution" (A^T B) that overwrites its output needs no second pass
  p.direct = (splits == 1 && taps == 1 && !accumulate && (reinterpret_cast<uintptr_t>(dw) & 15) == 0) ? dw : nullptr;

#define NRS_WG(PL)                                                                     \
  switch (stages) {                                                                    \
    case 2: st = launch_wgrad<PL, 2>(ctx, maps, p, splits, smem_bytes); break;         \
    case 3: st = launch_wgrad<PL, 3>(ctx, maps, p, splits, smem_bytes); break;         \
    case 4: st = launch_wgrad<PL, 4>(ctx, maps, p, splits, smem_bytes); break;         \
    case 5: st = launch_wgrad<PL, 5>(ctx, maps, p, splits, smem_bytes); break;         \
    default: st = launch_wgrad<PL, 6>(ctx, maps, p, splits, smem_bytes); break;        \
  }
  if (split3) { NRS_WG(2) } else { NRS_WG(1) }
#undef NRS_WG
  if (st != NRS_OK) return st;
  if (p.direct) return NRS_OK;
  const size_t total = (size_t)co * ci * taps;
  const int lanes = reduce_lanes(splits);
  NRS_PDL_LAUNCH(tc_wgrad_reduce_kernel, nrs_blocks(total / 4, kReduceThreads / lanes), kReduceThreads, 0, ctx->stream, p, splits, lanes, dw,
                 accumulate);
  NRS_LAUNCHED(ctx);
  return NRS_OK;
}

// C[m,n] (+)= A^T B for A stored [k][m] and B stored [k][n] (both row-major) without transposing either:
// the reduction index k is the slow index of both operands, which is what the weight-gradient kernel above
// consumes (a 1x1 convolution over k "pixels": rows = A's columns, columns = B's columns).  The weight
// gradient of a Linear layer, dW = x^T dz, is this product on the activations' own row-major planes.
// NRS_ERR_UNSUPPORTED (no error text) unless m and n are multiples of 32 and k of 8.
int nrs_tc_gemm_tn(nrs_ctx* ctx, int m, int n, int k, const float* a, const float* b, float* c, int accumulate) {
  if (m % 32 != 0 || n % 32 != 0 || k < 8 || (k < 32 && k % 8 != 0)) return NRS_ERR_UNSUPPORTED;
  // Outputs of up to 4 M elements (the Linear layers of the CNN and transformer configurations).  Larger ones
  // (4096 x 4096 hidden layers) stay on the persistent GEMM kernel: its rastered tiles reuse operands through L2,
  // and the transposes it needs are small beside such a product.
  if ((long)m * n > (4L << 20)) return NRS_ERR_UNSUPPORTED;
  return nrs_tc_conv_wgrad(ctx, /*x=*/b, /*dy=*/a, /*dw=*/c, /*n=*/k, /*ci=*/n, 1, 1, /*co=*/m, 1, 1, 1, 0, accumulate);
}
