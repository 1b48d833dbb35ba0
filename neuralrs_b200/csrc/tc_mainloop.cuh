// Shared tcgen05 main loop: D[128 x BN] (TMEM, f32) = sum over K-slices of
// A[128 x 32] . B[BN x 32]^T, both operands K-major in 128-byte-swizzled shared
// memory, fed by TMA, consumed by tcgen05.mma kind::tf32.
//
// Persistent CTAs (one per SM) walk a list of output tiles (row tile, column tile,
// batch x K-split).  Six warps, fixed roles:
//   warp 0     TMA producer (one thread): per K-slice, one mbarrier-tracked ring
//              slot holding the A and B slices (and their residual planes for 3xTF32);
//              the ring runs ahead across tile boundaries
//   warp 1     TMEM allocation; one thread issues the UMMAs (M=128, K=8) and commits
//              ring slots back to the producer, then the accumulator to the epilogue
//   warps 2-5  epilogue: tcgen05.ld (thread = accumulator row), policy-defined store
// TMEM holds two accumulators, so the epilogue of tile i runs under the main loop of
// tile i+1.
// A Policy supplies how an A slice is fetched (dense rows for GEMM, a shifted
// NHWC window for convolution) and what the epilogue does with a row of results.
// A policy with kCanEmit may also hand the finished values back: the epilogue warps then
// write them as TF32 high / residual planes ([row][32 columns], 128-byte swizzle) into a
// staging tile and one thread sends each tile to global memory with a TMA store — the
// operand planes of the next tensor-core kernel, written in full lines without a pass of
// their own.
//
// 3xTF32 (NPLANES == 2): the residual plane of B sits directly behind its high plane in
// the ring slot, so one UMMA of width 2*BN computes A_hi.[B_hi ; B_lo] (hi*hi in columns
// [0,BN), hi*lo in [BN,2BN)) and a second of width BN adds A_lo.B_hi onto the first half;
// the epilogue sums the halves.  Against three UMMAs of width BN this reads a quarter
// less shared memory per K-step, which is what bounds the narrow (BN = 64) tiles.
// The tensor core's f32 accumulation is not round-to-nearest; its error grows
// linearly with the length of one accumulation chain (about 7e-9 relative per K
// element), so callers keep a chain at or below kMaxChainK by splitting K across
// tiles, whose partial results are summed in f32 by tc_splitk_reduce_kernel in a
// fixed order.
//
// Every mbarrier wait is bounded: on expiry the kernel records an error code,
// waits (bounded) for TMA loads it already issued, frees its TMEM and returns.
#pragma once

#include "igemm_problems.cuh"
#include "nrs_internal.h"
#include "tc_common.cuh"

namespace tc {

constexpr int BM = 128, BK = 32;   // BK f32 = 128 bytes = one swizzle row
constexpr int kThreads = 192;
constexpr int kMaxChainK = 4096;   // longest single accumulation chain in 3xTF32 mode
constexpr int kGroupM = 16;        // row tiles per raster group (see TileMap)

template <int BN, int NPLANES, int EMIT_BYTES = 0>
struct SmemLayout {
  static constexpr int kATile = BM * BK * 4;   // 16 KB
  static constexpr int kBTile = BN * BK * 4;
  static constexpr int kStage = NPLANES * (kATile + kBTile);   // [A_hi][B_hi][B_lo][A_lo]
  static constexpr int kExtra = EMIT_BYTES /*plane staging tile*/ + 1024 /*align*/ + 256 /*barriers*/;
  static constexpr int kRing = 227 * 1024 - kExtra;
  static constexpr int kStages = kRing / kStage >= 8 ? 8 : kRing / kStage;
  static constexpr int kBytes = kStages * kStage + kExtra;
  static constexpr int kAccCols = NPLANES * BN;                 // one accumulator
  static constexpr int kTmemCols = 2 * kAccCols < 32 ? 32 : 2 * kAccCols;   // two of them
  static_assert((kTmemCols & (kTmemCols - 1)) == 0 && kTmemCols <= 512, "TMEM allocation must be a power of two <= 512");
};

struct SplitInfo {
  int splits;          // K-splits per (tile, batch)
  int kb_per_split;    // K-slices per split
  int kb_total;        // K-slices in all
  int batches;
  float* partial;      // [split][batch][tiles_m*128][n_total] when splits > 1
  int n_total;
  int rows_total;      // tiles_m * 128
};

// Tile list of one launch.  Within a (batch, split) plane tiles are visited in groups of
// kGroupM row tiles x all column tiles, row tile fastest, so the tiles in flight at any
// moment cover a compact block of the output and share operand slices through L2.
struct TileMap {
  int tiles_m, tiles_n;
  long total;          // tiles_m * tiles_n * batches * splits
  __device__ __forceinline__ void decode(long t, int* tile_m, int* tile_n, int* z) const {
    const int per_z = tiles_m * tiles_n;
    *z = (int)(t / per_z);
    const int r = (int)(t - (long)*z * per_z);
    const int group = r / (kGroupM * tiles_n);
    const int first = group * kGroupM;
    const int gm = min(kGroupM, tiles_m - first);
    const int rr = r - group * kGroupM * tiles_n;
    *tile_n = rr / gm;
    *tile_m = first + (rr - *tile_n * gm);
  }
};

// Shared memory of the plane-emission staging tile: one [128 rows][128 B] tile per plane.
template <int NPLANES, class Policy>
__host__ __device__ constexpr int emit_bytes() { return Policy::kCanEmit ? NPLANES * BM * 128 : 0; }

template <int BN, int NPLANES, class Policy>
__global__ void __launch_bounds__(kThreads, 1)
tc_kernel(const __grid_constant__ CUtensorMap tm_a_hi, const __grid_constant__ CUtensorMap tm_a_lo,
          const __grid_constant__ CUtensorMap tm_b_hi, const __grid_constant__ CUtensorMap tm_b_lo,
          const __grid_constant__ CUtensorMap tm_out_hi, const __grid_constant__ CUtensorMap tm_out_lo,
          const Policy pol, const SplitInfo sp, const TileMap tmap, const int emit /*planes to emit: 0, 1 or 2*/,
          int* __restrict__ err_flag) {
  constexpr int kEmitBytes = emit_bytes<NPLANES, Policy>();
  using L = SmemLayout<BN, NPLANES, kEmitBytes>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint8_t* emit_tile = smem + L::kStages * L::kStage;   // [planes][128 rows][128 B], 1024-byte aligned
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(emit_tile + kEmitBytes);
  uint64_t* empty_bar = full_bar + L::kStages;
  uint64_t* acc_full = empty_bar + L::kStages;   // [2] accumulator ready for the epilogue
  uint64_t* acc_empty = acc_full + 2;            // [2] accumulator drained by the epilogue
  uint64_t* emit_bar = acc_empty + 2;            // [2] staging tile free / staging tile written
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(emit_bar + 2);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (warp == 0 && lane == 0) {
    prefetch_tmap(&tm_a_hi);
    prefetch_tmap(&tm_b_hi);
    if (NPLANES == 2) { prefetch_tmap(&tm_a_lo); prefetch_tmap(&tm_b_lo); }
    if (emit >= 1) prefetch_tmap(&tm_out_hi);
    if (emit == 2) prefetch_tmap(&tm_out_lo);
    for (int s = 0; s < L::kStages; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
    for (int b = 0; b < 2; ++b) { mbar_init(&acc_full[b], 1); mbar_init(&acc_empty[b], 4); mbar_init(&emit_bar[b], 128); }
    fence_barrier_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, L::kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  // Everything above (barriers, tensor memory, descriptor prefetch) may overlap the tail of the kernel
  // before this one in the stream; from here on its results are needed.
  NRS_PDL_WAIT();
  NRS_PDL_TRIGGER();   // the next kernel may be scheduled as this grid's SMs free up

  if (warp == 0) {
    if (lane == 0) {
      // ---------------- TMA producer
      const uint32_t stage_bytes = (uint32_t)NPLANES * (pol.a_slice_bytes() + (uint32_t)L::kBTile);
      uint32_t it = 0;   // ring position, runs on across tiles
      bool ok = true;
      for (long t = blockIdx.x; t < tmap.total && ok; t += gridDim.x) {
        int tile_m, tile_n, z;
        tmap.decode(t, &tile_m, &tile_n, &z);
        const int batch = z / sp.splits, split = z - batch * sp.splits;
        const int kb_begin = split * sp.kb_per_split;
        const int kb_end = min(sp.kb_total, kb_begin + sp.kb_per_split);
        const int n0 = tile_n * BN;
        for (int kb = kb_begin; kb < kb_end; ++kb, ++it) {
          const int s = it % L::kStages;
          const uint32_t ph = (it / L::kStages) & 1u;
          if (!mbar_wait(&empty_bar[s], ph ^ 1u)) { atomicExch(err_flag, kErrProducerWait); ok = false; break; }
          uint8_t* st = smem + s * L::kStage;
          mbar_expect_tx(&full_bar[s], stage_bytes);
          pol.load_a(st, &tm_a_hi, &full_bar[s], kb, tile_m, batch);
          tma_load_3d(st + L::kATile, &tm_b_hi, &full_bar[s], kb * BK, n0, batch);
          if (NPLANES == 2) {
            tma_load_3d(st + L::kATile + L::kBTile, &tm_b_lo, &full_bar[s], kb * BK, n0, batch);
            pol.load_a(st + L::kATile + 2 * L::kBTile, &tm_a_lo, &full_bar[s], kb, tile_m, batch);
          }
        }
      }
      if (!ok) {
        // Loads already issued still land in this CTA's shared memory: wait for them
        // (bounded) before the CTA may retire.
        for (uint32_t j = (it > (uint32_t)L::kStages ? it - L::kStages : 0); j < it; ++j) {
          const int s = j % L::kStages;
          if (!mbar_wait(&full_bar[s], (j / L::kStages) & 1u)) { atomicExch(err_flag, kErrDrainWait); break; }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      // ---------------- UMMA issuer
      constexpr uint32_t idesc_wide = make_idesc_tf32(BM, NPLANES * BN, false, false);
      constexpr uint32_t idesc_half = make_idesc_tf32(BM, BN, false, false);
      uint32_t it = 0, local = 0;
      bool ok = true;
      for (long t = blockIdx.x; t < tmap.total && ok; t += gridDim.x, ++local) {
        int tile_m, tile_n, z;
        tmap.decode(t, &tile_m, &tile_n, &z);
        const int split = z % sp.splits;
        const int kb_begin = split * sp.kb_per_split;
        const int nkb = min(sp.kb_total, kb_begin + sp.kb_per_split) - kb_begin;   // >= 1 by construction
        const uint32_t buf = local & 1u, use = local >> 1;
        if (!mbar_wait(&acc_empty[buf], (use & 1u) ^ 1u)) { atomicExch(err_flag, kErrMmaWait); break; }
        tc_fence_after_sync();
        const uint32_t d = tmem_base + buf * (uint32_t)L::kAccCols;
        for (int i = 0; i < nkb; ++i, ++it) {
          const int s = it % L::kStages;
          const uint32_t ph = (it / L::kStages) & 1u;
          // (No tcgen05 fence here: the mbarrier's complete_tx orders the TMA writes before the
          // UMMAs, and a fence would make the issuing thread wait out the UMMAs in flight.)
          if (!mbar_wait(&full_bar[s], ph)) { atomicExch(err_flag, kErrMmaWait); ok = false; break; }
          const uint32_t a_hi = smem_u32(smem + s * L::kStage);
          const uint32_t b_hi = a_hi + L::kATile;                 // B_lo follows B_hi directly
          const uint32_t a_lo = b_hi + 2 * L::kBTile;
#pragma unroll
          for (int k = 0; k < BK / 8; ++k) {
            const uint32_t koff = k * 32;  // 8 f32 along K inside the 128-byte swizzle row
            const uint64_t da_hi = make_smem_desc_sw128(a_hi + koff, 16, 1024);
            const uint64_t db_hi = make_smem_desc_sw128(b_hi + koff, 16, 1024);
            umma_tf32(d, da_hi, db_hi, idesc_wide, (i | k) != 0);   // hi*hi | hi*lo
            if (NPLANES == 2) {
              const uint64_t da_lo = make_smem_desc_sw128(a_lo + koff, 16, 1024);
              umma_tf32(d, da_lo, db_hi, idesc_half, 1);             // + lo*hi
            }
          }
          umma_commit(&empty_bar[s]);  // slot reusable once these UMMAs have read it
        }
        if (ok) umma_commit(&acc_full[buf]);
      }
    }
  } else {
    // ---------------- epilogue: warp w owns TMEM lanes [32*(w%4), +32)
    const int q = warp & 3;
    const int row = q * 32 + lane;   // row inside the tile
    const bool emit_issuer = warp == 2 && lane == 0;
    uint32_t local = 0, emitted = 0;
    bool ok = true;
    for (long t = blockIdx.x; t < tmap.total && ok; t += gridDim.x, ++local) {
      int tile_m, tile_n, z;
      tmap.decode(t, &tile_m, &tile_n, &z);
      const int batch = z / sp.splits, split = z - batch * sp.splits;
      const int n0 = tile_n * BN;
      const uint32_t buf = local & 1u, use = local >> 1;
      if (!mbar_wait(&acc_full[buf], use & 1u)) {
        if (lane == 0) atomicExch(err_flag, kErrEpilogueWait);
        break;
      }
      tc_fence_after_sync();
      const uint32_t acc = tmem_base + buf * (uint32_t)L::kAccCols + ((uint32_t)(q * 32) << 16);
#pragma unroll 1
      for (int c = 0; c < (BN + 31) / 32; ++c) {
        uint32_t r[32];
        tmem_ld_32x32(acc + (uint32_t)(c * 32), r);
        if (NPLANES == 2) {
          uint32_t r2[32];
          tmem_ld_32x32(acc + (uint32_t)(BN + c * 32), r2);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 32; ++j) r[j] = __float_as_uint(__uint_as_float(r[j]) + __uint_as_float(r2[j]));
        } else {
          tmem_ld_wait();
        }
        if (c == (BN + 31) / 32 - 1) {
          // Everything this warp needs is in registers: hand the accumulator back.
          tc_fence_before_sync();
          __syncwarp();
          if (lane == 0) mbar_arrive(&acc_empty[buf]);
        }
        const int ncols = (BN - c * 32) < 32 ? (BN - c * 32) : 32;
        if (sp.splits > 1) {
          float* dst = sp.partial + (((size_t)split * sp.batches + batch) * sp.rows_total + (size_t)tile_m * BM + row) * sp.n_total;
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            const int n = n0 + c * 32 + j;
            if (c * 32 + j < BN && n < sp.n_total) dst[n] = __uint_as_float(r[j]);
          }
        } else if constexpr (Policy::kCanEmit) {
          float v[32];
          pol.epilogue(tile_m, batch, row, n0 + c * 32, ncols, r, v);
          if (float* cs = pol.colsum_row(tile_m, q)) {
            // Sum over this warp's 32 rows, one channel per lane: a 32 x 32 transpose-reduce in 31
            // shuffles (each stage halves the values a lane holds; fixed order, deterministic).
            float s[32];
#pragma unroll
            for (int j = 0; j < 32; ++j) s[j] = v[j];
#pragma unroll
            for (int d = 16; d >= 1; d >>= 1) {
              const bool up = (lane & d) != 0;
#pragma unroll
              for (int i = 0; i < d; ++i) {
                const float keep = up ? s[i + d] : s[i];
                const float send = up ? s[i] : s[i + d];
                s[i] = keep + __shfl_xor_sync(0xffffffffu, send, d);
              }
            }
            cs[n0 + c * 32 + lane] = s[0];
          }
          if (emit) {
            // The staging tile is free once the previous TMA store has read it; the issuer
            // arrives on emit_bar[0] only after that.
            const uint32_t ph = emitted & 1u;
            ++emitted;
            if (emit_issuer) bulk_wait_read();
            mbar_arrive(&emit_bar[0]);
            if (!mbar_wait(&emit_bar[0], ph)) { atomicExch(err_flag, kErrEpilogueWait); ok = false; break; }
            uint8_t* row_hi = emit_tile + row * 128;
#pragma unroll
            for (int g = 0; g < 8; ++g) {
              const int chunk = (g ^ (row & 7)) * 16;   // 128-byte swizzle: 16-byte chunk index XOR row % 8
              const float4 h = make_float4(tf32_rn(v[4 * g]), tf32_rn(v[4 * g + 1]), tf32_rn(v[4 * g + 2]), tf32_rn(v[4 * g + 3]));
              *reinterpret_cast<float4*>(row_hi + chunk) = h;
              if (NPLANES == 2 && emit == 2)
                *reinterpret_cast<float4*>(row_hi + BM * 128 + chunk) =
                    make_float4(v[4 * g] - h.x, v[4 * g + 1] - h.y, v[4 * g + 2] - h.z, v[4 * g + 3] - h.w);
            }
            fence_proxy_async();   // generic-proxy writes -> visible to the TMA engine
            mbar_arrive(&emit_bar[1]);
            if (emit_issuer) {
              if (!mbar_wait(&emit_bar[1], ph)) { atomicExch(err_flag, kErrEpilogueWait); ok = false; break; }
              int c1, c2, c3;
              pol.out_origin(tile_m, &c1, &c2, &c3);
              tma_store_4d(&tm_out_hi, emit_tile, n0 + c * 32, c1, c2, c3);
              if (NPLANES == 2 && emit == 2) tma_store_4d(&tm_out_lo, emit_tile + BM * 128, n0 + c * 32, c1, c2, c3);
              bulk_commit();
            }
          }
        } else {
          pol.epilogue(tile_m, batch, row, n0 + c * 32, ncols, r);
        }
      }
    }
    if (emit_issuer) bulk_wait_all();   // shared memory must outlive the stores that read it
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, L::kTmemCols);
  }
}

// out(row, n) = policy.store(sum over splits of partial), fixed summation order.
template <class Policy>
__global__ void __launch_bounds__(256)
tc_splitk_reduce_kernel(const Policy pol, const SplitInfo sp) {
  NRS_PDL_PROLOGUE();
  const size_t per = (size_t)sp.batches * sp.rows_total * sp.n_total;
  const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= per) return;
  float s = 0.0f;
  for (int z = 0; z < sp.splits; ++z) s += sp.partial[(size_t)z * per + idx];
  const int n = (int)(idx % sp.n_total);
  const size_t t = idx / sp.n_total;
  const int row_lin = (int)(t % sp.rows_total);
  const int b = (int)(t / sp.rows_total);
  pol.store(row_lin / BM, b, row_lin % BM, n, s);
}

// Chooses the K-split: enough CTAs to fill the GPU, and no accumulation chain longer
// than kMaxChainK elements when `limit_chain`.
inline void plan_split(const nrs_ctx* ctx, long tiles, int kb_total, bool limit_chain, int* splits, int* kb_per_split) {
  int s = 1;
  // (More than half a wave of tiles runs unsplit: the second pass over the partial tiles costs more
  // than the idle SMs.)
  if (2 * tiles <= ctx->sm_count && kb_total >= 32) {
    s = (int)(ctx->sm_count / tiles);
    if (s > kb_total / 16) s = kb_total / 16;   // a split shorter than 16 K-blocks is all prologue and second pass
  }
  if (limit_chain) {
    const int need = (kb_total * BK + kMaxChainK - 1) / kMaxChainK;
    if (s < need) s = need;
  }
  if (s < 1) s = 1;
  int per = (kb_total + s - 1) / s;
  if (per < 1) per = 1;
  *kb_per_split = per;
  *splits = (kb_total + per - 1) / per;
}

// Work units (pixel tiles, image rows) per CTA for a reduction that is split across CTAs, `ctas`
// CTAs per split and one CTA per SM at a time.  Candidates put the CTA count just under a whole
// number of waves (a count just over one costs a whole extra round); a CTA's fixed cost
// (prologue, partial-tile store) is weighed in as `overhead_units`; more than max_units per CTA
// (the accumulation-chain limit) is not allowed, fewer than min_units not worthwhile.
inline int plan_units_per_cta(int sm_count, int ctas, long units, int min_units, int max_units, int overhead_units) {
  if (units < 1) return 1;
  long best_u = -1, best_cost = 0;
  for (int w = 1; w <= 64; ++w) {
    const long splits = (long)w * sm_count / ctas;
    if (splits < 1) continue;
    long u = (units + splits - 1) / splits;
    if (u < min_units) u = min_units;
    if (u > units) u = units;
    if (u > max_units) continue;
    const long actual = (units + u - 1) / u;
    const long rounds = (actual * ctas + sm_count - 1) / sm_count;
    const long cost = rounds * (u + overhead_units);
    if (best_u < 0 || cost < best_cost) { best_u = u; best_cost = cost; }
  }
  if (best_u < 0) best_u = max_units < units ? max_units : units;
  return (int)(best_u < 1 ? 1 : best_u);
}

template <int BN, int NPLANES, class Policy>
int launch(nrs_ctx* ctx, const CUtensorMap& ta_hi, const CUtensorMap& ta_lo, const CUtensorMap& tb_hi,
           const CUtensorMap& tb_lo, const Policy& pol, int tiles_m, int n_total, int batches, int kb_total,
           const CUtensorMap* out_hi = nullptr, const CUtensorMap* out_lo = nullptr, int* splits_out = nullptr) {
  using L = SmemLayout<BN, NPLANES, emit_bytes<NPLANES, Policy>()>;
  constexpr int kSmem = L::kBytes;
  static_assert(kSmem <= 227 * 1024 && L::kStages >= 2, "shared memory budget");
  static NrsSmemAttr attr;
  NRS_ENSURE_SMEM(ctx, attr, (tc_kernel<BN, NPLANES, Policy>), kSmem);
  const int tiles_n = (n_total + BN - 1) / BN;
  SplitInfo sp{};
  plan_split(ctx, (long)tiles_m * tiles_n * batches, kb_total, NPLANES == 2, &sp.splits, &sp.kb_per_split);
  sp.kb_total = kb_total;
  sp.batches = batches;
  sp.n_total = n_total;
  sp.rows_total = tiles_m * BM;
  sp.partial = nullptr;
  if (splits_out) *splits_out = sp.splits;
  if (sp.splits > 1) {
    void* ws = nullptr;
    const int st = nrs_ws_slot(ctx, NRS_WS_PARTIAL, (size_t)sp.splits * batches * sp.rows_total * n_total * sizeof(float), &ws);
    if (st != NRS_OK) return st;
    sp.partial = (float*)ws;
  }
  int* err = nullptr;
  int st = nrs_err_flag(ctx, &err);
  if (st != NRS_OK) return st;
  TileMap tmap{tiles_m, tiles_n, (long)tiles_m * tiles_n * batches * sp.splits};
  const unsigned grid = (unsigned)(tmap.total < ctx->sm_count ? tmap.total : ctx->sm_count);
  // Planes can only be emitted by the direct epilogue; with a K-split the policy's store() writes them.
  const int emit = (Policy::kCanEmit && out_hi && sp.splits == 1) ? (out_lo && NPLANES == 2 ? 2 : 1) : 0;
  NRS_PDL_LAUNCH((tc_kernel<BN, NPLANES, Policy>), grid, kThreads, kSmem, ctx->stream, ta_hi, ta_lo, tb_hi, tb_lo,
                 out_hi ? *out_hi : ta_hi, out_lo ? *out_lo : ta_hi, pol, sp, tmap, emit, err);
  NRS_LAUNCHED(ctx);
  if (sp.splits > 1) {
    const size_t per = (size_t)batches * sp.rows_total * n_total;
    NRS_PDL_LAUNCH((tc_splitk_reduce_kernel<Policy>), nrs_blocks(per, 256), 256, 0, ctx->stream, pol, sp);
    NRS_LAUNCHED(ctx);
  }
  return NRS_OK;
}

}  // namespace tc

// Operand staging (tc_stage.cu).  Planes are [batch][rows][ldk] f32 with ldk a multiple of
// 32 and zeros beyond K; `lo == nullptr` means no split (hi = the values themselves).
// src_k_by_rows: the source is stored [K][rows] (transposed) instead of [rows][K].
int nrs_tc_stage(nrs_ctx* ctx, const float* src, float* hi, float* lo, int rows, int K, int ldk, int batch,
                 size_t src_bstride, size_t dst_bstride, bool src_k_by_rows);
// Masked gradient staging (see stage_masked_kernel): mode 0 = ReLU mask of dy[n,c,h,w] by y;
// mode 1 = gradient of a k x k / stride-k max-pool (g[n,c,h/k,w/k], argmax) followed by the ReLU
// mask, taken from the pooled output y[n,c,h/k,w/k].  nchw_out and the planes are each optional
// (lo only with hi).  chan_partial (optional, nrs_stage_masked_partial_rows(...) x c floats): per-block
// channel sums of the result, for the bias gradient; *chan_partial_rows receives how many rows
// were written (0: this path does not produce them and the caller sums the NCHW gradient).
int nrs_tc_stage_masked(nrs_ctx* ctx, int mode, const float* g, const float* y, const int32_t* argmax, int n, int c,
                        int h, int w, int k, float* nchw_out, float* hi, float* lo, float* chan_partial = nullptr,
                        int* chan_partial_rows = nullptr);
// 2x2 / stride-2 max-pool forward that also writes the NHWC planes of the pooled output
// (NRS_ERR_UNSUPPORTED for odd image sizes).
int nrs_tc_pool2_fwd_planes(nrs_ctx* ctx, const float* x, float* y, int32_t* argmax, float* hi, float* lo, int n, int c,
                            int h, int w);
inline size_t nrs_stage_masked_partial_rows(int n, int h, int w) { return ((size_t)n * (h / 2) * (w / 2) + 31) / 32; }
// Conv weights w[co][ci][kh][kw] -> K-major planes.
//  for_dgrad == 0: out[co][(i*kw + j)*ci_n + ci]   (forward B operand)
//  for_dgrad == 1: out[ci][(i*kw + j)*co_n + co]   (data-gradient B operand)
int nrs_tc_stage_conv_weight(nrs_ctx* ctx, const float* w, float* hi, float* lo, int co, int ci, int kh, int kw,
                             int for_dgrad);
