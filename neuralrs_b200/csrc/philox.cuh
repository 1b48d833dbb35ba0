// Philox-4x32-10 (Salmon, Moraes, Dror, Shaw: "Parallel random numbers: as easy as 1, 2, 3", SC'11), the
// counter-based generator behind the dropout masks and the augmentation draws: ten rounds of two
// 32x32->64-bit multiplies, the key bumped by the Weyl constants between rounds.  A block is addressed by
// a 64-bit counter under a 64-bit key (the context's seed); uniform01 maps a word to [0, 1).
#pragma once
#include <cstdint>

namespace nrs_rng {

__host__ __device__ __forceinline__ void philox4x32_10(uint32_t (&ctr)[4], uint32_t k0, uint32_t k1) {
#pragma unroll
  for (int r = 0; r < 10; ++r) {
    const uint64_t p0 = (uint64_t)0xD2511F53u * ctr[0];
    const uint64_t p1 = (uint64_t)0xCD9E8D57u * ctr[2];
    const uint32_t n0 = (uint32_t)(p1 >> 32) ^ ctr[1] ^ k0;
    const uint32_t n1 = (uint32_t)p1;
    const uint32_t n2 = (uint32_t)(p0 >> 32) ^ ctr[3] ^ k1;
    const uint32_t n3 = (uint32_t)p0;
    ctr[0] = n0; ctr[1] = n1; ctr[2] = n2; ctr[3] = n3;
    k0 += 0x9E3779B9u;
    k1 += 0xBB67AE85u;
  }
}

// The four words of block `at` under `seed`.
__host__ __device__ __forceinline__ void block(uint64_t seed, uint64_t at, uint32_t (&out)[4]) {
  out[0] = (uint32_t)at; out[1] = (uint32_t)(at >> 32); out[2] = 0u; out[3] = 0u;
  philox4x32_10(out, (uint32_t)seed, (uint32_t)(seed >> 32));
}

__host__ __device__ __forceinline__ float uniform01(uint32_t word) { return (float)(word >> 8) * (1.0f / 16777216.0f); }

}  // namespace nrs_rng
