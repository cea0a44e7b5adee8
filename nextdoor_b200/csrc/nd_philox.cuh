// Counter-based RNG of the sampling kernels: Philox4x32-10 keyed by (sample, step, slot).
//
// Replaces the per-thread XORWOW state of the reference (init_curand_states,
// src/nextdoor.cu:1838-1843: 48 bytes per thread, draws tied to the thread id).  Draw contract:
// key = 64-bit run seed, counter = (global sample index, step, slot, draw/4), lane = draw%4,
// where `draw` counts the uniform draws inside one next() invocation from 0.  A draw is mapped
// to (0,1] exactly like curand_uniform: x * 2^-32 + 2^-33 in fp32.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

namespace ndrng {

__host__ __device__ __forceinline__ void philox4x32_10(uint32_t c0, uint32_t c1, uint32_t c2,
                                                       uint32_t c3, uint32_t k0, uint32_t k1,
                                                       uint32_t out[4]) {
#pragma unroll
  for (int r = 0; r < 10; r++) {
#ifdef __CUDA_ARCH__
    const uint32_t hi0 = __umulhi(0xD2511F53u, c0), lo0 = 0xD2511F53u * c0;
    const uint32_t hi1 = __umulhi(0xCD9E8D57u, c2), lo1 = 0xCD9E8D57u * c2;
#else
    const uint64_t p0 = (uint64_t)0xD2511F53u * c0, p1 = (uint64_t)0xCD9E8D57u * c2;
    const uint32_t hi0 = (uint32_t)(p0 >> 32), lo0 = (uint32_t)p0;
    const uint32_t hi1 = (uint32_t)(p1 >> 32), lo1 = (uint32_t)p1;
#endif
    const uint32_t n0 = hi1 ^ c1 ^ k0;
    const uint32_t n2 = hi0 ^ c3 ^ k1;
    c0 = n0; c1 = lo1; c2 = n2; c3 = lo0;
    k0 += 0x9E3779B9u;
    k1 += 0xBB67AE85u;
  }
  out[0] = c0; out[1] = c1; out[2] = c2; out[3] = c3;
}

__device__ __forceinline__ float u32_to_uniform(uint32_t x) {
  // one exact power-of-two scaling and one rounded add: identical to the host oracle
  return __fadd_rn(__fmul_rn(__uint2float_rn(x), 2.3283064365386963e-10f), 1.1641532182693481e-10f);
}

// RandNumGen::rand_int (src/rand_num_gen.cuh:117-122): min((int)(u*n), n-1), a lone fp32 multiply
__device__ __forceinline__ int32_t rand_int_from(float u, int32_t n) {
  const int32_t id = __float2int_rz(__fmul_rn(u, __int2float_rn(n)));
  return id < n - 1 ? id : n - 1;
}

// Handle one next() invocation draws from.  Caches the four lanes of the current block.
struct Rng {
  uint32_t k0, k1, sample, step, slot, draw;
  uint32_t lanes[4];

  __device__ __forceinline__ Rng(uint64_t seed, uint32_t sample_, uint32_t step_, uint32_t slot_)
      : k0((uint32_t)seed), k1((uint32_t)(seed >> 32)), sample(sample_), step(step_), slot(slot_), draw(0) {}

  __device__ __forceinline__ uint32_t next_u32() {
    if ((draw & 3u) == 0u) philox4x32_10(sample, step, slot, draw >> 2, k0, k1, lanes);
    // lane select without dynamic register indexing
    const uint32_t l = draw & 3u;
    const uint32_t x = l == 0 ? lanes[0] : (l == 1 ? lanes[1] : (l == 2 ? lanes[2] : lanes[3]));
    draw++;
    return x;
  }
  // continue at draw `d` of the invocation (the draws before it were consumed elsewhere)
  __device__ __forceinline__ void seek(uint32_t d) {
    draw = d;
    if (d & 3u) philox4x32_10(sample, step, slot, d >> 2, k0, k1, lanes);
  }
  __device__ __forceinline__ float uniform() { return u32_to_uniform(next_u32()); }
  __device__ __forceinline__ int32_t rand_int(int32_t n) { return rand_int_from(uniform(), n); }
};

}  // namespace ndrng
