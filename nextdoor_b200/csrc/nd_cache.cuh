// L2 residency hints for the per-step arrays of the walk kernels.
//
// A next() launch streams tens to hundreds of MB of single-use gather sectors (neighbour ids,
// weight records, set buckets) through the L2, which is about as large; without a hint those
// sectors push out the arrays that ARE used again a few microseconds later (the transit maps the
// scatter kernel just wrote, the row offsets, the ticket counters, the staged output row), and
// every one of their reads becomes a DRAM access.  Loads, stores and atomics of those arrays go
// through the ops below, which carry an L2 cache policy made by createpolicy (evict_last); the
// gathers carry evict_first.  ND_TUNE_KEEP=0 turns the ops into plain accesses.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#ifndef ND_TUNE_KEEP
#define ND_TUNE_KEEP 1
#endif

namespace ndmem {

struct Keep {
  uint64_t pol;
  __device__ __forceinline__ Keep() {
#if ND_TUNE_KEEP
    asm("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(pol));
#else
    pol = 0;
#endif
  }
  __device__ __forceinline__ int32_t ld(const int32_t *p) const {
#if ND_TUNE_KEEP
    int32_t v;
    asm("ld.global.L2::cache_hint.s32 %0, [%1], %2;" : "=r"(v) : "l"(p), "l"(pol));
    return v;
#else
    return *p;
#endif
  }
  // read-only for the whole kernel (row offsets)
  __device__ __forceinline__ int32_t ld_const(const int32_t *p) const {
#if ND_TUNE_KEEP
    int32_t v;
    asm("ld.global.nc.L2::cache_hint.s32 %0, [%1], %2;" : "=r"(v) : "l"(p), "l"(pol));
    return v;
#else
    return __ldg(p);
#endif
  }
  __device__ __forceinline__ uint32_t ld(const uint32_t *p) const { return (uint32_t)ld(reinterpret_cast<const int32_t *>(p)); }
  __device__ __forceinline__ int2 ld(const int2 *p) const {
#if ND_TUNE_KEEP
    int2 v;
    asm("ld.global.L2::cache_hint.v2.s32 {%0, %1}, [%2], %3;" : "=r"(v.x), "=r"(v.y) : "l"(p), "l"(pol));
    return v;
#else
    return *p;
#endif
  }
  __device__ __forceinline__ int4 ld(const int4 *p) const {
#if ND_TUNE_KEEP
    int4 v;
    asm("ld.global.L2::cache_hint.v4.s32 {%0, %1, %2, %3}, [%4], %5;" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p), "l"(pol));
    return v;
#else
    return *p;
#endif
  }
  __device__ __forceinline__ void st(int4 *p, int4 v) const {
#if ND_TUNE_KEEP
    asm volatile("st.global.L2::cache_hint.v4.s32 [%0], {%1, %2, %3, %4}, %5;" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w), "l"(pol) : "memory");
#else
    *p = v;
#endif
  }
  __device__ __forceinline__ void st(int32_t *p, int32_t v) const {
#if ND_TUNE_KEEP
    asm volatile("st.global.L2::cache_hint.s32 [%0], %1, %2;" ::"l"(p), "r"(v), "l"(pol) : "memory");
#else
    *p = v;
#endif
  }
  __device__ __forceinline__ void st(int2 *p, int2 v) const {
#if ND_TUNE_KEEP
    asm volatile("st.global.L2::cache_hint.v2.s32 [%0], {%1, %2}, %3;" ::"l"(p), "r"(v.x), "r"(v.y), "l"(pol) : "memory");
#else
    *p = v;
#endif
  }
  __device__ __forceinline__ uint32_t atom_add(uint32_t *p, uint32_t v) const {
#if ND_TUNE_KEEP
    uint32_t old;
    asm volatile("atom.global.add.L2::cache_hint.u32 %0, [%1], %2, %3;" : "=r"(old) : "l"(p), "r"(v), "l"(pol) : "memory");
    return old;
#else
    return atomicAdd(p, v);
#endif
  }
};

}  // namespace ndmem
