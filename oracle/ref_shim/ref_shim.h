/*
 * ref_shim.h -- lets the reference's app sources (their next() bodies) and its host graph
 * loader compile with g++ so that they can serve as the oracle's ground truth.
 * TEST INFRASTRUCTURE ONLY.  Nothing from the reference is copied: its files are included
 * from where they lie at build time.
 *
 * What is restated here because the reference's own definitions sit in files full of CUDA
 * runtime calls: RandNumGen::rand_int (src/rand_num_gen.cuh:117-122), utils::binarySearch
 * (src/utils.hpp:30-48) and the two enums (src/nextdoor.cu:64-72).
 */
#ifndef REF_SHIM_H
#define REF_SHIM_H

#include <algorithm>
#include <cassert>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <vector>

#define __host__
#define __device__
#define __global__
#define __forceinline__ inline

using std::max;
using std::min;

extern "C" float ndo_uniform(uint64_t seed, uint32_t sample, uint32_t step, uint32_t slot, uint32_t draw);

/* keyed draw handle standing in for cuRAND's per-thread state */
struct curandState {
  uint64_t seed;
  uint32_t sample, step, slot, draw;
};
static inline float curand_uniform(curandState *s) {
  return ndo_uniform(s->seed, s->sample, s->step, s->slot, s->draw++);
}

#include "csr.hpp" /* the reference's, from -I<reference>/src */

namespace utils {
template <typename F, typename T> inline bool binarySearch(F &array, T x, int size) {
  EdgePos_t l = 0, r = size - 1;
  while (l <= r) {
    EdgePos_t m = l + (r - l) / 2;
    if (array[m] == x) return true;
    if (array[m] < x) l = m + 1; else r = m - 1;
  }
  return false;
}
}  // namespace utils

struct RandNumGen {
  static inline EdgePos_t rand_int(curandState *state, const EdgePos_t n) {
    float ff = curand_uniform(state) * n;
    return min((EdgePos_t)ff, n - 1);
  }
};

enum SamplingType { IndividualNeighborhood, CollectiveNeighborhood };
enum OutputFormat { SampledVertices, AdjacencyMatrix };

#endif
