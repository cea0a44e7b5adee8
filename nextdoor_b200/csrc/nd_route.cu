// Routing of walkers between the ranks of a partitioned sampling job.
//
// A walker is one 64-bit word: (global sample id << 32) | vertex; all ones = the walk has ended.
// After a step every rank sorts its surviving walkers by the rank that owns their new vertex
// (contiguous vertex ranges, `bounds`) so that one all-to-all delivers them; at the end of the job
// the (sample, vertex) records of every step are routed the same way by SAMPLE id to the samples'
// home ranks.  Two kernels: count per destination (shared-memory counters, one global atomic per
// destination and CTA), then scatter into the destination's segment (warp-aggregated cursor).
// The order of walkers inside a segment is irrelevant: every draw is keyed by the sample id.
//
// The reference has no such step: its multi-GPU path replicates the graph (src/nextdoor.cu:1893-1911)
// and its partitioner (src/graph_partitioner.cuh:1-173) only feeds a stub (src/csr.hpp:371-374).
#include "nd_common.cuh"

namespace {

constexpr int RTHREADS = 256;
constexpr int MAX_PARTS = 1024;
constexpr unsigned long long DEAD = ~0ull;

__device__ __forceinline__ int route_dest(unsigned long long wk, int by_sample, const int64_t *__restrict__ bounds, int parts) {
  const int64_t key = by_sample ? (int64_t)(wk >> 32) : (int64_t)(uint32_t)wk;
  int lo = 0, hi = parts;  // last part with bounds[part] <= key
  while (hi - lo > 1) {
    const int mid = (lo + hi) >> 1;
    if (bounds[mid] <= key) lo = mid; else hi = mid;
  }
  return lo;
}

__global__ void __launch_bounds__(RTHREADS)
route_count_kernel(int64_t n, const unsigned long long *__restrict__ wk, int by_sample, const int64_t *__restrict__ bounds,
                   int parts, unsigned long long *__restrict__ counts) {
  extern __shared__ unsigned int sh_cnt[];
  for (int p = threadIdx.x; p < parts; p += RTHREADS) sh_cnt[p] = 0u;
  __syncthreads();
  for (int64_t i = blockIdx.x * (int64_t)RTHREADS + threadIdx.x; i < n; i += (int64_t)gridDim.x * RTHREADS) {
    const unsigned long long x = wk[i];
    if (x != DEAD) atomicAdd(&sh_cnt[route_dest(x, by_sample, bounds, parts)], 1u);
  }
  __syncthreads();
  for (int p = threadIdx.x; p < parts; p += RTHREADS)
    if (sh_cnt[p]) atomicAdd(&counts[p], (unsigned long long)sh_cnt[p]);
}

__global__ void __launch_bounds__(RTHREADS)
route_scatter_kernel(int64_t n, const unsigned long long *__restrict__ wk, int by_sample, const int64_t *__restrict__ bounds,
                     int parts, const unsigned long long *__restrict__ counts, unsigned long long *__restrict__ cursor,
                     unsigned long long *__restrict__ out) {
  extern __shared__ unsigned long long sh_start[];  // first slot of every destination's segment
  if (threadIdx.x == 0) {
    unsigned long long run = 0;
    for (int p = 0; p < parts; p++) { sh_start[p] = run; run += counts[p]; }
  }
  __syncthreads();
  const int lane = threadIdx.x & 31;
  const int64_t stride = (int64_t)gridDim.x * RTHREADS;
  for (int64_t i0 = blockIdx.x * (int64_t)RTHREADS; i0 < n; i0 += stride) {  // whole warps stay in the loop
    const int64_t i = i0 + threadIdx.x;
    const unsigned long long x = i < n ? wk[i] : DEAD;
    const int dest = x != DEAD ? route_dest(x, by_sample, bounds, parts) : -1;
    const unsigned peers = __match_any_sync(0xffffffffu, dest);
    if (dest >= 0) {
      const int leader = __ffs(peers) - 1;
      unsigned long long base = 0;
      if (lane == leader) base = atomicAdd(&cursor[dest], (unsigned long long)__popc(peers));
      base = __shfl_sync(peers, base, leader);
      out[sh_start[dest] + base + __popc(peers & ((1u << lane) - 1u))] = x;
    }
  }
}

// records (sample << 32 | vertex) of one step -> the step's column of the home rank's sample rows
__global__ void __launch_bounds__(RTHREADS)
records_store_kernel(int64_t n, const unsigned long long *__restrict__ rec, int step, int64_t first_sample, int64_t count,
                     int steps, int32_t *__restrict__ out) {
  for (int64_t i = blockIdx.x * (int64_t)RTHREADS + threadIdx.x; i < n; i += (int64_t)gridDim.x * RTHREADS) {
    const unsigned long long x = rec[i];
    if (x == DEAD) continue;
    const int64_t s = (int64_t)(x >> 32) - first_sample;
    if (s >= 0 && s < count) out[s * steps + step] = (int32_t)(uint32_t)x;
  }
}

}  // namespace

extern "C" {

int nd_records_store(int device, int64_t n, const uint64_t *d_records, int step, int64_t first_sample, int64_t count,
                     int steps, int32_t *d_out, void *stream) {
  ND_REQUIRE(n >= 0 && step >= 0 && step < steps && count >= 0 && (n == 0 || (d_records && d_out)), ND_ERR_ARG,
             "nd_records_store: bad argument");
  ND_CUDA(cudaSetDevice(device));
  if (n == 0) return ND_OK;
  NdDeviceInfo dev;
  ND_TRY(nd_device_info(device, &dev));
  const int64_t blocks = (n + RTHREADS - 1) / RTHREADS;
  const int grid = (int)(blocks < (int64_t)dev.sms * 8 ? blocks : (int64_t)dev.sms * 8);
  records_store_kernel<<<grid, RTHREADS, 0, (cudaStream_t)stream>>>(n, (const unsigned long long *)d_records, step, first_sample,
                                                                    count, steps, d_out);
  nd_count_launches(1);
  ND_CUDA(cudaGetLastError());
  return ND_OK;
}


int nd_route_count(int device, int64_t n, const uint64_t *d_walkers, int by_sample, const int64_t *d_bounds, int parts,
                   uint64_t *d_counts, void *stream) {
  ND_REQUIRE(n >= 0 && parts >= 1 && parts <= MAX_PARTS && d_bounds && d_counts && (n == 0 || d_walkers), ND_ERR_ARG,
             "nd_route_count: bad argument");
  ND_CUDA(cudaSetDevice(device));
  cudaStream_t st = (cudaStream_t)stream;
  ND_CUDA(cudaMemsetAsync(d_counts, 0, sizeof(uint64_t) * (size_t)parts, st));
  if (n == 0) return ND_OK;
  NdDeviceInfo dev;
  ND_TRY(nd_device_info(device, &dev));
  const int64_t blocks = (n + RTHREADS - 1) / RTHREADS;
  const int grid = (int)(blocks < (int64_t)dev.sms * 8 ? blocks : (int64_t)dev.sms * 8);
  route_count_kernel<<<grid, RTHREADS, sizeof(unsigned int) * parts, st>>>(n, (const unsigned long long *)d_walkers, by_sample,
                                                                          d_bounds, parts, (unsigned long long *)d_counts);
  nd_count_launches(1);
  ND_CUDA(cudaGetLastError());
  return ND_OK;
}

int nd_route_scatter(int device, int64_t n, const uint64_t *d_walkers, int by_sample, const int64_t *d_bounds, int parts,
                     const uint64_t *d_counts, uint64_t *d_cursor, uint64_t *d_out, void *stream) {
  ND_REQUIRE(n >= 0 && parts >= 1 && parts <= MAX_PARTS && d_bounds && d_counts && d_cursor && (n == 0 || (d_walkers && d_out)),
             ND_ERR_ARG, "nd_route_scatter: bad argument");
  ND_CUDA(cudaSetDevice(device));
  cudaStream_t st = (cudaStream_t)stream;
  ND_CUDA(cudaMemsetAsync(d_cursor, 0, sizeof(uint64_t) * (size_t)parts, st));
  if (n == 0) return ND_OK;
  NdDeviceInfo dev;
  ND_TRY(nd_device_info(device, &dev));
  const int64_t blocks = (n + RTHREADS - 1) / RTHREADS;
  const int grid = (int)(blocks < (int64_t)dev.sms * 8 ? blocks : (int64_t)dev.sms * 8);
  route_scatter_kernel<<<grid, RTHREADS, sizeof(unsigned long long) * parts, st>>>(
      n, (const unsigned long long *)d_walkers, by_sample, d_bounds, parts, (const unsigned long long *)d_counts,
      (unsigned long long *)d_cursor, (unsigned long long *)d_out);
  nd_count_launches(1);
  ND_CUDA(cudaGetLastError());
  return ND_OK;
}

}  // extern "C"
