// Measurement aid of bench.py, not part of the sampling library: the rate (gathers per second)
// at which this GPU serves independent random 4-byte gathers from an array of a given footprint.
// A walk step is a few such gathers per (transit, sample) pair, so this rate -- one
// implementation's, not a hardware bound -- is reported beside the HBM roofline of the next()
// kernels.  Built into libnd_bench_probe.so by __graft_entry__.build().
#include <cuda_runtime.h>
#include <stdint.h>

namespace {
// one load per thread and loop trip, the index a hash of the trip
__global__ void random_gather_kernel(const int32_t *__restrict__ a, uint64_t words, int64_t total, int32_t *sink, uint32_t salt) {
  int32_t acc = 0;
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    uint32_t x = (uint32_t)i ^ (salt * 0x9e3779b9u), y = (uint32_t)(i >> 32) + salt;
    x ^= x >> 16; x *= 0x7feb352du; x ^= x >> 15; x *= 0x846ca68bu; x ^= x >> 16;
    y = (y ^ x) * 0x85ebca6bu; y ^= y >> 13;
    const uint64_t idx = (((uint64_t)y << 32) | x) % words;
    acc ^= __ldg(a + idx);
  }
  if (acc == 0x5a5a5a5a) *sink = acc;  // never true for the fill pattern: keeps the loads alive
}
}  // namespace

// returns 0 and the rate, or a cudaError_t value (1 = bad argument)
extern "C" int nd_bench_random_gather(int device, int64_t footprint_bytes, int64_t n_gathers, int repeats,
                                      double *gathers_per_second) {
  if (footprint_bytes < 4 || n_gathers <= 0 || repeats <= 0 || !gathers_per_second) return 1;
  cudaError_t e = cudaSetDevice(device);
  if (e != cudaSuccess) return (int)e;
  int sms = 0;
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
  const uint64_t words = (uint64_t)footprint_bytes / 4;
  int32_t *a = nullptr, *sink = nullptr;
  if ((e = cudaMalloc(&a, words * 4)) != cudaSuccess) return (int)e;
  if ((e = cudaMalloc(&sink, 4)) != cudaSuccess) { cudaFree(a); return (int)e; }
  cudaMemset(a, 1, words * 4);
  cudaEvent_t e0, e1;
  cudaEventCreate(&e0);
  cudaEventCreate(&e1);
  const int64_t blocks = (n_gathers + 255) / 256;
  const int grid = (int)(blocks < (int64_t)sms * 8 ? blocks : (int64_t)sms * 8);
  for (int r = 0; r < 2; r++) random_gather_kernel<<<grid, 256>>>(a, words, n_gathers, sink, (uint32_t)r);
  cudaEventRecord(e0);
  for (int r = 0; r < repeats; r++) random_gather_kernel<<<grid, 256>>>(a, words, n_gathers, sink, (uint32_t)(r + 2));
  cudaEventRecord(e1);
  e = cudaEventSynchronize(e1);
  float ms = 0.f;
  cudaEventElapsedTime(&ms, e0, e1);
  cudaEventDestroy(e0);
  cudaEventDestroy(e1);
  cudaFree(a);
  cudaFree(sink);
  if (e != cudaSuccess) return (int)e;
  if (!(ms > 0.f)) return 1;
  *gathers_per_second = (double)n_gathers * repeats / ((double)ms * 1e-3);
  return 0;
}
