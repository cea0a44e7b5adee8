// nd_invert_map_static: the map inversion for callers that must not allocate device memory.
//
// Who they are: a sampler that runs beside a training job in one process.  There, cudaMalloc and
// cudaFree are not just slow, they synchronise the whole device, so every call of the ordinary
// nd_invert_map (which allocates its histograms and frees them again) would stall the training
// streams; and once the framework's caching allocator has taken nearly all of HBM for itself, a
// raw cudaMalloc of a few MB can simply fail.  This entry point therefore keeps its scratch in a
// fixed array that is part of the loaded library image.
//
// Cost and limits: the array below (about 2 MB) is resident on every GPU that loads the library,
// until the process exits.  At most ND_STATIC_MAX_PAIRS pairs per call.  All calls on a device
// share the one array: a call clears the counters it needs before use, and two calls that overlap
// on the GPU (different streams or threads) race on it -- run them one after the other.
// nd_invert_map_static_on takes the stream to work on: everything is enqueued there with
// asynchronous copies and only that stream is waited for, so the training job's other streams
// are not held up (the legacy default stream, which nd_invert_map_static uses, synchronises with
// every blocking stream of the device -- prefer a non-blocking stream of your own).
//
// Set-up: in host code the name of a __device__ array is only a host-side stand-in, not an
// address a kernel may dereference.  The device address is looked up once per device with
// cudaGetSymbolAddress (with that device current) on the first call made for that device, which
// should therefore come before any stream capture begins.
#include <mutex>

#include "nd_common.cuh"

namespace {

constexpr int64_t MAX_PAIRS = (int64_t)1 << 20;
constexpr int MAX_BINS = 1024;                       // widest digit a plan over <= 4M pairs picks
constexpr int64_t MAX_TILES = MAX_PAIRS / 2048;      // radix tile = 2048 pairs
constexpr size_t HIST_WORDS = (size_t)MAX_BINS * MAX_TILES;
constexpr size_t GHIST_WORDS = (size_t)8 * MAX_BINS;
constexpr size_t SCRATCH_WORDS = HIST_WORDS + GHIST_WORDS + 64;  // + element counts

static __device__ __align__(256) uint32_t g_static_scratch[SCRATCH_WORDS];

constexpr int MAX_DEVICES = 64;
std::mutex g_mu;
uint32_t *g_scratch_ptr[MAX_DEVICES] = {nullptr};

// device address of the array on `device` (which must be current); looked up once per device
int scratch_for(int device, uint32_t **out) {
  std::lock_guard<std::mutex> lock(g_mu);
  if (!g_scratch_ptr[device]) {
    void *p = nullptr;
    ND_CUDA(cudaGetSymbolAddress(&p, g_static_scratch));
    g_scratch_ptr[device] = (uint32_t *)p;
  }
  *out = g_scratch_ptr[device];
  return ND_OK;
}

}  // namespace

extern "C" {

int64_t nd_static_max_pairs(void) { return MAX_PAIRS; }

int nd_invert_map_static_on(int device, void *stream, int64_t n, int32_t *keys_in, int32_t *vals_in, int32_t invalid,
                            int32_t *keys_out, int32_t *vals_out, int64_t *n_live_out) {
  ND_REQUIRE(n >= 0 && invalid >= 1, ND_ERR_ARG, "nd_invert_map_static: bad size or invalid id");
  ND_REQUIRE(n <= MAX_PAIRS, ND_ERR_RANGE,
             "nd_invert_map_static: %lld pairs exceed the fixed scratch (limit %lld); use nd_invert_map",
             (long long)n, (long long)MAX_PAIRS);
  ND_REQUIRE(n == 0 || (keys_in && vals_in && keys_out && vals_out), ND_ERR_ARG, "nd_invert_map_static: null pointer");
  ND_REQUIRE(device >= 0 && device < MAX_DEVICES, ND_ERR_ARG, "nd_invert_map_static: device %d out of range", device);
  ND_CUDA(cudaSetDevice(device));
  if (n == 0) { if (n_live_out) *n_live_out = 0; return ND_OK; }
  cudaStream_t st = (cudaStream_t)stream;
  NdDeviceInfo dev;
  ND_TRY(nd_device_info(device, &dev));
  uint32_t *base = nullptr;
  ND_TRY(scratch_for(device, &base));
  // carve the array; the plan's tile count is pinned to the array's so that the row stride of
  // the histogram matrix is the same whatever n is
  NdRadixScratch scr;
  scr.tile_hist = base;
  scr.ghist = base + HIST_WORDS;
  scr.cap_bins = MAX_BINS;
  scr.plan = nd_radix_plan(nd_bit_length((uint32_t)(invalid > 1 ? invalid - 1 : 1)), MAX_PAIRS);
  int32_t *d_n = (int32_t *)(base + HIST_WORDS + GHIST_WORDS);
  // the array keeps what the last call left: the digit counters must start at zero
  ND_CUDA(cudaMemsetAsync(scr.ghist, 0, sizeof(uint32_t) * GHIST_WORDS, st));
  const int32_t n32[2] = {(int32_t)n, 0};
  ND_CUDA(cudaMemcpyAsync(d_n, n32, sizeof(n32), cudaMemcpyHostToDevice, st));  // pageable source: staged before the call returns
  NdSortArrays arr;
  arr.nwords = 2;
  arr.a[0] = (uint32_t *)keys_in; arr.a[1] = (uint32_t *)vals_in; arr.a[2] = nullptr;
  arr.b[0] = (uint32_t *)keys_out; arr.b[1] = (uint32_t *)vals_out; arr.b[2] = nullptr;
  bool in_b = false;
  ND_TRY(nd_radix_sort(dev, st, &scr, scr.plan, arr, 0, d_n, d_n + 1, true, (uint32_t)invalid, false, &in_b));
  if (!in_b) {  // an even number of passes left the result in the input arrays: copy all n slots, the tail is unused
    ND_CUDA(cudaMemcpyAsync(keys_out, keys_in, sizeof(int32_t) * (size_t)n, cudaMemcpyDeviceToDevice, st));
    ND_CUDA(cudaMemcpyAsync(vals_out, vals_in, sizeof(int32_t) * (size_t)n, cudaMemcpyDeviceToDevice, st));
  }
  int32_t live = 0;
  ND_CUDA(cudaMemcpyAsync(&live, d_n + 1, sizeof(int32_t), cudaMemcpyDeviceToHost, st));
  ND_CUDA(cudaStreamSynchronize(st));  // this stream only: other streams of the device keep running
  if (n_live_out) *n_live_out = live;
  return ND_OK;
}

int nd_invert_map_static(int device, int64_t n, int32_t *keys_in, int32_t *vals_in, int32_t invalid,
                         int32_t *keys_out, int32_t *vals_out, int64_t *n_live_out) {
  return nd_invert_map_static_on(device, nullptr, n, keys_in, vals_in, invalid, keys_out, vals_out, n_live_out);
}

}  // extern "C"
