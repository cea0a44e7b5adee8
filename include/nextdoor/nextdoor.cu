// nextdoor.cu -- source-compatibility layer: lets an application written against NextDoor's App
// struct contract (steps / stepSize / next / samplingType / outputFormat / numSamples /
// initialSample / initialSampleSize / hasExplicitTransits / stepTransits / initializeSample,
// see the reference's example/uniformRandWalk.cu:15-93) compile unchanged and run on
// libnextdoor_b200.so.  The application file keeps its `#include "nextdoor.cu"`; put this
// directory first on the include path and link the library:
//
//   nvcc -gencode arch=compute_100a,code=sm_100a -fmad=false -I include/nextdoor -I include app.cu \
//        -L nextdoor_b200 -lnextdoor_b200
//
// What comes from where: graph loading, CSR construction and the map inversion are calls into the
// library's C ABI (nextdoor_b200.h); the kernels that call the user's next() are templates here,
// because the App type is only known in the user's translation unit.  next() receives a keyed
// counter-based generator through the names `curandState` / `curand_uniform`: draws depend on
// (seed, sample, step, slot) only, never on the thread that happens to run them, so the
// sample-parallel and transit-parallel paths produce identical samples.
// Output layout: finalSamples[s*finalSampleSize + prefix_k + parent*stepSize(k) + j]; empty slots
// hold INVALID_VERTEX = number of vertices (the reference's convention, src/nextdoor.cu:1993).
#ifndef NEXTDOOR_B200_COMPAT_NEXTDOOR_CU
#define NEXTDOOR_B200_COMPAT_NEXTDOOR_CU

#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include <iostream>
#include <sstream>
#include <string>
#include <vector>
#include <assert.h>

#include "nextdoor_b200.h"

typedef int32_t VertexID;
typedef int32_t EdgePos_t;
typedef VertexID VertexID_t;

const int ALL_NEIGHBORS = -1;

enum SamplingType { IndividualNeighborhood, CollectiveNeighborhood };
enum OutputFormat { SampledVertices, AdjacencyMatrix };

// ------------------------------------------------------------------ keyed generator behind the cuRAND names

struct nd_rng {
  uint64_t seed;
  uint32_t sample, step, slot, draw;
  uint32_t lanes[4];
};

__host__ __device__ inline void nd_rng_block(nd_rng *r) {
  uint32_t c0 = r->sample, c1 = r->step, c2 = r->slot, c3 = r->draw >> 2;
  uint32_t k0 = (uint32_t)r->seed, k1 = (uint32_t)(r->seed >> 32);
  for (int round = 0; round < 10; round++) {
    const uint64_t p0 = (uint64_t)0xD2511F53u * c0, p1 = (uint64_t)0xCD9E8D57u * c2;
    const uint32_t n0 = (uint32_t)(p1 >> 32) ^ c1 ^ k0, n2 = (uint32_t)(p0 >> 32) ^ c3 ^ k1;
    c1 = (uint32_t)p1; c3 = (uint32_t)p0; c0 = n0; c2 = n2;
    k0 += 0x9E3779B9u; k1 += 0xBB67AE85u;
  }
  r->lanes[0] = c0; r->lanes[1] = c1; r->lanes[2] = c2; r->lanes[3] = c3;
}

// (0,1], x * 2^-32 + 2^-33 in fp32: the mapping of cuRAND's curand_uniform
__host__ __device__ inline float nd_uniform(nd_rng *r) {
  if ((r->draw & 3u) == 0u) nd_rng_block(r);
  const uint32_t x = r->lanes[r->draw & 3u];
  r->draw++;
#ifdef __CUDA_ARCH__
  return __fadd_rn(__fmul_rn(__uint2float_rn(x), 2.3283064365386963e-10f), 1.1641532182693481e-10f);
#else
  volatile float f = (float)x * 2.3283064365386963e-10f;
  return f + 1.1641532182693481e-10f;
#endif
}

#define curandState nd_rng
#define curand_uniform nd_uniform

struct RandNumGen {
  // min((int)(u*n), n-1) with a lone fp32 multiply (the reference's rand_int, src/rand_num_gen.cuh:117-122)
  __host__ __device__ static inline EdgePos_t rand_int(curandState *state, const EdgePos_t n) {
#ifdef __CUDA_ARCH__
    const EdgePos_t id = __float2int_rz(__fmul_rn(curand_uniform(state), __int2float_rn(n)));
#else
    volatile float ff = curand_uniform(state) * (float)n;
    const EdgePos_t id = (EdgePos_t)ff;
#endif
    return id < n - 1 ? id : n - 1;
  }
};

namespace utils {
template <typename F, typename T>
__host__ __device__ inline bool binarySearch(F &array, T x, int size) {
  int lo = 0, hi = size - 1;
  while (lo <= hi) {
    const int mid = lo + (hi - lo) / 2;
    if (array[mid] == x) return true;
    if (array[mid] < x) lo = mid + 1; else hi = mid - 1;
  }
  return false;
}
// is_cuda_error / printCudaMemInfo (src/utils.hpp:16-30, 352-357)
inline bool is_cuda_error(cudaError_t status, int line) {
  if (status != cudaSuccess) {
    printf("CUDA error at line %d: %s\n", line, cudaGetErrorString(status));
    return true;
  }
  return false;
}
inline void printCudaMemInfo() {
  size_t free_b = 0, total_b = 0;
  if (cudaMemGetInfo(&free_b, &total_b) == cudaSuccess) printf("free memory %ld\n", (long)free_b);
}
}  // namespace utils
using namespace utils;  // src/nextdoor.cu:40

#ifndef DIVUP
#define DIVUP(x, y) (((x) + ((y) - 1)) / (y))  // src/utils.hpp:12
#endif
#ifndef CHK_CU
#define CHK_CU(x) if (utils::is_cuda_error((x), __LINE__) == true) { assert(false); }  // src/utils.hpp:16
#endif

// ------------------------------------------------------------------ graph types the App bodies see

// Host CSR: what numSamples / initialSample / initializeSample receive.
class CSR {
 public:
  typedef VertexID Edge;
  std::vector<int32_t> row_ptr;
  std::vector<Edge> edges;
  std::vector<float> weights;
  std::vector<float> max_weights;
  int n_vertices = 0;
  EdgePos_t n_edges = 0;
  __host__ VertexID get_n_vertices() const { return n_vertices; }
  __host__ int get_n_edges() const { return n_edges; }
  __host__ EdgePos_t n_edges_for_vertex(VertexID v) const { return row_ptr[v + 1] - row_ptr[v]; }
  __host__ EdgePos_t get_start_edge_idx(VertexID v) const { return row_ptr[v]; }
  __host__ EdgePos_t get_end_edge_idx(VertexID v) const { return row_ptr[v + 1] > row_ptr[v] ? row_ptr[v + 1] - 1 : -1; }
  __host__ const Edge *get_edges() const { return edges.data(); }
  __host__ const float *get_weights() const { return weights.data(); }
  __host__ bool has_vertex(VertexID v) const { return v >= 0 && v < n_vertices; }
  __host__ bool has_edge(VertexID u, VertexID v) const {
    for (EdgePos_t e = row_ptr[u]; e < row_ptr[u + 1]; e++) if (edges[e] == v) return true;
    return false;
  }
};

// Device view handed to next(): the whole graph is one partition (replica per GPU).
class CSRPartition {
 public:
  VertexID first_vertex_id, last_vertex_id;
  EdgePos_t first_edge_idx, last_edge_idx;
  const int32_t *row_ptr;
  const CSR::Edge *edges;
  const float *weights;
  const float *max_weights;
  __host__ __device__ VertexID get_n_vertices() const { return last_vertex_id - first_vertex_id + 1; }
  __host__ __device__ EdgePos_t get_n_edges() const { return last_edge_idx - first_edge_idx + 1; }
  __host__ __device__ bool has_vertex(int v) const { return v >= first_vertex_id && v <= last_vertex_id; }
  __host__ __device__ EdgePos_t get_start_edge_idx(int v) const { return row_ptr[v]; }
  __host__ __device__ EdgePos_t get_end_edge_idx(int v) const { return row_ptr[v + 1] > row_ptr[v] ? row_ptr[v + 1] - 1 : -1; }
  __host__ __device__ EdgePos_t get_n_edges_for_vertex(VertexID v) const { return row_ptr[v + 1] - row_ptr[v]; }
  __host__ __device__ float get_max_weight(int v) const { return max_weights[v]; }
  __host__ __device__ CSR::Edge get_edge(EdgePos_t i) const { return edges[i]; }
  __host__ __device__ float get_weight(EdgePos_t i) const { return weights[i]; }
  __host__ __device__ const CSR::Edge *get_edges() const { return edges; }
  __host__ __device__ const float *get_weights() const { return weights; }
  __host__ __device__ const CSR::Edge *get_edges(VertexID v) const { return edges + row_ptr[v]; }
  __host__ __device__ const float *get_weights(VertexID v) const { return weights + row_ptr[v]; }
  __host__ __device__ VertexID get_invalid_vertex() const { return get_n_vertices() + 1; }
  __host__ __device__ bool has_edge(VertexID s, VertexID d) const {
    for (EdgePos_t e = row_ptr[s]; e < row_ptr[s + 1]; e++) if (edges[e] == d) return true;
    return false;
  }
  __host__ __device__ bool has_edge_logn(VertexID s, VertexID d) const {
    EdgePos_t lo = row_ptr[s], hi = row_ptr[s + 1] - 1;
    while (lo <= hi) {
      const EdgePos_t mid = lo + (hi - lo) / 2;
      const CSR::Edge e = edges[mid];
      if (e == d) return true;
      if (e < d) lo = mid + 1; else hi = mid - 1;
    }
    return false;
  }
};

struct GPUCSRPartition {
  CSRPartition *device_csr;   // unused: the view travels to the kernels by value
  const int32_t *device_row_ptr;
  const CSR::Edge *device_edge_array;
  const float *device_weights_array;
  nd_graph *handle;
  CSRPartition view;
};

// Stand-in for the reference's host Graph class (the loader runs on the device here).
class Graph {
 public:
  int n_vertices = 0;
  int n_edges = 0;
  int get_n_edges() const { return n_edges; }
  struct VertexList { size_t n; size_t size() const { return n; } };
  VertexList get_vertices() const { return VertexList{(size_t)n_vertices}; }
};

// ------------------------------------------------------------------ NextDoorData (src/libNextDoor.hpp:13-37)

template <class SampleType, typename App>
struct NextDoorData {
  CSR *csr = nullptr;
  std::vector<SampleType> samples;
  std::vector<VertexID_t> hFinalSamples;
  std::vector<VertexID_t> initialContents;
  std::vector<VertexID_t> initialTransitToSampleValues;
  std::vector<int> devices;
  // per device
  std::vector<SampleType *> dOutputSamples;
  std::vector<VertexID_t *> dFinalSamples;
  std::vector<VertexID_t *> dInitialSamples;
  std::vector<VertexID_t *> dMapKeys[2];
  std::vector<VertexID_t *> dMapVals[2];
  std::vector<cudaStream_t> streams;       // one per device: the devices' step loops run side by side
  std::vector<nd_inverter *> inverters;    // map inversion with its scratch allocated once per device
  int INVALID_VERTEX = 0;
  int maxBits = 0;
  std::vector<GPUCSRPartition> gpuCSRPartitions;
  const char *graphFile = nullptr;
};

// run seed of the keyed generator; NEXTDOOR_SEED in the environment overrides it
inline uint64_t &nextdoor_seed() {
  static uint64_t seed = getenv("NEXTDOOR_SEED") ? strtoull(getenv("NEXTDOOR_SEED"), nullptr, 10) : 0;
  return seed;
}

#define NDC_CHECK(call)                                                                    \
  do {                                                                                     \
    cudaError_t e__ = (call);                                                              \
    if (e__ != cudaSuccess) {                                                              \
      printf("%s failed: %s (%s:%d)\n", #call, cudaGetErrorString(e__), __FILE__, __LINE__); \
      return false;                                                                        \
    }                                                                                      \
  } while (0)

// ------------------------------------------------------------------ sizes derived from the App

template <typename App>
int getFinalSampleSize() {
  size_t total = 0, n = 1;
  for (int step = 0; step < App().steps(); step++) {
    if (App().samplingType() == CollectiveNeighborhood) n = App().stepSize(step);
    else n *= App().stepSize(step);
    total += n;
  }
  return (int)total;
}

namespace ndc {

template <typename App>
__host__ __device__ inline int pairs_per_sample(int step, int isz = 1) {  // transits of a sample entering `step`
  if (App().samplingType() == CollectiveNeighborhood) return 1;
  int n = isz;  // individual-neighbourhood apps may start from several vertices (MVS, ClusterGCN: 32)
  for (int k = 0; k < step; k++) n *= App().stepSize(k);
  return n;
}
template <typename App>
__host__ __device__ inline int hop_size(int step) {  // slots hop `step` has in a sample's row (getFinalSampleSize)
  int n = 1;
  for (int k = 0; k <= step; k++) n *= App().stepSize(k);
  return n;
}
template <typename App>
__host__ __device__ inline int prefix_of(int step) {  // offset of hop `step` inside a sample's row
  int off = 0, n = 1;
  for (int k = 0; k < step; k++) {
    if (App().samplingType() == CollectiveNeighborhood) n = App().stepSize(k); else n *= App().stepSize(k);
    off += n;
  }
  return off;
}

// One thread per (pair, slot) -- the shape of the reference's samplingKernel / sampleParallelKernel
// (src/nextdoor.cu:212-336, 1348-1518).  FROM_MAP: pair i of the transit-sorted map.
template <class SampleType, typename App, bool FROM_MAP>
__global__ void step_kernel(CSRPartition part, int step, uint64_t seed, int64_t first_sample, int64_t n_pairs,
                            const int32_t *d_n_pairs, const VertexID_t *in_key, const VertexID_t *in_val, const VertexID_t *initial,
                            SampleType *samples, VertexID_t *out, int fs, VertexID_t *mkey, VertexID_t *mval,
                            bool write_map, const VertexID_t *explicit_prev, int isz) {
  const int f = App().stepSize(step);
  const int64_t tid = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
  if (d_n_pairs) n_pairs = *d_n_pairs;  // live pairs of the sorted map, left on the device by the inversion
  if (tid >= n_pairs * f) return;
  const int64_t i = tid / f;
  const int j = (int)(tid - i * f);
  const int32_t INV = part.get_n_vertices();
  const int n_prev = pairs_per_sample<App>(step, isz);
  VertexID_t q, transit;
  if (FROM_MAP) { transit = in_key[i]; q = in_val[i]; }
  else {
    q = (VertexID_t)i;
    const int64_t s = q / n_prev;
    // apps with explicit transits walk from what stepTransits returned at the previous step
    // (kept per pair id), the others from the vertex sampled at the previous hop
    if (step == 0) transit = initial[q];  // q = s * isz + index inside the initial sample
    else if (explicit_prev) transit = explicit_prev[q];
    else transit = out[s * fs + prefix_of<App>(step - 1) + (q - s * n_prev)];
  }
  const int64_t s = q / n_prev;
  const int parent = (int)(q - s * n_prev);
  const int slot = parent * f + j;
  VertexID_t nbr = -1;
  nd_rng rng;
  rng.seed = seed; rng.sample = (uint32_t)(first_sample + s); rng.step = (uint32_t)step; rng.slot = (uint32_t)slot; rng.draw = 0;
  if (transit >= 0 && transit < INV) {
    const EdgePos_t n = part.get_n_edges_for_vertex(transit);
    if (n != 0) {  // next() only runs on transits with edges (src/nextdoor.cu:255)
      const CSR::Edge *edges = part.get_edges(transit);
      const float *weights = part.get_weights(transit);
      nbr = App().template next<SampleType, const CSR::Edge *, const float *>(
          step, &part, &transit, (VertexID)(first_sample + s), &samples[s], part.get_max_weight(transit), edges, weights, n, j, &rng);
    }
  }
  // with several initial vertices a hop has more (pair, slot) combinations than slots in the row
  // (the reference sizes the row without them, src/nextdoor.cu:1914-1929): those are not stored
  if (slot < hop_size<App>(step)) out[s * fs + prefix_of<App>(step) + slot] = nbr != -1 ? nbr : INV;
  if (write_map) {  // apps with explicit transits get their keys from transits_kernel instead
    const int64_t c = (int64_t)q * f + j;
    mkey[c] = nbr != -1 ? nbr : INV;
    mval[c] = (VertexID_t)c;
  }
}

// Explicit transits (hasExplicitTransits / stepTransits, src/nextdoor.cu:1285-1323): the transit of
// every (sample, index) pair of the next step, computed by a kernel of its own AFTER the step's
// next() calls have all finished -- apps such as ClusterGCN read in stepTransits() what next()
// accumulated in the sample.  The draws of stepTransits come from the pair's keyed stream at an
// offset no next() reaches.
constexpr uint32_t NDC_TRANSIT_DRAW_BASE = 1u << 16;
template <class SampleType, typename App>
__global__ void transits_kernel(int next_step, uint64_t seed, int64_t first_sample, int64_t total, int per_sample,
                                SampleType *samples, VertexID_t *mkey, VertexID_t *mval, VertexID_t INV) {
  const int64_t c = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
  if (c >= total) return;
  const int64_t s = c / per_sample;
  const int slot = (int)(c - s * per_sample);
  nd_rng rng;
  rng.seed = seed; rng.sample = (uint32_t)(first_sample + s); rng.step = (uint32_t)(next_step - 1); rng.slot = (uint32_t)slot;
  rng.draw = NDC_TRANSIT_DRAW_BASE;
  const VertexID_t key = App().template stepTransits<SampleType>(next_step, (VertexID_t)(first_sample + s), samples[s], slot, &rng);
  mkey[c] = key != -1 ? key : INV;
  mval[c] = (VertexID_t)c;
}

// Collective apps: one thread per (sample, slot); the transits are the sample's previous layer
// (src/nextdoor.cu:1402-1411) and next() gets the summed degree, no edge array.
template <class SampleType, typename App>
__global__ void collective_kernel(CSRPartition part, int step, uint64_t seed, int64_t first_sample, int64_t S,
                                  const VertexID_t *initial, SampleType *samples, VertexID_t *out, int fs, int isz) {
  const int f = App().stepSize(step);
  const int64_t tid = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
  if (tid >= S * f) return;
  const int64_t s = tid / f;
  const int j = (int)(tid - s * f);
  const int32_t INV = part.get_n_vertices();
  const VertexID_t *transits = step == 0 ? initial + s * isz : out + s * fs + prefix_of<App>(step - 1);
  const int ntr = step == 0 ? isz : App().stepSize(step - 1);
  VertexID_t nbr = INV;
  if (transits[0] != INV && transits[0] != -1) {
    EdgePos_t total = 0;
    for (int i = 0; i < ntr; i++) if (part.has_vertex(transits[i])) total += part.get_n_edges_for_vertex(transits[i]);
    nd_rng rng;
    rng.seed = seed; rng.sample = (uint32_t)(first_sample + s); rng.step = (uint32_t)step; rng.slot = (uint32_t)j; rng.draw = 0;
    const CSR::Edge *edges = nullptr;
    const float *weights = nullptr;
    nbr = App().template next<SampleType, const CSR::Edge *, const float *>(
        step, &part, transits, (VertexID)(first_sample + s), &samples[s], 0.0f, edges, weights, total, j, &rng);
    if (nbr == -1) nbr = INV;
  }
  out[s * fs + prefix_of<App>(step) + j] = nbr;
}

template <typename T>
__global__ void fill_kernel(T *p, int64_t n, T v) {
  const int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
  if (i < n) p[i] = v;
}

inline int64_t part_start(int64_t total, int idx, int parts) { int64_t f = 0, c = 0; nd_shard_range(total, idx, parts, &f, &c); return f; }
inline int64_t part_size(int64_t total, int idx, int parts) { int64_t f = 0, c = 0; nd_shard_range(total, idx, parts, &f, &c); return c; }

}  // namespace ndc

// ------------------------------------------------------------------ the host functions of src/libNextDoor.hpp

// loadGraph (src/nextdoor.cu:1845-1891): the file is read and turned into a CSR on GPU 0 by the
// library; the host CSR the App's host functions need is copied back from it.
inline CSR *loadGraph(Graph &graph, char *graph_file, char *graph_type, char *graph_format) {
  if (strcmp(graph_type, "edge-list") != 0 && strcmp(graph_type, "adj-list") != 0) {
    printf("Incorrect graph file type '%s'\n", graph_type);
    return nullptr;
  }
  const bool known = (strcmp(graph_type, "edge-list") == 0 && (strcmp(graph_format, "binary") == 0 || strcmp(graph_format, "text") == 0)) ||
                     (strcmp(graph_type, "adj-list") == 0 && strcmp(graph_format, "text") == 0);
  if (!known) {
    printf("graph_format '%s' not supported for graph_type '%s'\n", graph_format, graph_type);
    return nullptr;
  }
  nd_graph *g = nullptr;
  if (nd_graph_load(0, graph_file, graph_type, graph_format, &g) != ND_OK) {
    std::cout << nd_last_error() << std::endl;
    return nullptr;
  }
  int32_t V = 0; int64_t E = 0;
  nd_graph_info(g, &V, &E, nullptr, nullptr);
  CSR *csr = new CSR();
  csr->n_vertices = V; csr->n_edges = (EdgePos_t)E;
  csr->row_ptr.resize((size_t)V + 1); csr->edges.resize((size_t)E); csr->weights.resize((size_t)E); csr->max_weights.resize((size_t)V);
  nd_graph_to_host(g, csr->row_ptr.data(), csr->edges.data(), csr->weights.data(), csr->max_weights.data());
  nd_graph_destroy(g);
  graph.n_vertices = V; graph.n_edges = (int)E;
  return csr;
}

// allocNextDoorDataOnGPU (src/nextdoor.cu:1931-2086)
template <class SampleType, typename App>
bool allocNextDoorDataOnGPU(CSR *csr, NextDoorData<SampleType, App> &data) {
  data.devices.clear();
  if (const char *list = getenv("CUDA_DEVICES")) {  // e.g. "0,1,3" or "[0,1,3]" (src/nextdoor.cu:1934-1950)
    std::stringstream ss(list);
    if (ss.peek() == '[') ss.ignore();
    for (int d; ss >> d;) { data.devices.push_back(d); if (ss.peek() == ',') ss.ignore(); }
  }
  if (data.devices.empty()) data.devices = {0};
  data.csr = csr;
  data.samples.clear(); data.initialContents.clear(); data.initialTransitToSampleValues.clear();
  const EdgePos_t isz = App().initialSampleSize(csr);
  const int64_t S = App().numSamples(csr);
  if (App().samplingType() == IndividualNeighborhood && isz != 1 && App().steps() > 1 && !App().hasExplicitTransits()) {
    printf("initialSampleSize '%d' > 1 with several steps needs hasExplicitTransits() for IndividualNeighborhood apps\n", isz);
    return false;
  }
  for (int step = 0; step < App().steps(); step++)
    if (App().stepSize(step) == ALL_NEIGHBORS) { printf("stepSize ALL_NEIGHBORS is not supported\n"); return false; }
  for (int64_t s = 0; s < S; s++) {
    data.samples.push_back(App().template initializeSample<SampleType>(csr, (VertexID_t)s));
    std::vector<VertexID_t> init = App().initialSample((int)s, csr, data.samples.back());
    if ((EdgePos_t)init.size() != isz) {
      printf("initialSampleSize '%d' != initialSample(%ld).size() '%ld'\n", isz, (long)s, (long)init.size());
      return false;
    }
    for (VertexID_t v : init) { data.initialContents.push_back(v); data.initialTransitToSampleValues.push_back((VertexID_t)s); }
  }
  const int fs = getFinalSampleSize<App>();
  data.INVALID_VERTEX = csr->get_n_vertices();
  data.maxBits = 0;
  while ((data.INVALID_VERTEX >> data.maxBits) != 0) data.maxBits++;
  data.hFinalSamples.assign((size_t)fs * S, data.INVALID_VERTEX);
  size_t max_pairs = App().samplingType() == IndividualNeighborhood ? (size_t)isz : 1;  // pairs per sample at the widest step that still feeds a map
  for (int step = 0; step + 1 < App().steps(); step++) max_pairs *= App().stepSize(step);
  const int P = (int)data.devices.size();
  data.dOutputSamples.assign(P, nullptr); data.dFinalSamples.assign(P, nullptr); data.dInitialSamples.assign(P, nullptr);
  for (int b = 0; b < 2; b++) { data.dMapKeys[b].assign(P, nullptr); data.dMapVals[b].assign(P, nullptr); }
  for (int d = 0; d < P; d++) {
    NDC_CHECK(cudaSetDevice(data.devices[d]));
    const int64_t n = ndc::part_size(S, d, P), first = ndc::part_start(S, d, P);
    const size_t n1 = (size_t)(n > 0 ? n : 1);
    NDC_CHECK(cudaMalloc(&data.dInitialSamples[d], sizeof(VertexID_t) * n1 * isz));
    NDC_CHECK(cudaMemcpy(data.dInitialSamples[d], data.initialContents.data() + first * isz, sizeof(VertexID_t) * (size_t)n * isz, cudaMemcpyHostToDevice));
    NDC_CHECK(cudaMalloc(&data.dOutputSamples[d], sizeof(SampleType) * n1));
    NDC_CHECK(cudaMemcpy(data.dOutputSamples[d], data.samples.data() + first, sizeof(SampleType) * (size_t)n, cudaMemcpyHostToDevice));
    NDC_CHECK(cudaMalloc(&data.dFinalSamples[d], sizeof(VertexID_t) * n1 * fs));
    for (int b = 0; b < 2; b++) {
      NDC_CHECK(cudaMalloc(&data.dMapKeys[b][d], sizeof(VertexID_t) * n1 * max_pairs));
      NDC_CHECK(cudaMalloc(&data.dMapVals[b][d], sizeof(VertexID_t) * n1 * max_pairs));
    }
    cudaStream_t st = nullptr;
    NDC_CHECK(cudaStreamCreateWithFlags(&st, cudaStreamNonBlocking));
    data.streams.push_back(st);
    nd_inverter *inv = nullptr;
    if (nd_inverter_create(data.devices[d], (int64_t)(n1 * max_pairs), data.INVALID_VERTEX, &inv) != ND_OK) { std::cout << nd_last_error() << std::endl; return false; }
    data.inverters.push_back(inv);
  }
  std::cout << "Final Size of each sample: " << fs << std::endl;
  std::cout << "Number of Samples: " << S << std::endl;
  return true;
}

// transferCSRToGPUs (src/nextdoor.cu:1893-1911): one replica per device
template <typename NextDoorDataT>
std::vector<GPUCSRPartition> transferCSRToGPUs(NextDoorDataT &data, CSR *csr) {
  std::vector<GPUCSRPartition> parts;
  for (int dev : data.devices) {
    GPUCSRPartition p;
    memset(&p, 0, sizeof(p));
    if (nd_graph_from_csr(dev, csr->n_vertices, csr->n_edges, csr->row_ptr.data(), csr->edges.data(), csr->weights.data(),
                          csr->max_weights.data(), &p.handle) != ND_OK) {
      std::cout << nd_last_error() << std::endl;
      return parts;
    }
    const float *mw = nullptr;
    nd_graph_device_ptrs(p.handle, &p.device_row_ptr, &p.device_edge_array, &p.device_weights_array, &mw);
    p.view.first_vertex_id = 0; p.view.last_vertex_id = csr->n_vertices - 1;
    p.view.first_edge_idx = 0; p.view.last_edge_idx = csr->n_edges - 1;
    p.view.row_ptr = p.device_row_ptr; p.view.edges = p.device_edge_array; p.view.weights = p.device_weights_array; p.view.max_weights = mw;
    parts.push_back(p);
  }
  return parts;
}

namespace ndc {
// The step loop.  Every device's whole job is enqueued on that device's stream before any device is
// waited for, so the devices work side by side (the reference runs one host thread per device,
// src/nextdoor.cu:2363-2963); inside a job nothing comes back to the host: the map inversion keeps
// its scratch between steps and leaves the live count on the device, where the next step's kernel
// reads it (the reference copies counts to the host and allocates per step, :2413-2429, 2515-2567).
template <class SampleType, typename App>
bool run(CSR *csr, NextDoorData<SampleType, App> &data, bool transit_parallel) {
  const int P = (int)data.devices.size();
  if ((int)data.gpuCSRPartitions.size() != P) { printf("transferCSRToGPUs has not been called\n"); return false; }
  if ((int)data.streams.size() != P) { printf("allocNextDoorDataOnGPU has not been called\n"); return false; }
  const int64_t S = (int64_t)data.samples.size();
  const int fs = getFinalSampleSize<App>();
  const int isz = App().initialSampleSize(csr);
  const int32_t INV = data.INVALID_VERTEX;
  const bool collective = App().samplingType() == CollectiveNeighborhood;
  std::vector<VertexID_t> ids;   // pair ids of the initial map; must outlive the asynchronous copies
  if (transit_parallel && !collective) {
    int64_t longest = 0;
    for (int d = 0; d < P; d++) longest = std::max<int64_t>(longest, part_size(S, d, P) * isz);
    ids.resize((size_t)longest);
    for (int64_t i = 0; i < longest; i++) ids[(size_t)i] = (VertexID_t)i;
  }
  for (int d = 0; d < P; d++) {
    NDC_CHECK(cudaSetDevice(data.devices[d]));
    cudaStream_t st = data.streams[d];
    const int64_t n = part_size(S, d, P), first = part_start(S, d, P);
    if (n == 0) continue;
    const CSRPartition part = data.gpuCSRPartitions[d].view;
    VertexID_t *out = data.dFinalSamples[d];
    fill_kernel<VertexID_t><<<(unsigned)((n * fs + 255) / 256), 256, 0, st>>>(out, n * fs, INV);
    NDC_CHECK(cudaMemcpyAsync(data.dOutputSamples[d], data.samples.data() + first, sizeof(SampleType) * (size_t)n, cudaMemcpyHostToDevice, st));
    if (collective) {  // next() of collective apps always runs sample-parallel (src/nextdoor.cu:2900-2916)
      for (int step = 0; step < App().steps(); step++) {
        const int64_t threads = n * App().stepSize(step);
        collective_kernel<SampleType, App><<<(unsigned)((threads + 255) / 256), 256, 0, st>>>(part, step, nextdoor_seed(), first, n, data.dInitialSamples[d], data.dOutputSamples[d], out, fs, isz);
      }
      NDC_CHECK(cudaGetLastError());
      continue;
    }
    const int64_t n0 = n * isz;   // initial pairs: every vertex of every initial sample
    int cur = 0;
    const VertexID_t *in_key = nullptr, *in_val = nullptr;
    const int32_t *d_live = nullptr;   // live pairs of the sorted map (device), transit-parallel only
    if (transit_parallel) {   // initial transit -> sample map, sorted by transit
      VertexID_t *k0 = data.dMapKeys[0][d], *v0 = data.dMapVals[0][d];
      NDC_CHECK(cudaMemcpyAsync(k0, data.initialContents.data() + first * isz, sizeof(VertexID_t) * (size_t)n0, cudaMemcpyHostToDevice, st));
      NDC_CHECK(cudaMemcpyAsync(v0, ids.data(), sizeof(VertexID_t) * (size_t)n0, cudaMemcpyHostToDevice, st));
      if (nd_inverter_run(data.inverters[d], st, n0, k0, v0, data.dMapKeys[1][d], data.dMapVals[1][d], &d_live) != ND_OK) { std::cout << nd_last_error() << std::endl; return false; }
      in_key = data.dMapKeys[1][d]; in_val = data.dMapVals[1][d];
      cur = 0;
    }
    for (int step = 0; step < App().steps(); step++) {
      const bool last = step == App().steps() - 1;
      const int f = App().stepSize(step);
      const int64_t full_pairs = n * pairs_per_sample<App>(step, isz);
      const bool explicit_tr = App().hasExplicitTransits();
      const bool write_map = (transit_parallel || explicit_tr) && !last;
      // sample-parallel runs of explicit-transit apps ping-pong the unsorted per-pair transits
      if (!transit_parallel && explicit_tr) cur = step & 1;
      VertexID_t *mk = data.dMapKeys[cur][d], *mv = data.dMapVals[cur][d];
      const VertexID_t *explicit_prev = (!transit_parallel && explicit_tr && step > 0) ? data.dMapKeys[cur ^ 1][d] : nullptr;
      if (write_map) fill_kernel<VertexID_t><<<(unsigned)((full_pairs * f + 255) / 256), 256, 0, st>>>(mk, full_pairs * f, INV);
      const int64_t threads = full_pairs * f;   // the grid covers every pair; transit-parallel threads beyond the live count return
      if (threads > 0) {
        if (transit_parallel) step_kernel<SampleType, App, true><<<(unsigned)((threads + 255) / 256), 256, 0, st>>>(part, step, nextdoor_seed(), first, full_pairs, d_live, in_key, in_val, data.dInitialSamples[d], data.dOutputSamples[d], out, fs, mk, mv, write_map, nullptr, isz);
        else step_kernel<SampleType, App, false><<<(unsigned)((threads + 255) / 256), 256, 0, st>>>(part, step, nextdoor_seed(), first, full_pairs, nullptr, nullptr, nullptr, data.dInitialSamples[d], data.dOutputSamples[d], out, fs, mk, mv, write_map, explicit_prev, isz);
      }
      if (write_map && explicit_tr) {
        const int64_t total = full_pairs * f;
        transits_kernel<SampleType, App><<<(unsigned)((total + 255) / 256), 256, 0, st>>>(step + 1, nextdoor_seed(), first, total, (int)(total / n),
                                                                                         data.dOutputSamples[d], mk, mv, INV);
      }
      NDC_CHECK(cudaGetLastError());
      if (write_map && transit_parallel) {  // the map inversion of the step loop (src/nextdoor.cu:2924-2939)
        // buffer 0 = unsorted pairs just written, buffer 1 = sorted map (its old content, this step's
        // input, is dead once the step kernel has run)
        if (nd_inverter_run(data.inverters[d], st, full_pairs * f, mk, mv, data.dMapKeys[1][d], data.dMapVals[1][d], &d_live) != ND_OK) { std::cout << nd_last_error() << std::endl; return false; }
      }
    }
  }
  for (int d = 0; d < P; d++) {  // only now wait: every device has its whole job
    NDC_CHECK(cudaSetDevice(data.devices[d]));
    NDC_CHECK(cudaStreamSynchronize(data.streams[d]));
    const int64_t n = part_size(S, d, P), first = part_start(S, d, P);
    if (n > 0) NDC_CHECK(cudaMemcpy(data.samples.data() + first, data.dOutputSamples[d], sizeof(SampleType) * (size_t)n, cudaMemcpyDeviceToHost));
  }
  return true;
}
}  // namespace ndc

// doTransitParallelSampling / doSampleParallelSampling (src/nextdoor.cu:2191-3006, 3009-3209)
template <class SampleType, typename App>
bool doTransitParallelSampling(CSR *csr, NextDoorData<SampleType, App> &data, bool enableLoadBalancing) {
  (void)enableLoadBalancing;  // user Apps run the generic kernels; the binned kernels serve the built-in apps of the library
  return ndc::run<SampleType, App>(csr, data, true);
}
template <class SampleType, typename App>
bool doSampleParallelSampling(CSR *csr, NextDoorData<SampleType, App> &data) {
  return ndc::run<SampleType, App>(csr, data, false);
}

// getFinalSamples (src/nextdoor.cu:3211-3237): library-owned host vector, shards in device order
template <class SampleType, typename App>
std::vector<VertexID_t> &getFinalSamples(NextDoorData<SampleType, App> &data) {
  const int P = (int)data.devices.size();
  const int64_t S = (int64_t)data.samples.size();
  const int fs = getFinalSampleSize<App>();
  for (int d = 0; d < P; d++) {
    cudaSetDevice(data.devices[d]);
    const int64_t n = ndc::part_size(S, d, P), first = ndc::part_start(S, d, P);
    if (n > 0) cudaMemcpy(data.hFinalSamples.data() + first * fs, data.dFinalSamples[d], sizeof(VertexID_t) * (size_t)n * fs, cudaMemcpyDeviceToHost);
    if (n > 0) cudaMemcpy(data.samples.data() + first, data.dOutputSamples[d], sizeof(SampleType) * (size_t)n, cudaMemcpyDeviceToHost);
  }
  return data.hFinalSamples;
}

// freeDeviceData (src/nextdoor.cu:2088-2115)
template <class SampleType, typename App>
void freeDeviceData(NextDoorData<SampleType, App> &data) {
  for (size_t d = 0; d < data.devices.size(); d++) {
    cudaSetDevice(data.devices[d]);
    if (d < data.dFinalSamples.size()) {
      cudaFree(data.dFinalSamples[d]); cudaFree(data.dInitialSamples[d]); cudaFree(data.dOutputSamples[d]);
      for (int b = 0; b < 2; b++) { cudaFree(data.dMapKeys[b][d]); cudaFree(data.dMapVals[b][d]); }
    }
    if (d < data.gpuCSRPartitions.size()) nd_graph_destroy(data.gpuCSRPartitions[d].handle);
    if (d < data.inverters.size()) nd_inverter_destroy(data.inverters[d]);
    if (d < data.streams.size()) cudaStreamDestroy(data.streams[d]);
  }
  data.inverters.clear(); data.streams.clear();
  data.dFinalSamples.clear(); data.dInitialSamples.clear(); data.dOutputSamples.clear();
  for (int b = 0; b < 2; b++) { data.dMapKeys[b].clear(); data.dMapVals[b].clear(); }
  data.gpuCSRPartitions.clear();
}

// nextdoor<>() (src/nextdoor.cu:3239-3306)
template <class SampleType, typename App>
bool nextdoor(const char *graph_file, const char *graph_type, const char *graph_format, const int nruns,
              const bool chk_results, const bool print_samples, const char *kernelType, const bool enableLoadBalancing,
              bool (*checkResultsFunc)(NextDoorData<SampleType, App> &)) {
  Graph graph;
  CSR *csr = loadGraph(graph, (char *)graph_file, (char *)graph_type, (char *)graph_format);
  if (csr == nullptr) return false;
  std::cout << "Graph has " << graph.get_n_edges() << " edges and " << graph.get_vertices().size() << " vertices " << std::endl;
  NextDoorData<SampleType, App> data;
  if (!allocNextDoorDataOnGPU<SampleType, App>(csr, data)) return false;
  data.gpuCSRPartitions = transferCSRToGPUs(data, csr);
  if (data.gpuCSRPartitions.size() != data.devices.size()) return false;
  for (int i = 0; i < nruns; i++) {
    bool ok;
    if (strcmp(kernelType, "TransitParallel") == 0) ok = doTransitParallelSampling<SampleType, App>(csr, data, enableLoadBalancing);
    else if (strcmp(kernelType, "SampleParallel") == 0) ok = doSampleParallelSampling<SampleType, App>(csr, data);
    else { printf("unknown kernel type '%s'\n", kernelType); return false; }
    if (!ok) return false;
  }
  getFinalSamples(data);
  const size_t fs = (size_t)getFinalSampleSize<App>();
  size_t total = 0;
  for (VertexID_t v : data.hFinalSamples) total += v != data.INVALID_VERTEX;
  if (print_samples) {
    for (size_t s = 0; s < data.hFinalSamples.size(); s += fs) {
      std::cout << "Contents of sample " << s / fs << " [";
      for (size_t v = s; v < s + fs; v++) std::cout << data.hFinalSamples[v] << ", ";
      std::cout << "]" << std::endl;
    }
  }
  std::cout << "totalSampledVertices " << total << std::endl;
  freeDeviceData(data);
  if (chk_results && checkResultsFunc) return checkResultsFunc(data);
  return true;
}

#endif
