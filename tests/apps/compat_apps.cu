// Test applications written against NextDoor's App struct contract, compiled through the
// source-compatibility headers of include/nextdoor/ and run on the GPU by tests/test_gpu_compat.py.
// The first group is this project's own; with -DNDC_WITH_REFERENCE the reference's application
// files are compiled in as well, unchanged, from the reference tree (never copied into the repo).
#include <chrono>

#include "nextdoor.cu"
#include "libNextDoor.hpp"
#include "main.cu"

// ---------------------------------------------------------------- own apps

struct PlainSample {};

struct WalkBase {
  __host__ __device__ int stepSize(int) { return 1; }
  __host__ __device__ int samplingType() { return SamplingType::IndividualNeighborhood; }
  __host__ __device__ OutputFormat outputFormat() { return SampledVertices; }
  __host__ __device__ EdgePos_t numSamples(CSR *graph) { return 3 * graph->get_n_vertices() + 7; }
  template <class SampleType>
  __host__ std::vector<VertexID_t> initialSample(int sampleIdx, CSR *graph, SampleType &) {
    return std::vector<VertexID_t>(1, sampleIdx % graph->get_n_vertices());
  }
  __host__ __device__ EdgePos_t initialSampleSize(CSR *) { return 1; }
  __host__ __device__ bool hasExplicitTransits() { return false; }
  template <class SampleType>
  __host__ __device__ VertexID_t stepTransits(int, const VertexID_t, SampleType &, int, curandState *) { return -1; }
  template <class SampleType>
  __host__ SampleType initializeSample(CSR *, const VertexID_t) { return SampleType(); }
};

// uniform neighbour, 40 steps
struct OwnUniformWalk : WalkBase {
  __host__ __device__ int steps() { return 40; }
  template <typename SampleType, typename EdgeArray, typename WeightArray>
  __device__ inline VertexID next(int, CSRPartition *, const VertexID *, const VertexID, SampleType *, const float,
                                  EdgeArray &edges, WeightArray &, const EdgePos_t numEdges, const VertexID_t, curandState *state) {
    return edges[RandNumGen::rand_int(state, numEdges)];
  }
};

// weight-proportional neighbour by rejection against the row's maximum weight, 30 steps
struct OwnWeightedWalk : WalkBase {
  __host__ __device__ int steps() { return 30; }
  template <typename SampleType, typename EdgeArray, typename WeightArray>
  __device__ inline VertexID next(int, CSRPartition *, const VertexID *, const VertexID, SampleType *, const float maxW,
                                  EdgeArray &edges, WeightArray &weights, const EdgePos_t numEdges, const VertexID_t, curandState *state) {
    if (numEdges == 1) return edges[0];
    for (;;) {
      const EdgePos_t pick = RandNumGen::rand_int(state, numEdges);
      const float bar = curand_uniform(state) * maxW;
      if (!(bar > weights[pick])) return edges[pick];
    }
  }
};

// second-order walk with return/in-out biases; the previous vertex lives in the sample
struct PrevSample { VertexID prev; };
struct OwnSecondOrderWalk : WalkBase {
  __host__ __device__ int steps() { return 25; }
  template <typename SampleType, typename EdgeArray, typename WeightArray>
  __device__ inline VertexID next(int step, CSRPartition *csr, const VertexID *transit, const VertexID, SampleType *sample,
                                  const float, EdgeArray &edges, WeightArray &, const EdgePos_t numEdges, const VertexID_t,
                                  curandState *state) {
    const float p = 0.5f, q = 2.0f;
    if (numEdges == 1 || step == 0) { sample->prev = *transit; return edges[0]; }
    const float bound = fmaxf(fmaxf(p, 1.0f / q), 1.0f);
    const VertexID before = sample->prev;
    for (;;) {
      const EdgePos_t pick = RandNumGen::rand_int(state, numEdges);
      const VertexID cand = edges[pick];
      const float bar = curand_uniform(state) * bound;
      float keep = 1.0f;
      if (cand == before) keep = p;
      else {
        const CSR::Edge *lst = csr->get_edges(before);
        if (utils::binarySearch(lst, cand, csr->get_n_edges_for_vertex(before))) keep = 1.0f / q;
      }
      if (bar < keep) { sample->prev = *transit; return cand; }
    }
  }
};

// three hops, fan-outs 4, 3, 2, with replacement
struct OwnKHop : WalkBase {
  __host__ __device__ int steps() { return 3; }
  __host__ __device__ int stepSize(int k) { return k == 0 ? 4 : (k == 1 ? 3 : 2); }
  __host__ __device__ EdgePos_t numSamples(CSR *graph) { return graph->get_n_vertices(); }
  template <typename SampleType, typename EdgeArray, typename WeightArray>
  __device__ inline VertexID next(int, CSRPartition *, const VertexID *, const VertexID, SampleType *, const float,
                                  EdgeArray &edges, WeightArray &, const EdgePos_t numEdges, const VertexID_t, curandState *state) {
    return edges[RandNumGen::rand_int(state, numEdges)];
  }
};

// collective layer sampling, 2 layers of 8 from batches of 8: a vertex uniform over the graph plus
// the batch-to-layer adjacency kept in the sample
struct OwnLayerSample { int row[2][64]; int col[2][64]; };
struct OwnLayerApp {
  __host__ __device__ int steps() { return 2; }
  __host__ __device__ int stepSize(int) { return 8; }
  __host__ __device__ int samplingType() { return SamplingType::CollectiveNeighborhood; }
  __host__ __device__ OutputFormat outputFormat() { return AdjacencyMatrix; }
  __host__ EdgePos_t numSamples(CSR *) { return 500; }
  __host__ __device__ EdgePos_t initialSampleSize(CSR *) { return 8; }
  __host__ __device__ bool hasExplicitTransits() { return false; }
  template <class SampleType>
  __device__ VertexID_t stepTransits(int, const VertexID_t, SampleType &, int, curandState *) { return -1; }
  template <class SampleType>
  __host__ std::vector<VertexID_t> initialSample(int sampleIdx, CSR *graph, SampleType &) {
    std::vector<VertexID_t> v;
    for (int i = 0; i < 8; i++) v.push_back((sampleIdx * 8 + i) % graph->get_n_vertices());
    return v;
  }
  template <class SampleType>
  __host__ SampleType initializeSample(CSR *, const VertexID_t) {
    SampleType s;
    for (int l = 0; l < 2; l++) for (int e = 0; e < 64; e++) { s.row[l][e] = -1; s.col[l][e] = -1; }
    return s;
  }
  template <typename SampleType, typename EdgeArray, typename WeightArray>
  __device__ inline VertexID next(int step, CSRPartition *csr, const VertexID *transits, const VertexID, SampleType *sample,
                                  const float, EdgeArray &, WeightArray &, const EdgePos_t, const VertexID_t slot, curandState *state) {
    const VertexID pick = RandNumGen::rand_int(state, csr->get_n_vertices());
    for (int i = 0; i < 8; i++) {
      const bool e = csr->has_edge_logn(transits[i], pick);
      sample->row[step][i * 8 + slot] = e ? i : -1;
      sample->col[step][i * 8 + slot] = e ? slot : -1;
    }
    return pick;
  }
};

// walk that teleports: after every step the next transit is one of four roots kept in the sample
// (explicit transits, the mechanism of the reference's multiRW app), and the vertex just sampled
// replaces the root the walk came from
struct TeleportSample { int roots[4]; int last; };
struct OwnTeleportWalk : WalkBase {
  __host__ __device__ int steps() { return 12; }
  __host__ __device__ EdgePos_t numSamples(CSR *graph) { return graph->get_n_vertices(); }
  __host__ __device__ bool hasExplicitTransits() { return true; }
  template <class SampleType>
  __host__ SampleType initializeSample(CSR *graph, const VertexID_t id) {
    SampleType s;
    for (int i = 0; i < 4; i++) s.roots[i] = (id * 7 + i * 13) % graph->get_n_vertices();
    s.last = 0;
    return s;
  }
  template <class SampleType>
  __host__ std::vector<VertexID_t> initialSample(int, CSR *, SampleType &sample) { return std::vector<VertexID_t>(1, sample.roots[0]); }
  template <class SampleType>
  __device__ VertexID_t stepTransits(int, const VertexID_t, SampleType &sample, int, curandState *state) {
    const int pick = RandNumGen::rand_int(state, 4);
    sample.last = pick;
    return sample.roots[pick];
  }
  template <typename SampleType, typename EdgeArray, typename WeightArray>
  __device__ inline VertexID next(int step, CSRPartition *, const VertexID *, const VertexID, SampleType *sample, const float,
                                  EdgeArray &edges, WeightArray &, const EdgePos_t numEdges, const VertexID_t, curandState *state) {
    const VertexID v = numEdges == 1 ? edges[0] : edges[RandNumGen::rand_int(state, numEdges)];
    if (step > 0) sample->roots[sample->last] = v;
    return v;
  }
};

// ---------------------------------------------------------------- the reference's own application files
#ifdef NDC_WITH_REFERENCE
#include "apps/randomwalks/randomWalks.cu"
#undef VERTICES_PER_SAMPLE
#include "apps/khop/khop.cu"
#undef VERTICES_PER_SAMPLE
#define main ndc_reference_example_main
#include "uniformRandWalk.cu"
#undef main
#include "apps/multiRW/multiRW.cu"
#undef VERTICES_PER_SAMPLE
#include "apps/layer/layerSampling.cu"
// The two subgraph apps keep file-scope globals with the same names (dRowStorage, dColStorage, foo):
// each gets a namespace of its own.
#undef VERTICES_PER_SAMPLE
namespace ref_mvs {
#include "apps/mvs/mvsSampling.cu"
}
#undef VERTICES_PER_SAMPLE
namespace ref_cluster {
#include "apps/clustergcn/clusterGCNSampling.cu"
}
#undef VERTICES_PER_SAMPLE
#endif

// ---------------------------------------------------------------- runners

template <class SampleType, typename App>
static int run_app(const char *file, const char *kernel, int lb, int32_t *out, int64_t cap, int64_t *n_out, int *fs_out,
                   NextDoorData<SampleType, App> *keep = nullptr) {
  Graph graph;
  CSR *csr = loadGraph(graph, (char *)file, (char *)"edge-list", (char *)"binary");
  if (!csr) return 1;
  srand(1);  // apps that seed their samples with rand() start from the same state on every run
  NextDoorData<SampleType, App> local;
  NextDoorData<SampleType, App> &data = keep ? *keep : local;
  if (!allocNextDoorDataOnGPU<SampleType, App>(csr, data)) return 2;
  data.gpuCSRPartitions = transferCSRToGPUs(data, csr);
  bool ok = strcmp(kernel, "SampleParallel") == 0 ? doSampleParallelSampling<SampleType, App>(csr, data)
                                                  : doTransitParallelSampling<SampleType, App>(csr, data, lb != 0);
  if (!ok) return 3;
  std::vector<VertexID_t> &fin = getFinalSamples(data);
  *n_out = (int64_t)fin.size();
  *fs_out = getFinalSampleSize<App>();
  if ((int64_t)fin.size() > cap) return 4;
  memcpy(out, fin.data(), sizeof(int32_t) * fin.size());
  freeDeviceData(data);
  delete csr;
  return 0;
}

// Times the sampling call alone, the way the reference prints its "End to end time"
// (src/nextdoor.cu:2363, 2963-2965: a host clock around the step loop): `nruns` calls after one
// warm-up call; seconds per call and the valid vertices of the last call's final samples.
template <class SampleType, typename App>
static int time_app(const char *file, const char *kernel, int lb, int nruns, double *seconds, int64_t *sampled) {
  Graph graph;
  CSR *csr = loadGraph(graph, (char *)file, (char *)"edge-list", (char *)"binary");
  if (!csr) return 1;
  NextDoorData<SampleType, App> data;
  if (!allocNextDoorDataOnGPU<SampleType, App>(csr, data)) return 2;
  data.gpuCSRPartitions = transferCSRToGPUs(data, csr);
  const bool sp = strcmp(kernel, "SampleParallel") == 0;
  double total = 0.0;
  for (int i = 0; i <= nruns; i++) {
    const auto t0 = std::chrono::steady_clock::now();
    const bool ok = sp ? doSampleParallelSampling<SampleType, App>(csr, data) : doTransitParallelSampling<SampleType, App>(csr, data, lb != 0);
    const auto t1 = std::chrono::steady_clock::now();
    if (!ok) return 3;
    if (i > 0) total += std::chrono::duration<double>(t1 - t0).count();
  }
  *seconds = total / (nruns > 0 ? nruns : 1);
  std::vector<VertexID_t> &fin = getFinalSamples(data);
  int64_t c = 0;
  for (VertexID_t v : fin) c += v != data.INVALID_VERTEX && v != -1;
  *sampled = c;
  freeDeviceData(data);
  delete csr;
  return 0;
}

extern "C" int ndc_time(int which, const char *file, const char *kernel, int lb, int nruns, double *seconds, int64_t *sampled) {
  switch (which) {
    case 0: return time_app<PlainSample, OwnUniformWalk>(file, kernel, lb, nruns, seconds, sampled);
    case 1: return time_app<PlainSample, OwnWeightedWalk>(file, kernel, lb, nruns, seconds, sampled);
#ifdef NDC_WITH_REFERENCE
    case 10: return time_app<UniformRandomWalkSample, UniformRandomWalkApp>(file, kernel, lb, nruns, seconds, sampled);
    case 11: return time_app<DummySample, DeepWalkApp>(file, kernel, lb, nruns, seconds, sampled);
    case 13: return time_app<Node2VecSample, Node2VecApp>(file, kernel, lb, nruns, seconds, sampled);
#endif
    default: return -1;
  }
}

extern "C" int ndc_run(int which, const char *file, const char *kernel, int lb, int32_t *out, int64_t cap, int64_t *n_out,
                       int *fs_out, int32_t *adj_row, int32_t *adj_col) {
  switch (which) {
    case 0: return run_app<PlainSample, OwnUniformWalk>(file, kernel, lb, out, cap, n_out, fs_out);
    case 1: return run_app<PlainSample, OwnWeightedWalk>(file, kernel, lb, out, cap, n_out, fs_out);
    case 2: return run_app<PrevSample, OwnSecondOrderWalk>(file, kernel, lb, out, cap, n_out, fs_out);
    case 3: return run_app<PlainSample, OwnKHop>(file, kernel, lb, out, cap, n_out, fs_out);
    case 4: {
      NextDoorData<OwnLayerSample, OwnLayerApp> data;
      int rc = run_app<OwnLayerSample, OwnLayerApp>(file, kernel, lb, out, cap, n_out, fs_out, &data);
      if (rc == 0 && adj_row)
        for (size_t s = 0; s < data.samples.size(); s++) {
          memcpy(adj_row + s * 128, data.samples[s].row, sizeof(int) * 128);
          memcpy(adj_col + s * 128, data.samples[s].col, sizeof(int) * 128);
        }
      return rc;
    }
    case 5: return run_app<TeleportSample, OwnTeleportWalk>(file, kernel, lb, out, cap, n_out, fs_out);
#ifdef NDC_WITH_REFERENCE
    case 16: return run_app<LayerSample, LayerSamplingApp>(file, kernel, lb, out, cap, n_out, fs_out);
    case 15: return run_app<MultiRWSample, MultiRWApp>(file, kernel, lb, out, cap, n_out, fs_out);
    case 10: return run_app<UniformRandomWalkSample, UniformRandomWalkApp>(file, kernel, lb, out, cap, n_out, fs_out);
    case 11: return run_app<DummySample, DeepWalkApp>(file, kernel, lb, out, cap, n_out, fs_out);
    case 12: return run_app<DummySample, PPRApp>(file, kernel, lb, out, cap, n_out, fs_out);
    case 13: return run_app<Node2VecSample, Node2VecApp>(file, kernel, lb, out, cap, n_out, fs_out);
    case 14: return run_app<KHopSample, KHopApp>(file, kernel, lb, out, cap, n_out, fs_out);
#endif
    default: return -1;
  }
}

#ifdef NDC_WITH_REFERENCE
// The reference's MVS app (src/apps/mvs/mvsSampling.cu) driven as its own test does
// (src/tests/multiGPU/mvs.cu:116-167): COO side buffers allocated by the caller, every sample
// appends the edges of its 32 batch vertices.  Returns the buffers and the per-sample records.
extern "C" int ndc_run_mvs(const char *file, const char *kernel, int lb, int64_t cap, int32_t *rows, int32_t *cols,
                           int64_t max_samples, int32_t *pos, int32_t *len, int32_t *vertices, int64_t *n_samples) {
  using namespace ref_mvs;
  Graph graph;
  CSR *csr = loadGraph(graph, (char *)file, (char *)"edge-list", (char *)"binary");
  if (!csr) return 1;
  const int64_t S = MVSSamplingApp().numSamples(csr);
  const int64_t storage = (int64_t)graph.get_n_edges() * DIVUP(S * 32, csr->get_n_vertices());
  if (storage > cap || S > max_samples) return 4;
  storagePosition = 0;
  cudaMalloc(&dRowStorage, sizeof(VertexID_t) * storage);
  cudaMalloc(&dColStorage, sizeof(VertexID_t) * storage);
  NextDoorData<MVSSample, MVSSamplingApp> data;
  data.csr = csr;
  data.gpuCSRPartitions = transferCSRToGPUs(data, csr);
  if (!allocNextDoorDataOnGPU<MVSSample, MVSSamplingApp>(csr, data)) return 2;
  if (data.gpuCSRPartitions.empty()) data.gpuCSRPartitions = transferCSRToGPUs(data, csr);
  bool ok = strcmp(kernel, "SampleParallel") == 0 ? doSampleParallelSampling<MVSSample, MVSSamplingApp>(csr, data)
                                                  : doTransitParallelSampling<MVSSample, MVSSamplingApp>(csr, data, lb != 0);
  if (!ok) return 3;
  getFinalSamples(data);
  cudaMemcpy(rows, dRowStorage, sizeof(int32_t) * storage, cudaMemcpyDeviceToHost);
  cudaMemcpy(cols, dColStorage, sizeof(int32_t) * storage, cudaMemcpyDeviceToHost);
  *n_samples = (int64_t)data.samples.size();
  for (size_t i = 0; i < data.samples.size(); i++) {
    pos[i] = data.samples[i].posInStorage;
    len[i] = data.samples[i].length;
    memcpy(vertices + i * 32, data.samples[i].vertices, sizeof(int32_t) * 32);
  }
  cudaFree(dRowStorage);
  cudaFree(dColStorage);
  freeDeviceData(data);
  delete csr;
  return 0;
}

// The reference's ClusterGCN app (src/apps/clustergcn/clusterGCNSampling.cu), set up as its foo()
// does (:141-208): clusters of 16 consecutive vertices, two clusters per sample, the induced
// subgraph of a sample appended to the COO buffers at a position claimed in stepTransits().
extern "C" int ndc_run_cluster(const char *file, const char *kernel, int lb, int64_t cap, int32_t *rows, int32_t *cols,
                               int64_t max_samples, int32_t *pos, int32_t *len, int32_t *vertices, int64_t *n_samples) {
  using namespace ref_cluster;
  Graph graph;
  CSR *csr = loadGraph(graph, (char *)file, (char *)"edge-list", (char *)"binary");
  if (!csr) return 1;
  clusters = std::vector<std::vector<VertexID_t>>(csr->get_n_vertices() / VERTICES_IN_CLUSTERS);
  for (int c = 0; c < (int)clusters.size(); c++)
    for (int v = 0; v < VERTICES_IN_CLUSTERS; v++) clusters[c].push_back(c * VERTICES_IN_CLUSTERS + v);
  const int64_t S = SubGraphSamplingAppI().numSamples(csr);
  const int64_t storage = (int64_t)graph.get_n_edges() * DIVUP(S * 32, csr->get_n_vertices());
  if (storage > cap || S > max_samples) return 4;
  NextDoorData<SubGraphSample, SubGraphSamplingAppI> data;
  data.devices = {0};
  data.csr = csr;
  data.gpuCSRPartitions = transferCSRToGPUs(data, csr);
  cudaMalloc(&dAdjMatrixTotalLen, sizeof(int));
  cudaMemset(dAdjMatrixTotalLen, 0, sizeof(int));
  cudaMalloc(&dRowStorage, sizeof(VertexID_t) * storage);
  cudaMalloc(&dColStorage, sizeof(VertexID_t) * storage);
  if (!allocNextDoorDataOnGPU<SubGraphSample, SubGraphSamplingAppI>(csr, data)) return 2;
  if (data.gpuCSRPartitions.empty()) data.gpuCSRPartitions = transferCSRToGPUs(data, csr);
  bool ok = strcmp(kernel, "SampleParallel") == 0 ? doSampleParallelSampling<SubGraphSample, SubGraphSamplingAppI>(csr, data)
                                                  : doTransitParallelSampling<SubGraphSample, SubGraphSamplingAppI>(csr, data, lb != 0);
  if (!ok) return 3;
  getFinalSamples(data);
  cudaMemcpy(rows, dRowStorage, sizeof(int32_t) * storage, cudaMemcpyDeviceToHost);
  cudaMemcpy(cols, dColStorage, sizeof(int32_t) * storage, cudaMemcpyDeviceToHost);
  *n_samples = (int64_t)data.samples.size();
  for (size_t i = 0; i < data.samples.size(); i++) {
    pos[i] = data.samples[i].adjMatrixPos;
    len[i] = data.samples[i].adjacencyMatrixLen;
    memcpy(vertices + i * 32, data.samples[i].vertices, sizeof(int32_t) * 32);
  }
  cudaFree(dRowStorage);
  cudaFree(dColStorage);
  cudaFree(dAdjMatrixTotalLen);
  freeDeviceData(data);
  delete csr;
  return 0;
}
#endif

extern "C" int ndc_has_reference_apps(void) {
#ifdef NDC_WITH_REFERENCE
  return 1;
#else
  return 0;
#endif
}

// the command line of the reference's per-app binaries, for the own uniform walk
extern "C" int ndc_app_main(int argc, char **argv) { return appMain<PlainSample, OwnUniformWalk>(argc, argv, nullptr); }
