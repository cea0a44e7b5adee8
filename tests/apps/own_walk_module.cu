// A uniform random walk written against NextDoor's App struct contract and turned into a CPython
// extension module the way the reference's README describes (README.md:73-95,
// example/Makefile:5-11): define INIT_FUNC_NAME, `moduleName` and a static `nextDoorData`, then
// include nextDoorPythonModule.cu at the end of the application file.  Built by build_apps.py into
// NdOwnWalkPy3.so and imported by tests/test_gpu_module.py.
#include "nextdoor.cu"

struct OwnModuleSample {};

struct OwnModuleWalk {
  __host__ __device__ int steps() { return 12; }
  __host__ __device__ int stepSize(int) { return 1; }
  template <typename SampleType, typename EdgeArray, typename WeightArray>
  __device__ inline VertexID next(int, CSRPartition *, const VertexID *, const VertexID, SampleType *, const float,
                                  EdgeArray &edges, WeightArray &, const EdgePos_t numEdges, const VertexID_t, curandState *state) {
    return edges[RandNumGen::rand_int(state, numEdges)];
  }
  __host__ __device__ int samplingType() { return SamplingType::IndividualNeighborhood; }
  __host__ __device__ OutputFormat outputFormat() { return SampledVertices; }
  __host__ __device__ EdgePos_t numSamples(CSR *graph) { return graph->get_n_vertices(); }
  template <class SampleType>
  __host__ std::vector<VertexID_t> initialSample(int sampleIdx, CSR *, SampleType &) { return std::vector<VertexID_t>(1, sampleIdx); }
  __host__ __device__ EdgePos_t initialSampleSize(CSR *) { return 1; }
  __host__ __device__ bool hasExplicitTransits() { return false; }
  template <class SampleType>
  __host__ __device__ VertexID_t stepTransits(int, const VertexID_t, SampleType &, int, curandState *) { return -1; }
  template <class SampleType>
  __host__ SampleType initializeSample(CSR *, const VertexID_t) { return SampleType(); }
};

#define INIT_FUNC_NAME PyInit_NdOwnWalkPy3
const char *moduleName = "NdOwnWalkPy3";
static NextDoorData<OwnModuleSample, OwnModuleWalk> nextDoorData;
#include "nextDoorPythonModule.cu"
