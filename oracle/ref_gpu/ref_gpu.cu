// Builds the reference's own GPU code for sm_100 and runs nextdoor<SampleType, App>() on a binary
// edge-list file.  TEST / MEASUREMENT INFRASTRUCTURE ONLY: the reference sources are included from
// their own tree (the include path is given by oracle/Makefile), none of them is copied here, and
// nothing of the product links against this program.  It is the "reference GPU build timed on the
// same synthetic graph" leg of the measurements; the reference prints its own "End to end time".
//
// usage: ref_gpu_<app> <graph.bin> <TransitParallel|SampleParallel> <load balancing 0|1> <runs>
// REF_APP: 1 DeepWalk, 2 PPR, 3 node2vec (apps/randomwalks), 4 k-hop (apps/khop), 0 uniform walk (example/)
#include "nextdoor.cu"   // the reference's src/nextdoor.cu

#if REF_APP == 0
#define main ref_example_main
#include "uniformRandWalk.cu"   // example/uniformRandWalk.cu (its main() renamed away)
#undef main
typedef UniformRandomWalkApp TheApp;
typedef UniformRandomWalkSample TheSample;
#elif REF_APP == 4
#include "apps/khop/khop.cu"
typedef KHopApp TheApp;
typedef KHopSample TheSample;
#else
#include "apps/randomwalks/randomWalks.cu"
#if REF_APP == 1
typedef DeepWalkApp TheApp;
typedef DummySample TheSample;
#elif REF_APP == 2
typedef PPRApp TheApp;
typedef DummySample TheSample;
#else
typedef Node2VecApp TheApp;
typedef Node2VecSample TheSample;
#endif
#endif

int main(int argc, char **argv) {
  if (argc < 5) {
    fprintf(stderr, "usage: %s <graph.bin> <TransitParallel|SampleParallel> <lb 0|1> <runs>\n", argv[0]);
    return 2;
  }
  const bool ok = nextdoor<TheSample, TheApp>(argv[1], "edge-list", "binary", atoi(argv[4]), false, false, argv[2],
                                              atoi(argv[3]) != 0, nullptr);
  return ok ? 0 : 1;
}
