// placeholder until the collective kernels land
#include "nd_common.cuh"
int nd_collective_alloc(nd_sampler *) { nd_set_error("collective kernels are not built yet"); return ND_ERR_ARG; }
int nd_collective_sample(nd_sampler *, int) { nd_set_error("collective kernels are not built yet"); return ND_ERR_ARG; }
