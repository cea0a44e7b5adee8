// placeholder until the k-hop kernels land
#include "nd_common.cuh"
int nd_khop_alloc(nd_sampler *) { nd_set_error("k-hop kernels are not built yet"); return ND_ERR_ARG; }
int nd_khop_sample(nd_sampler *, int) { nd_set_error("k-hop kernels are not built yet"); return ND_ERR_ARG; }
