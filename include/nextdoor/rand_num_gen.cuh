// rand_num_gen.cuh -- applications that include the reference's rand_num_gen.cuh directly get the same types from nextdoor.cu.
#include "nextdoor.cu"
