// csr.hpp -- applications that include the reference's csr.hpp directly get the same types from nextdoor.cu.
#include "nextdoor.cu"
