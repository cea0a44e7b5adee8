// graph.hpp -- applications that include the reference's graph.hpp directly get the same types from nextdoor.cu.
#include "nextdoor.cu"
