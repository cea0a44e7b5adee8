// utils.hpp -- applications that include the reference's utils.hpp directly get the same types from nextdoor.cu.
#include "nextdoor.cu"
