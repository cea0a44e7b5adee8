// libNextDoor.hpp -- the public declarations of the reference's library header
// (src/libNextDoor.hpp:13-50: NextDoorData, loadGraph, transferCSRToGPUs, allocNextDoorDataOnGPU,
// doSampleParallelSampling, getFinalSamples, getFinalSampleSize, freeDeviceData) live, together
// with their definitions, in nextdoor.cu of this directory: everything is a template over the
// user's App type and must be visible in the user's translation unit.
#ifndef NEXTDOOR_B200_COMPAT_LIBNEXTDOOR_HPP
#define NEXTDOOR_B200_COMPAT_LIBNEXTDOOR_HPP
#include "nextdoor.cu"
#endif
