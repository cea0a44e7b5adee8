/* Stand-in for the reference's src/libNextDoor.hpp on the host oracle build. */
#ifndef REF_SHIM_LIBNEXTDOOR_STUB
#define REF_SHIM_LIBNEXTDOOR_STUB
template <class SampleType, typename App> struct NextDoorData {};
#endif
