/* Stand-in for the reference's src/main.cu (needs the absent AnyOption submodule). */
#ifndef REF_SHIM_MAIN_STUB
#define REF_SHIM_MAIN_STUB
template <class SampleType, typename App> int appMain(int, char **, void *) { return 0; }
#endif
