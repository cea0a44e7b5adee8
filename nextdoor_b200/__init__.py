"""nextdoor_b200 -- B200-native (sm_100a) implementation of NextDoor's graph-sampling path.

The compute lives in libnextdoor_b200.so (hand-written CUDA, C ABI in include/nextdoor_b200.h);
this package is the thin host-side mirror of the reference's C++ / Python surface.  Importing
`nextdoor_b200.api` loads the shared library and raises if it has not been built.
"""
__all__ = ["api", "build"]
