"""metalhlo_b200 — B200 (sm_100a) execution backend behind MetalHLO's operator surface.

The product is native: ``lib/libmhlo_cuda.so`` (device runtime and hand-written kernels, C ABI in
``include/mhlo_cuda.h``) and ``lib/libCMetalHLO.so`` (StableHLO compiler + executor behind the ``mhlo_*`` C API
of ``include/metalhlo.h``). The Python modules here are ctypes views of those libraries for tests and benchmarks.
"""
__version__ = "0.1.0"
