"""B200 (sm_100a) epilogue kernels for PixieNN's per-layer path, behind a C ABI.

``capi``  -- ctypes declarations of ``libpxe.so`` (``include/pxe.h``)
``ops``   -- the operators on torch CUDA tensors
``synth`` -- seeded synthetic inputs and weights
"""
__version__ = "0.1.0"
