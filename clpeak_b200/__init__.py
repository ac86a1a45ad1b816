"""clpeak_b200: a Blackwell (sm_100a) backend for the clpeak benchmark.

The product is native: CUDA kernels behind the C ABI of
``include/clpeak_b200_kernels.h`` and a C++ host (options, logger, result
store, backend) behind the ``clpeak_ffi`` C ABI of ``include/clpeak_ffi.h``.
This Python package only builds those libraries (``clpeak_b200.build``) and
binds them with ctypes (``clpeak_b200.native``) for tests and ``bench.py``.
There is no CPU fallback: every compute entry point fails without an sm_100 GPU.
"""

__all__ = ["build", "native"]
