"""ccglib_b200: B200 (sm_100a) complex-GEMM hot path behind a C ABI.

The product is the shared library ``ccglib_b200/lib/libccglib_b200.so`` (C ABI declared in
``include/ccglib_b200.h``) plus the C++ classes in ``include/ccglib`` that mirror the reference's
API.  This Python package only binds the C ABI with ctypes for tests and benchmarks; there is no
CPU or framework fallback -- importing ``ccglib_b200.capi`` raises if the library is not built.
"""
