// Shared host/device helpers of the ccglib_b200 CUDA library.
#ifndef CCGLIB_B200_COMMON_CUH_
#define CCGLIB_B200_COMMON_CUH_

#include <cstdarg>
#include <cstddef>
#include <cstdint>
#include <cstdio>

#include <cuda_runtime.h>

#include "../../include/ccglib_b200.h"

namespace ccglib_b200 {

// Status-word codes written by kernels.
enum DeviceStatus : unsigned {
  kDevOk = 0u,
  kDevTimeoutProducer = 1u << 0,  // TMA producer waited too long for a free stage
  kDevTimeoutMma = 1u << 1,       // MMA issuer waited too long for a full stage / free accumulator
  kDevTimeoutEpilogue = 1u << 2,  // epilogue waited too long for a finished accumulator
  kDevTimeoutDrain = 1u << 3,     // drain of in-flight copies after an abort gave up
};

void set_last_error(const char *fmt, ...);

inline int cuda_fail(cudaError_t err, const char *what) {
  set_last_error("%s: %s", what, cudaGetErrorString(err));
  return CCGLIB_B200_CUDA_ERROR;
}

#define CCGLIB_CUDA_TRY(expr)                                                                    \
  do {                                                                                           \
    cudaError_t err__ = (expr);                                                                  \
    if (err__ != cudaSuccess) return ::ccglib_b200::cuda_fail(err__, #expr);                     \
  } while (0)

template <typename T> __host__ __device__ constexpr T ceil_div(T a, T b) { return (a + b - 1) / b; }

inline bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// Number of SMs of the current device (cached per device ordinal).
int sm_count();

// Launchers implemented in the individual .cu files (host side, no extern "C").
int launch_expand_bits(const void *d_in, void *d_out, size_t batch, size_t rows, size_t k_bits,
                       size_t out_row_bytes, int planes_out, bool tiled, size_t blk, size_t k_c_bits,
                       cudaStream_t stream, bool nibbles = false);
int launch_pad_rows(const void *d_in, void *d_out, size_t rows, size_t row_bytes,
                    size_t out_row_bytes, cudaStream_t stream);

} // namespace ccglib_b200
#endif
