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
// One-byte samples (non-zero = +1) in planar [batch][2][rows][k] or interleaved
// [batch][rows][k][2] order -> the operand planes of the 1-bit GEMM (see staging.cu).
int launch_expand_bytes(const void *d_in, void *d_out, size_t batch, size_t rows, size_t k,
                        size_t out_row_bytes, int planes_out, bool interleaved, cudaStream_t stream,
                        bool nibbles);
int launch_pad_rows(const void *d_in, void *d_out, size_t rows, size_t row_bytes,
                    size_t out_row_bytes, cudaStream_t stream);

// One entry of a tuning table (see capi.cu): tile width in columns (0 = leave to the model), one
// CTA or a CTA pair per tile (-1 = leave to the model), column-panel width of the tile walk
// (0 = leave to the model), split-K factor.  Looked up by (types, M, N, log2 bucket of the row bytes, log2 bucket
// of the batch); returns 1 when an entry matched.
struct TuneChoice {
  int bn = 0, pair = -1, group_n = 0;
  int split_k = 0;  // CTAs sharing the K of one tile (0 = leave to the model)
};
int tune_table_lookup(const char *path, const ccglib_b200_gemm_desc &d, size_t k_bytes,
                      TuneChoice *choice);

// Input forms the public GEMM description cannot express; used by the Pipeline.
struct PlanOptions {
  bool int1_bytes_in = false;           // 1-bit A and B arrive as one byte per sample
  bool int1_bytes_interleaved = false;  // ... in [batch][rows][K][2] order (else [batch][2][rows][K])
};

// ccglib_b200_gemm_plan_create with options; ccglib_b200_gemm_run on the first `items` batch
// items of a plan (items <= the plan's batch).
int create_gemm_plan(const ccglib_b200_gemm_desc *desc, const PlanOptions &opt,
                     ccglib_b200_gemm_plan **out);
int run_gemm_items(ccglib_b200_gemm_plan *plan, const void *d_a, const void *d_b, void *d_c,
                   size_t items, void *stream);

} // namespace ccglib_b200
#endif
