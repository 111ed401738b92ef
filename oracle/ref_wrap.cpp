// TEST INFRASTRUCTURE ONLY -- never linked into, loaded by or called from the
// product library.  C entry points around the reference's own CPU GEMM
// (ccglib::reference::GEMM::Run, declared in include/ccglib/gemm/reference.h:14-53
// and defined in src/reference/GEMM.cpp:229-287 of the reference project), so
// that tests and the CPU-baseline leg of the benchmark can call the unmodified
// reference through ctypes.  The reference sources are compiled where they lie;
// nothing of them is copied here.
//
// Storage types cross the boundary as raw bit patterns: half / bf16 as
// uint16_t, fp8 as uint8_t, 1-bit samples as packed uint32_t words.
#include <complex>
#include <cstddef>
#include <cstdint>

#include <omp.h>

#include <ccglib/gemm/reference.h>

// Thread count of the OpenMP runtime the reference GEMM runs on: set explicitly (launchers such
// as torchrun export OMP_NUM_THREADS=1) and read back, so a benchmark reports what it used.
extern "C" void ref_omp_set_threads(int n) {
  if (n > 0) omp_set_num_threads(n);
}
extern "C" int ref_omp_max_threads(void) { return omp_get_max_threads(); }

namespace {
inline ccglib::mma::MemOrder order(int c_col_major) {
  return c_col_major ? ccglib::mma::col_major : ccglib::mma::row_major;
}
} // namespace

#define REF_WRAP(NAME, TIN, TOUT)                                              \
  extern "C" void NAME(const void *a, const void *b, void *c, size_t M,        \
                       size_t N, size_t K, int c_col_major, float alpha_re,    \
                       float alpha_im, float beta_re, float beta_im) {         \
    ccglib::reference::GEMM gemm;                                              \
    gemm.Run(static_cast<const TIN *>(a), static_cast<const TIN *>(b),         \
             static_cast<TOUT *>(c), M, N, K, order(c_col_major),              \
             {alpha_re, alpha_im}, {beta_re, beta_im});                        \
  }

REF_WRAP(ref_gemm_e4m3_f32, fp8_e4m3, float)
REF_WRAP(ref_gemm_e5m2_f32, fp8_e5m2, float)
REF_WRAP(ref_gemm_f16_f16, half, half)
REF_WRAP(ref_gemm_f16_f32, half, float)
REF_WRAP(ref_gemm_f32_f16, float, half)
REF_WRAP(ref_gemm_bf16_bf16, bf16, bf16)
REF_WRAP(ref_gemm_bf16_f32, bf16, float)
REF_WRAP(ref_gemm_f32_bf16, float, bf16)
REF_WRAP(ref_gemm_f32_f32, float, float)
REF_WRAP(ref_gemm_int1_s32, unsigned, int)
