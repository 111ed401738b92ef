// ccglib::reference::GEMM -- the CPU complex GEMM that callers of the reference use to verify
// device results, with the reference's class name, its ten Run() overloads and their argument
// order (reference include/ccglib/gemm/reference.h:12-53, src/reference/GEMM.cpp:16-287).
// Header-only and host-only: it is a verification aid for callers, not a fallback of the device
// path (ccglib::mma::GEMM never calls it).
//
// Semantics kept from the reference:
//   * operands are planar, A [2][M][K] and B [2][N][K] (both K-contiguous); C is [2][M][N]
//     (row-major) or [2][N][M] (col-major);
//   * floating point: one serial sum over k per output element, each term formed as
//     ar*br - ai*bi and ar*bi + ai*br; arithmetic in float when the output is 16 bits wide,
//     otherwise in the output type; alpha is applied only when it differs from (1, 0), beta only
//     when it differs from (0, 0);
//   * 1-bit: bit 1 is +1 and bit 0 is -1, 32 samples per word; rows are padded to whole words
//     with zero bits, whose contribution cancels in the real part and is subtracted from the
//     imaginary part; alpha and beta are truncated to int and always applied.
// Compiled with OpenMP it runs the (m, n) loop in parallel, as the reference does.
#pragma once

#include <climits>
#include <complex>
#include <cstddef>
#include <cstdint>
#include <type_traits>

#include <ccglib/bf16.h>
#include <ccglib/fp16.h>
#include <ccglib/fp8.h>
#include <ccglib/gemm/mem_order.h>

namespace ccglib::reference {

namespace detail {

template <typename Tout>
using compute_t = std::conditional_t<std::is_same_v<Tout, half> || std::is_same_v<Tout, bf16>,
                                     float, Tout>;

template <typename Tin, typename Tout>
void cgemm(const Tin *a, const Tin *b, Tout *c, size_t M, size_t N, size_t K, bool c_col_major,
           std::complex<float> alpha, std::complex<float> beta) {
  using T = compute_t<Tout>;
  const Tin *a_re = a, *a_im = a + M * K;
  const Tin *b_re = b, *b_im = b + N * K;
  Tout *c_re = c, *c_im = c + M * N;
  const T alpha_re = alpha.real(), alpha_im = alpha.imag();
  const T beta_re = beta.real(), beta_im = beta.imag();
  const bool scale = alpha_re != T(1) || alpha_im != T(0);
  const bool accumulate = beta_re != T(0) || beta_im != T(0);
  const std::ptrdiff_t outputs = static_cast<std::ptrdiff_t>(M * N);
#ifdef _OPENMP
#pragma omp parallel for schedule(static)
#endif
  for (std::ptrdiff_t o = 0; o < outputs; ++o) {
    const size_t m = static_cast<size_t>(o) / N, n = static_cast<size_t>(o) % N;
    const Tin *ar = a_re + m * K, *ai = a_im + m * K;
    const Tin *br = b_re + n * K, *bi = b_im + n * K;
    T re = T(0), im = T(0);
    for (size_t k = 0; k < K; ++k) {
      const T x_re = static_cast<T>(ar[k]), x_im = static_cast<T>(ai[k]);
      const T y_re = static_cast<T>(br[k]), y_im = static_cast<T>(bi[k]);
      const T term_re = x_re * y_re - x_im * y_im;
      const T term_im = x_re * y_im + x_im * y_re;
      re += term_re;
      im += term_im;
    }
    if (scale) {
      const T unscaled_re = re;
      re = alpha_re * re - alpha_im * im;
      im = alpha_im * unscaled_re + alpha_re * im;
    }
    const size_t at = c_col_major ? n * M + m : m * N + n;
    if (accumulate) {
      const T old_re = static_cast<T>(c_re[at]), old_im = static_cast<T>(c_im[at]);
      re += beta_re * old_re - beta_im * old_im;
      im += beta_im * old_re + beta_re * old_im;
    }
    c_re[at] = static_cast<Tout>(re);
    c_im[at] = static_cast<Tout>(im);
  }
}

inline int differing_bits(unsigned x, unsigned y) { return __builtin_popcount(x ^ y); }

inline void cgemm_1bit(const unsigned *a, const unsigned *b, int *c, size_t M, size_t N, size_t K,
                       bool c_col_major, std::complex<float> alpha, std::complex<float> beta) {
  constexpr size_t kWordBits = sizeof(unsigned) * CHAR_BIT;
  const size_t words = (K + kWordBits - 1) / kWordBits;
  const long long k_padded = static_cast<long long>(words * kWordBits);
  const long long k_valid = static_cast<long long>(K);
  const unsigned *a_re = a, *a_im = a + M * words;
  const unsigned *b_re = b, *b_im = b + N * words;
  int *c_re = c, *c_im = c + M * N;
  const int alpha_re = static_cast<int>(alpha.real()), alpha_im = static_cast<int>(alpha.imag());
  const int beta_re = static_cast<int>(beta.real()), beta_im = static_cast<int>(beta.imag());
  const std::ptrdiff_t outputs = static_cast<std::ptrdiff_t>(M * N);
#ifdef _OPENMP
#pragma omp parallel for schedule(static)
#endif
  for (std::ptrdiff_t o = 0; o < outputs; ++o) {
    const size_t m = static_cast<size_t>(o) / N, n = static_cast<size_t>(o) % N;
    const unsigned *ar = a_re + m * words, *ai = a_im + m * words;
    const unsigned *br = b_re + n * words, *bi = b_im + n * words;
    // a product of two +-1 samples is -1 exactly where their bits differ; the subtraction of
    // ai*bi is a sum against the complemented bi
    long long diff_re = 0, diff_im = 0;
    for (size_t w = 0; w < words; ++w) {
      diff_re += differing_bits(ar[w], br[w]) + differing_bits(ai[w], ~bi[w]);
      diff_im += differing_bits(ar[w], bi[w]) + differing_bits(ai[w], br[w]);
    }
    const int dot_re = static_cast<int>(2 * (k_padded - diff_re));
    const int dot_im = static_cast<int>(2 * (k_valid - diff_im));
    const int re = alpha_re * dot_re - alpha_im * dot_im;
    const int im = alpha_im * dot_re + alpha_re * dot_im;
    const size_t at = c_col_major ? n * M + m : m * N + n;
    const int old_re = c_re[at], old_im = c_im[at];
    c_re[at] = re + beta_re * old_re - beta_im * old_im;
    c_im[at] = im + beta_im * old_re + beta_re * old_im;
  }
}

} // namespace detail

class GEMM {
public:
  virtual ~GEMM() = default;

#define CCGLIB_B200_REFERENCE_RUN(TIN, TOUT)                                                     \
  virtual void Run(const TIN *a, const TIN *b, TOUT *c, size_t M, size_t N, size_t K,            \
                   ccglib::mma::MemOrder output_mem_order = ccglib::mma::row_major,              \
                   std::complex<float> alpha = {1, 0}, std::complex<float> beta = {0, 0}) {      \
    detail::cgemm<TIN, TOUT>(a, b, c, M, N, K, output_mem_order == ccglib::mma::col_major,       \
                             alpha, beta);                                                       \
  }
  CCGLIB_B200_REFERENCE_RUN(fp8_e4m3, float)
  CCGLIB_B200_REFERENCE_RUN(fp8_e5m2, float)
  CCGLIB_B200_REFERENCE_RUN(half, half)
  CCGLIB_B200_REFERENCE_RUN(half, float)
  CCGLIB_B200_REFERENCE_RUN(float, half)
  CCGLIB_B200_REFERENCE_RUN(bf16, bf16)
  CCGLIB_B200_REFERENCE_RUN(bf16, float)
  CCGLIB_B200_REFERENCE_RUN(float, bf16)
  CCGLIB_B200_REFERENCE_RUN(float, float)
#undef CCGLIB_B200_REFERENCE_RUN

  virtual void Run(const unsigned *a, const unsigned *b, int *c, size_t M, size_t N, size_t K,
                   ccglib::mma::MemOrder output_mem_order = ccglib::mma::row_major,
                   std::complex<float> alpha = {1, 0}, std::complex<float> beta = {0, 0}) {
    detail::cgemm_1bit(a, b, c, M, N, K, output_mem_order == ccglib::mma::col_major, alpha, beta);
  }
};

} // namespace ccglib::reference
