/*
 * TEST INFRASTRUCTURE ONLY.  CPU restatement of the reference algorithms on the
 * complex-GEMM hot path, used as the checker for the CUDA library and as the
 * timed CPU baseline.  Nothing in the product library links, loads or calls
 * this file; the product fails loudly when its CUDA library is missing.
 *
 * Parity pin: every function here is checked (tests/test_oracle.py) against
 * the golden vectors of the reference's own tests (test/gemm/reference.cpp)
 * and, where the reference CPU GEMM could be compiled from its own sources
 * (oracle/_ref), against that binary on random inputs.
 *
 * Each function cites the reference file:line whose behaviour it restates.
 */
#include <stddef.h>
#include <stdint.h>
#include <string.h>

/* ---- storage-type decoders -------------------------------------------- */

static float bits_to_float(uint32_t u) {
  float f;
  memcpy(&f, &u, sizeof f);
  return f;
}

static uint32_t float_to_bits(float f) {
  uint32_t u;
  memcpy(&u, &f, sizeof u);
  return u;
}

/* IEEE binary16 -> binary32 (exact). */
static float half_to_float(uint16_t h) {
  const uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
  uint32_t exp = (h >> 10) & 0x1Fu;
  uint32_t man = h & 0x3FFu;
  if (exp == 0x1Fu) {
    return bits_to_float(sign | 0x7F800000u | (man << 13));
  }
  if (exp == 0) {
    if (man == 0) {
      return bits_to_float(sign);
    }
    /* subnormal: normalise */
    int shift = 0;
    while ((man & 0x400u) == 0) {
      man <<= 1;
      ++shift;
    }
    man &= 0x3FFu;
    exp = (uint32_t)(1 - shift);
    return bits_to_float(sign | ((exp + 112u) << 23) | (man << 13));
  }
  return bits_to_float(sign | ((exp + 112u) << 23) | (man << 13));
}

/* binary32 -> binary16, round to nearest even (what __float2half does). */
static uint16_t float_to_half(float f) {
  const uint32_t x = float_to_bits(f);
  const uint16_t sign = (uint16_t)((x >> 16) & 0x8000u);
  const uint32_t abs = x & 0x7FFFFFFFu;
  if (abs >= 0x7F800000u) { /* inf / nan */
    return (uint16_t)(sign | 0x7C00u | ((abs > 0x7F800000u) ? 0x200u : 0u));
  }
  if (abs >= 0x477FF000u) { /* rounds to >= 65520 -> inf */
    return (uint16_t)(sign | 0x7C00u);
  }
  if (abs < 0x33000001u) { /* < 2^-25 (or exactly 2^-25: ties to even 0) */
    return sign;
  }
  int32_t exp = (int32_t)(abs >> 23) - 127;
  uint32_t man = (abs & 0x7FFFFFu) | 0x800000u;
  uint32_t shift;
  uint32_t base;
  if (exp < -14) { /* subnormal half */
    shift = (uint32_t)(13 + (-14 - exp));
    base = 0;
  } else {
    shift = 13;
    base = (uint32_t)(exp + 15) << 10;
    man &= 0x7FFFFFu;
  }
  uint32_t q = man >> shift;
  const uint32_t rem = man & ((1u << shift) - 1u);
  const uint32_t halfway = 1u << (shift - 1);
  if (rem > halfway || (rem == halfway && (q & 1u))) {
    ++q;
  }
  return (uint16_t)(sign | (base + q));
}

static float bf16_to_float(uint16_t h) { return bits_to_float((uint32_t)h << 16); }

/* binary32 -> bfloat16, round to nearest even (what __float2bfloat16 does). */
static uint16_t float_to_bf16(float f) {
  const uint32_t x = float_to_bits(f);
  if ((x & 0x7FFFFFFFu) > 0x7F800000u) {
    return (uint16_t)((x >> 16) | 0x40u);
  }
  const uint32_t lsb = (x >> 16) & 1u;
  return (uint16_t)((x + 0x7FFFu + lsb) >> 16);
}

/* OCP FP8 E4M3 (bias 7, no inf, 0x7F/0xFF = NaN) -> binary32 (exact). */
static float e4m3_to_float(uint8_t v) {
  const uint32_t sign = (uint32_t)(v & 0x80u) << 24;
  const uint32_t exp = (v >> 3) & 0xFu;
  const uint32_t man = v & 0x7u;
  if (exp == 0xFu && man == 0x7u) {
    return bits_to_float(sign | 0x7FC00000u);
  }
  if (exp == 0) {
    /* subnormal: man * 2^-9 */
    const float mag = (float)man * (1.0f / 512.0f);
    return sign ? -mag : mag;
  }
  return bits_to_float(sign | ((exp + 120u) << 23) | (man << 20));
}

/* OCP FP8 E5M2 (bias 15, IEEE-like inf/nan) -> binary32 (exact). */
static float e5m2_to_float(uint8_t v) { return half_to_float((uint16_t)((uint16_t)v << 8)); }

/* Storage type codes follow the reference's ValueType enum
 * (include/ccglib/common/value_type.h:14-22). */
enum { VT_INT1 = 0, VT_INT32 = 1, VT_BF16 = 2, VT_E4M3 = 3, VT_E5M2 = 4, VT_F16 = 5, VT_F32 = 6 };

/* Widen n stored values of the given type to float, as the reference's
 * static_cast<ComputeType>(a_view(...)) does (src/reference/GEMM.cpp:52-55). */
int oracle_widen(const void *src, float *dst, size_t n, int value_type) {
  size_t i;
  switch (value_type) {
  case VT_F32:
    memcpy(dst, src, n * sizeof(float));
    return 0;
  case VT_F16:
    for (i = 0; i < n; ++i) dst[i] = half_to_float(((const uint16_t *)src)[i]);
    return 0;
  case VT_BF16:
    for (i = 0; i < n; ++i) dst[i] = bf16_to_float(((const uint16_t *)src)[i]);
    return 0;
  case VT_E4M3:
    for (i = 0; i < n; ++i) dst[i] = e4m3_to_float(((const uint8_t *)src)[i]);
    return 0;
  case VT_E5M2:
    for (i = 0; i < n; ++i) dst[i] = e5m2_to_float(((const uint8_t *)src)[i]);
    return 0;
  default:
    return 1;
  }
}

/* Narrow float results to the stored output type, as the reference's implicit
 * conversion in c_view(...) = sum does (src/reference/GEMM.cpp:87-88). */
int oracle_narrow(const float *src, void *dst, size_t n, int value_type) {
  size_t i;
  switch (value_type) {
  case VT_F32:
    memcpy(dst, src, n * sizeof(float));
    return 0;
  case VT_F16:
    for (i = 0; i < n; ++i) ((uint16_t *)dst)[i] = float_to_half(src[i]);
    return 0;
  case VT_BF16:
    for (i = 0; i < n; ++i) ((uint16_t *)dst)[i] = float_to_bf16(src[i]);
    return 0;
  default:
    return 1;
  }
}

/* ---- OpenMP thread count: set explicitly, read back for the benchmark record ---- */

#include <omp.h>

void oracle_omp_set_threads(int n) {
  if (n > 0) omp_set_num_threads(n);
}

int oracle_omp_max_threads(void) { return omp_get_max_threads(); }

/* ---- complex GEMM, floating point --------------------------------------- */

/*
 * One batch item of C = alpha * A x B^T + beta * C on planar complex data.
 * a: [2][M][K], b: [2][N][K] (both K-contiguous), c: [2][M][N] (row-major) or
 * [2][N][M] (col-major), all already widened to float.
 *
 * Follows src/reference/GEMM.cpp:45-90: per output element a serial k-loop in
 * float; the complex product term is formed first (two products and one
 * add/sub per part) and then added to the running sum; alpha is applied only
 * when it differs from (1,0) and beta only when it differs from (0,0).
 * Compile with -ffp-contract=off so that no fused multiply-add changes the
 * rounding sequence (the reference build has none on baseline x86-64).
 */
void oracle_cgemm_f32(const float *a, const float *b, float *c, size_t M, size_t N, size_t K,
                      int c_col_major, float alpha_re, float alpha_im, float beta_re,
                      float beta_im) {
  const float *a_re = a;
  const float *a_im = a + M * K;
  const float *b_re = b;
  const float *b_im = b + N * K;
  float *c_re = c;
  float *c_im = c + M * N;
  ptrdiff_t mn;
#pragma omp parallel for schedule(static)
  for (mn = 0; mn < (ptrdiff_t)(M * N); ++mn) {
    const size_t m = (size_t)mn / N;
    const size_t n = (size_t)mn % N;
    float sum_re = 0.0f;
    float sum_im = 0.0f;
    size_t k;
    for (k = 0; k < K; ++k) {
      const float ar = a_re[m * K + k];
      const float ai = a_im[m * K + k];
      const float br = b_re[n * K + k];
      const float bi = b_im[n * K + k];
      const float term_re = ar * br - ai * bi;
      const float term_im = ar * bi + ai * br;
      sum_re += term_re;
      sum_im += term_im;
    }
    if (alpha_re != 1.0f || alpha_im != 0.0f) {
      const float copy = sum_re;
      sum_re = alpha_re * sum_re - alpha_im * sum_im;
      sum_im = alpha_im * copy + alpha_re * sum_im;
    }
    {
      const size_t idx = c_col_major ? n * M + m : m * N + n;
      if (beta_re != 0.0f || beta_im != 0.0f) {
        const float old_re = c_re[idx];
        const float old_im = c_im[idx];
        sum_re += beta_re * old_re - beta_im * old_im;
        sum_im += beta_im * old_re + beta_re * old_im;
      }
      c_re[idx] = sum_re;
      c_im[idx] = sum_im;
    }
  }
}

/* ---- complex GEMM, 1-bit samples ---------------------------------------- */

static int popcount32(uint32_t x) {
  x = x - ((x >> 1) & 0x55555555u);
  x = (x & 0x33333333u) + ((x >> 2) & 0x33333333u);
  x = (x + (x >> 4)) & 0x0F0F0F0Fu;
  return (int)((x * 0x01010101u) >> 24);
}

/*
 * One batch item of the +-1 complex GEMM on packed bits (bit 1 = +1, bit 0 =
 * -1, sample i in bit i%32 of word i/32).  K counts 1-bit samples; rows hold
 * ceil(K/32) words and padding bits are zero.
 *
 * Follows run_binary, src/reference/GEMM.cpp:106-224: XOR + popcount per word
 * with the imaginary part of B complemented for the real sum, then
 * re = 2*(K_padded - sum_re), im = 2*(K_padded - K_padding - sum_im); alpha
 * and beta are truncated to int and always applied.
 */
void oracle_cgemm_int1(const uint32_t *a, const uint32_t *b, int32_t *c, size_t M, size_t N,
                       size_t K, int c_col_major, float alpha_re_f, float alpha_im_f,
                       float beta_re_f, float beta_im_f) {
  const size_t k_packed = (K + 31) / 32;
  const size_t k_padded = k_packed * 32;
  const size_t k_padding = k_padded - K;
  const uint32_t *a_re = a;
  const uint32_t *a_im = a + M * k_packed;
  const uint32_t *b_re = b;
  const uint32_t *b_im = b + N * k_packed;
  int32_t *c_re = c;
  int32_t *c_im = c + M * N;
  const int alpha_re = (int)alpha_re_f;
  const int alpha_im = (int)alpha_im_f;
  const int beta_re = (int)beta_re_f;
  const int beta_im = (int)beta_im_f;
  ptrdiff_t mn;
#pragma omp parallel for schedule(static)
  for (mn = 0; mn < (ptrdiff_t)(M * N); ++mn) {
    const size_t m = (size_t)mn / N;
    const size_t n = (size_t)mn % N;
    int sum_re = 0;
    int sum_im = 0;
    size_t k;
    for (k = 0; k < k_packed; ++k) {
      const uint32_t ar = a_re[m * k_packed + k];
      const uint32_t ai = a_im[m * k_packed + k];
      const uint32_t br = b_re[n * k_packed + k];
      const uint32_t bi = b_im[n * k_packed + k];
      sum_re += popcount32(ar ^ br) + popcount32(ai ^ ~bi);
      sum_im += popcount32(ar ^ bi) + popcount32(ai ^ br);
    }
    sum_re = 2 * ((int)k_padded - sum_re);
    sum_im = 2 * ((int)k_padded - (int)k_padding - sum_im);
    {
      const int copy = sum_re;
      const size_t idx = c_col_major ? n * M + m : m * N + n;
      int old_re, old_im;
      sum_re = alpha_re * sum_re - alpha_im * sum_im;
      sum_im = alpha_im * copy + alpha_re * sum_im;
      old_re = c_re[idx];
      old_im = c_im[idx];
      c_re[idx] = sum_re + beta_re * old_re - beta_im * old_im;
      c_im[idx] = sum_im + beta_im * old_re + beta_re * old_im;
    }
  }
}

/* ---- bit packing --------------------------------------------------------- */

/*
 * n one-byte samples -> ceil(n/32) words; sample i goes to bit i%32 of word
 * i/32 and is 1 when the byte is non-zero (kernels/packing_kernel.cu:7-49:
 * warp ballot, lane i -> bit i).  With interleaved input the whole buffer is
 * read as [n/2][2] (re, im pairs) and written as [2][n/2]: output sample t
 * reads input 2t for t < n/2 and 2t - (n-1) otherwise (:15-22).
 */
void oracle_pack_bits(const uint8_t *in, uint32_t *out, size_t n, int input_interleaved) {
  size_t t;
  const size_t words = (n + 31) / 32;
  memset(out, 0, words * sizeof(uint32_t));
  for (t = 0; t < n; ++t) {
    size_t src = t;
    if (input_interleaved) {
      src = 2 * t;
      if (src >= n) {
        src -= n - 1;
      }
    }
    if (in[src] != 0) {
      out[t / 32] |= 1u << (t % 32);
    }
  }
}

/* ceil(n/32) words -> n bytes of 0/1 (kernels/packing_kernel.cu:51-62). */
void oracle_unpack_bits(const uint32_t *in, uint8_t *out, size_t n) {
  size_t t;
  for (t = 0; t < n; ++t) {
    out[t] = (uint8_t)((in[t / 32] >> (t % 32)) & 1u);
  }
}

/* ---- tile transpose ------------------------------------------------------- */

/*
 * [B][2][M][N] (planar) or [B][M][N][2] (interleaved) ->
 * [B][ceil(M/Mc)][ceil(N/Nc)][2][Mc][Nc], zero padded; elements are moved by
 * size only (kernels/transpose_kernel.cu:40-82).  For 1-bit data the element
 * is a 32-bit word of 32 samples: N and Nc count samples and must be multiples
 * of 32 (:28,54).  elem_bytes is 1, 2 or 4; for nr_bits == 1 pass the sample
 * counts and this routine divides by 32 itself.
 */
int oracle_transpose(const void *in, void *out, size_t B, size_t M, size_t N, size_t Mc, size_t Nc,
                     size_t nr_bits, int input_interleaved) {
  size_t es, n_el, nc_el, b, c, m, n;
  const uint8_t *src = (const uint8_t *)in;
  uint8_t *dst = (uint8_t *)out;
  if (nr_bits == 1) {
    if (N % 32 != 0 || Nc % 32 != 0) return 1;
    es = 4;
    n_el = N / 32;
    nc_el = Nc / 32;
  } else if (nr_bits == 8 || nr_bits == 16 || nr_bits == 32) {
    es = nr_bits / 8;
    n_el = N;
    nc_el = Nc;
  } else {
    return 1;
  }
  {
    const size_t mt = (M + Mc - 1) / Mc;
    const size_t nt = (n_el + nc_el - 1) / nc_el;
    memset(dst, 0, B * mt * nt * 2 * Mc * nc_el * es);
    for (b = 0; b < B; ++b)
      for (c = 0; c < 2; ++c)
        for (m = 0; m < M; ++m)
          for (n = 0; n < n_el; ++n) {
            const size_t si = input_interleaved ? (((b * M + m) * n_el + n) * 2 + c)
                                                : (((b * 2 + c) * M + m) * n_el + n);
            const size_t di =
                ((((b * mt + m / Mc) * nt + n / nc_el) * 2 + c) * Mc + m % Mc) * nc_el + n % nc_el;
            memcpy(dst + di * es, src + si * es, es);
          }
  }
  return 0;
}
