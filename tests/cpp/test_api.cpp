// Self-checking program for the C++ classes in <ccglib/...>: the cases of the reference's
// raw-CUDA-handle tests (test/cuda/mma.cpp, pipeline.cpp, transpose.cpp, packing.cpp) and of its
// pipeline integration tests (test/pipeline/pipeline.cpp:17-187), checked against the CPU oracle
// (oracle/oracle.c, linked here as the checker).  Prints one line per case; exit code = failures.
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <functional>
#include <random>
#include <string>
#include <vector>

#include <cuda.h>
#include <cuda_fp16.h>

#include <cudawrappers/cu.hpp>

#include <ccglib/ccglib.hpp>
#include <ccglib/common/arch.h>
#include <ccglib/fp16.h>

extern "C" {
void oracle_cgemm_f32(const float *a, const float *b, float *c, size_t M, size_t N, size_t K,
                      int c_col_major, float ar, float ai, float br, float bi);
void oracle_cgemm_int1(const uint32_t *a, const uint32_t *b, int32_t *c, size_t M, size_t N,
                       size_t K, int c_col_major, float ar, float ai, float br, float bi);
void oracle_pack_bits(const uint8_t *in, uint32_t *out, size_t n, int interleaved);
void oracle_unpack_bits(const uint32_t *in, uint8_t *out, size_t n);
int oracle_transpose(const void *in, void *out, size_t B, size_t M, size_t N, size_t Mc, size_t Nc,
                     size_t nr_bits, int interleaved);
}

namespace {

int failures = 0;

void report(const char *name, bool ok, const std::string &detail = "") {
  std::printf("%s %s %s\n", ok ? "PASS" : "FAIL", name, detail.c_str());
  if (!ok) ++failures;
}

void run_case(const char *name, const std::function<bool()> &body) {
  try {
    report(name, body());
  } catch (const std::exception &e) {
    report(name, false, std::string("exception: ") + e.what());
  }
}

// the reference's acceptance rule (test/gemm/fpequals.h:38-53) for float32 output of f16 input
bool close_f16(float x, float y) {
  const double rel = std::fabs(double(x) - y) / (std::fabs(double(x)) + std::fabs(double(y)) + 1.0);
  return rel <= 10.0 * 0.000976562;
}

struct Cuda {
  CUdevice device{};
  CUcontext context{};
  CUstream stream{};
  Cuda() {
    cu::checkCudaCall(cuInit(0));
    cu::checkCudaCall(cuDeviceGet(&device, 0));
    cu::checkCudaCall(cuDevicePrimaryCtxRetain(&context, device));
    cu::checkCudaCall(cuCtxSetCurrent(context));
    cu::checkCudaCall(cuStreamCreate(&stream, CU_STREAM_DEFAULT));
  }
};

bool all_ones_gemm(Cuda &cuda) {
  // test/cuda/mma.cpp: all-ones input gives Re = 0, Im = 2K
  const size_t B = 3, M = 512, N = 512, K = 512;
  ccglib::mma::GEMM gemm(B, M, N, K, cuda.device, cuda.stream, ccglib::ValueType::float16,
                         ccglib::mma::basic);
  std::vector<half> ones(B * 2 * M * K, __float2half(1.0f));
  std::vector<float> c(B * 2 * M * N, -1.0f);
  CUdeviceptr d_a, d_b, d_c;
  cu::checkCudaCall(cuMemAlloc(&d_a, ones.size() * sizeof(half)));
  cu::checkCudaCall(cuMemAlloc(&d_b, ones.size() * sizeof(half)));
  cu::checkCudaCall(cuMemAlloc(&d_c, c.size() * sizeof(float)));
  cu::checkCudaCall(cuMemcpyHtoD(d_a, ones.data(), ones.size() * sizeof(half)));
  cu::checkCudaCall(cuMemcpyHtoD(d_b, ones.data(), ones.size() * sizeof(half)));
  gemm.Run(d_a, d_b, d_c);
  cu::checkCudaCall(cuStreamSynchronize(cuda.stream));
  cu::checkCudaCall(cuMemcpyDtoH(c.data(), d_c, c.size() * sizeof(float)));
  cuMemFree(d_a);
  cuMemFree(d_b);
  cuMemFree(d_c);
  for (size_t b = 0; b < B; ++b)
    for (size_t i = 0; i < M * N; ++i)
      if (c[(b * 2) * M * N + i] != 0.0f || c[(b * 2 + 1) * M * N + i] != 2.0f * K) return false;
  return true;
}

bool all_ones_pipeline(Cuda &cuda) {
  // test/cuda/pipeline.cpp: planar f16 -> f32, opt variant, device pointers
  const size_t B = 3, M = 512, N = 512, K = 512;
  ccglib::pipeline::Pipeline pipeline(B, M, N, K, cuda.device, cuda.stream, ccglib::complex_planar,
                                      ccglib::complex_planar, ccglib::mma::row_major,
                                      ccglib::mma::col_major, ccglib::mma::row_major,
                                      ccglib::float16, ccglib::float32, ccglib::mma::opt);
  std::vector<half> ones(B * 2 * M * K, __float2half(1.0f));
  std::vector<float> c(B * 2 * M * N, -1.0f);
  CUdeviceptr d_a, d_b, d_c;
  cu::checkCudaCall(cuMemAlloc(&d_a, ones.size() * sizeof(half)));
  cu::checkCudaCall(cuMemAlloc(&d_b, ones.size() * sizeof(half)));
  cu::checkCudaCall(cuMemAlloc(&d_c, c.size() * sizeof(float)));
  cu::checkCudaCall(cuMemcpyHtoD(d_a, ones.data(), ones.size() * sizeof(half)));
  cu::checkCudaCall(cuMemcpyHtoD(d_b, ones.data(), ones.size() * sizeof(half)));
  pipeline.Run(d_a, d_b, d_c);
  cu::checkCudaCall(cuStreamSynchronize(cuda.stream));
  cu::checkCudaCall(cuMemcpyDtoH(c.data(), d_c, c.size() * sizeof(float)));
  cuMemFree(d_a);
  cuMemFree(d_b);
  cuMemFree(d_c);
  for (size_t b = 0; b < B; ++b)
    for (size_t i = 0; i < M * N; ++i)
      if (c[(b * 2) * M * N + i] != 0.0f || c[(b * 2 + 1) * M * N + i] != 2.0f * K) return false;
  return true;
}

bool pipeline_f16_host(ccglib::ComplexAxisLocation in_axis) {
  // test/pipeline/pipeline.cpp:17-86: f16 -> f32, opt, unaligned 300 x 200 x 100, alpha/beta set,
  // host-memory Run through the cu:: overloads
  cu::init();
  cu::Device device(0);
  cu::Context context(CU_CTX_SCHED_BLOCKING_SYNC, device);
  cu::Stream stream;
  const size_t B = 2, M = 300, N = 200, K = 100;
  const std::complex<float> alpha(0.5f, 2.0f), beta(-1.5f, 0.25f);
  ccglib::pipeline::Pipeline pipeline(B, M, N, K, device, stream, in_axis, ccglib::complex_planar,
                                      ccglib::mma::row_major, ccglib::mma::col_major,
                                      ccglib::mma::row_major, ccglib::float16, ccglib::float32,
                                      ccglib::mma::opt, alpha, beta);
  cu::HostMemory h_a(B * 2 * M * K * sizeof(half)), h_b(B * 2 * N * K * sizeof(half)),
      h_c(B * 2 * M * N * sizeof(float));
  std::mt19937 rng(3);
  std::uniform_real_distribution<float> dist(-1.0f, 1.0f);
  std::vector<float> a(B * 2 * M * K), b(B * 2 * N * K), c0(B * 2 * M * N);
  for (auto &x : a) x = __half2float(__float2half(dist(rng)));
  for (auto &x : b) x = __half2float(__float2half(dist(rng)));
  for (auto &x : c0) x = dist(rng);
  half *pa = h_a, *pb = h_b;
  float *pc = h_c;
  auto fill = [&](half *dst, const std::vector<float> &src, size_t rows) {
    for (size_t bb = 0; bb < B; ++bb)
      for (size_t c = 0; c < 2; ++c)
        for (size_t r = 0; r < rows; ++r)
          for (size_t k = 0; k < K; ++k) {
            const float v = src[((bb * 2 + c) * rows + r) * K + k];
            const size_t idx = in_axis == ccglib::complex_planar
                                   ? ((bb * 2 + c) * rows + r) * K + k
                                   : ((bb * rows + r) * K + k) * 2 + c;
            dst[idx] = __float2half(v);
          }
  };
  fill(pa, a, M);
  fill(pb, b, N);
  std::memcpy(pc, c0.data(), c0.size() * sizeof(float));
  pipeline.Run(h_a, h_b, h_c);
  std::vector<float> want = c0;
  for (size_t bb = 0; bb < B; ++bb)
    oracle_cgemm_f32(&a[bb * 2 * M * K], &b[bb * 2 * N * K], &want[bb * 2 * M * N], M, N, K, 0,
                     alpha.real(), alpha.imag(), beta.real(), beta.imag());
  for (size_t i = 0; i < want.size(); ++i)
    if (!close_f16(pc[i], want[i])) return false;
  return true;
}

bool pipeline_int1_host() {
  // test/pipeline/pipeline.cpp:88-187: 1-bit input given as one byte per sample, B = 2, 512^3
  cu::init();
  cu::Device device(0);
  cu::Context context(CU_CTX_SCHED_BLOCKING_SYNC, device);
  cu::Stream stream;
  const size_t B = 2, M = 512, N = 512, K = 512;
  ccglib::pipeline::Pipeline pipeline(B, M, N, K, device, stream, ccglib::complex_planar,
                                      ccglib::complex_planar, ccglib::mma::row_major,
                                      ccglib::mma::col_major, ccglib::mma::row_major, ccglib::int1,
                                      ccglib::int32, ccglib::mma::opt);
  cu::HostMemory h_a(B * 2 * M * K), h_b(B * 2 * N * K), h_c(B * 2 * M * N * sizeof(int));
  std::mt19937 rng(5);
  unsigned char *pa = h_a, *pb = h_b;
  for (size_t i = 0; i < h_a.size(); ++i) pa[i] = rng() & 1;
  for (size_t i = 0; i < h_b.size(); ++i) pb[i] = rng() & 1;
  pipeline.Run(h_a, h_b, h_c);
  std::vector<uint32_t> wa(h_a.size() / 32), wb(h_b.size() / 32);
  oracle_pack_bits(pa, wa.data(), h_a.size(), 0);
  oracle_pack_bits(pb, wb.data(), h_b.size(), 0);
  std::vector<int32_t> want(B * 2 * M * N, 0);
  for (size_t bb = 0; bb < B; ++bb)
    oracle_cgemm_int1(&wa[bb * 2 * M * K / 32], &wb[bb * 2 * N * K / 32], &want[bb * 2 * M * N], M,
                      N, K, 0, 1, 0, 0, 0);
  return std::memcmp(static_cast<int *>(h_c), want.data(), want.size() * sizeof(int)) == 0;
}

// The cu::Stream overloads must enqueue on the CALLER's stream.  A non-blocking stream is not
// ordered against the NULL stream, so an object that silently fell back to stream 0 would read
// the device input before the (long) asynchronous copy on the caller's stream has filled it.
bool packing_on_nonblocking_cu_stream() {
  cu::init();
  cu::Device device(0);
  cu::Context context(CU_CTX_SCHED_BLOCKING_SYNC, device);
  cu::Stream stream(CU_STREAM_NON_BLOCKING);
  const size_t N = size_t{96} << 20;  // 96 Mi samples: the copy in takes milliseconds
  ccglib::packing::Packing pack(N, ccglib::forward, device, stream);
  if (pack.stream() != static_cast<CUstream>(stream)) return false;  // host-only check
  cu::HostMemory h_in(N), h_out(N / 8);
  unsigned char *in = h_in;
  std::mt19937 rng(21);
  for (size_t i = 0; i < N; i += 4) {
    const uint32_t r = rng();
    in[i] = r & 1, in[i + 1] = (r >> 1) & 1, in[i + 2] = (r >> 2) & 1, in[i + 3] = (r >> 3) & 1;
  }
  cu::DeviceMemory d_in(N), d_out(N / 8);
  cu::checkCudaCall(cuMemsetD8(d_in, 0xFF, N));  // what a racing kernel would read
  cu::checkCudaCall(cuMemsetD8(d_out, 0, N / 8));
  cu::checkCudaCall(cuCtxSynchronize());
  stream.memcpyHtoDAsync(d_in, in, N);
  pack.Run(d_in, d_out);
  stream.memcpyDtoHAsync(h_out, d_out, N / 8);
  stream.synchronize();  // only the caller's stream
  std::vector<uint32_t> want(N / 32);
  oracle_pack_bits(in, want.data(), N, 0);
  return std::memcmp(static_cast<uint32_t *>(h_out), want.data(), N / 8) == 0;
}

bool pipeline_on_nonblocking_cu_stream() {
  cu::init();
  cu::Device device(0);
  cu::Context context(CU_CTX_SCHED_BLOCKING_SYNC, device);
  cu::Stream stream(CU_STREAM_NON_BLOCKING);
  const size_t B = 8, M = 512, N = 512, K = 4096;  // 64 MiB per operand
  ccglib::pipeline::Pipeline pipeline(B, M, N, K, device, stream, ccglib::complex_planar,
                                      ccglib::complex_planar, ccglib::mma::row_major,
                                      ccglib::mma::col_major, ccglib::mma::row_major,
                                      ccglib::float16, ccglib::float32, ccglib::mma::opt);
  if (pipeline.stream() != static_cast<CUstream>(stream)) return false;  // host-only check
  ccglib::mma::GEMM gemm(B, M, N, K, device, stream, ccglib::ValueType::float16);
  ccglib::transpose::Transpose transpose(B, M, K, 128, 64, 16, device, stream);
  if (gemm.stream() != static_cast<CUstream>(stream) ||
      transpose.stream() != static_cast<CUstream>(stream)) {
    return false;
  }
  const size_t na = B * 2 * M * K, nb = B * 2 * N * K, nc = B * 2 * M * N;
  cu::HostMemory h_a(na * sizeof(half)), h_b(nb * sizeof(half)), h_c(nc * sizeof(float));
  half *pa = h_a, *pb = h_b;
  float *pc = h_c;
  std::mt19937 rng(23);
  std::uniform_real_distribution<float> dist(-1.0f, 1.0f);
  for (size_t i = 0; i < na; ++i) pa[i] = __float2half(dist(rng));
  for (size_t i = 0; i < nb; ++i) pb[i] = __float2half(dist(rng));
  cu::DeviceMemory d_a(na * sizeof(half)), d_b(nb * sizeof(half)), d_c(nc * sizeof(float));
  cu::checkCudaCall(cuMemsetD8(d_a, 0, na * sizeof(half)));  // a racing kernel would compute 0
  cu::checkCudaCall(cuMemsetD8(d_b, 0, nb * sizeof(half)));
  cu::checkCudaCall(cuCtxSynchronize());
  stream.memcpyHtoDAsync(d_a, pa, na * sizeof(half));
  stream.memcpyHtoDAsync(d_b, pb, nb * sizeof(half));
  pipeline.Run(d_a, d_b, d_c);
  stream.memcpyDtoHAsync(pc, d_c, nc * sizeof(float));
  stream.synchronize();  // only the caller's stream
  // sampled float64 dot products of the same inputs
  for (int s = 0; s < 4000; ++s) {
    const size_t b = rng() % B, m = rng() % M, n = rng() % N;
    double re = 0, im = 0;
    for (size_t k = 0; k < K; ++k) {
      const double ar = __half2float(pa[((b * 2) * M + m) * K + k]);
      const double ai = __half2float(pa[((b * 2 + 1) * M + m) * K + k]);
      const double br = __half2float(pb[((b * 2) * N + n) * K + k]);
      const double bi = __half2float(pb[((b * 2 + 1) * N + n) * K + k]);
      re += ar * br - ai * bi;
      im += ar * bi + ai * br;
    }
    const double tol = 4.0 * std::sqrt(2.0 * K) * 5.96e-8 * K;  // S <= 2K for |values| <= 1
    if (std::fabs(pc[((b * 2) * M + m) * N + n] - re) > tol ||
        std::fabs(pc[((b * 2 + 1) * M + m) * N + n] - im) > tol) {
      return false;
    }
  }
  return true;
}

bool pipeline_int1_interleaved_in_and_out() {
  // byte samples [B][M][K][2] in (any non-zero byte = +1), interleaved int32 C [B][M][N][2] out
  cu::init();
  cu::Device device(0);
  cu::Context context(CU_CTX_SCHED_BLOCKING_SYNC, device);
  cu::Stream stream(CU_STREAM_NON_BLOCKING);
  const size_t B = 5, M = 200, N = 136, K = 1056;
  ccglib::pipeline::Pipeline pipeline(B, M, N, K, device, stream, ccglib::complex_interleaved,
                                      ccglib::complex_interleaved, ccglib::mma::row_major,
                                      ccglib::mma::col_major, ccglib::mma::row_major, ccglib::int1,
                                      ccglib::int32, ccglib::mma::basic);
  cu::HostMemory h_a(B * 2 * M * K), h_b(B * 2 * N * K), h_c(B * 2 * M * N * sizeof(int));
  std::mt19937 rng(29);
  unsigned char *pa = h_a, *pb = h_b;
  for (size_t i = 0; i < h_a.size(); ++i) pa[i] = (rng() & 1) * (1 + rng() % 200);  // non-zero = +1
  for (size_t i = 0; i < h_b.size(); ++i) pb[i] = rng() & 1;
  pipeline.Run(h_a, h_b, h_c);
  // oracle: de-interleave per batch item, pack, multiply
  std::vector<int32_t> want(2 * M * N);
  const int *got = h_c;
  for (size_t bb = 0; bb < B; ++bb) {
    std::vector<uint8_t> a_pl(2 * M * K), b_pl(2 * N * K);
    for (size_t r = 0; r < M; ++r)
      for (size_t k = 0; k < K; ++k)
        for (size_t c = 0; c < 2; ++c) a_pl[(c * M + r) * K + k] = pa[((bb * M + r) * K + k) * 2 + c];
    for (size_t r = 0; r < N; ++r)
      for (size_t k = 0; k < K; ++k)
        for (size_t c = 0; c < 2; ++c) b_pl[(c * N + r) * K + k] = pb[((bb * N + r) * K + k) * 2 + c];
    std::vector<uint32_t> wa(2 * M * K / 32), wb(2 * N * K / 32);
    oracle_pack_bits(a_pl.data(), wa.data(), a_pl.size(), 0);
    oracle_pack_bits(b_pl.data(), wb.data(), b_pl.size(), 0);
    std::fill(want.begin(), want.end(), 0);
    oracle_cgemm_int1(wa.data(), wb.data(), want.data(), M, N, K, 0, 1, 0, 0, 0);
    for (size_t m = 0; m < M; ++m)
      for (size_t n = 0; n < N; ++n)
        for (size_t c = 0; c < 2; ++c)
          if (got[((bb * M + m) * N + n) * 2 + c] != want[(c * M + m) * N + n]) return false;
  }
  return true;
}

bool transpose_cases(Cuda &cuda) {
  // test/transpose/transpose.cpp:37-46 (B=2, 256 x 128, chunks 64 x 64), host and device input
  const size_t B = 2, M = 256, N = 128, Mc = 64, Nc = 64;
  bool ok = true;
  for (int interleaved = 0; interleaved < 2; ++interleaved) {
    std::vector<uint16_t> in(B * 2 * M * N), want(in.size()), got(in.size());
    std::mt19937 rng(7 + interleaved);
    for (auto &x : in) x = static_cast<uint16_t>(rng());
    oracle_transpose(in.data(), want.data(), B, M, N, Mc, Nc, 16, interleaved);
    ccglib::transpose::Transpose transpose(
        B, M, N, Mc, Nc, 16, cuda.device, cuda.stream,
        interleaved ? ccglib::complex_interleaved : ccglib::complex_planar);
    CUdeviceptr d_in, d_out;
    cu::checkCudaCall(cuMemAlloc(&d_in, in.size() * 2));
    cu::checkCudaCall(cuMemAlloc(&d_out, in.size() * 2));
    cu::checkCudaCall(cuMemcpyHtoD(d_in, in.data(), in.size() * 2));
    transpose.Run(d_in, d_out);
    cu::checkCudaCall(cuStreamSynchronize(cuda.stream));
    cu::checkCudaCall(cuMemcpyDtoH(got.data(), d_out, got.size() * 2));
    ok = ok && got == want;
    cu::checkCudaCall(cuMemsetD8(d_out, 0, in.size() * 2));
    transpose.Run(static_cast<const void *>(in.data()), d_out);  // host input overload
    cu::checkCudaCall(cuStreamSynchronize(cuda.stream));
    cu::checkCudaCall(cuMemcpyDtoH(got.data(), d_out, got.size() * 2));
    ok = ok && got == want;
    cuMemFree(d_in);
    cuMemFree(d_out);
  }
  return ok;
}

bool packing_cases(Cuda &cuda) {
  // test/packing/packing.cpp:22-204 (N = 2048): pack, unpack, round trip, interleaved pack
  const size_t N = 2048;
  std::vector<uint8_t> bytes(N), back(N);
  std::mt19937 rng(9);
  for (auto &x : bytes) x = rng() & 1;
  std::vector<uint32_t> want(N / 32), got(N / 32), want_il(N / 32);
  oracle_pack_bits(bytes.data(), want.data(), N, 0);
  oracle_pack_bits(bytes.data(), want_il.data(), N, 1);
  CUdeviceptr d_bytes, d_words;
  cu::checkCudaCall(cuMemAlloc(&d_bytes, N));
  cu::checkCudaCall(cuMemAlloc(&d_words, N / 8));
  bool ok = true;
  {
    ccglib::packing::Packing pack(N, ccglib::forward, cuda.device, cuda.stream);
    pack.Run(bytes.data(), d_words);  // host input overload
    cu::checkCudaCall(cuStreamSynchronize(cuda.stream));
    cu::checkCudaCall(cuMemcpyDtoH(got.data(), d_words, N / 8));
    ok = ok && got == want;
    ccglib::packing::Packing unpack(N, ccglib::backward, cuda.device, cuda.stream);
    unpack.Run(d_words, d_bytes);
    cu::checkCudaCall(cuStreamSynchronize(cuda.stream));
    cu::checkCudaCall(cuMemcpyDtoH(back.data(), d_bytes, N));
    ok = ok && back == bytes;
  }
  {
    ccglib::packing::Packing pack(N, ccglib::forward, cuda.device, cuda.stream,
                                  ccglib::complex_interleaved);
    cu::checkCudaCall(cuMemcpyHtoD(d_bytes, bytes.data(), N));
    pack.Run(d_bytes, d_words);
    cu::checkCudaCall(cuStreamSynchronize(cuda.stream));
    cu::checkCudaCall(cuMemcpyDtoH(got.data(), d_words, N / 8));
    ok = ok && got == want_il;
  }
  cuMemFree(d_bytes);
  cuMemFree(d_words);
  return ok;
}

bool throws_with(const std::function<void()> &body, const char *needle) {
  try {
    body();
  } catch (const std::exception &e) {
    return std::strstr(e.what(), needle) != nullptr;
  }
  return false;
}

bool error_cases(Cuda &cuda) {
  bool ok = true;
  // test/gemm/mma.cpp:598-643: A col-major is reported under the reference's error name
  ok = ok && throws_with(
                 [&] {
                   ccglib::mma::GEMM(16, 16, 16, 256, cuda.device, cuda.stream,
                                     ccglib::ValueType::float16, ccglib::mma::basic,
                                     ccglib::complex_planar, ccglib::mma::row_major,
                                     ccglib::mma::col_major, ccglib::mma::col_major);
                 },
                 "NVRTC_ERROR_COMPILATION");
  ok = ok && throws_with(
                 [&] {
                   ccglib::mma::GEMM(16, 16, 16, 256, cuda.device, cuda.stream,
                                     {ccglib::ValueType::int1, ccglib::ValueType::int32},
                                     ccglib::mma::basic, ccglib::complex_planar,
                                     ccglib::mma::row_major, ccglib::mma::col_major,
                                     ccglib::mma::col_major);
                 },
                 "NVRTC_ERROR_COMPILATION");
  // src/mma/GEMM.cpp:77-80
  ok = ok && throws_with(
                 [&] {
                   ccglib::mma::GEMM(1, 16, 16, 64, cuda.device, cuda.stream,
                                     ccglib::ValueType::float16, ccglib::mma::basic,
                                     ccglib::complex_interleaved);
                 },
                 "complex-interleaved output is not supported in basic variant");
  // src/packing/Packing.cpp:49-53
  ok = ok && throws_with(
                 [&] {
                   ccglib::packing::Packing(64, ccglib::backward, cuda.device, cuda.stream,
                                            ccglib::complex_interleaved);
                 },
                 "complex-interleaved input is not supported in unpacking kernel");
  const dim3 dims = ccglib::mma::GEMM::GetDimensions(ccglib::ValueType::float16);
  ok = ok && dims.x == 128 && dims.y == 256 && dims.z == 64;
  ok = ok && ccglib::helper::ceildiv(10, 3) == 4 && ccglib::helper::ceildiv(9, 3) == 3;
  // the architecture predicates reference tests skip on (test/gemm/mma.cpp:530-591)
  {
    cu::Device device(0);
    ok = ok && ccglib::isBlackwell(device.getArch()) && ccglib::hasFP8(device) &&
         !ccglib::isVolta(device) && !ccglib::isCDNA(device) && !ccglib::isUnsupported(device);
  }
  // the CPU verification class is part of the umbrella header
  {
    const float a[4] = {1, 2, 3, 4}, b[4] = {5, 6, 7, 8};  // [2][1][2] each
    float c[2] = {0, 0};
    ccglib::reference::GEMM().Run(a, b, c, 1, 1, 2);
    ok = ok && c[0] == (1 * 5 + 2 * 6) - (3 * 7 + 4 * 8) && c[1] == (1 * 7 + 2 * 8) + (3 * 5 + 4 * 6);
  }
  return ok;
}

} // namespace

int main() {
  Cuda cuda;
  run_case("gemm_all_ones_raw_handles", [&] { return all_ones_gemm(cuda); });
  run_case("pipeline_all_ones_raw_handles", [&] { return all_ones_pipeline(cuda); });
  run_case("pipeline_f16_host_planar", [] { return pipeline_f16_host(ccglib::complex_planar); });
  run_case("pipeline_f16_host_interleaved",
           [] { return pipeline_f16_host(ccglib::complex_interleaved); });
  run_case("pipeline_int1_host", [] { return pipeline_int1_host(); });
  run_case("packing_on_nonblocking_cu_stream", [] { return packing_on_nonblocking_cu_stream(); });
  run_case("pipeline_on_nonblocking_cu_stream", [] { return pipeline_on_nonblocking_cu_stream(); });
  run_case("pipeline_int1_interleaved_in_and_out",
           [] { return pipeline_int1_interleaved_in_and_out(); });
  run_case("transpose_host_and_device", [&] { return transpose_cases(cuda); });
  run_case("packing_host_and_device", [&] { return packing_cases(cuda); });
  run_case("error_cases_and_dims", [&] { return error_cases(cuda); });
  unsigned word = 0;
  ccglib_b200_device_status(&word);
  report("device_status_clean", word == 0);
  std::printf("%d failure(s)\n", failures);
  return failures;
}
