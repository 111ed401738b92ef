// C++ classes with the names, constructor arguments and Run() overloads of the reference's public
// API, implemented header-only on top of the C ABI in <ccglib_b200.h>:
//
//   ccglib::mma::GEMM                (reference include/ccglib/gemm/mma.h:27-68)
//   ccglib::transpose::Transpose     (reference include/ccglib/transpose/transpose.h:14-54)
//   ccglib::packing::Packing         (reference include/ccglib/packing/packing.h:25-54)
//   ccglib::pipeline::Pipeline       (reference include/ccglib/pipeline/pipeline.h:28-73)
//   value types / enums              (reference include/ccglib/common/*.h, gemm/mem_order.h,
//                                     gemm/variant.h)
//
// Callers keep ownership of devices, streams and A/B/C; objects enqueue work on the caller's
// stream in call order and never synchronise, except the host-memory overload of Pipeline::Run
// (as in the reference, src/pipeline/Pipeline.cpp:162-176).  Errors are C++ exceptions
// (std::runtime_error) carrying the C ABI's message text.
//
// The cu::Device / cu::Stream / cu::DeviceMemory / cu::HostMemory overloads are compiled when
// <cudawrappers/cu.hpp> can be included; they use nothing of those classes beyond their
// conversion operators to the raw CUDA handles and size().  Programs link libccglib_b200 and
// libcuda.
#ifndef CCGLIB_B200_API_HPP_
#define CCGLIB_B200_API_HPP_

#include <climits>
#include <complex>
#include <cstddef>
#include <stdexcept>
#include <string>

#include <cuda.h>
#include <vector_types.h>  // dim3

#include <ccglib_b200.h>

#if !defined(CCGLIB_B200_NO_CUDAWRAPPERS) && defined(__has_include)
#if __has_include(<cudawrappers/cu.hpp>)
#include <cudawrappers/cu.hpp>
#define CCGLIB_B200_HAVE_CUDAWRAPPERS 1
#endif
#endif

namespace ccglib {

// ---- vocabulary: the enumerator values are part of the C ABI -----------------------------------

enum ValueType { int1, int32, bfloat16, float8e4m3, float8e5m2, float16, float32 };

constexpr size_t CalculateBitWidth(ValueType type) {
  return type == int1 ? 1
         : (type == float8e4m3 || type == float8e5m2) ? 8
         : (type == bfloat16 || type == float16)      ? 16
         : (type == float32 || type == int32)         ? 32
                                                      : 0;
}

struct ValuePrecision {
  constexpr ValuePrecision(ValueType t) : type(t), num_bits(CalculateBitWidth(t)) {}
  constexpr ValuePrecision(ValueType t, size_t bits) : type(t), num_bits(bits) {}
  constexpr bool operator==(const ValuePrecision &other) const { return type == other.type; }
  constexpr bool operator==(const ValueType &other) const { return type == other; }
  constexpr operator ValueType() const { return type; }
  constexpr size_t GetBitWidth() const { return num_bits; }

private:
  const ValueType type;
  const size_t num_bits;
};

// Input and output value types of a GEMM; the output defaults to float32.
struct Precision {
  constexpr Precision(const ValueType in) : input_type(in), output_type(float32) {}
  constexpr Precision(const ValueType in, const ValueType out) : input_type(in), output_type(out) {}
  constexpr Precision(const ValuePrecision in) : input_type(in), output_type(float32) {}
  constexpr Precision(const ValuePrecision in, const ValuePrecision out)
      : input_type(in), output_type(out) {}
  constexpr size_t GetInputBits() const { return input_type.GetBitWidth(); }
  constexpr size_t GetOutputBits() const { return output_type.GetBitWidth(); }
  const ValuePrecision input_type;
  const ValuePrecision output_type;
};

// complex_planar: [batch][2][...]; complex_interleaved: [batch][...][2]
enum ComplexAxisLocation { complex_planar, complex_interleaved };
enum Direction { forward, backward };

namespace helper {
template <typename T> inline T ceildiv(T a, T b) { return a / b + (a % b != 0); }
inline size_t ceildiv(size_t a, unsigned int b) { return ceildiv(a, static_cast<size_t>(b)); }
} // namespace helper

namespace mma {
enum MemOrder { row_major, col_major };
enum Variant { basic, opt };
} // namespace mma

namespace detail {

inline void check(int status) {
  if (status == CCGLIB_B200_OK) return;
  std::string text = ccglib_b200_last_error();
  if (status == CCGLIB_B200_UNSUPPORTED && text.find("-major") != std::string::npos) {
    // The reference rejects these layouts inside its run-time kernel compilation and existing
    // callers match on that error name (reference test/gemm/mma.cpp:598-643).
    text = "NVRTC_ERROR_COMPILATION: " + text;
  }
  throw std::runtime_error(text);
}

inline void check(CUresult result, const char *what) {
  if (result == CUDA_SUCCESS) return;
  const char *name = nullptr;
  cuGetErrorString(result, &name);
  throw std::runtime_error(std::string(what) + ": " + (name ? name : "unknown CUDA error"));
}

inline void *ptr(CUdeviceptr p) { return reinterpret_cast<void *>(p); }

} // namespace detail

// ---- GEMM ---------------------------------------------------------------------------------------

namespace mma {

class GEMM {
public:
  GEMM(size_t B_, size_t M_, size_t N_, size_t K_, CUdevice &device, CUstream &stream,
       Precision precision, Variant variant = Variant::opt,
       ComplexAxisLocation c_complex_axis_location = ComplexAxisLocation::complex_planar,
       MemOrder c_mem_order = MemOrder::row_major, MemOrder a_mem_order = MemOrder::row_major,
       MemOrder b_mem_order = MemOrder::col_major, std::complex<float> alpha = {1, 0},
       std::complex<float> beta = {0, 0})
      : stream_(stream) {
    (void)device;  // the current context's device is used, as with the reference
    create(B_, M_, N_, K_, precision, variant, c_complex_axis_location, c_mem_order, a_mem_order,
           b_mem_order, alpha, beta);
  }
  ~GEMM() { ccglib_b200_gemm_plan_destroy(plan_); }
  GEMM(const GEMM &) = delete;
  GEMM &operator=(const GEMM &) = delete;

  // Asynchronous on the stream given at construction; no allocation, no synchronisation.
  void Run(CUdeviceptr d_a, CUdeviceptr d_b, CUdeviceptr d_c) {
    detail::check(ccglib_b200_gemm_run(plan_, detail::ptr(d_a), detail::ptr(d_b),
                                       detail::ptr(d_c), stream_));
  }

  // The stream this object enqueues on (the handle given at construction).
  CUstream stream() const { return stream_; }

  // (m_per_block, n_per_block, k_per_chunk) of the tiled layout the opt variant reads.
  static dim3 GetDimensions(Precision precision, Variant variant = Variant::opt) {
    unsigned d[3];
    detail::check(ccglib_b200_gemm_dims(static_cast<ValueType>(precision.input_type),
                                        static_cast<ValueType>(precision.output_type), variant, d));
    return dim3(d[0], d[1], d[2]);
  }

#ifdef CCGLIB_B200_HAVE_CUDAWRAPPERS
  GEMM(size_t B_, size_t M_, size_t N_, size_t K_, cu::Device &device, cu::Stream &stream,
       Precision precision, Variant variant = Variant::opt,
       ComplexAxisLocation c_complex_axis_location = ComplexAxisLocation::complex_planar,
       MemOrder c_mem_order = MemOrder::row_major, MemOrder a_mem_order = MemOrder::row_major,
       MemOrder b_mem_order = MemOrder::col_major, std::complex<float> alpha = {1, 0},
       std::complex<float> beta = {0, 0})
      : stream_(static_cast<CUstream>(stream)) {
    (void)device;
    create(B_, M_, N_, K_, precision, variant, c_complex_axis_location, c_mem_order, a_mem_order,
           b_mem_order, alpha, beta);
  }
  void Run(cu::DeviceMemory &d_a, cu::DeviceMemory &d_b, cu::DeviceMemory &d_c) {
    Run(static_cast<CUdeviceptr>(d_a), static_cast<CUdeviceptr>(d_b),
        static_cast<CUdeviceptr>(d_c));
  }
#endif

private:
  void create(size_t B_, size_t M_, size_t N_, size_t K_, Precision precision, Variant variant,
              ComplexAxisLocation c_axis, MemOrder c_order, MemOrder a_order, MemOrder b_order,
              std::complex<float> alpha, std::complex<float> beta) {
    ccglib_b200_gemm_desc d{};
    d.batch = B_;
    d.m = M_;
    d.n = N_;
    d.k = K_;
    d.type_in = static_cast<ValueType>(precision.input_type);
    d.type_out = static_cast<ValueType>(precision.output_type);
    d.variant = variant;
    d.c_complex_axis = c_axis;
    d.a_mem_order = a_order;
    d.b_mem_order = b_order;
    d.c_mem_order = c_order;
    d.alpha_re = alpha.real();
    d.alpha_im = alpha.imag();
    d.beta_re = beta.real();
    d.beta_im = beta.imag();
    detail::check(ccglib_b200_gemm_plan_create(&d, &plan_));
  }

  ccglib_b200_gemm_plan *plan_ = nullptr;
  CUstream stream_;
};

} // namespace mma

// ---- Transpose ----------------------------------------------------------------------------------

namespace transpose {

class Transpose {
public:
  Transpose(size_t B, size_t M, size_t N, size_t M_chunk, size_t N_chunk, size_t nr_bits,
            CUdevice &device, CUstream &stream,
            ComplexAxisLocation input_complex_axis_location = ComplexAxisLocation::complex_planar)
      : B_(B), M_(M), N_(N), M_chunk_(M_chunk), N_chunk_(N_chunk), nr_bits_(nr_bits),
        axis_(input_complex_axis_location), stream_(stream) {
    (void)device;
  }

  void Run(CUdeviceptr d_input, CUdeviceptr d_output) {
    detail::check(ccglib_b200_transpose_run(B_, M_, N_, M_chunk_, N_chunk_, nr_bits_, axis_,
                                            detail::ptr(d_input), detail::ptr(d_output), stream_));
  }

  // Host input: stream-ordered temporary, copy, transpose, free (no synchronisation).
  void Run(const void *h_input, CUdeviceptr d_output) {
    const size_t bytes = InputBytes();
    CUdeviceptr tmp = 0;
    detail::check(cuMemAllocAsync(&tmp, bytes, stream_), "cuMemAllocAsync");
    detail::check(cuMemcpyHtoDAsync(tmp, h_input, bytes, stream_), "cuMemcpyHtoDAsync");
    Run(tmp, d_output);
    detail::check(cuMemFreeAsync(tmp, stream_), "cuMemFreeAsync");
  }

  // The stream this object enqueues on (the handle given at construction).
  CUstream stream() const { return stream_; }

  // Bytes of the input array ([B][2][M][N] elements of nr_bits each).
  size_t InputBytes() const { return B_ * 2 * M_ * N_ * nr_bits_ / CHAR_BIT; }
  // Bytes of the zero-padded tiled output.
  size_t OutputBytes() const {
    return B_ * 2 * helper::ceildiv(M_, M_chunk_) * M_chunk_ * helper::ceildiv(N_, N_chunk_) *
           N_chunk_ * nr_bits_ / CHAR_BIT;
  }

#ifdef CCGLIB_B200_HAVE_CUDAWRAPPERS
  Transpose(size_t B, size_t M, size_t N, size_t M_chunk, size_t N_chunk, size_t nr_bits,
            cu::Device &device, cu::Stream &stream,
            ComplexAxisLocation input_complex_axis_location = ComplexAxisLocation::complex_planar)
      : B_(B), M_(M), N_(N), M_chunk_(M_chunk), N_chunk_(N_chunk), nr_bits_(nr_bits),
        axis_(input_complex_axis_location), stream_(static_cast<CUstream>(stream)) {
    (void)device;
  }
  void Run(cu::HostMemory &h_input, cu::DeviceMemory &d_output) {
    Run(static_cast<const void *>(static_cast<void *>(h_input)),
        static_cast<CUdeviceptr>(d_output));
  }
  void Run(cu::DeviceMemory &d_input, cu::DeviceMemory &d_output) {
    Run(static_cast<CUdeviceptr>(d_input), static_cast<CUdeviceptr>(d_output));
  }
#endif

protected:
  size_t B_, M_, N_, M_chunk_, N_chunk_, nr_bits_;

private:
  ComplexAxisLocation axis_;
  CUstream stream_;
};

} // namespace transpose

// ---- Packing ------------------------------------------------------------------------------------

namespace packing {

class Packing {
public:
  Packing(size_t N, Direction direction, CUdevice &device, CUstream &stream,
          ComplexAxisLocation input_complex_axis_location = ComplexAxisLocation::complex_planar)
      : Packing(FromHandles{}, N, direction, device, stream, input_complex_axis_location) {}

  void Run(CUdeviceptr d_input, CUdeviceptr d_output) {
    detail::check(ccglib_b200_pack_run(N_, direction_, axis_, detail::ptr(d_input),
                                       detail::ptr(d_output), stream_));
  }

  // Host input: N bytes when packing, ceil(N/32) words when unpacking.
  void Run(unsigned char *h_input, CUdeviceptr d_output) {
    const size_t bytes = direction_ == Direction::forward ? N_ : 4 * helper::ceildiv(N_, size_t{32});
    CUdeviceptr tmp = 0;
    detail::check(cuMemAllocAsync(&tmp, bytes, stream_), "cuMemAllocAsync");
    detail::check(cuMemcpyHtoDAsync(tmp, h_input, bytes, stream_), "cuMemcpyHtoDAsync");
    Run(tmp, d_output);
    detail::check(cuMemFreeAsync(tmp, stream_), "cuMemFreeAsync");
  }

#ifdef CCGLIB_B200_HAVE_CUDAWRAPPERS
  Packing(size_t N, Direction direction, cu::Device &device, cu::Stream &stream,
          ComplexAxisLocation input_complex_axis_location = ComplexAxisLocation::complex_planar)
      : Packing(FromHandles{}, N, direction, static_cast<CUdevice>(device),
                static_cast<CUstream>(stream), input_complex_axis_location) {}
  void Run(cu::HostMemory &h_input, cu::DeviceMemory &d_output) {
    Run(static_cast<unsigned char *>(static_cast<void *>(h_input)),
        static_cast<CUdeviceptr>(d_output));
  }
  void Run(cu::DeviceMemory &d_input, cu::DeviceMemory &d_output) {
    Run(static_cast<CUdeviceptr>(d_input), static_cast<CUdeviceptr>(d_output));
  }
#endif

  // The stream this object enqueues on (the handle given at construction).
  CUstream stream() const { return stream_; }

private:
  // Both public constructors delegate here with the raw handles taken BY VALUE, so the stored
  // stream is the caller's whichever overload was used.
  struct FromHandles {};
  Packing(FromHandles, size_t N, Direction direction, CUdevice device, CUstream stream,
          ComplexAxisLocation input_complex_axis_location)
      : N_(N), direction_(direction), axis_(input_complex_axis_location), stream_(stream) {
    (void)device;
    if (direction == Direction::backward &&
        input_complex_axis_location == ComplexAxisLocation::complex_interleaved) {
      throw std::runtime_error("complex-interleaved input is not supported in unpacking kernel");
    }
  }

  size_t N_;
  Direction direction_;
  ComplexAxisLocation axis_;
  CUstream stream_;
};

} // namespace packing

// ---- Pipeline -----------------------------------------------------------------------------------

namespace pipeline {

// The caller's matrices in their natural layout -> C: for floating-point input transpose (opt
// variant only) -> gemm; for 1-bit input, given as one byte per sample, the GEMM's own front end
// turns the bytes into tensor-core operands, so nothing is packed or tiled first.  The object
// owns the intermediate buffers (allocated once at construction; the device slices of the
// host-memory Run at its first call).
class Pipeline {
public:
  Pipeline(size_t B, size_t M, size_t N, size_t K, CUdevice &device, CUstream &stream,
           ComplexAxisLocation input_complex_axis_location,
           ComplexAxisLocation output_complex_axis_location, mma::MemOrder a_mem_order,
           mma::MemOrder b_mem_order, mma::MemOrder c_mem_order, ValuePrecision input_precision,
           ValuePrecision output_precision, mma::Variant variant = mma::Variant::opt,
           std::complex<float> alpha = {1, 0}, std::complex<float> beta = {0, 0})
      : stream_(stream) {
    (void)device;  // the current context's device is used, as with the reference
    create(B, M, N, K, input_complex_axis_location, output_complex_axis_location, a_mem_order,
           b_mem_order, c_mem_order, input_precision, output_precision, variant, alpha, beta);
  }
  ~Pipeline() { ccglib_b200_pipeline_destroy(pipeline_); }
  Pipeline(const Pipeline &) = delete;
  Pipeline &operator=(const Pipeline &) = delete;

  // Device operands: asynchronous on the stream given at construction, no allocation.
  void Run(CUdeviceptr d_a, CUdeviceptr d_b, CUdeviceptr d_c) {
    detail::check(ccglib_b200_pipeline_run(pipeline_, detail::ptr(d_a), detail::ptr(d_b),
                                           detail::ptr(d_c), stream_));
  }

  // Host operands: batch slices are copied in, run and copied back double-buffered; returns when
  // C is complete in host memory (as the reference's host-memory Run, which synchronises too).
  void RunHost(const void *a, const void *b, void *c) {
    detail::check(ccglib_b200_pipeline_run_host(pipeline_, a, b, c, stream_));
  }

  // The stream this object enqueues on (the handle given at construction).
  CUstream stream() const { return stream_; }

#ifdef CCGLIB_B200_HAVE_CUDAWRAPPERS
  Pipeline(size_t B, size_t M, size_t N, size_t K, cu::Device &device, cu::Stream &stream,
           ComplexAxisLocation input_complex_axis_location,
           ComplexAxisLocation output_complex_axis_location, mma::MemOrder a_mem_order,
           mma::MemOrder b_mem_order, mma::MemOrder c_mem_order, ValuePrecision input_precision,
           ValuePrecision output_precision, mma::Variant variant = mma::Variant::opt,
           std::complex<float> alpha = {1, 0}, std::complex<float> beta = {0, 0})
      : stream_(static_cast<CUstream>(stream)) {
    (void)device;
    create(B, M, N, K, input_complex_axis_location, output_complex_axis_location, a_mem_order,
           b_mem_order, c_mem_order, input_precision, output_precision, variant, alpha, beta);
  }
  void Run(cu::HostMemory &a, cu::HostMemory &b, cu::HostMemory &c) {
    RunHost(static_cast<void *>(a), static_cast<void *>(b), static_cast<void *>(c));
  }
  void Run(cu::DeviceMemory &d_a, cu::DeviceMemory &d_b, cu::DeviceMemory &d_c) {
    Run(static_cast<CUdeviceptr>(d_a), static_cast<CUdeviceptr>(d_b),
        static_cast<CUdeviceptr>(d_c));
  }
#endif

private:
  void create(size_t B, size_t M, size_t N, size_t K, ComplexAxisLocation in_axis,
              ComplexAxisLocation out_axis, mma::MemOrder a_order, mma::MemOrder b_order,
              mma::MemOrder c_order, ValuePrecision in, ValuePrecision out, mma::Variant variant,
              std::complex<float> alpha, std::complex<float> beta) {
    ccglib_b200_pipeline_desc d{};
    d.batch = B;
    d.m = M;
    d.n = N;
    d.k = K;
    d.type_in = static_cast<ValueType>(in);
    d.type_out = static_cast<ValueType>(out);
    d.variant = variant;
    d.input_complex_axis = in_axis;
    d.output_complex_axis = out_axis;
    d.a_mem_order = a_order;
    d.b_mem_order = b_order;
    d.c_mem_order = c_order;
    d.alpha_re = alpha.real();
    d.alpha_im = alpha.imag();
    d.beta_re = beta.real();
    d.beta_im = beta.imag();
    detail::check(ccglib_b200_pipeline_create(&d, &pipeline_));
  }

  ccglib_b200_pipeline *pipeline_ = nullptr;
  CUstream stream_;
};

} // namespace pipeline
} // namespace ccglib
#endif // CCGLIB_B200_API_HPP_
