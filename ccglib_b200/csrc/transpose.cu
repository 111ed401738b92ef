// Tile transpose into the layout the opt GEMM variant consumes:
//   [B][2][M][N] (planar) or [B][M][N][2] (interleaved)
//     -> [B][ceil(M/Mc)][ceil(N/Nc)][2][Mc][Nc], zero padded.
// Pure data movement, bounded by HBM bandwidth: every thread moves 16 bytes of the real plane and
// 16 bytes of the imaginary plane with 128-bit loads and stores; consecutive threads write
// consecutive 16-byte vectors of the output, so stores are fully coalesced and loads come in runs
// of Nc elements.  Interleaved input is de-interleaved in registers with byte permutes.
// A scalar kernel covers shapes whose rows are not multiples of 16 bytes.
//
// Replaces the reference's transpose kernel (kernels/transpose_kernel.cu:50-82, one element per
// thread) and its launcher (src/transpose/Transpose.cpp:58-73).
#include "common.cuh"

namespace ccglib_b200 {
namespace {

struct TransposeParams {
  const uint8_t *in;
  uint8_t *out;
  size_t B, M, N;      // N in elements (words for 1-bit data)
  size_t Mc, Nc;       // chunk sizes in elements
  size_t Mt, Nt;       // chunks per dimension
};

template <int ES> __device__ __forceinline__ void deinterleave(const uint4 &lo, const uint4 &hi,
                                                               uint4 &re, uint4 &im) {
  if constexpr (ES == 4) {
    re = make_uint4(lo.x, lo.z, hi.x, hi.z);
    im = make_uint4(lo.y, lo.w, hi.y, hi.w);
  } else {
    constexpr uint32_t kRe = (ES == 2) ? 0x5410u : 0x6420u;
    constexpr uint32_t kIm = (ES == 2) ? 0x7632u : 0x7531u;
    re = make_uint4(__byte_perm(lo.x, lo.y, kRe), __byte_perm(lo.z, lo.w, kRe),
                    __byte_perm(hi.x, hi.y, kRe), __byte_perm(hi.z, hi.w, kRe));
    im = make_uint4(__byte_perm(lo.x, lo.y, kIm), __byte_perm(lo.z, lo.w, kIm),
                    __byte_perm(hi.x, hi.y, kIm), __byte_perm(hi.z, hi.w, kIm));
  }
}

// Requires: Nc*ES and N*ES multiples of 16, 16-byte aligned pointers.
template <int ES, bool INTERLEAVED>
__global__ void __launch_bounds__(256) transpose_vec_kernel(const TransposeParams p) {
  constexpr size_t kPerVec = 16 / ES;
  const size_t vpr = p.Nc / kPerVec;  // vectors per chunk row
  const size_t total = p.B * p.Mt * p.Nt * p.Mc * vpr;
  const size_t plane_bytes = p.Mc * p.Nc * ES;
  for (size_t gid = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; gid < total;
       gid += static_cast<size_t>(gridDim.x) * blockDim.x) {
    const size_t j = gid % vpr;
    size_t t = gid / vpr;
    const size_t mc = t % p.Mc;
    t /= p.Mc;
    const size_t nt = t % p.Nt;
    t /= p.Nt;
    const size_t mt = t % p.Mt;
    const size_t b = t / p.Mt;
    const size_t m = mt * p.Mc + mc;
    const size_t n = nt * p.Nc + j * kPerVec;
    uint4 re = make_uint4(0, 0, 0, 0), im = make_uint4(0, 0, 0, 0);
    if (m < p.M && n < p.N) {
      if constexpr (INTERLEAVED) {
        const uint4 *src =
            reinterpret_cast<const uint4 *>(p.in + (((b * p.M + m) * p.N + n) * 2) * ES);
        const uint4 lo = __ldg(src);
        const uint4 hi = __ldg(src + 1);
        deinterleave<ES>(lo, hi, re, im);
      } else {
        const uint8_t *src = p.in + (((b * 2) * p.M + m) * p.N + n) * ES;
        re = __ldg(reinterpret_cast<const uint4 *>(src));
        im = __ldg(reinterpret_cast<const uint4 *>(src + p.M * p.N * ES));
      }
    }
    uint8_t *dst = p.out + (((b * p.Mt + mt) * p.Nt + nt) * 2) * plane_bytes +
                   (mc * p.Nc + j * kPerVec) * ES;
    *reinterpret_cast<uint4 *>(dst) = re;
    *reinterpret_cast<uint4 *>(dst + plane_bytes) = im;
  }
}

// Any shape: one thread per output element pair (re, im).
template <typename T, bool INTERLEAVED>
__global__ void __launch_bounds__(256) transpose_scalar_kernel(const TransposeParams p) {
  const T *in = reinterpret_cast<const T *>(p.in);
  T *out = reinterpret_cast<T *>(p.out);
  const size_t total = p.B * p.Mt * p.Nt * p.Mc * p.Nc;
  const size_t plane = p.Mc * p.Nc;
  for (size_t gid = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; gid < total;
       gid += static_cast<size_t>(gridDim.x) * blockDim.x) {
    const size_t nc = gid % p.Nc;
    size_t t = gid / p.Nc;
    const size_t mc = t % p.Mc;
    t /= p.Mc;
    const size_t nt = t % p.Nt;
    t /= p.Nt;
    const size_t mt = t % p.Mt;
    const size_t b = t / p.Mt;
    const size_t m = mt * p.Mc + mc;
    const size_t n = nt * p.Nc + nc;
    T re = 0, im = 0;
    if (m < p.M && n < p.N) {
      if constexpr (INTERLEAVED) {
        const size_t s = ((b * p.M + m) * p.N + n) * 2;
        re = in[s];
        im = in[s + 1];
      } else {
        const size_t s = ((b * 2) * p.M + m) * p.N + n;
        re = in[s];
        im = in[s + p.M * p.N];
      }
    }
    const size_t d = (((b * p.Mt + mt) * p.Nt + nt) * 2) * plane + mc * p.Nc + nc;
    out[d] = re;
    out[d + plane] = im;
  }
}

template <int ES, typename T>
int launch(const TransposeParams &p, bool interleaved, bool vec, cudaStream_t stream) {
  const size_t total = p.B * p.Mt * p.Nt * p.Mc * (vec ? p.Nc / (16 / ES) : p.Nc);
  const size_t blocks = ceil_div<size_t>(total, 256);
  const size_t cap = static_cast<size_t>(sm_count()) * 32;
  const unsigned grid = static_cast<unsigned>(blocks < cap ? (blocks ? blocks : 1) : cap);
  if (vec) {
    if (interleaved) {
      transpose_vec_kernel<ES, true><<<grid, 256, 0, stream>>>(p);
    } else {
      transpose_vec_kernel<ES, false><<<grid, 256, 0, stream>>>(p);
    }
  } else {
    if (interleaved) {
      transpose_scalar_kernel<T, true><<<grid, 256, 0, stream>>>(p);
    } else {
      transpose_scalar_kernel<T, false><<<grid, 256, 0, stream>>>(p);
    }
  }
  CCGLIB_CUDA_TRY(cudaGetLastError());
  return CCGLIB_B200_OK;
}

} // namespace
} // namespace ccglib_b200

using namespace ccglib_b200;

extern "C" int ccglib_b200_transpose_run(size_t batch, size_t m, size_t n, size_t m_chunk,
                                         size_t n_chunk, size_t nr_bits, int input_complex_axis,
                                         const void *d_in, void *d_out, void *stream_v) {
  if (d_in == nullptr || d_out == nullptr || batch == 0 || m == 0 || n == 0 || m_chunk == 0 ||
      n_chunk == 0) {
    set_last_error("transpose_run: null pointer or zero size");
    return CCGLIB_B200_INVALID_ARGUMENT;
  }
  if (input_complex_axis != CCGLIB_B200_PLANAR && input_complex_axis != CCGLIB_B200_INTERLEAVED) {
    set_last_error("transpose_run: unknown complex axis location %d", input_complex_axis);
    return CCGLIB_B200_INVALID_ARGUMENT;
  }
  size_t es;
  size_t n_el = n, nc_el = n_chunk;
  if (nr_bits == 1) {
    if (n % 32 != 0 || n_chunk % 32 != 0) {
      set_last_error("transpose_run: for 1-bit data N and N_chunk must be multiples of 32");
      return CCGLIB_B200_INVALID_ARGUMENT;
    }
    es = 4;
    n_el = n / 32;
    nc_el = n_chunk / 32;
  } else if (nr_bits == 8 || nr_bits == 16 || nr_bits == 32) {
    es = nr_bits / 8;
  } else {
    set_last_error("transpose_run: nr_bits must be 1, 8, 16 or 32");
    return CCGLIB_B200_INVALID_ARGUMENT;
  }
  TransposeParams p{};
  p.in = static_cast<const uint8_t *>(d_in);
  p.out = static_cast<uint8_t *>(d_out);
  p.B = batch;
  p.M = m;
  p.N = n_el;
  p.Mc = m_chunk;
  p.Nc = nc_el;
  p.Mt = ceil_div(m, m_chunk);
  p.Nt = ceil_div(n_el, nc_el);
  const bool interleaved = input_complex_axis == CCGLIB_B200_INTERLEAVED;
  const bool vec = (nc_el * es) % 16 == 0 && (n_el * es) % 16 == 0 && aligned16(d_in) &&
                   aligned16(d_out);
  cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
  switch (es) {
  case 1:
    return launch<1, uint8_t>(p, interleaved, vec, stream);
  case 2:
    return launch<2, uint16_t>(p, interleaved, vec, stream);
  default:
    return launch<4, uint32_t>(p, interleaved, vec, stream);
  }
}
