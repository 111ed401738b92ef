// Bit packing / unpacking of 1-bit samples.
//   forward : n bytes (non-zero = 1) -> ceil(n/32) words, sample i in bit i%32 of word i/32;
//             interleaved input [n/2][2] is written planar [2][n/2]
//   backward: words -> n bytes of 0/1
// Pure data movement bounded by HBM bandwidth: each thread handles 16 samples with one 128-bit
// load (forward) or store (backward); bytes are squeezed to bits with a multiply instead of a
// warp ballot.  Scalar kernels cover sizes that are not multiples of the vector width.
//
// Replaces the reference's pack_bits / unpack_bits (kernels/packing_kernel.cu:7-62, one byte per
// thread) and their launcher (src/packing/Packing.cpp:65-74).
#include "common.cuh"

namespace ccglib_b200 {
namespace {

// 4 bytes (non-zero = set) -> 4 bits (byte i -> bit i).
__device__ __forceinline__ uint32_t squeeze4(uint32_t x) {
  const uint32_t nz = ((x | ((x & 0x7F7F7F7Fu) + 0x7F7F7F7Fu)) & 0x80808080u) >> 7;
  return ((nz * 0x00204081u) >> 21) & 0xFu;
}

__device__ __forceinline__ uint32_t squeeze16(const uint4 &v) {
  return squeeze4(v.x) | (squeeze4(v.y) << 4) | (squeeze4(v.z) << 8) | (squeeze4(v.w) << 12);
}

// 4 bits -> 4 bytes of 0/1.
__device__ __forceinline__ uint32_t spread4(uint32_t nibble) {
  return (nibble * 0x00204081u) & 0x01010101u;
}

// Planar forward: unit = 16 input bytes; lane pairs combine their 16 bits into one word.
// `units` is even (n multiple of 32) and the block size a multiple of 32, so both lanes of a
// pair are always active together.
__global__ void __launch_bounds__(256)
pack_planar_kernel(const uint4 *__restrict__ in, uint32_t *__restrict__ out, size_t units) {
  constexpr int kUnroll = 4;  // independent 16-byte loads in flight per thread
  const size_t span = static_cast<size_t>(blockDim.x) * kUnroll;
  for (size_t base = blockIdx.x * span; base < units; base += static_cast<size_t>(gridDim.x) * span) {
    uint32_t bits[kUnroll];
#pragma unroll
    for (int j = 0; j < kUnroll; ++j) {
      const size_t u = base + j * blockDim.x + threadIdx.x;
      bits[j] = u < units ? squeeze16(__ldg(in + u)) : 0u;
    }
#pragma unroll
    for (int j = 0; j < kUnroll; ++j) {
      const size_t u = base + j * blockDim.x + threadIdx.x;
      const uint32_t other = __shfl_xor_sync(0xFFFFFFFFu, bits[j], 1);
      if (u < units && (threadIdx.x & 1) == 0) out[u >> 1] = bits[j] | (other << 16);
    }
  }
}

// Interleaved forward (n multiple of 64): unit = 16 input bytes = 8 (re, im) pairs -> 8 real bits
// and 8 imaginary bits; four lanes combine into one real word and one imaginary word.
__global__ void __launch_bounds__(256)
pack_interleaved_kernel(const uint4 *__restrict__ in, uint32_t *__restrict__ out, size_t units,
                        size_t imag_word_offset) {
  constexpr int kUnroll = 4;
  const size_t span = static_cast<size_t>(blockDim.x) * kUnroll;
  for (size_t base = blockIdx.x * span; base < units; base += static_cast<size_t>(gridDim.x) * span) {
    uint4 v[kUnroll];
#pragma unroll
    for (int j = 0; j < kUnroll; ++j) {
      const size_t u = base + j * blockDim.x + threadIdx.x;
      v[j] = u < units ? __ldg(in + u) : make_uint4(0, 0, 0, 0);
    }
#pragma unroll
    for (int j = 0; j < kUnroll; ++j) {
      const size_t u = base + j * blockDim.x + threadIdx.x;
      // bytes r0 i0 r1 i1 | ... : gather real bytes and imaginary bytes, then squeeze
      const uint32_t r01 = __byte_perm(v[j].x, v[j].y, 0x6420u);
      const uint32_t i01 = __byte_perm(v[j].x, v[j].y, 0x7531u);
      const uint32_t r23 = __byte_perm(v[j].z, v[j].w, 0x6420u);
      const uint32_t i23 = __byte_perm(v[j].z, v[j].w, 0x7531u);
      uint32_t re = squeeze4(r01) | (squeeze4(r23) << 4);
      uint32_t im = squeeze4(i01) | (squeeze4(i23) << 4);
      const uint32_t shift = (threadIdx.x & 3) * 8;
      re <<= shift;
      im <<= shift;
      re |= __shfl_xor_sync(0xFFFFFFFFu, re, 1);
      im |= __shfl_xor_sync(0xFFFFFFFFu, im, 1);
      re |= __shfl_xor_sync(0xFFFFFFFFu, re, 2);
      im |= __shfl_xor_sync(0xFFFFFFFFu, im, 2);
      if (u < units && (threadIdx.x & 3) == 0) {
        out[u >> 2] = re;
        out[(u >> 2) + imag_word_offset] = im;
      }
    }
  }
}

// Any n: one thread per output word, byte loads.
__global__ void __launch_bounds__(256)
pack_scalar_kernel(const uint8_t *__restrict__ in, uint32_t *__restrict__ out, size_t n,
                   int interleaved) {
  const size_t words = ceil_div<size_t>(n, 32);
  for (size_t w = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; w < words;
       w += static_cast<size_t>(gridDim.x) * blockDim.x) {
    uint32_t bits = 0;
    for (int i = 0; i < 32; ++i) {
      const size_t t = w * 32 + i;
      if (t >= n) break;
      size_t src = t;
      if (interleaved) {
        src = 2 * t;
        if (src >= n) src -= n - 1;
      }
      if (in[src] != 0) bits |= 1u << i;
    }
    out[w] = bits;
  }
}

// Backward: unit = 16 output bytes.
__global__ void __launch_bounds__(256)
unpack_kernel(const uint32_t *__restrict__ in, uint8_t *__restrict__ out, size_t n) {
  constexpr int kUnroll = 4;  // independent loads, then independent 16-byte stores, per thread
  const size_t units = n / 16;
  const size_t span = static_cast<size_t>(blockDim.x) * kUnroll;
  for (size_t base = blockIdx.x * span; base < units; base += static_cast<size_t>(gridDim.x) * span) {
    uint32_t half[kUnroll];
#pragma unroll
    for (int j = 0; j < kUnroll; ++j) {
      const size_t u = base + j * blockDim.x + threadIdx.x;
      half[j] = u < units ? (__ldg(in + (u >> 1)) >> ((u & 1) * 16)) & 0xFFFFu : 0u;
    }
#pragma unroll
    for (int j = 0; j < kUnroll; ++j) {
      const size_t u = base + j * blockDim.x + threadIdx.x;
      if (u < units) {
        *reinterpret_cast<uint4 *>(out + u * 16) =
            make_uint4(spread4(half[j] & 0xFu), spread4((half[j] >> 4) & 0xFu),
                       spread4((half[j] >> 8) & 0xFu), spread4((half[j] >> 12) & 0xFu));
      }
    }
  }
  if (blockIdx.x == 0 && threadIdx.x == 0) {
    for (size_t t = units * 16; t < n; ++t) out[t] = (in[t / 32] >> (t % 32)) & 1u;
  }
}

unsigned grid_for(size_t units) {
  const size_t blocks = ceil_div<size_t>(units, 256);
  const size_t cap = static_cast<size_t>(sm_count()) * 32;
  return static_cast<unsigned>(blocks < cap ? (blocks ? blocks : 1) : cap);
}

} // namespace
} // namespace ccglib_b200

using namespace ccglib_b200;

extern "C" int ccglib_b200_pack_run(size_t n, int direction, int input_complex_axis,
                                    const void *d_in, void *d_out, void *stream_v) {
  if (d_in == nullptr || d_out == nullptr || n == 0) {
    set_last_error("pack_run: null pointer or zero size");
    return CCGLIB_B200_INVALID_ARGUMENT;
  }
  if (input_complex_axis != CCGLIB_B200_PLANAR && input_complex_axis != CCGLIB_B200_INTERLEAVED) {
    set_last_error("pack_run: unknown complex axis location %d", input_complex_axis);
    return CCGLIB_B200_INVALID_ARGUMENT;
  }
  cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
  const bool interleaved = input_complex_axis == CCGLIB_B200_INTERLEAVED;
  if (direction == CCGLIB_B200_BACKWARD) {
    if (interleaved) {
      set_last_error("complex-interleaved input is not supported in unpacking kernel");
      return CCGLIB_B200_UNSUPPORTED;
    }
    if (!aligned16(d_out)) {
      set_last_error("pack_run: output must be 16-byte aligned");
      return CCGLIB_B200_INVALID_ARGUMENT;
    }
    unpack_kernel<<<grid_for(ceil_div<size_t>(n / 16, 4) + 1), 256, 0, stream>>>(static_cast<const uint32_t *>(d_in),
                                                           static_cast<uint8_t *>(d_out), n);
  } else if (direction == CCGLIB_B200_FORWARD) {
    const bool vec = aligned16(d_in) && (interleaved ? n % 64 == 0 : n % 32 == 0);
    if (!vec) {
      pack_scalar_kernel<<<grid_for(ceil_div<size_t>(n, 32)), 256, 0, stream>>>(
          static_cast<const uint8_t *>(d_in), static_cast<uint32_t *>(d_out), n,
          interleaved ? 1 : 0);
    } else if (interleaved) {
      pack_interleaved_kernel<<<grid_for(ceil_div<size_t>(n / 16, 4)), 256, 0, stream>>>(
          static_cast<const uint4 *>(d_in), static_cast<uint32_t *>(d_out), n / 16, n / 64);
    } else {
      pack_planar_kernel<<<grid_for(ceil_div<size_t>(n / 16, 4)), 256, 0, stream>>>(
          static_cast<const uint4 *>(d_in), static_cast<uint32_t *>(d_out), n / 16);
    }
  } else {
    set_last_error("pack_run: unknown direction %d", direction);
    return CCGLIB_B200_INVALID_ARGUMENT;
  }
  CCGLIB_CUDA_TRY(cudaGetLastError());
  return CCGLIB_B200_OK;
}
