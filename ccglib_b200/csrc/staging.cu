// Re-staging kernels used by the GEMM plan when the caller's operands cannot be read by TMA as
// they are:
//   * expand_bits: packed 1-bit samples (bit 1 = +1, bit 0 = -1) -> one signed byte (or one e2m1
//     nibble) per sample, planes (re, im[, -im]); tcgen05 has no 1-bit MMA and its integer kind
//     has no negate bit, so the +-1 values (and the negated imaginary plane of A) are produced
//     here.
//   * pad_rows: copies rows whose byte length is not a multiple of 16 to a 16-byte pitch.
// Both are pure data movement bounded by HBM bandwidth.
#include "common.cuh"

namespace ccglib_b200 {
namespace {

// 4 bits -> 4 bytes of 0/1 (bit i -> byte i).
__device__ __forceinline__ uint32_t spread_nibble(uint32_t nibble) {
  return (nibble * 0x00204081u) & 0x01010101u;
}

// 8 bits -> 8 nibbles (bit j -> bit 4j).
__device__ __forceinline__ uint32_t spread_byte(uint32_t v) {
  uint32_t x = (v | (v << 12)) & 0x000F000Fu;
  x = (x | (x << 6)) & 0x03030303u;
  x = (x | (x << 3)) & 0x11111111u;
  return x;
}

// One word of 32 samples (bit set = +1, clear = -1; only the first `valid` count) -> the operand
// bytes of unit `u` of `out_row`, and of the same row of the next plane negated when
// `negated_plane`.  NIBBLES: 16 bytes, sample i in nibble i, +1 = 0x2 (e2m1 1.0), -1 = 0xA,
// padding = 0.  Else 32 signed bytes, +1 = 0x01, -1 = 0xFF, padding = 0.
template <bool NIBBLES>
__device__ __forceinline__ void emit_word(uint32_t w, int valid, int8_t *out_row, size_t u,
                                          size_t out_row_bytes, bool negated_plane,
                                          size_t plane_bytes) {
  if constexpr (NIBBLES) {
    uint32_t pos[4], neg[4];
    if (valid == 32) {  // every word but possibly the last of a row: no padding mask
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const uint32_t sign = spread_byte(__byte_perm(w, 0, 0x4440 + q));  // bit j -> bit 4j
        neg[q] = 0x22222222u | (sign << 3);
        pos[q] = neg[q] ^ 0x88888888u;
      }
    } else {
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const uint32_t sign = spread_byte((w >> (8 * q)) & 0xFFu);
        uint32_t mask = 0xFFFFFFFFu;
        if (8 * q + 8 > valid) mask = (8 * q >= valid) ? 0u : ((1u << (4 * (valid - 8 * q))) - 1u);
        pos[q] = (0x22222222u | ((~sign & 0x11111111u) << 3)) & mask;
        neg[q] = (0x22222222u | (sign << 3)) & mask;
      }
    }
    uint4 *dst = reinterpret_cast<uint4 *>(out_row + u * 16);
    *dst = make_uint4(pos[0], pos[1], pos[2], pos[3]);
    if (negated_plane) {
      *reinterpret_cast<uint4 *>(reinterpret_cast<int8_t *>(dst) + plane_bytes) =
          make_uint4(neg[0], neg[1], neg[2], neg[3]);
    }
  } else {
    uint32_t pos[8], neg[8];
#pragma unroll
    for (int q = 0; q < 8; ++q) {
      const uint32_t y = spread_nibble((w >> (4 * q)) & 0xFu);
      uint32_t mask = 0xFFFFFFFFu;
      if (4 * q + 4 > valid) mask = (4 * q >= valid) ? 0u : ((1u << (8 * (valid - 4 * q))) - 1u);
      pos[q] = (0xFFFFFFFFu - y * 0xFEu) & mask;  // 1 -> 0x01, 0 -> 0xFF
      neg[q] = (0x01010101u + y * 0xFEu) & mask;  // 1 -> 0xFF, 0 -> 0x01
    }
    int8_t *dst = out_row + u * 32;
    const bool second = u * 32 + 16 < out_row_bytes;  // the row pitch is a multiple of 16
    *reinterpret_cast<uint4 *>(dst) = make_uint4(pos[0], pos[1], pos[2], pos[3]);
    if (second) *reinterpret_cast<uint4 *>(dst + 16) = make_uint4(pos[4], pos[5], pos[6], pos[7]);
    if (negated_plane) {
      int8_t *dn = dst + plane_bytes;
      *reinterpret_cast<uint4 *>(dn) = make_uint4(neg[0], neg[1], neg[2], neg[3]);
      if (second) {
        *reinterpret_cast<uint4 *>(dn + 16) = make_uint4(neg[4], neg[5], neg[6], neg[7]);
      }
    }
  }
}

struct ExpandParams {
  const uint32_t *in;
  int8_t *out;
  size_t batch, rows, k_bits, out_row_bytes;
  size_t units;      // 32-byte output units (= input words) per row
  size_t words;      // input words per row
  int planes_out;    // 2: (re, im); 3: (re, im, -im)
  int nibbles;       // 0: one signed byte per sample; 1: one e2m1 nibble per sample (+-1.0)
  int tiled;
  size_t blk, kc_words, row_tiles, k_tiles;
};

// A warp expands a block of 128 consecutive words of one row, lane l taking words l, l + 32,
// l + 64, l + 96, so every load instruction reads 128 contiguous bytes and every store instruction
// writes 512 (nibbles) or 2 x 512 (bytes) contiguous bytes.  One warp per block (no grid-stride
// loop): the row/plane arithmetic is two divisions per 4096 samples, in 32 bits whenever the
// number of blocks allows.
template <bool NIBBLES, typename Index>
__global__ void __launch_bounds__(256) expand_bits_warp_kernel(const ExpandParams p) {
  const Index blocks_per_row = static_cast<Index>(ceil_div<size_t>(p.words, 128));
  const Index rows = static_cast<Index>(p.rows);
  const size_t unit = blockIdx.x * static_cast<size_t>(blockDim.x / 32) + (threadIdx.x >> 5);
  if (unit >= p.batch * 2 * p.rows * static_cast<size_t>(blocks_per_row)) return;
  const uint32_t lane = threadIdx.x & 31;
  const Index row_id = static_cast<Index>(unit) / blocks_per_row;
  const size_t blk = static_cast<Index>(unit) - row_id * blocks_per_row;
  const Index plane_id = row_id / rows;
  const size_t r = row_id - plane_id * rows;
  const size_t c = plane_id & 1;
  const size_t b = plane_id >> 1;
  const size_t plane_bytes = p.rows * p.out_row_bytes;
  const bool negated_plane = c == 1 && p.planes_out == 3;
  int8_t *out_row = p.out + ((b * p.planes_out + c) * p.rows + r) * p.out_row_bytes;
  const size_t rt = r / p.blk, rr = r - rt * p.blk;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const size_t u = blk * 128 + i * 32 + lane;  // word within the row
    if (u >= p.words) continue;
    size_t src;
    if (p.tiled) {
      const size_t kt = u / p.kc_words, uu = u - kt * p.kc_words;
      src = ((((b * p.row_tiles + rt) * p.k_tiles + kt) * 2 + c) * p.blk + rr) * p.kc_words + uu;
    } else {
      src = ((b * 2 + c) * p.rows + r) * p.words + u;
    }
    const uint32_t w = __ldg(p.in + src);
    const size_t bit0 = u * 32;
    const int valid = static_cast<int>(p.k_bits - bit0 < 32 ? p.k_bits - bit0 : 32);
    emit_word<NIBBLES>(w, valid, out_row, u, p.out_row_bytes, negated_plane, plane_bytes);
  }
}

// 4 bytes (non-zero = set) -> 4 bits (byte i -> bit i), the packing rule of the reference's
// pack_bits (kernels/packing_kernel.cu:25-29: a ballot over "byte != 0").
__device__ __forceinline__ uint32_t squeeze4(uint32_t x) {
  const uint32_t nz = ((x | ((x & 0x7F7F7F7Fu) + 0x7F7F7F7Fu)) & 0x80808080u) >> 7;
  return ((nz * 0x00204081u) >> 21) & 0xFu;
}

__device__ __forceinline__ uint32_t squeeze16(const uint4 &v) {
  return squeeze4(v.x) | (squeeze4(v.y) << 4) | (squeeze4(v.z) << 8) | (squeeze4(v.w) << 12);
}

// 8 samples (bit set = +1, clear = -1; only the first `valid` count) -> 8 e2m1 nibbles, sample j
// in nibble j: +1 = 0x2 (1.0), -1 = 0xA (-1.0), padding = 0.  `neg` is the negated row.
__device__ __forceinline__ void nibbles8(uint32_t bits, int valid, uint32_t &pos, uint32_t &neg) {
  const uint32_t sign = spread_byte(bits & 0xFFu);
  const uint32_t mask = valid >= 8 ? 0xFFFFFFFFu : (valid <= 0 ? 0u : ((1u << (4 * valid)) - 1u));
  neg = (0x22222222u | (sign << 3)) & mask;
  pos = (neg ^ 0x88888888u) & mask;
}

// 4 samples -> 4 signed bytes: +1 = 0x01, -1 = 0xFF, padding = 0.
__device__ __forceinline__ void bytes4(uint32_t bits, int valid, uint32_t &pos, uint32_t &neg) {
  const uint32_t y = spread_nibble(bits & 0xFu);
  const uint32_t mask = valid >= 4 ? 0xFFFFFFFFu : (valid <= 0 ? 0u : ((1u << (8 * valid)) - 1u));
  pos = (0xFFFFFFFFu - y * 0xFEu) & mask;
  neg = (0x01010101u + y * 0xFEu) & mask;
}

// 4 one-byte samples -> the low nibble of each byte holds the e2m1 code of the sample:
// non-zero = +1.0 = 0x2, zero = -1.0 = 0xA (high nibbles are 0).
__device__ __forceinline__ uint32_t nibble_codes4(uint32_t w) {
  const uint32_t nz = ((w & 0x7F7F7F7Fu) + 0x7F7F7F7Fu) | w;  // bit 7 of a byte: byte != 0
  return ((~nz >> 4) & 0x08080808u) | 0x02020202u;
}

// 16 samples of one plane (one 16-byte piece) -> 16 nibbles, sample j in nibble j.
__device__ __forceinline__ uint2 nibbles_of_piece(const uint4 &x) {
  uint32_t t[4];
  const uint32_t w[4] = {x.x, x.y, x.z, x.w};
#pragma unroll
  for (int q = 0; q < 4; ++q) {
    const uint32_t v = nibble_codes4(w[q]);
    t[q] = v | (v >> 4);  // byte 0 = samples 0, 1; byte 2 = samples 2, 3
  }
  return make_uint2(__byte_perm(t[0], t[1], 0x6420u), __byte_perm(t[2], t[3], 0x6420u));
}

// 8 (re, im) pairs (one 16-byte piece of interleaved input) -> 8 real and 8 imaginary nibbles.
__device__ __forceinline__ void nibbles_of_pairs(const uint4 &x, uint32_t &re, uint32_t &im) {
  uint32_t t[4];
  const uint32_t w[4] = {x.x, x.y, x.z, x.w};
#pragma unroll
  for (int q = 0; q < 4; ++q) {
    const uint32_t v = nibble_codes4(w[q]);  // bytes: re0, im0, re1, im1
    t[q] = v | (v >> 12);                    // byte 0 = re0 | re1 << 4, byte 1 = im0 | im1 << 4
  }
  const uint32_t lo = __byte_perm(t[0], t[1], 0x5140u);  // re(t0), re(t1), im(t0), im(t1)
  const uint32_t hi = __byte_perm(t[2], t[3], 0x5140u);
  re = __byte_perm(lo, hi, 0x5410u);
  im = __byte_perm(lo, hi, 0x7632u);
}

struct ExpandBytesParams {
  const uint8_t *in;
  int8_t *out;
  size_t batch, rows, k, out_row_bytes;
  size_t pieces;   // 16-byte input pieces per output row (covers the whole row pitch)
  int planes_out;  // 2: (re, im); 3: (re, im, -im)
  int vec_ok;      // every row of the input starts on a 16-byte boundary
};

// The fused front end of the 1-bit Pipeline: one-byte samples (non-zero = +1, zero = -1, the
// rule of the reference's pack_bits), planar [batch][2][rows][K] or interleaved
// [batch][rows][K][2], straight to the planes the tensor cores read, without the packed words in
// between.  The unit of work is one 16-byte piece of an input row: 16 samples of one plane, or 8
// (re, im) pairs.  A warp takes 128 consecutive pieces of a row, lane l the pieces l, l + 32,
// l + 64, l + 96, so every load instruction reads 512 contiguous bytes and every store
// instruction 128 to 512 contiguous bytes of each output plane.  Pieces past K (row padding up to
// the 16-byte pitch) are written as zeros.
template <bool NIBBLES, bool INTERLEAVED>
__global__ void __launch_bounds__(256) expand_bytes_warp_kernel(const ExpandBytesParams p) {
  constexpr int kSamples = INTERLEAVED ? 8 : 16;                       // samples per piece
  constexpr int kOutBytes = NIBBLES ? kSamples / 2 : kSamples;         // per piece and plane
  const size_t blocks_per_row = ceil_div<size_t>(p.pieces, 128);
  const size_t planes_in = INTERLEAVED ? 1 : 2;
  const size_t unit = blockIdx.x * static_cast<size_t>(blockDim.x / 32) + (threadIdx.x >> 5);
  if (unit >= p.batch * planes_in * p.rows * blocks_per_row) return;
  const uint32_t lane = threadIdx.x & 31;
  const size_t row_id = unit / blocks_per_row;
  const size_t blk = unit - row_id * blocks_per_row;
  const size_t plane_id = row_id / p.rows;
  const size_t r = row_id - plane_id * p.rows;
  const size_t c = INTERLEAVED ? 0 : (plane_id & 1);
  const size_t b = INTERLEAVED ? plane_id : (plane_id >> 1);
  const size_t plane_bytes = p.rows * p.out_row_bytes;
  int8_t *out_row = p.out + ((b * p.planes_out + c) * p.rows + r) * p.out_row_bytes;
  const uint8_t *in_row = INTERLEAVED ? p.in + (b * p.rows + r) * p.k * 2
                                      : p.in + ((b * 2 + c) * p.rows + r) * p.k;
  // full pieces of nibble output take the direct route (about two integer operations per
  // sample, so that the pass stays bound by memory); ragged tails and the signed-byte form go
  // through the bit masks
  uint4 raw[4];
  uint32_t re[4], im[4];
  int valid[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const size_t u = blk * 128 + i * 32 + lane;  // piece within the row
    const size_t k0 = u * kSamples;
    valid[i] = (u < p.pieces && k0 < p.k)
                   ? static_cast<int>(p.k - k0 < kSamples ? p.k - k0 : kSamples)
                   : 0;
    re[i] = im[i] = 0;
    raw[i] = make_uint4(0, 0, 0, 0);
    if (valid[i] == kSamples && p.vec_ok) {
      raw[i] = __ldg(reinterpret_cast<const uint4 *>(in_row) + u);
      if constexpr (!NIBBLES) {
        if constexpr (INTERLEAVED) {
          re[i] = squeeze4(__byte_perm(raw[i].x, raw[i].y, 0x6420u)) |
                  (squeeze4(__byte_perm(raw[i].z, raw[i].w, 0x6420u)) << 4);
          im[i] = squeeze4(__byte_perm(raw[i].x, raw[i].y, 0x7531u)) |
                  (squeeze4(__byte_perm(raw[i].z, raw[i].w, 0x7531u)) << 4);
        } else {
          re[i] = squeeze16(raw[i]);
        }
      }
    } else {
      for (int j = 0; j < valid[i]; ++j) {
        if constexpr (INTERLEAVED) {
          re[i] |= (in_row[2 * (k0 + j)] != 0 ? 1u : 0u) << j;
          im[i] |= (in_row[2 * (k0 + j) + 1] != 0 ? 1u : 0u) << j;
        } else {
          re[i] |= (in_row[k0 + j] != 0 ? 1u : 0u) << j;
        }
      }
    }
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const size_t u = blk * 128 + i * 32 + lane;
    if (u >= p.pieces) continue;
    int8_t *dst = out_row + u * kOutBytes;
    if constexpr (NIBBLES) {
      if (valid[i] == kSamples && p.vec_ok) {
        if constexpr (INTERLEAVED) {
          uint32_t r, m;
          nibbles_of_pairs(raw[i], r, m);
          *reinterpret_cast<uint32_t *>(dst) = r;
          *reinterpret_cast<uint32_t *>(dst + plane_bytes) = m;
          if (p.planes_out == 3) *reinterpret_cast<uint32_t *>(dst + 2 * plane_bytes) = m ^ 0x88888888u;
        } else {
          const uint2 v = nibbles_of_piece(raw[i]);
          *reinterpret_cast<uint2 *>(dst) = v;
          if (p.planes_out == 3 && c == 1) {
            *reinterpret_cast<uint2 *>(dst + plane_bytes) =
                make_uint2(v.x ^ 0x88888888u, v.y ^ 0x88888888u);
          }
        }
        continue;
      }
    }
    // plane `c` from re[]; with interleaved input also plane 1 from im[]
#pragma unroll
    for (int part = 0; part < (INTERLEAVED ? 2 : 1); ++part) {
      const uint32_t bits = part == 0 ? re[i] : im[i];
      int8_t *d = dst + part * plane_bytes;
      const bool negated = p.planes_out == 3 && (INTERLEAVED ? part == 1 : c == 1);
      uint32_t pos[4], neg[4];
      if constexpr (NIBBLES) {
#pragma unroll
        for (int q = 0; q < kSamples / 8; ++q) {
          nibbles8(bits >> (8 * q), valid[i] - 8 * q, pos[q], neg[q]);
        }
        if constexpr (INTERLEAVED) {
          *reinterpret_cast<uint32_t *>(d) = pos[0];
          if (negated) *reinterpret_cast<uint32_t *>(d + plane_bytes) = neg[0];
        } else {
          *reinterpret_cast<uint2 *>(d) = make_uint2(pos[0], pos[1]);
          if (negated) *reinterpret_cast<uint2 *>(d + plane_bytes) = make_uint2(neg[0], neg[1]);
        }
      } else {
#pragma unroll
        for (int q = 0; q < kSamples / 4; ++q) {
          bytes4(bits >> (4 * q), valid[i] - 4 * q, pos[q], neg[q]);
        }
        if constexpr (INTERLEAVED) {
          *reinterpret_cast<uint2 *>(d) = make_uint2(pos[0], pos[1]);
          if (negated) *reinterpret_cast<uint2 *>(d + plane_bytes) = make_uint2(neg[0], neg[1]);
        } else {
          *reinterpret_cast<uint4 *>(d) = make_uint4(pos[0], pos[1], pos[2], pos[3]);
          if (negated) {
            *reinterpret_cast<uint4 *>(d + plane_bytes) = make_uint4(neg[0], neg[1], neg[2], neg[3]);
          }
        }
      }
    }
  }
}

__global__ void __launch_bounds__(256)
pad_rows_kernel(const uint8_t *__restrict__ in, uint8_t *__restrict__ out, size_t rows,
                size_t row_bytes, size_t out_row_bytes) {
  const size_t vec_per_row = out_row_bytes / 16;
  const size_t total = rows * vec_per_row;
  for (size_t gid = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; gid < total;
       gid += static_cast<size_t>(gridDim.x) * blockDim.x) {
    const size_t r = gid / vec_per_row;
    const size_t off = (gid - r * vec_per_row) * 16;
    const uint8_t *src = in + r * row_bytes + off;
    uint32_t w[4] = {0, 0, 0, 0};
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      if (off + i < row_bytes) w[i >> 2] |= static_cast<uint32_t>(src[i]) << (8 * (i & 3));
    }
    *reinterpret_cast<uint4 *>(out + r * out_row_bytes + off) = make_uint4(w[0], w[1], w[2], w[3]);
  }
}

unsigned grid_for(size_t total, int threads) {
  const size_t blocks = ceil_div<size_t>(total, threads);
  const size_t cap = static_cast<size_t>(sm_count()) * 32;
  return static_cast<unsigned>(blocks < cap ? (blocks ? blocks : 1) : cap);
}

} // namespace

int launch_expand_bits(const void *d_in, void *d_out, size_t batch, size_t rows, size_t k_bits,
                       size_t out_row_bytes, int planes_out, bool tiled, size_t blk,
                       size_t k_c_bits, cudaStream_t stream, bool nibbles) {
  ExpandParams p{};
  p.in = static_cast<const uint32_t *>(d_in);
  p.out = static_cast<int8_t *>(d_out);
  p.batch = batch;
  p.rows = rows;
  p.k_bits = k_bits;
  p.out_row_bytes = out_row_bytes;
  p.words = ceil_div<size_t>(k_bits, 32);
  p.units = p.words;
  p.planes_out = planes_out;
  p.nibbles = nibbles ? 1 : 0;
  p.tiled = tiled ? 1 : 0;
  p.blk = blk;
  p.kc_words = k_c_bits / 32;
  p.row_tiles = ceil_div<size_t>(rows, blk);
  p.k_tiles = ceil_div<size_t>(p.words, p.kc_words);
  const size_t units = batch * 2 * rows * ceil_div<size_t>(p.words, 128);  // one warp each
  const size_t blocks = ceil_div<size_t>(units, 8);
  if (blocks > 0x7FFFFFFFull) {
    set_last_error("expand_bits: too many rows for one launch");
    return CCGLIB_B200_INVALID_ARGUMENT;
  }
  const unsigned grid = static_cast<unsigned>(blocks);
  const bool narrow = units <= 0xFFFFFFFFull;
  if (nibbles) {
    if (narrow) {
      expand_bits_warp_kernel<true, uint32_t><<<grid, 256, 0, stream>>>(p);
    } else {
      expand_bits_warp_kernel<true, size_t><<<grid, 256, 0, stream>>>(p);
    }
  } else {
    if (narrow) {
      expand_bits_warp_kernel<false, uint32_t><<<grid, 256, 0, stream>>>(p);
    } else {
      expand_bits_warp_kernel<false, size_t><<<grid, 256, 0, stream>>>(p);
    }
  }
  CCGLIB_CUDA_TRY(cudaGetLastError());
  return CCGLIB_B200_OK;
}

int launch_expand_bytes(const void *d_in, void *d_out, size_t batch, size_t rows, size_t k,
                        size_t out_row_bytes, int planes_out, bool interleaved, cudaStream_t stream,
                        bool nibbles) {
  ExpandBytesParams p{};
  p.in = static_cast<const uint8_t *>(d_in);
  p.out = static_cast<int8_t *>(d_out);
  p.batch = batch;
  p.rows = rows;
  p.k = k;
  p.out_row_bytes = out_row_bytes;
  // output bytes per 16-byte input piece and plane: 16 or 8 samples as nibbles or bytes
  const size_t out_per_piece = (interleaved ? 8 : 16) / (nibbles ? 2 : 1);
  p.pieces = out_row_bytes / out_per_piece;
  p.planes_out = planes_out;
  p.vec_ok = (aligned16(d_in) && (interleaved ? 2 * k : k) % 16 == 0) ? 1 : 0;
  const size_t units = batch * (interleaved ? 1 : 2) * rows * ceil_div<size_t>(p.pieces, 128);
  const size_t blocks = ceil_div<size_t>(units, 8);
  if (blocks > 0x7FFFFFFFull) {
    set_last_error("expand_bytes: too many rows for one launch");
    return CCGLIB_B200_INVALID_ARGUMENT;
  }
  const unsigned grid = static_cast<unsigned>(blocks);
  if (nibbles) {
    if (interleaved) {
      expand_bytes_warp_kernel<true, true><<<grid, 256, 0, stream>>>(p);
    } else {
      expand_bytes_warp_kernel<true, false><<<grid, 256, 0, stream>>>(p);
    }
  } else {
    if (interleaved) {
      expand_bytes_warp_kernel<false, true><<<grid, 256, 0, stream>>>(p);
    } else {
      expand_bytes_warp_kernel<false, false><<<grid, 256, 0, stream>>>(p);
    }
  }
  CCGLIB_CUDA_TRY(cudaGetLastError());
  return CCGLIB_B200_OK;
}

int launch_pad_rows(const void *d_in, void *d_out, size_t rows, size_t row_bytes,
                    size_t out_row_bytes, cudaStream_t stream) {
  const size_t total = rows * (out_row_bytes / 16);
  pad_rows_kernel<<<grid_for(total, 256), 256, 0, stream>>>(
      static_cast<const uint8_t *>(d_in), static_cast<uint8_t *>(d_out), rows, row_bytes,
      out_row_bytes);
  CCGLIB_CUDA_TRY(cudaGetLastError());
  return CCGLIB_B200_OK;
}

} // namespace ccglib_b200
