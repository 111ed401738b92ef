// Device side of the batched complex GEMM for sm_100a: kernel parameters, shared-memory
// geometry, the epilogue, and the two kernels (one CTA per tile; a cluster of two CTAs per tile).
// Included by gemm.cu only, which instantiates the kernels and owns the host-side plan.
//
// One persistent CTA per SM, warp-specialised:
//   warp 0      TMA producer   -- stages [planes][rows][SW bytes] tiles of A and B in swizzled
//                                 shared memory (one 3-D cp.async.bulk.tensor per operand)
//   warp 1      MMA issuer     -- one thread issues tcgen05.mma; per 32-byte k-step four real MMAs
//                                 Re += Ar.Br, Im += Ar.Bi, Im += Ai.Br, Re += (-Ai).Bi into two
//                                 fp32 (or s32) accumulators in tensor memory
//   warps 2..5  epilogue       -- tcgen05.ld the accumulators, apply alpha/beta, convert, and
//                                 store planar/interleaved, row/col-major C
// Stage hand-over uses mbarrier rings (full: TMA complete_tx, empty: tcgen05.commit); the
// accumulator is handed to the epilogue by tcgen05.commit and back by one arrival per warp.
//
// Every wait is bounded: a wait that runs out sets a shared abort flag and a bit in the global
// status word, after which all roles fall through to the common tear-down (TMEM is always freed).
//
// Replaces the reference's wmma_complex_gemm_basic / wmma_complex_gemm_opt
// (kernels/gemm_kernel_float.cu:35-355, kernels/gemm_kernel_int1.cu:64-356) and their
// epilogues (kernels/matrix_operations.h:37-178).
#pragma once

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include "common.cuh"
#include "ptx.cuh"

namespace ccglib_b200 {

// Sticky device-side status word: kernels OR a code into it when a bounded wait gives up.
__device__ unsigned int g_device_status = 0;

#ifdef CCGLIB_B200_TRACE
// Instrumented builds only (-DCCGLIB_B200_TRACE; never in the shipped library): SM clock stamps of
// the first tiles of every CTA of cgemm_tcgen05_kernel: [0] tile start at the MMA issuer,
// [1] last MMA issued, [2] accumulator complete at the epilogue, [3] epilogue done.
constexpr int kTraceTiles = 48;
__device__ long long g_trace[160][kTraceTiles][4];
#define CCGLIB_TRACE(iter, slot)                                                         \
  do {                                                                                   \
    if ((iter) < kTraceTiles && blockIdx.x < 160) g_trace[blockIdx.x][(iter)][(slot)] = clock64(); \
  } while (0)
#else
#define CCGLIB_TRACE(iter, slot) \
  do {                           \
  } while (0)
#endif

namespace {

using namespace ptx;

constexpr int kBlockM = 128;       // rows of A per tile = TMEM lanes
constexpr int kThreads = 192;      // producer warp, MMA warp, four epilogue warps
constexpr int kTmemCols = 512;     // whole tensor memory of the SM
constexpr int kMaxSmem = 227 * 1024;
constexpr long long kWaitLimitCycles = 4000000000ll;  // default wait limit: ~2 s at boost clock

enum CLayout { kPlanarRow = 0, kPlanarCol = 1, kInterRow = 2, kInterCol = 3 };

struct GemmParams {
  uint32_t M, N;
  uint32_t k_blocks;   // k-blocks of SW bytes per tile
  uint32_t tiles_m, tiles_n, group_n;
  uint32_t num_tiles;
  // operand coordinates
  uint32_t tiled;          // 0: [batch][planes][rows][K] arrays, 1: slab layout of the opt variant
  uint32_t k_per_slab;     // tiled: k-blocks per 128-byte slab row (128 / SW)
  uint32_t slabs_k;        // tiled: slabs along K
  uint32_t a_slabs_m;      // tiled: slabs along M
  uint32_t b_slabs_n;      // tiled: slabs along N
  uint32_t b_slab_rows;    // tiled: rows per B slab (n_blk of the layout contract)
  uint32_t idesc, idesc_neg_a;
  // epilogue
  void *c;
  uint32_t c_layout;
  uint32_t have_alpha, have_beta, vec_ok;
  uint32_t epi_tma;  // stage C through shared memory and store it with TMA (row-major, 4-byte)
  uint32_t prefetch;  // k-blocks the producer asks L2 to fetch ahead of its own loads (0 = off)
  float alpha_re, alpha_im, beta_re, beta_im;
  unsigned int *status;
  long long wait_cycles;  // SM clock cycles after which a wait on an mbarrier gives up
};

constexpr int kStagingTile = 32 * 128;  // one staging tile: 32 rows x 128 B
constexpr int kStagingBytes = 4 * 2 * kStagingTile;  // two tiles for each of the four epilogue warps

template <int BN, int SW, int A_PLANES, int EPI> struct Cfg {
  static constexpr int kAPlane = kBlockM * SW;
  static constexpr int kBPlane = BN * SW;
  static constexpr int kABytes = A_PLANES * kAPlane;
  static constexpr int kBBytes = 2 * kBPlane;
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kBarrierBytes = 256;
  static constexpr int kStaging = 4 * EPI * kStagingTile;  // EPI tiles per epilogue warp
  static constexpr int kStagesRaw = (kMaxSmem - 1024 - kBarrierBytes - kStaging) / kStageBytes;
  static constexpr int kStages = kStagesRaw > 8 ? 8 : kStagesRaw;
  static constexpr int kAccStages = (BN <= 128) ? 2 : 1;
  static constexpr int kSmemBytes = kStages * kStageBytes + kStaging + 1024 + kBarrierBytes;
  static_assert(kStages >= 2, "need at least two stages");
  static_assert(2 * BN * kAccStages <= kTmemCols, "accumulators exceed tensor memory");
};

// Bounded wait on an mbarrier phase.  Returns false when the abort flag is up or the wait ran out
// after `limit` cycles (in which case it raises the flag and records `code`).  In a CTA pair
// `peer_abort` is the shared::cluster address of the other CTA's abort flag (0: none): the CTA
// that gives up raises it too, so the pair stops together instead of each role of the peer sitting
// out its own full limit.  The peer cannot have left: both CTAs meet at the closing cluster barrier.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int *abort_flag,
                                          unsigned int *status, unsigned code, long long limit,
                                          uint32_t peer_abort = 0) {
  if (mbar_try_wait(bar, parity)) return true;
  const long long t0 = clock64();
  for (uint32_t spin = 1;; ++spin) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((spin & 0x3Fu) == 0) {
      if (*abort_flag) return false;
      if (clock64() - t0 > limit) {
        *abort_flag = 1;
        if (peer_abort != 0) st_shared_cluster_u32(peer_abort, 1u);
        atomicOr(status, code);
        return false;
      }
    }
  }
}

struct TileCoord {
  uint32_t b, mt, nt;
};

// Tiles are walked batch by batch, and inside a batch item in column panels of `group_n` tiles
// so that CTAs running at the same time share A row-blocks and B column-blocks in L2.
__device__ __forceinline__ TileCoord decode_tile(const GemmParams &p, uint32_t tile) {
  const uint32_t per_batch = p.tiles_m * p.tiles_n;
  TileCoord t;
  t.b = tile / per_batch;
  const uint32_t r = tile - t.b * per_batch;
  const uint32_t panel = p.group_n * p.tiles_m;
  const uint32_t g = r / panel;
  const uint32_t first_n = g * p.group_n;
  const uint32_t width = min(p.group_n, p.tiles_n - first_n);
  const uint32_t rr = r - g * panel;
  t.mt = rr / width;
  t.nt = first_n + (rr - t.mt * width);
  return t;
}

template <typename T> struct OutTraits;
template <> struct OutTraits<float> {
  using Acc = float;
  static __device__ __forceinline__ float from_bits(uint32_t u) { return __uint_as_float(u); }
  static __device__ __forceinline__ float to_out(float v) { return v; }
  static __device__ __forceinline__ float to_acc(float v) { return v; }
};
template <> struct OutTraits<__half> {
  using Acc = float;
  static __device__ __forceinline__ float from_bits(uint32_t u) { return __uint_as_float(u); }
  static __device__ __forceinline__ __half to_out(float v) { return __float2half_rn(v); }
  static __device__ __forceinline__ float to_acc(__half v) { return __half2float(v); }
};
template <> struct OutTraits<__nv_bfloat16> {
  using Acc = float;
  static __device__ __forceinline__ float from_bits(uint32_t u) { return __uint_as_float(u); }
  static __device__ __forceinline__ __nv_bfloat16 to_out(float v) {
    return __float2bfloat16_rn(v);
  }
  static __device__ __forceinline__ float to_acc(__nv_bfloat16 v) { return __bfloat162float(v); }
};
template <> struct OutTraits<int> {
  using Acc = int;
  static __device__ __forceinline__ int from_bits(uint32_t u) { return static_cast<int>(u); }
  static __device__ __forceinline__ int to_out(int v) { return v; }
  static __device__ __forceinline__ int to_acc(int v) { return v; }
};

// int32 output whose tensor-memory accumulator is fp32 (the block-scaled 4-bit path): the sums are
// integers below 2^24, so the conversion is exact.
struct IntFromFloat {
  int v;
};
template <> struct OutTraits<IntFromFloat> {
  using Acc = int;
  static __device__ __forceinline__ int from_bits(uint32_t u) {
    return __float2int_rn(__uint_as_float(u));
  }
  static __device__ __forceinline__ IntFromFloat to_out(int v) { return IntFromFloat{v}; }
  static __device__ __forceinline__ int to_acc(IntFromFloat v) { return v.v; }
};

// Pack two consecutive accumulator values into output words (one word per value for 32-bit
// outputs, one word per pair for 16-bit outputs).
template <typename OutT> struct Packer;
template <> struct Packer<float> {
  static constexpr int kPerWord = 1;
  static __device__ __forceinline__ uint32_t word(const float *v) { return __float_as_uint(v[0]); }
};
template <> struct Packer<int> {
  static constexpr int kPerWord = 1;
  static __device__ __forceinline__ uint32_t word(const int *v) {
    return static_cast<uint32_t>(v[0]);
  }
};
template <> struct Packer<IntFromFloat> : Packer<int> {};
template <> struct Packer<__half> {
  static constexpr int kPerWord = 2;
  static __device__ __forceinline__ uint32_t word(const float *v) {
    const __half2 h = __floats2half2_rn(v[0], v[1]);
    return *reinterpret_cast<const uint32_t *>(&h);
  }
};
template <> struct Packer<__nv_bfloat16> {
  static constexpr int kPerWord = 2;
  static __device__ __forceinline__ uint32_t word(const float *v) {
    const __nv_bfloat162 h = __floats2bfloat162_rn(v[0], v[1]);
    return *reinterpret_cast<const uint32_t *>(&h);
  }
};

// Store `COUNT` consecutive output elements held in registers; 16-byte stores when allowed.
template <typename OutT, int COUNT, typename Acc>
__device__ __forceinline__ void store_run(OutT *dst, const Acc (&v)[COUNT], int valid, bool vec) {
  using P = Packer<OutT>;
  constexpr int kPerVec = 4 * P::kPerWord;
  if (vec && valid == COUNT) {
    uint4 *d = reinterpret_cast<uint4 *>(dst);
#pragma unroll
    for (int i = 0; i < COUNT / kPerVec; ++i) {
      uint4 q;
      q.x = P::word(&v[i * kPerVec + 0 * P::kPerWord]);
      q.y = P::word(&v[i * kPerVec + 1 * P::kPerWord]);
      q.z = P::word(&v[i * kPerVec + 2 * P::kPerWord]);
      q.w = P::word(&v[i * kPerVec + 3 * P::kPerWord]);
      d[i] = q;
    }
  } else {
#pragma unroll
    for (int i = 0; i < COUNT; ++i) {
      if (i < valid) dst[i] = OutTraits<OutT>::to_out(v[i]);
    }
  }
}

// Element offsets of C for (row m, column n0) of batch item b in the requested layout.
struct COffsets {
  size_t base_re, stride_j, off_im;
};

__device__ __forceinline__ COffsets c_offsets(const GemmParams &p, uint32_t b, uint32_t m,
                                              uint32_t n0) {
  const size_t M = p.M, N = p.N;
  COffsets o;
  switch (p.c_layout) {
  case kPlanarRow:
    o.base_re = ((size_t)b * 2 * M + m) * N + n0;
    o.stride_j = 1;
    o.off_im = M * N;
    break;
  case kPlanarCol:
    o.base_re = ((size_t)b * 2 * N + n0) * M + m;
    o.stride_j = M;
    o.off_im = M * N;
    break;
  case kInterRow:
    o.base_re = (((size_t)b * M + m) * N + n0) * 2;
    o.stride_j = 2;
    o.off_im = 1;
    break;
  default:
    o.base_re = (((size_t)b * N + n0) * M + m) * 2;
    o.stride_j = 2 * M;
    o.off_im = 1;
    break;
  }
  return o;
}

// Accumulator bits -> values with alpha and beta applied (row m, 32 columns from n0).
template <typename OutT>
__device__ __forceinline__ void epilogue_values(const GemmParams &p, const COffsets &o, bool row_ok,
                                                int valid, const uint32_t (&bits_re)[32],
                                                const uint32_t (&bits_im)[32],
                                                typename OutTraits<OutT>::Acc (&re)[32],
                                                typename OutTraits<OutT>::Acc (&im)[32]) {
  using Tr = OutTraits<OutT>;
  using Acc = typename Tr::Acc;
  const OutT *C = static_cast<const OutT *>(p.c);
#pragma unroll
  for (int j = 0; j < 32; ++j) {
    re[j] = Tr::from_bits(bits_re[j]);
    im[j] = Tr::from_bits(bits_im[j]);
  }
  if (p.have_alpha) {
    const Acc ar = static_cast<Acc>(p.alpha_re), ai = static_cast<Acc>(p.alpha_im);
#pragma unroll
    for (int j = 0; j < 32; ++j) {
      const Acc r = re[j];
      re[j] = ar * r - ai * im[j];
      im[j] = ai * r + ar * im[j];
    }
  }
  if (p.have_beta && row_ok) {
    const Acc br = static_cast<Acc>(p.beta_re), bi = static_cast<Acc>(p.beta_im);
#pragma unroll
    for (int j = 0; j < 32; ++j) {
      if (j < valid) {
        const Acc cr = Tr::to_acc(C[o.base_re + j * o.stride_j]);
        const Acc ci = Tr::to_acc(C[o.base_re + j * o.stride_j + o.off_im]);
        re[j] += br * cr - bi * ci;
        im[j] += bi * cr + br * ci;
      }
    }
  }
}

// Epilogue for one row (m) and 32 consecutive columns starting at n0 of batch item b, stored
// straight from registers.
template <typename OutT>
__device__ __forceinline__ void epilogue_chunk(const GemmParams &p, uint32_t b, uint32_t m,
                                               uint32_t n0, const uint32_t (&bits_re)[32],
                                               const uint32_t (&bits_im)[32]) {
  using Tr = OutTraits<OutT>;
  using Acc = typename Tr::Acc;
  if (m >= p.M) return;
  OutT *C = static_cast<OutT *>(p.c);
  const int valid = static_cast<int>(min(32u, p.N - n0));
  const COffsets o = c_offsets(p, b, m, n0);
  Acc re[32], im[32];
  epilogue_values<OutT>(p, o, true, valid, bits_re, bits_im, re, im);
  if (p.c_layout == kPlanarRow) {
    store_run<OutT, 32>(C + o.base_re, re, valid, p.vec_ok != 0);
    store_run<OutT, 32>(C + o.base_re + o.off_im, im, valid, p.vec_ok != 0);
  } else if (p.c_layout == kInterRow) {
    Acc both[64];
#pragma unroll
    for (int j = 0; j < 32; ++j) {
      both[2 * j] = re[j];
      both[2 * j + 1] = im[j];
    }
    store_run<OutT, 64>(C + o.base_re, both, 2 * valid, p.vec_ok != 0);
  } else {
    // column-major: consecutive lanes hold consecutive m, so each store is coalesced as is
#pragma unroll
    for (int j = 0; j < 32; ++j) {
      if (j < valid) {
        C[o.base_re + j * o.stride_j] = Tr::to_out(re[j]);
        C[o.base_re + j * o.stride_j + o.off_im] = Tr::to_out(im[j]);
      }
    }
  }
}

// One lane writes its row of 32 four-byte values into a 4 KiB staging tile laid out the way a
// 128-byte-swizzled TMA store reads it (16-byte chunk j of row r sits at chunk j ^ (r & 7)).
template <typename Acc>
__device__ __forceinline__ void stage_row(uint32_t tile, uint32_t lane, const Acc (&v)[32]) {
  const uint32_t row = tile + lane * 128;
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    st_shared_v4(row + ((j ^ (lane & 7)) << 4), Packer<Acc>::word(&v[4 * j]),
                 Packer<Acc>::word(&v[4 * j + 1]), Packer<Acc>::word(&v[4 * j + 2]),
                 Packer<Acc>::word(&v[4 * j + 3]));
  }
}

// Epilogue for 32 rows (one per lane, first row m0) and 32 columns from n0, stored through the
// warp's staging tiles with TMA (row-major C, planar or interleaved, four-byte elements).  The two
// tiles of a chunk (real and imaginary plane, or the two halves of an interleaved row) are written
// side by side, made visible to the async proxy with one fence, and
// stored as one bulk group.  A warp rotates through DEPTH / 2 tile pairs and reuses a pair only
// after the group issued from it has finished reading shared memory.
template <typename OutT, int DEPTH>
__device__ __forceinline__ void epilogue_chunk_staged(const GemmParams &p, const CUtensorMap *tm_c,
                                                      uint32_t staging, uint32_t &slot,
                                                      uint32_t lane, uint32_t b, uint32_t m0,
                                                      uint32_t n0, const uint32_t (&bits_re)[32],
                                                      const uint32_t (&bits_im)[32]) {
  using Acc = typename OutTraits<OutT>::Acc;
  static_assert(sizeof(OutT) == 4, "staged epilogue is for four-byte outputs");
  static_assert(DEPTH >= 2 && DEPTH % 2 == 0, "staging tiles come in (re, im) pairs");
  const uint32_t m = m0 + lane;
  const int valid = static_cast<int>(min(32u, p.N - n0));
  const COffsets o = c_offsets(p, b, m, n0);
  Acc re[32], im[32];
  epilogue_values<OutT>(p, o, m < p.M, valid, bits_re, bits_im, re, im);
  const uint32_t tiles = staging + (slot % (DEPTH / 2)) * (2 * kStagingTile);
  ++slot;
  if (lane == 0) bulk_wait_group_read<DEPTH / 2 - 1>();
  __syncwarp();
  if (p.c_layout == kInterRow) {
    // [m][n][2]: a row of 32 complex values is 256 bytes = two tiles of 16 (re, im) pairs
    Acc lo[32], hi[32];
#pragma unroll
    for (int j = 0; j < 16; ++j) {
      lo[2 * j] = re[j];
      lo[2 * j + 1] = im[j];
      hi[2 * j] = re[16 + j];
      hi[2 * j + 1] = im[16 + j];
    }
    stage_row<Acc>(tiles, lane, lo);
    stage_row<Acc>(tiles + kStagingTile, lane, hi);
  } else {
    stage_row<Acc>(tiles, lane, re);
    stage_row<Acc>(tiles + kStagingTile, lane, im);
  }
  fence_proxy_async_smem();
  __syncwarp();
  if (lane == 0 && m0 < p.M) {
    // the tensor map is byte-typed: planar (N*4, M, 2*batch), interleaved (N*8, M, batch)
    if (p.c_layout == kInterRow) {
      const int32_t x = static_cast<int32_t>(n0 * 8);
      tma_store_3d(tm_c, tiles, x, static_cast<int32_t>(m0), static_cast<int32_t>(b));
      if (n0 + 16 < p.N) {
        tma_store_3d(tm_c, tiles + kStagingTile, x + 128, static_cast<int32_t>(m0),
                     static_cast<int32_t>(b));
      }
    } else {
      const int32_t x = static_cast<int32_t>(n0 * 4);
      tma_store_3d(tm_c, tiles, x, static_cast<int32_t>(m0), static_cast<int32_t>(2 * b));
      tma_store_3d(tm_c, tiles + kStagingTile, x, static_cast<int32_t>(m0),
                   static_cast<int32_t>(2 * b + 1));
    }
    bulk_commit_group();
  }
}

template <int KIND, int BN, int SW, int A_PLANES, typename OutT, int EPI>
__global__ void __launch_bounds__(kThreads, 1)
cgemm_tcgen05_kernel(const __grid_constant__ CUtensorMap tm_a,
                     const __grid_constant__ CUtensorMap tm_b,
                     const __grid_constant__ CUtensorMap tm_c, const GemmParams p) {
  using C = Cfg<BN, SW, A_PLANES, EPI>;
  constexpr bool EPI_TMA = EPI > 0;
  constexpr int kStages = C::kStages;
  // the block-scaled kind keeps 32 tensor-memory columns for its (all-ones) scale factors
  constexpr int kAccStages = (KIND == kKindMXF4) ? 1 : C::kAccStages;
  constexpr int kScaleCol = 2 * BN * kAccStages;
  static_assert(KIND != kKindMXF4 || kScaleCol + 32 <= kTmemCols, "no room for scale factors");
  constexpr int kSub = SW / 32;  // 32-byte MMA k-steps per stage

  extern __shared__ uint8_t smem_raw[];
  uint8_t *smem = reinterpret_cast<uint8_t *>(
      (reinterpret_cast<uintptr_t>(smem_raw) + 1023u) & ~static_cast<uintptr_t>(1023u));
  uint64_t *bars = reinterpret_cast<uint64_t *>(smem + kStages * C::kStageBytes + C::kStaging);
  const uint32_t bar_full = smem_u32(bars);
  const uint32_t bar_empty = bar_full + 8 * kStages;
  const uint32_t bar_acc_full = bar_empty + 8 * kStages;
  const uint32_t bar_acc_empty = bar_acc_full + 8 * kAccStages;
  const uint32_t bar_borrow = bar_acc_empty + 8 * kAccStages;
  uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + 2 * kStages + 2 * kAccStages + 1);
  volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);
  const uint32_t smem_base = smem_u32(smem);

  const uint32_t warp = threadIdx.x >> 5;
  const uint32_t lane = threadIdx.x & 31;

  // With one accumulator stage the epilogue is exposed: the MMAs of the next tile wait for it.
  // Its speed is set by how many TMA stores a warp may have in flight, i.e. by staging space, so
  // for the tile's epilogue the warps borrow the pipeline stage that the tile's last k-block
  // used (free once the accumulator is complete): six staging tiles per warp instead of two.
  // The producer's next load into that stage (k-block kStages - 1 of the next tile) waits until
  // the stores have read it (bar_borrow); the next tile's first k-blocks sit in the other stages
  // and were prefetched during the epilogue.
  constexpr int kBorrowDepth = 6;
  constexpr bool BORROW = EPI_TMA && kAccStages == 1 && KIND != kKindMXF4 &&
                          C::kStageBytes >= 4 * kBorrowDepth * kStagingTile;
  const bool borrow = BORROW && p.epi_tma && p.k_blocks >= static_cast<uint32_t>(kStages);

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(bar_full + 8 * s, 1);
      mbar_init(bar_empty + 8 * s, 1);
    }
    for (int s = 0; s < kAccStages; ++s) {
      mbar_init(bar_acc_full + 8 * s, 1);
      mbar_init(bar_acc_empty + 8 * s, 4);  // one arrival per epilogue warp
    }
    mbar_init(bar_borrow, 4);  // one arrival per epilogue warp and tile
    *abort_flag = 0;
    fence_mbar_init();
    prefetch_tensormap(&tm_a);
    prefetch_tensormap(&tm_b);
    if (EPI_TMA && p.epi_tma) prefetch_tensormap(&tm_c);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(tmem_slot), kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  if constexpr (KIND == kKindMXF4) {
    // Scale factors are ue8m0 bytes; 0x7F = 2^0.  Every byte of the 32 columns is 1.0, so whichever
    // bytes the MMA picks for its rows and 32-element blocks, the operands are used unscaled.
    if (warp >= 2) {
      const uint32_t t_sf = tmem_base + (((warp & 3) * 32) << 16) + kScaleCol;
      tmem_st_32x32b_x16_fill(t_sf, 0x7F7F7F7Fu);
      tmem_st_32x32b_x16_fill(t_sf + 16, 0x7F7F7F7Fu);
      tmem_wait_st();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
  }

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    uint32_t stage = 0, phase = 0;
    uint32_t issued = 0;  // stages that have carried at least one load
    bool ok = true;
    // operand coordinates of k-block kb of tile t
    auto coords = [&](const TileCoord &t, uint32_t kb, int32_t &ax, int32_t &ay, int32_t &az,
                      int32_t &bx, int32_t &by, int32_t &bz) {
      if (p.tiled) {
        const uint32_t slab = kb / p.k_per_slab;
        ax = bx = static_cast<int32_t>((kb - slab * p.k_per_slab) * SW);
        ay = 0;
        az = static_cast<int32_t>(2 * ((t.b * p.a_slabs_m + t.mt) * p.slabs_k + slab));
        const uint32_t n_glob = t.nt * BN;
        const uint32_t slab_n = n_glob / p.b_slab_rows;
        by = static_cast<int32_t>(n_glob - slab_n * p.b_slab_rows);
        bz = static_cast<int32_t>(2 * ((t.b * p.b_slabs_n + slab_n) * p.slabs_k + slab));
      } else {
        ax = bx = static_cast<int32_t>(kb * SW);
        ay = static_cast<int32_t>(t.mt * kBlockM);
        az = static_cast<int32_t>(t.b * A_PLANES);
        by = static_cast<int32_t>(t.nt * BN);
        bz = static_cast<int32_t>(t.b * 2);
      }
    };
    // Optional second cursor that runs p.prefetch k-blocks ahead of the loads and only asks L2 for
    // the tiles (an experiment for short-K shapes whose loads mostly miss L2; see launch_gemm).
    uint32_t pf_tile = blockIdx.x, pf_kb = 0;
    auto prefetch_next = [&]() {
      if (pf_tile >= p.num_tiles) return;
      int32_t ax, ay, az, bx, by, bz;
      coords(decode_tile(p, pf_tile), pf_kb, ax, ay, az, bx, by, bz);
      tma_prefetch_3d(&tm_a, ax, ay, az);
      tma_prefetch_3d(&tm_b, bx, by, bz);
      if (++pf_kb == p.k_blocks) {
        pf_kb = 0;
        pf_tile += gridDim.x;
      }
    };
    if (lane == 0) {
      for (uint32_t i = 0; i < p.prefetch; ++i) prefetch_next();
    }
    uint32_t tile_iter = 0;
    for (uint32_t tile = blockIdx.x; ok && tile < p.num_tiles; tile += gridDim.x, ++tile_iter) {
      const TileCoord t = decode_tile(p, tile);
      for (uint32_t kb = 0; kb < p.k_blocks; ++kb) {
        if (!mbar_wait(bar_empty + 8 * stage, phase ^ 1, abort_flag, p.status,
                       kDevTimeoutProducer, p.wait_cycles)) {
          ok = false;
          break;
        }
        if (borrow && tile_iter > 0 && kb == static_cast<uint32_t>(kStages - 1)) {
          // this stage was the previous tile's last one: its epilogue staged C in it
          if (!mbar_wait(bar_borrow, (tile_iter - 1) & 1, abort_flag, p.status,
                         kDevTimeoutProducer, p.wait_cycles)) {
            ok = false;
            break;
          }
        }
        if (lane == 0) {
          int32_t ax, ay, az, bx, by, bz;
          coords(t, kb, ax, ay, az, bx, by, bz);
          const uint32_t full = bar_full + 8 * stage;
          const uint32_t dst = smem_base + stage * C::kStageBytes;
          mbar_arrive_expect_tx(full, C::kStageBytes);
          tma_load_3d(dst, &tm_a, ax, ay, az, full);
          tma_load_3d(dst + C::kABytes, &tm_b, bx, by, bz, full);
          if (p.prefetch) prefetch_next();
        }
        __syncwarp();
        issued |= 1u << stage;
        if (++stage == kStages) {
          stage = 0;
          phase ^= 1;
        }
      }
    }
    if (*abort_flag) {
      // Do not leave the CTA while our own bulk copies may still be landing in its shared memory:
      // wait (bounded) for the last load issued into every stage.
      for (int s = 0; s < kStages; ++s) {
        if (!(issued & (1u << s))) continue;
        // stages before `stage` were last filled in the current phase, the others one phase back
        const uint32_t last_parity = (static_cast<uint32_t>(s) < stage) ? phase : (phase ^ 1);
        const long long t0 = clock64();
        while (!mbar_try_wait(bar_full + 8 * s, last_parity)) {
          if (clock64() - t0 > p.wait_cycles) {
            atomicOr(p.status, kDevTimeoutDrain);
            break;
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    uint32_t stage = 0, phase = 0, acc = 0, acc_phase = 0;
    bool ok = true;
    [[maybe_unused]] uint32_t iter = 0;
    for (uint32_t tile = blockIdx.x; ok && tile < p.num_tiles; tile += gridDim.x, ++iter) {
      if (!mbar_wait(bar_acc_empty + 8 * acc, acc_phase ^ 1, abort_flag, p.status,
                     kDevTimeoutMma, p.wait_cycles)) {
        break;
      }
      tc_fence_after();
      if (lane == 0) CCGLIB_TRACE(iter, 0);
      const uint32_t d_re = tmem_base + acc * (2 * BN);
      const uint32_t d_im = d_re + BN;
      for (uint32_t kb = 0; kb < p.k_blocks; ++kb) {
        if (!mbar_wait(bar_full + 8 * stage, phase, abort_flag, p.status, kDevTimeoutMma,
                       p.wait_cycles)) {
          ok = false;
          break;
        }
        tc_fence_after();
        if (lane == 0) {
          const uint32_t a_base = smem_base + stage * C::kStageBytes;
          const uint32_t b_base = a_base + C::kABytes;
#pragma unroll
          for (int k = 0; k < kSub; ++k) {
            const uint64_t a_re = smem_desc<SW>(a_base + k * 32);
            const uint64_t a_im = smem_desc<SW>(a_base + C::kAPlane + k * 32);
            const uint64_t b_re = smem_desc<SW>(b_base + k * 32);
            const uint64_t b_im = smem_desc<SW>(b_base + C::kBPlane + k * 32);
            const uint32_t accum = (kb | static_cast<uint32_t>(k)) != 0 ? 1u : 0u;
            if constexpr (KIND == kKindMXF4) {
              const uint32_t sf = tmem_base + kScaleCol;
              tc_mma_mxf4(d_re, a_re, b_re, p.idesc, sf, sf + 16, accum);
              tc_mma_mxf4(d_im, a_re, b_im, p.idesc, sf, sf + 16, accum);
              tc_mma_mxf4(d_im, a_im, b_re, p.idesc, sf, sf + 16, 1u);
              if constexpr (A_PLANES == 3) {
                const uint64_t a_neg = smem_desc<SW>(a_base + 2 * C::kAPlane + k * 32);
                tc_mma_mxf4(d_re, a_neg, b_im, p.idesc, sf, sf + 16, 1u);
              } else {
                tc_mma_mxf4(d_re, a_im, b_im, p.idesc_neg_a, sf, sf + 16, 1u);
              }
            } else {
              tc_mma<KIND>(d_re, a_re, b_re, p.idesc, accum);
              tc_mma<KIND>(d_im, a_re, b_im, p.idesc, accum);
              tc_mma<KIND>(d_im, a_im, b_re, p.idesc, 1u);
              if constexpr (A_PLANES == 3) {
                // third plane already holds -Ai (integer kinds have no negate bit)
                const uint64_t a_neg = smem_desc<SW>(a_base + 2 * C::kAPlane + k * 32);
                tc_mma<KIND>(d_re, a_neg, b_im, p.idesc, 1u);
              } else {
                tc_mma<KIND>(d_re, a_im, b_im, p.idesc_neg_a, 1u);
              }
            }
          }
          tc_commit(bar_empty + 8 * stage);  // stage reusable once these MMAs have read it
          if (kb + 1 == p.k_blocks) {
            tc_commit(bar_acc_full + 8 * acc);
            CCGLIB_TRACE(iter, 1);
          }
        }
        __syncwarp();
        if (++stage == kStages) {
          stage = 0;
          phase ^= 1;
        }
      }
      if (++acc == kAccStages) {
        acc = 0;
        acc_phase ^= 1;
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue warps
    const uint32_t quad = warp & 3;  // TMEM lanes [32*quad, 32*quad+32) belong to this warp
    uint32_t acc = 0, acc_phase = 0;
    uint32_t slot = 0;  // staging tile rotation
    [[maybe_unused]] uint32_t iter = 0;
    for (uint32_t tile = blockIdx.x; tile < p.num_tiles; tile += gridDim.x, ++iter) {
      const TileCoord t = decode_tile(p, tile);
      if (!mbar_wait(bar_acc_full + 8 * acc, acc_phase, abort_flag, p.status,
                     kDevTimeoutEpilogue, p.wait_cycles)) {
        break;
      }
      tc_fence_after();
      if (warp == 2 && lane == 0) CCGLIB_TRACE(iter, 2);
      const uint32_t m = t.mt * kBlockM + quad * 32 + lane;
      const uint32_t t_re = tmem_base + ((quad * 32) << 16) + acc * (2 * BN);
#pragma unroll 1
      for (uint32_t c0 = 0; c0 < BN; c0 += 32) {
        const uint32_t n0 = t.nt * BN + c0;
        if (n0 >= p.N) break;
        uint32_t bits_re[32], bits_im[32];
        tmem_ld_32x32b_x32(t_re + c0, bits_re);
        tmem_ld_32x32b_x32(t_re + BN + c0, bits_im);
        tmem_wait_ld();
        if constexpr (EPI_TMA) {
          if (p.epi_tma) {
            if constexpr (BORROW) {
              if (borrow) {
                // the stage of this tile's last k-block (global k-block (iter + 1) * k_blocks - 1)
                const uint32_t last_stage = static_cast<uint32_t>(
                    (static_cast<uint64_t>(iter + 1) * p.k_blocks - 1) % kStages);
                const uint32_t staging = smem_base + last_stage * C::kStageBytes +
                                         quad * (kBorrowDepth * kStagingTile);
                epilogue_chunk_staged<OutT, kBorrowDepth>(p, &tm_c, staging, slot, lane, t.b,
                                                          t.mt * kBlockM + quad * 32, n0, bits_re,
                                                          bits_im);
                continue;
              }
            }
            const uint32_t staging =
                smem_base + kStages * C::kStageBytes + quad * (EPI * kStagingTile);
            epilogue_chunk_staged<OutT, (EPI > 0 ? EPI : 2)>(p, &tm_c, staging, slot, lane, t.b,
                                                             t.mt * kBlockM + quad * 32, n0,
                                                             bits_re, bits_im);
            continue;
          }
        }
        epilogue_chunk<OutT>(p, t.b, m, n0, bits_re, bits_im);
      }
      tc_fence_before();
      __syncwarp();
      if (warp == 2 && lane == 0) CCGLIB_TRACE(iter, 3);
      if (lane == 0) mbar_arrive(bar_acc_empty + 8 * acc);
      if constexpr (BORROW) {
        if (borrow) {
          // hand the borrowed stage back once this warp's stores have read it
          if (lane == 0) {
            bulk_wait_group_read<0>();
            mbar_arrive(bar_borrow);
          }
          __syncwarp();
        }
      }
      if (++acc == kAccStages) {
        acc = 0;
        acc_phase ^= 1;
      }
    }
    if constexpr (EPI_TMA) {
      // the staging tiles must outlive the stores that read them
      if (p.epi_tma && lane == 0) bulk_wait_group<0>();
      __syncwarp();
    }
  }

  // ------------------------------------------------------------------ tear-down
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

// ------------------------------------------------------------------------------ CTA pairs
//
// Same computation with the two SMs of a TPC working as one: a cluster of two CTAs shares one
// 256 x BN tile.  Each CTA stages its own 128 rows of A and only half of the B tile (BN/2 rows);
// one thread of the leader CTA (cluster rank 0) issues tcgen05.mma.cta_group::2 with M = 256, which
// makes each SM multiply its A rows by the whole B tile, reading the other half from the peer's
// shared memory.  Per flop this halves the B bytes fetched from L2 and cuts the operand bytes
// read from shared memory by a third, which is what the clock under the power cap and the L2
// bandwidth of short-K problems are limited by.
//
// Hand-over: both producers arm and fill the LEADER's full barrier (2 arrivals + both CTAs' bytes;
// loads carry .cta_group::2 so that they may signal the peer's barrier, never multicast); the
// leader's commits arrive on each CTA's own empty / acc_full barriers; the eight epilogue warps
// of the pair arrive on the leader's acc_empty barrier.  Set-up and tear-down are cluster-wide
// barriers, so neither CTA leaves while the other may still touch its shared memory.

template <int BN, int A_PLANES, bool EPI_TMA> struct PairCfg {
  static constexpr int kSw = 128;
  static constexpr int kAPlane = kBlockM * kSw;
  static constexpr int kBPlane = (BN / 2) * kSw;
  static constexpr int kABytes = A_PLANES * kAPlane;
  static constexpr int kBBytes = 2 * kBPlane;
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kBarrierBytes = 256;
  static constexpr int kStaging = EPI_TMA ? kStagingBytes : 0;
  static constexpr int kStagesRaw = (kMaxSmem - 1024 - kBarrierBytes - kStaging) / kStageBytes;
  static constexpr int kStages = kStagesRaw > 8 ? 8 : kStagesRaw;
  static constexpr int kAccStages = (BN == 128) ? 2 : 1;
  static constexpr int kSmemBytes = kStages * kStageBytes + kStaging + 1024 + kBarrierBytes;
  static_assert(kStages >= 2, "need at least two stages");
};

template <int KIND, int BN, int A_PLANES, typename OutT, bool EPI_TMA>
__global__ void __launch_bounds__(kThreads, 1)
cgemm_pair_kernel(const __grid_constant__ CUtensorMap tm_a,
                  const __grid_constant__ CUtensorMap tm_b,
                  const __grid_constant__ CUtensorMap tm_c, const GemmParams p) {
  using C = PairCfg<BN, A_PLANES, EPI_TMA>;
  constexpr int kStages = C::kStages;
  constexpr int kAccStages = (KIND == kKindMXF4) ? 1 : C::kAccStages;
  constexpr int kScaleCol = 2 * BN * kAccStages;  // scale-factor columns of the block-scaled kind
  static_assert(KIND != kKindMXF4 || kScaleCol + 32 <= kTmemCols, "no room for scale factors");
  constexpr int SW = C::kSw;
  constexpr int kSub = SW / 32;

  extern __shared__ uint8_t smem_raw[];
  uint8_t *smem = reinterpret_cast<uint8_t *>(
      (reinterpret_cast<uintptr_t>(smem_raw) + 1023u) & ~static_cast<uintptr_t>(1023u));
  uint64_t *bars = reinterpret_cast<uint64_t *>(smem + kStages * C::kStageBytes + C::kStaging);
  const uint32_t bar_full = smem_u32(bars);
  const uint32_t bar_empty = bar_full + 8 * kStages;
  const uint32_t bar_acc_full = bar_empty + 8 * kStages;
  const uint32_t bar_acc_empty = bar_acc_full + 8 * kAccStages;
  uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + 2 * kStages + 2 * kAccStages);
  volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);
  const uint32_t smem_base = smem_u32(smem);

  const uint32_t warp = threadIdx.x >> 5;
  const uint32_t lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();  // 0 = leader
  const uint32_t pair = cluster_id_x();
  const uint32_t num_pairs = cluster_count_x();
  const uint32_t peer_abort = map_to_cta(smem_u32(const_cast<int *>(abort_flag)), rank ^ 1u);

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(bar_full + 8 * s, 2);  // one arrival per producer of the pair (used in the leader)
      mbar_init(bar_empty + 8 * s, 1);
    }
    for (int s = 0; s < kAccStages; ++s) {
      mbar_init(bar_acc_full + 8 * s, 1);
      mbar_init(bar_acc_empty + 8 * s, 8);  // epilogue warps of both CTAs (used in the leader)
    }
    *abort_flag = 0;
    fence_mbar_init();
    prefetch_tensormap(&tm_a);
    prefetch_tensormap(&tm_b);
    if (EPI_TMA && p.epi_tma) prefetch_tensormap(&tm_c);
  }
  if (warp == 1) {
    tmem_alloc_pair(smem_u32(tmem_slot), kTmemCols);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  cluster_sync();  // the peer's barriers must be initialised before anything arrives on them
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  if constexpr (KIND == kKindMXF4) {
    // all-ones (ue8m0 0x7F) scale factors in each CTA's own tensor memory
    if (warp >= 2) {
      const uint32_t t_sf = tmem_base + (((warp & 3) * 32) << 16) + kScaleCol;
      tmem_st_32x32b_x16_fill(t_sf, 0x7F7F7F7Fu);
      tmem_st_32x32b_x16_fill(t_sf + 16, 0x7F7F7F7Fu);
      tmem_wait_st();
    }
    tc_fence_before();
    cluster_sync();
    tc_fence_after();
  }

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer (both CTAs)
    uint32_t stage = 0, phase = 0;
    uint32_t issued = 0;
    bool ok = true;
    for (uint32_t tile = pair; ok && tile < p.num_tiles; tile += num_pairs) {
      const TileCoord t = decode_tile(p, tile);
      const uint32_t mt = t.mt * 2 + rank;  // this CTA's 128-row block
      for (uint32_t kb = 0; kb < p.k_blocks; ++kb) {
        if (!mbar_wait(bar_empty + 8 * stage, phase ^ 1, abort_flag, p.status,
                       kDevTimeoutProducer, p.wait_cycles)) {
          ok = false;
          break;
        }
        if (lane == 0) {
          int32_t ax, ay, az, bx, by, bz;
          const uint32_t n_glob = t.nt * BN + rank * (BN / 2);
          if (p.tiled) {
            const uint32_t slab = kb / p.k_per_slab;
            ax = bx = static_cast<int32_t>((kb - slab * p.k_per_slab) * SW);
            // a row block past the last slab reads nothing this CTA will store; keep it in range
            const uint32_t mt_slab = min(mt, p.a_slabs_m - 1);
            ay = 0;
            az = static_cast<int32_t>(2 * ((t.b * p.a_slabs_m + mt_slab) * p.slabs_k + slab));
            const uint32_t slab_n = min(n_glob / p.b_slab_rows, p.b_slabs_n - 1);
            by = static_cast<int32_t>(n_glob - (n_glob / p.b_slab_rows) * p.b_slab_rows);
            bz = static_cast<int32_t>(2 * ((t.b * p.b_slabs_n + slab_n) * p.slabs_k + slab));
          } else {
            ax = bx = static_cast<int32_t>(kb * SW);
            ay = static_cast<int32_t>(mt * kBlockM);
            az = static_cast<int32_t>(t.b * A_PLANES);
            by = static_cast<int32_t>(n_glob);
            bz = static_cast<int32_t>(t.b * 2);
          }
          const uint32_t full = map_to_cta(bar_full + 8 * stage, 0);
          const uint32_t dst = smem_base + stage * C::kStageBytes;
          mbar_arrive_expect_tx_cluster(full, C::kStageBytes);
          tma_load_3d_pair(dst, &tm_a, ax, ay, az, full);
          tma_load_3d_pair(dst + C::kABytes, &tm_b, bx, by, bz, full);
        }
        __syncwarp();
        issued |= 1u << stage;
        if (++stage == kStages) {
          stage = 0;
          phase ^= 1;
        }
      }
    }
    if (*abort_flag && rank == 0) {
      // The leader's full barriers count the bytes of both CTAs: wait (bounded) for the last
      // load of every stage before the pair meets at the closing cluster barrier.
      for (int s = 0; s < kStages; ++s) {
        if (!(issued & (1u << s))) continue;
        const uint32_t last_parity = (static_cast<uint32_t>(s) < stage) ? phase : (phase ^ 1);
        const long long t0 = clock64();
        while (!mbar_try_wait(bar_full + 8 * s, last_parity)) {
          if (clock64() - t0 > p.wait_cycles) {
            atomicOr(p.status, kDevTimeoutDrain);
            break;
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer (leader only)
    if (rank == 0) {
      uint32_t stage = 0, phase = 0, acc = 0, acc_phase = 0;
      bool ok = true;
      [[maybe_unused]] uint32_t iter = 0;
      for (uint32_t tile = pair; ok && tile < p.num_tiles; tile += num_pairs, ++iter) {
        if (!mbar_wait(bar_acc_empty + 8 * acc, acc_phase ^ 1, abort_flag, p.status,
                       kDevTimeoutMma, p.wait_cycles, peer_abort)) {
          break;
        }
        tc_fence_after();
        if (lane == 0) CCGLIB_TRACE(iter, 0);
        const uint32_t d_re = tmem_base + acc * (2 * BN);
        const uint32_t d_im = d_re + BN;
        for (uint32_t kb = 0; kb < p.k_blocks; ++kb) {
          if (!mbar_wait(bar_full + 8 * stage, phase, abort_flag, p.status, kDevTimeoutMma,
                       p.wait_cycles)) {
            ok = false;
            break;
          }
          tc_fence_after();
          if (lane == 0) {
            const uint32_t a_base = smem_base + stage * C::kStageBytes;
            const uint32_t b_base = a_base + C::kABytes;
#pragma unroll
            for (int k = 0; k < kSub; ++k) {
              const uint64_t a_re = smem_desc<SW>(a_base + k * 32);
              const uint64_t a_im = smem_desc<SW>(a_base + C::kAPlane + k * 32);
              const uint64_t b_re = smem_desc<SW>(b_base + k * 32);
              const uint64_t b_im = smem_desc<SW>(b_base + C::kBPlane + k * 32);
              const uint32_t accum = (kb | static_cast<uint32_t>(k)) != 0 ? 1u : 0u;
              if constexpr (KIND == kKindMXF4) {
                const uint32_t sf = tmem_base + kScaleCol;
                tc_mma_mxf4_pair(d_re, a_re, b_re, p.idesc, sf, sf + 16, accum);
                tc_mma_mxf4_pair(d_im, a_re, b_im, p.idesc, sf, sf + 16, accum);
                tc_mma_mxf4_pair(d_im, a_im, b_re, p.idesc, sf, sf + 16, 1u);
                if constexpr (A_PLANES == 3) {
                  const uint64_t a_neg = smem_desc<SW>(a_base + 2 * C::kAPlane + k * 32);
                  tc_mma_mxf4_pair(d_re, a_neg, b_im, p.idesc, sf, sf + 16, 1u);
                } else {
                  tc_mma_mxf4_pair(d_re, a_im, b_im, p.idesc_neg_a, sf, sf + 16, 1u);
                }
              } else {
                tc_mma_pair<KIND>(d_re, a_re, b_re, p.idesc, accum);
                tc_mma_pair<KIND>(d_im, a_re, b_im, p.idesc, accum);
                tc_mma_pair<KIND>(d_im, a_im, b_re, p.idesc, 1u);
                if constexpr (A_PLANES == 3) {
                  const uint64_t a_neg = smem_desc<SW>(a_base + 2 * C::kAPlane + k * 32);
                  tc_mma_pair<KIND>(d_re, a_neg, b_im, p.idesc, 1u);
                } else {
                  tc_mma_pair<KIND>(d_re, a_im, b_im, p.idesc_neg_a, 1u);
                }
              }
            }
            // the stage is free in both CTAs once these MMAs have read it
            tc_commit_pair(map_to_cta(bar_empty + 8 * stage, 0));
            tc_commit_pair(map_to_cta(bar_empty + 8 * stage, 1));
            if (kb + 1 == p.k_blocks) {
              tc_commit_pair(map_to_cta(bar_acc_full + 8 * acc, 0));
              tc_commit_pair(map_to_cta(bar_acc_full + 8 * acc, 1));
              CCGLIB_TRACE(iter, 1);
            }
          }
          __syncwarp();
          if (++stage == kStages) {
            stage = 0;
            phase ^= 1;
          }
        }
        if (++acc == kAccStages) {
          acc = 0;
          acc_phase ^= 1;
        }
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue warps (both CTAs)
    const uint32_t quad = warp & 3;
    uint32_t acc = 0, acc_phase = 0;
    uint32_t slot = 0;
    [[maybe_unused]] uint32_t iter = 0;
    for (uint32_t tile = pair; tile < p.num_tiles; tile += num_pairs, ++iter) {
      const TileCoord t = decode_tile(p, tile);
      if (!mbar_wait(bar_acc_full + 8 * acc, acc_phase, abort_flag, p.status,
                     kDevTimeoutEpilogue, p.wait_cycles, peer_abort)) {
        break;
      }
      tc_fence_after();
      if (rank == 0 && warp == 2 && lane == 0) CCGLIB_TRACE(iter, 2);
      const uint32_t m0 = (t.mt * 2 + rank) * kBlockM + quad * 32;
      const uint32_t t_re = tmem_base + ((quad * 32) << 16) + acc * (2 * BN);
#pragma unroll 1
      for (uint32_t c0 = 0; c0 < BN; c0 += 32) {
        const uint32_t n0 = t.nt * BN + c0;
        if (n0 >= p.N) break;
        uint32_t bits_re[32], bits_im[32];
        tmem_ld_32x32b_x32(t_re + c0, bits_re);
        tmem_ld_32x32b_x32(t_re + BN + c0, bits_im);
        tmem_wait_ld();
        if constexpr (EPI_TMA) {
          if (p.epi_tma) {
            const uint32_t staging = smem_base + kStages * C::kStageBytes + quad * 8192;
            epilogue_chunk_staged<OutT, 2>(p, &tm_c, staging, slot, lane, t.b, m0, n0, bits_re,
                                           bits_im);
            continue;
          }
        }
        epilogue_chunk<OutT>(p, t.b, m0 + lane, n0, bits_re, bits_im);
      }
      tc_fence_before();
      __syncwarp();
      if (rank == 0 && warp == 2 && lane == 0) CCGLIB_TRACE(iter, 3);
      if (lane == 0) mbar_arrive_cluster(map_to_cta(bar_acc_empty + 8 * acc, 0));
      if (++acc == kAccStages) {
        acc = 0;
        acc_phase ^= 1;
      }
    }
    if constexpr (EPI_TMA) {
      if (p.epi_tma && lane == 0) bulk_wait_group<0>();
      __syncwarp();
    }
  }

  // ------------------------------------------------------------------ tear-down
  tc_fence_before();
  cluster_sync();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, kTmemCols);
  }
}

} // namespace

} // namespace ccglib_b200
