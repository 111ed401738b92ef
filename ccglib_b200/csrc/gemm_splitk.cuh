// Split-K form of the complex GEMM kernel for problems too small to fill the device: a cluster of
// SPLIT CTAs shares one 128 x 128 output tile, each CTA multiplying a 1/SPLIT share of K into its
// own tensor-memory accumulators; the partial sums are then reduce-scattered through distributed
// shared memory (plain st.shared::cluster stores, no multicast), every CTA finishing 128 / SPLIT
// of the tile's columns: it adds the SPLIT - 1 partials it received to its own and runs the
// usual epilogue on them.  Compared with one CTA per (smaller) tile this halves or quarters the
// MMA chain per SM and moves fewer operand bytes from L2 in total, at the price of one exchange
// of accumulators inside the cluster.
//
// One tile per cluster (not persistent).  Roles as in cgemm_tcgen05_kernel: warp 0 TMA producer,
// warp 1 MMA issuer, warps 2..5 epilogue.  The exchange is bracketed by two cluster barriers that
// every thread reaches on every path (time-outs included): the first says "all MMAs of the
// cluster are done, the stage memory may be reused as receive buffers", the second "all partials
// have been delivered".
//
// Included by gemm.cu after gemm_kernels.cuh.
#pragma once

#include "gemm_kernels.cuh"

namespace ccglib_b200 {
namespace {

template <int SPLIT, bool EPI_TMA> struct SplitCfg {
  static constexpr int kBN = 128;
  static constexpr int kSw = 128;
  static constexpr int kW = kBN / SPLIT;  // columns each CTA of the cluster finishes
  static constexpr int kAPlane = kBlockM * kSw;
  static constexpr int kBPlane = kBN * kSw;
  static constexpr int kABytes = 2 * kAPlane;
  static constexpr int kStageBytes = 2 * kAPlane + 2 * kBPlane;
  static constexpr int kStages = 3;
  static constexpr int kBarrierBytes = 256;
  static constexpr int kStaging = EPI_TMA ? kStagingBytes : 0;
  // one 4 KiB tile (32 rows x 32 floats) per (source, plane, 32-column chunk, epilogue warp);
  // the receive buffers reuse the stage memory once the main loop is over
  static constexpr int kRecvBytes = (SPLIT - 1) * 2 * (kW / 32) * 4 * kStagingTile;
  static constexpr int kSmemBytes = kStages * kStageBytes + kStaging + 1024 + kBarrierBytes;
  static_assert(kW % 32 == 0, "each CTA finishes whole 32-column chunks");
  static_assert(kRecvBytes <= kStages * kStageBytes, "receive buffers exceed the stage memory");
};

template <int KIND, int SPLIT, typename OutT, bool EPI_TMA>
__global__ void __launch_bounds__(kThreads, 1)
cgemm_splitk_kernel(const __grid_constant__ CUtensorMap tm_a,
                    const __grid_constant__ CUtensorMap tm_b,
                    const __grid_constant__ CUtensorMap tm_c, const GemmParams p) {
  using C = SplitCfg<SPLIT, EPI_TMA>;
  constexpr int BN = C::kBN, SW = C::kSw, kStages = C::kStages, kSub = SW / 32;
  static_assert(sizeof(typename OutTraits<OutT>::Acc) == 4 && KIND != kKindI8 && KIND != kKindMXF4,
                "split-K adds float partial sums");

  extern __shared__ uint8_t smem_raw[];
  uint8_t *smem = reinterpret_cast<uint8_t *>(
      (reinterpret_cast<uintptr_t>(smem_raw) + 1023u) & ~static_cast<uintptr_t>(1023u));
  uint64_t *bars = reinterpret_cast<uint64_t *>(smem + kStages * C::kStageBytes + C::kStaging);
  const uint32_t bar_full = smem_u32(bars);
  const uint32_t bar_empty = bar_full + 8 * kStages;
  const uint32_t bar_acc_full = bar_empty + 8 * kStages;
  uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + 2 * kStages + 1);
  volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);
  const uint32_t smem_base = smem_u32(smem);

  const uint32_t warp = threadIdx.x >> 5;
  const uint32_t lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const uint32_t tile = cluster_id_x();
  // this CTA's share of the k-blocks (every share is non-empty: the host asks k_blocks >= SPLIT)
  const uint32_t kb0 = rank * p.k_blocks / SPLIT;
  const uint32_t kb1 = (rank + 1) * p.k_blocks / SPLIT;
  const TileCoord t = decode_tile(p, tile);

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(bar_full + 8 * s, 1);
      mbar_init(bar_empty + 8 * s, 1);
    }
    mbar_init(bar_acc_full, 1);
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
  bool done = false;  // epilogue warps: the accumulators of this CTA are complete

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    uint32_t stage = 0, phase = 0, issued = 0;
    for (uint32_t kb = kb0; kb < kb1; ++kb) {
      if (!mbar_wait(bar_empty + 8 * stage, phase ^ 1, abort_flag, p.status, kDevTimeoutProducer,
                     p.wait_cycles)) {
        break;
      }
      if (lane == 0) {
        int32_t ax, ay, az, bx, by, bz;
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
          az = static_cast<int32_t>(t.b * 2);
          by = static_cast<int32_t>(t.nt * BN);
          bz = static_cast<int32_t>(t.b * 2);
        }
        const uint32_t full = bar_full + 8 * stage;
        const uint32_t dst = smem_base + stage * C::kStageBytes;
        mbar_arrive_expect_tx(full, C::kStageBytes);
        tma_load_3d(dst, &tm_a, ax, ay, az, full);
        tma_load_3d(dst + C::kABytes, &tm_b, bx, by, bz, full);
      }
      __syncwarp();
      issued |= 1u << stage;
      if (++stage == kStages) {
        stage = 0;
        phase ^= 1;
      }
    }
    if (*abort_flag) {
      // wait (bounded) for our own bulk copies before the stage memory is reused
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
    // ------------------------------------------------------------------ MMA issuer
    uint32_t stage = 0, phase = 0;
    const uint32_t d_re = tmem_base, d_im = tmem_base + BN;
    for (uint32_t kb = kb0; kb < kb1; ++kb) {
      if (!mbar_wait(bar_full + 8 * stage, phase, abort_flag, p.status, kDevTimeoutMma,
                     p.wait_cycles)) {
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
          const uint32_t accum = (kb != kb0 || k != 0) ? 1u : 0u;
          tc_mma<KIND>(d_re, a_re, b_re, p.idesc, accum);
          tc_mma<KIND>(d_im, a_re, b_im, p.idesc, accum);
          tc_mma<KIND>(d_im, a_im, b_re, p.idesc, 1u);
          tc_mma<KIND>(d_re, a_im, b_im, p.idesc_neg_a, 1u);
        }
        tc_commit(bar_empty + 8 * stage);
        if (kb + 1 == kb1) tc_commit(bar_acc_full);
      }
      __syncwarp();
      if (++stage == kStages) {
        stage = 0;
        phase ^= 1;
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue warps, part 1
    done = mbar_wait(bar_acc_full, 0, abort_flag, p.status, kDevTimeoutEpilogue, p.wait_cycles);
  }

  // ---- every MMA of the cluster is done (or its CTA gave up): stage memory becomes receive buffers
  tc_fence_before();
  cluster_sync();
  tc_fence_after();

  const uint32_t quad = warp & 3;
  const uint32_t t_lane = tmem_base + ((quad * 32) << 16);
  constexpr uint32_t kChunks = C::kW / 32;
  // receive tile of (source index i, plane, chunk c, epilogue warp): see SplitCfg::kRecvBytes
  auto recv_tile = [&](uint32_t i, uint32_t plane, uint32_t c) {
    return smem_base + ((((i * 2 + plane) * kChunks + c) * 4 + quad) * kStagingTile);
  };
  if (warp >= 2 && done) {
    // send the columns the other CTAs finish: row = lane, 32 floats per chunk, written in the
    // 16-byte-chunk XOR pattern of the staging tiles so that neither side has bank conflicts
    for (uint32_t step = 1; step < SPLIT; ++step) {
      const uint32_t dest = (rank + step) % SPLIT;
      const uint32_t idx = rank - (rank > dest ? 1u : 0u);  // our slot among dest's sources
#pragma unroll 1
      for (uint32_t c = 0; c < kChunks; ++c) {
        uint32_t re[32], im[32];
        const uint32_t col = dest * C::kW + c * 32;
        tmem_ld_32x32b_x32(t_lane + col, re);
        tmem_ld_32x32b_x32(t_lane + BN + col, im);
        tmem_wait_ld();
        const uint32_t row_re = map_to_cta(recv_tile(idx, 0, c) + lane * 128, dest);
        const uint32_t row_im = map_to_cta(recv_tile(idx, 1, c) + lane * 128, dest);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const uint32_t off = (j ^ (lane & 7)) << 4;
          st_shared_cluster_v4(row_re + off, re[4 * j], re[4 * j + 1], re[4 * j + 2], re[4 * j + 3]);
          st_shared_cluster_v4(row_im + off, im[4 * j], im[4 * j + 1], im[4 * j + 2], im[4 * j + 3]);
        }
      }
    }
  }

  // ---- all partial sums have been delivered
  cluster_sync();

  if (warp >= 2 && done && !*abort_flag) {
    // ------------------------------------------------------------------ epilogue warps, part 2
    uint32_t slot = 0;
#pragma unroll 1
    for (uint32_t c = 0; c < kChunks; ++c) {
      const uint32_t col = rank * C::kW + c * 32;
      const uint32_t n0 = t.nt * BN + col;
      if (n0 >= p.N) break;
      uint32_t bits_re[32], bits_im[32];
      tmem_ld_32x32b_x32(t_lane + col, bits_re);
      tmem_ld_32x32b_x32(t_lane + BN + col, bits_im);
      tmem_wait_ld();
      for (uint32_t i = 0; i + 1 < SPLIT; ++i) {
        const uint32_t row_re = recv_tile(i, 0, c) + lane * 128;
        const uint32_t row_im = recv_tile(i, 1, c) + lane * 128;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const uint32_t off = (j ^ (lane & 7)) << 4;
          uint32_t r[4], q[4];
          ld_shared_v4(row_re + off, r[0], r[1], r[2], r[3]);
          ld_shared_v4(row_im + off, q[0], q[1], q[2], q[3]);
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            bits_re[4 * j + e] = __float_as_uint(__uint_as_float(bits_re[4 * j + e]) +
                                                 __uint_as_float(r[e]));
            bits_im[4 * j + e] = __float_as_uint(__uint_as_float(bits_im[4 * j + e]) +
                                                 __uint_as_float(q[e]));
          }
        }
      }
      if constexpr (EPI_TMA) {
        if (p.epi_tma) {
          const uint32_t staging = smem_base + kStages * C::kStageBytes + quad * (2 * kStagingTile);
          epilogue_chunk_staged<OutT, 2>(p, &tm_c, staging, slot, lane, t.b,
                                         t.mt * kBlockM + quad * 32, n0, bits_re, bits_im);
          continue;
        }
      }
      epilogue_chunk<OutT>(p, t.b, t.mt * kBlockM + quad * 32 + lane, n0, bits_re, bits_im);
    }
    if constexpr (EPI_TMA) {
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

} // namespace
} // namespace ccglib_b200
