// Host side of the batched complex GEMM: C[b] = alpha * A[b] x B[b]^T + beta * C[b].
// Tensor-map encoding, the table of kernel instantiations, the plan (validation, tensor route and
// tile choice, staging scratch), the launch, and the C entry points.  The kernels are in
// gemm_kernels.cuh.
//
// Replaces ccglib::mma::GEMM (reference src/mma/GEMM.cpp:56-108,231-275) and its per-type kernel
// tables (src/mma/Kernel.cpp:7-73).
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <new>

#include "gemm_kernels.cuh"
#include "gemm_splitk.cuh"

namespace ccglib_b200 {

namespace {

using namespace ptx;

// ------------------------------------------------------------------------------ host side

using EncodeTiledFn = CUresult (*)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *,
                                   const cuuint64_t *, const cuuint64_t *, const cuuint32_t *,
                                   const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                   CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (fn == nullptr) {
    void *sym = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &qres) !=
            cudaSuccess ||
        qres != cudaDriverEntryPointSuccess) {
      return nullptr;
    }
    fn = reinterpret_cast<EncodeTiledFn>(sym);
  }
  return fn;
}

// Byte-typed 3-D tensor map: dims (row bytes, rows, slices), box (sw bytes, box_rows, box_slices).
int make_map(CUtensorMap *tm, const void *base, uint64_t row_bytes, uint64_t rows, uint64_t slices,
             uint64_t row_pitch, uint64_t slice_pitch, uint32_t sw, uint32_t box_rows,
             uint32_t box_slices) {
  EncodeTiledFn encode = get_encode_fn();
  if (encode == nullptr) {
    set_last_error("cuTensorMapEncodeTiled is not available from the installed driver");
    return CCGLIB_B200_CUDA_ERROR;
  }
  const cuuint64_t dims[3] = {row_bytes, rows, slices};
  const cuuint64_t strides[2] = {row_pitch, slice_pitch};
  const cuuint32_t box[3] = {sw, box_rows, box_slices};
  const cuuint32_t elem_strides[3] = {1, 1, 1};
  const CUresult r = encode(
      tm, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, const_cast<void *>(base), dims, strides, box,
      elem_strides, CU_TENSOR_MAP_INTERLEAVE_NONE,
      sw == 128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B,
      sw == 128 ? CU_TENSOR_MAP_L2_PROMOTION_L2_256B : CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
      CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    set_last_error("cuTensorMapEncodeTiled failed with CUresult %d (row_bytes=%llu rows=%llu "
                   "slices=%llu pitch=%llu)",
                   static_cast<int>(r), (unsigned long long)row_bytes, (unsigned long long)rows,
                   (unsigned long long)slices, (unsigned long long)row_pitch);
    return CCGLIB_B200_CUDA_ERROR;
  }
  return CCGLIB_B200_OK;
}

using KernelFn = void (*)(const CUtensorMap, const CUtensorMap, const CUtensorMap,
                          const GemmParams);

struct KernelEntry {
  KernelFn fn;
  int smem;
  bool epi_tma;  // the instance reserves staging tiles for the TMA-store epilogue
  bool pair;     // CTA-pair kernel: launched as clusters of two, tiles are 256 rows high
  int split;     // split-K kernel: clusters of `split` CTAs per 128 x 128 tile (else 1)
};

// Four-byte outputs get the TMA-store epilogue wherever its 32 KiB of staging costs no pipeline
// stage; that is everywhere except three A planes with 256-column tiles.
template <int KIND, int BN, int SW, int A_PLANES, typename OutT, int DEPTH = 2>
KernelEntry entry() {
  constexpr int kEpi = (sizeof(OutT) == 4 && !(A_PLANES == 3 && BN == 256)) ? DEPTH : 0;
  return {cgemm_tcgen05_kernel<KIND, BN, SW, A_PLANES, OutT, kEpi>,
          Cfg<BN, SW, A_PLANES, kEpi>::kSmemBytes, kEpi > 0, false, 1};
}

// Split-K instances exist for float32 output of the floating-point kinds.
template <int KIND> KernelEntry splitk_entry(int split) {
  if (split == 4) {
    return {cgemm_splitk_kernel<KIND, 4, float, true>, SplitCfg<4, true>::kSmemBytes, true, false,
            4};
  }
  return {cgemm_splitk_kernel<KIND, 2, float, true>, SplitCfg<2, true>::kSmemBytes, true, false, 2};
}

template <int KIND, int BN, int A_PLANES, typename OutT, bool EPI_TMA = (sizeof(OutT) == 4)>
KernelEntry pair_entry() {
  return {cgemm_pair_kernel<KIND, BN, A_PLANES, OutT, EPI_TMA>,
          PairCfg<BN, A_PLANES, EPI_TMA>::kSmemBytes, EPI_TMA, true, 1};
}

template <int KIND, int A_PLANES, typename OutT>
KernelEntry pick_tile(int bn, int sw, bool pair = false) {
  if (pair) {
    return bn == 256 ? pair_entry<KIND, 256, A_PLANES, OutT>()
                     : pair_entry<KIND, 128, A_PLANES, OutT>();
  }
  if (bn == 256) {
    return sw == 128 ? entry<KIND, 256, 128, A_PLANES, OutT>()
                     : entry<KIND, 256, 64, A_PLANES, OutT>();
  }
  if (bn == 64) return entry<KIND, 64, 128, A_PLANES, OutT>();
  return sw == 128 ? entry<KIND, 128, 128, A_PLANES, OutT>()
                   : entry<KIND, 128, 64, A_PLANES, OutT>();
}

template <int KIND> KernelEntry pick_float_out(int type_out, int bn, int sw, bool pair) {
  switch (type_out) {
  case CCGLIB_B200_FLOAT32:
    return pick_tile<KIND, 2, float>(bn, sw, pair);
  case CCGLIB_B200_FLOAT16:
    return pick_tile<KIND, 2, __half>(bn, sw, pair);
  case CCGLIB_B200_BFLOAT16:
    return pick_tile<KIND, 2, __nv_bfloat16>(bn, sw, pair);
  default:
    return {nullptr, 0, false, false, 1};
  }
}

int env_int(const char *name, int fallback) {
  const char *v = std::getenv(name);
  return (v != nullptr && *v != '\0') ? std::atoi(v) : fallback;
}

// Limit of the device-side waits in SM clock cycles: CCGLIB_B200_WAIT_CYCLES, else about two
// seconds.  Never unbounded: values below 1 fall back to the default.
long long wait_limit_cycles() {
  const char *v = std::getenv("CCGLIB_B200_WAIT_CYCLES");
  const long long n = (v != nullptr && *v != '\0') ? std::atoll(v) : 0;
  return n > 0 ? n : kWaitLimitCycles;
}

size_t type_bits(int t) {
  switch (t) {
  case CCGLIB_B200_INT1:
    return 1;
  case CCGLIB_B200_FLOAT8E4M3:
  case CCGLIB_B200_FLOAT8E5M2:
    return 8;
  case CCGLIB_B200_BFLOAT16:
  case CCGLIB_B200_FLOAT16:
    return 16;
  case CCGLIB_B200_INT32:
  case CCGLIB_B200_FLOAT32:
    return 32;
  default:
    return 0;
  }
}

// Time per flop of a 64-column tile relative to 128 columns: an N = 64 MMA takes as long as an
// N = 128 one (measured 823 against 1537 TFLOP/s on full waves), so the narrow tile only pays
// when it turns idle SMs into a shorter single wave.
constexpr double kCost64 = 1.9;

constexpr unsigned kSlabRowBytes = 128;  // bytes per slab row of the opt layout
constexpr unsigned kSlabRowsA = 128;     // m_blk
constexpr unsigned kSlabRowsB = 256;     // n_blk

enum StageMode { kDirect = 0, kPadRows = 1, kExpandBits = 2 };

} // namespace

} // namespace ccglib_b200

using namespace ccglib_b200;

struct ccglib_b200_gemm_plan {
  ccglib_b200_gemm_desc desc;
  KernelEntry kernel;
  int bn, sw, a_planes;
  int group_n;            // column-panel width of the tile walk from a tuning table (0: heuristic)
  int tuned;              // the tile choice came from a tuning table
  int max_clusters;       // CTA-pair kernels: co-resident clusters of two
  int nibbles;            // 1-bit input expanded to e2m1 nibbles (block-scaled 4-bit MMA path)
  int bytes_in;           // 1-bit input arrives as one byte per sample (Pipeline), not packed words
  int bytes_interleaved;  // ... in [batch][rows][K][2] order
  int stage_mode;
  size_t k_bytes;         // bytes per operand row as the kernel reads it (before any padding)
  size_t pitch;           // row pitch in bytes of what the kernel reads (basic layout)
  size_t batch_chunk;     // batch items per kernel launch (== batch in direct mode)
  void *scratch_a, *scratch_b;
  size_t scratch_bytes;
  // Staged modes with several chunks run on two lanes: lane j owns one scratch buffer and one
  // internal stream and handles chunks j, j + 2, ...; while one lane's GEMM holds the SMs the
  // other lane re-stages its next chunk beside it, and its GEMM's CTAs move in as the first
  // one's drain.  lanes < 2: one buffer, everything on the caller's stream.
  int lanes;
  void *lane_a[2], *lane_b[2];
  cudaStream_t lane_stream[2];
  cudaEvent_t ev_fork, ev_join[2];
  size_t out_elem_bytes;
  uint32_t idesc, idesc_neg_a;
  int device;
  int sms;
  long long wait_cycles;  // limit of every device-side wait of this plan's kernels
  // per-plan caches: the status word's device address and the tensor maps of the last operands
  mutable unsigned int *status_ptr;
  mutable const void *map_a, *map_b;
  mutable void *map_c;
  mutable size_t map_nb;
  mutable CUtensorMap tm_a, tm_b, tm_c;
};

namespace {

void release_plan_resources(ccglib_b200_gemm_plan &plan) {
  if (plan.lanes == 2) {
    for (int j = 0; j < 2; ++j) {
      if (plan.lane_stream[j] != nullptr) {
        cudaStreamSynchronize(plan.lane_stream[j]);
        cudaStreamDestroy(plan.lane_stream[j]);
      }
      if (plan.ev_join[j] != nullptr) cudaEventDestroy(plan.ev_join[j]);
    }
    if (plan.ev_fork != nullptr) cudaEventDestroy(plan.ev_fork);
  }
  if (plan.scratch_a != nullptr) cudaFree(plan.scratch_a);
  plan.scratch_a = nullptr;
}

} // namespace

extern "C" int ccglib_b200_gemm_dims(int type_in, int type_out, int variant, unsigned dims[3]) {
  (void)type_out;
  (void)variant;
  const size_t bits = type_bits(type_in);
  if (dims == nullptr || bits == 0 || type_in == CCGLIB_B200_INT32) {
    set_last_error("gemm_dims: unsupported input type %d", type_in);
    return CCGLIB_B200_INVALID_ARGUMENT;
  }
  dims[0] = kSlabRowsA;
  dims[1] = kSlabRowsB;
  dims[2] = static_cast<unsigned>(kSlabRowBytes * 8 / bits);
  return CCGLIB_B200_OK;
}

extern "C" int ccglib_b200_gemm_plan_create(const ccglib_b200_gemm_desc *desc,
                                            ccglib_b200_gemm_plan **out) {
  return create_gemm_plan(desc, PlanOptions{}, out);
}

int ccglib_b200::create_gemm_plan(const ccglib_b200_gemm_desc *desc, const PlanOptions &opt,
                                  ccglib_b200_gemm_plan **out) {
  if (desc == nullptr || out == nullptr) {
    set_last_error("gemm_plan_create: null argument");
    return CCGLIB_B200_INVALID_ARGUMENT;
  }
  *out = nullptr;
  const ccglib_b200_gemm_desc &d = *desc;
  if (d.batch == 0 || d.m == 0 || d.n == 0 || d.k == 0) {
    set_last_error("gemm_plan_create: batch, M, N and K must be positive");
    return CCGLIB_B200_INVALID_ARGUMENT;
  }
  if (d.m > 0x7FFFFFFFull || d.n > 0x7FFFFFFFull || d.k > 0x7FFFFFFFull ||
      d.batch > 0x3FFFFFFFull) {
    set_last_error("gemm_plan_create: dimension too large");
    return CCGLIB_B200_INVALID_ARGUMENT;
  }
  if (d.variant != CCGLIB_B200_BASIC && d.variant != CCGLIB_B200_OPT) {
    set_last_error("gemm_plan_create: unknown variant %d", d.variant);
    return CCGLIB_B200_INVALID_ARGUMENT;
  }
  if (d.variant == CCGLIB_B200_BASIC && d.c_complex_axis == CCGLIB_B200_INTERLEAVED &&
      !opt.int1_bytes_in) {
    set_last_error("complex-interleaved output is not supported in basic variant");
    return CCGLIB_B200_UNSUPPORTED;
  }
  if (d.a_mem_order != CCGLIB_B200_ROW_MAJOR) {
    set_last_error("GEMM does not support col-major A matrix");
    return CCGLIB_B200_UNSUPPORTED;
  }
  if (d.b_mem_order != CCGLIB_B200_COL_MAJOR) {
    set_last_error("GEMM does not support row-major B matrix");
    return CCGLIB_B200_UNSUPPORTED;
  }
  if (opt.int1_bytes_in && d.type_in != CCGLIB_B200_INT1) {
    set_last_error("gemm_plan_create: one-byte samples are a 1-bit input form");
    return CCGLIB_B200_INVALID_ARGUMENT;
  }

  ccglib_b200_gemm_plan plan{};
  plan.desc = d;
  plan.bytes_in = opt.int1_bytes_in ? 1 : 0;
  plan.bytes_interleaved = opt.int1_bytes_interleaved ? 1 : 0;
  CCGLIB_CUDA_TRY(cudaGetDevice(&plan.device));
  plan.sms = sm_count();
  if (plan.sms <= 0) return CCGLIB_B200_CUDA_ERROR;
  int cc_major = 0;
  CCGLIB_CUDA_TRY(cudaDeviceGetAttribute(&cc_major, cudaDevAttrComputeCapabilityMajor, plan.device));
  if (cc_major != 10) {
    set_last_error("This architecture is not supported (need compute capability 10.x)");
    return CCGLIB_B200_UNSUPPORTED;
  }
  plan.wait_cycles = wait_limit_cycles();

  // ---- kernel family and instruction descriptor
  // idesc: [4,6) D format, [7,10) A format, [10,13) B format, bit 13 negate A, bit 15/16 majors
  // (0 = K-major), [17,23) N>>3, [24,29) M>>4.
  uint32_t d_fmt = 1, ab_fmt = 0;  // fp32 accumulate
  int kind = kKindF16;
  plan.a_planes = 2;
  const size_t in_bits = type_bits(d.type_in);
  switch (d.type_in) {
  case CCGLIB_B200_FLOAT16:
    kind = kKindF16;
    ab_fmt = 0;
    break;
  case CCGLIB_B200_BFLOAT16:
    kind = kKindF16;
    ab_fmt = 1;
    break;
  case CCGLIB_B200_FLOAT32:
    kind = kKindTF32;
    ab_fmt = 2;
    break;
  case CCGLIB_B200_FLOAT8E4M3:
    kind = kKindF8F6F4;
    ab_fmt = 0;
    break;
  case CCGLIB_B200_FLOAT8E5M2:
    kind = kKindF8F6F4;
    ab_fmt = 1;
    break;
  case CCGLIB_B200_INT1:
    // +-1 samples run either as signed bytes on the integer kind (s32 accumulators) or, opt-in, as
    // e2m1 nibbles on the block-scaled 4-bit kind with all scale factors 1.0 (fp32 accumulators)
    // The fp32 accumulator of the 4-bit path holds the integer sums exactly while 2K < 2^24
    // (verified bit-exact against the CPU oracle up to K = 65536); beyond K = 2^22 samples the
    // integer kind takes over.  The 4-bit path runs at twice the rate and a fraction of the power.
    plan.nibbles = (env_int("CCGLIB_B200_INT1_MXF4", 1) != 0 && d.k <= (size_t{1} << 22)) ? 1 : 0;
    kind = plan.nibbles ? kKindMXF4 : kKindI8;
    ab_fmt = 1;  // signed 8-bit, resp. e2m1
    d_fmt = 2;   // s32 accumulate (unused by the block-scaled descriptor)
    // the integer kind has no negate bit and reads -Ai from a third plane; the 4-bit kind negates
    // in the instruction descriptor (a third plane remains selectable for cross-checking)
    plan.a_planes = (plan.nibbles && env_int("CCGLIB_B200_MXF4_NEGATE", 1) != 0) ? 2 : 3;
    break;
  default:
    set_last_error("No kernel available for input type %d", d.type_in);
    return CCGLIB_B200_UNSUPPORTED;
  }
  bool out_ok = false;
  switch (d.type_in) {
  case CCGLIB_B200_INT1:
    out_ok = d.type_out == CCGLIB_B200_INT32;
    break;
  case CCGLIB_B200_FLOAT16:
    out_ok = d.type_out == CCGLIB_B200_FLOAT32 || d.type_out == CCGLIB_B200_FLOAT16;
    break;
  case CCGLIB_B200_BFLOAT16:
    out_ok = d.type_out == CCGLIB_B200_FLOAT32 || d.type_out == CCGLIB_B200_BFLOAT16;
    break;
  case CCGLIB_B200_FLOAT32:
    out_ok = d.type_out == CCGLIB_B200_FLOAT32 || d.type_out == CCGLIB_B200_FLOAT16 ||
             d.type_out == CCGLIB_B200_BFLOAT16;
    break;
  default:
    out_ok = d.type_out == CCGLIB_B200_FLOAT32;
    break;
  }
  if (!out_ok) {
    set_last_error("Unsupported combination of input/output data types (%d -> %d)", d.type_in,
                   d.type_out);
    return CCGLIB_B200_UNSUPPORTED;
  }
  plan.out_elem_bytes = type_bits(d.type_out) / 8;

  // ---- staging mode and operand geometry
  if (d.type_in == CCGLIB_B200_INT1) {
    plan.stage_mode = kExpandBits;
    // one signed byte, resp. one nibble, per sample after expansion
    plan.k_bytes = plan.nibbles ? ceil_div<size_t>(d.k, 2) : d.k;
    plan.pitch = ceil_div<size_t>(plan.k_bytes, 16) * 16;
  } else {
    plan.k_bytes = d.k * in_bits / 8;
    if (d.variant == CCGLIB_B200_OPT) {
      plan.stage_mode = kDirect;
      plan.pitch = kSlabRowBytes;
    } else if (plan.k_bytes % 16 == 0) {
      plan.stage_mode = kDirect;
      plan.pitch = plan.k_bytes;
    } else {
      plan.stage_mode = kPadRows;
      plan.pitch = ceil_div<size_t>(plan.k_bytes, 16) * 16;
    }
  }

  // ---- tile shape
  // BN = 256 halves the shared-memory traffic per flop; BN = 128 double-buffers the accumulators
  // so the epilogue overlaps the next tile's main loop (short K), wastes less on a ragged N and
  // gives more tiles (small M*N).  Compare waves of tiles x relative time per tile; the two
  // efficiency factors are measured: at 2 KB rows the 256-wide tile is 5-8 % slower per flop, at
  // 4 KB rows and beyond 3-7 % faster.
  const size_t tiles_m = d.batch * ceil_div<size_t>(d.m, kBlockM);
  const size_t sms = static_cast<size_t>(plan.sms);
  const bool short_k = plan.k_bytes <= 2048;
  const double cost_128 = static_cast<double>(ceil_div(tiles_m * ceil_div<size_t>(d.n, 128), sms)) *
                          (short_k ? 1.0 : 1.05);
  // (short rows of 32-bit input are the exception: twice the operand bytes per flop make the
  // narrow tile's extra traffic from L2 cost more, in time and under the power cap in clock,
  // than the wide tile's exposed epilogue: 518 against 479-507 TFLOP/s sustained on
  // 256 x 2048 x 512 tf32)
  const double wide_short = in_bits >= 32 ? 0.97 : 1.06;
  const double cost_256 = static_cast<double>(ceil_div(tiles_m * ceil_div<size_t>(d.n, 256), sms)) *
                          2.0 * (short_k ? wide_short : 1.0);
  // 64-column tiles double the tile count once more for problems that cannot fill the SMs (a
  // single 1024^3 product is 64 tiles of 128 x 128: 466 against 419 TFLOP/s).
  const double cost_64 = static_cast<double>(ceil_div(tiles_m * ceil_div<size_t>(d.n, 64), sms)) *
                         0.5 * kCost64;
  int bn = cost_256 <= cost_128 ? 256 : 128;
  if (cost_64 < (bn == 256 ? cost_256 : cost_128)) bn = 64;
  int sw = 128;
  // A tuning table (CCGLIB_B200_TUNE_TABLE, written by `python -m ccglib_b200.tune --write`)
  // overrides the model for the problems it lists; the environment overrides both.
  TuneChoice tuned;
  plan.tuned = tune_table_lookup(std::getenv("CCGLIB_B200_TUNE_TABLE"), d,
                                 ceil_div<size_t>(d.k * in_bits, 8), &tuned);
  if (!plan.tuned) tuned = TuneChoice{};
  if (tuned.bn != 0) bn = tuned.bn;
  plan.group_n = tuned.group_n > 0 ? tuned.group_n : 0;
  const bool bn_forced = env_int("CCGLIB_B200_BN", 0) != 0 || tuned.bn != 0;
  bn = env_int("CCGLIB_B200_BN", bn);
  sw = env_int("CCGLIB_B200_SW", sw);
  const int pair_default = tuned.pair >= 0 ? tuned.pair : (kind == kKindMXF4 ? 1 : 0);
  const bool want_pair = env_int("CCGLIB_B200_PAIR", pair_default) != 0 && d.m > kBlockM;
  if (kind == kKindMXF4) {
    // two accumulators plus 32 scale-factor columns must fit 512 tensor-memory columns: 224
    // columns for a CTA pair (N of a 256-row MMA is a multiple of 32), else 192
    if (bn == 256) bn = 192;
    if (want_pair && !bn_forced) {
      // The pair kernel is bound by operand traffic from L2: time per 256 x bn tile goes as
      // bn / 256 + 1, and there are sms / 2 clusters.  Wider tiles move fewer bytes per flop
      // (224 columns: 8 % fewer than 192) but may quantise worse on a few waves (4096^2,
      // batch 1: 1.44 ms with 192 columns, 1.80 ms with 128).
      const size_t clusters = sms / 2;
      const size_t rows = d.batch * ceil_div<size_t>(d.m, 2 * kBlockM);
      double best = 0.0;
      for (int cand : {224, 192, 128}) {
        if (cand == 224 && plan.a_planes != 2) continue;
        const double cost = static_cast<double>(ceil_div(rows * ceil_div<size_t>(d.n, cand), clusters)) *
                            (cand / 256.0 + 1.0);
        if (best == 0.0 || cost < best) {
          best = cost;
          bn = cand;
        }
      }
    }
    if (bn == 64) bn = 128;
    sw = 128;
  }
  if (bn == 64) sw = 128;
  const bool bn_ok = bn == 64 || bn == 128 || bn == 256 ||
                     (kind == kKindMXF4 && (bn == 192 || (bn == 224 && want_pair &&
                                                          plan.a_planes == 2)));
  if (!bn_ok || (sw != 64 && sw != 128)) {
    set_last_error("CCGLIB_B200_BN must be 64, 128 or 256 and CCGLIB_B200_SW 64 or 128");
    return CCGLIB_B200_INVALID_ARGUMENT;
  }
  // CTA pairs (cta_group::2, 256-row tiles) are opt-in: they reach a higher tensor-pipe duty cycle
  // per clock (95.8 % against 91.8 % on 8192^3 f16), but every MMA reads half of B over the
  // SM-to-SM network, twice per k-step in the four-product complex scheme, which costs about 20 %
  // more energy per flop.  While the 1 kW cap does not bind (constant operand bytes) the pair is
  // 1-8 % ahead; on normally distributed operands the cap pulls its clock to 1.0 GHz against
  // 1.25 GHz and it delivers 1116 against 1341 TFLOP/s.
  // The 4-bit path is the exception: it is bound by operand traffic from L2, not by power, and a
  // pair halves the B bytes each SM fetches (5.6 against 5.3 POPS at 4096 x 4096 x 65536).
  const bool pair = want_pair && sw == 128 && bn != 64;
  // Split-K for problems that leave most SMs idle: when even 128 x 128 tiles fill less than half
  // (a quarter) of the device and K is long enough to share, a cluster of 2 (4) CTAs per tile
  // shortens the MMA chain per SM and moves fewer operand bytes out of L2 than narrower tiles
  // would (1024^3, batch 1: 64 tiles x 2 CTAs instead of 128 tiles of 128 x 64).  The exchange
  // costs about 4 us per call, a K-block about 0.35 us less per CTA: measured on 1024 x 1024,
  // f16, split 2 against 128 x 64 tiles: K = 512 14.3 against 12.3 us, K = 1024 16.4 against
  // 18.4 us, K = 4096 33.7 against 53.2 us.
  int split = 1;
  {
    const size_t tiles128 = tiles_m * ceil_div<size_t>(d.n, 128);
    const size_t k_blocks = ceil_div<size_t>(plan.k_bytes, 128);
    const bool can_split = kind != kKindI8 && kind != kKindMXF4 &&
                           d.type_out == CCGLIB_B200_FLOAT32 && !pair && sw == 128 &&
                           !bn_forced;
    if (can_split && 4 * tiles128 <= sms && k_blocks >= 24) {
      split = 4;
    } else if (can_split && 2 * tiles128 <= sms && k_blocks >= 12) {
      split = 2;
    }
    if (tuned.split_k > 0) split = tuned.split_k;
    split = env_int("CCGLIB_B200_SPLITK", split);
    if (split != 1 && split != 2 && split != 4) {
      set_last_error("CCGLIB_B200_SPLITK must be 1, 2 or 4");
      return CCGLIB_B200_INVALID_ARGUMENT;
    }
    if (split > 1 && (kind == kKindI8 || kind == kKindMXF4 || d.type_out != CCGLIB_B200_FLOAT32 ||
                      k_blocks < static_cast<size_t>(split))) {
      split = 1;  // no such instance: integer sums, 16-bit output, or less K than CTAs
    }
  }
  if (split > 1) {
    bn = 128;
    sw = 128;
  }
  plan.bn = bn;
  plan.sw = sw;
  switch (split > 1 ? -1 : kind) {
  case -1:
    plan.kernel = kind == kKindF16    ? splitk_entry<kKindF16>(split)
                  : kind == kKindTF32 ? splitk_entry<kKindTF32>(split)
                                      : splitk_entry<kKindF8F6F4>(split);
    break;
  case kKindF16:
    plan.kernel = pick_float_out<kKindF16>(d.type_out, bn, sw, pair);
    break;
  case kKindTF32:
    plan.kernel = pick_float_out<kKindTF32>(d.type_out, bn, sw, pair);
    break;
  case kKindF8F6F4:
    plan.kernel = pick_tile<kKindF8F6F4, 2, float>(bn, sw, pair);
    break;
  case kKindMXF4:
    if (plan.a_planes == 3) {
      plan.kernel = pair ? (bn == 192 ? pair_entry<kKindMXF4, 192, 3, IntFromFloat>()
                                      : pair_entry<kKindMXF4, 128, 3, IntFromFloat>())
                         : (bn == 192 ? entry<kKindMXF4, 192, 128, 3, IntFromFloat>()
                                      : entry<kKindMXF4, 128, 128, 3, IntFromFloat>());
    } else {
      plan.kernel = pair ? (bn == 224   ? pair_entry<kKindMXF4, 224, 2, IntFromFloat>()
                            : bn == 192 ? pair_entry<kKindMXF4, 192, 2, IntFromFloat>()
                                        : pair_entry<kKindMXF4, 128, 2, IntFromFloat>())
                         : (bn == 192 ? entry<kKindMXF4, 192, 128, 2, IntFromFloat>()
                                      : entry<kKindMXF4, 128, 128, 2, IntFromFloat>());
    }
    break;
  default:
    plan.kernel = pick_tile<kKindI8, 3, int>(bn, sw, pair);
    break;
  }
  if (plan.kernel.fn == nullptr) {
    set_last_error("no kernel instance for this type combination");
    return CCGLIB_B200_UNSUPPORTED;
  }
  const uint32_t mma_m = plan.kernel.pair ? 2 * kBlockM : kBlockM;
  plan.idesc = (d_fmt << 4) | (ab_fmt << 7) | (ab_fmt << 10) |
               (static_cast<uint32_t>(bn >> 3) << 17) | ((mma_m >> 4) << 24);
  plan.idesc_neg_a = plan.idesc | (1u << 13);
  if (kind == kKindMXF4) {
    // block-scaled descriptor: [7,10)/[10,13) operand formats (1 = e2m1), [17,23) N>>3, bit 23
    // scale format (1 = ue8m0), [24,29) M>>4; scale-factor byte ids and K size stay 0
    plan.idesc = (1u << 7) | (1u << 10) | (static_cast<uint32_t>(bn >> 3) << 17) | (1u << 23) |
                 ((mma_m >> 4) << 24);
    plan.idesc_neg_a = plan.idesc | (1u << 13);
  }
  CCGLIB_CUDA_TRY(cudaFuncSetAttribute(reinterpret_cast<const void *>(plan.kernel.fn),
                                       cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       plan.kernel.smem));
  if (plan.kernel.pair) {
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(static_cast<unsigned>(plan.sms & ~1));
    cfg.blockDim = dim3(kThreads);
    cfg.dynamicSmemBytes = plan.kernel.smem;
    cudaLaunchAttribute attr{};
    attr.id = cudaLaunchAttributeClusterDimension;
    attr.val.clusterDim.x = 2;
    attr.val.clusterDim.y = 1;
    attr.val.clusterDim.z = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    int clusters = 0;
    CCGLIB_CUDA_TRY(cudaOccupancyMaxActiveClusters(
        &clusters, reinterpret_cast<const void *>(plan.kernel.fn), &cfg));
    if (clusters < 1) {
      set_last_error("gemm_plan_create: the device cannot co-schedule a CTA pair");
      return CCGLIB_B200_UNSUPPORTED;
    }
    plan.max_clusters = clusters;
  }

  // ---- scratch for the staged modes, processed in batch chunks of bounded size
  plan.batch_chunk = d.batch;
  plan.lanes = 1;
  if (plan.stage_mode != kDirect) {
    const size_t per_item_a = plan.a_planes * d.m * plan.pitch;
    const size_t per_item_b = 2 * d.n * plan.pitch;
    const size_t per_item = per_item_a + per_item_b;
    const size_t cap = static_cast<size_t>(env_int("CCGLIB_B200_SCRATCH_MB", 8192)) << 20;
    // Two lanes pay when every chunk still fills the device several times over: aim at eight
    // chunks of at least eight waves of tiles each, within half the scratch cap per lane.
    const size_t tiles_per_item = ceil_div<size_t>(d.m, plan.kernel.pair ? 2 * kBlockM : kBlockM) *
                                  ceil_div<size_t>(d.n, plan.bn);
    const size_t ctas = plan.kernel.pair ? static_cast<size_t>(plan.sms) / 2 : plan.sms;
    size_t lane_chunk = ceil_div<size_t>(d.batch, 8);
    const size_t waves = static_cast<size_t>(env_int("CCGLIB_B200_LANE_WAVES", 8));
    const size_t min_items = ceil_div<size_t>(waves * ctas, tiles_per_item);
    if (lane_chunk < min_items) lane_chunk = min_items;
    if (lane_chunk * per_item > cap / 2) lane_chunk = cap / 2 / per_item;
    const bool two_lanes = env_int("CCGLIB_B200_LANES", 2) >= 2 && lane_chunk >= 1 &&
                           ceil_div<size_t>(d.batch, lane_chunk) >= 2;
    size_t chunk;
    if (two_lanes) {
      chunk = ceil_div(d.batch, ceil_div(d.batch, lane_chunk));  // equal chunks
      plan.lanes = 2;
    } else {
      chunk = cap / per_item;
      if (chunk < 1) chunk = 1;
      if (chunk > d.batch) chunk = d.batch;
      chunk = ceil_div(d.batch, ceil_div(d.batch, chunk));  // equal chunks: no short last launch
    }
    plan.batch_chunk = chunk;
    plan.scratch_bytes = plan.lanes * chunk * per_item;
    if (cudaMalloc(&plan.scratch_a, plan.scratch_bytes) != cudaSuccess) {
      cudaGetLastError();
      set_last_error("gemm_plan_create: could not allocate %zu bytes of staging scratch",
                     plan.scratch_bytes);
      return CCGLIB_B200_OUT_OF_MEMORY;
    }
    plan.scratch_b = static_cast<char *>(plan.scratch_a) + chunk * per_item_a;
    for (int j = 0; j < plan.lanes; ++j) {
      plan.lane_a[j] = static_cast<char *>(plan.scratch_a) + j * chunk * per_item;
      plan.lane_b[j] = static_cast<char *>(plan.lane_a[j]) + chunk * per_item_a;
    }
    if (plan.lanes == 2) {
      cudaError_t err = cudaEventCreateWithFlags(&plan.ev_fork, cudaEventDisableTiming);
      for (int j = 0; j < 2 && err == cudaSuccess; ++j) {
        err = cudaStreamCreateWithFlags(&plan.lane_stream[j], cudaStreamNonBlocking);
        if (err == cudaSuccess) {
          err = cudaEventCreateWithFlags(&plan.ev_join[j], cudaEventDisableTiming);
        }
      }
      if (err != cudaSuccess) {
        release_plan_resources(plan);
        return cuda_fail(err, "creating the staging lanes");
      }
    }
  }

  if (env_int("CCGLIB_B200_VERBOSE", 0) != 0) {
    // the counterpart of the reference's DEBUG print of its launch geometry (src/mma/GEMM.cpp:84-95)
    std::fprintf(stderr,
                 "ccglib_b200 plan: batch %zu M %zu N %zu K %zu types %d->%d variant %d | tile %d x "
                 "%d, stage rows %d B, %s%s, split-K %d, %s | staging mode %d, %d lane(s), chunk "
                 "%zu item(s), scratch %zu bytes | shared memory %d B, %d SMs\n",
                 d.batch, d.m, d.n, d.k, d.type_in, d.type_out, d.variant,
                 plan.kernel.pair ? 2 * kBlockM : kBlockM, plan.bn, plan.sw,
                 plan.kernel.pair ? "CTA pair" : "one CTA", plan.nibbles ? ", e2m1 operands" : "",
                 plan.kernel.split, plan.tuned ? "from the tuning table" : "built-in model",
                 plan.stage_mode, plan.lanes, plan.batch_chunk, plan.scratch_bytes,
                 plan.kernel.smem, plan.sms);
  }
  *out = new (std::nothrow) ccglib_b200_gemm_plan(plan);
  if (*out == nullptr) {
    release_plan_resources(plan);
    return CCGLIB_B200_OUT_OF_MEMORY;
  }
  return CCGLIB_B200_OK;
}

extern "C" size_t ccglib_b200_gemm_plan_scratch_bytes(const ccglib_b200_gemm_plan *plan) {
  return plan != nullptr ? plan->scratch_bytes : 0;
}

extern "C" int ccglib_b200_gemm_plan_tile(const ccglib_b200_gemm_plan *plan, int tile[5]) {
  if (plan == nullptr || tile == nullptr) {
    set_last_error("gemm_plan_tile: null argument");
    return CCGLIB_B200_INVALID_ARGUMENT;
  }
  tile[0] = plan->bn;
  tile[1] = plan->kernel.pair ? 1 : 0;
  tile[2] = plan->group_n;
  tile[3] = plan->tuned;
  tile[4] = plan->kernel.split;
  return CCGLIB_B200_OK;
}

extern "C" size_t ccglib_b200_gemm_plan_launches(const ccglib_b200_gemm_plan *plan) {
  if (plan == nullptr) return 0;
  if (plan->stage_mode == kDirect) return 1;
  return 3 * ceil_div<size_t>(plan->desc.batch, plan->batch_chunk);
}

extern "C" int ccglib_b200_gemm_plan_destroy(ccglib_b200_gemm_plan *plan) {
  if (plan == nullptr) return CCGLIB_B200_OK;
  release_plan_resources(*plan);
  delete plan;
  return CCGLIB_B200_OK;
}

namespace {

// Launch the GEMM kernel on `nb` batch items whose operands the kernel can read directly.
int launch_gemm(const ccglib_b200_gemm_plan &plan, const void *a, const void *b, void *c,
                size_t nb, bool tiled, cudaStream_t stream) {
  const ccglib_b200_gemm_desc &d = plan.desc;
  GemmParams p{};
  p.M = static_cast<uint32_t>(d.m);
  p.N = static_cast<uint32_t>(d.n);
  const bool pair = plan.kernel.pair;
  p.tiles_m = static_cast<uint32_t>(ceil_div<size_t>(d.m, pair ? 2 * kBlockM : kBlockM));
  p.tiles_n = static_cast<uint32_t>(ceil_div<size_t>(d.n, plan.bn));
  // column-panel width of the tile walk: 4 for 256-column tiles; 8 for narrower ones, except
  // on short matrices (one or two row tiles: +2 % on 256 x 2048 x 512)
  p.group_n = static_cast<uint32_t>(env_int(
      "CCGLIB_B200_GROUP",
      plan.group_n > 0 ? plan.group_n : ((plan.bn == 256 || p.tiles_m <= 2) ? 4 : 8)));
  if (p.group_n == 0) p.group_n = 1;
  const size_t tiles = nb * p.tiles_m * p.tiles_n;
  if (tiles > 0x7FFFFFFFull) {
    set_last_error("gemm_run: too many tiles");
    return CCGLIB_B200_INVALID_ARGUMENT;
  }
  p.num_tiles = static_cast<uint32_t>(tiles);
  p.tiled = tiled ? 1u : 0u;
  CUtensorMap &tm_a = plan.tm_a, &tm_b = plan.tm_b, &tm_c = plan.tm_c;
  const bool maps_cached = plan.map_a == a && plan.map_b == b && plan.map_c == c &&
                           plan.map_nb == nb && a != nullptr;
  int rc = CCGLIB_B200_OK;
  if (tiled) {
    const size_t slabs_k = ceil_div<size_t>(plan.k_bytes, kSlabRowBytes);
    const size_t slabs_m = ceil_div<size_t>(d.m, kSlabRowsA);
    const size_t slabs_n = ceil_div<size_t>(d.n, kSlabRowsB);
    p.k_per_slab = kSlabRowBytes / plan.sw;
    p.slabs_k = static_cast<uint32_t>(slabs_k);
    p.a_slabs_m = static_cast<uint32_t>(slabs_m);
    p.b_slabs_n = static_cast<uint32_t>(slabs_n);
    p.b_slab_rows = kSlabRowsB;
    p.k_blocks = static_cast<uint32_t>(slabs_k * p.k_per_slab);
    if (!maps_cached) rc = make_map(&tm_a, a, kSlabRowBytes, kSlabRowsA, 2 * nb * slabs_m * slabs_k, kSlabRowBytes,
                  kSlabRowBytes * kSlabRowsA, plan.sw, kBlockM, 2);
    if (!maps_cached && rc != CCGLIB_B200_OK) return rc;
    if (!maps_cached) rc = make_map(&tm_b, b, kSlabRowBytes, kSlabRowsB, 2 * nb * slabs_n * slabs_k, kSlabRowBytes,
                  kSlabRowBytes * kSlabRowsB, plan.sw, pair ? plan.bn / 2 : plan.bn, 2);
    if (!maps_cached && rc != CCGLIB_B200_OK) return rc;
  } else {
    p.k_blocks = static_cast<uint32_t>(ceil_div<size_t>(plan.k_bytes, plan.sw));
    if (!maps_cached) rc = make_map(&tm_a, a, plan.k_bytes, d.m, plan.a_planes * nb, plan.pitch, plan.pitch * d.m,
                  plan.sw, kBlockM, plan.a_planes);
    if (!maps_cached && rc != CCGLIB_B200_OK) return rc;
    if (!maps_cached) rc = make_map(&tm_b, b, plan.k_bytes, d.n, 2 * nb, plan.pitch, plan.pitch * d.n, plan.sw,
                  pair ? plan.bn / 2 : plan.bn, 2);
    if (!maps_cached && rc != CCGLIB_B200_OK) return rc;
  }
  p.idesc = plan.idesc;
  p.idesc_neg_a = plan.idesc_neg_a;
  p.c = c;
  const bool row = d.c_mem_order == CCGLIB_B200_ROW_MAJOR;
  const bool planar = d.c_complex_axis == CCGLIB_B200_PLANAR;
  p.c_layout = planar ? (row ? kPlanarRow : kPlanarCol) : (row ? kInterRow : kInterCol);
  const bool is_int = d.type_in == CCGLIB_B200_INT1;
  // the integer path always applies alpha and beta (as the reference CPU GEMM does), after
  // truncating them to int
  p.alpha_re = is_int ? static_cast<float>(static_cast<int>(d.alpha_re)) : d.alpha_re;
  p.alpha_im = is_int ? static_cast<float>(static_cast<int>(d.alpha_im)) : d.alpha_im;
  p.beta_re = is_int ? static_cast<float>(static_cast<int>(d.beta_re)) : d.beta_re;
  p.beta_im = is_int ? static_cast<float>(static_cast<int>(d.beta_im)) : d.beta_im;
  p.have_alpha = (p.alpha_re != 1.0f || p.alpha_im != 0.0f) ? 1u : 0u;
  p.have_beta = (p.beta_re != 0.0f || p.beta_im != 0.0f) ? 1u : 0u;
  // 16-byte stores need every row run to start on a 16-byte boundary
  const size_t run_bytes = (planar ? d.n : 2 * d.n) * plan.out_elem_bytes;
  p.vec_ok = (row && aligned16(c) && run_bytes % 16 == 0) ? 1u : 0u;
  // L2 prefetch distance in k-blocks; off by default: on the HBM-bound short-K shape (256 x 2048 x
  // 512, batch 4096) distances 3..24 were 12-34 % slower than none, and slower on the others too
  p.prefetch = static_cast<uint32_t>(env_int("CCGLIB_B200_PREFETCH", 0));
  // TMA-store epilogue: row-major C (planar or interleaved), four-byte elements, 16-byte aligned rows
  p.epi_tma = (plan.kernel.epi_tma && p.vec_ok && plan.out_elem_bytes == 4) ? 1u : 0u;
  if (!maps_cached) {
    if (p.epi_tma) {
      const size_t row_bytes = planar ? d.n * 4 : d.n * 8;
      rc = make_map(&tm_c, c, row_bytes, d.m, planar ? 2 * nb : nb, row_bytes, d.m * row_bytes,
                    128, 32, 1);
      if (rc != CCGLIB_B200_OK) return rc;
    } else {
      tm_c = tm_a;  // placeholder when the epilogue stores straight from registers
    }
    plan.map_a = a;
    plan.map_b = b;
    plan.map_c = c;
    plan.map_nb = nb;
  }
  if (plan.status_ptr == nullptr &&
      cudaGetSymbolAddress(reinterpret_cast<void **>(&plan.status_ptr), g_device_status) !=
          cudaSuccess) {
    return cuda_fail(cudaGetLastError(), "cudaGetSymbolAddress(g_device_status)");
  }
  p.status = plan.status_ptr;
  p.wait_cycles = plan.wait_cycles;
  if (pair) {
    const size_t clusters = tiles < static_cast<size_t>(plan.max_clusters)
                                ? tiles
                                : static_cast<size_t>(plan.max_clusters);
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(static_cast<unsigned>(2 * clusters));
    cfg.blockDim = dim3(kThreads);
    cfg.dynamicSmemBytes = plan.kernel.smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr{};
    attr.id = cudaLaunchAttributeClusterDimension;
    attr.val.clusterDim.x = 2;
    attr.val.clusterDim.y = 1;
    attr.val.clusterDim.z = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    CCGLIB_CUDA_TRY(cudaLaunchKernelEx(&cfg, plan.kernel.fn, tm_a, tm_b, tm_c, p));
    return CCGLIB_B200_OK;
  }
  if (plan.kernel.split > 1) {
    // one cluster per tile (not persistent); clusters beyond the co-resident ones run as they fit
    if (tiles * plan.kernel.split > 0x7FFFFFFFull) {
      set_last_error("gemm_run: too many tiles for the split-K form");
      return CCGLIB_B200_INVALID_ARGUMENT;
    }
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(static_cast<unsigned>(tiles * plan.kernel.split));
    cfg.blockDim = dim3(kThreads);
    cfg.dynamicSmemBytes = plan.kernel.smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr{};
    attr.id = cudaLaunchAttributeClusterDimension;
    attr.val.clusterDim.x = static_cast<unsigned>(plan.kernel.split);
    attr.val.clusterDim.y = 1;
    attr.val.clusterDim.z = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    CCGLIB_CUDA_TRY(cudaLaunchKernelEx(&cfg, plan.kernel.fn, tm_a, tm_b, tm_c, p));
    return CCGLIB_B200_OK;
  }
  const unsigned grid = static_cast<unsigned>(tiles < static_cast<size_t>(plan.sms) ? tiles
                                                                                   : plan.sms);
  plan.kernel.fn<<<grid, kThreads, plan.kernel.smem, stream>>>(tm_a, tm_b, tm_c, p);
  CCGLIB_CUDA_TRY(cudaGetLastError());
  return CCGLIB_B200_OK;
}

// Re-stage batch items [b0, b0 + nb) of A and B into (sa, sb) in the form the kernel reads.
int stage_chunk(const ccglib_b200_gemm_plan &plan, const void *d_a, const void *d_b, size_t b0,
                size_t nb, void *sa, void *sb, cudaStream_t stream) {
  const ccglib_b200_gemm_desc &d = plan.desc;
  const bool tiled_in = d.variant == CCGLIB_B200_OPT && !plan.bytes_in;
  int rc;
  if (plan.stage_mode == kExpandBits && plan.bytes_in) {
    // one byte per sample, 2 * rows * K bytes per batch item in either complex order
    rc = launch_expand_bytes(static_cast<const char *>(d_a) + b0 * 2 * d.m * d.k, sa, nb, d.m, d.k,
                             plan.pitch, plan.a_planes, plan.bytes_interleaved != 0, stream,
                             plan.nibbles != 0);
    if (rc != CCGLIB_B200_OK) return rc;
    return launch_expand_bytes(static_cast<const char *>(d_b) + b0 * 2 * d.n * d.k, sb, nb, d.n,
                               d.k, plan.pitch, 2, plan.bytes_interleaved != 0, stream,
                               plan.nibbles != 0);
  }
  if (plan.stage_mode == kExpandBits) {
    const size_t words = ceil_div<size_t>(d.k, 32);
    size_t a_item, b_item;
    if (tiled_in) {
      const size_t k_c_words = kSlabRowBytes / 4;
      const size_t slabs_k = ceil_div<size_t>(words, k_c_words);
      a_item = ceil_div<size_t>(d.m, kSlabRowsA) * slabs_k * 2 * kSlabRowsA * kSlabRowBytes;
      b_item = ceil_div<size_t>(d.n, kSlabRowsB) * slabs_k * 2 * kSlabRowsB * kSlabRowBytes;
    } else {
      a_item = 2 * d.m * words * 4;
      b_item = 2 * d.n * words * 4;
    }
    rc = launch_expand_bits(static_cast<const char *>(d_a) + b0 * a_item, sa, nb, d.m, d.k,
                            plan.pitch, plan.a_planes, tiled_in, kSlabRowsA, kSlabRowBytes * 8,
                            stream, plan.nibbles != 0);
    if (rc != CCGLIB_B200_OK) return rc;
    return launch_expand_bits(static_cast<const char *>(d_b) + b0 * b_item, sb, nb, d.n, d.k,
                              plan.pitch, 2, tiled_in, kSlabRowsB, kSlabRowBytes * 8, stream,
                              plan.nibbles != 0);
  }
  rc = launch_pad_rows(static_cast<const char *>(d_a) + b0 * 2 * d.m * plan.k_bytes, sa,
                       nb * 2 * d.m, plan.k_bytes, plan.pitch, stream);
  if (rc != CCGLIB_B200_OK) return rc;
  return launch_pad_rows(static_cast<const char *>(d_b) + b0 * 2 * d.n * plan.k_bytes, sb,
                         nb * 2 * d.n, plan.k_bytes, plan.pitch, stream);
}

} // namespace

extern "C" int ccglib_b200_gemm_run(ccglib_b200_gemm_plan *plan, const void *d_a, const void *d_b,
                                    void *d_c, void *stream_v) {
  if (plan == nullptr) {
    set_last_error("gemm_run: null argument");
    return CCGLIB_B200_INVALID_ARGUMENT;
  }
  return run_gemm_items(plan, d_a, d_b, d_c, plan->desc.batch, stream_v);
}

int ccglib_b200::run_gemm_items(ccglib_b200_gemm_plan *plan, const void *d_a, const void *d_b,
                                void *d_c, size_t items, void *stream_v) {
  if (plan == nullptr || d_a == nullptr || d_b == nullptr || d_c == nullptr) {
    set_last_error("gemm_run: null argument");
    return CCGLIB_B200_INVALID_ARGUMENT;
  }
  if (items == 0 || items > plan->desc.batch) {
    set_last_error("gemm_run: %zu batch items asked of a plan made for %zu", items,
                   plan->desc.batch);
    return CCGLIB_B200_INVALID_ARGUMENT;
  }
  cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
  // the first `items` batch items: the batch is the outermost axis of every operand
  ccglib_b200_gemm_desc d = plan->desc;
  d.batch = items;
  const bool tiled_in = d.variant == CCGLIB_B200_OPT && !plan->bytes_in;
  if (plan->stage_mode == kDirect) {
    if (!aligned16(d_a) || !aligned16(d_b)) {
      set_last_error("gemm_run: A and B must be 16-byte aligned");
      return CCGLIB_B200_INVALID_ARGUMENT;
    }
    return launch_gemm(*plan, d_a, d_b, d_c, d.batch, tiled_in, stream);
  }
  // Staged modes: re-stage a chunk of batch items into scratch, then multiply it.
  const size_t c_item_bytes = 2 * d.m * d.n * plan->out_elem_bytes;
  if (plan->lanes < 2) {
    for (size_t b0 = 0; b0 < d.batch; b0 += plan->batch_chunk) {
      const size_t nb = (d.batch - b0 < plan->batch_chunk) ? d.batch - b0 : plan->batch_chunk;
      int rc = stage_chunk(*plan, d_a, d_b, b0, nb, plan->scratch_a, plan->scratch_b, stream);
      if (rc != CCGLIB_B200_OK) return rc;
      rc = launch_gemm(*plan, plan->scratch_a, plan->scratch_b,
                       static_cast<char *>(d_c) + b0 * c_item_bytes, nb, false, stream);
      if (rc != CCGLIB_B200_OK) return rc;
    }
    return CCGLIB_B200_OK;
  }
  // Two lanes: fork both internal streams off the caller's stream, deal the chunks out
  // alternately, join both back.  Everything a lane does is ordered on its own stream, so its
  // buffer is never re-staged before the GEMM that read it has finished.
  CCGLIB_CUDA_TRY(cudaEventRecord(plan->ev_fork, stream));
  for (int j = 0; j < 2; ++j) {
    CCGLIB_CUDA_TRY(cudaStreamWaitEvent(plan->lane_stream[j], plan->ev_fork, 0));
  }
  int rc = CCGLIB_B200_OK;
  size_t ci = 0;
  for (size_t b0 = 0; b0 < d.batch && rc == CCGLIB_B200_OK; b0 += plan->batch_chunk, ++ci) {
    const size_t nb = (d.batch - b0 < plan->batch_chunk) ? d.batch - b0 : plan->batch_chunk;
    const int j = static_cast<int>(ci & 1);
    rc = stage_chunk(*plan, d_a, d_b, b0, nb, plan->lane_a[j], plan->lane_b[j],
                     plan->lane_stream[j]);
    if (rc == CCGLIB_B200_OK) {
      rc = launch_gemm(*plan, plan->lane_a[j], plan->lane_b[j],
                       static_cast<char *>(d_c) + b0 * c_item_bytes, nb, false,
                       plan->lane_stream[j]);
    }
  }
  // join even after a failed launch, so that the caller's stream stays ordered after the lanes
  for (int j = 0; j < 2; ++j) {
    CCGLIB_CUDA_TRY(cudaEventRecord(plan->ev_join[j], plan->lane_stream[j]));
    CCGLIB_CUDA_TRY(cudaStreamWaitEvent(stream, plan->ev_join[j], 0));
  }
  return rc;
}

extern "C" int ccglib_b200_device_status(unsigned *word) {
  if (word == nullptr) {
    set_last_error("device_status: null argument");
    return CCGLIB_B200_INVALID_ARGUMENT;
  }
  CCGLIB_CUDA_TRY(cudaDeviceSynchronize());
  unsigned value = 0;
  CCGLIB_CUDA_TRY(cudaMemcpyFromSymbol(&value, g_device_status, sizeof(value)));
  if (value != 0) {
    const unsigned zero = 0;
    CCGLIB_CUDA_TRY(cudaMemcpyToSymbol(g_device_status, &zero, sizeof(zero)));
    set_last_error("device status word 0x%x: a bounded device-side wait gave up", value);
  }
  *word = value;
  return value == 0 ? CCGLIB_B200_OK : CCGLIB_B200_DEVICE_TIMEOUT;
}

#ifdef CCGLIB_B200_TRACE
// Instrumented builds only: copy the clock stamps out (and clear them).
extern "C" __attribute__((visibility("default"))) int ccglib_b200_debug_trace_read(
    long long *host, size_t count) {
  const size_t all = sizeof(g_trace) / sizeof(long long);
  if (host == nullptr || count > all) return CCGLIB_B200_INVALID_ARGUMENT;
  CCGLIB_CUDA_TRY(cudaDeviceSynchronize());
  CCGLIB_CUDA_TRY(cudaMemcpyFromSymbol(host, g_trace, count * sizeof(long long)));
  return CCGLIB_B200_OK;
}
#endif

// ------------------------------------------------------------------------------------------
// Self-test of the time-out machinery: a wait that is guaranteed to run out, made on the host
// side of the contract (an mbarrier nobody arrives on), so that nothing faults or hangs.
namespace ccglib_b200 {
namespace {

__device__ long long g_selftest_waited[2];

// Warp 0 of CTA 0 (the cluster leader in the pair form) waits `limit` cycles on a barrier that
// never completes, with the same mbar_wait the GEMM kernels use; it must give up, raise the
// abort flag (its own and, in a pair, the peer's) and record kDevTimeoutProducer.  The second
// waiter (warp 1 of the same CTA, or warp 0 of the peer CTA) has a limit `other_limit` that is
// much longer and a different code: it must come back early through the abort flag, without
// recording its code.  Each waiter stores the cycles it spent.
template <bool PAIR>
__global__ void __launch_bounds__(64, 1)
wait_timeout_selftest_kernel(unsigned int *status, long long limit, long long other_limit) {
  __shared__ uint64_t bar;
  __shared__ int abort_word;
  volatile int *abort_flag = &abort_word;
  const uint32_t warp = threadIdx.x >> 5;
  uint32_t rank = 0, peer_abort = 0;
  if (threadIdx.x == 0) {
    mbar_init(smem_u32(&bar), 1);
    *abort_flag = 0;
    fence_mbar_init();
  }
  if constexpr (PAIR) {
    rank = cluster_ctarank();
    cluster_sync();
    peer_abort = map_to_cta(smem_u32(&abort_word), rank ^ 1u);
  } else {
    __syncthreads();
  }
  const bool first = rank == 0 && warp == 0;
  const bool second = PAIR ? (rank == 1 && warp == 0) : (warp == 1);
  if (first || second) {
    const long long t0 = clock64();
    mbar_wait(smem_u32(&bar), 0, abort_flag, status,
              first ? kDevTimeoutProducer : kDevTimeoutEpilogue, first ? limit : other_limit,
              first ? peer_abort : 0u);
    if ((threadIdx.x & 31) == 0) g_selftest_waited[first ? 0 : 1] = clock64() - t0;
  }
  if constexpr (PAIR) {
    cluster_sync();
  }
}

} // namespace
} // namespace ccglib_b200

extern "C" int ccglib_b200_selftest_wait_timeout(long long limit_cycles, int pair,
                                                 long long waited_cycles[2]) {
  if (limit_cycles < 1 || limit_cycles > 10000000ll || waited_cycles == nullptr) {
    set_last_error("selftest_wait_timeout: limit must be 1..1e7 cycles and the result array non-null");
    return CCGLIB_B200_INVALID_ARGUMENT;
  }
  unsigned int *status = nullptr;
  CCGLIB_CUDA_TRY(cudaGetSymbolAddress(reinterpret_cast<void **>(&status), g_device_status));
  const long long other_limit = 200 * limit_cycles;  // bounded as well: at most 2e9 cycles
  if (pair != 0) {
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(2);
    cfg.blockDim = dim3(64);
    cudaLaunchAttribute attr{};
    attr.id = cudaLaunchAttributeClusterDimension;
    attr.val.clusterDim.x = 2;
    attr.val.clusterDim.y = 1;
    attr.val.clusterDim.z = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    CCGLIB_CUDA_TRY(cudaLaunchKernelEx(&cfg, wait_timeout_selftest_kernel<true>, status,
                                       limit_cycles, other_limit));
  } else {
    wait_timeout_selftest_kernel<false><<<1, 64>>>(status, limit_cycles, other_limit);
    CCGLIB_CUDA_TRY(cudaGetLastError());
  }
  CCGLIB_CUDA_TRY(cudaDeviceSynchronize());
  CCGLIB_CUDA_TRY(cudaMemcpyFromSymbol(waited_cycles, g_selftest_waited, 2 * sizeof(long long)));
  return CCGLIB_B200_OK;
}

// ------------------------------------------------------------------------------------------
// Allocation-free 1-bit GEMM.
//
// Some callers must not allocate device memory at all once they are running: a streaming
// correlator or beamformer loop whose device memory was handed out in full at start-up (to its own
// ring buffers or to a framework's caching allocator, so a later cudaMalloc simply fails), and
// host threads for which the implicit device-wide synchronisation of cudaMalloc / cudaFree would
// stall every other stream of the process in the middle of an observation.  The 1-bit GEMM needs
// scratch (the +-1 byte expansion of A and B that the tensor cores read), which a plan normally
// allocates.  This entry point takes that scratch from a fixed array that is part of the library
// image instead: every device that loads the library holds kStaticScratchBytes for it until the
// process exits.
namespace {

constexpr size_t kStaticScratchBytes = 32u << 20;  // 32 MiB, fixed at build time

static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

constexpr int kMaxDevices = 64;
void *g_static_scratch_addr[kMaxDevices] = {nullptr};

// The array's name is only a host-side handle; the address kernels and tensor maps can use comes
// from cudaGetSymbolAddress, looked up once per device with that device current.
int static_scratch_address(void **out) {
  int dev = 0;
  CCGLIB_CUDA_TRY(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kMaxDevices) {
    set_last_error("gemm_int1_static_scratch: device ordinal %d out of range", dev);
    return CCGLIB_B200_INVALID_ARGUMENT;
  }
  if (g_static_scratch_addr[dev] == nullptr) {
    void *ptr = nullptr;
    const cudaError_t err = cudaGetSymbolAddress(&ptr, g_static_scratch);
    if (err != cudaSuccess) return cuda_fail(err, "cudaGetSymbolAddress(g_static_scratch)");
    g_static_scratch_addr[dev] = ptr;
  }
  *out = g_static_scratch_addr[dev];
  return CCGLIB_B200_OK;
}

} // namespace

extern "C" int ccglib_b200_gemm_int1_static_scratch(const ccglib_b200_gemm_desc *desc,
                                                    const void *d_a, const void *d_b, void *d_c,
                                                    void *stream) {
  if (desc == nullptr || d_a == nullptr || d_b == nullptr || d_c == nullptr) {
    set_last_error("gemm_int1_static_scratch: null argument");
    return CCGLIB_B200_INVALID_ARGUMENT;
  }
  const ccglib_b200_gemm_desc &d = *desc;
  if (d.type_in != CCGLIB_B200_INT1 || d.type_out != CCGLIB_B200_INT32) {
    set_last_error("gemm_int1_static_scratch: only 1-bit input with int32 output is supported");
    return CCGLIB_B200_UNSUPPORTED;
  }
  if (d.batch == 0 || d.m == 0 || d.n == 0 || d.k == 0 || d.m > 0x7FFFFFFFull ||
      d.n > 0x7FFFFFFFull || d.k > 0x7FFFFFFFull || d.batch > 0x3FFFFFFFull) {
    set_last_error("gemm_int1_static_scratch: batch, M, N and K must be positive and below 2^31");
    return CCGLIB_B200_INVALID_ARGUMENT;
  }
  if (d.variant != CCGLIB_B200_BASIC && d.variant != CCGLIB_B200_OPT) {
    set_last_error("gemm_int1_static_scratch: unknown variant %d", d.variant);
    return CCGLIB_B200_INVALID_ARGUMENT;
  }
  if (d.variant == CCGLIB_B200_BASIC && d.c_complex_axis == CCGLIB_B200_INTERLEAVED) {
    set_last_error("complex-interleaved output is not supported in basic variant");
    return CCGLIB_B200_UNSUPPORTED;
  }
  if (d.a_mem_order != CCGLIB_B200_ROW_MAJOR || d.b_mem_order != CCGLIB_B200_COL_MAJOR) {
    set_last_error("GEMM needs row-major A and col-major B");
    return CCGLIB_B200_UNSUPPORTED;
  }
  // A plan-shaped description on the stack; nothing here allocates on the host or the device.
  ccglib_b200_gemm_plan plan{};
  plan.desc = d;
  plan.a_planes = 3;
  plan.stage_mode = kExpandBits;
  plan.k_bytes = d.k;
  plan.pitch = ceil_div<size_t>(d.k, 16) * 16;
  plan.out_elem_bytes = 4;
  plan.wait_cycles = wait_limit_cycles();
  const size_t per_item_a = 3 * d.m * plan.pitch;
  const size_t per_item_b = 2 * d.n * plan.pitch;
  if (per_item_a + per_item_b > kStaticScratchBytes) {
    set_last_error("gemm_int1_static_scratch: one batch item needs (3*M + 2*N) * K = %zu bytes of "
                   "scratch but the built-in array holds %zu; use a plan (gemm_plan_create) for "
                   "this size",
                   per_item_a + per_item_b, kStaticScratchBytes);
    return CCGLIB_B200_INVALID_ARGUMENT;
  }
  CCGLIB_CUDA_TRY(cudaGetDevice(&plan.device));
  plan.sms = sm_count();
  if (plan.sms <= 0) return CCGLIB_B200_CUDA_ERROR;
  int cc_major = 0;
  CCGLIB_CUDA_TRY(cudaDeviceGetAttribute(&cc_major, cudaDevAttrComputeCapabilityMajor, plan.device));
  if (cc_major != 10) {
    set_last_error("This architecture is not supported (need compute capability 10.x)");
    return CCGLIB_B200_UNSUPPORTED;
  }
  const size_t tiles_256 = d.batch * ceil_div<size_t>(d.m, kBlockM) * ceil_div<size_t>(d.n, 256);
  plan.bn = (plan.k_bytes <= 2048 || tiles_256 < static_cast<size_t>(plan.sms)) ? 128 : 256;
  plan.sw = 128;
  plan.kernel = pick_tile<kKindI8, 3, int>(plan.bn, plan.sw);
  plan.idesc = (2u << 4) | (1u << 7) | (1u << 10) | (static_cast<uint32_t>(plan.bn >> 3) << 17) |
               (static_cast<uint32_t>(kBlockM >> 4) << 24);  // s32 accumulate, signed 8-bit A and B
  plan.idesc_neg_a = plan.idesc;
  CCGLIB_CUDA_TRY(cudaFuncSetAttribute(reinterpret_cast<const void *>(plan.kernel.fn),
                                       cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       plan.kernel.smem));
  void *scratch = nullptr;
  const int rc = static_scratch_address(&scratch);
  if (rc != CCGLIB_B200_OK) return rc;
  size_t chunk = kStaticScratchBytes / (per_item_a + per_item_b);
  if (chunk > d.batch) chunk = d.batch;
  plan.batch_chunk = chunk;
  plan.scratch_bytes = 0;  // nothing owned
  plan.scratch_a = scratch;
  plan.scratch_b = static_cast<char *>(scratch) + chunk * per_item_a;
  // Every byte the multiply reads from the array is rewritten by this call's own expansion pass
  // (rows are written in full, zero padding included), so nothing has to start at zero and
  // whatever an earlier call left behind is never read.
  return ccglib_b200_gemm_run(&plan, d_a, d_b, d_c, stream);
}
