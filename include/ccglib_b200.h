/*
 * ccglib_b200 -- C ABI of the B200 (sm_100a) complex-GEMM hot path.
 *
 * This is the boundary between host code (C++ classes mirroring the reference's
 * ccglib::mma::GEMM, ccglib::transpose::Transpose, ccglib::packing::Packing and
 * ccglib::pipeline::Pipeline, or any FFI) and the ahead-of-time compiled CUDA
 * kernels.  Plain pointers, sizes and ints only; no C++ or framework types.
 *
 * Every function returns a ccglib_b200_status (0 = success).  Device pointers
 * are passed as void* (the numeric value of a CUdeviceptr); streams as void*
 * (the value of a CUstream / cudaStream_t; NULL = default stream).  A CUDA
 * context must be current on the calling thread.  Functions that launch work
 * are asynchronous on the given stream and never synchronise; only the plan
 * constructor may allocate device memory.
 *
 * Integer codes of value types, variants, memory orders, complex-axis locations
 * and directions are the enumerator values of the reference's public enums
 * (include/ccglib/common/value_type.h:14-22, gemm/variant.h:6,
 * gemm/mem_order.h:6, common/complex_order.h:12, common/direction.h:6).
 */
#ifndef CCGLIB_B200_H_
#define CCGLIB_B200_H_

#include <stddef.h>

#if defined(__GNUC__)
#define CCGLIB_B200_API __attribute__((visibility("default")))
#else
#define CCGLIB_B200_API
#endif

#ifdef __cplusplus
extern "C" {
#endif

typedef enum ccglib_b200_status {
  CCGLIB_B200_OK = 0,
  CCGLIB_B200_INVALID_ARGUMENT = 1, /* bad size, pointer, alignment or enum value */
  CCGLIB_B200_UNSUPPORTED = 2,      /* combination the library has no kernel for */
  CCGLIB_B200_CUDA_ERROR = 3,       /* a CUDA runtime/driver call failed */
  CCGLIB_B200_DEVICE_TIMEOUT = 4,   /* a bounded device-side wait gave up */
  CCGLIB_B200_OUT_OF_MEMORY = 5     /* scratch allocation failed at plan creation */
} ccglib_b200_status;

enum { /* ccglib::ValueType */
  CCGLIB_B200_INT1 = 0,
  CCGLIB_B200_INT32 = 1,
  CCGLIB_B200_BFLOAT16 = 2,
  CCGLIB_B200_FLOAT8E4M3 = 3,
  CCGLIB_B200_FLOAT8E5M2 = 4,
  CCGLIB_B200_FLOAT16 = 5,
  CCGLIB_B200_FLOAT32 = 6
};
enum { CCGLIB_B200_BASIC = 0, CCGLIB_B200_OPT = 1 };                /* ccglib::mma::Variant */
enum { CCGLIB_B200_ROW_MAJOR = 0, CCGLIB_B200_COL_MAJOR = 1 };      /* ccglib::mma::MemOrder */
enum { CCGLIB_B200_PLANAR = 0, CCGLIB_B200_INTERLEAVED = 1 };       /* ccglib::ComplexAxisLocation */
enum { CCGLIB_B200_FORWARD = 0, CCGLIB_B200_BACKWARD = 1 };         /* ccglib::Direction */

/*
 * Problem description of one batched complex GEMM  C[b] = alpha * A[b] x B[b]^T + beta * C[b].
 * Replaces the constructor arguments of ccglib::mma::GEMM
 * (reference include/ccglib/gemm/mma.h:29-37, src/mma/GEMM.cpp:56-97), which the
 * reference turns into NVRTC -D macros (src/mma/GEMM.cpp:133-214).
 *
 * Layouts (reference kernels/type_selector.h:224-241, kernels/gemm_kernel_float.cu:28-33):
 *   basic A: [batch][2][M][K]   basic B: [batch][2][N][K]   (K contiguous; 1-bit: K/32 words)
 *   opt   A: [batch][ceil(M/m_blk)][ceil(K/k_c)][2][m_blk][k_c], opt B likewise with n_blk,
 *            zero padded, with (m_blk, n_blk, k_c) from ccglib_b200_gemm_dims
 *   C planar:      [batch][2][M][N] (row-major) or [batch][2][N][M] (col-major)
 *   C interleaved: [batch][M][N][2] (row-major) or [batch][N][M][2] (col-major)
 */
typedef struct ccglib_b200_gemm_desc {
  size_t batch;
  size_t m;
  size_t n;
  size_t k;           /* samples (bits for 1-bit input) */
  int type_in;        /* value type of A and B */
  int type_out;       /* value type of C */
  int variant;        /* CCGLIB_B200_BASIC / CCGLIB_B200_OPT */
  int c_complex_axis; /* CCGLIB_B200_PLANAR / CCGLIB_B200_INTERLEAVED */
  int a_mem_order;    /* must be row-major */
  int b_mem_order;    /* must be col-major */
  int c_mem_order;
  float alpha_re, alpha_im;
  float beta_re, beta_im;
} ccglib_b200_gemm_desc;

typedef struct ccglib_b200_gemm_plan ccglib_b200_gemm_plan;

/* Tile contract of the opt layout: dims = {m_blk, n_blk, k_c}.  Replaces
 * ccglib::mma::GEMM::GetDimensions (reference src/mma/GEMM.cpp:270-275). */
CCGLIB_B200_API int ccglib_b200_gemm_dims(int type_in, int type_out, int variant, unsigned dims[3]);

/* Validate the description, choose the kernel and (only where the input needs re-staging:
 * 1-bit input, or rows whose byte pitch is not a multiple of 16) allocate scratch.
 * Replaces GEMM::Impl::Impl + compile_kernel (reference src/mma/GEMM.cpp:56-97,133-229).
 * Errors the reference raises as exceptions come back as status codes: basic variant with
 * interleaved C -> UNSUPPORTED (:77-80); col-major A or row-major B -> UNSUPPORTED (the
 * reference fails in NVRTC, kernels/gemm_kernel_float.cu:20-25). */
CCGLIB_B200_API int ccglib_b200_gemm_plan_create(const ccglib_b200_gemm_desc *desc, ccglib_b200_gemm_plan **plan);

/* Enqueue the GEMM.  Replaces ccglib::mma::GEMM::Run(CUdeviceptr a, b, c)
 * (reference src/mma/GEMM.cpp:99-108,263-268).  Never allocates and never synchronises the
 * host.  All work is ordered after what `stream` holds at the call and before anything
 * enqueued on it afterwards; a staged plan with several batch chunks forks two internal streams
 * off `stream` for the chunks and joins them back before returning.  One plan must not run on
 * two streams at the same time (its scratch and tensor-map cache are per plan). */
CCGLIB_B200_API int ccglib_b200_gemm_run(ccglib_b200_gemm_plan *plan, const void *d_a, const void *d_b, void *d_c,
                         void *stream);

CCGLIB_B200_API int ccglib_b200_gemm_plan_destroy(ccglib_b200_gemm_plan *plan);

/* Bytes of device scratch the plan owns (0 for the direct TMA path). */
CCGLIB_B200_API size_t ccglib_b200_gemm_plan_scratch_bytes(const ccglib_b200_gemm_plan *plan);

/* Tile choice of the plan: tile = {columns per tile, 1 if a CTA pair works on a 256-row tile,
 * column-panel width of the tile walk from a tuning table (0: built-in rule), 1 if the choice
 * came from a tuning table, CTAs that share the K of one tile (split-K; 1 = none)}.
 * Introspection; no counterpart in the reference. */
CCGLIB_B200_API int ccglib_b200_gemm_plan_tile(const ccglib_b200_gemm_plan *plan, int tile[5]);

/* Look a problem up in a tuning table file (JSON written by `python -m ccglib_b200.tune
 * --write FILE`; plans consult the file named by the environment variable
 * CCGLIB_B200_TUNE_TABLE in the same way).  choice = {columns per tile, pair (0/1, -1 = model),
 * column-panel width (0 = built-in rule)}; UNSUPPORTED when no entry matches (types, M, N,
 * log2 bucket of the bytes per input row, log2 bucket of the batch).  Host only.  Takes the
 * place of the result files of the reference's tuner (tuning/tune_gemm.py:316-363). */
CCGLIB_B200_API int ccglib_b200_tune_table_lookup(const char *path,
                                                  const ccglib_b200_gemm_desc *desc,
                                                  int choice[3]);

/* Kernel launches one ccglib_b200_gemm_run of this plan enqueues: 1 on the direct TMA path,
 * 3 per batch chunk (re-stage A, re-stage B, multiply) on the staged paths.  Introspection for
 * benchmarks; no counterpart in the reference. */
CCGLIB_B200_API size_t ccglib_b200_gemm_plan_launches(const ccglib_b200_gemm_plan *plan);

/*
 * Tile transpose: [batch][2][M][N] (planar) or [batch][M][N][2] (interleaved) ->
 * [batch][ceil(M/m_chunk)][ceil(N/n_chunk)][2][m_chunk][n_chunk], zero padded.  Elements are
 * moved by width only: nr_bits in {8, 16, 32}, or 1 for 32-sample words (N and n_chunk then
 * count samples and must be multiples of 32).  Replaces ccglib::transpose::Transpose::Run
 * (reference src/transpose/Transpose.cpp:58-73, kernels/transpose_kernel.cu:50-82).
 */
CCGLIB_B200_API int ccglib_b200_transpose_run(size_t batch, size_t m, size_t n, size_t m_chunk, size_t n_chunk,
                              size_t nr_bits, int input_complex_axis, const void *d_in,
                              void *d_out, void *stream);

/*
 * Bit packing.  FORWARD: n one-byte samples -> ceil(n/32) words, sample i in bit i%32 of word
 * i/32, set when the byte is non-zero; with interleaved input the buffer [n/2][2] is written
 * as [2][n/2].  BACKWARD: words -> n bytes of 0/1 (planar only; interleaved -> UNSUPPORTED).
 * Replaces ccglib::packing::Packing::Run (reference src/packing/Packing.cpp:44-74,
 * kernels/packing_kernel.cu:7-62).
 */
CCGLIB_B200_API int ccglib_b200_pack_run(size_t n, int direction, int input_complex_axis, const void *d_in,
                         void *d_out, void *stream);

/*
 * The Pipeline: the caller's matrices in their natural layout -> C, as one object that owns the
 * intermediate buffers.  Replaces ccglib::pipeline::Pipeline (reference
 * include/ccglib/pipeline/pipeline.h:28-73, src/pipeline/Pipeline.cpp:44-188), whose chain is
 * Packing (1-bit input) -> Transpose (opt variant) -> GEMM as separate launches.
 *
 * Input A: [batch][2][M][K] (planar) or [batch][M][K][2] (interleaved) elements of type_in, B
 * likewise with N rows; 1-bit input is given as ONE BYTE PER SAMPLE (non-zero = +1, zero = -1),
 * as the reference's Pipeline takes it (src/pipeline/Pipeline.cpp:58-72).  C as for the GEMM.
 *   - floating point, opt variant: Transpose A, Transpose B (which also de-interleaves), GEMM.
 *   - floating point, basic variant: GEMM on the caller's buffers (planar input only).
 *   - 1-bit: the byte samples are turned into tensor-core operands by the GEMM's own front end,
 *     chunk by chunk; no packed or tiled copy of A and B is ever written, whatever the variant,
 *     and interleaved C is available with either variant.  Interleaved 1-bit input is
 *     de-interleaved per batch item (the reference's packing pass treats the whole buffer as one
 *     [n/2][2] array, kernels/packing_kernel.cu:15-22, which is the same thing for batch 1).
 */
typedef struct ccglib_b200_pipeline_desc {
  size_t batch;
  size_t m;
  size_t n;
  size_t k;
  int type_in;
  int type_out;
  int variant;
  int input_complex_axis;
  int output_complex_axis;
  int a_mem_order; /* must be row-major */
  int b_mem_order; /* must be col-major */
  int c_mem_order;
  float alpha_re, alpha_im;
  float beta_re, beta_im;
} ccglib_b200_pipeline_desc;

typedef struct ccglib_b200_pipeline ccglib_b200_pipeline;

/* A pipeline owns its scratch and internal streams: like the reference's objects it is not
 * thread-safe and must not run on two streams at the same time.
 *
 * Validates, creates the GEMM plan and allocates the tiled buffers of the device path.
 * Replaces Pipeline::Impl::Impl (reference src/pipeline/Pipeline.cpp:44-106). */
CCGLIB_B200_API int ccglib_b200_pipeline_create(const ccglib_b200_pipeline_desc *desc,
                                                ccglib_b200_pipeline **pipeline);

/* Device operands: enqueues the chain on `stream`; no allocation, no synchronisation.
 * Replaces Pipeline::Run(CUdeviceptr a, b, c) (reference src/pipeline/Pipeline.cpp:108-126,178-188). */
CCGLIB_B200_API int ccglib_b200_pipeline_run(ccglib_b200_pipeline *pipeline, const void *d_a,
                                             const void *d_b, void *d_c, void *stream);

/* Host operands (whole A, B, C in host memory; pinned memory lets the copies overlap the
 * kernels, pageable memory works but serialises).  The batch is cut into slices; each slice is
 * copied in, run through the chain and copied back on three internal streams with two sets of
 * device slice buffers, so host->device, kernels and device->host of neighbouring slices
 * overlap.  Ordered after what `stream` holds at the call; returns when C is complete in host
 * memory.  With beta != 0 the caller's C is copied in first.  The first call allocates the
 * device slices (kept until destroy).  Replaces Pipeline::Run(cu::HostMemory& a, b, c)
 * (reference src/pipeline/Pipeline.cpp:162-176: whole-buffer copies, run, copy back,
 * synchronise). */
CCGLIB_B200_API int ccglib_b200_pipeline_run_host(ccglib_b200_pipeline *pipeline, const void *h_a,
                                                  const void *h_b, void *h_c, void *stream);

/* Batch items per slice of the host path: read, or set before the first run_host (default: about
 * 1 GiB of operands per slice).  No counterpart in the reference. */
CCGLIB_B200_API size_t ccglib_b200_pipeline_host_slice(const ccglib_b200_pipeline *pipeline);
CCGLIB_B200_API int ccglib_b200_pipeline_set_host_slice(ccglib_b200_pipeline *pipeline, size_t items);

/* With the opt variant and a batch of several chunks (chunks of at least 2e13 operations, at most
 * eight), ccglib_b200_pipeline_run puts the transposes on an internal side stream, chunk by chunk,
 * so that those of later chunks run beside the GEMM of earlier ones; the caller still sees one
 * in-order stream.  on = 0 keeps the plain chain (all transposes, then one GEMM) on the caller's
 * stream; the environment variable CCGLIB_B200_PIPE_OVERLAP=0 does the same at creation.
 * No counterpart in the reference. */
CCGLIB_B200_API int ccglib_b200_pipeline_set_overlap(ccglib_b200_pipeline *pipeline, int on);

/* Benchmark hook: two caller-owned CUDA events (CUevent / cudaEvent_t values) that every
 * later run records on the run's stream just before and just after the GEMM stage of the chain
 * (for 1-bit input the stage includes the operand expansion); NULL, NULL switches it off.
 * No counterpart in the reference. */
CCGLIB_B200_API int ccglib_b200_pipeline_set_gemm_events(ccglib_b200_pipeline *pipeline,
                                                         void *begin, void *end);

/* Kernel launches one ccglib_b200_pipeline_run enqueues, and device bytes the pipeline owns.
 * Introspection for benchmarks; no counterpart in the reference. */
CCGLIB_B200_API size_t ccglib_b200_pipeline_launches(const ccglib_b200_pipeline *pipeline);
CCGLIB_B200_API size_t ccglib_b200_pipeline_scratch_bytes(const ccglib_b200_pipeline *pipeline);

CCGLIB_B200_API int ccglib_b200_pipeline_destroy(ccglib_b200_pipeline *pipeline);

/*
 * 1-bit complex GEMM that allocates nothing, for callers that cannot call cudaMalloc: a
 * correlator or beamformer loop whose device memory was handed out in full at start-up (a later
 * allocation would fail), or a host thread that cannot afford the device-wide synchronisation an
 * allocation or free implies while other streams are in the middle of an observation.  It has no
 * counterpart in the reference, whose GEMM needs no scratch.  Same arithmetic, layouts and
 * errors as a plan created from `desc` and run once (type_in must be INT1, type_out INT32), but
 * the scratch for the +-1 byte expansion of A and B is a fixed 32 MiB array inside the library
 * image (each GPU that loads the library holds it until the process exits) instead of a plan
 * allocation.
 *   - Limit: one batch item must fit, (3*M + 2*N) * round_up(K, 16) <= 32 MiB; larger problems
 *     get INVALID_ARGUMENT and should use a plan.  Batches are processed in chunks that fit.
 *   - The first call on each device looks up the array's device address (with that device
 *     current); make that first call before starting any stream capture on that device.  With
 *     CUDA's default lazy module loading the part of the library image that holds the array is
 *     loaded by the first call into the GEMM code, so a process whose very first library call is
 *     this one also pays that module load (and the 32 MiB) there.
 *   - All calls on a device share the one array and it keeps the last call's contents.  Nothing
 *     has to be cleared: each call rewrites every row it later reads, padding included.  Calls
 *     that can overlap on the GPU (different streams, or threads) race on it; serialise them.
 */
CCGLIB_B200_API int ccglib_b200_gemm_int1_static_scratch(const ccglib_b200_gemm_desc *desc,
                                                         const void *d_a, const void *d_b,
                                                         void *d_c, void *stream);

/*
 * Multi-GPU help.  Batch items are independent GEMMs and the batch is the outermost axis of
 * every layout, so a batch is spread over the GPUs of a node by giving each a contiguous slice;
 * nothing is exchanged between devices.  For device `rank` of `world`: the first item and the
 * number of items of its share (as even as possible, the first batch % world ranks take one
 * more), and where that share starts in whole-batch A, B and C arrays laid out as `desc` says
 * (basic or opt layout).  The caller creates one plan per device with batch = count.  Host only.
 * The reference has no multi-GPU support; no counterpart.
 */
typedef struct ccglib_b200_share {
  size_t first, count;
  size_t a_offset, b_offset, c_offset; /* bytes */
  size_t a_bytes, b_bytes, c_bytes;
} ccglib_b200_share;

CCGLIB_B200_API int ccglib_b200_batch_share(const ccglib_b200_gemm_desc *desc, int world,
                                            int rank, ccglib_b200_share *share);

/* Read and clear the sticky device-side status word of the current device (synchronises the
 * device).  Non-zero means a bounded wait inside a kernel gave up; its results are invalid. */
CCGLIB_B200_API int ccglib_b200_device_status(unsigned *word);

/* Self-test of the bounded device-side waits; no counterpart in the reference (its kernels
 * have no waits that can run out).  Launches a tiny kernel on the default stream in which one
 * waiter waits `limit_cycles` (1..1e7 SM clock cycles) on a barrier nobody arrives on, with the
 * same wait routine the GEMM kernels use, and a second waiter (another warp when pair == 0, the
 * other CTA of a two-CTA cluster when pair != 0) has a 200 times longer limit.  The first must
 * give up and set the time-out bit 1 in the device status word; the second must return early
 * through the abort flag without setting its own bit (4).  Nothing faults or hangs: the wait
 * simply runs out.  Synchronises the device; waited_cycles[0], [1] receive the cycles each
 * waiter spent.  The status word is left set: read it with ccglib_b200_device_status. */
CCGLIB_B200_API int ccglib_b200_selftest_wait_timeout(long long limit_cycles, int pair,
                                                      long long waited_cycles[2]);

CCGLIB_B200_API const char *ccglib_b200_status_string(int status);

/* Text of the last error raised on the calling thread ("" if none). */
CCGLIB_B200_API const char *ccglib_b200_last_error(void);

#ifdef __cplusplus
}
#endif
#endif /* CCGLIB_B200_H_ */
