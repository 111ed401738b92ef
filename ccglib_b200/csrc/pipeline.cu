// The Pipeline: from the caller's matrices in their natural layout to C, as one object.
//
//   floating point, opt variant : Transpose(A), Transpose(B) into pipeline-owned tiled buffers,
//                                 then the GEMM on them
//   floating point, basic       : the GEMM on the caller's buffers
//   1-bit (one byte per sample) : the GEMM's own front end turns the bytes into tensor-core
//                                 operands chunk by chunk (staging.cu: expand_bytes_warp_kernel),
//                                 so there is neither a packing nor a tiling pass over memory
//
// with device operands (asynchronous on the caller's stream, no allocation) or host operands
// (batch slices double-buffered over three internal streams, so that the copies in both
// directions overlap the kernels; blocks until C is back in host memory).
//
// Replaces ccglib::pipeline::Pipeline (reference src/pipeline/Pipeline.cpp:44-126 for the chain
// and the scratch ownership, :162-188 for the two Run forms), whose chain is
// Packing -> Transpose -> GEMM as separate passes over HBM.
#include <cstdlib>
#include <new>

#include "common.cuh"

using namespace ccglib_b200;

namespace {
constexpr int kMaxChunks = 8;
}

struct ccglib_b200_pipeline {
  ccglib_b200_pipeline_desc desc;
  ccglib_b200_gemm_plan *gemm;
  bool tiles;               // Transpose A and B into the opt layout before the GEMM
  unsigned m_blk, n_blk, k_c;
  size_t bits;              // bits per input element as the caller stores it (1-bit input: 8)
  size_t item_a, item_b, item_c;  // bytes per batch item of the caller's A, B, C
  size_t tiled_item_a, tiled_item_b;
  void *tiled_a, *tiled_b;  // pipeline-owned scratch of the device path (whole batch)
  int device;
  cudaEvent_t ev_gemm_begin, ev_gemm_end;  // caller-owned, optional: recorded around the GEMM stage
  // device path with tiling: the batch goes in chunks, the transposes of later chunks running on
  // a side stream beside the GEMM of earlier ones
  size_t chunk_items;
  bool overlap_on;  // ccglib_b200_pipeline_set_overlap
  cudaStream_t s_side;
  cudaEvent_t ev_call, ev_tiled[kMaxChunks];
  // host path, created by the first run_host
  size_t slice_items;
  void *slice_a[2], *slice_b[2], *slice_c[2];
  cudaStream_t s_in, s_cmp, s_out;
  cudaEvent_t ev_start, ev_in[2], ev_cmp[2], ev_out[2];
  bool host_ready;
};

namespace {

size_t type_bits_of(int t) {
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

void release(ccglib_b200_pipeline &p) {
  if (p.host_ready) {
    for (cudaStream_t s : {p.s_in, p.s_cmp, p.s_out}) {
      if (s != nullptr) {
        cudaStreamSynchronize(s);
        cudaStreamDestroy(s);
      }
    }
    for (int j = 0; j < 2; ++j) {
      for (cudaEvent_t e : {p.ev_in[j], p.ev_cmp[j], p.ev_out[j]}) {
        if (e != nullptr) cudaEventDestroy(e);
      }
    }
    if (p.ev_start != nullptr) cudaEventDestroy(p.ev_start);
    if (p.slice_a[0] != nullptr) cudaFree(p.slice_a[0]);
    p.host_ready = false;
  }
  if (p.s_side != nullptr) {
    cudaStreamSynchronize(p.s_side);
    cudaStreamDestroy(p.s_side);
    p.s_side = nullptr;
  }
  if (p.ev_call != nullptr) cudaEventDestroy(p.ev_call);
  p.ev_call = nullptr;
  for (cudaEvent_t &e : p.ev_tiled) {
    if (e != nullptr) cudaEventDestroy(e);
    e = nullptr;
  }
  if (p.tiled_a != nullptr) cudaFree(p.tiled_a);
  p.tiled_a = p.tiled_b = nullptr;
  if (p.gemm != nullptr) ccglib_b200_gemm_plan_destroy(p.gemm);
  p.gemm = nullptr;
}

// The chain on `items` batch items of device operands.  Everything is ordered after what
// `stream` holds at the call and before what is enqueued on it afterwards.  With tiling and a
// batch of several chunks the transposes run on the pipeline's side stream, chunk by chunk, and
// the GEMM of a chunk waits only for its own operands: the transposes (bound by HBM bandwidth)
// of later chunks then run beside the GEMM (bound by the tensor cores and the power cap) of
// earlier ones instead of in front of it.
int run_items(ccglib_b200_pipeline &p, const void *d_a, const void *d_b, void *d_c, size_t items,
              cudaStream_t stream) {
  const ccglib_b200_pipeline_desc &d = p.desc;
  if (!p.tiles) {
    if (p.ev_gemm_begin != nullptr) CCGLIB_CUDA_TRY(cudaEventRecord(p.ev_gemm_begin, stream));
    const int rc = run_gemm_items(p.gemm, d_a, d_b, d_c, items, stream);
    if (p.ev_gemm_end != nullptr) CCGLIB_CUDA_TRY(cudaEventRecord(p.ev_gemm_end, stream));
    return rc;
  }
  const size_t chunk =
      (p.s_side != nullptr && p.overlap_on && p.chunk_items < items) ? p.chunk_items : items;
  const bool overlap = chunk < items;
  cudaStream_t s_t = overlap ? p.s_side : stream;
  if (overlap) {
    // the side stream starts after everything the caller enqueued so far, which includes the
    // GEMMs of an earlier call that may still be reading the tiled buffers
    CCGLIB_CUDA_TRY(cudaEventRecord(p.ev_call, stream));
    CCGLIB_CUDA_TRY(cudaStreamWaitEvent(s_t, p.ev_call, 0));
  }
  int rc = CCGLIB_B200_OK;
  size_t ci = 0;
  for (size_t b0 = 0; b0 < items && rc == CCGLIB_B200_OK; b0 += chunk, ++ci) {
    const size_t nb = items - b0 < chunk ? items - b0 : chunk;
    char *ta = static_cast<char *>(p.tiled_a) + b0 * p.tiled_item_a;
    char *tb = static_cast<char *>(p.tiled_b) + b0 * p.tiled_item_b;
    rc = ccglib_b200_transpose_run(nb, d.m, d.k, p.m_blk, p.k_c, p.bits, d.input_complex_axis,
                                   static_cast<const char *>(d_a) + b0 * p.item_a, ta, s_t);
    if (rc != CCGLIB_B200_OK) break;
    rc = ccglib_b200_transpose_run(nb, d.n, d.k, p.n_blk, p.k_c, p.bits, d.input_complex_axis,
                                   static_cast<const char *>(d_b) + b0 * p.item_b, tb, s_t);
    if (rc != CCGLIB_B200_OK) break;
    if (overlap) {
      CCGLIB_CUDA_TRY(cudaEventRecord(p.ev_tiled[ci], s_t));
      CCGLIB_CUDA_TRY(cudaStreamWaitEvent(stream, p.ev_tiled[ci], 0));
    }
    if (ci == 0 && p.ev_gemm_begin != nullptr) {
      CCGLIB_CUDA_TRY(cudaEventRecord(p.ev_gemm_begin, stream));
    }
    rc = run_gemm_items(p.gemm, ta, tb, static_cast<char *>(d_c) + b0 * p.item_c, nb, stream);
  }
  if (overlap) {
    // after a failed launch the caller's stream must still come after the side stream
    CCGLIB_CUDA_TRY(cudaEventRecord(p.ev_call, s_t));
    CCGLIB_CUDA_TRY(cudaStreamWaitEvent(stream, p.ev_call, 0));
  }
  if (p.ev_gemm_end != nullptr) CCGLIB_CUDA_TRY(cudaEventRecord(p.ev_gemm_end, stream));
  return rc;
}

int prepare_host_path(ccglib_b200_pipeline &p) {
  if (p.host_ready) return CCGLIB_B200_OK;
  const size_t s = p.slice_items;
  const size_t bytes_a = s * p.item_a, bytes_b = s * p.item_b, bytes_c = s * p.item_c;
  auto up = [](size_t n) { return (n + 255) & ~size_t{255}; };
  const size_t per_buf = up(bytes_a) + up(bytes_b) + up(bytes_c);
  void *base = nullptr;
  if (cudaMalloc(&base, 2 * per_buf) != cudaSuccess) {
    cudaGetLastError();
    set_last_error("pipeline_run_host: could not allocate %zu bytes for the device slices",
                   2 * per_buf);
    return CCGLIB_B200_OUT_OF_MEMORY;
  }
  for (int j = 0; j < 2; ++j) {
    char *q = static_cast<char *>(base) + j * per_buf;
    p.slice_a[j] = q;
    p.slice_b[j] = q + up(bytes_a);
    p.slice_c[j] = q + up(bytes_a) + up(bytes_b);
  }
  p.host_ready = true;  // from here on release() cleans up whatever exists
  cudaError_t err = cudaEventCreateWithFlags(&p.ev_start, cudaEventDisableTiming);
  for (cudaStream_t *s_ptr : {&p.s_in, &p.s_cmp, &p.s_out}) {
    if (err == cudaSuccess) err = cudaStreamCreateWithFlags(s_ptr, cudaStreamNonBlocking);
  }
  for (int j = 0; j < 2; ++j) {
    for (cudaEvent_t *e : {&p.ev_in[j], &p.ev_cmp[j], &p.ev_out[j]}) {
      if (err == cudaSuccess) err = cudaEventCreateWithFlags(e, cudaEventDisableTiming);
    }
  }
  if (err != cudaSuccess) return cuda_fail(err, "creating the streams of the host path");
  return CCGLIB_B200_OK;
}

} // namespace

extern "C" int ccglib_b200_pipeline_create(const ccglib_b200_pipeline_desc *desc,
                                           ccglib_b200_pipeline **out) {
  if (desc == nullptr || out == nullptr) {
    set_last_error("pipeline_create: null argument");
    return CCGLIB_B200_INVALID_ARGUMENT;
  }
  *out = nullptr;
  const ccglib_b200_pipeline_desc &d = *desc;
  const size_t in_bits = type_bits_of(d.type_in), out_bits = type_bits_of(d.type_out);
  if (in_bits == 0 || out_bits == 0 || d.type_in == CCGLIB_B200_INT32) {
    set_last_error("pipeline_create: unsupported value types (%d -> %d)", d.type_in, d.type_out);
    return CCGLIB_B200_UNSUPPORTED;
  }
  if ((d.input_complex_axis != CCGLIB_B200_PLANAR &&
       d.input_complex_axis != CCGLIB_B200_INTERLEAVED) ||
      (d.output_complex_axis != CCGLIB_B200_PLANAR &&
       d.output_complex_axis != CCGLIB_B200_INTERLEAVED)) {
    set_last_error("pipeline_create: unknown complex axis location");
    return CCGLIB_B200_INVALID_ARGUMENT;
  }
  const bool one_bit = d.type_in == CCGLIB_B200_INT1;
  if (!one_bit && d.variant == CCGLIB_B200_BASIC &&
      d.input_complex_axis == CCGLIB_B200_INTERLEAVED) {
    set_last_error("complex-interleaved input needs the opt variant (its transpose pass "
                   "de-interleaves)");
    return CCGLIB_B200_UNSUPPORTED;
  }

  ccglib_b200_pipeline p{};
  p.desc = d;
  p.overlap_on = true;
  CCGLIB_CUDA_TRY(cudaGetDevice(&p.device));
  ccglib_b200_gemm_desc g{};
  g.batch = d.batch;
  g.m = d.m;
  g.n = d.n;
  g.k = d.k;
  g.type_in = d.type_in;
  g.type_out = d.type_out;
  // one-byte samples are re-staged by the GEMM whatever the variant; nothing is tiled first
  g.variant = one_bit ? CCGLIB_B200_BASIC : d.variant;
  g.c_complex_axis = d.output_complex_axis;
  g.a_mem_order = d.a_mem_order;
  g.b_mem_order = d.b_mem_order;
  g.c_mem_order = d.c_mem_order;
  g.alpha_re = d.alpha_re;
  g.alpha_im = d.alpha_im;
  g.beta_re = d.beta_re;
  g.beta_im = d.beta_im;
  PlanOptions opt;
  opt.int1_bytes_in = one_bit;
  opt.int1_bytes_interleaved = one_bit && d.input_complex_axis == CCGLIB_B200_INTERLEAVED;
  int rc = create_gemm_plan(&g, opt, &p.gemm);
  if (rc != CCGLIB_B200_OK) return rc;

  p.bits = one_bit ? 8 : in_bits;
  p.item_a = 2 * d.m * d.k * p.bits / 8;
  p.item_b = 2 * d.n * d.k * p.bits / 8;
  p.item_c = 2 * d.m * d.n * out_bits / 8;
  p.tiles = !one_bit && d.variant == CCGLIB_B200_OPT;
  if (p.tiles) {
    unsigned dims[3];
    rc = ccglib_b200_gemm_dims(d.type_in, d.type_out, d.variant, dims);
    if (rc != CCGLIB_B200_OK) {
      release(p);
      return rc;
    }
    p.m_blk = dims[0];
    p.n_blk = dims[1];
    p.k_c = dims[2];
    const size_t kt = ceil_div<size_t>(d.k, p.k_c) * p.k_c;
    p.tiled_item_a = 2 * ceil_div<size_t>(d.m, p.m_blk) * p.m_blk * kt * in_bits / 8;
    p.tiled_item_b = 2 * ceil_div<size_t>(d.n, p.n_blk) * p.n_blk * kt * in_bits / 8;
    const size_t bytes_a = (d.batch * p.tiled_item_a + 255) & ~size_t{255};
    if (cudaMalloc(&p.tiled_a, bytes_a + d.batch * p.tiled_item_b) != cudaSuccess) {
      cudaGetLastError();
      set_last_error("pipeline_create: could not allocate %zu bytes for the tiled operands",
                     bytes_a + d.batch * p.tiled_item_b);
      release(p);
      return CCGLIB_B200_OUT_OF_MEMORY;
    }
    p.tiled_b = static_cast<char *>(p.tiled_a) + bytes_a;
    // chunks of at least 2e13 operations (some ten milliseconds of GEMM), at most kMaxChunks
    const double ops_item = 8.0 * static_cast<double>(d.m) * d.n * d.k;
    size_t chunk = static_cast<size_t>(2e13 / ops_item) + 1;
    const char *forced = std::getenv("CCGLIB_B200_PIPE_CHUNK");  // items per chunk (experiments)
    if (forced != nullptr && std::atoi(forced) > 0) chunk = static_cast<size_t>(std::atoi(forced));
    if (chunk < ceil_div<size_t>(d.batch, kMaxChunks)) chunk = ceil_div<size_t>(d.batch, kMaxChunks);
    p.chunk_items = chunk;
    const char *env = std::getenv("CCGLIB_B200_PIPE_OVERLAP");
    const bool want = env == nullptr || *env == '\0' || std::atoi(env) != 0;
    if (want && chunk < d.batch) {
      cudaError_t err = cudaStreamCreateWithFlags(&p.s_side, cudaStreamNonBlocking);
      if (err == cudaSuccess) err = cudaEventCreateWithFlags(&p.ev_call, cudaEventDisableTiming);
      for (cudaEvent_t &e : p.ev_tiled) {
        if (err == cudaSuccess) err = cudaEventCreateWithFlags(&e, cudaEventDisableTiming);
      }
      if (err != cudaSuccess) {
        release(p);
        return cuda_fail(err, "creating the side stream of the pipeline");
      }
    }
  }
  // host path: slices of about 1 GiB of the larger of input and output, at least one item
  const size_t per_item = (p.item_a + p.item_b > p.item_c) ? p.item_a + p.item_b : p.item_c;
  size_t slice = (size_t{1} << 30) / (per_item ? per_item : 1);
  if (slice < 1) slice = 1;
  if (slice > d.batch) slice = d.batch;
  p.slice_items = ceil_div(d.batch, ceil_div(d.batch, slice));  // equal slices

  *out = new (std::nothrow) ccglib_b200_pipeline(p);
  if (*out == nullptr) {
    release(p);
    return CCGLIB_B200_OUT_OF_MEMORY;
  }
  return CCGLIB_B200_OK;
}

extern "C" int ccglib_b200_pipeline_destroy(ccglib_b200_pipeline *p) {
  if (p == nullptr) return CCGLIB_B200_OK;
  release(*p);
  delete p;
  return CCGLIB_B200_OK;
}

extern "C" int ccglib_b200_pipeline_run(ccglib_b200_pipeline *p, const void *d_a, const void *d_b,
                                        void *d_c, void *stream) {
  if (p == nullptr || d_a == nullptr || d_b == nullptr || d_c == nullptr) {
    set_last_error("pipeline_run: null argument");
    return CCGLIB_B200_INVALID_ARGUMENT;
  }
  return run_items(*p, d_a, d_b, d_c, p->desc.batch, static_cast<cudaStream_t>(stream));
}

extern "C" int ccglib_b200_pipeline_set_gemm_events(ccglib_b200_pipeline *p, void *begin,
                                                    void *end) {
  if (p == nullptr || (begin == nullptr) != (end == nullptr)) {
    set_last_error("pipeline_set_gemm_events: give both events or neither");
    return CCGLIB_B200_INVALID_ARGUMENT;
  }
  p->ev_gemm_begin = static_cast<cudaEvent_t>(begin);
  p->ev_gemm_end = static_cast<cudaEvent_t>(end);
  return CCGLIB_B200_OK;
}

extern "C" int ccglib_b200_pipeline_set_overlap(ccglib_b200_pipeline *p, int on) {
  if (p == nullptr) {
    set_last_error("pipeline_set_overlap: null argument");
    return CCGLIB_B200_INVALID_ARGUMENT;
  }
  p->overlap_on = on != 0;
  return CCGLIB_B200_OK;
}

extern "C" size_t ccglib_b200_pipeline_launches(const ccglib_b200_pipeline *p) {
  if (p == nullptr) return 0;
  if (!p->tiles) return ccglib_b200_gemm_plan_launches(p->gemm);
  const size_t chunks =
      (p->s_side != nullptr && p->overlap_on) ? ceil_div(p->desc.batch, p->chunk_items) : 1;
  return chunks * (2 + ccglib_b200_gemm_plan_launches(p->gemm));
}

extern "C" size_t ccglib_b200_pipeline_scratch_bytes(const ccglib_b200_pipeline *p) {
  if (p == nullptr) return 0;
  size_t n = ccglib_b200_gemm_plan_scratch_bytes(p->gemm);
  if (p->tiles) n += p->desc.batch * (p->tiled_item_a + p->tiled_item_b);
  if (p->host_ready) n += 2 * p->slice_items * (p->item_a + p->item_b + p->item_c);
  return n;
}

extern "C" int ccglib_b200_pipeline_set_host_slice(ccglib_b200_pipeline *p, size_t items) {
  if (p == nullptr || items == 0 || items > p->desc.batch) {
    set_last_error("pipeline_set_host_slice: the slice must hold 1..batch items");
    return CCGLIB_B200_INVALID_ARGUMENT;
  }
  if (p->host_ready) {
    set_last_error("pipeline_set_host_slice: the device slices already exist");
    return CCGLIB_B200_INVALID_ARGUMENT;
  }
  p->slice_items = items;
  return CCGLIB_B200_OK;
}

extern "C" size_t ccglib_b200_pipeline_host_slice(const ccglib_b200_pipeline *p) {
  return p != nullptr ? p->slice_items : 0;
}

extern "C" int ccglib_b200_pipeline_run_host(ccglib_b200_pipeline *p, const void *h_a,
                                             const void *h_b, void *h_c, void *stream_v) {
  if (p == nullptr || h_a == nullptr || h_b == nullptr || h_c == nullptr) {
    set_last_error("pipeline_run_host: null argument");
    return CCGLIB_B200_INVALID_ARGUMENT;
  }
  int rc = prepare_host_path(*p);
  if (rc != CCGLIB_B200_OK) return rc;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
  const ccglib_b200_pipeline_desc &d = p->desc;
  const bool copy_c_in = d.beta_re != 0.0f || d.beta_im != 0.0f;
  // everything the caller enqueued on its stream before this call comes first
  CCGLIB_CUDA_TRY(cudaEventRecord(p->ev_start, stream));
  for (cudaStream_t s : {p->s_in, p->s_cmp, p->s_out}) {
    CCGLIB_CUDA_TRY(cudaStreamWaitEvent(s, p->ev_start, 0));
  }
  const char *a = static_cast<const char *>(h_a), *b = static_cast<const char *>(h_b);
  char *c = static_cast<char *>(h_c);
  size_t i = 0;
  for (size_t b0 = 0; b0 < d.batch; b0 += p->slice_items, ++i) {
    const size_t nb = d.batch - b0 < p->slice_items ? d.batch - b0 : p->slice_items;
    const int j = static_cast<int>(i & 1);
    // copy in: the buffers are free once the GEMM two slices back has read A and B (and, when C
    // is an input too, once its copy-out has left the C buffer)
    if (i >= 2) {
      CCGLIB_CUDA_TRY(cudaStreamWaitEvent(p->s_in, p->ev_cmp[j], 0));
      if (copy_c_in) CCGLIB_CUDA_TRY(cudaStreamWaitEvent(p->s_in, p->ev_out[j], 0));
    }
    CCGLIB_CUDA_TRY(cudaMemcpyAsync(p->slice_a[j], a + b0 * p->item_a, nb * p->item_a,
                                    cudaMemcpyHostToDevice, p->s_in));
    CCGLIB_CUDA_TRY(cudaMemcpyAsync(p->slice_b[j], b + b0 * p->item_b, nb * p->item_b,
                                    cudaMemcpyHostToDevice, p->s_in));
    if (copy_c_in) {
      CCGLIB_CUDA_TRY(cudaMemcpyAsync(p->slice_c[j], c + b0 * p->item_c, nb * p->item_c,
                                      cudaMemcpyHostToDevice, p->s_in));
    }
    CCGLIB_CUDA_TRY(cudaEventRecord(p->ev_in[j], p->s_in));
    // compute: after this slice's copy-in, and after the copy-out that last used the C buffer
    CCGLIB_CUDA_TRY(cudaStreamWaitEvent(p->s_cmp, p->ev_in[j], 0));
    if (i >= 2) CCGLIB_CUDA_TRY(cudaStreamWaitEvent(p->s_cmp, p->ev_out[j], 0));
    rc = run_items(*p, p->slice_a[j], p->slice_b[j], p->slice_c[j], nb, p->s_cmp);
    if (rc != CCGLIB_B200_OK) break;
    CCGLIB_CUDA_TRY(cudaEventRecord(p->ev_cmp[j], p->s_cmp));
    // copy out
    CCGLIB_CUDA_TRY(cudaStreamWaitEvent(p->s_out, p->ev_cmp[j], 0));
    CCGLIB_CUDA_TRY(cudaMemcpyAsync(c + b0 * p->item_c, p->slice_c[j], nb * p->item_c,
                                    cudaMemcpyDeviceToHost, p->s_out));
    CCGLIB_CUDA_TRY(cudaEventRecord(p->ev_out[j], p->s_out));
  }
  // as the reference's host-memory Run: return when C is complete in host memory
  for (cudaStream_t s : {p->s_in, p->s_cmp, p->s_out}) {
    const cudaError_t err = cudaStreamSynchronize(s);
    if (err != cudaSuccess && rc == CCGLIB_B200_OK) rc = cuda_fail(err, "cudaStreamSynchronize");
  }
  return rc;
}
