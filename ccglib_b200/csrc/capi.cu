// Status handling and small utilities of the C ABI.
#include <cctype>
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>
#include <vector>

#include "common.cuh"

namespace ccglib_b200 {

namespace {
thread_local char g_last_error[512] = "";
}

void set_last_error(const char *fmt, ...) {
  va_list args;
  va_start(args, fmt);
  vsnprintf(g_last_error, sizeof(g_last_error), fmt, args);
  va_end(args);
}

int sm_count() {
  static int cached[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) {
    set_last_error("cudaGetDevice failed: %s", cudaGetErrorString(cudaGetLastError()));
    return -1;
  }
  if (dev >= 0 && dev < 64 && cached[dev] > 0) return cached[dev];
  int sms = 0;
  if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) {
    set_last_error("cudaDeviceGetAttribute failed: %s", cudaGetErrorString(cudaGetLastError()));
    return -1;
  }
  if (dev >= 0 && dev < 64) cached[dev] = sms;
  return sms;
}

// ---- tuning table ------------------------------------------------------------------------------
//
// A JSON file written by `python -m ccglib_b200.tune --write FILE`:
//   {"format": "ccglib_b200 tuning table 1",
//    "entries": [{"type_in": 5, "type_out": 6, "m": 8192, "n": 8192, "k_bucket": 14,
//                 "batch_bucket": 6, "bn": 256, "pair": 0, "group_n": 4, ...}, ...]}
// Only flat objects with integer members are read; other members (timings, notes) are skipped.
// Replaces the result files of the reference's tuner (tuning/tune_gemm.py:316-363), whose
// winners are hard-wired into its per-type kernel tables (src/mma/Kernel*.cpp).

namespace {

struct TuneEntry {
  long long type_in = -1, type_out = -1, m = -1, n = -1, k_bucket = -1, batch_bucket = -1;
  long long bn = 0, pair = -1, group_n = 0, split_k = 0;
};

unsigned log2_bucket(size_t v) {
  unsigned b = 0;
  while ((size_t{1} << b) < v) ++b;
  return b;
}

// Parse every {...} object that sits inside the "entries" array.
bool parse_table(const std::string &text, std::vector<TuneEntry> &out) {
  const size_t at = text.find("\"entries\"");
  if (at == std::string::npos) return false;
  size_t i = text.find('[', at);
  if (i == std::string::npos) return false;
  for (++i; i < text.size();) {
    while (i < text.size() && text[i] != '{' && text[i] != ']') ++i;
    if (i >= text.size() || text[i] == ']') break;
    const size_t end = text.find('}', i);
    if (end == std::string::npos) return false;
    TuneEntry e;
    size_t j = i + 1;
    while (j < end) {
      const size_t q0 = text.find('"', j);
      if (q0 == std::string::npos || q0 >= end) break;
      const size_t q1 = text.find('"', q0 + 1);
      if (q1 == std::string::npos || q1 >= end) break;
      const std::string key = text.substr(q0 + 1, q1 - q0 - 1);
      size_t v = text.find(':', q1);
      if (v == std::string::npos || v >= end) break;
      ++v;
      while (v < end && std::isspace(static_cast<unsigned char>(text[v]))) ++v;
      if (v < end && text[v] == '"') {  // a string member: skip it
        const size_t q2 = text.find('"', v + 1);
        j = (q2 == std::string::npos || q2 >= end) ? end : q2 + 1;
        continue;
      }
      char *stop = nullptr;
      const long long value = std::strtoll(text.c_str() + v, &stop, 10);
      j = static_cast<size_t>(stop - text.c_str());
      if (j <= v) {  // not a number (true / false / null / nested): skip to the next member
        const size_t comma = text.find(',', v);
        j = (comma == std::string::npos || comma >= end) ? end : comma + 1;
        continue;
      }
      if (key == "type_in") e.type_in = value;
      else if (key == "type_out") e.type_out = value;
      else if (key == "m") e.m = value;
      else if (key == "n") e.n = value;
      else if (key == "k_bucket") e.k_bucket = value;
      else if (key == "batch_bucket") e.batch_bucket = value;
      else if (key == "bn") e.bn = value;
      else if (key == "pair") e.pair = value;
      else if (key == "group_n") e.group_n = value;
      else if (key == "split_k") e.split_k = value;
    }
    out.push_back(e);
    i = end + 1;
  }
  return true;
}

} // namespace

int tune_table_lookup(const char *path, const ccglib_b200_gemm_desc &d, size_t k_bytes,
                      TuneChoice *choice) {
  if (path == nullptr || *path == '\0' || choice == nullptr) return 0;
  std::FILE *f = std::fopen(path, "rb");
  if (f == nullptr) return 0;
  std::string text;
  char buf[4096];
  size_t got;
  while ((got = std::fread(buf, 1, sizeof(buf), f)) > 0) text.append(buf, got);
  std::fclose(f);
  std::vector<TuneEntry> entries;
  if (!parse_table(text, entries)) return 0;
  const long long kb = log2_bucket(k_bytes), bb = log2_bucket(d.batch);
  for (const TuneEntry &e : entries) {
    if (e.type_in == d.type_in && e.type_out == d.type_out &&
        e.m == static_cast<long long>(d.m) && e.n == static_cast<long long>(d.n) &&
        e.k_bucket == kb && e.batch_bucket == bb) {
      choice->bn = static_cast<int>(e.bn);
      choice->pair = static_cast<int>(e.pair);
      choice->group_n = static_cast<int>(e.group_n);
      choice->split_k = static_cast<int>(e.split_k);
      return 1;
    }
  }
  return 0;
}

} // namespace ccglib_b200

using namespace ccglib_b200;

extern "C" int ccglib_b200_tune_table_lookup(const char *path, const ccglib_b200_gemm_desc *desc,
                                             int choice[3]) {
  if (path == nullptr || desc == nullptr || choice == nullptr) {
    set_last_error("tune_table_lookup: null argument");
    return CCGLIB_B200_INVALID_ARGUMENT;
  }
  size_t bits = 0;
  switch (desc->type_in) {
  case CCGLIB_B200_INT1: bits = 1; break;
  case CCGLIB_B200_FLOAT8E4M3:
  case CCGLIB_B200_FLOAT8E5M2: bits = 8; break;
  case CCGLIB_B200_BFLOAT16:
  case CCGLIB_B200_FLOAT16: bits = 16; break;
  case CCGLIB_B200_FLOAT32: bits = 32; break;
  default:
    set_last_error("tune_table_lookup: unsupported input type %d", desc->type_in);
    return CCGLIB_B200_INVALID_ARGUMENT;
  }
  TuneChoice c{};
  choice[0] = choice[1] = choice[2] = 0;
  if (!tune_table_lookup(path, *desc, (desc->k * bits + 7) / 8, &c)) {
    set_last_error("tune_table_lookup: no entry for this problem in %s", path);
    return CCGLIB_B200_UNSUPPORTED;
  }
  choice[0] = c.bn;
  choice[1] = c.pair;
  choice[2] = c.group_n;
  return CCGLIB_B200_OK;
}

extern "C" const char *ccglib_b200_status_string(int status) {
  switch (status) {
  case CCGLIB_B200_OK:
    return "success";
  case CCGLIB_B200_INVALID_ARGUMENT:
    return "invalid argument";
  case CCGLIB_B200_UNSUPPORTED:
    return "unsupported combination";
  case CCGLIB_B200_CUDA_ERROR:
    return "CUDA error";
  case CCGLIB_B200_DEVICE_TIMEOUT:
    return "device-side wait timed out";
  case CCGLIB_B200_OUT_OF_MEMORY:
    return "out of memory";
  default:
    return "unknown status";
  }
}

extern "C" const char *ccglib_b200_last_error(void) { return g_last_error; }

namespace {
size_t value_bits(int t) {
  switch (t) {
  case CCGLIB_B200_INT1: return 1;
  case CCGLIB_B200_FLOAT8E4M3:
  case CCGLIB_B200_FLOAT8E5M2: return 8;
  case CCGLIB_B200_BFLOAT16:
  case CCGLIB_B200_FLOAT16: return 16;
  case CCGLIB_B200_INT32:
  case CCGLIB_B200_FLOAT32: return 32;
  default: return 0;
  }
}
} // namespace

// Batch items are independent GEMMs and the batch is the outermost axis of every layout, so the
// share of one device is a contiguous slice of A, B and C: pure host arithmetic.
extern "C" int ccglib_b200_batch_share(const ccglib_b200_gemm_desc *desc, int world, int rank,
                                       ccglib_b200_share *out) {
  if (desc == nullptr || out == nullptr || world < 1 || rank < 0 || rank >= world) {
    set_last_error("batch_share: need a description, world >= 1 and 0 <= rank < world");
    return CCGLIB_B200_INVALID_ARGUMENT;
  }
  const size_t in_bits = value_bits(desc->type_in), out_bits = value_bits(desc->type_out);
  if (in_bits == 0 || out_bits == 0 || desc->type_in == CCGLIB_B200_INT32) {
    set_last_error("batch_share: unsupported value types (%d -> %d)", desc->type_in,
                   desc->type_out);
    return CCGLIB_B200_INVALID_ARGUMENT;
  }
  const size_t w = static_cast<size_t>(world), r = static_cast<size_t>(rank);
  const size_t base = desc->batch / w, extra = desc->batch % w;
  out->count = base + (r < extra ? 1 : 0);          // the first batch % world ranks take one more
  out->first = r * base + (r < extra ? r : extra);
  size_t a_item, b_item;
  if (desc->variant == CCGLIB_B200_OPT) {
    unsigned dims[3];
    const int rc = ccglib_b200_gemm_dims(desc->type_in, desc->type_out, desc->variant, dims);
    if (rc != CCGLIB_B200_OK) return rc;
    const size_t kp = ceil_div<size_t>(desc->k, dims[2]) * dims[2];
    a_item = 2 * ceil_div<size_t>(desc->m, dims[0]) * dims[0] * kp * in_bits / 8;
    b_item = 2 * ceil_div<size_t>(desc->n, dims[1]) * dims[1] * kp * in_bits / 8;
  } else {
    const size_t row = in_bits == 1 ? ceil_div<size_t>(desc->k, 32) * 4 : desc->k * in_bits / 8;
    a_item = 2 * desc->m * row;
    b_item = 2 * desc->n * row;
  }
  const size_t c_item = 2 * desc->m * desc->n * out_bits / 8;
  out->a_offset = out->first * a_item;
  out->b_offset = out->first * b_item;
  out->c_offset = out->first * c_item;
  out->a_bytes = out->count * a_item;
  out->b_bytes = out->count * b_item;
  out->c_bytes = out->count * c_item;
  return CCGLIB_B200_OK;
}
