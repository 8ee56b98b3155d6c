// rdna4::kv_* -- the reference's KV-cache launch API (its include/rdna4/kv.h) as thin
// C++17 inline wrappers over the C ABI in rd_attn.h, so that a caller written against
// the reference (graph.cuh-style code, the check/bench programs) compiles unchanged:
// same names, same argument order, `bool` results, a trailing stream that defaults to
// the default stream. cudaStream_t takes the place of hipStream_t.
#pragma once
#include <cuda_runtime.h>

#include <cstdint>
#include <cstdio>
#include <cstdlib>

#include "../rd_attn.h"

namespace rdna4 {

// Values and order of the reference enum (kv.h:89-98); never renumbered.
enum class KvType : std::uint32_t { F32 = 0, F16 = 1, Q8_0 = 2, Q4_0 = 3, Q5_0 = 4, Q4_1 = 5 };

// The reference's table functions abort on a value outside the enum instead of
// returning a plausible number (kv.h:58-69); dispatchers return false.
[[noreturn]] inline void kv_unreachable(const char *what) {
  std::fprintf(stderr, "rdna4: %s: unknown KvType\n", what);
  std::abort();
}

inline const char *kv_type_name(KvType t) {
  const char *n = rd_kv_type_name((int)t);
  return n ? n : "<unknown-kv-type>";
}

// nullptr on success, else the message to report (kv.h:129-137).
inline const char *kv_type_parse(const char *name, KvType *out) {
  int t = 0;
  if (rd_kv_type_parse(name, &t) == RD_OK) {
    *out = (KvType)t;
    return nullptr;
  }
  return "kv type must be one of f32, f16, q8_0, q4_0, q5_0, q4_1";
}

inline double kv_bytes_per_elem(KvType t) {
  const double b = rd_kv_bytes_per_elem((int)t);
  if (b == 0.0) kv_unreachable("kv_bytes_per_elem");
  return b;
}

inline std::uint64_t kv_row_bytes(KvType t, int head_dim) {
  if ((std::uint32_t)t > (std::uint32_t)KvType::Q4_1) kv_unreachable("kv_row_bytes");
  return rd_kv_row_bytes((int)t, head_dim);
}

// kv.h:682-694. `width` is the number of f32 values (a multiple of 32).
inline bool kv_store_row_launch(KvType t, const float *d_src, void *d_dst, int width,
                                cudaStream_t stream = nullptr) {
  return rd_kv_store_rows((int)t, d_src, d_dst, width, stream) == RD_OK;
}
template <KvType CT>
inline bool kv_store_row_launch(const float *d_src, void *d_dst, int width,
                                cudaStream_t stream = nullptr) {
  return kv_store_row_launch(CT, d_src, d_dst, width, stream);
}

// kv.h:632-671.
inline bool kv_fill_launch(KvType t, void *d_cache, std::int64_t n_rows, int head_dim,
                           unsigned seed, cudaStream_t stream = nullptr) {
  return rd_kv_fill((int)t, d_cache, n_rows, head_dim, seed, stream) == RD_OK;
}

}  // namespace rdna4
