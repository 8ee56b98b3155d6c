// rdna4::fa2_prefill_* -- the reference's causal prefill tile launcher (its
// include/rdna4/attn_fa2.cuh:174-207) over rd_attn.h. f16/f16 caches, 6 query heads per
// KV head, head_dim 256; `kmax` is the index of the last key, `keys_total` the count.
#pragma once
#include <cuda_runtime.h>

#include "../rd_attn.h"
#include "kv.h"

namespace rdna4 {

inline bool fa2_prefill_launch(const float *d_q, const void *d_k, const void *d_v, float *d_o,
                               const int *d_pos, int n_q, int kmax, int keys_total, int n_head,
                               int n_head_kv, int head_dim, float scale,
                               cudaStream_t stream = nullptr) {
  return rd_fa2_prefill(d_q, d_k, d_v, d_o, d_pos, n_q, kmax, keys_total, n_head, n_head_kv,
                        head_dim, scale, stream) == RD_OK;
}

// Fail-closed admission, as in the reference; the window is wider here (any chunk
// length and any key count) because the kernel behind it has no measured-only range.
inline bool fa2_prefill_usable(KvType kt, KvType vt, int n_q, int pos0, int n_head, int n_head_kv,
                               int head_dim) {
  return rd_fa2_prefill_usable((int)kt, (int)vt, n_q, pos0, n_head, n_head_kv, head_dim) != 0;
}

}  // namespace rdna4
