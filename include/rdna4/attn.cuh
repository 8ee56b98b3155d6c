// rdna4::rope_launch / attn_* -- the reference's attention launch API (its
// include/rdna4/attn.cuh) as C++17 inline wrappers over rd_attn.h. Signatures, argument
// meaning (`t` = index of the last attended key, device `pos[]`, caller-owned partial
// buffer, q and out may alias) and the bool result are the reference's.
//
// One behavioural note for callers that size `d_partial` with attn_partial_bytes: the
// B200 kernels keep one partial record per SM, not per requested split, in a per-device
// workspace that the library grows on first use; `d_partial` is only written when the
// caller asks for records without a merge (rd_attn_decode_split with out == nullptr).
#pragma once
#include <cuda_runtime.h>

#include <cstddef>
#include <cstdint>

#include "../rd_attn.h"
#include "kv.h"

namespace rdna4 {

// tuning.h:144-150 of the reference -- contract values kept for callers that read
// them (e.g. Graph::attn_splits_for); the split COUNT actually used is planned inside
// the library from the SM count.
namespace tuned {
inline constexpr int kAttnWarpsPerBlock = 8;
inline constexpr int kAttnSplitWpbLimit = 4;
inline constexpr int kAttnSplitWpbWide = 16;
inline constexpr int kAttnSplitMin = 512;
inline constexpr int kAttnMaxSplits = 16;
inline constexpr int kAttnSplitCtasDense = 96;
}  // namespace tuned
constexpr int kAttnWarpsPerBlock = tuned::kAttnWarpsPerBlock;
constexpr int kAttnSplitWpbLimit = tuned::kAttnSplitWpbLimit;
constexpr int kAttnSplitWpbWide = tuned::kAttnSplitWpbWide;

// attn.cuh:56-63
inline bool rope_launch(float *d_x, int n_tokens, int n_heads, int head_dim, int n_rot,
                        float freq_base, const int *d_pos, cudaStream_t stream = nullptr) {
  return rd_rope(d_x, n_tokens, n_heads, head_dim, n_rot, freq_base, d_pos, stream) == RD_OK;
}

// attn.cuh:201-249
inline bool attn_launch(const float *d_q, const void *d_k, const void *d_v, float *d_out, int t,
                        int n_head, int n_head_kv, int head_dim, float scale, KvType kt, KvType vt,
                        cudaStream_t stream = nullptr) {
  return rd_attn_decode(d_q, d_k, d_v, d_out, t, n_head, n_head_kv, head_dim, scale, (int)kt,
                        (int)vt, stream) == RD_OK;
}

// attn.cuh:373-424
inline bool attn_batch_launch(const float *d_q, const void *d_k, const void *d_v, float *d_out,
                              const int *d_pos, int n_tok, int n_head, int n_head_kv, int head_dim,
                              float scale, KvType kt, KvType vt, cudaStream_t stream = nullptr) {
  return rd_attn_batch(d_q, d_k, d_v, d_out, d_pos, n_tok, n_head, n_head_kv, head_dim, scale,
                       (int)kt, (int)vt, stream) == RD_OK;
}

// attn.cuh:665-667
inline std::size_t attn_partial_bytes(int n_head, int head_dim, int n_splits) {
  return rd_attn_partial_bytes(n_head, head_dim, n_splits);
}

// attn.cuh:895-901 (shape policy of the reference's split kernel; informational here)
// Graph::attn_splits_for (graph.cuh:495-526) as a free function: the split count a caller
// sizes its partial buffer for (the library plans its own internal split, rd_attn_plan).
inline int attn_splits_for(int keys, KvType kt, KvType vt, int n_head, int forced = 0) {
  return rd_attn_splits_for(keys, (int)kt, (int)vt, n_head, forced);
}
inline int attn_split_wpb(int n_splits) {
  if (n_splits <= kAttnSplitWpbLimit) return 16;
  if (n_splits >= kAttnSplitWpbWide) return 16;
  return kAttnWarpsPerBlock;
}

// attn.cuh:903-956
inline bool attn_launch_split(const float *d_q, const void *d_k, const void *d_v, float *d_out,
                              float *d_partial, int t, int n_head, int n_head_kv, int head_dim,
                              float scale, KvType kt, KvType vt, int n_splits,
                              cudaStream_t stream = nullptr) {
  if (d_out == nullptr) return false;
  return rd_attn_decode_split(d_q, d_k, d_v, d_out, d_partial, t, n_head, n_head_kv, head_dim,
                              scale, (int)kt, (int)vt, n_splits, stream) == RD_OK;
}

// attn.cuh:958-1049
inline bool attn_split_batch_launch(const float *d_q, const void *d_k, const void *d_v,
                                    float *d_out, float *d_partial, const int *d_pos, int n_tok,
                                    int n_head, int n_head_kv, int head_dim, float scale, KvType kt,
                                    KvType vt, int n_splits, cudaStream_t stream = nullptr) {
  if (d_out == nullptr) return false;
  return rd_attn_split_batch(d_q, d_k, d_v, d_out, d_partial, d_pos, n_tok, n_head, n_head_kv,
                             head_dim, scale, (int)kt, (int)vt, n_splits, stream) == RD_OK;
}

// The merge the reference launches as a bare kernel (attn.cuh:563-590, 605): records
// [n_head][n_splits][2+head_dim] -> out [n_head][head_dim].
inline bool attn_merge_launch(const float *d_partial, float *d_out, int n_head, int head_dim,
                              int n_splits, cudaStream_t stream = nullptr) {
  return rd_attn_merge(d_partial, d_out, n_head, head_dim, n_splits, nullptr, stream) == RD_OK;
}

// nn.cuh:414-420 and gdn.cuh:377-384, 853-862 of the reference: the gate glue around
// the attention call (kept here so that one include serves Graph::full_attn).
// nn.cuh:239-243 of the reference.
inline bool rms_norm_launch(const float *d_x, const float *d_w, float *d_y, std::int64_t nrows,
                            std::int64_t ncols, float eps, cudaStream_t stream = nullptr) {
  return rd_rms_norm(d_x, d_w, d_y, nrows, ncols, eps, stream) == RD_OK;
}
inline bool sigmoid_gate_launch(float *d_g_io, float *d_y_io, std::int64_t n,
                                cudaStream_t stream = nullptr) {
  return rd_sigmoid_gate(d_g_io, d_y_io, n, stream) == RD_OK;
}
inline bool deinterleave_q_gate_launch(const float *d_yq, float *d_q, float *d_gate, int n_head,
                                       int head_dim, cudaStream_t stream = nullptr) {
  return rd_deinterleave_q_gate(d_yq, d_q, d_gate, 1, n_head, head_dim, stream) == RD_OK;
}
inline bool deinterleave_q_gate_batch_launch(const float *d_yq, float *d_q, float *d_gate, int n_tok,
                                             int n_head, int head_dim,
                                             cudaStream_t stream = nullptr) {
  return rd_deinterleave_q_gate(d_yq, d_q, d_gate, n_tok, n_head, head_dim, stream) == RD_OK;
}

}  // namespace rdna4
