// Internal (C++) launch interface shared by the translation units of the library.
#pragma once
#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

namespace rd {

struct DeviceStatus;

// ---- rd_kv.cu
int launch_kv_append(int kt, int vt, const float *ks, const float *vs, void *kd, void *vd,
                     int64_t width, int head_dim, int heads_per_tok, const int32_t *pos, int n_rot,
                     float freq_base, cudaStream_t st);
int launch_kv_fill(int type, void *cache, int64_t n_rows, int head_dim, uint32_t seed,
                   cudaStream_t st);
int launch_rope(float *x, int n_tok, int n_heads, int head_dim, int n_rot, float freq_base,
                const int32_t *pos, cudaStream_t st);
int launch_deinterleave(const float *yq, float *q, float *gate, int64_t n_rows, int head_dim,
                        cudaStream_t st);
int launch_sigmoid_gate(float *g, float *y, int64_t n, cudaStream_t st);
// n_values stored values of `type` at src -> f16 at dst (the dequantizing loads of
// include/rdna4/kv.h:174-368, rounded once).
int launch_kv_dequant_f16(int type, const void *src, void *dst, int64_t n_values, cudaStream_t st);
int launch_kv_dequant_f16_pair(int kt, const void *k, void *kdst, int vt, const void *v, void *vdst,
                               int64_t n_values, cudaStream_t st);

// ---- rd_pre.cu
int launch_rms_norm(const float *x, const float *w, float *y, int64_t nrows, int64_t ncols, float eps,
                    cudaStream_t st);
// One launch for deinterleave + q/k RMS-norm + RoPE + K/V quantize-and-store of n_tok
// tokens (head_dim 256, n_rot a multiple of 64).
int launch_pre_attn(int kt, int vt, const float *qg, const float *k_src, const float *v_src,
                    const float *q_w, const float *k_w, float eps, float *q_out, float *gate_out,
                    void *k_rows, void *v_rows, const int32_t *pos, int n_tok, int n_head, int nkv,
                    int n_rot, float freq_base, cudaStream_t st);

// ---- rd_shard.cu (types)
// Exchange buffers of a context-sharded group, as mapped into this process: x[r] is
// rank r's buffer (x[rank] the local one): kShardHeaderBytes of header, then
// [2 parities][world][n_head][4 dim quarters][kXPart] record parts of 8-byte words
// (f32 value, epoch).
constexpr int kShardMaxWorld = 8;
constexpr int kShardMaxHeads = 32;
constexpr int kXPart = 2 + 64;  // (m, l) + one quarter of the accumulator
constexpr size_t kShardHeaderBytes = 256;
struct ShardPeers {
  unsigned char *x[kShardMaxWorld];
  int rank;
  int world;
  unsigned long long wait_ns;  // how long the merge waits for the other ranks' records
};
// ---- rd_decode_*.cu
// One launch of the split-KV decode kernel: grid (n_splits, n_tok). Token i attends
// keys key_begin..(pos ? pos[i] : t). Writes n_splits records per (token, head) into
// partial[n_tok][n_head][n_splits][258].
struct DecodeArgs {
  const float *q;
  const void *k;
  const void *v;
  float *partial;
  const int32_t *pos;  // device, may be null
  int t;
  int key_begin;
  int n_tok;
  int n_head;
  int n_head_kv;
  float scale;
  int n_splits;
  DeviceStatus *status;
  // Fused append (optional, single token only): the f32 rows k_new / v_new
  // [n_head_kv][256] are quantized and stored as cache row `new_row` by the first CTAs of
  // the launch; the keys attended are still key_begin..t (pass t = new_row - 1).
  const float *k_new = nullptr;
  const float *v_new = nullptr;
  int new_row = 0;
  // Context-sharded call (single token): the launch also runs the exchange -- reduces its
  // records per (head, dim quarter), stores the parts into every rank's buffer, waits for
  // the other ranks' parts and writes the merged (optionally gated) output to push_out.
  const ShardPeers *push = nullptr;
  float *push_out = nullptr;    // [n_head][256]
  float *push_gate = nullptr;   // optional
};
int launch_decode(int kt, int vt, const DecodeArgs &a, cudaStream_t st);

// One sequence of a multi-sequence launch, as the kernels read it from device memory.
// The last of the q_len new tokens attends keys 0..t, token i keys 0..t-(q_len-1-i).
// Its records live at records[rec_base ...] as [q_len][n_head][n_splits][258].
struct alignas(64) DecodeSeq {
  alignas(64) unsigned char tm_k[128];  // CUtensorMap over the K cache, if k_tmap
  alignas(64) unsigned char tm_v[128];
  const float *q;    // [q_len][n_head][256]
  const uint8_t *k;
  const uint8_t *v;
  float *out;        // [q_len][n_head][256]
  float *gate;       // optional, like out
  int t;
  int n_splits;
  int rec_base;      // in records
  int k_tmap;
  int v_tmap;
  int pad_;
};
static_assert(sizeof(DecodeSeq) == 320, "DecodeSeq layout");

// launch_decode_multi runs in two phases: with host_seqs set it only encodes the
// tensor maps into the host-side descriptors (k_tmap / v_tmap say which exist); with
// host_seqs null it launches n_items CTAs over the device copies.
struct MultiDecodeArgs {
  DecodeSeq *host_seqs;
  int n_seq;
  const DecodeSeq *dev_seqs;
  const int4 *dev_items;  // (sequence, token, split, 0)
  int n_items;
  int q_len;
  int n_head;
  int n_head_kv;
  float scale;
  float *records;
  DeviceStatus *status;
};
int launch_decode_multi(int kt, int vt, const MultiDecodeArgs &a, cudaStream_t st);
// Keys per tile of the (kt, vt) kernel: the granularity of the key split.
int decode_tile_keys(int kt, int vt);

// ---- rd_tmap.cu
// Tensor map over a KV cache viewed as u64 [n_rows][key bytes / 8] with a box of
// [tile_rows][key bytes / 8 + 2]: one copy brings a whole tile into shared memory with
// a key pitch of key bytes + 16 (the extra columns are outside the tensor: zeros).
// Returns RD_OK, or an error if the key is too wide for one box (f16 / f32 rows), the
// driver entry point is unavailable, or the encoder refuses.
int encode_kv_tmap(void *tmap_out, const void *base, int type, int n_head_kv, int64_t n_rows,
                   int tile_rows);

// Tensor map over an f16 KV cache [n_rows][n_head_kv * 256] with a box of
// [tile_rows][64 dims] and the hardware 128-byte swizzle (what tcgen05.mma descriptors
// with SWIZZLE_128B read).
int encode_f16_tmap(void *tmap_out, const void *base, int n_head_kv, int64_t n_rows, int tile_rows);

// ---- rd_prefill.cu
// Causal prefill attention over f16 caches on tcgen05: token i attends keys 0..pos[i]
// (pos on the device), keys_total rows exist in the cache. gate (optional) fuses
// out *= sigmoid(gate); n_rot > 0 applies the partial RoPE to the queries on load.
// n_splits > 1 (with `records`, prefill_record_bytes(...) bytes): the keys are also split
// over gridDim.z and a second launch merges the per-split records.
int launch_prefill(const float *q, const void *k, const void *v, float *out, const float *gate,
                   const int32_t *pos, int n_q, int keys_total, int n_head, int n_head_kv, float scale,
                   int n_rot, float freq_base, DeviceStatus *status, float *records, int n_splits, void *q16, const float *k_new, const float *v_new, void *k_dst, void *v_dst,
                   cudaStream_t st);
size_t prefill_rope_bytes(int n_q, int n_head);   // the f16 query copy launch_prefill needs when n_rot > 0
int prefill_splits(int n_q, int keys_total, int n_head, int sms);
size_t prefill_record_bytes(int n_q, int n_head, int splits);

// ---- rd_merge.cu
// partial [n_rows][n_splits][258] -> out [n_rows][256]; optional fused sigmoid gate.
int launch_merge(const float *partial, float *out, int n_rows, int n_splits, float *gate,
                 cudaStream_t st);
// The same merge with one more key folded in: the key stored at k_row / v_row (cache row
// of the newest position, types kt / vt, n_head_kv heads) attended by q [n_rows][256]
// with `scale`, as if it were one more record (m = score, l = 1, acc = v). q must not
// alias out.
struct ExtraKey {
  const float *q;
  const uint8_t *k_row;
  const uint8_t *v_row;
  int kt, vt, nkv;
  float scale;
};
int launch_merge_extra(const float *partial, float *out, int n_rows, int n_splits, float *gate,
                       const ExtraKey &x, cudaStream_t st);
// partial [n_rows][n_in][258] -> records [n_rows][n_out][258]: record j merges the
// input records [j*n_in/n_out, (j+1)*n_in/n_out).
int launch_merge_records(const float *partial, float *records, int n_rows, int n_in, int n_out,
                         cudaStream_t st);
// Multi-sequence merge: row (sequence, token, head) reads its n_splits records from the
// sequence's block of `records` and writes (optionally gated) into the sequence's out.
int launch_merge_multi(const DecodeSeq *dev_seqs, const float *records, int n_seq, int q_len,
                       int n_head, cudaStream_t st);

// ---- rd_shard.cu (launchers)
// partial [n_head][n_in][258] (this rank's split records) -> one record per head stored
// into every rank's buffer, then this call's epoch into every rank's flag.
int launch_shard_push(const float *partial, int n_in, int n_head, const ShardPeers &g,
                      cudaStream_t st);
// Waits (bounded) for all ranks' records of this call, merges them into out
// [n_head][256] (optional fused sigmoid gate) and advances the local epoch.
int launch_shard_merge(float *out, float *gate, int n_head, const ShardPeers &g,
                       DeviceStatus *status, cudaStream_t st);
// Both halves in one launch.
int launch_shard_exchange(const float *partial, int n_in, float *out, float *gate, int n_head,
                          const ShardPeers &g, DeviceStatus *status, cudaStream_t st);

}  // namespace rd
