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
};
int launch_decode(int kt, int vt, const DecodeArgs &a, cudaStream_t st);
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
int launch_prefill(const float *q, const void *k, const void *v, float *out, const float *gate,
                   const int32_t *pos, int n_q, int keys_total, int n_head, int n_head_kv, float scale,
                   int n_rot, float freq_base, DeviceStatus *status, cudaStream_t st);

// ---- rd_merge.cu
// partial [n_rows][n_splits][258] -> out [n_rows][256]; optional fused sigmoid gate.
int launch_merge(const float *partial, float *out, int n_rows, int n_splits, float *gate,
                 cudaStream_t st);
// partial [n_rows][n_in][258] -> records [n_rows][n_out][258]: record j merges the
// input records [j*n_in/n_out, (j+1)*n_in/n_out).
int launch_merge_records(const float *partial, float *records, int n_rows, int n_in, int n_out,
                         cudaStream_t st);

}  // namespace rd
