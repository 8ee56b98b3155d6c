/*
 * rd_attn.h -- C ABI of the B200 (sm_100a) attention / KV-cache library.
 *
 * This is the drop-in boundary for the attention hot path of rdna4-infer: every
 * entry point below replaces one launcher of the reference's
 * include/rdna4/{kv.h,attn.cuh,attn_fa2.cuh,nn.cuh,gdn.cuh} (cited per function,
 * paths relative to the reference project). The C++17 wrappers in
 * include/rdna4/ give the same names and signatures as the reference in
 * namespace rdna4 and forward here.
 *
 * Conventions kept from the reference:
 *   - all pointers are caller-owned DEVICE pointers unless a comment says host;
 *   - activations are f32; q and out may be the same buffer;
 *   - K/V caches are rows [key][n_head_kv] of `row_bytes(type, head_dim)` bytes in
 *     GGUF 32-element blocks (fp16 scale first), key j / kv head h at
 *     (j*n_head_kv + h) * row_bytes;
 *   - `t` is the index of the LAST attended key (n_keys = t + 1); `pos[]` is a device
 *     int32 array with one such index per query token;
 *   - `scale` is passed in, never recomputed; `stream` is a cudaStream_t (NULL = the
 *     default stream); launch order on the stream is the only synchronisation;
 *   - no host synchronisation and no allocation inside a call, with one documented
 *     exception: the launchers that keep the reference's small `partial` argument
 *     (rd_attn_decode, rd_attn_decode_split, rd_attn_batch, rd_attn_split_batch) grow
 *     a per-device workspace with cudaMalloc the first time a shape needs it, because
 *     148 SMs want more partial records than the reference's 16-split buffer holds.
 *     That workspace is ONE per device, shared by all streams and host threads: use
 *     these launchers (and rd_fa2_prefill / rd_attn_prefill_fused, which grow it the
 *     same way) from one stream per device, or order the streams yourself -- two calls
 *     whose kernels overlap race on the records. A later, larger shape frees and
 *     reallocates it, which leaves a CUDA graph captured earlier with the old pointer:
 *     warm up with the largest shape before capturing, or use the *_ws entry points,
 *     which take the workspace from the caller, never allocate and have no such
 *     sharing (multi-stream and graph users).
 *
 * Every function returns RD_OK (0) or a negative RD_ERR_* code; nothing aborts and
 * nothing traps on the device. Shapes outside the supported set are refused with
 * RD_ERR_UNSUPPORTED: head_dim must be 256, n_head == 6 * n_head_kv, n_head_kv in
 * {1, 2, 4}; all six K/V types in every combination for decode / batch attention
 * (attn.cuh:203-246), f16 / f16 for the prefill tile kernel (attn_fa2.cuh:177-180).
 */
#ifndef RD_ATTN_H
#define RD_ATTN_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* KvType of include/rdna4/kv.h:89-98 (values never renumbered). */
enum {
  RD_KV_F32 = 0,
  RD_KV_F16 = 1,
  RD_KV_Q8_0 = 2,
  RD_KV_Q4_0 = 3,
  RD_KV_Q5_0 = 4,
  RD_KV_Q4_1 = 5
};

enum {
  RD_OK = 0,
  RD_ERR_TYPE = -1,        /* KV type outside the enum */
  RD_ERR_SHAPE = -2,       /* negative / zero / non-multiple-of-32 sizes, n_splits < 1 ... */
  RD_ERR_UNSUPPORTED = -3, /* valid for the reference, not built here (see above) */
  RD_ERR_NULL = -4,        /* a required pointer is NULL */
  RD_ERR_ALIGN = -5,       /* a pointer is not aligned as the entry point requires */
  RD_ERR_CUDA = -6,        /* a CUDA runtime call or launch failed */
  RD_ERR_WORKSPACE = -7,   /* caller-provided workspace too small / workspace growth failed */
  RD_ERR_DEVICE = -8,      /* a kernel recorded a bounded-wait timeout (rd_device_status) */
  RD_ERR_LIMIT = -9        /* a size exceeds a fixed maximum (rd_attn_decode_noalloc, rd_attn_shard_*) */
};

const char *rd_strerror(int code);

/* ---- KV tables: kv_type_name / kv_type_parse / kv_bytes_per_elem / kv_row_bytes,
 * include/rdna4/kv.h:100-169. Unknown types return NULL / 0 here; the C++ wrapper
 * aborts on them as the reference does (kv.h:58-69). */
const char *rd_kv_type_name(int type);
int rd_kv_type_parse(const char *name, int *out_type);
double rd_kv_bytes_per_elem(int type);
uint64_t rd_kv_row_bytes(int type, int head_dim);

/* ---- KV append: kv_store_row_launch(t, src, dst, width), include/rdna4/kv.h:673-694.
 * `width` consecutive f32 values (n_tok * n_head_kv * head_dim, graph.cuh:1028) are
 * stored as width/32 blocks (or width scalars). Bit-exact with the reference
 * quantizers for all six types. src 4-byte, dst 2-byte aligned. */
int rd_kv_store_rows(int type, const float *src, void *dst, int64_t width, void *stream);

/* One launch for the K and the V rows of a chunk (the two calls of
 * Graph::kv_write_batch, graph.cuh:1011-1035), optionally applying RoPE to the K rows
 * first (pos != NULL): k_src is then [n_tok][n_head_kv][head_dim] and is NOT
 * modified. Without RoPE this is exactly two rd_kv_store_rows. */
int rd_kv_append(int k_type, int v_type, const float *k_src, const float *v_src, void *k_dst,
                 void *v_dst, int n_tok, int n_head_kv, int head_dim, const int32_t *pos,
                 int n_rot, float freq_base, void *stream);

/* ---- synthetic cache: kv_fill_launch, include/rdna4/kv.h:632-671. Row r, element e
 * holds kv_rand(r*head_dim+e, seed) stored with the real quantizer (the reference's
 * own q4_0 fill writes racing per-byte scales and is not reproduced). */
int rd_kv_fill(int type, void *cache, int64_t n_rows, int head_dim, uint32_t seed, void *stream);

/* ---- RoPE: rope_launch, include/rdna4/attn.cuh:56-63. In place on
 * x[n_tok][n_heads][head_dim], split-half pairs of the first n_rot dims. */
int rd_rope(float *x, int n_tok, int n_heads, int head_dim, int n_rot, float freq_base,
            const int32_t *pos, void *stream);

/* ---- gate glue: deinterleave_q_gate(_batch)_launch, include/rdna4/gdn.cuh:377-384,
 * 853-862, and sigmoid_gate_launch, include/rdna4/nn.cuh:414-420 (y *= sigmoid(g),
 * sigmoid stored back into g). */
int rd_deinterleave_q_gate(const float *yq, float *q, float *gate, int n_tok, int n_head,
                           int head_dim, void *stream);
int rd_sigmoid_gate(float *g_io, float *y_io, int64_t n, void *stream);

/* ---- RMS-norm (rms_norm_launch, nn.cuh:239-243; kernel :23-63): y = x / sqrt(mean(x^2)
 * + eps) (* w if w != NULL) per row of n_cols; x and y may alias. The sum of squares
 * keeps the reference kernel's order; the reciprocal square root is correctly rounded. */
int rd_rms_norm(const float *x, const float *w, float *y, int64_t n_rows, int64_t n_cols, float eps,
                void *stream);

/* ---- fused pre-attention stage of a full-attention layer (no single counterpart: the
 * reference runs seven launches here, graph.cuh:915-954 -- deinterleave_q_gate_launch,
 * two rms_norm_launch, two rope_launch, two kv_store_row_launch).
 *   q_gate   [n_tok][n_head][2*head_dim] f32: the q projection, q then gate per head
 *   k_src, v_src   [n_tok][n_head_kv][head_dim] f32: the k and v projections
 *   q_norm_w, k_norm_w   [head_dim] norm weights (NULL: none); eps the RMS epsilon
 *   q_out    [n_tok][n_head][head_dim]: normalised, rotated q (input of the attention)
 *   gate_out [n_tok][n_head][head_dim]: the gate logits, copied
 *   k_rows, v_rows   first cache row of the n_tok new tokens (cache + pos0 * n_head_kv *
 *                    row_bytes): k normalised, rotated, stored as k_type; v stored as v_type
 *   pos      device int32 [n_tok]; n_rot a multiple of 64 (0: no rotation).
 * Results equal the seven separate calls of this library bit for bit. head_dim 256. */
int rd_pre_attn_fused(const float *q_gate, const float *k_src, const float *v_src,
                      const float *q_norm_w, const float *k_norm_w, float eps, float *q_out,
                      float *gate_out, void *k_rows, void *v_rows, int k_type, int v_type,
                      const int32_t *pos, int n_tok, int n_head, int n_head_kv, int head_dim,
                      int n_rot, float freq_base, void *stream);

/* ---- split policy. rd_attn_splits_for is the reference's rule for how many partial
 * records per head a caller allocates (Graph::attn_splits_for, graph.cuh:495-526, constants
 * of tuning.h:144-150): 1 below 512 keys; ceil(96 / n_head) for f16 / f32 caches;
 * min(16, n_keys / 512) for quantized ones; forced > 0 overrides (the RD_ATTN_SPLITS
 * knob), capped at 16. Host arithmetic only.
 *
 * rd_attn_plan reports what THIS library does with a decode launch on a GPU of sm_count
 * SMs (<= 0: the current device): keys per shared-memory tile (16, 32 or 48 by K / V type),
 * stages of the TMA ring, and the internal split count (about one CTA per SM, never more
 * splits than key tiles). Any output pointer may be NULL. Host arithmetic only when
 * sm_count is given. */
int rd_attn_splits_for(int n_keys, int k_type, int v_type, int n_head, int forced);
/* What the prefill entries do with a chunk of n_q tokens over keys_total keys on a GPU of
 * sm_count SMs (<= 0: the current device): the key splits per (128-token tile, head) and
 * the CTAs of the tile-kernel launch. One split unless the cost model says that filling the
 * idle SMs outweighs a second wave of fixed costs and the records (from about 8192 keys for
 * 512 tokens x 24 heads on 148 SMs). Host arithmetic only when sm_count is given. */
int rd_attn_prefill_plan(int n_q, int keys_total, int n_head, int sm_count, int *n_splits, int *n_ctas);
int rd_attn_plan(int n_keys, int n_tok, int n_head_kv, int k_type, int v_type, int sm_count,
                 int *tile_keys, int *ring_stages, int *n_splits);

/* ---- partial records: attn_partial_bytes, include/rdna4/attn.cuh:665-667.
 * A record is (m, l, acc[head_dim]) f32 in natural-log units: m = max scaled score,
 * l = sum exp(s - m), acc = sum exp(s - m) * v; an empty record is (-inf, 0, 0...). */
size_t rd_attn_partial_bytes(int n_head, int head_dim, int n_splits);

/* Workspace the decode kernels want for `n_tok` query tokens on the current device
 * (internal split records + status word). Pass it to the *_ws entry points. */
size_t rd_attn_workspace_bytes(int n_tok, int n_head, int head_dim);

/* ---- single-token attention: attn_launch, include/rdna4/attn.cuh:201-249. */
int rd_attn_decode(const float *q, const void *k, const void *v, float *out, int t, int n_head,
                   int n_head_kv, int head_dim, float scale, int k_type, int v_type,
                   void *stream);

/* ---- split-KV single-token attention: attn_launch_split, include/rdna4/attn.cuh:903-956.
 * `n_splits` is a hint: the kernel spreads the keys over all SMs and merges. If
 * `out` is NULL, `partial` receives exactly n_splits records per head in the
 * reference layout [h][s][2+head_dim] (split s owns the s-th contiguous slice of the
 * keys) and no merge runs; otherwise `partial` may be NULL. */
int rd_attn_decode_split(const float *q, const void *k, const void *v, float *out,
                         float *partial, int t, int n_head, int n_head_kv, int head_dim,
                         float scale, int k_type, int v_type, int n_splits, void *stream);

/* The same with every option spelled out and no allocation:
 *   key_begin..t     the attended key range (key_begin > t gives the empty record);
 *   gate             optional [n_head][head_dim]: out *= sigmoid(gate) fused into the
 *                    merge, sigmoid stored back (nn.cuh:405-412);
 *   workspace/bytes  from rd_attn_workspace_bytes(1, ...), 256-byte aligned. */
int rd_attn_decode_ws(const float *q, const void *k, const void *v, float *out, float *partial,
                      int key_begin, int t, int n_head, int n_head_kv, int head_dim, float scale,
                      int k_type, int v_type, int n_splits, float *gate, void *workspace,
                      size_t workspace_bytes, void *stream);

/* ---- append + decode in two launches (no counterpart: the reference runs
 * kv_store_row_launch twice, then attn_launch_split, graph.cuh:1011-1035 and 958-977).
 * Stores k_new / v_new ([n_head_kv][head_dim] f32, K already normalised and rotated) as
 * row t of the caches and returns the attention of q over keys 0..t, the new one
 * included: the first CTAs of the split-KV launch quantize and store the row while the
 * launch attends keys 0..t-1, and the merge folds key t in from the cache. Cache bytes
 * equal rd_kv_append's; the output equals rd_attn_decode_ws after rd_kv_append within
 * the attention tolerance. q must not alias out (RD_ERR_UNSUPPORTED). gate as in
 * rd_attn_decode_ws; workspace from rd_attn_workspace_bytes(1, ...). */
int rd_attn_decode_append_ws(const float *q, const float *k_new, const float *v_new, void *k_cache,
                             void *v_cache, float *out, int t, int n_head, int n_head_kv, int head_dim,
                             float scale, int k_type, int v_type, float *gate, void *workspace,
                             size_t workspace_bytes, void *stream);

/* ---- many sequences in one launch (decode and short verify blocks).
 *
 * The reference serves one sequence per Graph (graph.cuh:958-977 decode,
 * :1479-1535 verify); a host that batches requests calls those once per sequence. This
 * entry takes the per-sequence caches as a host array of descriptors and runs ONE
 * decode launch plus ONE merge for all of them: the key ranges of all sequences are cut
 * into chunks of equal length, so ragged contexts load the SMs evenly.
 *
 * Sequence i has q_len new tokens; its LAST token attends keys 0..t of its cache and
 * token j keys 0..t-(q_len-1-j) (causal inside the block, as attn_batch_kernel with
 * pos[j] = t-(q_len-1-j)). t >= q_len-1. q / out / gate are [q_len][n_head][head_dim]
 * f32 on the device (q 16-byte aligned); gate may be NULL, else out *= sigmoid(gate)
 * and the sigmoid is stored back.
 *
 * The descriptor array is read on the host during the call; the workspace
 * (rd_attn_multi_workspace_bytes, 256-byte aligned, device memory) receives the device
 * copies, the work list and the partial records, and must stay untouched until the
 * stream has passed the call. The call enqueues a host-to-device copy from pageable
 * memory, so it cannot be part of a stream capture. */
typedef struct rd_attn_seq {
  const float *q;
  const void *k;
  const void *v;
  float *out;
  float *gate;
  int32_t t;
  int32_t reserved;
} rd_attn_seq;
size_t rd_attn_multi_workspace_bytes(int n_seq, int q_len, int n_head, int head_dim);
int rd_attn_decode_multi(const rd_attn_seq *seqs, int n_seq, int q_len, int n_head, int n_head_kv,
                         int head_dim, float scale, int k_type, int v_type, void *workspace,
                         size_t workspace_bytes, void *stream);

/* The same call in its two halves, for hosts that capture the decode step into a CUDA graph.
 *   rd_attn_multi_plan    host arithmetic only: checks the descriptors, cuts the key ranges
 *                         into work items and encodes the tensor maps into `plan`, host
 *                         memory of rd_attn_multi_plan_bytes(n_seq, q_len) bytes, 16-byte
 *                         aligned. pad_items > 0 pads the work list to exactly that many
 *                         items (the extra CTAs leave at once), so that the grid of a
 *                         captured launch stays valid while the contexts grow; a plan that
 *                         needs more items returns RD_ERR_LIMIT (capture again with more).
 *   rd_attn_multi_launch  one host-to-device copy of the plan into the workspace, the
 *                         decode launch and the merge, on `stream`. With the plan in PINNED
 *                         host memory the call can be captured, and a replay reads the plan
 *                         as it is then: rewrite it with rd_attn_multi_plan (same n_seq,
 *                         q_len, types and pad_items) between replays, after the previous
 *                         replay's copy has completed. From pageable memory it behaves as
 *                         rd_attn_decode_multi (which is these two calls in a row). */
size_t rd_attn_multi_plan_bytes(int n_seq, int q_len);
int rd_attn_multi_plan(const rd_attn_seq *seqs, int n_seq, int q_len, int n_head, int n_head_kv,
                       int head_dim, int k_type, int v_type, int pad_items, void *plan, size_t plan_bytes);
int rd_attn_multi_launch(const void *plan, float scale, void *workspace, size_t workspace_bytes,
                         void *stream);

/* ---- context-sharded decode over several GPUs, exchange fused into the merge.
 * (No counterpart in the reference, which is single-GPU.)
 *
 * One process per GPU; rank r holds a contiguous slice of every layer's keys. Each rank
 * calls this with ITS slice (k, v = start of the slice, t = index of the slice's last
 * row, -1 for an empty slice) and the same q; every rank receives the full attention
 * output. Instead of a library all-gather between two merges, each rank's kernel
 * stores its per-head record (m, l, acc) directly into every rank's exchange buffer
 * over NVLink, every value tagged with the call's sequence number in the same 8-byte
 * store; the final merge spins (bounded) on the tags of the values it needs.
 *
 *   group->xbuf[r]   rank r's exchange buffer AS MAPPED INTO THIS PROCESS (peer-mapped
 *                    or symmetric memory; xbuf[rank] is the local one), each
 *                    rd_shard_xbuf_bytes(...) bytes, 256-byte aligned. Zero all of them
 *                    once and synchronise the ranks before the first call; all ranks
 *                    must then make the same sequence of calls on the group.
 *   wait_limit_us    how long the merge waits for the other ranks (0: one second).
 *                    When it runs out the kernel stores zeros, records the event
 *                    (rd_device_status returns RD_ERR_DEVICE) and returns normally.
 *   workspace        rd_attn_workspace_bytes(1, ...), 256-byte aligned.
 * The call is ONE launch on `stream` and nothing else (no copy, no allocation): the
 * decode kernel's first n_head * 4 CTAs wait for the launch's records, reduce them, store
 * the parts into every rank's buffer, wait (bounded) for the other ranks' parts and merge.
 * The call counter lives in the exchange buffer, so the call can be captured into a CUDA
 * graph and replayed. world <= 8.
 *
 * rd_attn_shard_push / rd_attn_shard_merge are the two halves of the exchange for a
 * caller that computes the split records itself (rd_attn_decode_split with out == NULL,
 * partial [n_head][n_splits][2 + head_dim]) or wants other work between the halves.
 * On every rank each push must be followed by exactly one merge before the next push. */
typedef struct rd_shard_group {
  int32_t rank;
  int32_t world;
  void *const *xbuf;
  uint32_t wait_limit_us;
  uint32_t reserved;
} rd_shard_group;
size_t rd_shard_xbuf_bytes(int n_head, int head_dim, int world);
int rd_attn_decode_sharded(const float *q, const void *k, const void *v, float *out, int t,
                           int n_head, int n_head_kv, int head_dim, float scale, int k_type,
                           int v_type, float *gate, void *workspace, size_t workspace_bytes,
                           const rd_shard_group *group, void *stream);
/* The same for the rank that owns the newest position: k_new / v_new [n_head_kv][head_dim]
 * f32 are quantized and stored as row t of its slice inside the launch (bytes as
 * rd_kv_append writes them; rotate K beforehand if the model does), and that key joins the
 * exchange as one more record -- rd_kv_append (kv_store_row_launch, include/rdna4/kv.h:
 * 673-694) and rd_attn_decode_sharded in one launch. q must not alias out. */
int rd_attn_decode_sharded_append(const float *q, const float *k_new, const float *v_new, void *k, void *v,
                                  float *out, int t, int n_head, int n_head_kv, int head_dim, float scale,
                                  int k_type, int v_type, float *gate, void *workspace,
                                  size_t workspace_bytes, const rd_shard_group *group, void *stream);
int rd_attn_shard_push(const float *partial, int n_splits, int n_head, int head_dim,
                       const rd_shard_group *group, void *stream);
int rd_attn_shard_merge(float *out, float *gate, int n_head, int head_dim,
                        const rd_shard_group *group, void *stream);

/* ---- single-token attention that allocates nothing. (No counterpart in the reference.)
 *
 * Some hosts cannot let a library call cudaMalloc: a serving process whose memory
 * manager has already claimed the whole device, a latency-critical decode loop in which
 * the implicit device-wide synchronisation of cudaMalloc / cudaFree is not acceptable,
 * or an embedder with a no-allocation-after-start-up rule. For them this entry computes
 * exactly what rd_attn_decode_split does (optionally with the fused sigmoid gate of
 * rd_attn_decode_ws), but keeps its partial records in a fixed array that is part of
 * the library image: RD_NOALLOC_MAX_HEADS x RD_NOALLOC_MAX_SPLITS records, 3.96 MB,
 * resident on every GPU that loads the library until the process exits. It calls no
 * cudaMalloc, no cudaFree and no allocating library routine.
 *
 *   - n_head above RD_NOALLOC_MAX_HEADS returns RD_ERR_LIMIT; the key split is capped at
 *     RD_NOALLOC_MAX_SPLITS records per head (enough for one per SM on a B200).
 *   - The first call on a device looks the array's device address up (once per device);
 *     make that first call before any stream capture.
 *   - All calls on a device share the one array and it keeps the previous call's
 *     records. Nothing has to start at zero -- each call writes every record it later
 *     merges -- but two calls whose kernels overlap on the GPU (different streams) race
 *     on it. Calls on one stream are ordered and safe. */
#define RD_NOALLOC_MAX_HEADS 24
#define RD_NOALLOC_MAX_SPLITS 160
int rd_attn_decode_noalloc(const float *q, const void *k, const void *v, float *out, int t,
                           int n_head, int n_head_kv, int head_dim, float scale, int k_type,
                           int v_type, float *gate, void *stream);

/* ---- merge: attn_merge_kernel / attn_merge_batch_kernel launches,
 * include/rdna4/attn.cuh:563-590,795-827. partial [n_rows][n_splits][2+head_dim],
 * out [n_rows][head_dim] with n_rows = n_tok * n_head. Rows whose records are all
 * empty give zeros. `gate` as above (may be NULL). */
int rd_attn_merge(const float *partial, float *out, int n_rows, int head_dim, int n_splits,
                  float *gate, void *stream);

/* ---- multi-token attention (prefill chunk, speculative verify): attn_batch_launch,
 * include/rdna4/attn.cuh:373-424, and attn_split_batch_launch, :958-1049. Token i
 * attends keys 0..pos[i]. q/out [n_tok][n_head][head_dim]. */
int rd_attn_batch(const float *q, const void *k, const void *v, float *out, const int32_t *pos,
                  int n_tok, int n_head, int n_head_kv, int head_dim, float scale, int k_type,
                  int v_type, void *stream);
int rd_attn_split_batch(const float *q, const void *k, const void *v, float *out, float *partial,
                        const int32_t *pos, int n_tok, int n_head, int n_head_kv, int head_dim,
                        float scale, int k_type, int v_type, int n_splits, void *stream);

/* ---- causal prefill tile kernel: fa2_prefill_usable / fa2_prefill_launch,
 * include/rdna4/attn_fa2.cuh:174-207. f16/f16 caches; runs on tcgen05 tensor cores with
 * TMEM accumulators. The admission window is wider than the reference's (any n_q >= 1
 * and any key count), since the tensor-core kernel has no measured-only range to
 * protect. keys_total rows must exist in the caches; token i attends keys 0..pos[i].
 * When n_q * n_head / 128 CTAs would leave most SMs idle, the keys are split over more CTAs
 * and a second launch merges per-split records; rd_fa2_prefill and rd_attn_prefill_fused
 * keep those records in the library's own per-device workspace (grown on demand like that
 * of the allocating launchers above: warm up once before a stream capture), while
 * rd_attn_prefill_typed keeps them in the caller's workspace and never allocates. */
int rd_fa2_prefill_usable(int k_type, int v_type, int n_q, int pos0, int n_head, int n_head_kv,
                          int head_dim);
int rd_fa2_prefill(const float *q, const void *k, const void *v, float *o, const int32_t *pos,
                   int n_q, int kmax, int keys_total, int n_head, int n_head_kv, int head_dim,
                   float scale, void *stream);

/* The same kernel with its fused edges (no single counterpart in the reference: it is
 * rope_launch on q, include/rdna4/attn.cuh:56-63, + the prefill attention + the sigmoid
 * gate of nn.cuh:405-420 in one launch). n_rot > 0 (a multiple of 16, <= 64) rotates
 * the first n_rot dims of every query row by its pos[] -- in a pre-pass that writes the
 * rotated, scaled queries as f16 into the library's grown workspace (512 bytes per token
 * and head; the tile kernel starts under it as a programmatic dependent launch and loads
 * its query tile by TMA), so q itself is not modified unless it aliases o; the K rows in
 * the cache must already be rotated (use rd_kv_append with pos). gate != NULL multiplies
 * the output by sigmoid(gate); the gate buffer is read only. q, o and gate must be 16-byte
 * aligned. */
int rd_attn_prefill_fused(const float *q, const void *k, const void *v, float *o, const float *gate,
                          const int32_t *pos, int n_q, int keys_total, int n_head, int n_head_kv,
                          int head_dim, float scale, int n_rot, float freq_base, void *stream);

/* The chunk's cache append fused in as well (f16 caches): rd_kv_append(k_new, v_new -> rows
 * row0 .. row0 + n_q - 1, K rotated by pos[] when n_rot > 0; kv_store_row_launch,
 * include/rdna4/kv.h:673-694, + rope_launch on k) and rd_attn_prefill_fused in one call. The
 * pre-pass that rotates the queries stores the new rows too -- the (cos, sin) of a token
 * are computed once for its 24 query and 4 key rows -- and writes the bytes rd_kv_append
 * writes. k_new / v_new are [n_q][n_head_kv][head_dim] f32, 16-byte aligned;
 * row0 + n_q <= keys_total. */
int rd_attn_prefill_append_fused(const float *q, const float *k_new, const float *v_new, void *k, void *v,
                                 float *o, const float *gate, const int32_t *pos, int n_q, int row0,
                                 int keys_total, int n_head, int n_head_kv, int head_dim, float scale,
                                 int n_rot, float freq_base, void *stream);

/* ---- causal prefill over caches of ANY type pair on the tensor cores: what the reference
 * serves with its chunk path, attn_split_batch_launch (include/rdna4/attn.cuh:958-1049, all
 * 6 x 6 K x V types; dispatch src/graph.cuh:1486-1527), where every one of the n_q tokens
 * re-streams and re-expands its prefix. Here the caches that are not f16 are expanded ONCE
 * into `workspace` (rd_attn_prefill_workspace_bytes, which also covers the rotated f16
 * queries of a call with n_rot > 0 and the records of the key split) with the exact values of the reference's dequantizing loads
 * (kv.h:174-368) rounded to f16, and the tcgen05 prefill kernel runs over that copy. Arguments as rd_attn_prefill_fused; token i attends
 * keys 0..pos[i], keys_total rows must exist. No allocation, no host synchronisation. */
size_t rd_attn_prefill_workspace_bytes(int k_type, int v_type, int n_q, int keys_total, int n_head,
                                       int n_head_kv, int head_dim);
int rd_attn_prefill_typed(const float *q, const void *k, const void *v, float *o, const float *gate,
                          const int32_t *pos, int n_q, int keys_total, int n_head, int n_head_kv,
                          int head_dim, float scale, int k_type, int v_type, int n_rot, float freq_base,
                          void *workspace, size_t workspace_bytes, void *stream);

/* ---- device status: 0, or RD_ERR_DEVICE if any kernel launched through this
 * library on the current device gave up on a bounded wait since the last call.
 * Synchronises the device; meant for tests and debugging, not for the hot path. */
int rd_device_status(void);
/* Which wait gave up, for the last RD_ERR_DEVICE that rd_device_status returned: a small
 * site number from the kernel sources (prefill 11-23, decode 1-9 and 90, exchange 100 +
 * rank); 0 if none was ever reported. For bug reports. */
int rd_device_timeout_site(void);

/* Library identification ("rd_attn_b200 <version> sm_100a"). */
const char *rd_version(void);

#ifdef __cplusplus
}
#endif
#endif /* RD_ATTN_H */
