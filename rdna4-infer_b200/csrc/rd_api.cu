// extern "C" entry points: argument validation, split planning, per-device workspace.
#include <algorithm>
#include <mutex>
#include <vector>
#include <string.h>

#include "rd_common.cuh"
#include "rd_internal.h"

namespace {

using namespace rd;

constexpr int kMaxDevices = 32;

struct DeviceState {
  int sms = 0;
  DeviceStatus *status = nullptr;  // sticky status word
  void *ws = nullptr;              // grown on demand by the allocating entry points
  size_t ws_bytes = 0;
};
DeviceState g_dev[kMaxDevices];
std::mutex g_mu;

int current_device(int *dev) {
  if (cudaGetDevice(dev) != cudaSuccess) return RD_ERR_CUDA;
  if (*dev < 0 || *dev >= kMaxDevices) return RD_ERR_UNSUPPORTED;
  return RD_OK;
}

int sm_count(int dev) {
  std::lock_guard<std::mutex> lk(g_mu);
  if (g_dev[dev].sms == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0)
      n = 148;
    g_dev[dev].sms = n;
  }
  return g_dev[dev].sms;
}

// Status word of the bounded waits: part of the library image (zero-initialised when the
// module is loaded on a device), so every entry point has one without allocating -- also
// under stream capture and on a process's very first call. In host code the symbol's name
// is only a stand-in; its device address is looked up once per device.
static __device__ __align__(256) DeviceStatus g_status_word;

DeviceStatus *status_word(int dev) {
  std::lock_guard<std::mutex> lk(g_mu);
  if (g_dev[dev].status == nullptr) {
    void *p = nullptr;
    if (cudaGetSymbolAddress(&p, g_status_word) == cudaSuccess) g_dev[dev].status = (DeviceStatus *)p;
  }
  return g_dev[dev].status;
}

void *ensure_workspace(int dev, size_t bytes) {
  std::lock_guard<std::mutex> lk(g_mu);
  DeviceState &d = g_dev[dev];
  if (d.ws_bytes >= bytes) return d.ws;
  if (d.ws != nullptr) cudaFree(d.ws);  // synchronises with work still using it
  d.ws = nullptr;
  d.ws_bytes = 0;
  const size_t want = (bytes + (size_t)(1 << 20) - 1) & ~(size_t)((1 << 20) - 1);
  if (cudaMalloc(&d.ws, want) != cudaSuccess) {
    d.ws = nullptr;
    return nullptr;
  }
  d.ws_bytes = want;
  return d.ws;
}

bool known_type(int t) { return t >= RD_KV_F32 && t <= RD_KV_Q4_1; }
bool aligned(const void *p, size_t a) { return ((uintptr_t)p & (a - 1)) == 0; }

// Shape gate shared by every attention entry point.
int check_attn_shape(int n_head, int n_head_kv, int head_dim, int kt, int vt) {
  if (!known_type(kt) || !known_type(vt)) return RD_ERR_TYPE;
  if (head_dim <= 0 || head_dim % 32 != 0 || head_dim > 512) return RD_ERR_SHAPE;
  if (n_head <= 0 || n_head_kv <= 0 || n_head % n_head_kv != 0) return RD_ERR_SHAPE;
  if (head_dim != kHeadDim || n_head / n_head_kv != kGroup) return RD_ERR_UNSUPPORTED;
  if (n_head_kv != 1 && n_head_kv != 2 && n_head_kv != 4) return RD_ERR_UNSUPPORTED;
  return RD_OK;
}

// Internal split count: about one CTA per SM over the whole launch, never more
// splits than key tiles (when the key count is known on the host).
int plan_splits(int sms, int n_tok, int64_t tiles_known) {
  int s = sms / (n_tok > 0 ? n_tok : 1);
  if (s < 1) s = 1;
  if (tiles_known >= 0 && s > tiles_known) s = tiles_known > 0 ? (int)tiles_known : 1;
  return s;
}

size_t partial_floats(int n_tok, int n_head, int splits) {
  return (size_t)n_tok * n_head * splits * kRec;
}

// Core: attention of n_tok tokens over keys key_begin..(pos ? pos[i] : t).
//   out != null: merged (and optionally gated) output;
//   out == null: exactly n_rec records per (token, head) into `records`.
int attn_core(const float *q, const void *k, const void *v, float *out, float *records, int n_rec,
              const int32_t *pos, int t, int key_begin, int n_tok, int n_head, int n_head_kv,
              float scale, int kt, int vt, float *gate, void *ws, size_t ws_bytes,
              DeviceStatus *status, int sms, cudaStream_t st) {
  const int tile = decode_tile_keys(kt, vt);
  int64_t tiles = -1;
  if (pos == nullptr) {
    const int64_t n_keys = t >= key_begin ? (int64_t)t - key_begin + 1 : 0;
    tiles = (n_keys + tile - 1) / tile;
  }
  int S = plan_splits(sms, n_tok, tiles);
  if (out == nullptr) {
    // nest the internal splits inside the caller's: S = n_rec * r
    int r = S / n_rec;
    if (r < 1) r = 1;
    S = n_rec * r;
  }
  DecodeArgs a;
  a.q = q;
  a.k = k;
  a.v = v;
  a.pos = pos;
  a.t = t;
  a.key_begin = key_begin;
  a.n_tok = n_tok;
  a.n_head = n_head;
  a.n_head_kv = n_head_kv;
  a.scale = scale;
  a.n_splits = S;
  a.status = status;
  if (out == nullptr && S == n_rec) {
    a.partial = records;
    return launch_decode(kt, vt, a, st);
  }
  const size_t need = partial_floats(n_tok, n_head, S) * sizeof(float);
  if (ws == nullptr || ws_bytes < need) return RD_ERR_WORKSPACE;
  a.partial = (float *)ws;
  int rc = launch_decode(kt, vt, a, st);
  if (rc != RD_OK) return rc;
  if (out != nullptr) return launch_merge((const float *)ws, out, n_tok * n_head, S, gate, st);
  return launch_merge_records((const float *)ws, records, n_tok * n_head, S, n_rec, st);
}

size_t workspace_bytes_for(int sms, int n_tok, int n_head) {
  // the largest split count attn_core can pick for this token count, plus slack for
  // the "nest inside the caller's splits" rounding
  const int s = plan_splits(sms, n_tok, -1);
  return partial_floats(n_tok, n_head, s) * sizeof(float) + 256;
}

// Allocating flavour used by the reference-shaped launchers.
int attn_alloc(const float *q, const void *k, const void *v, float *out, float *records, int n_rec,
               const int32_t *pos, int t, int n_tok, int n_head, int n_head_kv, int head_dim,
               float scale, int kt, int vt, void *stream) {
  int rc = check_attn_shape(n_head, n_head_kv, head_dim, kt, vt);
  if (rc != RD_OK) return rc;
  if (q == nullptr || k == nullptr || v == nullptr) return RD_ERR_NULL;
  if (out == nullptr && records == nullptr) return RD_ERR_NULL;
  if (n_tok < 1 || n_rec < 1) return RD_ERR_SHAPE;
  if (!aligned(q, 4) || !aligned(out, 4) || !aligned(records, 4)) return RD_ERR_ALIGN;
  if (!aligned(k, 16) || !aligned(v, 16)) return RD_ERR_ALIGN;
  int dev;
  if ((rc = current_device(&dev)) != RD_OK) return rc;
  DeviceStatus *status = status_word(dev);   // every launch reports its bounded waits
  if (status == nullptr) return RD_ERR_CUDA;
  const int sms = sm_count(dev);
  size_t bytes = workspace_bytes_for(sms, n_tok, n_head);
  if (out == nullptr) {
    const size_t nested = partial_floats(n_tok, n_head, sms + n_rec) * sizeof(float);
    if (nested > bytes) bytes = nested;
  }
  void *ws = ensure_workspace(dev, bytes);
  if (ws == nullptr) return RD_ERR_WORKSPACE;
  return attn_core(q, k, v, out, records, n_rec, pos, t, 0, n_tok, n_head, n_head_kv, scale, kt, vt,
                   nullptr, ws, bytes, status, sms, (cudaStream_t)stream);
}

// ---- allocation-free decode (rd_attn_decode_noalloc) --------------------------------
// Partial records of the allocation-free entry point: part of the library image, so no
// call ever has to allocate them. In host code the array's NAME is only a host-side
// stand-in -- handing it to a kernel would pass a host address -- so the device address
// is looked up once per device with cudaGetSymbolAddress and cached.
constexpr size_t kNoAllocFloats =
    (size_t)RD_NOALLOC_MAX_HEADS * RD_NOALLOC_MAX_SPLITS * kRec;
static __device__ __align__(256) float g_noalloc_records[kNoAllocFloats];
float *g_noalloc_ptr[kMaxDevices] = {};

// Device address of the record array on the current device (dev); nullptr on failure.
float *noalloc_records(int dev) {
  std::lock_guard<std::mutex> lk(g_mu);
  if (g_noalloc_ptr[dev] == nullptr) {
    void *p = nullptr;
    if (cudaGetSymbolAddress(&p, g_noalloc_records) != cudaSuccess) return nullptr;
    g_noalloc_ptr[dev] = (float *)p;
  }
  return g_noalloc_ptr[dev];
}

}  // namespace

extern "C" {

const char *rd_version(void) { return "rd_attn_b200 0.1 sm_100a"; }

const char *rd_strerror(int code) {
  switch (code) {
    case RD_OK: return "ok";
    case RD_ERR_TYPE: return "KV type outside the enum";
    case RD_ERR_SHAPE: return "bad shape or size";
    case RD_ERR_UNSUPPORTED: return "shape or type not built in this library";
    case RD_ERR_NULL: return "required pointer is NULL";
    case RD_ERR_ALIGN: return "pointer not aligned as required";
    case RD_ERR_CUDA: return "CUDA runtime error";
    case RD_ERR_WORKSPACE: return "workspace missing or too small";
    case RD_ERR_DEVICE: return "a kernel gave up on a bounded wait";
    case RD_ERR_LIMIT: return "size beyond a fixed maximum of the entry point";
  }
  return "unknown error code";
}

const char *rd_kv_type_name(int type) {
  static const char *names[] = {"f32", "f16", "q8_0", "q4_0", "q5_0", "q4_1"};
  return known_type(type) ? names[type] : nullptr;
}

int rd_kv_type_parse(const char *name, int *out_type) {
  if (name == nullptr || out_type == nullptr) return RD_ERR_NULL;
  for (int t = RD_KV_F32; t <= RD_KV_Q4_1; ++t) {
    if (strcmp(name, rd_kv_type_name(t)) == 0) {
      *out_type = t;
      return RD_OK;
    }
  }
  return RD_ERR_TYPE;
}

double rd_kv_bytes_per_elem(int type) {
  switch (type) {
    case RD_KV_F32: return 4.0;
    case RD_KV_F16: return 2.0;
    case RD_KV_Q8_0: return 34.0 / 32.0;
    case RD_KV_Q4_0: return 18.0 / 32.0;
    case RD_KV_Q5_0: return 22.0 / 32.0;
    case RD_KV_Q4_1: return 20.0 / 32.0;
  }
  return 0.0;
}

uint64_t rd_kv_row_bytes(int type, int head_dim) {
  if (head_dim < 0) return 0;
  const uint64_t blocks = (uint64_t)(head_dim + 31) / 32;
  switch (type) {
    case RD_KV_F32: return (uint64_t)head_dim * 4;
    case RD_KV_F16: return (uint64_t)head_dim * 2;
    case RD_KV_Q8_0: return blocks * 34;
    case RD_KV_Q4_0: return blocks * 18;
    case RD_KV_Q5_0: return blocks * 22;
    case RD_KV_Q4_1: return blocks * 20;
  }
  return 0;
}

int rd_kv_store_rows(int type, const float *src, void *dst, int64_t width, void *stream) {
  if (!known_type(type)) return RD_ERR_TYPE;
  if (width < 0 || width % 32 != 0) return RD_ERR_SHAPE;
  if (width == 0) return RD_OK;
  if (src == nullptr || dst == nullptr) return RD_ERR_NULL;
  if (!aligned(src, 4) || !aligned(dst, type == RD_KV_F32 ? 4 : 2)) return RD_ERR_ALIGN;
  return launch_kv_append(type, type, src, nullptr, dst, nullptr, width, kHeadDim, 1, nullptr, 0,
                          0.f, (cudaStream_t)stream);
}

int rd_kv_append(int k_type, int v_type, const float *k_src, const float *v_src, void *k_dst,
                 void *v_dst, int n_tok, int n_head_kv, int head_dim, const int32_t *pos, int n_rot,
                 float freq_base, void *stream) {
  if (!known_type(k_type) || !known_type(v_type)) return RD_ERR_TYPE;
  if (n_tok < 0 || n_head_kv < 1 || head_dim < 32 || head_dim % 32 != 0) return RD_ERR_SHAPE;
  if (pos != nullptr && (n_rot < 2 || n_rot % 2 != 0 || n_rot > head_dim)) return RD_ERR_SHAPE;
  if (pos != nullptr && n_rot > 512) return RD_ERR_UNSUPPORTED;  // frequency table of 256 pairs
  if (n_tok == 0) return RD_OK;
  if (k_src == nullptr || v_src == nullptr || k_dst == nullptr || v_dst == nullptr)
    return RD_ERR_NULL;
  if (!aligned(k_src, 4) || !aligned(v_src, 4) || !aligned(k_dst, k_type == RD_KV_F32 ? 4 : 2) ||
      !aligned(v_dst, v_type == RD_KV_F32 ? 4 : 2))
    return RD_ERR_ALIGN;
  const int64_t width = (int64_t)n_tok * n_head_kv * head_dim;
  return launch_kv_append(k_type, v_type, k_src, v_src, k_dst, v_dst, width, head_dim, n_head_kv,
                          pos, n_rot, freq_base, (cudaStream_t)stream);
}

int rd_kv_fill(int type, void *cache, int64_t n_rows, int head_dim, uint32_t seed, void *stream) {
  if (!known_type(type)) return RD_ERR_TYPE;
  if (n_rows < 0 || head_dim < 32 || head_dim % 32 != 0) return RD_ERR_SHAPE;
  if (n_rows == 0) return RD_OK;
  if (cache == nullptr) return RD_ERR_NULL;
  if (!aligned(cache, type == RD_KV_F32 ? 4 : 2)) return RD_ERR_ALIGN;
  return launch_kv_fill(type, cache, n_rows, head_dim, seed, (cudaStream_t)stream);
}

int rd_rope(float *x, int n_tok, int n_heads, int head_dim, int n_rot, float freq_base,
            const int32_t *pos, void *stream) {
  if (n_tok < 0 || n_heads < 1 || head_dim < 2 || n_rot < 2 || n_rot % 2 != 0 || n_rot > head_dim)
    return RD_ERR_SHAPE;
  if (n_rot > 512) return RD_ERR_UNSUPPORTED;  // frequency table of 256 pairs
  if (n_tok == 0) return RD_OK;
  if (x == nullptr || pos == nullptr) return RD_ERR_NULL;
  if (!aligned(x, 4) || !aligned(pos, 4)) return RD_ERR_ALIGN;
  return launch_rope(x, n_tok, n_heads, head_dim, n_rot, freq_base, pos, (cudaStream_t)stream);
}

int rd_deinterleave_q_gate(const float *yq, float *q, float *gate, int n_tok, int n_head,
                           int head_dim, void *stream) {
  if (n_tok < 0 || n_head < 1 || head_dim < 4 || head_dim % 4 != 0) return RD_ERR_SHAPE;
  if (n_tok == 0) return RD_OK;
  if (yq == nullptr || q == nullptr || gate == nullptr) return RD_ERR_NULL;
  if (!aligned(yq, 16) || !aligned(q, 16) || !aligned(gate, 16)) return RD_ERR_ALIGN;
  return launch_deinterleave(yq, q, gate, (int64_t)n_tok * n_head, head_dim, (cudaStream_t)stream);
}

int rd_sigmoid_gate(float *g_io, float *y_io, int64_t n, void *stream) {
  if (n < 0) return RD_ERR_SHAPE;
  if (n == 0) return RD_OK;
  if (g_io == nullptr || y_io == nullptr) return RD_ERR_NULL;
  return launch_sigmoid_gate(g_io, y_io, n, (cudaStream_t)stream);
}

int rd_rms_norm(const float *x, const float *w, float *y, int64_t n_rows, int64_t n_cols, float eps,
                void *stream) {
  if (n_rows < 0 || n_cols < 1) return RD_ERR_SHAPE;
  if (n_rows == 0) return RD_OK;
  if (x == nullptr || y == nullptr) return RD_ERR_NULL;
  if (!aligned(x, 4) || !aligned(y, 4) || !aligned(w, 4)) return RD_ERR_ALIGN;
  return launch_rms_norm(x, w, y, n_rows, n_cols, eps, (cudaStream_t)stream);
}

int rd_pre_attn_fused(const float *q_gate, const float *k_src, const float *v_src,
                      const float *q_norm_w, const float *k_norm_w, float eps, float *q_out,
                      float *gate_out, void *k_rows, void *v_rows, int k_type, int v_type,
                      const int32_t *pos, int n_tok, int n_head, int n_head_kv, int head_dim,
                      int n_rot, float freq_base, void *stream) {
  if (!known_type(k_type) || !known_type(v_type)) return RD_ERR_TYPE;
  if (n_tok < 0 || n_head < 1 || n_head_kv < 1 || head_dim < 32 || head_dim % 32 != 0)
    return RD_ERR_SHAPE;
  if (n_rot < 0 || n_rot > head_dim) return RD_ERR_SHAPE;
  if (head_dim != kHeadDim || n_rot % 64 != 0) return RD_ERR_UNSUPPORTED;
  if (n_tok == 0) return RD_OK;
  if (q_gate == nullptr || k_src == nullptr || v_src == nullptr || q_out == nullptr ||
      gate_out == nullptr || k_rows == nullptr || v_rows == nullptr || pos == nullptr)
    return RD_ERR_NULL;
  if (!aligned(q_gate, 4) || !aligned(k_src, 4) || !aligned(v_src, 4) || !aligned(q_out, 4) ||
      !aligned(gate_out, 4) || !aligned(q_norm_w, 4) || !aligned(k_norm_w, 4) || !aligned(pos, 4))
    return RD_ERR_ALIGN;
  if (!aligned(k_rows, 4) || !aligned(v_rows, 4)) return RD_ERR_ALIGN;
  return launch_pre_attn(k_type, v_type, q_gate, k_src, v_src, q_norm_w, k_norm_w, eps, q_out,
                         gate_out, k_rows, v_rows, pos, n_tok, n_head, n_head_kv, n_rot, freq_base,
                         (cudaStream_t)stream);
}

int rd_attn_splits_for(int n_keys, int k_type, int v_type, int n_head, int forced) {
  // Graph::attn_splits_for (graph.cuh:495-526) with the constants of tuning.h:144-150
  constexpr int kSplitMin = 512, kMaxSplits = 16, kCtasDense = 96;
  if (!known_type(k_type) || !known_type(v_type)) return RD_ERR_TYPE;
  if (n_keys < 0 || n_head < 1) return RD_ERR_SHAPE;
  if (forced > 0) return forced > kMaxSplits ? kMaxSplits : forced;
  if (n_keys < kSplitMin) return 1;
  const bool dense = (k_type == RD_KV_F16 || k_type == RD_KV_F32) &&
                     (v_type == RD_KV_F16 || v_type == RD_KV_F32);
  int sp = dense ? (kCtasDense + n_head - 1) / n_head : n_keys / kSplitMin;
  if (sp < 1) sp = 1;
  return sp > kMaxSplits ? kMaxSplits : sp;
}

int rd_attn_plan(int n_keys, int n_tok, int n_head_kv, int k_type, int v_type, int sm_count,
                 int *tile_keys, int *ring_stages, int *n_splits) {
  if (!known_type(k_type) || !known_type(v_type)) return RD_ERR_TYPE;
  if (n_keys < 0 || n_tok < 1) return RD_ERR_SHAPE;
  if (n_head_kv != 1 && n_head_kv != 2 && n_head_kv != 4) return RD_ERR_UNSUPPORTED;
  if (sm_count <= 0) {
    int dev;
    const int rc = current_device(&dev);
    if (rc != RD_OK) return rc;
    sm_count = ::sm_count(dev);
  }
  const int tile = decode_tile_keys(k_type, v_type);
  const int stages = ring_depth(k_type, v_type, n_head_kv);
  if (stages < 1) return RD_ERR_UNSUPPORTED;
  const int64_t tiles = ((int64_t)n_keys + tile - 1) / tile;
  if (tile_keys != nullptr) *tile_keys = tile;
  if (ring_stages != nullptr) *ring_stages = stages;
  if (n_splits != nullptr) *n_splits = plan_splits(sm_count, n_tok, tiles);
  return RD_OK;
}

int rd_attn_prefill_plan(int n_q, int keys_total, int n_head, int sm_count, int *n_splits, int *n_ctas) {
  if (n_q < 1 || keys_total < 1 || n_head < 1) return RD_ERR_SHAPE;
  if (sm_count <= 0) {
    int dev;
    const int rc = current_device(&dev);
    if (rc != RD_OK) return rc;
    sm_count = ::sm_count(dev);
  }
  const int z = prefill_splits(n_q, keys_total, n_head, sm_count);
  if (n_splits != nullptr) *n_splits = z;
  if (n_ctas != nullptr) *n_ctas = ((n_q + 127) / 128) * n_head * z;
  return RD_OK;
}

size_t rd_attn_partial_bytes(int n_head, int head_dim, int n_splits) {
  if (n_head < 0 || head_dim < 0 || n_splits < 0) return 0;
  return (size_t)n_head * (size_t)n_splits * (2 + (size_t)head_dim) * sizeof(float);
}

size_t rd_attn_workspace_bytes(int n_tok, int n_head, int head_dim) {
  int dev;
  if (n_tok < 1 || n_head < 1 || head_dim != kHeadDim || current_device(&dev) != RD_OK) return 0;
  const int sms = sm_count(dev);
  // room for the largest nested split count as well (records-only calls)
  return partial_floats(n_tok, n_head, 2 * sms) * sizeof(float) + 256;
}

int rd_attn_decode(const float *q, const void *k, const void *v, float *out, int t, int n_head,
                   int n_head_kv, int head_dim, float scale, int k_type, int v_type,
                   void *stream) {
  if (out == nullptr) return RD_ERR_NULL;
  return attn_alloc(q, k, v, out, nullptr, 1, nullptr, t, 1, n_head, n_head_kv, head_dim, scale,
                    k_type, v_type, stream);
}

int rd_attn_decode_split(const float *q, const void *k, const void *v, float *out, float *partial,
                         int t, int n_head, int n_head_kv, int head_dim, float scale, int k_type,
                         int v_type, int n_splits, void *stream) {
  if (n_splits < 1) return RD_ERR_SHAPE;
  return attn_alloc(q, k, v, out, partial, n_splits, nullptr, t, 1, n_head, n_head_kv, head_dim,
                    scale, k_type, v_type, stream);
}

int rd_attn_decode_ws(const float *q, const void *k, const void *v, float *out, float *partial,
                      int key_begin, int t, int n_head, int n_head_kv, int head_dim, float scale,
                      int k_type, int v_type, int n_splits, float *gate, void *workspace,
                      size_t workspace_bytes, void *stream) {
  int rc = check_attn_shape(n_head, n_head_kv, head_dim, k_type, v_type);
  if (rc != RD_OK) return rc;
  if (n_splits < 1 || key_begin < 0) return RD_ERR_SHAPE;
  if (q == nullptr || k == nullptr || v == nullptr) return RD_ERR_NULL;
  if (out == nullptr && partial == nullptr) return RD_ERR_NULL;
  if (workspace == nullptr) return RD_ERR_WORKSPACE;
  if (!aligned(q, 4) || !aligned(out, 4) || !aligned(partial, 4) || !aligned(gate, 4))
    return RD_ERR_ALIGN;
  if (!aligned(k, 16) || !aligned(v, 16) || !aligned(workspace, 256)) return RD_ERR_ALIGN;
  int dev;
  if ((rc = current_device(&dev)) != RD_OK) return rc;
  DeviceStatus *status = status_word(dev);   // every launch reports its bounded waits
  if (status == nullptr) return RD_ERR_CUDA;
  return attn_core(q, k, v, out, partial, n_splits, nullptr, t, key_begin, 1, n_head, n_head_kv,
                   scale, k_type, v_type, gate, workspace, workspace_bytes, status,
                   sm_count(dev), (cudaStream_t)stream);
}

int rd_attn_decode_append_ws(const float *q, const float *k_new, const float *v_new, void *k_cache,
                             void *v_cache, float *out, int t, int n_head, int n_head_kv, int head_dim,
                             float scale, int k_type, int v_type, float *gate, void *workspace,
                             size_t workspace_bytes, void *stream) {
  int rc = check_attn_shape(n_head, n_head_kv, head_dim, k_type, v_type);
  if (rc != RD_OK) return rc;
  if (t < 0) return RD_ERR_SHAPE;
  if (q == nullptr || k_new == nullptr || v_new == nullptr || k_cache == nullptr ||
      v_cache == nullptr || out == nullptr)
    return RD_ERR_NULL;
  if (q == out) return RD_ERR_UNSUPPORTED;  // the merge reads whole query rows while it writes out
  if (workspace == nullptr) return RD_ERR_WORKSPACE;
  if (!aligned(q, 4) || !aligned(out, 4) || !aligned(gate, 4) || !aligned(k_new, 4) || !aligned(v_new, 4))
    return RD_ERR_ALIGN;
  if (!aligned(k_cache, 16) || !aligned(v_cache, 16) || !aligned(workspace, 256)) return RD_ERR_ALIGN;
  int dev;
  if ((rc = current_device(&dev)) != RD_OK) return rc;
  DeviceStatus *status = status_word(dev);   // every launch reports its bounded waits
  if (status == nullptr) return RD_ERR_CUDA;
  // keys 0..t-1 through the split-KV kernel (whose first CTAs also store row t), then the
  // merge with row t folded in
  const int tile = decode_tile_keys(k_type, v_type);
  const int64_t tiles = ((int64_t)t + tile - 1) / tile;
  const int S = plan_splits(sm_count(dev), 1, tiles);
  if (workspace_bytes < partial_floats(1, n_head, S) * sizeof(float)) return RD_ERR_WORKSPACE;
  DecodeArgs a;
  a.q = q;
  a.k = k_cache;
  a.v = v_cache;
  a.partial = (float *)workspace;
  a.pos = nullptr;
  a.t = t - 1;
  a.key_begin = 0;
  a.n_tok = 1;
  a.n_head = n_head;
  a.n_head_kv = n_head_kv;
  a.scale = scale;
  a.n_splits = S;
  a.status = status;
  a.k_new = k_new;
  a.v_new = v_new;
  a.new_row = t;
  cudaStream_t st = (cudaStream_t)stream;
  if ((rc = launch_decode(k_type, v_type, a, st)) != RD_OK) return rc;
  ExtraKey x;
  x.q = q;
  x.k_row = (const uint8_t *)k_cache + (size_t)t * n_head_kv * row_bytes(k_type);
  x.v_row = (const uint8_t *)v_cache + (size_t)t * n_head_kv * row_bytes(v_type);
  x.kt = k_type;
  x.vt = v_type;
  x.nkv = n_head_kv;
  x.scale = scale;
  return launch_merge_extra((const float *)workspace, out, n_head, S, gate, x, st);
}

int rd_attn_decode_noalloc(const float *q, const void *k, const void *v, float *out, int t,
                           int n_head, int n_head_kv, int head_dim, float scale, int k_type,
                           int v_type, float *gate, void *stream) {
  // the fixed array's own limit first: a size beyond it is refused as such, whatever
  // else the shape check would say about it
  if (n_head > RD_NOALLOC_MAX_HEADS) return RD_ERR_LIMIT;
  int rc = check_attn_shape(n_head, n_head_kv, head_dim, k_type, v_type);
  if (rc != RD_OK) return rc;
  if (q == nullptr || k == nullptr || v == nullptr || out == nullptr) return RD_ERR_NULL;
  if (!aligned(q, 4) || !aligned(out, 4) || !aligned(gate, 4)) return RD_ERR_ALIGN;
  if (!aligned(k, 16) || !aligned(v, 16)) return RD_ERR_ALIGN;
  int dev;
  if ((rc = current_device(&dev)) != RD_OK) return rc;
  DeviceStatus *status = status_word(dev);   // every launch reports its bounded waits
  if (status == nullptr) return RD_ERR_CUDA;
  float *records = noalloc_records(dev);  // first call on this device: address look-up
  if (records == nullptr) return RD_ERR_CUDA;
  // Planning with at most RD_NOALLOC_MAX_SPLITS "SMs" caps the records per head, so the
  // fixed array always holds them: n_head * splits * 258 floats <= kNoAllocFloats.
  int sms = sm_count(dev);
  if (sms > RD_NOALLOC_MAX_SPLITS) sms = RD_NOALLOC_MAX_SPLITS;
  return attn_core(q, k, v, out, nullptr, 1, nullptr, t, 0, 1, n_head, n_head_kv, scale, k_type,
                   v_type, gate, records, kNoAllocFloats * sizeof(float), status,
                   sms, (cudaStream_t)stream);
}

// ---- multi-sequence decode / verify -------------------------------------------------
// Workspace layout: [n_seq descriptors][work items][records]; every part 256-aligned.
static size_t align256(size_t x) { return (x + 255) & ~(size_t)255; }
static int multi_max_items(int sms, int n_seq, int q_len) { return 4 * sms + n_seq * q_len; }

size_t rd_attn_multi_workspace_bytes(int n_seq, int q_len, int n_head, int head_dim) {
  int dev;
  if (n_seq < 1 || q_len < 1 || n_head < 1 || head_dim != kHeadDim ||
      current_device(&dev) != RD_OK)
    return 0;
  const size_t items = (size_t)multi_max_items(sm_count(dev), n_seq, q_len);
  return align256((size_t)n_seq * sizeof(DecodeSeq)) + align256(items * sizeof(int4)) +
         align256(items * (size_t)n_head * kRec * sizeof(float));
}

// Plan of one multi-sequence call, in HOST memory: a header, then exactly the bytes the
// launch copies to the start of the workspace (sequence descriptors with their tensor
// maps, then the work list).
struct MultiPlanHeader {
  uint32_t magic;
  int32_t n_seq, q_len, n_head, n_head_kv, k_type, v_type;
  int32_t n_items, max_items;
  uint64_t off_items, copy_bytes;
};
constexpr uint32_t kMultiPlanMagic = 0x52444d50u;   // "RDMP"
constexpr size_t kMultiPlanHeaderBytes = 256;
static_assert(sizeof(MultiPlanHeader) <= kMultiPlanHeaderBytes, "plan header");

size_t rd_attn_multi_plan_bytes(int n_seq, int q_len) {
  int dev;
  if (n_seq < 1 || q_len < 1 || current_device(&dev) != RD_OK) return 0;
  const size_t items = (size_t)multi_max_items(sm_count(dev), n_seq, q_len);
  return kMultiPlanHeaderBytes + align256((size_t)n_seq * sizeof(DecodeSeq)) + align256(items * sizeof(int4));
}

int rd_attn_multi_plan(const rd_attn_seq *seqs, int n_seq, int q_len, int n_head, int n_head_kv,
                       int head_dim, int k_type, int v_type, int pad_items, void *plan, size_t plan_bytes) {
  int rc = check_attn_shape(n_head, n_head_kv, head_dim, k_type, v_type);
  if (rc != RD_OK) return rc;
  if (n_seq < 1 || q_len < 1 || pad_items < 0) return RD_ERR_SHAPE;
  if (seqs == nullptr || plan == nullptr) return RD_ERR_NULL;
  if (!aligned(plan, 16)) return RD_ERR_ALIGN;
  for (int i = 0; i < n_seq; ++i) {
    const rd_attn_seq &s = seqs[i];
    if (s.q == nullptr || s.k == nullptr || s.v == nullptr || s.out == nullptr) return RD_ERR_NULL;
    if (!aligned(s.q, 16) || !aligned(s.out, 4) || !aligned(s.gate, 4)) return RD_ERR_ALIGN;
    if (!aligned(s.k, 16) || !aligned(s.v, 16)) return RD_ERR_ALIGN;
    if (s.t < q_len - 1) return RD_ERR_SHAPE;  // every new token needs at least its own key
  }
  int dev;
  if ((rc = current_device(&dev)) != RD_OK) return rc;
  const int sms = sm_count(dev);
  const int max_items = multi_max_items(sms, n_seq, q_len);
  const size_t off_items = align256((size_t)n_seq * sizeof(DecodeSeq));
  if (plan_bytes < kMultiPlanHeaderBytes + off_items + align256((size_t)max_items * sizeof(int4)))
    return RD_ERR_WORKSPACE;
  if (pad_items > max_items) return RD_ERR_LIMIT;

  // Key split: chunks of equal length over all sequences, about four CTAs per SM in
  // total, so that a 32k-key sequence and a 1k-key one load the SMs evenly.
  const int tile = decode_tile_keys(k_type, v_type);
  std::vector<int> tiles(n_seq);
  int64_t total = 0;
  for (int i = 0; i < n_seq; ++i) {
    tiles[i] = (seqs[i].t + tile) / tile;  // ceil((t + 1) / tile)
    total += (int64_t)tiles[i] * q_len;
  }
  int64_t chunk = (total + 4 * sms - 1) / (4 * sms);
  if (chunk < 4) chunk = 4;
  unsigned char *body = (unsigned char *)plan + kMultiPlanHeaderBytes;
  DecodeSeq *hs = reinterpret_cast<DecodeSeq *>(body);
  int4 *hi = reinterpret_cast<int4 *>(body + off_items);
  std::vector<int> order(n_seq);
  for (int i = 0; i < n_seq; ++i) order[i] = i;
  std::stable_sort(order.begin(), order.end(), [&](int a, int b) { return tiles[a] > tiles[b]; });
  int64_t rec_base = 0;
  int n_items = 0;
  for (int i = 0; i < n_seq; ++i) {
    DecodeSeq &d = hs[i];
    memset(&d, 0, sizeof(d));
    d.q = seqs[i].q;
    d.k = (const uint8_t *)seqs[i].k;
    d.v = (const uint8_t *)seqs[i].v;
    d.out = seqs[i].out;
    d.gate = seqs[i].gate;
    d.t = seqs[i].t;
    int ns = (int)((tiles[i] + chunk - 1) / chunk);
    d.n_splits = ns < 1 ? 1 : ns;
    d.rec_base = (int)rec_base;
    rec_base += (int64_t)d.n_splits * q_len * n_head;
  }
  for (int oi = 0; oi < n_seq; ++oi) {  // longest sequences first
    const int i = order[oi];
    for (int sp = 0; sp < hs[i].n_splits; ++sp)
      for (int tok = 0; tok < q_len; ++tok) {
        if (n_items >= max_items) return RD_ERR_WORKSPACE;  // cannot happen by the bound above
        hi[n_items++] = make_int4(i, tok, sp, 0);
      }
  }
  // a fixed item count keeps the grid of a captured launch valid while the contexts grow:
  // the padding items name no sequence and their CTAs leave at once
  if (pad_items > 0) {
    if (n_items > pad_items) return RD_ERR_LIMIT;
    while (n_items < pad_items) hi[n_items++] = make_int4(-1, 0, 0, 0);
  }
  MultiDecodeArgs a;   // host pass: the tensor maps of every sequence, into its descriptor
  memset(&a, 0, sizeof(a));
  a.host_seqs = hs;
  a.n_seq = n_seq;
  a.n_head_kv = n_head_kv;
  if ((rc = launch_decode_multi(k_type, v_type, a, nullptr)) != RD_OK) return rc;
  MultiPlanHeader h;
  memset(&h, 0, sizeof(h));
  h.magic = kMultiPlanMagic;
  h.n_seq = n_seq;
  h.q_len = q_len;
  h.n_head = n_head;
  h.n_head_kv = n_head_kv;
  h.k_type = k_type;
  h.v_type = v_type;
  h.n_items = n_items;
  h.max_items = max_items;
  h.off_items = off_items;
  h.copy_bytes = off_items + (size_t)n_items * sizeof(int4);
  memcpy(plan, &h, sizeof(h));
  return RD_OK;
}

int rd_attn_multi_launch(const void *plan, float scale, void *workspace, size_t workspace_bytes, void *stream) {
  if (plan == nullptr) return RD_ERR_NULL;
  MultiPlanHeader h;
  memcpy(&h, plan, sizeof(h));
  if (h.magic != kMultiPlanMagic || h.n_seq < 1 || h.q_len < 1 || h.n_items < 1 || h.n_items > h.max_items ||
      h.off_items != align256((size_t)h.n_seq * sizeof(DecodeSeq)) ||
      h.copy_bytes != h.off_items + (size_t)h.n_items * sizeof(int4) ||
      check_attn_shape(h.n_head, h.n_head_kv, kHeadDim, h.k_type, h.v_type) != RD_OK)
    return RD_ERR_SHAPE;   // not a plan of rd_attn_multi_plan, or damaged
  if (workspace == nullptr) return RD_ERR_WORKSPACE;
  if (!aligned(workspace, 256)) return RD_ERR_ALIGN;
  int dev, rc;
  if ((rc = current_device(&dev)) != RD_OK) return rc;
  DeviceStatus *status = status_word(dev);   // every launch reports its bounded waits
  if (status == nullptr) return RD_ERR_CUDA;
  const size_t off_rec = h.off_items + align256((size_t)h.max_items * sizeof(int4));
  const size_t need = off_rec + align256((size_t)h.max_items * h.n_head * kRec * sizeof(float));
  if (workspace_bytes < need) return RD_ERR_WORKSPACE;
  // From pageable memory the copy has left the plan when cudaMemcpyAsync returns; from
  // pinned memory it reads the plan when the stream (or a replayed graph) reaches it.
  if (cudaMemcpyAsync(workspace, (const unsigned char *)plan + kMultiPlanHeaderBytes, h.copy_bytes,
                      cudaMemcpyHostToDevice, (cudaStream_t)stream) != cudaSuccess)
    return RD_ERR_CUDA;
  MultiDecodeArgs a;
  memset(&a, 0, sizeof(a));
  a.n_seq = h.n_seq;
  a.n_head_kv = h.n_head_kv;
  a.dev_seqs = reinterpret_cast<const DecodeSeq *>(workspace);
  a.dev_items = reinterpret_cast<const int4 *>((const unsigned char *)workspace + h.off_items);
  a.n_items = h.n_items;
  a.q_len = h.q_len;
  a.n_head = h.n_head;
  a.scale = scale;
  a.records = reinterpret_cast<float *>((unsigned char *)workspace + off_rec);
  a.status = status;
  if ((rc = launch_decode_multi(h.k_type, h.v_type, a, (cudaStream_t)stream)) != RD_OK) return rc;
  return launch_merge_multi(a.dev_seqs, a.records, h.n_seq, h.q_len, h.n_head, (cudaStream_t)stream);
}

int rd_attn_decode_multi(const rd_attn_seq *seqs, int n_seq, int q_len, int n_head, int n_head_kv,
                         int head_dim, float scale, int k_type, int v_type, void *workspace,
                         size_t workspace_bytes, void *stream) {
  if (n_seq < 0 || q_len < 1) {
    const int rc = check_attn_shape(n_head, n_head_kv, head_dim, k_type, v_type);
    return rc != RD_OK ? rc : RD_ERR_SHAPE;
  }
  if (n_seq == 0) return check_attn_shape(n_head, n_head_kv, head_dim, k_type, v_type);
  const size_t plan_bytes = rd_attn_multi_plan_bytes(n_seq, q_len);
  if (plan_bytes == 0) return RD_ERR_CUDA;
  // 16-byte aligned pageable plan of this call
  std::vector<uint4> plan((plan_bytes + sizeof(uint4) - 1) / sizeof(uint4));
  int rc = rd_attn_multi_plan(seqs, n_seq, q_len, n_head, n_head_kv, head_dim, k_type, v_type, 0, plan.data(),
                              plan_bytes);
  if (rc != RD_OK) return rc;
  return rd_attn_multi_launch(plan.data(), scale, workspace, workspace_bytes, stream);
}

// ---- context-sharded decode with the exchange fused into the merge -------------------
size_t rd_shard_xbuf_bytes(int n_head, int head_dim, int world) {
  if (n_head < 1 || n_head > kShardMaxHeads || head_dim != kHeadDim || world < 1 ||
      world > kShardMaxWorld)
    return 0;
  return align256(kShardHeaderBytes + (size_t)2 * world * n_head * 4 * kXPart * 8);
}

// Validates a group and converts it; RD_OK or an error.
static int shard_peers(const rd_shard_group *group, ShardPeers *g) {
  if (group == nullptr || group->xbuf == nullptr) return RD_ERR_NULL;
  if (group->world < 1 || group->world > kShardMaxWorld || group->rank < 0 ||
      group->rank >= group->world)
    return RD_ERR_SHAPE;
  memset(g, 0, sizeof(*g));
  for (int r = 0; r < group->world; ++r) {
    if (group->xbuf[r] == nullptr) return RD_ERR_NULL;
    if (!aligned(group->xbuf[r], 256)) return RD_ERR_ALIGN;
    g->x[r] = (unsigned char *)group->xbuf[r];
  }
  g->rank = group->rank;
  g->world = group->world;
  g->wait_ns = 1000ull * (group->wait_limit_us != 0 ? group->wait_limit_us : 1000000u);
  return RD_OK;
}

int rd_attn_shard_push(const float *partial, int n_splits, int n_head, int head_dim,
                       const rd_shard_group *group, void *stream) {
  if (n_head < 1 || n_splits < 1) return RD_ERR_SHAPE;
  if (head_dim != kHeadDim) return RD_ERR_UNSUPPORTED;
  if (n_head > kShardMaxHeads) return RD_ERR_LIMIT;
  if (partial == nullptr) return RD_ERR_NULL;
  if (!aligned(partial, 4)) return RD_ERR_ALIGN;
  ShardPeers g;
  const int rc = shard_peers(group, &g);
  if (rc != RD_OK) return rc;
  return launch_shard_push(partial, n_splits, n_head, g, (cudaStream_t)stream);
}

int rd_attn_shard_merge(float *out, float *gate, int n_head, int head_dim,
                        const rd_shard_group *group, void *stream) {
  if (n_head < 1) return RD_ERR_SHAPE;
  if (head_dim != kHeadDim) return RD_ERR_UNSUPPORTED;
  if (n_head > kShardMaxHeads) return RD_ERR_LIMIT;
  if (out == nullptr) return RD_ERR_NULL;
  if (!aligned(out, 4) || !aligned(gate, 4)) return RD_ERR_ALIGN;
  ShardPeers g;
  int rc = shard_peers(group, &g);
  if (rc != RD_OK) return rc;
  int dev;
  if ((rc = current_device(&dev)) != RD_OK) return rc;
  DeviceStatus *status = status_word(dev);   // every launch reports its bounded waits
  if (status == nullptr) return RD_ERR_CUDA;
  return launch_shard_merge(out, gate, n_head, g, status, (cudaStream_t)stream);
}

// k_new / v_new != NULL: the rank that owns the newest position; row t of its slice is
// stored by the same launch and joins the exchange as one more record.
static int decode_sharded(const float *q, const float *k_new, const float *v_new, const void *k, const void *v,
                          float *out, int t, int n_head, int n_head_kv, int head_dim, float scale, int k_type,
                          int v_type, float *gate, void *workspace, size_t workspace_bytes,
                          const rd_shard_group *group, void *stream);

int rd_attn_decode_sharded(const float *q, const void *k, const void *v, float *out, int t,
                           int n_head, int n_head_kv, int head_dim, float scale, int k_type,
                           int v_type, float *gate, void *workspace, size_t workspace_bytes,
                           const rd_shard_group *group, void *stream) {
  return decode_sharded(q, nullptr, nullptr, k, v, out, t, n_head, n_head_kv, head_dim, scale, k_type, v_type,
                        gate, workspace, workspace_bytes, group, stream);
}

int rd_attn_decode_sharded_append(const float *q, const float *k_new, const float *v_new, void *k, void *v,
                                  float *out, int t, int n_head, int n_head_kv, int head_dim, float scale,
                                  int k_type, int v_type, float *gate, void *workspace,
                                  size_t workspace_bytes, const rd_shard_group *group, void *stream) {
  if (k_new == nullptr || v_new == nullptr) return RD_ERR_NULL;
  if (t < 0) return RD_ERR_SHAPE;
  if (q == out) return RD_ERR_UNSUPPORTED;   // the exchange reads whole query rows while it writes out
  if (!aligned(k_new, 4) || !aligned(v_new, 4)) return RD_ERR_ALIGN;
  return decode_sharded(q, k_new, v_new, k, v, out, t, n_head, n_head_kv, head_dim, scale, k_type, v_type, gate,
                        workspace, workspace_bytes, group, stream);
}

static int decode_sharded(const float *q, const float *k_new, const float *v_new, const void *k, const void *v,
                          float *out, int t, int n_head, int n_head_kv, int head_dim, float scale, int k_type,
                          int v_type, float *gate, void *workspace, size_t workspace_bytes,
                          const rd_shard_group *group, void *stream) {
  int rc = check_attn_shape(n_head, n_head_kv, head_dim, k_type, v_type);
  if (rc != RD_OK) return rc;
  if (q == nullptr || k == nullptr || v == nullptr || out == nullptr) return RD_ERR_NULL;
  if (t < -1) return RD_ERR_SHAPE;
  ShardPeers g;
  if ((rc = shard_peers(group, &g)) != RD_OK) return rc;
  if (workspace == nullptr) return RD_ERR_WORKSPACE;
  if (!aligned(q, 4) || !aligned(out, 4) || !aligned(gate, 4)) return RD_ERR_ALIGN;
  if (!aligned(k, 16) || !aligned(v, 16) || !aligned(workspace, 256)) return RD_ERR_ALIGN;
  int dev;
  if ((rc = current_device(&dev)) != RD_OK) return rc;
  DeviceStatus *status = status_word(dev);   // every launch reports its bounded waits
  if (status == nullptr) return RD_ERR_CUDA;
  // with a fused append the split-KV loop attends keys 0..t-1; row t joins in the exchange
  const int t_loop = k_new != nullptr ? t - 1 : t;
  const int tile = decode_tile_keys(k_type, v_type);
  const int64_t tiles = ((int64_t)t_loop + tile) / tile;  // ceil((t_loop + 1) / tile); 0 for an empty slice
  // The exchange runs as n_head * 4 roles on the launch's first CTAs: a short slice still
  // gets that many CTAs (the ones without keys write empty records) instead of a few CTAs
  // walking the roles one after another.
  int S = plan_splits(sm_count(dev), 1, tiles);
  const int roles = std::min(n_head * (head_dim / 64), sm_count(dev));
  if (S < roles) S = roles;
  if (workspace_bytes < partial_floats(1, n_head, S) * sizeof(float)) return RD_ERR_WORKSPACE;
  DecodeArgs a;
  a.q = q;
  a.k = k;
  a.v = v;
  a.partial = (float *)workspace;
  a.pos = nullptr;
  a.t = t_loop;
  a.k_new = k_new;
  a.v_new = v_new;
  a.new_row = t;
  a.key_begin = 0;
  a.n_tok = 1;
  a.n_head = n_head;
  a.n_head_kv = n_head_kv;
  a.scale = scale;
  a.n_splits = S;
  a.status = status;
  a.push = &g;   // the decode launch runs the whole exchange in its epilogue
  a.push_out = out;
  a.push_gate = gate;
  return launch_decode(k_type, v_type, a, (cudaStream_t)stream);
}

int rd_attn_merge(const float *partial, float *out, int n_rows, int head_dim, int n_splits,
                  float *gate, void *stream) {
  if (n_rows < 0 || n_splits < 1) return RD_ERR_SHAPE;
  if (head_dim != kHeadDim) return head_dim > 0 && head_dim % 32 == 0 ? RD_ERR_UNSUPPORTED
                                                                      : RD_ERR_SHAPE;
  if (n_rows == 0) return RD_OK;
  if (partial == nullptr || out == nullptr) return RD_ERR_NULL;
  if (!aligned(partial, 4) || !aligned(out, 4) || !aligned(gate, 4)) return RD_ERR_ALIGN;
  return launch_merge(partial, out, n_rows, n_splits, gate, (cudaStream_t)stream);
}

int rd_attn_batch(const float *q, const void *k, const void *v, float *out, const int32_t *pos,
                  int n_tok, int n_head, int n_head_kv, int head_dim, float scale, int k_type,
                  int v_type, void *stream) {
  if (out == nullptr || pos == nullptr) return RD_ERR_NULL;
  return attn_alloc(q, k, v, out, nullptr, 1, pos, 0, n_tok, n_head, n_head_kv, head_dim, scale,
                    k_type, v_type, stream);
}

int rd_attn_split_batch(const float *q, const void *k, const void *v, float *out, float *partial,
                        const int32_t *pos, int n_tok, int n_head, int n_head_kv, int head_dim,
                        float scale, int k_type, int v_type, int n_splits, void *stream) {
  if (n_splits < 1 || n_tok < 1) return RD_ERR_SHAPE;
  if (pos == nullptr) return RD_ERR_NULL;
  return attn_alloc(q, k, v, out, partial, n_splits, pos, 0, n_tok, n_head, n_head_kv, head_dim,
                    scale, k_type, v_type, stream);
}

int rd_fa2_prefill_usable(int k_type, int v_type, int n_q, int pos0, int n_head, int n_head_kv,
                          int head_dim) {
  if (k_type != RD_KV_F16 || v_type != RD_KV_F16) return 0;
  if (n_q < 1 || pos0 < 0) return 0;
  return check_attn_shape(n_head, n_head_kv, head_dim, k_type, v_type) == RD_OK ? 1 : 0;
}

// records / record_bytes: caller memory for the key-split records, or NULL: the library's
// own grown workspace is used then (see the note on allocating launchers in rd_attn.h).
static int prefill_common(const float *q, const void *k, const void *v, float *o, const float *gate,
                          const int32_t *pos, int n_q, int keys_total, int n_head, int n_head_kv,
                          int head_dim, float scale, int n_rot, float freq_base, void *stream,
                          void *records = nullptr, size_t record_bytes = 0, const float *k_new = nullptr,
                          const float *v_new = nullptr, int row0 = 0) {
  int rc = check_attn_shape(n_head, n_head_kv, head_dim, RD_KV_F16, RD_KV_F16);
  if (rc != RD_OK) return rc;
  if (n_q < 1 || keys_total <= 0) return RD_ERR_SHAPE;
  if (n_rot < 0 || n_rot % 16 != 0 || n_rot > 64) return RD_ERR_SHAPE;
  if (q == nullptr || k == nullptr || v == nullptr || o == nullptr || pos == nullptr) return RD_ERR_NULL;
  if (!aligned(q, 16) || !aligned(o, 16) || !aligned(gate, 16) || !aligned(pos, 4)) return RD_ERR_ALIGN;
  if (!aligned(k, 16) || !aligned(v, 16)) return RD_ERR_ALIGN;
  int dev;
  if ((rc = current_device(&dev)) != RD_OK) return rc;
  DeviceStatus *status = status_word(dev);   // every launch reports its bounded waits
  if (status == nullptr) return RD_ERR_CUDA;
  // scratch: [rotated f16 queries, if the call rotates][key-split records, if any]
  int splits = prefill_splits(n_q, keys_total, n_head, sm_count(dev));
  const size_t rope_need = (n_rot > 0 || k_new != nullptr) ? align256(prefill_rope_bytes(n_q, n_head)) : 0;
  const size_t need = prefill_record_bytes(n_q, n_head, splits);
  if (records == nullptr && rope_need + (splits > 1 ? need : 0) > 0) {
    records = ensure_workspace(dev, rope_need + need);
    record_bytes = records != nullptr ? rope_need + need : 0;
  }
  if (record_bytes < rope_need) return records == nullptr ? RD_ERR_CUDA : RD_ERR_WORKSPACE;
  void *rope_cs = rope_need > 0 ? records : nullptr;
  float *recs = (float *)((unsigned char *)records + rope_need);
  if (splits > 1 && record_bytes - rope_need < need) splits = 1;   // no room: one CTA per (token tile, head) walks all keys
  // a fused append stores rows row0 .. row0 + n_q - 1 of the (f16) caches
  const size_t row_bytes = (size_t)n_head_kv * kHeadDim * 2;
  void *k_dst = k_new != nullptr ? (void *)((unsigned char *)const_cast<void *>(k) + (size_t)row0 * row_bytes) : nullptr;
  void *v_dst = k_new != nullptr ? (void *)((unsigned char *)const_cast<void *>(v) + (size_t)row0 * row_bytes) : nullptr;
  return launch_prefill(q, k, v, o, gate, pos, n_q, keys_total, n_head, n_head_kv, scale, n_rot,
                        freq_base, status, recs, splits, rope_cs, k_new, v_new, k_dst, v_dst,
                        (cudaStream_t)stream);
}

int rd_fa2_prefill(const float *q, const void *k, const void *v, float *o, const int32_t *pos,
                   int n_q, int kmax, int keys_total, int n_head, int n_head_kv, int head_dim,
                   float scale, void *stream) {
  if (kmax < 0) return RD_ERR_SHAPE;
  return prefill_common(q, k, v, o, nullptr, pos, n_q, keys_total, n_head, n_head_kv, head_dim, scale,
                        0, 0.f, stream);
}

int rd_attn_prefill_fused(const float *q, const void *k, const void *v, float *o, const float *gate,
                          const int32_t *pos, int n_q, int keys_total, int n_head, int n_head_kv,
                          int head_dim, float scale, int n_rot, float freq_base, void *stream) {
  return prefill_common(q, k, v, o, gate, pos, n_q, keys_total, n_head, n_head_kv, head_dim, scale,
                        n_rot, freq_base, stream);
}

int rd_attn_prefill_append_fused(const float *q, const float *k_new, const float *v_new, void *k, void *v,
                                 float *o, const float *gate, const int32_t *pos, int n_q, int row0,
                                 int keys_total, int n_head, int n_head_kv, int head_dim, float scale,
                                 int n_rot, float freq_base, void *stream) {
  if (k_new == nullptr || v_new == nullptr) return RD_ERR_NULL;
  if (!aligned(k_new, 16) || !aligned(v_new, 16)) return RD_ERR_ALIGN;
  if (row0 < 0 || n_q < 1 || (int64_t)row0 + n_q > keys_total) return RD_ERR_SHAPE;
  return prefill_common(q, k, v, o, gate, pos, n_q, keys_total, n_head, n_head_kv, head_dim, scale,
                        n_rot, freq_base, stream, nullptr, 0, k_new, v_new, row0);
}

// f16 copies of the caches that are not f16, then the key-split records
static size_t prefill_copy_bytes(int k_type, int v_type, int keys_total, int n_head_kv) {
  const size_t one = align256((size_t)keys_total * n_head_kv * kHeadDim * 2);
  return (k_type != RD_KV_F16 ? one : 0) + (v_type != RD_KV_F16 ? one : 0);
}
size_t rd_attn_prefill_workspace_bytes(int k_type, int v_type, int n_q, int keys_total, int n_head,
                                       int n_head_kv, int head_dim) {
  int dev;
  if (!known_type(k_type) || !known_type(v_type) || n_q < 1 || keys_total <= 0 || n_head < 1 ||
      n_head_kv < 1 || head_dim != kHeadDim || current_device(&dev) != RD_OK)
    return 0;
  return prefill_copy_bytes(k_type, v_type, keys_total, n_head_kv) + align256(prefill_rope_bytes(n_q, n_head)) +
         align256(prefill_record_bytes(n_q, n_head, prefill_splits(n_q, keys_total, n_head, sm_count(dev))));
}

int rd_attn_prefill_typed(const float *q, const void *k, const void *v, float *o, const float *gate,
                          const int32_t *pos, int n_q, int keys_total, int n_head, int n_head_kv,
                          int head_dim, float scale, int k_type, int v_type, int n_rot, float freq_base,
                          void *workspace, size_t workspace_bytes, void *stream) {
  int rc = check_attn_shape(n_head, n_head_kv, head_dim, k_type, v_type);
  if (rc != RD_OK) return rc;
  if (n_q < 1 || keys_total <= 0) return RD_ERR_SHAPE;
  if (k == nullptr || v == nullptr) return RD_ERR_NULL;
  if (!aligned(k, 16) || !aligned(v, 16)) return RD_ERR_ALIGN;
  const size_t copies = prefill_copy_bytes(k_type, v_type, keys_total, n_head_kv);
  const size_t need = rd_attn_prefill_workspace_bytes(k_type, v_type, n_q, keys_total, n_head, n_head_kv, head_dim);
  if (need > 0) {
    if (workspace == nullptr || workspace_bytes < need) return RD_ERR_WORKSPACE;
    if (!aligned(workspace, 256)) return RD_ERR_ALIGN;
  }
  // caches that are not f16 are expanded once into the workspace -- one pass shared by
  // every query tile and every head, where the per-token path re-reads and re-expands
  // the prefix for each of the n_q tokens
  const int64_t n_values = (int64_t)keys_total * n_head_kv * kHeadDim;
  unsigned char *w = (unsigned char *)workspace;
  const void *k16 = k, *v16 = v;
  cudaStream_t st = (cudaStream_t)stream;
  void *kdst = nullptr, *vdst = nullptr;
  if (k_type != RD_KV_F16) {
    kdst = w;
    k16 = w;
    w += align256((size_t)n_values * 2);
  }
  if (v_type != RD_KV_F16) {
    vdst = w;
    v16 = w;
  }
  if (kdst != nullptr || vdst != nullptr) {   // one launch for both tensors
    if ((rc = launch_kv_dequant_f16_pair(k_type, kdst != nullptr ? k : nullptr, kdst, v_type,
                                         vdst != nullptr ? v : nullptr, vdst, n_values, st)) != RD_OK)
      return rc;
  }
  // what follows the copies holds the key-split records (never the library's own workspace:
  // this entry allocates nothing)
  unsigned char *rec = workspace != nullptr ? (unsigned char *)workspace + copies : nullptr;
  static float s_dummy;   // non-null marker when no records are needed
  return prefill_common(q, k16, v16, o, gate, pos, n_q, keys_total, n_head, n_head_kv, head_dim, scale,
                        n_rot, freq_base, stream, rec != nullptr ? (void *)rec : (void *)&s_dummy,
                        need > copies ? need - copies : 0);
}

static int g_last_site = 0;   // `where` of the last time-out rd_device_status reported

int rd_device_status(void) {
  int dev;
  int rc = current_device(&dev);
  if (rc != RD_OK) return rc;
  DeviceStatus *st = status_word(dev);
  if (st == nullptr) return RD_ERR_CUDA;
  if (cudaDeviceSynchronize() != cudaSuccess) return RD_ERR_CUDA;
  DeviceStatus h;
  if (cudaMemcpy(&h, st, sizeof(h), cudaMemcpyDeviceToHost) != cudaSuccess) return RD_ERR_CUDA;
  if (h.timeout_flag != 0) {
    g_last_site = h.where;
    cudaMemset(st, 0, sizeof(h));
    return RD_ERR_DEVICE;
  }
  return RD_OK;
}

int rd_device_timeout_site(void) { return g_last_site; }

}  // extern "C"
