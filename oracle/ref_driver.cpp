// Runs the REFERENCE project's own attention / KV kernels on the CPU.
//
// TEST INFRASTRUCTURE ONLY (parity pin of the oracle, generator of the golden
// vectors). The reference ships no CPU implementation of this path: it is HIP
// device code. Its headers are compiled here, from where they lie in the
// reference checkout, with g++ against a stand-in <hip/hip_runtime.h> (ref_shim/)
// after the Makefile strips the `<<<grid, block, smem, stream>>>` launch chevrons
// into a scratch copy under _ref/gen/. Each simulated GPU thread is a ucontext
// fiber; __syncthreads() and __shfl_xor_sync() yield to a round-robin scheduler,
// so the kernels execute exactly their own statements, lane by lane.
//
// Nothing of the reference is copied into this file: it only includes the
// headers and calls the kernels the way their launchers do (grid/block shapes are
// cited beside each call).
#include <ucontext.h>

#include <functional>
#include <vector>

#include "hip/hip_runtime.h"

rdshim_dim3 threadIdx, blockIdx, blockDim, gridDim;

#include "rdna4/attn.cuh"
#include "rdna4/attn_fa2.cuh"
#include "rdna4/kv.h"
#include "rdna4/nn.cuh"

namespace rdna4 {
// Dynamic shared memory of the attention kernels (`extern __shared__ float smem[]`
// inside namespace rdna4 resolves to these): 16 warps * (2+512) floats is the
// largest request (attn.cuh:601), the FA2 tile is 64 KiB (attn_fa2.cuh:182).
float smem[32 * (2 + 512)];
uint4 lds4[2 * 64 * 32];
}  // namespace rdna4

namespace {

// ------------------------------------------------------------ fiber runtime --
struct Fiber {
  ucontext_t ctx;
  std::vector<char> stack;
  bool done = false;
};

ucontext_t g_main;
std::vector<Fiber> g_fibers;
int g_cur = -1;
int g_live = 0;
std::function<void()> g_body;

// block barrier
int g_bar_count = 0;
unsigned g_bar_gen = 0;
// per-warp shuffle exchange
struct WarpX {
  float val[32];
  int count = 0;
  unsigned gen = 0;
};
std::vector<WarpX> g_warp;

void yield_to_main() { swapcontext(&g_fibers[g_cur].ctx, &g_main); }

void fiber_entry() {
  g_body();
  g_fibers[g_cur].done = true;
  --g_live;
  // a thread that exits no longer takes part in block barriers
  if (g_live > 0 && g_bar_count == g_live) {
    g_bar_count = 0;
    ++g_bar_gen;
  }
  swapcontext(&g_fibers[g_cur].ctx, &g_main);
}

void warp_barrier(int w) {
  WarpX &x = g_warp[w];
  const unsigned gen = x.gen;
  if (++x.count == 32) {
    x.count = 0;
    ++x.gen;
    return;
  }
  while (x.gen == gen) yield_to_main();
}

// Runs one CTA of `nthreads` simulated threads over `body`.
void run_cta(int nthreads, const std::function<void()> &body) {
  g_body = body;
  g_fibers.resize(nthreads);
  g_warp.assign((nthreads + 31) / 32, WarpX());
  g_bar_count = 0;
  g_live = nthreads;
  for (int i = 0; i < nthreads; ++i) {
    Fiber &f = g_fibers[i];
    f.done = false;
    if (f.stack.empty()) f.stack.resize(256 * 1024);
    getcontext(&f.ctx);
    f.ctx.uc_stack.ss_sp = f.stack.data();
    f.ctx.uc_stack.ss_size = f.stack.size();
    f.ctx.uc_link = &g_main;
    makecontext(&f.ctx, fiber_entry, 0);
  }
  while (g_live > 0) {
    for (int i = 0; i < nthreads; ++i) {
      if (g_fibers[i].done) continue;
      g_cur = i;
      threadIdx = rdshim_dim3((unsigned)i, 0, 0);
      swapcontext(&g_main, &g_fibers[i].ctx);
    }
  }
  g_cur = -1;
}

template <typename F>
void run_grid(dim3 grid, int nthreads, F &&body) {
  gridDim = grid;
  blockDim = rdshim_dim3((unsigned)nthreads, 1, 1);
  for (unsigned z = 0; z < grid.z; ++z)
    for (unsigned y = 0; y < grid.y; ++y)
      for (unsigned x = 0; x < grid.x; ++x) {
        blockIdx = rdshim_dim3(x, y, z);
        run_cta(nthreads, body);
      }
}

// Kernels without any synchronisation: plain loops over the thread index.
template <typename F>
void run_grid_nosync(dim3 grid, int nthreads, F &&body) {
  gridDim = grid;
  blockDim = rdshim_dim3((unsigned)nthreads, 1, 1);
  for (unsigned z = 0; z < grid.z; ++z)
    for (unsigned y = 0; y < grid.y; ++y)
      for (unsigned x = 0; x < grid.x; ++x) {
        blockIdx = rdshim_dim3(x, y, z);
        for (int i = 0; i < nthreads; ++i) {
          threadIdx = rdshim_dim3((unsigned)i, 0, 0);
          body();
        }
      }
}

using rdna4::KvType;

#define RD_KV4(M, ...)                                                                    \
  switch (kt_) {                                                                          \
    case 0: M(KvType::F32, __VA_ARGS__); break;                                            \
    case 1: M(KvType::F16, __VA_ARGS__); break;                                            \
    case 2: M(KvType::Q8_0, __VA_ARGS__); break;                                           \
    case 3: M(KvType::Q4_0, __VA_ARGS__); break;                                           \
    case 4: M(KvType::Q5_0, __VA_ARGS__); break;                                           \
    case 5: M(KvType::Q4_1, __VA_ARGS__); break;                                           \
    default: return -1;                                                                   \
  }

// Two-level dispatch over (K type, V type): calls fn.template operator()<KT,VT>().
template <KvType KT, typename Fn>
int dispatch_v(int vt, Fn &&fn) {
  switch (vt) {
    case 0: fn.template operator()<KT, KvType::F32>(); return 0;
    case 1: fn.template operator()<KT, KvType::F16>(); return 0;
    case 2: fn.template operator()<KT, KvType::Q8_0>(); return 0;
    case 3: fn.template operator()<KT, KvType::Q4_0>(); return 0;
    case 4: fn.template operator()<KT, KvType::Q5_0>(); return 0;
    case 5: fn.template operator()<KT, KvType::Q4_1>(); return 0;
  }
  return -1;
}
template <typename Fn>
int dispatch_kv(int kt, int vt, Fn &&fn) {
  switch (kt) {
    case 0: return dispatch_v<KvType::F32>(vt, fn);
    case 1: return dispatch_v<KvType::F16>(vt, fn);
    case 2: return dispatch_v<KvType::Q8_0>(vt, fn);
    case 3: return dispatch_v<KvType::Q4_0>(vt, fn);
    case 4: return dispatch_v<KvType::Q5_0>(vt, fn);
    case 5: return dispatch_v<KvType::Q4_1>(vt, fn);
  }
  return -1;
}

}  // namespace

void rdshim_syncthreads() {
  const unsigned gen = g_bar_gen;
  if (++g_bar_count == g_live) {
    g_bar_count = 0;
    ++g_bar_gen;
    return;
  }
  while (g_bar_gen == gen) yield_to_main();
}

float rdshim_shfl_xor(float v, int lane_mask) {
  const int w = g_cur >> 5, lane = g_cur & 31;
  g_warp[w].val[lane] = v;
  warp_barrier(w);
  const float r = g_warp[w].val[lane ^ lane_mask];
  warp_barrier(w);
  return r;
}

extern "C" {

uint16_t ref_float_to_fp16(float f) { return rdna4::float_to_fp16(f); }
float ref_fp16_to_float(uint16_t h) { return rdna4::fp16_to_float(h); }
float ref_kv_rand(unsigned idx, unsigned seed) { return rdna4::kv_rand(idx, seed); }

// kv_row_bytes aborts on a type outside the enum (kv.h:58-69); callers pass 0..5.
uint64_t ref_kv_row_bytes(int type, int head_dim) {
  return rdna4::kv_row_bytes((KvType)type, head_dim);
}
double ref_kv_bytes_per_elem(int type) { return rdna4::kv_bytes_per_elem((KvType)type); }
const char *ref_kv_type_name(int type) { return rdna4::kv_type_name((KvType)type); }
int ref_kv_type_parse(const char *name, int *out) {
  KvType t;
  if (rdna4::kv_type_parse(name, &t) != nullptr) return 1;
  *out = (int)t;
  return 0;
}
int ref_attn_split_wpb(int n_splits) { return rdna4::attn_split_wpb(n_splits); }
uint64_t ref_attn_partial_bytes(int n_head, int head_dim, int n_splits) {
  return rdna4::attn_partial_bytes(n_head, head_dim, n_splits);
}

// kv_store_row_launch (kv.h:673-680): grid ceil(units/128) x 128 threads,
// units = width for f32/f16, width/32 for the block types.
int ref_kv_store_rows(int kt_, const float *src, void *dst, int width) {
#define STORE(T, ...)                                                                      \
  {                                                                                       \
    const int units = (T == KvType::F32 || T == KvType::F16) ? width : width / 32;        \
    run_grid_nosync(dim3((units + 127) / 128), 128,                                       \
                    [&] { rdna4::kv_store_row_kernel<T>(src, dst, width); });             \
  }
  RD_KV4(STORE, 0)
#undef STORE
  return 0;
}

// kv_fill_launch (kv.h:632-671): one warp per 32-element block, 4 warps per CTA.
int ref_kv_fill(int kt_, void *cache, int64_t n_rows, int head_dim, unsigned seed) {
  const int64_t total_warps = n_rows * ((head_dim + 31) / 32);
  const unsigned blocks = (unsigned)((total_warps + 3) / 4);
#define FILL(T, ...)                                                                       \
  run_grid(dim3(blocks), 128, [&] { rdna4::kv_fill_kernel<T>(cache, n_rows, head_dim, seed); });
  RD_KV4(FILL, 0)
#undef FILL
  return 0;
}

// rope_launch (attn.cuh:56-63).
int ref_rope(float *x, int n_tok, int n_heads, int head_dim, int n_rot, float freq_base,
             const int *pos) {
  const int total = n_tok * n_heads * (n_rot / 2);
  run_grid_nosync(dim3((total + 127) / 128), 128, [&] {
    rdna4::rope_kernel(x, n_tok, n_heads, head_dim, n_rot, freq_base, pos);
  });
  return 0;
}

// rms_norm_launch (nn.cuh:94-101): one block of 256 threads per row.
int ref_rms_norm(const float *x, const float *w, float *y, int64_t nrows, int64_t ncols, float eps) {
  run_grid(dim3((unsigned)nrows), rdna4::kRmsNormThreads,
           [&] { rdna4::rms_norm_kernel(x, w, y, ncols, eps); });
  return 0;
}

// sigmoid_gate_launch (nn.cuh:414-420).
int ref_sigmoid_gate(float *g_io, float *y_io, int64_t n) {
  run_grid_nosync(dim3((unsigned)((n + 255) / 256)), 256,
                  [&] { rdna4::sigmoid_gate_kernel(g_io, y_io, n); });
  return 0;
}

// attn_launch_typed (attn.cuh:187-199): grid n_head x 256 threads.
int ref_attn(const float *q, const void *k, const void *v, float *out, int t, int n_head,
             int n_head_kv, int head_dim, float scale, int kt, int vt) {
  if (head_dim % 32 != 0 || head_dim / 32 > rdna4::kAttnMaxDimsPerLane) return -1;
  auto fn = [&]<KvType KT, KvType VT>() {
    run_grid(dim3(n_head), rdna4::kAttnWarpsPerBlock * 32, [&] {
      rdna4::attn_kernel<KT, VT>(q, k, v, out, t, n_head, n_head_kv, head_dim, scale);
    });
  };
  return dispatch_kv(kt, vt, fn);
}

// attn_batch_launch_typed (attn.cuh:357-371): grid (n_head, n_tok).
int ref_attn_batch(const float *q, const void *k, const void *v, float *out, const int *pos,
                   int n_tok, int n_head, int n_head_kv, int head_dim, float scale, int kt,
                   int vt) {
  if (head_dim % 32 != 0 || head_dim / 32 > rdna4::kAttnMaxDimsPerLane) return -1;
  auto fn = [&]<KvType KT, KvType VT>() {
    run_grid(dim3(n_head, n_tok), rdna4::kAttnWarpsPerBlock * 32, [&] {
      rdna4::attn_batch_kernel<KT, VT>(q, k, v, out, pos, n_head, n_head_kv, head_dim, scale);
    });
  };
  return dispatch_kv(kt, vt, fn);
}

// attn_merge_kernel launch (attn.cuh:605): grid n_head x 32 threads.
int ref_attn_merge(const float *partial, float *out, int n_head, int head_dim, int n_splits) {
  run_grid_nosync(dim3(n_head), 32, [&] {
    rdna4::attn_merge_kernel(partial, out, n_head, head_dim, n_splits);
  });
  return 0;
}

// attn_launch_split (attn.cuh:903-956): WPB from attn_split_wpb, grid
// (n_head, n_splits) x WPB*32 threads, then the merge.
int ref_attn_split(const float *q, const void *k, const void *v, float *out, float *partial,
                   int t, int n_head, int n_head_kv, int head_dim, float scale, int kt, int vt,
                   int n_splits) {
  if (head_dim % 32 != 0 || head_dim / 32 > rdna4::kAttnMaxDimsPerLane || n_splits < 1) return -1;
  const int wpb = rdna4::attn_split_wpb(n_splits);
  auto fn = [&]<KvType KT, KvType VT>() {
    if (wpb == 16) {
      run_grid(dim3(n_head, n_splits), 16 * 32, [&] {
        rdna4::attn_split_kernel<KT, VT, 16>(q, k, v, partial, t, n_head, n_head_kv, head_dim,
                                             scale, n_splits);
      });
    } else {
      run_grid(dim3(n_head, n_splits), 8 * 32, [&] {
        rdna4::attn_split_kernel<KT, VT, 8>(q, k, v, partial, t, n_head, n_head_kv, head_dim,
                                            scale, n_splits);
      });
    }
  };
  const int rc = dispatch_kv(kt, vt, fn);
  if (rc != 0) return rc;
  if (out) return ref_attn_merge(partial, out, n_head, head_dim, n_splits);
  return 0;
}

// attn_split_batch_launch (attn.cuh:958-1049): grid (n_head, n_splits, n_tok),
// merge grid (n_head, n_tok).
int ref_attn_split_batch(const float *q, const void *k, const void *v, float *out,
                         float *partial, const int *pos, int n_tok, int n_head, int n_head_kv,
                         int head_dim, float scale, int kt, int vt, int n_splits) {
  if (head_dim % 32 != 0 || head_dim / 32 > rdna4::kAttnMaxDimsPerLane) return -1;
  if (n_splits < 1 || n_tok < 1) return -1;
  const int wpb = rdna4::attn_split_wpb(n_splits);
  auto fn = [&]<KvType KT, KvType VT>() {
    if (wpb == 16) {
      run_grid(dim3(n_head, n_splits, n_tok), 16 * 32, [&] {
        rdna4::attn_split_batch_kernel<KT, VT, 16>(q, k, v, partial, pos, n_head, n_head_kv,
                                                   head_dim, scale, n_splits);
      });
    } else {
      run_grid(dim3(n_head, n_splits, n_tok), 8 * 32, [&] {
        rdna4::attn_split_batch_kernel<KT, VT, 8>(q, k, v, partial, pos, n_head, n_head_kv,
                                                  head_dim, scale, n_splits);
      });
    }
  };
  const int rc = dispatch_kv(kt, vt, fn);
  if (rc != 0) return rc;
  run_grid_nosync(dim3(n_head, n_tok), 32, [&] {
    rdna4::attn_merge_batch_kernel(partial, out, head_dim, n_splits);
  });
  return 0;
}

// fa2_prefill_launch (attn_fa2.cuh:174-187): f16/f16, grid (n_head_kv,
// ceil(n_q/16)) x 512 threads, 64-key tiles.
int ref_fa2_prefill(const float *q, const void *k, const void *v, float *o, const int *pos,
                    int n_q, int kmax, int keys_total, int n_head, int n_head_kv, int head_dim,
                    float scale) {
  if (head_dim != 256 || n_head_kv <= 0 || n_head / n_head_kv != 6 || n_head % n_head_kv != 0 ||
      n_q < 1 || kmax < 0 || keys_total <= 0)
    return -1;
  run_grid(dim3(n_head_kv, (n_q + 15) / 16), 16 * 32, [&] {
    rdna4::attn_fa2_prefill_kernel<KvType::F16, KvType::F16, 64, 6, false, 16>(
        q, k, v, o, pos, n_head, n_head_kv, head_dim, scale, n_q, kmax, keys_total);
  });
  return 0;
}

int ref_fa2_prefill_usable(int kt, int vt, int n_q, int pos0, int n_head, int n_head_kv,
                           int head_dim) {
  return rdna4::fa2_prefill_usable((KvType)kt, (KvType)vt, n_q, pos0, n_head, n_head_kv,
                                   head_dim)
             ? 1
             : 0;
}

}  // extern "C"
