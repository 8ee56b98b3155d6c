// The reference project's own GPU launchers (include/rdna4/attn.cuh, attn_fa2.cuh, kv.h of
// the reference checkout, compiled unmodified against ref_gpu_shim/) behind a C ABI, so
// that the tests can cross-check the product kernels against them on the same GPU and
// bench.py can time them beside the product ("reference kernel on this box"). Test
// infrastructure only: built by `make -C oracle ref_gpu` into the git-ignored _ref/.
#include <cstdint>
#include <cstdio>

#include "rdna4/attn.cuh"
#include "rdna4/attn_fa2.cuh"
#include "rdna4/kv.h"

using rdna4::KvType;

extern "C" {

// attn_launch (attn.cuh:201-249)
int refgpu_attn(const float *q, const void *k, const void *v, float *out, int t, int n_head,
                int n_head_kv, int head_dim, float scale, int kt, int vt, void *stream) {
  return rdna4::attn_launch(q, k, v, out, t, n_head, n_head_kv, head_dim, scale, (KvType)kt, (KvType)vt,
                            (hipStream_t)stream)
             ? 0
             : -1;
}

// attn_launch_split (attn.cuh:903-956): split kernel + merge
int refgpu_attn_split(const float *q, const void *k, const void *v, float *out, float *partial, int t,
                      int n_head, int n_head_kv, int head_dim, float scale, int kt, int vt, int n_splits,
                      void *stream) {
  return rdna4::attn_launch_split(q, k, v, out, partial, t, n_head, n_head_kv, head_dim, scale, (KvType)kt,
                                  (KvType)vt, n_splits, (hipStream_t)stream)
             ? 0
             : -1;
}

// fa2_prefill_launch (attn_fa2.cuh:171-207). Its kernel asks for 64 KiB of dynamic shared
// memory, which a CUDA device grants only after an opt-in on the kernel; the reference's
// launcher has no such call (HIP needs none), so it is made here, once, on the one
// instantiation that launcher dispatches.
int refgpu_fa2_prefill(const float *q, const void *k, const void *v, float *o, const int *pos, int n_q,
                       int kmax, int keys_total, int n_head, int n_head_kv, int head_dim, float scale,
                       void *stream) {
  static const cudaError_t optin = cudaFuncSetAttribute(
      rdna4::attn_fa2_prefill_kernel<KvType::F16, KvType::F16, 64, 6, false, 16>,
      cudaFuncAttributeMaxDynamicSharedMemorySize, 2 * 64 * 256 * 2);
  if (optin != cudaSuccess) {
    std::fprintf(stderr, "refgpu_fa2_prefill: shared-memory opt-in failed: %s\n", cudaGetErrorString(optin));
    return -2;
  }
  (void)cudaGetLastError();
  if (rdna4::fa2_prefill_launch(q, k, v, o, pos, n_q, kmax, keys_total, n_head, n_head_kv, head_dim, scale,
                                (hipStream_t)stream))
    return 0;
  std::fprintf(stderr, "refgpu_fa2_prefill: launch refused: %s\n", cudaGetErrorString(cudaPeekAtLastError()));
  return -1;
}

// kv_store_row_launch (kv.h:673-694)
int refgpu_kv_store_rows(int type, const float *src, void *dst, int width, void *stream) {
  return rdna4::kv_store_row_launch((KvType)type, src, dst, width, (hipStream_t)stream) ? 0 : -1;
}

}  // extern "C"
