// A caller shaped like the reference's Graph::full_attn (graph.cuh:901-988) and
// Graph::forward_batch_layer (graph.cuh:1429-1540), written ONLY against the reference's
// names (namespace rdna4, KvType, *_launch returning bool) and linked to the C-ABI
// library: what a maintainer's code looks like after swapping the headers.
//
//   graph_caller <out.bin> <k_type> <v_type> <n_prefix> <n_batch> <n_layers>
//
// Per layer: the cache is pre-filled for n_prefix positions (kv_fill_launch, the
// reference's --fill-cache hook), then
//   (1) a batch of n_batch tokens at positions n_prefix.. goes through the batch path:
//       deinterleave, q/k norm, RoPE, KV write, attention (fa2_prefill_launch when
//       usable, else attn_split_batch_launch), gate;
//   (2) one more token goes through the decode path: the same steps with n_tok = 1,
//       attn_splits_for -> attn_launch_split / attn_launch, sigmoid_gate_launch.
// Inputs come from the LCG of the reference's tests (check_rope_gpu.hip:36-39). The
// file receives, per layer, the batch outputs [n_batch][NH][HD] and the decode output
// [NH][HD] as f32; the Python test recomputes them with the CPU oracle.
#include <cuda_runtime.h>

#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <string>
#include <vector>

#include "rdna4/attn.cuh"
#include "rdna4/attn_fa2.cuh"

using namespace rdna4;

#define CK(call)                                                          \
  do {                                                                    \
    if (!(call)) {                                                        \
      std::fprintf(stderr, "FAILED %s:%d: %s\n", __FILE__, __LINE__, #call); \
      return 2;                                                           \
    }                                                                     \
  } while (0)
#define CU(call) CK((call) == cudaSuccess)

static uint32_t g_lcg = 12345u;
static float lcg_next() {
  g_lcg = g_lcg * 1664525u + 1013904223u;
  return ((float)(g_lcg >> 8) / 16777216.0f - 0.5f) * 2.0f;
}
static void fill(std::vector<float> &v, float amp) {
  for (auto &x : v) x = amp * lcg_next();
}

int main(int argc, char **argv) {
  if (argc != 7) {
    std::fprintf(stderr, "usage: graph_caller out.bin k_type v_type n_prefix n_batch n_layers\n");
    return 1;
  }
  KvType kt, vt;
  CK(kv_type_parse(argv[2], &kt) == nullptr);
  CK(kv_type_parse(argv[3], &vt) == nullptr);
  const int n_prefix = std::atoi(argv[4]), n_batch = std::atoi(argv[5]), n_layers = std::atoi(argv[6]);
  const int NH = 24, NKV = 4, HD = 256, n_rot = 64;
  const float base = 1e7f, eps = 1e-6f, scale = 1.0f / std::sqrt((float)HD);
  const int max_ctx = n_prefix + n_batch + 1;
  const size_t krow = kv_row_bytes(kt, HD) * NKV, vrow = kv_row_bytes(vt, HD) * NKV;

  float *d_proj, *d_kst, *d_vst, *d_q, *d_gate, *d_qw, *d_kw, *d_partial, *d_out;
  int *d_pos;
  void *d_k, *d_v;
  const int max_tok = n_batch > 1 ? n_batch : 1;
  CU(cudaMalloc(&d_proj, sizeof(float) * max_tok * NH * 2 * HD));
  CU(cudaMalloc(&d_kst, sizeof(float) * max_tok * NKV * HD));
  CU(cudaMalloc(&d_vst, sizeof(float) * max_tok * NKV * HD));
  CU(cudaMalloc(&d_q, sizeof(float) * max_tok * NH * HD));
  CU(cudaMalloc(&d_out, sizeof(float) * max_tok * NH * HD));
  CU(cudaMalloc(&d_gate, sizeof(float) * max_tok * NH * HD));
  CU(cudaMalloc(&d_qw, sizeof(float) * HD));
  CU(cudaMalloc(&d_kw, sizeof(float) * HD));
  CU(cudaMalloc(&d_pos, sizeof(int) * max_tok));
  // the reference sizes its partial buffer for 16 splits per (token, head)
  CU(cudaMalloc(&d_partial, (size_t)max_tok * attn_partial_bytes(NH, HD, tuned::kAttnMaxSplits)));
  CU(cudaMalloc(&d_k, krow * max_ctx));
  CU(cudaMalloc(&d_v, vrow * max_ctx));

  FILE *f = std::fopen(argv[1], "wb");
  CK(f != nullptr);
  std::vector<float> h_proj, h_k, h_v, h_w(HD), h_out;
  for (int il = 0; il < n_layers; ++il) {
    CK(kv_fill_launch(kt, d_k, (std::int64_t)n_prefix * NKV, HD, 100u + il));
    CK(kv_fill_launch(vt, d_v, (std::int64_t)n_prefix * NKV, HD, 200u + il));
    for (auto &x : h_w) x = 1.0f + 0.1f * lcg_next();
    CU(cudaMemcpy(d_qw, h_w.data(), sizeof(float) * HD, cudaMemcpyHostToDevice));
    for (auto &x : h_w) x = 1.0f + 0.1f * lcg_next();
    CU(cudaMemcpy(d_kw, h_w.data(), sizeof(float) * HD, cudaMemcpyHostToDevice));

    for (int phase = 0; phase < 2; ++phase) {
      const int n = phase == 0 ? n_batch : 1;
      const int pos0 = phase == 0 ? n_prefix : n_prefix + n_batch;
      if (n == 0) continue;
      h_proj.assign((size_t)n * NH * 2 * HD, 0.f);
      h_k.assign((size_t)n * NKV * HD, 0.f);
      h_v.assign((size_t)n * NKV * HD, 0.f);
      fill(h_proj, 2.0f);
      fill(h_k, 2.0f);
      fill(h_v, 1.0f);
      std::vector<int> h_pos(n);
      for (int i = 0; i < n; ++i) h_pos[i] = pos0 + i;
      CU(cudaMemcpy(d_proj, h_proj.data(), sizeof(float) * h_proj.size(), cudaMemcpyHostToDevice));
      CU(cudaMemcpy(d_kst, h_k.data(), sizeof(float) * h_k.size(), cudaMemcpyHostToDevice));
      CU(cudaMemcpy(d_vst, h_v.data(), sizeof(float) * h_v.size(), cudaMemcpyHostToDevice));
      CU(cudaMemcpy(d_pos, h_pos.data(), sizeof(int) * n, cudaMemcpyHostToDevice));

      // qk_norm_rope_kv (graph.cuh:915-954 decode, :1446-1476 batch)
      CK(deinterleave_q_gate_batch_launch(d_proj, d_q, d_gate, n, NH, HD));
      CK(rms_norm_launch(d_q, d_qw, d_q, (std::int64_t)n * NH, HD, eps));
      CK(rms_norm_launch(d_kst, d_kw, d_kst, (std::int64_t)n * NKV, HD, eps));
      CK(rope_launch(d_q, n, NH, HD, n_rot, base, d_pos));
      CK(rope_launch(d_kst, n, NKV, HD, n_rot, base, d_pos));
      CK(kv_store_row_launch(kt, d_kst, (char *)d_k + krow * pos0, n * NKV * HD));
      CK(kv_store_row_launch(vt, d_vst, (char *)d_v + vrow * pos0, n * NKV * HD));

      if (phase == 0) {
        // forward_batch_layer (graph.cuh:1479-1535)
        const int kmax = pos0 + n - 1;
        if (fa2_prefill_usable(kt, vt, n, pos0, NH, NKV, HD)) {
          CK(fa2_prefill_launch(d_q, d_k, d_v, d_out, d_pos, n, kmax, kmax + 1, NH, NKV, HD, scale));
        } else {
          const int splits = attn_splits_for(kmax + 1, kt, vt, NH);
          if (splits > 1)
            CK(attn_split_batch_launch(d_q, d_k, d_v, d_out, d_partial, d_pos, n, NH, NKV, HD, scale, kt,
                                       vt, splits));
          else
            CK(attn_batch_launch(d_q, d_k, d_v, d_out, d_pos, n, NH, NKV, HD, scale, kt, vt));
        }
      } else {
        // full_attn (graph.cuh:958-977): q and out alias, as in the reference
        const int splits = attn_splits_for(pos0 + 1, kt, vt, NH);
        if (splits > 1)
          CK(attn_launch_split(d_q, d_k, d_v, d_q, d_partial, pos0, NH, NKV, HD, scale, kt, vt, splits));
        else
          CK(attn_launch(d_q, d_k, d_v, d_q, pos0, NH, NKV, HD, scale, kt, vt));
        CU(cudaMemcpy(d_out, d_q, sizeof(float) * NH * HD, cudaMemcpyDeviceToDevice));
      }
      CK(sigmoid_gate_launch(d_gate, d_out, (std::int64_t)n * NH * HD));
      h_out.resize((size_t)n * NH * HD);
      CU(cudaMemcpy(h_out.data(), d_out, sizeof(float) * h_out.size(), cudaMemcpyDeviceToHost));
      CK(std::fwrite(h_out.data(), sizeof(float), h_out.size(), f) == h_out.size());
    }
  }
  std::fclose(f);
  CU(cudaDeviceSynchronize());
  std::printf("graph_caller OK\n");
  return 0;
}
