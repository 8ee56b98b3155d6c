// RMS-norm (replaces rms_norm_kernel, include/rdna4/nn.cuh:23-63 and rms_norm_launch,
// :239-243 of the reference) and the fused pre-attention stage of a full-attention
// layer: what Graph::full_attn does in seven launches between the projections and
// the attention call (include/rdna4/graph.cuh:915-954) --
//   deinterleave [q | gate] per head, RMS-norm of every q and k head row with its weight,
//   partial RoPE of q and k, quantize-and-store of the k and v rows into the caches --
// in ONE launch, one warp per 256-wide head row.
//
// The sum of squares keeps the reference kernel's order (256 threads each squaring one
// element, then a shared-memory tree over strides 128 .. 1), so it is bit-identical to
// it; rsqrt is the correctly rounded 1 / sqrt (the reference's device intrinsic is
// approximate). A warp lane L holds elements L, L+32, .. L+224 of the row, which makes
// the first three tree levels and the RoPE pairs (p, p + n_rot/2 with n_rot/2 a multiple
// of 32) lane-local and gives the quantizer its native layout (lane j = element j of a
// 32-value block).
#include "rd_common.cuh"
#include "rd_internal.h"
#include "rd_quant.cuh"

namespace rd {

constexpr int kRmsThreads = 256;

__global__ void __launch_bounds__(kRmsThreads)
rms_norm_kernel(const float *__restrict__ x, const float *__restrict__ w, float *__restrict__ y,
                int64_t ncols, float eps) {
  __shared__ float partial[kRmsThreads];
  const float *xr = x + (int64_t)blockIdx.x * ncols;
  float *yr = y + (int64_t)blockIdx.x * ncols;
  float acc = 0.0f;
  for (int64_t i = threadIdx.x; i < ncols; i += kRmsThreads) acc = __fmaf_rn(xr[i], xr[i], acc);
  partial[threadIdx.x] = acc;
  __syncthreads();
  for (int stride = kRmsThreads / 2; stride > 0; stride >>= 1) {
    if ((int)threadIdx.x < stride)
      partial[threadIdx.x] = __fadd_rn(partial[threadIdx.x], partial[threadIdx.x + stride]);
    __syncthreads();
  }
  const float scale =
      __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(partial[0], (float)ncols), eps)));
  for (int64_t i = threadIdx.x; i < ncols; i += kRmsThreads) {
    const float v = __fmul_rn(xr[i], scale);
    yr[i] = w != nullptr ? __fmul_rn(v, w[i]) : v;
  }
}

int launch_rms_norm(const float *x, const float *w, float *y, int64_t nrows, int64_t ncols, float eps,
                    cudaStream_t st) {
  if (nrows == 0) return RD_OK;
  rms_norm_kernel<<<(unsigned)nrows, kRmsThreads, 0, st>>>(x, w, y, ncols, eps);
  return cudaGetLastError() == cudaSuccess ? RD_OK : RD_ERR_CUDA;
}

struct PreAttnArgs {
  const float *qg;      // [n_tok][n_head][2 * 256]: q then gate per head
  const float *k_src;   // [n_tok][nkv][256]
  const float *v_src;   // [n_tok][nkv][256]
  const float *q_w;     // [256] or null
  const float *k_w;     // [256] or null
  float *q_out;         // [n_tok][n_head][256]
  float *gate_out;      // [n_tok][n_head][256]
  uint8_t *k_rows;      // cache rows of the n_tok new tokens, [n_tok][nkv] rows
  uint8_t *v_rows;
  const int32_t *pos;   // [n_tok]
  int n_tok, n_head, nkv, n_rot;
  float eps, freq_base;
  RopeTable rope;
};

// Normalise (optional) and rotate the 8 values a lane holds of one head row.
__device__ __forceinline__ void norm_rope_row(float (&x)[8], const float *__restrict__ w, float eps,
                                              int n_rot, float fpos, const RopeTable &tab,
                                              float freq_base, int lane) {
  float p[8];
#pragma unroll
  for (int k = 0; k < 8; ++k) p[k] = __fmul_rn(x[k], x[k]);
#pragma unroll
  for (int k = 0; k < 4; ++k) p[k] = __fadd_rn(p[k], p[k + 4]);   // stride 128
  p[0] = __fadd_rn(p[0], p[2]);                                   // stride 64
  p[1] = __fadd_rn(p[1], p[3]);
  float s = __fadd_rn(p[0], p[1]);                                // stride 32
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) s = __fadd_rn(s, __shfl_down_sync(0xffffffffu, s, o));
  s = __shfl_sync(0xffffffffu, s, 0);
  const float scale = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(s, (float)kHeadDim), eps)));
#pragma unroll
  for (int k = 0; k < 8; ++k) {
    x[k] = __fmul_rn(x[k], scale);
    if (w != nullptr) x[k] = __fmul_rn(x[k], w[lane + 32 * k]);
  }
  const int hk = n_rot / 64;   // registers per half: pairs (k, k + hk), k < hk
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    if (k < hk) {
      const int pidx = lane + 32 * k;
      const float freq = pidx < kRopeTablePairs
                             ? tab.f[pidx]
                             : (float)pow((double)freq_base, (double)(-2.0f * (float)pidx / (float)n_rot));
      float c, sn;
      sincosf(fpos * freq, &sn, &c);
#pragma unroll
      for (int h = 1; h <= 4; ++h) {
        if (h == hk && k + h < 8) {
          const float x0 = x[k], x1 = x[k + h];
          x[k] = __fsub_rn(__fmul_rn(x0, c), __fmul_rn(x1, sn));
          x[k + h] = __fadd_rn(__fmul_rn(x0, sn), __fmul_rn(x1, c));
        }
      }
    }
  }
}

template <int KT, int VT>
__global__ void __launch_bounds__(256) pre_attn_kernel(const __grid_constant__ PreAttnArgs a) {
  const int lane = threadIdx.x & 31;
  const int64_t row = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int per_tok = a.n_head + 2 * a.nkv;
  if (row >= (int64_t)a.n_tok * per_tok) return;
  const int tok = (int)(row / per_tok), r = (int)(row % per_tok);
  float x[8];
  if (r < a.n_head) {
    // a query head: split off the gate, normalise, rotate
    const float *src = a.qg + ((size_t)tok * a.n_head + r) * (2 * kHeadDim);
    float *qo = a.q_out + ((size_t)tok * a.n_head + r) * kHeadDim;
    float *go = a.gate_out + ((size_t)tok * a.n_head + r) * kHeadDim;
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      x[k] = src[lane + 32 * k];
      go[lane + 32 * k] = src[kHeadDim + lane + 32 * k];
    }
    norm_rope_row(x, a.q_w, a.eps, a.n_rot, (float)a.pos[tok], a.rope, a.freq_base, lane);
#pragma unroll
    for (int k = 0; k < 8; ++k) qo[lane + 32 * k] = x[k];
  } else if (r < a.n_head + a.nkv) {
    const int kvh = r - a.n_head;
    const float *src = a.k_src + ((size_t)tok * a.nkv + kvh) * kHeadDim;
#pragma unroll
    for (int k = 0; k < 8; ++k) x[k] = src[lane + 32 * k];
    norm_rope_row(x, a.k_w, a.eps, a.n_rot, (float)a.pos[tok], a.rope, a.freq_base, lane);
    uint8_t *dst = a.k_rows + ((size_t)tok * a.nkv + kvh) * row_bytes(KT);
#pragma unroll
    for (int k = 0; k < 8; ++k) store_block<KT>(x[k], dst, k, lane);
  } else {
    const int kvh = r - a.n_head - a.nkv;
    const float *src = a.v_src + ((size_t)tok * a.nkv + kvh) * kHeadDim;
    uint8_t *dst = a.v_rows + ((size_t)tok * a.nkv + kvh) * row_bytes(VT);
#pragma unroll
    for (int k = 0; k < 8; ++k) store_block<VT>(src[lane + 32 * k], dst, k, lane);
  }
}

template <int KT>
static int pre_attn_v(int vt, const PreAttnArgs &a, unsigned grid, cudaStream_t st) {
#define RD_V(VT)                                  \
  case VT:                                        \
    pre_attn_kernel<KT, VT><<<grid, 256, 0, st>>>(a); \
    break;
  switch (vt) {
    RD_V(RD_KV_F32)
    RD_V(RD_KV_F16)
    RD_V(RD_KV_Q8_0)
    RD_V(RD_KV_Q4_0)
    RD_V(RD_KV_Q5_0)
    RD_V(RD_KV_Q4_1)
    default: return RD_ERR_TYPE;
  }
#undef RD_V
  return cudaGetLastError() == cudaSuccess ? RD_OK : RD_ERR_CUDA;
}

int launch_pre_attn(int kt, int vt, const float *qg, const float *k_src, const float *v_src,
                    const float *q_w, const float *k_w, float eps, float *q_out, float *gate_out,
                    void *k_rows, void *v_rows, const int32_t *pos, int n_tok, int n_head, int nkv,
                    int n_rot, float freq_base, cudaStream_t st) {
  if (n_tok == 0) return RD_OK;
  PreAttnArgs a;
  a.qg = qg;
  a.k_src = k_src;
  a.v_src = v_src;
  a.q_w = q_w;
  a.k_w = k_w;
  a.q_out = q_out;
  a.gate_out = gate_out;
  a.k_rows = (uint8_t *)k_rows;
  a.v_rows = (uint8_t *)v_rows;
  a.pos = pos;
  a.n_tok = n_tok;
  a.n_head = n_head;
  a.nkv = nkv;
  a.n_rot = n_rot;
  a.eps = eps;
  a.freq_base = freq_base;
  a.rope = make_rope_table(n_rot, freq_base);
  const int64_t warps = (int64_t)n_tok * (n_head + 2 * nkv);
  const unsigned grid = (unsigned)((warps * 32 + 255) / 256);
#define RD_K(KT) \
  case KT: return pre_attn_v<KT>(vt, a, grid, st);
  switch (kt) {
    RD_K(RD_KV_F32)
    RD_K(RD_KV_F16)
    RD_K(RD_KV_Q8_0)
    RD_K(RD_KV_Q4_0)
    RD_K(RD_KV_Q5_0)
    RD_K(RD_KV_Q4_1)
    default: return RD_ERR_TYPE;
  }
#undef RD_K
}

}  // namespace rd
