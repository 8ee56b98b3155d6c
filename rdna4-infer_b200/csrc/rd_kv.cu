// KV-append (quantize-on-store), synthetic cache fill, RoPE and the gate glue.
//
// KV append is the bit-exact part of the path: every block of 32 values must come
// out byte-identical to the reference quantizers (include/rdna4/kv.h:386-501). The
// reference runs one THREAD per block with serial 32-element loops; here one WARP
// owns a block, lane j holds element j, the block statistics are warp shuffles and
// every lane stores its own byte. The arithmetic is pinned with explicit
// round-to-nearest intrinsics so that no multiply-add is contracted into an FMA:
// `x*id + 8.5f` is two roundings in the reference's host mirror, and a fused form
// changes the byte whenever the sum lands within an ulp of an integer.
#include "rd_common.cuh"
#include "rd_internal.h"
#include "rd_quant.cuh"

namespace rd {


// RoPE angle factor: freq = base^(-2p/n_rot). The reference calls f32 powf
// (attn.cuh:39); the correctly rounded value is what a good host libm returns, and
// a one-ulp difference here moves theta by several milliradians at position 131000,
// so it is computed in double and rounded once.
__device__ __forceinline__ float rope_freq(float freq_base, int p, int n_rot) {
  const float e = -2.0f * (float)p / (float)n_rot;
  return (float)pow((double)freq_base, (double)e);
}
constexpr int kMaxRopePairs = 256;  // n_rot <= head_dim <= 512

// sin/cos of the f32 angle with the accurate f32 routine (full-range argument
// reduction, <= 2 ulp): what the reference's cosf/sinf do (attn.cuh:40-41), and far
// cheaper than double for the 10^5..10^6 angles a prefill chunk needs.
__device__ __forceinline__ void rope_cs(float theta, float &c, float &s) { sincosf(theta, &s, &c); }

// One warp per 32-element block of K (blockIdx.y == 0) or V (blockIdx.y == 1).
// With pos != nullptr the K value is rotated first (attn.cuh:30-54): element e of a
// head pairs with e +- n_rot/2 inside the first n_rot dims, which for n_rot == 64 is
// the neighbouring block, so the partner is read from global memory.
template <int KT, int VT>
__global__ void __launch_bounds__(256)
kv_append_kernel(const float *__restrict__ ksrc, const float *__restrict__ vsrc,
                 uint8_t *__restrict__ kdst, uint8_t *__restrict__ vdst, int64_t n_blocks,
                 int head_dim, int heads_per_tok, const int32_t *__restrict__ pos, int n_rot,
                 float freq_base, const __grid_constant__ RopeTable tab) {
  // the n_rot/2 frequencies once per CTA (a double pow per element would dominate a
  // 512-token append)
  __shared__ float s_freq[kMaxRopePairs];
  pdl_launch_dependents();
  pdl_wait();
  if (pos != nullptr && blockIdx.y == 0 && (int)threadIdx.x < n_rot / 2)
    s_freq[threadIdx.x] = (int)threadIdx.x < kRopeTablePairs ? tab.f[threadIdx.x]
                                                             : rope_freq(freq_base, threadIdx.x, n_rot);
  __syncthreads();
  const int lane = threadIdx.x & 31;
  const int64_t blk = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  if (blk >= n_blocks) return;
  if (blockIdx.y == 0) {
    if (ksrc == nullptr) return;
    const int64_t e = blk * 32 + lane;
    float x = ksrc[e];
    if (pos != nullptr) {
      const int d = (int)(e % head_dim);
      if (d < n_rot) {
        const int half = n_rot / 2;
        const int p = d < half ? d : d - half;
        const int tok = (int)(e / ((int64_t)head_dim * heads_per_tok));
        const float theta = (float)pos[tok] * s_freq[p];
        float c, s;
        rope_cs(theta, c, s);
        const float other = ksrc[d < half ? e + half : e - half];
        // (x0, x1) -> (x0*c - x1*s, x0*s + x1*c), products rounded separately
        x = d < half ? __fsub_rn(__fmul_rn(x, c), __fmul_rn(other, s))
                     : __fadd_rn(__fmul_rn(other, s), __fmul_rn(x, c));
      }
    }
    store_block<KT>(x, kdst, blk, lane);
  } else {
    if (vsrc == nullptr) return;
    store_block<VT>(vsrc[blk * 32 + lane], vdst, blk, lane);
  }
}

// include/rdna4/kv.h:508-513.
__device__ __forceinline__ float kv_rand_dev(unsigned idx, unsigned seed) {
  unsigned h = idx * 2654435761u ^ seed * 2246822519u;
  h ^= h >> 13;
  h *= 1274126177u;
  return __fsub_rn(__fdiv_rn((float)(h >> 8), 8388608.0f), 1.0f);
}

template <int T>
__global__ void __launch_bounds__(256)
kv_fill_kernel(uint8_t *__restrict__ cache, int64_t n_blocks, unsigned seed) {
  const int lane = threadIdx.x & 31;
  const int64_t blk = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  if (blk >= n_blocks) return;
  // rows are contiguous and head_dim is a multiple of 32, so block b of the cache
  // holds elements 32b..32b+31 of the flat index the hash is fed with.
  const float x = kv_rand_dev((unsigned)(blk * 32 + lane), seed);
  store_block<T>(x, cache, blk, lane);
}

__global__ void __launch_bounds__(128)
rope_kernel(float *__restrict__ x, int n_tok, int n_heads, int head_dim, int n_rot,
            float freq_base, const int32_t *__restrict__ pos, const __grid_constant__ RopeTable tab) {
  const int pairs = n_rot / 2;
  __shared__ float s_freq[kMaxRopePairs];
  for (int i = threadIdx.x; i < pairs; i += blockDim.x)
    s_freq[i] = i < kRopeTablePairs ? tab.f[i] : rope_freq(freq_base, i, n_rot);
  __syncthreads();
  const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (int64_t)n_tok * n_heads * pairs) return;
  const int p = (int)(idx % pairs);
  const int64_t th = idx / pairs;  // token * n_heads + head
  const int tok = (int)(th / n_heads);
  const float theta = (float)pos[tok] * s_freq[p];
  float c, s;
  rope_cs(theta, c, s);
  float *base = x + th * head_dim;
  const float x0 = base[p], x1 = base[p + pairs];
  base[p] = __fsub_rn(__fmul_rn(x0, c), __fmul_rn(x1, s));
  base[p + pairs] = __fadd_rn(__fmul_rn(x0, s), __fmul_rn(x1, c));
}

__global__ void deinterleave_kernel(const float4 *__restrict__ yq, float4 *__restrict__ q,
                                    float4 *__restrict__ gate, int64_t n_rows, int hd4) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n_rows * hd4) return;
  const int64_t r = i / hd4;
  const int d = (int)(i % hd4);
  q[i] = yq[r * 2 * hd4 + d];
  gate[i] = yq[r * 2 * hd4 + hd4 + d];
}

__global__ void sigmoid_gate_kernel(float *__restrict__ g, float *__restrict__ y, int64_t n) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const float s = __fdiv_rn(1.0f, 1.0f + expf(-g[i]));
  g[i] = s;
  y[i] = y[i] * s;
}

// ---- host launchers ---------------------------------------------------------------

template <int KT>
static int append_dispatch_v(int vt, const float *ks, const float *vs, uint8_t *kd, uint8_t *vd,
                             int64_t n_blocks, int head_dim, int heads_per_tok, const int32_t *pos,
                             int n_rot, float freq_base, cudaStream_t st) {
  const dim3 grid((unsigned)((n_blocks * 32 + 255) / 256), 2);
  const RopeTable tab = make_rope_table(pos != nullptr ? n_rot : 0, freq_base);
  cudaError_t err = cudaSuccess;
#define RD_V(VT)                                                                              \
  case VT:                                                                                    \
    err = launch_pdl(1, kv_append_kernel<KT, VT>, grid, dim3(256), 0, st, ks, vs, kd, vd, n_blocks, \
                     head_dim, heads_per_tok, pos, n_rot, freq_base, tab);                      \
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
  return err == cudaSuccess ? RD_OK : RD_ERR_CUDA;
}

int launch_kv_append(int kt, int vt, const float *ks, const float *vs, void *kd, void *vd,
                     int64_t width, int head_dim, int heads_per_tok, const int32_t *pos, int n_rot,
                     float freq_base, cudaStream_t st) {
  const int64_t n_blocks = width / 32;
  if (n_blocks == 0) return RD_OK;
#define RD_K(KT)                                                                               \
  case KT:                                                                                     \
    return append_dispatch_v<KT>(vt, ks, vs, (uint8_t *)kd, (uint8_t *)vd, n_blocks, head_dim, \
                                 heads_per_tok, pos, n_rot, freq_base, st);
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

int launch_kv_fill(int type, void *cache, int64_t n_rows, int head_dim, uint32_t seed,
                   cudaStream_t st) {
  const int64_t n_blocks = n_rows * (head_dim / 32);
  if (n_blocks == 0) return RD_OK;
  const unsigned grid = (unsigned)((n_blocks * 32 + 255) / 256);
#define RD_F(T)                                                                       \
  case T:                                                                             \
    kv_fill_kernel<T><<<grid, 256, 0, st>>>((uint8_t *)cache, n_blocks, seed);        \
    break;
  switch (type) {
    RD_F(RD_KV_F32)
    RD_F(RD_KV_F16)
    RD_F(RD_KV_Q8_0)
    RD_F(RD_KV_Q4_0)
    RD_F(RD_KV_Q5_0)
    RD_F(RD_KV_Q4_1)
    default: return RD_ERR_TYPE;
  }
#undef RD_F
  return cudaGetLastError() == cudaSuccess ? RD_OK : RD_ERR_CUDA;
}

int launch_rope(float *x, int n_tok, int n_heads, int head_dim, int n_rot, float freq_base,
                const int32_t *pos, cudaStream_t st) {
  const int64_t total = (int64_t)n_tok * n_heads * (n_rot / 2);
  if (total == 0) return RD_OK;
  rope_kernel<<<(unsigned)((total + 127) / 128), 128, 0, st>>>(x, n_tok, n_heads, head_dim, n_rot,
                                                               freq_base, pos,
                                                               make_rope_table(n_rot, freq_base));
  return cudaGetLastError() == cudaSuccess ? RD_OK : RD_ERR_CUDA;
}

int launch_deinterleave(const float *yq, float *q, float *gate, int64_t n_rows, int head_dim,
                        cudaStream_t st) {
  const int64_t n = n_rows * (head_dim / 4);
  if (n == 0) return RD_OK;
  deinterleave_kernel<<<(unsigned)((n + 255) / 256), 256, 0, st>>>(
      (const float4 *)yq, (float4 *)q, (float4 *)gate, n_rows, head_dim / 4);
  return cudaGetLastError() == cudaSuccess ? RD_OK : RD_ERR_CUDA;
}

int launch_sigmoid_gate(float *g, float *y, int64_t n, cudaStream_t st) {
  if (n == 0) return RD_OK;
  sigmoid_gate_kernel<<<(unsigned)((n + 255) / 256), 256, 0, st>>>(g, y, n);
  return cudaGetLastError() == cudaSuccess ? RD_OK : RD_ERR_CUDA;
}

// ---- stored rows -> f16 rows (the dequantizing loads of include/rdna4/kv.h:174-368) ------
// One thread per 8 consecutive elements (one 16-byte store); the value is formed in f32
// exactly as kv_load does (d * q, d * (n - 8), d * (n5 - 16), d * n + m) and rounded once to
// f16 -- the same value the decode kernel's fragment loaders hand to the tensor cores. Feeds
// the tensor-core prefill kernel when the caches are not f16.
__device__ __forceinline__ uint32_t ld16(const uint8_t *p) { return *reinterpret_cast<const uint16_t *>(p); }

// elements [8 * oct, 8 * oct + 8) of the 32-value block at b
template <int T>
__device__ __forceinline__ void dequant8(const uint8_t *b, int oct, float (&x)[8]) {
  if (T == RD_KV_Q8_0) {
    const float d = f16_bits_to_f32((uint16_t)ld16(b));
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const uint32_t w = ld16(b + 2 + 8 * oct + 2 * i);
      x[2 * i] = d * (float)(int8_t)(w & 0xff);
      x[2 * i + 1] = d * (float)(int8_t)(w >> 8);
    }
    return;
  }
  // 4-bit layouts: element j < 16 is the low nibble of byte j, element j + 16 the high one
  constexpr int QS = T == RD_KV_Q4_0 ? 2 : T == RD_KV_Q4_1 ? 4 : 6;
  const float d = f16_bits_to_f32((uint16_t)ld16(b));
  const float m = T == RD_KV_Q4_1 ? f16_bits_to_f32((uint16_t)ld16(b + 2)) : 0.f;
  const uint32_t qh = T == RD_KV_Q5_0 ? (ld16(b + 2) | (ld16(b + 4) << 16)) : 0u;
  const int sh = oct >= 2 ? 4 : 0;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const uint32_t w = ld16(b + QS + 8 * (oct & 1) + 2 * i);
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      int n = (int)((w >> (8 * h + sh)) & 15u);
      const int j = 8 * oct + 2 * i + h;
      if (T == RD_KV_Q4_0) x[2 * i + h] = d * (float)(n - 8);
      if (T == RD_KV_Q4_1) x[2 * i + h] = __fadd_rn(__fmul_rn(d, (float)n), m);
      if (T == RD_KV_Q5_0) {
        n |= (int)((qh >> j) & 1u) << 4;
        x[2 * i + h] = d * (float)(n - 16);
      }
    }
  }
}

// One CTA = one tile of 256 blocks (8192 values) of one tensor. Quantized types: the tile's
// source bytes (a multiple of 16, 16-byte aligned like the cache) are staged in shared
// memory with coalesced 16-byte loads, then every thread expands four groups of 8 values
// and stores 16 bytes each, coalesced. HBM-bound: one read of the cache, one write of the
// copy. (The first version read the blocks with 2-byte global loads, 8 values per thread:
// 22 us per tensor for 8192 keys where this takes the time of the traffic.)
constexpr int kDqTileBlocks = 256;
template <int T>
__device__ __forceinline__ void dequant_tile(const uint8_t *__restrict__ src, uint4 *__restrict__ dst,
                                             int64_t n_blocks, int64_t tile, uint8_t *stage) {
  const int64_t b0 = tile * kDqTileBlocks;
  const int nb = (int)((n_blocks - b0) < kDqTileBlocks ? (n_blocks - b0) : kDqTileBlocks);
  if (T == RD_KV_F32) {
    for (int o = threadIdx.x; o < nb * 4; o += blockDim.x) {
      const float4 *s4 = reinterpret_cast<const float4 *>(src) + (b0 * 4 + o) * 2;
      const float4 a = s4[0], c = s4[1];
      dst[b0 * 4 + o] = make_uint4(pack_h2(a.x, a.y), pack_h2(a.z, a.w), pack_h2(c.x, c.y), pack_h2(c.z, c.w));
    }
    return;
  }
  if (T == RD_KV_F16) {
    for (int o = threadIdx.x; o < nb * 4; o += blockDim.x)
      dst[b0 * 4 + o] = reinterpret_cast<const uint4 *>(src)[b0 * 4 + o];
    return;
  }
  constexpr int BB = row_bytes(T) / 8;   // bytes per 32-value block: 34 / 18 / 22 / 20
  static_assert((kDqTileBlocks * BB) % 16 == 0, "a tile starts on a 16-byte boundary");
  const uint8_t *tsrc = src + b0 * BB;
  const int n16 = nb * BB / 16, tail = nb * BB - 16 * n16;   // a short last tile may end unaligned
  for (int i = threadIdx.x; i < n16; i += blockDim.x)
    reinterpret_cast<uint4 *>(stage)[i] = reinterpret_cast<const uint4 *>(tsrc)[i];
  if ((int)threadIdx.x < tail) stage[16 * n16 + threadIdx.x] = tsrc[16 * n16 + threadIdx.x];
  __syncthreads();
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const int o = j * (int)blockDim.x + (int)threadIdx.x;   // group of 8 values inside the tile
    if (o < nb * 4) {
      float x[8];
      dequant8<T>(stage + (o >> 2) * BB, o & 3, x);
      dst[b0 * 4 + o] = make_uint4(pack_h2(x[0], x[1]), pack_h2(x[2], x[3]), pack_h2(x[4], x[5]), pack_h2(x[6], x[7]));
    }
  }
}

// blockIdx.y = tensor (0: K, 1: V), each with its own type; a tensor that is f16 already
// (or absent) has src == nullptr and its CTAs leave at once.
__global__ void __launch_bounds__(256)
kv_dequant_f16_kernel(const uint8_t *__restrict__ ksrc, uint4 *__restrict__ kdst, int kt,
                      const uint8_t *__restrict__ vsrc, uint4 *__restrict__ vdst, int vt, int64_t n_blocks) {
  __shared__ __align__(16) uint8_t stage[kDqTileBlocks * 34];
  const uint8_t *src = blockIdx.y == 0 ? ksrc : vsrc;
  uint4 *dst = blockIdx.y == 0 ? kdst : vdst;
  const int type = blockIdx.y == 0 ? kt : vt;
  if (src == nullptr) return;
  switch (type) {   // the same for the whole CTA
    case RD_KV_F32: dequant_tile<RD_KV_F32>(src, dst, n_blocks, blockIdx.x, stage); break;
    case RD_KV_F16: dequant_tile<RD_KV_F16>(src, dst, n_blocks, blockIdx.x, stage); break;
    case RD_KV_Q8_0: dequant_tile<RD_KV_Q8_0>(src, dst, n_blocks, blockIdx.x, stage); break;
    case RD_KV_Q4_0: dequant_tile<RD_KV_Q4_0>(src, dst, n_blocks, blockIdx.x, stage); break;
    case RD_KV_Q5_0: dequant_tile<RD_KV_Q5_0>(src, dst, n_blocks, blockIdx.x, stage); break;
    case RD_KV_Q4_1: dequant_tile<RD_KV_Q4_1>(src, dst, n_blocks, blockIdx.x, stage); break;
    default: break;
  }
}

// Expands K (type kt) into kdst and V (type vt) into vdst as f16, one launch for both; a null
// source skips that tensor. n_values per tensor.
int launch_kv_dequant_f16_pair(int kt, const void *k, void *kdst, int vt, const void *v, void *vdst,
                               int64_t n_values, cudaStream_t st) {
  if (n_values % 32 != 0) return RD_ERR_SHAPE;
  if ((k != nullptr && (kt < 0 || kt > RD_KV_Q4_1)) || (v != nullptr && (vt < 0 || vt > RD_KV_Q4_1))) return RD_ERR_TYPE;
  const int64_t n_blocks = n_values / 32;
  if (n_blocks == 0 || (k == nullptr && v == nullptr)) return RD_OK;
  const dim3 grid((unsigned)((n_blocks + kDqTileBlocks - 1) / kDqTileBlocks), 2);
  kv_dequant_f16_kernel<<<grid, 256, 0, st>>>((const uint8_t *)k, (uint4 *)kdst, kt, (const uint8_t *)v,
                                              (uint4 *)vdst, vt, n_blocks);
  return cudaGetLastError() == cudaSuccess ? RD_OK : RD_ERR_CUDA;
}

int launch_kv_dequant_f16(int type, const void *src, void *dst, int64_t n_values, cudaStream_t st) {
  if (type < 0 || type > RD_KV_Q4_1) return RD_ERR_TYPE;
  return launch_kv_dequant_f16_pair(type, src, dst, RD_KV_F16, nullptr, nullptr, n_values, st);
}

}  // namespace rd
