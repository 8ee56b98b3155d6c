// Quantize-on-store of one 32-value block by one warp (shared by the KV-append kernels
// and the fused pre-attention kernel). Every block must come out byte-identical to the
// reference quantizers (include/rdna4/kv.h:386-501): lane j holds element j, the block
// statistics are warp shuffles, every lane stores its own byte, and the arithmetic is
// pinned with explicit round-to-nearest intrinsics so that no multiply-add is contracted
// into an FMA.
#pragma once
#include "rd_common.cuh"

namespace rd {

// Lane j holds x = element j of the block; writes the block at `dst`.
template <int T>
__device__ __forceinline__ void quant_block_warp(float x, uint8_t *dst, int lane) {
  constexpr unsigned FULL = 0xffffffffu;
  if (T == RD_KV_Q8_0) {
    // kv.h:402-411: amax/127, roundf(x*id).
    float amax = fabsf(x);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(FULL, amax, o));
    const float d = __fdiv_rn(amax, 127.0f);
    const float id = d != 0.0f ? __fdiv_rn(1.0f, d) : 0.0f;
    if (lane == 0) *(uint16_t *)dst = f32_to_f16_bits(d);
    dst[2 + lane] = (uint8_t)(int8_t)__float2int_rz(roundf(__fmul_rn(x, id)));
    return;
  }
  if (T == RD_KV_Q4_1) {
    // kv.h:445-467: affine grid [min, max].
    float vmin = x, vmax = x;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      vmin = fminf(vmin, __shfl_xor_sync(FULL, vmin, o));
      vmax = fmaxf(vmax, __shfl_xor_sync(FULL, vmax, o));
    }
    const float d = __fdiv_rn(__fsub_rn(vmax, vmin), 15.0f);
    const float id = d != 0.0f ? __fdiv_rn(1.0f, d) : 0.0f;
    int q = __float2int_rz(__fadd_rn(__fmul_rn(__fsub_rn(x, vmin), id), 0.5f));
    q = q > 15 ? 15 : (q < 0 ? 0 : q);
    const int qhi = __shfl_down_sync(FULL, q, 16);
    if (lane == 0) {
      *(uint16_t *)dst = f32_to_f16_bits(d);
      *(uint16_t *)(dst + 2) = f32_to_f16_bits(vmin);
    }
    if (lane < 16) dst[4 + lane] = (uint8_t)(q | (qhi << 4));
    return;
  }
  // Q4_0 / Q5_0 (kv.h:412-444, 476-499): the SIGNED value of largest magnitude,
  // first one on ties (the serial scan uses a strict '<'), NaN never selected.
  float a = (x == x) ? fabsf(x) : -1.0f;
  float v = x;
  int idx = lane;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float oa = __shfl_xor_sync(FULL, a, o);
    const float ov = __shfl_xor_sync(FULL, v, o);
    const int oi = __shfl_xor_sync(FULL, idx, o);
    if (oa > a || (oa == a && oi < idx)) {
      a = oa;
      v = ov;
      idx = oi;
    }
  }
  const float vmax = a > 0.0f ? v : 0.0f;
  if (T == RD_KV_Q4_0) {
    const float d = __fdiv_rn(vmax, -8.0f);
    const float id = d != 0.0f ? __fdiv_rn(1.0f, d) : 0.0f;
    int q = __float2int_rz(__fadd_rn(__fmul_rn(x, id), 8.5f));
    q = q > 15 ? 15 : (q < 0 ? 0 : q);
    const int qhi = __shfl_down_sync(FULL, q, 16);
    if (lane == 0) *(uint16_t *)dst = f32_to_f16_bits(d);
    if (lane < 16) dst[2 + lane] = (uint8_t)(q | (qhi << 4));
  } else {  // Q5_0
    const float d = __fdiv_rn(vmax, -16.0f);
    const float id = d != 0.0f ? __fdiv_rn(1.0f, d) : 0.0f;
    int q = __float2int_rz(__fadd_rn(__fmul_rn(x, id), 16.5f));
    q = q > 31 ? 31 : (q < 0 ? 0 : q);
    const int qhi = __shfl_down_sync(FULL, q, 16);
    const unsigned qh = __ballot_sync(FULL, (q & 0x10) != 0);  // bit j = 5th bit of element j
    if (lane == 0) *(uint16_t *)dst = f32_to_f16_bits(d);
    if (lane < 4) dst[2 + lane] = (uint8_t)((qh >> (8 * lane)) & 0xffu);
    if (lane < 16) dst[6 + lane] = (uint8_t)((q & 0x0f) | ((qhi & 0x0f) << 4));
  }
}

template <int T>
__device__ __forceinline__ void store_block(float x, uint8_t *dst_base, int64_t blk, int lane) {
  if (T == RD_KV_F32) {
    ((float *)dst_base)[blk * 32 + lane] = x;
  } else if (T == RD_KV_F16) {
    ((uint16_t *)dst_base)[blk * 32 + lane] = f32_to_f16_bits(x);
  } else {
    constexpr int BB = row_bytes(T) / 8;
    quant_block_warp<T>(x, dst_base + blk * BB, lane);
  }
}

}  // namespace rd
