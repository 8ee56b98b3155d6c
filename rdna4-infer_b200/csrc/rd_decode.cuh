// Split-KV decode attention for sm_100a: one query token (per grid row) against a
// quantized KV cache, all 6 query heads of a GQA group sharing every loaded KV tile.
//
// Shape of the computation (replaces attn_split_kernel, include/rdna4/attn.cuh:445-560,
// and the unsplit attn_kernel, :95-185):
//   * grid (n_splits, n_tok): CTA s owns a contiguous slice of the key tiles and
//     writes one partial record (m, l, acc[256]) per query head;
//   * the CTA's warps form key groups of four (one warp per kv head); every group streams
//     16-key slots through its own ring in shared memory -- one tensor-map (TMA) copy per
//     slot and tensor, the n_head_kv rows of a key being contiguous in the cache, or one
//     bulk copy per key for wide rows -- completion counted on an mbarrier; the warp that
//     finishes a slot last issues the slot's next load, so no warp is only a producer;
//   * warp (kv head, key group) dequantizes its rows IN REGISTERS straight
//     into mma.sync m16n8k16 f16 fragments: QK^T with the 16 keys on M and the 6 heads
//     (padded to 8) on N, then P*V with V^T on M (dims) and the keys on K. The
//     arithmetic intensity of q4_0 (21 flop/byte) is beyond the FP32 pipe at HBM
//     speed, hence tensor-core fragments even for a single query token;
//   * scores live in log2 units (scale*log2e folded into Q), softmax statistics in
//     f32, online rescale only when a running maximum actually moves.
//
// Dequantization in two instructions per pair of values: masking a nibble (or
// placing a byte) into the low mantissa bits of a half gives the SUBNORMAL n * 2^-24
// exactly, and one HFMA2 with the block scale turns it into the value:
//   q4_0: fma(n * 2^-24, d * 2^12, -d * 2^-9)  = d * (n - 8)   * 2^-12
//   q8_0: fma(u * 2^-24, d * 2^12, -d * 2^-5)  = d * (u - 128) * 2^-12   (u = q ^ 0x80)
// rounded once, i.e. as exact as an f16 can hold the dequantized value. The common
// factor 2^-12 keeps every constant a power-of-two multiple of d inside the f16 range
// (block scales up to 16, i.e. |x| < 128 for q4_0) and is undone for free: Q is
// pre-multiplied by 2^12 for the scores, the output accumulator is multiplied by
// 2^12 once at the end.
//
// Index freedom used throughout: the contraction index of an MMA can be permuted
// freely as long as A and B agree, and the M index of P*V (the output dim) can be
// permuted freely as long as the epilogue writes each value to its true dim. Each
// loader below therefore defines `dim()` -- which true dim a fragment slot holds --
// and the Q fragments / epilogue are built from it.
#pragma once
#include "rd_common.cuh"
#include <stdlib.h>
#include <string.h>

#include <type_traits>

#include "rd_internal.h"
#include "rd_quant.cuh"
#include "rd_shard.cuh"

namespace rd {

constexpr uint32_t kH4096 = 0x6C006C00u;    // half2(2^12, 2^12)
constexpr uint32_t kH256 = 0x5C005C00u;     // half2(2^8, 2^8)
constexpr uint32_t kHNeg2m9 = 0x98009800u;  // half2(-2^-9, -2^-9)
constexpr uint32_t kHNeg2m5 = 0xA800A800u;  // half2(-2^-5, -2^-5)
constexpr float kQuantUnscale = 4096.0f;    // undoes the 2^-12 of the quantized loaders

// Per-block constants of the 4-bit path from the half2 scale d.
struct Q4Scale {
  uint32_t lo, hi, c;
  __device__ __forceinline__ explicit Q4Scale(uint32_t d)
      : lo(hmul2(d, kH4096)), hi(hmul2(d, kH256)), c(hmul2(d, kHNeg2m9)) {}
};
// q4_1: value = d*n + m (kv.h:219-229), same trick with the block minimum as the addend:
//   fma(n * 2^-24, d * 2^12, m * 2^-12) = (d*n + m) * 2^-12.
// (m * 2^-12 is a subnormal half for |m| < 1/4: at most 2^-13 of absolute error in the
// value, far inside the attention gates.)
constexpr uint32_t kH2m12 = 0x0C000C00u;    // half2(2^-12, 2^-12)
struct Q41Scale {
  uint32_t lo, hi, c;
  __device__ __forceinline__ Q41Scale(uint32_t d, uint32_t m)
      : lo(hmul2(d, kH4096)), hi(hmul2(d, kH256)), c(hmul2(m, kH2m12)) {}
};
// q5_0: value = d * ((nibble | bit5 << 4) - 16) (kv.h:203-216). The fifth bits of the four
// low-nibble and the four high-nibble elements of a word (bit i = byte i, bits above 7
// clear) are spread to bit 4 of each byte with one multiply -- bit i * 2^(4+7j) lands on
// 4+8j exactly for i == j and on positions the mask drops otherwise -- and OR-ed under the
// masked nibbles; the rest is the q4_0 trick with a 5-bit mantissa field:
//   fma(v * 2^-24, d * 2^12, -d * 2^-8) = d * (v - 16) * 2^-12.
constexpr uint32_t kHNeg2m8 = 0x9C009C00u;  // half2(-2^-8, -2^-8)
struct Q5Scale {
  uint32_t m, c;
  __device__ __forceinline__ explicit Q5Scale(uint32_t d) : m(hmul2(d, kH4096)), c(hmul2(d, kHNeg2m8)) {}
};
//   l0 = (B0.lo, B2.lo), h0 = (B0.hi, B2.hi), l1 = (B1.lo, B3.lo), h1 = (B1.hi, B3.hi)
__device__ __forceinline__ void dq5(uint32_t x, uint32_t bl, uint32_t bh, const Q5Scale &s, uint32_t &l0,
                                    uint32_t &h0, uint32_t &l1, uint32_t &h1) {
  const uint32_t xl = (x & 0x0F0F0F0Fu) | ((bl * 0x02040810u) & 0x10101010u);
  const uint32_t xh = ((x >> 4) & 0x0F0F0F0Fu) | ((bh * 0x02040810u) & 0x10101010u);
  l0 = hfma2(xl & 0x001F001Fu, s.m, s.c);
  l1 = hfma2((xl >> 8) & 0x001F001Fu, s.m, s.c);
  h0 = hfma2(xh & 0x001F001Fu, s.m, s.c);
  h1 = hfma2((xh >> 8) & 0x001F001Fu, s.m, s.c);
}
// One word of 8 nibbles, bytes (B0,B1,B2,B3) -> four half2 of d*(n-8)*2^-12 (Q4Scale) or
// (d*n+m)*2^-12 (Q41Scale):
//   l0 = (B0.lo, B2.lo), h0 = (B0.hi, B2.hi), l1 = (B1.lo, B3.lo), h1 = (B1.hi, B3.hi)
template <class Scale>
__device__ __forceinline__ void dq4(uint32_t x, const Scale &s, uint32_t &l0, uint32_t &h0,
                                    uint32_t &l1, uint32_t &h1) {
  const uint32_t y = x >> 8;
  l0 = hfma2(x & 0x000F000Fu, s.lo, s.c);
  h0 = hfma2(x & 0x00F000F0u, s.hi, s.c);
  l1 = hfma2(y & 0x000F000Fu, s.lo, s.c);
  h1 = hfma2(y & 0x00F000F0u, s.hi, s.c);
}
// Per-block constants of the 8-bit path.
struct Q8Scale {
  uint32_t m, c;
  __device__ __forceinline__ explicit Q8Scale(uint32_t d)
      : m(hmul2(d, kH4096)), c(hmul2(d, kHNeg2m5)) {}
};
// Four biased bytes u = q ^ 0x80: lo = (B0, B1), hi = (B2, B3), each d*q*2^-12.
__device__ __forceinline__ void dq8(uint32_t u, const Q8Scale &s, uint32_t &lo, uint32_t &hi) {
  lo = hfma2(prmt(u, 0u, 0x4140u), s.m, s.c);
  hi = hfma2(prmt(u, 0u, 0x4342u), s.m, s.c);
}

// =============================== K loaders =======================================
// A fragment of Q*K^T for MMA n (0..15): rows = keys g / g+8 of the 16-key group,
// k-slots (2t, 2t+1, 2t+8, 2t+9) = four dims chosen by the loader. run() calls
// mma(n, a0, a1, a2, a3) for n = 0..15. Values come out multiplied by 1/kUnscale.
template <int T>
struct KLoad;

template <>
struct KLoad<RD_KV_Q4_0> {
  static constexpr float kUnscale = kQuantUnscale;
  // lane t owns blocks 2t and 2t+1 of the row: 36 bytes at 36t (4-byte aligned).
  __device__ static int dim(int t, int n, int e) {
    const int x = n >> 1, odd = n & 1;
    int blk, i0, i2;
    if (x < 3) {
      blk = 2 * t; i0 = 4 * x + 2 + odd; i2 = i0 + 2;
    } else if (x == 3) {
      blk = 2 * t; i0 = odd; i2 = 14 + odd;
    } else {
      blk = 2 * t + 1; i0 = 4 * (x - 4) + odd; i2 = i0 + 2;
    }
    return blk * 32 + ((e & 1) ? i2 : i0) + ((e & 2) ? 16 : 0);
  }
  template <class F>
  __device__ static void run(uint32_t row_g, uint32_t row_h, int t, F &&mma) {
    uint32_t wg[9], wh[9];
    row_g += 36 * t;
    row_h += 36 * t;
#pragma unroll
    for (int i = 0; i < 9; ++i) {
      wg[i] = lds32(row_g + 4 * i);
      wh[i] = lds32(row_h + 4 * i);
    }
#pragma unroll
    for (int b = 0; b < 2; ++b) {
      const uint32_t dg = b == 0 ? prmt(wg[0], wg[0], 0x1010u) : prmt(wg[4], wg[4], 0x3232u);
      const uint32_t dh = b == 0 ? prmt(wh[0], wh[0], 0x1010u) : prmt(wh[4], wh[4], 0x3232u);
      const Q4Scale sg(dg), sh(dh);
#pragma unroll
      for (int xx = 0; xx < 4; ++xx) {
        const int x = 4 * b + xx;
        const uint32_t xg = (x == 3) ? prmt(wg[0], wg[4], 0x5432u) : wg[x + 1];
        const uint32_t xh = (x == 3) ? prmt(wh[0], wh[4], 0x5432u) : wh[x + 1];
        uint32_t l0g, h0g, l1g, h1g, l0h, h0h, l1h, h1h;
        dq4(xg, sg, l0g, h0g, l1g, h1g);
        dq4(xh, sh, l0h, h0h, l1h, h1h);
        mma(2 * x, l0g, l0h, h0g, h0h);
        mma(2 * x + 1, l1g, l1h, h1g, h1h);
      }
    }
  }
};

template <>
struct KLoad<RD_KV_Q8_0> {
  static constexpr float kUnscale = kQuantUnscale;
  // lane t owns blocks 2t and 2t+1: 68 bytes at 68t.
  __device__ static int dim(int t, int n, int e) {
    if (n < 7) return (2 * t) * 32 + 4 * n + 2 + e;
    if (n == 7) return (2 * t) * 32 + (e < 2 ? e : 28 + e);
    return (2 * t + 1) * 32 + 4 * (n - 8) + e;
  }
  template <class F>
  __device__ static void run(uint32_t row_g, uint32_t row_h, int t, F &&mma) {
    uint32_t wg[17], wh[17];
    row_g += 68 * t;
    row_h += 68 * t;
#pragma unroll
    for (int i = 0; i < 17; ++i) {
      wg[i] = lds32(row_g + 4 * i);
      wh[i] = lds32(row_h + 4 * i);
    }
#pragma unroll
    for (int b = 0; b < 2; ++b) {
      const uint32_t dg = b == 0 ? prmt(wg[0], wg[0], 0x1010u) : prmt(wg[8], wg[8], 0x3232u);
      const uint32_t dh = b == 0 ? prmt(wh[0], wh[0], 0x1010u) : prmt(wh[8], wh[8], 0x3232u);
      const Q8Scale sg(dg), sh(dh);
#pragma unroll
      for (int xx = 0; xx < 8; ++xx) {
        const int x = 8 * b + xx;
        uint32_t xg = (x == 7) ? prmt(wg[0], wg[8], 0x5432u) : wg[x + 1];
        uint32_t xh = (x == 7) ? prmt(wh[0], wh[8], 0x5432u) : wh[x + 1];
        xg ^= 0x80808080u;
        xh ^= 0x80808080u;
        uint32_t log_, hig, loh, hih;
        dq8(xg, sg, log_, hig);
        dq8(xh, sh, loh, hih);
        mma(x, log_, loh, hig, hih);
      }
    }
  }
};

template <>
struct KLoad<RD_KV_F16> {
  static constexpr float kUnscale = 1.0f;
  // lane t owns the 16-byte chunks 8*(i>>1) + 2t + (i&1), i = 0..7 (conflict-free with
  // a key pitch of 16 bytes mod 128).
  __device__ static int dim(int t, int n, int e) {
    const int i = n >> 1;
    const int c = 8 * (i >> 1) + 2 * t + (i & 1);
    return 8 * c + 4 * (n & 1) + e;
  }
  template <class F>
  __device__ static void run(uint32_t row_g, uint32_t row_h, int t, F &&mma) {
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int c = 8 * (i >> 1) + 2 * t + (i & 1);
      const uint4 vg = lds128(row_g + 16 * c);
      const uint4 vh = lds128(row_h + 16 * c);
      mma(2 * i, vg.x, vh.x, vg.y, vh.y);
      mma(2 * i + 1, vg.z, vh.z, vg.w, vh.w);
    }
  }
};

template <>
struct KLoad<RD_KV_F32> {
  static constexpr float kUnscale = 1.0f;
  // lane t owns the 16-byte chunks (4 dims) 4i + t, i = 0..15. Values are rounded to
  // f16 for the tensor core (f32 caches are a debugging format in the reference).
  __device__ static int dim(int t, int n, int e) { return 4 * (4 * n + t) + e; }
  template <class F>
  __device__ static void run(uint32_t row_g, uint32_t row_h, int t, F &&mma) {
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      const uint4 vg = lds128(row_g + 16 * (4 * i + t));
      const uint4 vh = lds128(row_h + 16 * (4 * i + t));
      mma(i, pack_h2(__uint_as_float(vg.x), __uint_as_float(vg.y)),
          pack_h2(__uint_as_float(vh.x), __uint_as_float(vh.y)),
          pack_h2(__uint_as_float(vg.z), __uint_as_float(vg.w)),
          pack_h2(__uint_as_float(vh.z), __uint_as_float(vh.w)));
    }
  }
};

// ---- q5_0 / q4_1: the reference's default 131K configuration stores K as q5_0 and V as
// q4_1 (include/rdna4/kv.h:75-98); kv_load of kv.h:203-229 restated on fragments.
template <>
struct KLoad<RD_KV_Q5_0> {
  static constexpr float kUnscale = kQuantUnscale;
  // lane t owns blocks 2t and 2t+1 of the row: 44 bytes at 44t = eleven aligned words.
  // Block 2t is d | qh | 16 nibble bytes from byte 0, so its qh and nibble words straddle
  // two loaded words (realigned with PRMT); block 2t+1 starts at byte 22: d is the upper
  // half of word 5, qh is word 6 and the nibbles are words 7..10.
  __device__ static int dim(int t, int n, int e) {
    const int x = n >> 1;
    return (2 * t + (x >> 2)) * 32 + 4 * (x & 3) + (n & 1) + ((e & 1) ? 2 : 0) + ((e & 2) ? 16 : 0);
  }
  template <class F>
  __device__ static void run(uint32_t row_g, uint32_t row_h, int t, F &&mma) {
    uint32_t wg[11], wh[11];
#pragma unroll
    for (int i = 0; i < 11; ++i) {
      wg[i] = lds32(row_g + 44 * t + 4 * i);
      wh[i] = lds32(row_h + 44 * t + 4 * i);
    }
#pragma unroll
    for (int b = 0; b < 2; ++b) {
      const Q5Scale sg(b == 0 ? prmt(wg[0], wg[0], 0x1010u) : prmt(wg[5], wg[5], 0x3232u));
      const Q5Scale sh(b == 0 ? prmt(wh[0], wh[0], 0x1010u) : prmt(wh[5], wh[5], 0x3232u));
      const uint32_t qhg = b == 0 ? prmt(wg[0], wg[1], 0x5432u) : wg[6];
      const uint32_t qhh = b == 0 ? prmt(wh[0], wh[1], 0x5432u) : wh[6];
#pragma unroll
      for (int xx = 0; xx < 4; ++xx) {
        const int x = 4 * b + xx;
        const uint32_t xg = b == 0 ? prmt(wg[1 + xx], wg[2 + xx], 0x5432u) : wg[7 + xx];
        const uint32_t xh = b == 0 ? prmt(wh[1 + xx], wh[2 + xx], 0x5432u) : wh[7 + xx];
        uint32_t l0g, h0g, l1g, h1g, l0h, h0h, l1h, h1h;
        dq5(xg, (qhg >> (4 * xx)) & 0xFu, (qhg >> (16 + 4 * xx)) & 0xFu, sg, l0g, h0g, l1g, h1g);
        dq5(xh, (qhh >> (4 * xx)) & 0xFu, (qhh >> (16 + 4 * xx)) & 0xFu, sh, l0h, h0h, l1h, h1h);
        mma(2 * x, l0g, l0h, h0g, h0h);
        mma(2 * x + 1, l1g, l1h, h1g, h1h);
      }
    }
  }
};
template <>
struct KLoad<RD_KV_Q4_1> {
  static constexpr float kUnscale = kQuantUnscale;
  // lane t owns blocks t and t+4 of the row: five aligned words each ((d, m), then four
  // words of nibbles) at 20t and 20t + 80. (Blocks 2t and 2t+1 would put the four lanes
  // of a row 10 words apart: with the row pitch of 4 words mod 32 that is a 2-way bank
  // conflict on every load; 5 words apart is conflict-free.)
  __device__ static int dim(int t, int n, int e) {
    const int x = n >> 1;
    return (t + 4 * (x >> 2)) * 32 + 4 * (x & 3) + (n & 1) + ((e & 1) ? 2 : 0) + ((e & 2) ? 16 : 0);
  }
  template <class F>
  __device__ static void run(uint32_t row_g, uint32_t row_h, int t, F &&mma) {
#pragma unroll
    for (int b = 0; b < 2; ++b) {   // one block at a time: ten words live, not twenty
      uint32_t wg[5], wh[5];
#pragma unroll
      for (int i = 0; i < 5; ++i) {
        wg[i] = lds32(row_g + 20 * t + 80 * b + 4 * i);
        wh[i] = lds32(row_h + 20 * t + 80 * b + 4 * i);
      }
      const Q41Scale sg(prmt(wg[0], wg[0], 0x1010u), prmt(wg[0], wg[0], 0x3232u));
      const Q41Scale sh(prmt(wh[0], wh[0], 0x1010u), prmt(wh[0], wh[0], 0x3232u));
#pragma unroll
      for (int xx = 0; xx < 4; ++xx) {
        const int x = 4 * b + xx;
        uint32_t l0g, h0g, l1g, h1g, l0h, h0h, l1h, h1h;
        dq4(wg[1 + xx], sg, l0g, h0g, l1g, h1g);
        dq4(wh[1 + xx], sh, l0h, h0h, l1h, h1h);
        mma(2 * x, l0g, l0h, h0g, h0h);
        mma(2 * x + 1, l1g, l1h, h1g, h1h);
      }
    }
  }
};

// =============================== V loaders =======================================
// A fragment of V^T*P for M-tile m (0..15): rows g / g+8 = two true dims chosen by
// the loader (dim(g, m, r)), k-slots = keys (2t, 2t+1, 2t+8, 2t+9) of the group.
// kPairM says which two accumulator values of a lane are neighbours in memory (the
// epilogue stores them as one 8-byte word): true, dim(g, m + 1, r) = dim(g, m, r) + 1 for
// even m; false, dim(g, m, 1) = dim(g, m, 0) + 1. Either way the first dim is even.
// rows[j] is the shared address of the stored row of key j of those four. run()
// calls mma(m, a0, a1, a2, a3) for m = 0..15. Values come out multiplied by 1/kUnscale.
template <int T>
struct VLoad;

template <>
struct VLoad<RD_KV_Q4_0> {
  static constexpr bool kPairM = true;
  static constexpr float kUnscale = kQuantUnscale;
  // lane g owns block g of each key: 18 bytes at 18g, read as 5 aligned words from
  // (18g & ~3); for odd g the block starts in the upper half of the first word.
  __device__ static int hidx(int s, int par) { return s <= 6 ? s + 1 - par : (par ? 7 : 0); }
  __device__ static int dim(int g, int m, int r) {
    return 32 * g + 2 * hidx(m >> 1, g & 1) + (m & 1) + (r ? 16 : 0);
  }
  template <class F>
  __device__ static void run(const uint32_t (&rows)[4], int g, F &&mma) {
    const uint32_t off = (18u * g) & ~3u;
    const bool par = g & 1;
    uint32_t w[4][5];
#pragma unroll
    for (int j = 0; j < 4; ++j)
#pragma unroll
      for (int i = 0; i < 5; ++i) w[j][i] = lds32(rows[j] + off + 4 * i);
    const uint32_t seld = par ? 0x7632u : 0x5410u;
    const uint32_t dab = prmt(w[0][0], w[1][0], seld);
    const uint32_t dcd = prmt(w[2][0], w[3][0], seld);
    const Q4Scale sab(dab), scd(dcd);
#pragma unroll
    for (int s = 0; s < 8; ++s) {
      uint32_t xab, xcd;
      if (s < 7) {
        const int i = 1 + (s >> 1);
        const uint32_t sel = (s & 1) ? 0x7632u : 0x5410u;
        xab = prmt(w[0][i], w[1][i], sel);
        xcd = prmt(w[2][i], w[3][i], sel);
      } else {
        xab = prmt(par ? w[0][4] : w[0][0], par ? w[1][4] : w[1][0], 0x7632u);
        xcd = prmt(par ? w[2][4] : w[2][0], par ? w[3][4] : w[3][0], 0x7632u);
      }
      uint32_t l0a, h0a, l1a, h1a, l0c, h0c, l1c, h1c;
      dq4(xab, sab, l0a, h0a, l1a, h1a);
      dq4(xcd, scd, l0c, h0c, l1c, h1c);
      mma(2 * s, l0a, h0a, l0c, h0c);
      mma(2 * s + 1, l1a, h1a, l1c, h1c);
    }
  }
};

template <>
struct VLoad<RD_KV_Q8_0> {
  static constexpr bool kPairM = false;
  static constexpr float kUnscale = kQuantUnscale;
  // lane g owns block g: 34 bytes at 34g, read as 9 aligned words from (34g & ~3).
  __device__ static int hidx(int s, int par) { return s <= 14 ? s + 1 - par : (par ? 15 : 0); }
  __device__ static int dim(int g, int m, int r) { return 32 * g + 2 * hidx(m, g & 1) + r; }
  template <class F>
  __device__ static void run(const uint32_t (&rows)[4], int g, F &&mma) {
    const uint32_t off = (34u * g) & ~3u;
    const bool par = g & 1;
    uint32_t w[4][9];
#pragma unroll
    for (int j = 0; j < 4; ++j)
#pragma unroll
      for (int i = 0; i < 9; ++i) w[j][i] = lds32(rows[j] + off + 4 * i);
    const uint32_t seld = par ? 0x7632u : 0x5410u;
    const uint32_t dab = prmt(w[0][0], w[1][0], seld);
    const uint32_t dcd = prmt(w[2][0], w[3][0], seld);
    const Q8Scale sab(dab), scd(dcd);
#pragma unroll
    for (int s = 0; s < 16; ++s) {
      uint32_t tab, tcd;  // bytes (a.b0, b.b0, a.b1, b.b1) of the 2-byte slot
      if (s < 15) {
        const int i = 1 + (s >> 1);
        const uint32_t sel = (s & 1) ? 0x7362u : 0x5140u;
        tab = prmt(w[0][i], w[1][i], sel);
        tcd = prmt(w[2][i], w[3][i], sel);
      } else {
        tab = prmt(par ? w[0][8] : w[0][0], par ? w[1][8] : w[1][0], 0x7362u);
        tcd = prmt(par ? w[2][8] : w[2][0], par ? w[3][8] : w[3][0], 0x7362u);
      }
      tab ^= 0x80808080u;
      tcd ^= 0x80808080u;
      uint32_t e0a, e1a, e0c, e1c;
      dq8(tab, sab, e0a, e1a);
      dq8(tcd, scd, e0c, e1c);
      mma(s, e0a, e1a, e0c, e1c);
    }
  }
};

template <>
struct VLoad<RD_KV_F16> {
  static constexpr bool kPairM = false;
  static constexpr float kUnscale = 1.0f;
  // lane g owns the 16-byte chunks g + 8*ci, ci = 0..3, of each key.
  __device__ static int dim(int g, int m, int r) { return 8 * (g + 8 * (m >> 2)) + 2 * (m & 3) + r; }
  template <class F>
  __device__ static void run(const uint32_t (&rows)[4], int g, F &&mma) {
#pragma unroll
    for (int ci = 0; ci < 4; ++ci) {
      const uint32_t o = 16 * (g + 8 * ci);
      const uint4 a = lds128(rows[0] + o), b = lds128(rows[1] + o);
      const uint4 c = lds128(rows[2] + o), d = lds128(rows[3] + o);
      mma(4 * ci + 0, prmt(a.x, b.x, 0x5410u), prmt(a.x, b.x, 0x7632u), prmt(c.x, d.x, 0x5410u),
          prmt(c.x, d.x, 0x7632u));
      mma(4 * ci + 1, prmt(a.y, b.y, 0x5410u), prmt(a.y, b.y, 0x7632u), prmt(c.y, d.y, 0x5410u),
          prmt(c.y, d.y, 0x7632u));
      mma(4 * ci + 2, prmt(a.z, b.z, 0x5410u), prmt(a.z, b.z, 0x7632u), prmt(c.z, d.z, 0x5410u),
          prmt(c.z, d.z, 0x7632u));
      mma(4 * ci + 3, prmt(a.w, b.w, 0x5410u), prmt(a.w, b.w, 0x7632u), prmt(c.w, d.w, 0x5410u),
          prmt(c.w, d.w, 0x7632u));
    }
  }
};

template <>
struct VLoad<RD_KV_F32> {
  static constexpr bool kPairM = false;
  static constexpr float kUnscale = 1.0f;
  // lane g owns the 16-byte chunks (4 dims) g + 8*ci, ci = 0..7.
  __device__ static int dim(int g, int m, int r) { return 4 * (g + 8 * (m >> 1)) + 2 * (m & 1) + r; }
  template <class F>
  __device__ static void run(const uint32_t (&rows)[4], int g, F &&mma) {
#pragma unroll
    for (int ci = 0; ci < 8; ++ci) {
      const uint32_t o = 16 * (g + 8 * ci);
      const uint4 a = lds128(rows[0] + o), b = lds128(rows[1] + o);
      const uint4 c = lds128(rows[2] + o), d = lds128(rows[3] + o);
#define RD_F(x) __uint_as_float(x)
      mma(2 * ci, pack_h2(RD_F(a.x), RD_F(b.x)), pack_h2(RD_F(a.y), RD_F(b.y)),
          pack_h2(RD_F(c.x), RD_F(d.x)), pack_h2(RD_F(c.y), RD_F(d.y)));
      mma(2 * ci + 1, pack_h2(RD_F(a.z), RD_F(b.z)), pack_h2(RD_F(a.w), RD_F(b.w)),
          pack_h2(RD_F(c.z), RD_F(d.z)), pack_h2(RD_F(c.w), RD_F(d.w)));
#undef RD_F
    }
  }
};

template <>
struct VLoad<RD_KV_Q5_0> {
  static constexpr bool kPairM = true;
  static constexpr float kUnscale = kQuantUnscale;
  // lane g owns block g of each key: 22 bytes at 22g, read as six aligned words from
  // (22g & ~3); for odd g the block starts in the upper half of the first word, which
  // shifts d, qh and the nibble words by two bytes (one PRMT selector per case).
  __device__ static int dim(int g, int m, int r) { return 32 * g + m + 16 * r; }
  template <class F>
  __device__ static void run(const uint32_t (&rows)[4], int g, F &&mma) {
    const uint32_t off = (22u * g) & ~3u;
    const bool par = g & 1;
    const uint32_t sel = par ? 0x7654u : 0x5432u;   // odd g: the next word is already aligned
    uint32_t dd[4], qh[4], qs[4][4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      uint32_t w[6];
#pragma unroll
      for (int i = 0; i < 6; ++i) w[i] = lds32(rows[j] + off + 4 * i);
      dd[j] = prmt(w[0], w[0], par ? 0x3232u : 0x1010u);
      qh[j] = prmt(w[0], w[1], sel);
#pragma unroll
      for (int x = 0; x < 4; ++x) qs[j][x] = prmt(w[1 + x], w[2 + x], sel);
    }
    const Q5Scale sab(prmt(dd[0], dd[1], 0x5410u)), scd(prmt(dd[2], dd[3], 0x5410u));
    // fifth bits of element pairs, two keys side by side: nibble (s & ~1) * 2 of pe (even
    // slots s) / po (odd slots) holds (key0 bits 2s, 2s+1 | key1 bits 2s, 2s+1)
    const uint32_t pe_ab = (qh[0] & 0x33333333u) | ((qh[1] & 0x33333333u) << 2);
    const uint32_t po_ab = ((qh[0] >> 2) & 0x33333333u) | (qh[1] & 0xCCCCCCCCu);
    const uint32_t pe_cd = (qh[2] & 0x33333333u) | ((qh[3] & 0x33333333u) << 2);
    const uint32_t po_cd = ((qh[2] >> 2) & 0x33333333u) | (qh[3] & 0xCCCCCCCCu);
#pragma unroll
    for (int s = 0; s < 8; ++s) {   // bytes 2s, 2s+1 of the nibbles: elements 2s, 2s+1 (+16)
      const uint32_t psel = (s & 1) ? 0x7632u : 0x5410u;
      const uint32_t xab = prmt(qs[0][s >> 1], qs[1][s >> 1], psel);
      const uint32_t xcd = prmt(qs[2][s >> 1], qs[3][s >> 1], psel);
      const int sh = 4 * (s >> 1);
      const uint32_t bab = (s & 1) ? po_ab : pe_ab, bcd = (s & 1) ? po_cd : pe_cd;
      uint32_t l0a, h0a, l1a, h1a, l0c, h0c, l1c, h1c;
      dq5(xab, (bab >> sh) & 0xFu, (bab >> (16 + sh)) & 0xFu, sab, l0a, h0a, l1a, h1a);
      dq5(xcd, (bcd >> sh) & 0xFu, (bcd >> (16 + sh)) & 0xFu, scd, l0c, h0c, l1c, h1c);
      mma(2 * s, l0a, h0a, l0c, h0c);
      mma(2 * s + 1, l1a, h1a, l1c, h1c);
    }
  }
};
template <>
struct VLoad<RD_KV_Q4_1> {
  static constexpr bool kPairM = true;
  static constexpr float kUnscale = kQuantUnscale;
  // lane g owns block g of each key: 20 bytes at 20g = five aligned words.
  __device__ static int dim(int g, int m, int r) { return 32 * g + m + 16 * r; }
  template <class F>
  __device__ static void run(const uint32_t (&rows)[4], int g, F &&mma) {
    uint32_t w[4][5];
#pragma unroll
    for (int j = 0; j < 4; ++j)
#pragma unroll
      for (int i = 0; i < 5; ++i) w[j][i] = lds32(rows[j] + 20u * g + 4 * i);
    // half2 across two keys: (key a, key b) and (key c, key d), each with its own (d, m)
    const Q41Scale sab(prmt(w[0][0], w[1][0], 0x5410u), prmt(w[0][0], w[1][0], 0x7632u));
    const Q41Scale scd(prmt(w[2][0], w[3][0], 0x5410u), prmt(w[2][0], w[3][0], 0x7632u));
#pragma unroll
    for (int s = 0; s < 8; ++s) {   // bytes 2s, 2s+1 of the nibbles: elements 2s, 2s+1 (+16)
      const int i = 1 + (s >> 1);
      const uint32_t sel = (s & 1) ? 0x7632u : 0x5410u;
      const uint32_t xab = prmt(w[0][i], w[1][i], sel);
      const uint32_t xcd = prmt(w[2][i], w[3][i], sel);
      uint32_t l0a, h0a, l1a, h1a, l0c, h0c, l1c, h1c;
      dq4(xab, sab, l0a, h0a, l1a, h1a);
      dq4(xcd, scd, l0c, h0c, l1c, h1c);
      mma(2 * s, l0a, h0a, l0c, h0c);
      mma(2 * s + 1, l1a, h1a, l1c, h1c);
    }
  }
};

// =============================== kernel ==========================================
struct DecodeKernelArgs {
  // Tensor maps over the K / V caches (see encode_kv_tmap): one box = one slot of 16
  // keys in the padded shared-memory layout; used when k_tmap / v_tmap is set.
  alignas(64) CUtensorMap tm_k;
  alignas(64) CUtensorMap tm_v;
  int k_tmap;
  int v_tmap;
  const float *q;
  const uint8_t *k;
  const uint8_t *v;
  float *partial;
  const int32_t *pos;
  int t;
  int key_begin;
  int n_head;
  int nkv;
  float qscale;  // scale * log2(e)
  int depth;     // ring slots per key group
  int group_bytes;  // shared memory per key group: its ring, at least one epilogue plane
#ifdef RD_TIMING_SWITCHES
  int debug;  // timing experiments only, bit mask: 1 skip all math, 2 skip the copies, 4 skip QK,
              // 8 skip PV, 32 thread 0 overwrites its first record with clock readings
#endif
  DeviceStatus *status;
  // Multi-sequence launches (MULTI): one CTA per work item (sequence, token, split);
  // everything per-sequence comes from the descriptor instead of the fields above.
  const DecodeSeq *seqs;
  const int4 *items;
  int q_len;
  // Fused append (single-sequence launches): quantize k_new / v_new [nkv][256] into cache
  // row new_row; null = nothing to append.
  const float *k_new;
  const float *v_new;
  int new_row;
  // Context-sharded calls (single-sequence launches, push.world > 0): once every CTA's
  // records are written, the first n_head * 4 CTAs reduce them per (head, dim quarter),
  // store the parts into every rank's exchange buffer, wait for the other ranks' parts and
  // merge -- the whole exchange of rd_shard.cu inside this launch.
  ShardPeers push;
  float *x_out;    // [n_head][256]: the merged output of a context-sharded call
  float *x_gate;   // optional fused sigmoid gate of that output
};

// acq_rel: the slot reads of the arriving warp happen before the refill the last
// arriver issues.
__device__ __forceinline__ uint32_t atom_add_acq_rel_shared(uint32_t addr, uint32_t v) {
  uint32_t old;
  asm volatile("atom.acq_rel.cta.shared::cta.add.u32 %0, [%1], %2;" : "=r"(old) : "r"(addr), "r"(v) : "memory");
  return old;
}
__device__ __forceinline__ void sts32(uint32_t addr, uint32_t v) {
  asm volatile("st.shared.u32 [%0], %1;" ::"r"(addr), "r"(v) : "memory");
}
__device__ __forceinline__ void st_global_f2(float *p, float a, float b) {
  *reinterpret_cast<float2 *>(p) = make_float2(a, b);
}

// Warps: 4 per key group (one per kv head), G groups. Nobody is only a producer: the
// warp that is last to finish a slot re-arms it and issues the slot's next load, so a
// CTA of 12 warps leaves each of them 168 registers (13 warps would cap them at 128:
// the register file is split four ways and one quarter would hold four warps).
//
// Softmax reference: p = exp2(s - m) is taken against a reference m that is only moved
// (and the accumulators rescaled) when a score exceeds it by more than kRefSlack, so
// p <= 2^kRefSlack -- exact enough in f16 and far from overflow -- and the rescale runs
// once or twice per CTA instead of on every new maximum. The true running maximum is
// kept per lane and becomes the record's m at the end.
constexpr float kRefSlack = 8.0f;
constexpr int kPlaneHead = 268;   // floats per head in the epilogue planes (12 mod 32)

template <int KT, int VT, bool MULTI>
__global__ void __launch_bounds__(4 * key_groups(KT, VT) * 32, 1)
decode_kernel(const __grid_constant__ DecodeKernelArgs p) {
  constexpr int G = key_groups(KT, VT);
  constexpr int NW = 4 * G;
  constexpr int NT = NW * 32;
  constexpr int RK = row_bytes(KT), RV = row_bytes(VT);
  using KL = KLoad<KT>;
  using VL = VLoad<VT>;
  constexpr unsigned FULL = 0xffffffffu;

  extern __shared__ __align__(128) uint8_t smem[];
  __shared__ int s_abort;
  // per (group, kv head * 8 + column): softmax reference, true maximum, row sum
  __shared__ float s_m[kMaxGroups][32], s_t[kMaxGroups][32], s_l[kMaxGroups][32];
  pdl_launch_dependents();
  if constexpr (!MULTI) {
    // the tensor maps are kernel parameters: start fetching them now
    if (threadIdx.x == 0 && p.k_tmap) asm volatile("prefetch.tensormap [%0];" ::"l"(&p.tm_k) : "memory");
    if (threadIdx.x == 32 && p.v_tmap) asm volatile("prefetch.tensormap [%0];" ::"l"(&p.tm_v) : "memory");
  }
#ifdef RD_TIMING_SWITCHES
  long long tr[8];
  unsigned long long gt0;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(gt0));
  tr[0] = clock64();
#define RD_TRACE(i) tr[i] = clock64()
#else
#define RD_TRACE(i)
#endif

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, tq = lane & 3;
  const int gi = warp >> 2, kvh = warp & 3;
  const int nkv = p.nkv;
  const bool active = kvh < nkv;
  const int D = p.depth;
  const int pitch_k = nkv * RK + 16, pitch_v = nkv * RV + 16;
  const uint32_t slot_sz = (uint32_t)kSlotKeys * (pitch_k + pitch_v);
  const uint32_t v_slot_off = kSlotKeys * pitch_k;
  // Shared-memory layout: ring position (group, d) = index group * D + d owns a full
  // barrier, an arrival counter, a fill count and the number of the slot it holds; then
  // the query fragments; then the rings, group
  // after group (p.group_bytes apart: a group's ring also holds its epilogue plane).
  const uint32_t bar_full = smem_u32(smem);                       // 24 x 8 bytes
  const uint32_t cnt0 = bar_full + 8 * kMaxPos;   // 24 x 4 bytes
  const uint32_t nfill0 = cnt0 + 4 * kMaxPos;     // 24 x 4 bytes
  const uint32_t sid0 = nfill0 + 4 * kMaxPos;     // 24 x 4 bytes: slot held, or -1
  uint8_t *qstage = smem + kBarBytes;
  const uint32_t ring0 = bar_full + kRingOffset;                  // 128-byte aligned
  const uint32_t group_bytes = (uint32_t)p.group_bytes;

  // ---- set-up that needs nothing from global memory --------------------------------
  if (threadIdx.x == 0) {
    s_abort = 0;
    for (int i = 0; i < G * D; ++i) {
      mbar_init(bar_full + 8 * i, 1);
      sts32(cnt0 + 4 * i, 0u);
      sts32(nfill0 + 4 * i, 0u);
    }
    fence_barrier_init();
  }
  // Query fragments. Lane (g, tq) of every warp of a kv head needs the same 32 words:
  // head g's values at the dims KL::dim(tq, n, 0..3), n = 0..15, as f16 pairs pre-scaled
  // into log2 units (and by the loader's fixed-point factor). The threads build them
  // cooperatively: a 256-entry table inverts KL::dim (dim -> fragment slot), every thread
  // then loads query values coalesced and drops each as an f16 into its slot, 144 bytes
  // per (head, tq), and every lane reads its 32 words with 8 conflict-free 16-byte loads
  // -- instead of 64 scalar gathers per lane, repeated by every key-group warp.
  unsigned short *inv = reinterpret_cast<unsigned short *>(qstage);           // 512 bytes
  const uint32_t frag0 = smem_u32(qstage) + 512;
  for (int i = threadIdx.x; i < 256; i += NT) {
    const int tq_i = i >> 6, n_i = (i >> 2) & 15, e_i = i & 3;
    // byte offset of the half inside the (head, tq) block: word 2n + (e >> 1), half e & 1
    inv[KL::dim(tq_i, n_i, e_i)] = (unsigned short)(tq_i * kFragPitch + (2 * n_i + (e_i >> 1)) * 4 +
                                                    (e_i & 1) * 2);
  }
  pdl_wait();   // everything below reads what earlier kernels of the stream wrote
  RD_TRACE(1);

  // What this CTA works on: token qt, split s of S, keys key_begin..t_last of the caches
  // at kbase / vbase (or behind the tensor maps tmk / tmv), one record per head at
  // rec0 + head * S * kRec.
  int qt, s, S, t_last, key_begin, use_tk, use_tv;
  const float *qsrc;
  const uint8_t *kbase, *vbase;
  const CUtensorMap *tmk, *tmv;
  float *rec0;
  if constexpr (MULTI) {
    const int4 item = p.items[blockIdx.x];
    if (item.x < 0) return;   // padding of a plan with a fixed item count
    const DecodeSeq &d = p.seqs[item.x];
    qt = item.y;
    s = item.z;
    S = d.n_splits;
    t_last = d.t - (p.q_len - 1 - qt);  // causal inside the block of q_len new tokens
    key_begin = 0;
    use_tk = d.k_tmap;
    use_tv = d.v_tmap;
    qsrc = d.q + (size_t)qt * p.n_head * kHeadDim;
    kbase = d.k;
    vbase = d.v;
    tmk = reinterpret_cast<const CUtensorMap *>(d.tm_k);
    tmv = reinterpret_cast<const CUtensorMap *>(d.tm_v);
    rec0 = p.partial + ((size_t)d.rec_base + (size_t)qt * p.n_head * S + s) * kRec;
    // These descriptors were written to global memory by an ordinary copy and may have
    // been rewritten since an earlier launch read them: make the copy visible to the
    // tensor-map proxy of every thread that may issue a load through them.
    if (lane == 0 || lane == 16) {
      if (use_tk)
        asm volatile("fence.proxy.tensormap::generic.acquire.gpu [%0], 128;" ::"l"(tmk) : "memory");
      if (use_tv)
        asm volatile("fence.proxy.tensormap::generic.acquire.gpu [%0], 128;" ::"l"(tmv) : "memory");
    }
  } else {
    qt = blockIdx.y;
    s = blockIdx.x;
    S = gridDim.x;
    t_last = p.pos != nullptr ? p.pos[qt] : p.t;
    key_begin = p.key_begin;
    use_tk = p.k_tmap;
    use_tv = p.v_tmap;
    qsrc = p.q + (size_t)qt * p.n_head * kHeadDim;
    kbase = p.k;
    vbase = p.v;
    tmk = &p.tm_k;
    tmv = &p.tm_v;
    rec0 = p.partial + ((size_t)qt * p.n_head * S + s) * kRec;
  }
  // Key split in 16-key slots: CTA s owns slots [c_b, c_e) of the attended range and
  // deals them round-robin to its key groups (group x: local slots x, x + G, ...), so the
  // order of every sum is fixed by the shape alone.
  const int n_keys = t_last >= key_begin ? t_last - key_begin + 1 : 0;
  const int slots_total = (n_keys + kSlotKeys - 1) / kSlotKeys;
  const int c_b = (int)(((int64_t)slots_total * s) / S);
  const int c_e = (int)(((int64_t)slots_total * (s + 1)) / S);
  const int n_slots = c_e - c_b;
  const int key0 = key_begin + c_b * kSlotKeys;
  const uint32_t kb = (uint32_t)nkv * RK, vb = (uint32_t)nkv * RV;

  // The query rows of this token: requested before anything else, so that they do not
  // queue behind the first lap of slot loads.
  const float4 *q4 = reinterpret_cast<const float4 *>(qsrc);
  const int n_q4 = nkv * kGroup * (kHeadDim / 4);
  float4 qv[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const int i = threadIdx.x + j * NT;
    qv[j] = i < n_q4 ? q4[i] : make_float4(0.f, 0.f, 0.f, 0.f);
  }

  // Loads group fgi's next slot for ring position d -- on the position's lap-th fill
  // that is the group's slot lap * D + d -- or, once the group's slots have run out,
  // completes the position empty (slot number -1), which is the group's signal to stop.
  // Warp-collective.
  auto fill = [&](int fgi, int d) {
    const int pos = fgi * D + d;
    const uint32_t bar = bar_full + 8 * pos;
    const uint32_t sk = ring0 + fgi * group_bytes + d * slot_sz, sv = sk + v_slot_off;
    int c = 0;
    if (lane == 0) {
      const uint32_t lap = lds32(nfill0 + 4 * pos);
      c = fgi + G * ((int)lap * D + d);
      if (c >= n_slots) c = -1;
      sts32(sid0 + 4 * pos, (uint32_t)c);
      sts32(nfill0 + 4 * pos, lap + 1u);
#ifdef RD_TIMING_SWITCHES
      if (c >= 0 && (p.debug & 2)) {   // no copies: the barrier completes at once
        mbar_arrive(bar);
        c = -1;
      } else
#endif
      if (c < 0)
        mbar_arrive(bar);
      else  // a tensor-map box counts its zero-filled padding columns too
        mbar_expect_tx(bar, kSlotKeys * ((use_tk ? pitch_k : kb) + (use_tv ? pitch_v : vb)));
    }
    c = __shfl_sync(FULL, c, 0);
    if (c < 0) return;
    const int row0 = key0 + c * kSlotKeys;
    if (use_tk) {
      if (lane == 0) tma_load_2d(sk, tmk, 0, row0, bar);
    } else if (lane < kSlotKeys) {
      const int key = row0 + lane > t_last ? t_last : row0 + lane;  // tail rows repeat the last key
      bulk_g2s(sk + lane * pitch_k, kbase + (size_t)key * kb, kb, bar);
    }
    if (use_tv) {
      if (lane == 16) tma_load_2d(sv, tmv, 0, row0, bar);
    } else if (lane >= 16) {
      const int key = row0 + lane - 16 > t_last ? t_last : row0 + lane - 16;
      bulk_g2s(sv + (lane - 16) * pitch_v, vbase + (size_t)key * vb, vb, bar);
    }
  };

  __syncthreads();   // barriers, counters and the table are in place
  // every group's first slot first; the rest of the first lap follows the query build
  if (warp == 0)
    for (int fgi = 0; fgi < G; ++fgi) fill(fgi, 0);
  {
    const float qmul = p.qscale * KL::kUnscale;
    auto scatter = [&](int i, const float4 &v) {
      const int head = i >> 6, c4 = i & 63;
      const uint32_t hb = frag0 + (uint32_t)head * (4 * kFragPitch);
      const float x[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const unsigned short hbits = __half_as_ushort(__float2half_rn(x[j] * qmul));
        asm volatile("st.shared.u16 [%0], %1;" ::"r"(hb + inv[4 * c4 + j]), "h"(hbits) : "memory");
      }
    };
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int i = threadIdx.x + j * NT;
      if (i < n_q4) scatter(i, qv[j]);
    }
    for (int i = threadIdx.x + 4 * NT; i < n_q4; i += NT) scatter(i, q4[i]);   // G < 3 only
  }
  // Fused append: the newest position's K and V rows are quantized by the warps of the
  // first CTAs (one 32-value block per warp) while the first slots are in flight.
  // Nobody in this launch reads that row: the keys attended end before it, and the merge
  // that follows folds it in from the cache.
  if constexpr (!MULTI) {
    if (p.k_new != nullptr && blockIdx.y == 0) {
      const int per_tensor = nkv * (kHeadDim / 32);
      for (int b = (int)blockIdx.x * NW + warp; b < 2 * per_tensor; b += (int)gridDim.x * NW) {
        if (b < per_tensor)
          store_block<KT>(p.k_new[b * 32 + lane], const_cast<uint8_t *>(p.k) + (size_t)p.new_row * nkv * RK, b,
                          lane);
        else
          store_block<VT>(p.v_new[(b - per_tensor) * 32 + lane],
                          const_cast<uint8_t *>(p.v) + (size_t)p.new_row * nkv * RV, b - per_tensor, lane);
      }
    }
  }
  __syncthreads();
  RD_TRACE(2);
  // rest of the first lap: ring position x of a group by the group's warp x & 3
  for (int x = 1; x < D; ++x)
    if ((x & 3) == kvh) fill(gi, x);

  // ---- per-warp state ----
  float O[16][4];
  // Maxima start at a large finite negative instead of -inf: exp2(m_old - m_new) and
  // exp2(s - m) then need no special cases (an all-masked step keeps p = 0).
  constexpr float kNegBig = -1.0e30f;
  float m0 = kNegBig, m1 = kNegBig;       // softmax references of the lane's two head columns
  float run0 = kNegBig, run1 = kNegBig;   // lane-local true maxima
  float l0 = 0.f, l1 = 0.f;
#pragma unroll
  for (int i = 0; i < 16; ++i) O[i][0] = O[i][1] = O[i][2] = O[i][3] = 0.f;

  if (active) {
    // Q fragments (B operand): lane (g, tq) holds head g's 32 words; padding heads are 0.
    uint32_t qb[16][2];
    {
      const uint32_t fa =
          frag0 + (uint32_t)((kvh * kGroup + (g < kGroup ? g : 0)) * 4 + tq) * kFragPitch;
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const uint4 v = lds128(fa + 16 * i);
        qb[2 * i][0] = g < kGroup ? v.x : 0u;
        qb[2 * i][1] = g < kGroup ? v.y : 0u;
        qb[2 * i + 1][0] = g < kGroup ? v.z : 0u;
        qb[2 * i + 1][1] = g < kGroup ? v.w : 0u;
      }
    }
    const uint32_t my_ring = ring0 + gi * group_bytes;
    const uint32_t k_row_off = (uint32_t)g * pitch_k + kvh * RK;
    const uint32_t v_row_off = (uint32_t)(2 * tq) * pitch_v + kvh * RV;
    // One step consumes NS consecutive ring positions (pos[j], holding slot cs[j]). Two
    // per step give the scheduler two independent dequantize -> MMA streams per warp and
    // halve the softmax and hand-back bookkeeping.
    auto step = [&](auto nsc, const int (&pos)[2], const int (&dd)[2], const int (&cs)[2]) {
      constexpr int NS = decltype(nsc)::value;
#ifdef RD_TIMING_SWITCHES
      if (!(p.debug & 1)) {
#endif
      // ---- S = K Q^T (16 keys x 8 heads per slot), two accumulator chains each ----
      float Sv[NS][4];
#pragma unroll
      for (int j = 0; j < NS; ++j) {
        float Sc[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
        const uint32_t row_g = my_ring + dd[j] * slot_sz + k_row_off;
        const uint32_t row_h = row_g + 8 * pitch_k;
#ifdef RD_TIMING_SWITCHES
        if (!(p.debug & 4))
#endif
        KL::run(row_g, row_h, tq, [&](int n, uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3) {
          mma16816(Sc[n & 1], a0, a1, a2, a3, qb[n][0], qb[n][1]);
        });
#pragma unroll
        for (int e = 0; e < 4; ++e) Sv[j][e] = Sc[0][e] + Sc[1][e];
        const int kfirst = key0 + cs[j] * kSlotKeys;  // first key of the slot
        if (kfirst + 15 > t_last) {  // tail slot: keys beyond the last attended one
          if (kfirst + g > t_last) Sv[j][0] = Sv[j][1] = -INFINITY;
          if (kfirst + g + 8 > t_last) Sv[j][2] = Sv[j][3] = -INFINITY;
        }
        run0 = fmaxf(run0, fmaxf(Sv[j][0], Sv[j][2]));
        run1 = fmaxf(run1, fmaxf(Sv[j][1], Sv[j][3]));
      }
      // ---- online softmax (per head: columns 2t and 2t+1 of this lane) ----
      if (__any_sync(FULL, run0 > m0 + kRefSlack || run1 > m1 + kRefSlack)) {
        // move the references to the current maxima of the columns (over the 8 row lanes)
        float n0 = run0, n1 = run1;
#pragma unroll
        for (int o = 4; o < 32; o <<= 1) {
          n0 = fmaxf(n0, __shfl_xor_sync(FULL, n0, o));
          n1 = fmaxf(n1, __shfl_xor_sync(FULL, n1, o));
        }
        n0 = fmaxf(n0, m0);
        n1 = fmaxf(n1, m1);
        const float c0 = ex2(m0 - n0), c1 = ex2(m1 - n1);
        m0 = n0;
        m1 = n1;
        l0 *= c0;
        l1 *= c1;
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          O[j][0] *= c0;
          O[j][1] *= c1;
          O[j][2] *= c0;
          O[j][3] *= c1;
        }
      }
      uint32_t pb[NS][2];
#pragma unroll
      for (int j = 0; j < NS; ++j) {
        const float p0 = ex2(Sv[j][0] - m0), p1 = ex2(Sv[j][1] - m1);
        const float p2 = ex2(Sv[j][2] - m0), p3 = ex2(Sv[j][3] - m1);
        l0 += p0 + p2;
        l1 += p1 + p3;
        // P^T fragments: (keys 2t,2t+1 | head g) and (keys 2t+8,2t+9 | head g)
        pb[j][0] = movmatrix_trans(pack_h2(p0, p1));
        pb[j][1] = movmatrix_trans(pack_h2(p2, p3));
      }
      // ---- O^T += V^T P^T (256 dims x 8 heads) ----
#pragma unroll
      for (int j = 0; j < NS; ++j) {
        uint32_t rows[4];
        const uint32_t r0 = my_ring + dd[j] * slot_sz + v_slot_off + v_row_off;
        rows[0] = r0;
        rows[1] = r0 + pitch_v;
        rows[2] = r0 + 8 * pitch_v;
        rows[3] = r0 + 9 * pitch_v;
#ifdef RD_TIMING_SWITCHES
        if (!(p.debug & 8))
#endif
        VL::run(rows, g, [&](int m, uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3) {
          mma16816(O[m], a0, a1, a2, a3, pb[j][0], pb[j][1]);
        });
      }
#ifdef RD_TIMING_SWITCHES
      }
#endif
      // ---- hand the slots back; the last of the group's warps refills each ----
      __syncwarp();
      uint32_t last = 0;
      if (lane == 0) {
#pragma unroll
        for (int j = 0; j < NS; ++j)
          last |= (uint32_t)(atom_add_acq_rel_shared(cnt0 + 4 * pos[j], 1u) == (uint32_t)(nkv - 1)) << j;
      }
      last = __shfl_sync(FULL, last, 0);
#pragma unroll
      for (int j = 0; j < NS; ++j) {
        if (last & (1u << j)) {
          if (lane == 0) sts32(cnt0 + 4 * pos[j], 0u);
          fill(gi, dd[j]);
        }
      }
    };
    int d = 0;         // ring position of the next slot to consume
    uint32_t ph = 0;   // and the parity its full barrier completes with
    constexpr int kPerStep = G == 1 ? 2 : 1;   // two streams per warp where there are only four warps
    for (int i = 0;; ++i) {
      int pos[2], dd[2], cs[2];
      int got = 0;
      bool ok = true;
      const int want = (kPerStep > 1 && D >= 3) ? kPerStep : 1;   // keep one slot of a short ring in flight
      for (; got < want; ++got) {
        pos[got] = gi * D + d;
        dd[got] = d;
        if (!mbar_wait(bar_full + 8 * pos[got], ph, p.status, 2)) {
          ok = false;
          break;
        }
        cs[got] = (int)lds32(sid0 + 4 * pos[got]);
        if (cs[got] < 0) break;   // the group's slots have run out
        if (++d == D) {
          d = 0;
          ph ^= 1;
        }
      }
      if (!ok) {
        s_abort = 1;
        break;
      }
#ifdef RD_TIMING_SWITCHES
      if (i == 0) tr[3] = clock64();
#endif
      if (got == 2)
        step(std::integral_constant<int, 2>(), pos, dd, cs);
      else if (got == 1)
        step(std::integral_constant<int, 1>(), pos, dd, cs);
      if (got < want) break;
    }
    RD_TRACE(4);
    // row sums and true maxima: over the 8 key-row lanes of each head column
#pragma unroll
    for (int o = 4; o < 32; o <<= 1) {
      l0 += __shfl_xor_sync(FULL, l0, o);
      l1 += __shfl_xor_sync(FULL, l1, o);
      run0 = fmaxf(run0, __shfl_xor_sync(FULL, run0, o));
      run1 = fmaxf(run1, __shfl_xor_sync(FULL, run1, o));
    }
    if (g == 0) {
      const int c = kvh * 8 + 2 * tq;
      s_m[gi][c] = m0, s_m[gi][c + 1] = m1;
      s_t[gi][c] = run0, s_t[gi][c + 1] = run1;
      s_l[gi][c] = l0, s_l[gi][c + 1] = l1;
    }
    // Park the accumulators (still relative to this warp's references) in the group's
    // plane [head][dim], which lies over the group's own ring: the group's warps meet
    // first, so nobody still reads a slot. Dim d of a head sits at 33 * (d >> 5) +
    // (d & 31) and heads are kPlaneHead floats apart, which spreads the 8 row lanes (32
    // dims apart for the block loaders) and the quad lanes (two heads apart) over
    // different banks.
    asm volatile("bar.sync %0, %1;" ::"r"(1 + gi), "r"(nkv * 32) : "memory");
    if (!*(volatile int *)&s_abort && tq < kGroup / 2) {
      float *plane = reinterpret_cast<float *>(smem + kRingOffset + (size_t)gi * group_bytes) +
                     (kvh * kGroup + 2 * tq) * kPlaneHead;
#pragma unroll
      for (int m = 0; m < 16; ++m) {
        const int d0 = VL::dim(g, m, 0), d1 = VL::dim(g, m, 1);
        const int a0 = 33 * (d0 >> 5) + (d0 & 31), a1 = 33 * (d1 >> 5) + (d1 & 31);
        plane[a0] = O[m][0];
        plane[a0 + kPlaneHead] = O[m][1];
        plane[a1] = O[m][2];
        plane[a1 + kPlaneHead] = O[m][3];
      }
    }
  }

  // ---- combine the key groups of each kv head and write one record per head ----
  __syncthreads();  // every slot has been consumed (or the CTA is unwinding)
  RD_TRACE(5);
  const bool aborted = s_abort != 0;
  if (aborted) {
    // Unwinding after a bounded wait ran out: give copies still in flight one more
    // bounded chance to land before the CTA (and its shared memory) goes away.
    if (threadIdx.x == 0) {
      for (int i = 0; i < G * D; ++i) {
        const uint32_t nf = lds32(nfill0 + 4 * i);
        if (nf > 0) mbar_wait(bar_full + 8 * i, (nf - 1) & 1, nullptr, 0);
      }
    }
    __syncthreads();
  }
  {
    const size_t head_stride = (size_t)S * kRec;
    const bool wide = (reinterpret_cast<uintptr_t>(rec0) & 7) == 0;  // always true for the library's workspace
    const float *planes = reinterpret_cast<const float *>(smem + kRingOffset);
    const size_t plane_stride = group_bytes / sizeof(float);
    for (int idx = threadIdx.x; idx < nkv * kGroup * (kHeadDim / 2); idx += NT) {
      const int h = idx >> 7, dd = 2 * (idx & 127);
      const int c = (h / kGroup) * 8 + h % kGroup;
      float mm = kNegBig;
#pragma unroll
      for (int w = 0; w < G; ++w) mm = fmaxf(mm, s_t[w][c]);
      const bool empty = aborted || mm <= 0.5f * kNegBig;
      const int off = h * kPlaneHead + 33 * (dd >> 5) + (dd & 31);
      float a0 = 0.f, a1 = 0.f, ll = 0.f;
#pragma unroll
      for (int w = 0; w < G; ++w) {
        const float wg = ex2(s_m[w][c] - mm);   // references never exceed the true maximum
        ll += s_l[w][c] * wg;
        if (!empty) {
          a0 += planes[w * plane_stride + off] * wg;
          a1 += planes[w * plane_stride + off + 1] * wg;
        }
      }
      a0 *= VL::kUnscale;
      a1 *= VL::kUnscale;
      float *rec = rec0 + h * head_stride;
      if (dd == 0) {
        rec[0] = empty ? -INFINITY : mm * 0.6931471805599453f;  // natural log
        rec[1] = empty ? 0.f : ll;
      }
      if (wide) {
        *reinterpret_cast<float2 *>(rec + 2 + dd) = make_float2(a0, a1);
      } else {
        rec[2 + dd] = a0;
        rec[3 + dd] = a1;
      }
    }
  }
  if constexpr (!MULTI) {
    if (p.push.world > 0) {
      // Context-sharded call: the exchange of rd_shard.cu inside this launch. Every CTA
      // reports its records written; the first n_head * 4 CTAs then take one (head, dim
      // quarter) each: wait (bounded) for all CTAs, reduce the launch's records to one part,
      // store it into every rank's buffer, wait (bounded) for the other ranks' parts and
      // merge them into the output quarter.
      constexpr int NGW = NT / 16;
      float *s_pacc = reinterpret_cast<float *>(smem + kRingOffset);   // over the ring: the planes
      float *s_pl = s_pacc + NGW * kPushDims;                          // have been read by the time
      float *s_pgm = s_pl + NGW;                                       // the barrier below is passed
      int &s_go = s_abort;   // free again: the abort state was read into `aborted` above
      XHeader *me = reinterpret_cast<XHeader *>(p.push.x[p.push.rank]);
      const uint32_t epoch = *reinterpret_cast<volatile uint32_t *>(&me->epoch) + 1;
      uint32_t *arrived = &me->push_count[epoch & 1];
      __syncthreads();   // this CTA's record stores are issued
      if (threadIdx.x == 0) {
        __threadfence();
        atomicAdd(arrived, 1u);
      }
      const int n_roles = p.n_head * kQuarters;
      if ((int)blockIdx.x < n_roles) {
        if (threadIdx.x == 0) {
          int ok = 1;
          if (*reinterpret_cast<volatile uint32_t *>(arrived) < gridDim.x) {
            const unsigned long long t0 = global_ns();
            unsigned polls = 0;
            while (*reinterpret_cast<volatile uint32_t *>(arrived) < gridDim.x) {
              if ((++polls & 63u) == 0 && global_ns() - t0 > p.push.wait_ns) {
                ok = 0;
                break;
              }
            }
          }
          if (!ok && p.status != nullptr && atomicExch(&p.status->timeout_flag, 1) == 0) p.status->where = 90;
          __threadfence();
          s_go = ok;
        }
        __syncthreads();
        // Every CTA of the launch has read the epoch by now (it did before it arrived), so
        // the call can be counted: the last of the role CTAs to get here resets the counters
        // and advances the epoch. Done by a thread that takes no part in the merge below, so
        // that the round trip of its atomic is on nobody's path.
        // (the atomic is issued here and its result looked at after the exchange)
        const uint32_t cnt_mine = (uint32_t)((n_roles - 1 - (int)blockIdx.x) / (int)gridDim.x + 1);
        uint32_t cnt_prev = 0;
        if (threadIdx.x == kPushDims) cnt_prev = atomicAdd(&me->merge_count, cnt_mine);
        for (int role = blockIdx.x; role < n_roles; role += gridDim.x) {
          const int row = role / kQuarters, quarter = role % kQuarters;
          // a fused append: the new row (stored by this launch's first CTAs, not attended by
          // any of them) joins here as one more record; its score = scale * q . k: every
          // thread requests its share of the products here, the push sums them
          float x_prod = 0.f;
          const uint8_t *xv = nullptr;
          if (p.k_new != nullptr) {
            const int kvh_x = row / kGroup;
            for (int dd = threadIdx.x; dd < kHeadDim; dd += NT)
              x_prod += __ldcg(p.q + (size_t)row * kHeadDim + dd) *
                        load_cache_value(p.k + ((size_t)p.new_row * nkv + kvh_x) * RK, KT, dd);
            xv = p.v + ((size_t)p.new_row * nkv + kvh_x) * RV;
          }
          if (s_go)   // qscale = scale * log2(e): x ln 2 brings the score back to natural-log units
            shard_push_part_wide<NT>(p.partial, (int)gridDim.x, p.n_head, row, quarter, p.push, epoch, s_pacc, s_pl,
                                     s_pgm, 8, x_prod, p.qscale * 0.6931471805599453f, xv, VT);
          if (threadIdx.x < kPushDims)
            shard_merge_part(p.x_out, p.x_gate, p.n_head, row, quarter, threadIdx.x, p.push, epoch, p.status);
        }
        if (threadIdx.x == kPushDims && cnt_prev + cnt_mine == (uint32_t)n_roles) {
          me->merge_count = 0;
          me->push_count[epoch & 1] = 0;
          __threadfence();
          me->epoch = epoch;
        }
      }
    }
  }
#ifdef RD_TIMING_SWITCHES
  if (p.debug & 32) {
    __syncthreads();
    if (threadIdx.x == 0) {
      RD_TRACE(6);
      unsigned *o = reinterpret_cast<unsigned *>(rec0 + 2);
      o[0] = (unsigned)gt0;
      for (int i = 1; i < 7; ++i) o[i] = (unsigned)(tr[i] - tr[0]);
      o[7] = (unsigned)n_slots;
    }
  }
#endif
}
#undef RD_TRACE

#ifdef RD_TIMING_SWITCHES
}  // namespace rd
// Experimental tensor-memory flavour of the kernel (tcgen05.mma with the dequantized
// fragments in TMEM): correct, slower than this kernel so far, built only into
// timing-switch builds and taken there with RD_TC_DECODE=1.
#include "rd_decode_tc.cuh"
namespace rd {
inline bool tc_decode_enabled() {
  const char *e = getenv("RD_TC_DECODE");
  return e != nullptr && atoi(e) != 0;
}
#endif

// Shared-memory plan of one (KT, VT) instantiation and the opt-in for it.
template <int KT, int VT, bool MULTI>
int prepare_decode(int n_head_kv, int *depth_out, int *group_bytes_out, size_t *smem_out) {
  constexpr int G = key_groups(KT, VT);
  const int depth = ring_depth(KT, VT, n_head_kv);
  if (depth < 1) return RD_ERR_UNSUPPORTED;
  // a group's ring doubles as its epilogue plane [head][kPlaneHead] of f32
  size_t group_bytes = (size_t)depth * slot_bytes(KT, VT, n_head_kv);
  const size_t plane_bytes = (size_t)n_head_kv * kGroup * kPlaneHead * sizeof(float);
  if (group_bytes < plane_bytes) group_bytes = (plane_bytes + 127) & ~(size_t)127;
  const size_t smem = kRingOffset + (size_t)G * group_bytes;
  if (smem > (size_t)kSmemBudget) return RD_ERR_UNSUPPORTED;
  static bool attr_set[8] = {false, false, false, false, false, false, false, false};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return RD_ERR_CUDA;
  if (dev < 0 || dev >= 8 || !attr_set[dev]) {
    if (cudaFuncSetAttribute(decode_kernel<KT, VT, MULTI>,
                             cudaFuncAttributeMaxDynamicSharedMemorySize,
                             kSmemBudget) != cudaSuccess)
      return RD_ERR_CUDA;
    if (dev >= 0 && dev < 8) attr_set[dev] = true;
  }
  *depth_out = depth;
  *group_bytes_out = (int)group_bytes;
  *smem_out = smem;
  return RD_OK;
}

#ifdef RD_TIMING_SWITCHES
inline int decode_debug_mask() {
  const char *e = getenv("RD_DECODE_DEBUG");
  return e ? atoi(e) : 0;
}
#endif

// Host side of one (KT, VT) instantiation.
template <int KT, int VT>
int launch_decode_typed(const DecodeArgs &a, cudaStream_t st) {
  constexpr int G = key_groups(KT, VT);
  int depth = 0, group_bytes = 0;
  size_t smem = 0;
  const int rc = prepare_decode<KT, VT, false>(a.n_head_kv, &depth, &group_bytes, &smem);
  if (rc != RD_OK) return rc;
  DecodeKernelArgs k;
  memset(&k, 0, sizeof(k));
  // Quantized keys are small (576 / 1088 bytes for 4 kv heads), so a whole slot comes in
  // as one tensor-map copy; f16 / f32 keys are too wide for one box and large enough for
  // one plain bulk copy per key. Tensor maps need the key count on the host, so
  // launches that take it from a device array use bulk copies as well.
  const bool host_keys = a.pos == nullptr;
  const int64_t n_rows = (int64_t)a.t + 1;
  k.k_tmap = host_keys && n_rows > 0 && KT >= RD_KV_Q8_0 &&
             encode_kv_tmap(&k.tm_k, a.k, KT, a.n_head_kv, n_rows, kSlotKeys) == RD_OK;
  k.v_tmap = host_keys && n_rows > 0 && VT >= RD_KV_Q8_0 &&
             encode_kv_tmap(&k.tm_v, a.v, VT, a.n_head_kv, n_rows, kSlotKeys) == RD_OK;
  k.q = a.q;
  k.k = (const uint8_t *)a.k;
  k.v = (const uint8_t *)a.v;
  k.partial = a.partial;
  k.pos = a.pos;
  k.t = a.t;
  k.key_begin = a.key_begin;
  k.n_head = a.n_head;
  k.nkv = a.n_head_kv;
  k.qscale = a.scale * 1.4426950408889634f;
  k.depth = depth;
  k.group_bytes = group_bytes;
#ifdef RD_TIMING_SWITCHES
  k.debug = decode_debug_mask();
#endif
  k.status = a.status;
  k.k_new = a.k_new;
  k.v_new = a.v_new;
  k.new_row = a.new_row;
  if (a.push != nullptr && a.n_tok == 1) {   // memset above: world 0 = no exchange
    k.push = *a.push;
    k.x_out = a.push_out;
    k.x_gate = a.push_gate;
  }
#ifdef RD_TIMING_SWITCHES
  if constexpr (tc_decode_usable(KT, VT)) {
    if (tc_decode_enabled() && a.n_head_kv == 4 && a.n_tok == 1 && k.k_tmap && k.v_tmap && a.push == nullptr &&
        a.k_new == nullptr)
      return launch_decode_tc<KT, VT>(k, a.n_splits, st);
  }
#endif
  const dim3 grid((unsigned)a.n_splits, (unsigned)a.n_tok);
  return launch_pdl(2, decode_kernel<KT, VT, false>, grid, dim3(4 * G * 32), smem, st, k) == cudaSuccess
             ? RD_OK
             : RD_ERR_CUDA;
}

// Multi-sequence flavour: fills the tensor maps of the host-side descriptors (prepare)
// and launches one CTA per work item (launch).
template <int KT, int VT>
int multi_decode_typed(const MultiDecodeArgs &a, cudaStream_t st) {
  constexpr int G = key_groups(KT, VT);
  if (a.host_seqs != nullptr) {
    for (int i = 0; i < a.n_seq; ++i) {
      DecodeSeq &d = a.host_seqs[i];
      const int64_t n_rows = (int64_t)d.t + 1;
      d.k_tmap = n_rows > 0 && KT >= RD_KV_Q8_0 &&
                 encode_kv_tmap(d.tm_k, d.k, KT, a.n_head_kv, n_rows, kSlotKeys) == RD_OK;
      d.v_tmap = n_rows > 0 && VT >= RD_KV_Q8_0 &&
                 encode_kv_tmap(d.tm_v, d.v, VT, a.n_head_kv, n_rows, kSlotKeys) == RD_OK;
    }
    return RD_OK;
  }
  int depth = 0, group_bytes = 0;
  size_t smem = 0;
  const int rc = prepare_decode<KT, VT, true>(a.n_head_kv, &depth, &group_bytes, &smem);
  if (rc != RD_OK) return rc;
  DecodeKernelArgs k;
  memset(&k, 0, sizeof(k));
  k.partial = a.records;
  k.n_head = a.n_head;
  k.nkv = a.n_head_kv;
  k.qscale = a.scale * 1.4426950408889634f;
  k.depth = depth;
  k.group_bytes = group_bytes;
#ifdef RD_TIMING_SWITCHES
  k.debug = decode_debug_mask();
#endif
  k.status = a.status;
  k.seqs = a.dev_seqs;
  k.items = a.dev_items;
  k.q_len = a.q_len;
  return launch_pdl(2, decode_kernel<KT, VT, true>, dim3((unsigned)a.n_items), dim3(4 * G * 32), smem, st,
                    k) == cudaSuccess
             ? RD_OK
             : RD_ERR_CUDA;
}

}  // namespace rd
