// Causal prefill attention on the 5th-generation tensor cores (tcgen05 + TMEM + TMA).
//
// Replaces attn_fa2_prefill_kernel (include/rdna4/attn_fa2.cuh:30-169 of the reference)
// for f16 K/V caches. One CTA owns a tile of 128 query tokens of ONE query head and walks
// the keys in tiles of 128. Tensor memory (512 columns x 128 lanes, lane = query row):
//   columns   0..255  O, the f32 output accumulator
//   columns 256..511  two score buffers of 128 f32 columns; the f16 P of a tile is written
//                     over the first 64 columns of its buffer (the A operand of O += P V,
//                     read from TMEM)
// Shared memory (224 KB): Q as f16 in the K-major 128-byte-swizzled layout (64 KB), a ring
// of three K units of [128 keys][128 dims] (96 KB) and a ring of two V units of 64 keys
// (64 KB), all filled by TMA with the hardware 128B swizzle.
//
//   prologue   the 128 x 256 f32 query rows -> optional partial RoPE, scale*log2(e), f16,
//              swizzled into shared memory (8 warps, 16 rows each);
//   per 128-key tile j:
//     warp 9     S = Q K_j^T        16 x tcgen05.mma M128 N128 K16, four per K chunk, each
//                                   chunk handed back to the TMA producer as soon as its
//                                   four MMAs are done (N = 128 keeps the tensor core busy
//                                   for as long as the 128 x 16 A slice takes to fetch)
//     warps 0-7  two threads per query row, 64 score columns each (row max exchanged
//                through shared memory): tcgen05.ld the scores, causal mask
//                (key <= pos[r]), running max with LAZY rescale (the reference point only
//                moves when a row's max grows by more than 2^8, so P stays below 256 in
//                f16 and O in TMEM is rarely touched), P -> f16 pairs, tcgen05.st
//     warp 11    O += P V_j          8 x tcgen05.mma M128 N256 K16 (A = P from TMEM, B = V
//                                   MN-major), four per V unit
//   epilogue   O / l (times sigmoid(gate) if asked) through a swizzled staging tile to
//              coalesced f32 stores.
// Warps 8 and 10 are the K and V TMA producers (separate warps: a lane parked in
// mbarrier.try_wait parks its whole warp). The two contractions have their own issuing
// threads because issuing a tcgen05.mma costs the issuing thread tens of cycles.
//
// Scores are double-buffered: the tensor core computes S of tile j+1 while the softmax
// warps work on tile j. S of tile j+2 waits for P V of tile j, which reads the P that
// lives in its buffer.
//
// Synchronisation is mbarriers only (TMA transaction counts, tcgen05.commit); every wait
// is bounded and a timeout unwinds the CTA (TMEM is always freed). No cluster launch, no
// multicast.
#include <stdlib.h>
#include <string.h>

#include "rd_common.cuh"
#include "rd_internal.h"
#include "rd_tc.cuh"

// Timing experiments (skip one pipeline stage, bit mask in PrefillArgs::debug) exist only
// in builds with -DRD_TIMING_SWITCHES; a default build compiles them out.
#ifdef RD_TIMING_SWITCHES
#define RD_PF_DEBUG(p) ((p).debug)
#else
#define RD_PF_DEBUG(p) 0
#endif
// -DRD_PF_TRACING (timing builds only): phase trace of CTA (0, 0, 0),
// [role 0..3][tile 0..47][point 0..7] clock64 values, read back with rd_debug_pf_trace
#ifdef RD_PF_TRACING
__device__ unsigned long long g_pf_trace[4][48][8];
#define RD_PF_TRACE(role, j, pt)                                                  \
  do {                                                                            \
    if (blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0 && (j) < 48)        \
      g_pf_trace[role][j][pt] = clock64();                                        \
  } while (0)
#else
#define RD_PF_TRACE(role, j, pt) do { } while (0)
#endif

namespace rd {

constexpr int kPfM = 128;                 // query rows per CTA
constexpr int kPfN = 128;                 // keys per tile
constexpr int kPfQBytes = kPfM * kHeadDim * 2;             // 65536 (also the epilogue staging)
constexpr int kPfKChunkBytes = kPfN * 128;                 // [128 keys][64 dims] f16: 16384
constexpr int kPfKUnitBytes = 2 * kPfKChunkBytes;          // K unit: [128 keys][128 dims], two chunks
constexpr int kPfKSlots = 3;                               // 1.5 tiles of K in flight
constexpr int kPfVUnitKeys = 64;
constexpr int kPfVUnitBytes = kPfVUnitKeys * kHeadDim * 2; // 32768
constexpr int kPfVSlots = 2;
// 224 KB of dynamic shared memory + < 3 KB static = the 227 KB an sm_100 CTA may use
constexpr int kPfSmemBytes = kPfQBytes + kPfKSlots * kPfKUnitBytes + kPfVSlots * kPfVUnitBytes;
constexpr int kPfThreads = 384;           // 8 softmax warps, K TMA, S MMA, V TMA, PV MMA warps
constexpr uint32_t kTmemCols = 512;
constexpr uint32_t kTmemO = 0;            // columns [0, 256): output accumulator
constexpr uint32_t kTmemS = 256;          // columns [256, 512): two score buffers of 128; the
                                          // f16 P of a tile overwrites its first 64 columns
constexpr float kLazyThreshold = 8.0f;    // log2 units
constexpr int kPfMaxSplits = 8;           // key splits per (token tile, head) at most

struct PrefillArgs {
  alignas(64) CUtensorMap tm_k;
  alignas(64) CUtensorMap tm_v;
  const float *q;
  float *out;
  const float *gate;     // optional [n_q][n_head][256]
  const int32_t *pos;    // device, one per query token
  int n_q;
  int n_head;
  int nkv;
  float qscale;          // scale * log2(e)
  alignas(64) CUtensorMap tm_q;  // q16 != 0: the rotated, scaled f16 queries q_prep_kernel wrote
  int q16;               // 1: Q tile by TMA from tm_q; 0: converted from `q` (f32, no rotation) here
  int kv_wait;           // 1: that pre-pass also stored cache rows: the K / V loads wait for it too
  int debug;             // timing experiments only (bit mask), 0 in production
  DeviceStatus *status;
  // Split over the keys (gridDim.z > 1): CTA (tile, head, z) walks only its share of the
  // key tiles and writes an un-normalised record (m, l, acc) per row instead of the
  // output; prefill_merge_kernel combines the records. Fills the SMs when n_q * n_head /
  // 128 CTAs would leave many idle.
  float *records;        // [n_q * n_head][gridDim.z][2 + 256]
};

// Barrier slots (8 bytes each).
enum { kBarKFull = 0, kBarKFree = 6, kBarVFull = 12, kBarVFree = 14, kBarS = 16, kBarP = 18, kBarO = 22,
       kBarQ = 24, kBarR = 25, kBarCount = 33 };   // kBarP: [score buffer][64-key half of P];
                                                   // kBarR: [warp pair 0..3][tile parity]

__global__ void __launch_bounds__(kPfThreads, 1) prefill_kernel(const __grid_constant__ PrefillArgs p) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  __shared__ __align__(8) unsigned long long s_bars[kBarCount];
  __shared__ uint32_t s_tmem_base;
  __shared__ int s_maxpos;
  __shared__ int s_abort;
  __shared__ float s_ref[2][kPfM];     // [tile parity][row]: the reference maximum that tile left

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  pdl_launch_dependents();   // the merge pass of a key split may be scheduled under this kernel
  if (threadIdx.x == 0) RD_PF_TRACE(0, 47, 0);   // kernel entry
  const int tile = (int)gridDim.x - 1 - (int)blockIdx.x;  // heaviest (latest) tiles first
  const int head = blockIdx.y;
  const int kvh = head / kGroup;
  const int row0 = tile * kPfM;

  // carve-up of dynamic shared memory; 128B-swizzle atoms need the base 1 KB aligned
  const uint32_t base = smem_u32(smem_raw);
  if ((base & 1023u) != 0) {  // cannot happen with the declared alignment; refuse, do not corrupt
    if (threadIdx.x == 0 && p.status != nullptr && atomicExch(&p.status->timeout_flag, 1) == 0)
      p.status->where = 99;
    return;
  }
  const uint32_t sQ = base;
  const uint32_t sK = sQ + kPfQBytes;                       // slot s at + s * 32 KB
  const uint32_t sV = sK + kPfKSlots * kPfKUnitBytes;       // slot s at + s * 32 KB
  uint8_t *gQ = smem_raw;                                   // generic pointer to sQ
  const uint32_t bars = smem_u32(s_bars);

  // Requested first, so that their latency runs under the set-up below: the positions of
  // this tile's rows and -- where the tile is converted here -- all 16 query rows of the
  // warp (32 float4 per lane; the conversion is bound by the latency of these loads).
  int my_pos = -1;
  if (threadIdx.x < 2 * kPfM) {
    const int r = row0 + (threadIdx.x & (kPfM - 1));
    if (r < p.n_q) my_pos = p.pos[r];
  }
  float4 qa[16], qb[16];
  if (!p.q16 && warp < 8) {
#pragma unroll
    for (int rr = 0; rr < 16; ++rr) {
      const int gr = row0 + warp * 16 + rr;
      qa[rr] = qb[rr] = make_float4(0.f, 0.f, 0.f, 0.f);
      if (gr < p.n_q) {
        const float4 *src = reinterpret_cast<const float4 *>(p.q + ((size_t)gr * p.n_head + head) * kHeadDim);
        qa[rr] = src[2 * lane];
        qb[rr] = src[2 * lane + 1];
      }
    }
  }

  if (threadIdx.x == 0) {
    s_maxpos = -1;
    s_abort = 0;
    for (int i = 0; i < kPfKSlots; ++i) {
      mbar_init(bars + 8 * (kBarKFull + i), 1);
      mbar_init(bars + 8 * (kBarKFree + i), 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(bars + 8 * (kBarVFull + i), 1);
      mbar_init(bars + 8 * (kBarVFree + i), 1);
      mbar_init(bars + 8 * (kBarS + i), 1);
      mbar_init(bars + 8 * (kBarP + 2 * i), 4);       // one elected lane per softmax warp of the
      mbar_init(bars + 8 * (kBarP + 2 * i + 1), 4);   // tile's set, per 64-key half of P
      mbar_init(bars + 8 * (kBarO + i), 1);
    }
    for (int i = 0; i < 8; ++i) mbar_init(bars + 8 * (kBarR + i), 1);
    mbar_init(bars + 8 * kBarQ, p.q16 ? 1 : 8);   // the TMA issuer, or one per converting warp
    fence_barrier_init();
  }
  if (warp == 9) {  // TMEM: 512 columns for this CTA (one CTA per SM: no contention)
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                     smem_u32(&s_tmem_base)),
                 "r"(kTmemCols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  __syncthreads();
  if (threadIdx.x == 0) RD_PF_TRACE(0, 47, 1);   // barriers + TMEM allocated

  // ---- the last key any row of this tile attends ----
  if (threadIdx.x < kPfM) {
    int mx = my_pos;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mx = max(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    if (lane == 0) atomicMax(&s_maxpos, mx);
  }
  tc_fence_before();
  __syncthreads();
  if (threadIdx.x == 0) RD_PF_TRACE(0, 47, 2);   // positions known
  tc_fence_after();
  const uint32_t tmem = s_tmem_base;
  const int maxpos = s_maxpos;
  const int nt_all = maxpos >= 0 ? maxpos / kPfN + 1 : 0;  // key tiles the rows of this tile attend
  const int jt0 = (int)(((int64_t)nt_all * blockIdx.z) / gridDim.z);        // this CTA's share of them
  const int nt = (int)(((int64_t)nt_all * (blockIdx.z + 1)) / gridDim.z) - jt0;

  // ---- prologue: the Q tile as f16 in the swizzled K-major layout ----
  if (p.q16) {
    // rotated, scaled and rounded by q_prep_kernel: four TMA boxes of [128 rows][64 dims]
    // (rows past n_q are filled with zeros). Only this thread waits for that pass: the K
    // and V producers are already loading.
    if (threadIdx.x == 0) {
      pdl_wait();   // that pass has completed (this launch may have started under it)
      const uint32_t full = bars + 8 * kBarQ;
      mbar_expect_tx(full, kPfQBytes);
#pragma unroll
      for (int c = 0; c < 4; ++c)
        tma_load_2d(sQ + c * (kPfM * 128), &p.tm_q, head * kHeadDim + 64 * c, row0, full);
    }
  } else if (warp < 8) {
    // f32 rows -> x scale * log2(e) -> f16, warps 0-7, 16 rows each
#pragma unroll
    for (int rr = 0; rr < 16; ++rr) {
      const int r = warp * 16 + rr;      // row inside the tile
      const uint32_t w0 = pack_h2(qa[rr].x * p.qscale, qa[rr].y * p.qscale);
      const uint32_t w1 = pack_h2(qa[rr].z * p.qscale, qa[rr].w * p.qscale);
      const uint32_t w2 = pack_h2(qb[rr].x * p.qscale, qb[rr].y * p.qscale);
      const uint32_t w3 = pack_h2(qb[rr].z * p.qscale, qb[rr].w * p.qscale);
      // lane = 16-byte chunk of the row: sub-tile lane/8, chunk lane%8, swizzled by the row
      const uint32_t dst = sQ + (lane >> 3) * (kPfM * 128) + r * 128 + (((lane & 7) ^ (r & 7)) << 4);
      sts128(dst, w0, w1, w2, w3);
    }
    fence_proxy_async();  // generic-proxy writes -> visible to the tensor core's async proxy
    __syncwarp();
    if (lane == 0) mbar_arrive(bars + 8 * kBarQ);  // the S MMAs wait for all 8 warps
    if (threadIdx.x == 0) RD_PF_TRACE(0, 47, 3);   // this warp's Q rows converted
  }

  float l_run = 0.f;                 // softmax threads: row sum
  float m_ref = -1.0e30f;            //                  reference maximum (log2 units)

  if (warp >= 8) {
  if (warp == 8) {
    // =============================== K producer ====================================
    // unit g = 2 j + u: keys of tile j, dims [128 u, 128 u + 128) as two 64-dim chunks, into
    // slot g % 3 -- one barrier per unit: the issuing thread pays for every wait and commit
    if (lane == 0) {
      if (p.kv_wait) pdl_wait();   // the pre-pass of this call appended rows to the caches
      int slot = 0, use = 0;
      for (int g = 0; g < 2 * nt; ++g) {
        if (use > 0 && !mbar_wait(bars + 8 * (kBarKFree + slot), (use - 1) & 1, p.status, 11)) {
          s_abort = 1;
          break;
        }
        if (*(volatile int *)&s_abort) break;
        const uint32_t full = bars + 8 * (kBarKFull + slot);
        if (RD_PF_DEBUG(p) & 32) {
          mbar_arrive(full);
        } else {
          mbar_expect_tx(full, kPfKUnitBytes);
#pragma unroll
          for (int h = 0; h < 2; ++h)
            tma_load_2d(sK + slot * kPfKUnitBytes + h * kPfKChunkBytes, &p.tm_k,
                        kvh * kHeadDim + 128 * (g & 1) + 64 * h, (jt0 + (g >> 1)) * kPfN, full);
        }
        if (++slot == kPfKSlots) {
          slot = 0;
          ++use;
        }
      }
    }
  } else if (warp == 10) {
    // =============================== V producer ====================================
    // unit g = 2 j + u: keys [128 j + 64 u, + 64) of all 256 dims, into slot g % 2
    if (lane == 0) {
      bool ok = true;
      if (p.kv_wait) pdl_wait();
      for (int g = 0; g < 2 * nt && ok; ++g) {
        const int slot = g & 1;
        if (g >= 2 && !mbar_wait(bars + 8 * (kBarVFree + slot), ((g >> 1) - 1) & 1, p.status, 22)) {
          ok = false;
          break;
        }
        if (*(volatile int *)&s_abort) break;
        const uint32_t full = bars + 8 * (kBarVFull + slot);
        if (RD_PF_DEBUG(p) & 32) {
          mbar_arrive(full);
          continue;
        }
        mbar_expect_tx(full, kPfVUnitBytes);
#pragma unroll
        for (int c = 0; c < 4; ++c)  // four [64 keys][64 dims] sub-tiles
          tma_load_2d(sV + slot * kPfVUnitBytes + c * (kPfVUnitKeys * 128), &p.tm_v, kvh * kHeadDim + 64 * c,
                      (2 * jt0 + g) * kPfVUnitKeys, full);
      }
      if (!ok) s_abort = 1;
    }
  } else if (warp == 9) {
    // ============================ MMA issuer: S = Q K^T =============================
    if (lane == 0) {
      constexpr uint32_t idesc_s = idesc_f16(kPfM, kPfN, false);
      // Descriptors differ only in the 16-byte-granular start address (low 14 bits, and
      // every address here is below 256 KB), so each one is a base plus a constant.
      const uint64_t dq = smem_desc(sQ, 16, 1024);
      const uint64_t dk = smem_desc(sK, 16, 1024);
      bool ok = mbar_wait(bars + 8 * kBarQ, 0, p.status, 18);  // Q tile written by warps 0-3
      tc_fence_after();
      int slot = 0, use = 0;
      for (int j = 0; j < nt && ok; ++j) {
        const int st = j & 1;
        RD_PF_TRACE(2, j, 0);
        // score buffer st still holds P(j-2) until P V of tile j-2 has read it
        if (j >= 2 && !mbar_wait(bars + 8 * (kBarO + st), ((j - 2) >> 1) & 1, p.status, 15)) {
          ok = false;
          break;
        }
        const uint32_t d_s = tmem + kTmemS + 128 * st;
        RD_PF_TRACE(2, j, 1);
        for (int u = 0; u < 2 && ok; ++u) {
          if (!mbar_wait(bars + 8 * (kBarKFull + slot), use & 1, p.status, 12)) {
            ok = false;
            break;
          }
          tc_fence_after();
          if (u == 0) RD_PF_TRACE(2, j, 3);
          // per 64-dim chunk c = 2 u + h: A = Q sub-tile c ([128 rows][64 dims]), B = K chunk
          // ([128 keys][64 dims]), both K-major with 8-row groups 1 KB apart; four steps of
          // 16 dims = 32 bytes each
          if (!(RD_PF_DEBUG(p) & 8)) {
#pragma unroll
            for (int h = 0; h < 2; ++h) {
              const uint64_t a0 = dq + (uint64_t)(((2 * u + h) * (kPfM * 128)) >> 4);
              const uint64_t b0 = dk + (uint64_t)((slot * kPfKUnitBytes + h * kPfKChunkBytes) >> 4);
#pragma unroll
              for (int kk = 0; kk < 4; ++kk)
                tc_mma_f16(d_s, a0 + (uint64_t)(2 * kk), b0 + (uint64_t)(2 * kk), idesc_s,
                           (u > 0 || h > 0 || kk > 0) ? 1u : 0u);
            }
          }
          if (u == 0) RD_PF_TRACE(2, j, 4);
          tc_commit(bars + 8 * (kBarKFree + slot));  // the unit can be refilled
          if (u == 0) RD_PF_TRACE(2, j, 5);
          if (++slot == kPfKSlots) {
            slot = 0;
            ++use;
          }
        }
        tc_commit(bars + 8 * (kBarS + st));
        RD_PF_TRACE(2, j, 2);
      }
      if (!ok) s_abort = 1;
    }
  } else if (warp == 11) {
    // ============================ MMA issuer: O += P V ==============================
    if (lane == 0) {
      constexpr uint32_t idesc_o = idesc_f16(kPfM, kHeadDim, true);
      const uint64_t dv = smem_desc(sV, kPfVUnitKeys * 128, 1024);
      bool ok = true;
      for (int j = 0; j < nt && ok; ++j) {
        const int st = j & 1;
        RD_PF_TRACE(3, j, 0);
        for (int u = 0; u < 2 && ok; ++u) {
          // P arrives in two halves of 64 keys: P V of the first runs while the softmax
          // threads are still on the second
          if (!mbar_wait(bars + 8 * (kBarP + 2 * st + u), (j >> 1) & 1, p.status, 13)) {
            ok = false;
            break;
          }
          if (u == 0) RD_PF_TRACE(3, j, 1);
          const int g = 2 * j + u, slot = g & 1;
          if (!mbar_wait(bars + 8 * (kBarVFull + slot), (g >> 1) & 1, p.status, 19)) {
            ok = false;
            break;
          }
          tc_fence_after();
          // A = P(j) from TMEM (16 keys = 8 columns per step), B = V unit MN-major: 64-dim
          // groups 8 KB apart (LBO), 8-key groups 1 KB apart (SBO); 4 steps of 16 keys
          const uint64_t dvs = dv + (uint64_t)((slot * kPfVUnitBytes) >> 4);
          const uint32_t a_p = tmem + kTmemS + 128 * st + 32 * u;
          if (!(RD_PF_DEBUG(p) & 4)) {
#pragma unroll
            for (int kk = 0; kk < 4; ++kk)
              tc_mma_f16_ts(tmem + kTmemO, a_p + 8 * kk, dvs + (uint64_t)((kk * 2048) >> 4), idesc_o,
                            (j > 0 || u > 0 || kk > 0) ? 1u : 0u);
          }
          tc_commit(bars + 8 * (kBarVFree + slot));  // the V unit can be refilled
        }
        tc_commit(bars + 8 * (kBarO + st));  // score buffer reusable, O settled
        RD_PF_TRACE(3, j, 2);
      }
      if (!ok) s_abort = 1;
    }
  }
  } else {
    // ========= softmax: thread = (row r, tile parity): warps 0-3 take the even key =========
    // tiles of this CTA, warps 4-7 the odd ones, a whole 128-key row of scores per thread.
    // The two sets run one tile apart, so the tensor-memory loads, the maxima and the waits
    // of tile j + 1 overlap the exponentials of tile j. What the tiles of a row share is the
    // reference maximum of the one accumulator: it is handed from tile to tile through
    // s_ref and one mbarrier per (warp pair, parity) -- after a tile's maxima are known,
    // before its exponentials.
    const int r = threadIdx.x & (kPfM - 1), set = threadIdx.x >> 7;
    const uint32_t lane_addr = tmem + ((uint32_t)((warp & 3) * 32) << 16);
    const uint32_t bar_ref = bars + 8 * (kBarR + 2 * (warp & 3));
    bool ok = true;
    for (int j = set; j < nt && ok; j += 2) {
      const int st = set;   // tile j's score buffer: j & 1
      if ((threadIdx.x & 127) == 0) RD_PF_TRACE(set, j, 0);
      // the reference tile j - 1 left: its set published it right after its own maxima,
      // long before this tile's scores are ready -- fetched first, off the critical path
      float m_prev = -1.0e30f;
      if (j > 0) {
        if (!mbar_wait(bar_ref + 8 * ((j - 1) & 1), ((j - 1) >> 1) & 1, p.status, 20)) { ok = false; break; }
        m_prev = s_ref[(j - 1) & 1][r];
      }
      if (!mbar_wait(bars + 8 * (kBarS + st), (j >> 1) & 1, p.status, 14)) { ok = false; break; }
      tc_fence_after();
      if ((threadIdx.x & 127) == 0) RD_PF_TRACE(set, j, 1);
      uint32_t sc[4][32];
      const uint32_t scol = lane_addr + kTmemS + 128 * st;
#pragma unroll
      for (int c = 0; c < 4; ++c) tmem_ld32(scol + 32 * c, sc[c]);
      tmem_wait_ld();
      if ((threadIdx.x & 127) == 0) RD_PF_TRACE(set, j, 2);
      const int key0 = (jt0 + j) * kPfN;
      // only tiles that reach past some row's last key need the causal mask
      if (__any_sync(0xffffffffu, key0 + kPfN - 1 > my_pos)) {
#pragma unroll
        for (int c = 0; c < 4; ++c)
#pragma unroll
          for (int i = 0; i < 32; ++i)
            if (key0 + 32 * c + i > my_pos) sc[c][i] = 0xff800000u;  // -inf
      }
      // eight independent chains of three-input maxima
      float mx[8];
#pragma unroll
      for (int k = 0; k < 8; ++k) mx[k] = -INFINITY;
#pragma unroll
      for (int c = 0; c < 4; ++c)
#pragma unroll
        for (int i = 0; i < 32; i += 2)
          mx[(i >> 1) & 7] = max3(mx[(i >> 1) & 7], __uint_as_float(sc[c][i]), __uint_as_float(sc[c][i + 1]));
      const float mt = fmaxf(max3(mx[0], mx[1], mx[2]), fmaxf(max3(mx[3], mx[4], mx[5]), fmaxf(mx[6], mx[7])));
      const bool grow = __any_sync(0xffffffffu, mt > m_prev + kLazyThreshold);
      const float m_new = grow ? fmaxf(m_prev, mt) : m_prev;
      s_ref[j & 1][r] = m_new;
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_ref + 8 * (j & 1));
      if ((threadIdx.x & 127) == 0) RD_PF_TRACE(set, j, 3);
      l_run *= ex2(m_ref - m_new);   // this set's sum moves to the new reference (m_ref: its last one)
      m_ref = m_new;
      if (grow && j > 0) {
        // O is rescaled in tensor memory: P V of tile j - 1 must be done, and no later one
        // can start before this tile's P arrives
        const float f = ex2(m_prev - m_new);   // 1 for rows that keep their reference
        if (!mbar_wait(bars + 8 * (kBarO + ((j - 1) & 1)), ((j - 1) >> 1) & 1, p.status, 17)) {
          ok = false;
          break;
        }
        tc_fence_after();
#pragma unroll 1
        for (int c = 0; c < kHeadDim / 32; ++c) {
          uint32_t o[32];
          tmem_ld32(lane_addr + kTmemO + 32 * c, o);
          tmem_wait_ld();
#pragma unroll
          for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * f);
          tmem_st32(lane_addr + kTmemO + 32 * c, o);
        }
        tmem_wait_st();
      }
      // P = 2^(s - m_ref) as f16 pairs, written over the score buffer: key k of row r
      // becomes half k & 1 of column k / 2 (the A operand of P V, read from TMEM); the
      // columns a chunk overwrites hold scores that are already in registers
      // (s - m) and the row sum go through the packed f32x2 adds, two scores per
      // instruction: measured alone, one warp then needs ~1200 cycles per 128-score row
      // (the 128 exponentials alone are 1024 on the special-function unit) against ~1600
      // with scalar adds
      unsigned long long neg_m = f2_pack(-m_new, -m_new);
      unsigned long long ls2[4] = {0ull, 0ull, 0ull, 0ull};
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        uint32_t pw[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          float x0, x1;
          f2_unpack(f2_add(f2_pack(__uint_as_float(sc[c][2 * i]), __uint_as_float(sc[c][2 * i + 1])), neg_m), x0, x1);
          if (!(RD_PF_DEBUG(p) & 1)) {
            x0 = ex2(x0);
            x1 = ex2(x1);
          }
          ls2[i & 3] = f2_add(ls2[i & 3], f2_pack(x0, x1));
          pw[i] = (RD_PF_DEBUG(p) & 2) ? __float_as_uint(x0) : pack_h2(x0, x1);
        }
        if (!(RD_PF_DEBUG(p) & 16)) tmem_st16(scol + 16 * c, pw);
        else if (pw[0] == 0x12345678u && pw[7] == 0x9abcdefu) l_run += 1.f;   // keeps the values live
        if (c == 1) {   // the first 64 keys of P are complete: hand them to the P V issuer
          tmem_wait_st();
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(bars + 8 * (kBarP + 2 * st));
          // keeps the second half's arithmetic behind the hand-over (the compiler would
          // otherwise hoist all 128 exponentials above the first store)
          asm volatile("mov.b64 %0, %0;" : "+l"(neg_m)::"memory");
        }
      }
      {
        float a0, a1, a2, a3;
        f2_unpack(f2_add(ls2[0], ls2[1]), a0, a1);
        f2_unpack(f2_add(ls2[2], ls2[3]), a2, a3);
        l_run += (a0 + a1) + (a2 + a3);
      }
      if ((threadIdx.x & 127) == 0) RD_PF_TRACE(set, j, 4);
      tmem_wait_st();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bars + 8 * (kBarP + 2 * st + 1));
      if ((threadIdx.x & 127) == 0) RD_PF_TRACE(set, j, 5);
    }
    if (ok && nt > 0 && !mbar_wait(bars + 8 * (kBarO + ((nt - 1) & 1)), ((nt - 1) >> 1) & 1, p.status, 16))
      ok = false;
    if (!ok) s_abort = 1;
    tc_fence_after();
  }

  // With the queries coming from the pre-pass, nothing may be stored before that pass has
  // completed: o may alias q, which it is still reading. A CTA with key tiles knows this from
  // its Q tile; one without (no row attends a key) waits for the tile here -- its TMA load was
  // issued behind the dependency wait all the same.
  if (p.q16 && nt == 0 && threadIdx.x == 0 && !mbar_wait(bars + 8 * kBarQ, 0, p.status, 23)) s_abort = 1;
  __syncthreads();
  const bool aborted = s_abort != 0;
  // the two sets' row sums, each with the reference it is expressed in: [set][sum,
  // reference][row], over the K ring (every load into it has been consumed by now)
  float (*s_fin)[2][kPfM] = reinterpret_cast<float (*)[2][kPfM]>(smem_raw + kPfQBytes);
  if (warp < 8) {
    s_fin[threadIdx.x >> 7][0][threadIdx.x & (kPfM - 1)] = l_run;
    s_fin[threadIdx.x >> 7][1][threadIdx.x & (kPfM - 1)] = m_ref;
  }
  __syncthreads();
  if (threadIdx.x == 0) RD_PF_TRACE(0, 47, 4);   // main loop done, sums exchanged

  // ---- epilogue: O / l (x sigmoid(gate)) -> global, 64 columns at a time ----
  // staging tile [128 rows][64 floats] aliases the Q region; 16-byte chunk q of row r is
  // stored at q ^ (r & 15), so both the row-wise writes and the coalesced reads are
  // conflict-free.
  if (warp < 8) {
    // warpgroup ch stores output columns [64*(2c+ch), +64), c = 0..1, through its own
    // staging tile and named barrier
    const int r = threadIdx.x & (kPfM - 1), ch = threadIdx.x >> 7, gt = threadIdx.x & (kPfM - 1);
    const uint32_t lane_addr = tmem + ((uint32_t)((warp & 3) * 32) << 16);
    // both sums at the reference the last tile left (a set without tiles: sum 0)
    const float m_fin = nt > 0 ? s_ref[(nt - 1) & 1][r] : -1.0e30f;
    const float l_tot = s_fin[0][0][r] * ex2(s_fin[0][1][r] - m_fin) + s_fin[1][0][r] * ex2(s_fin[1][1][r] - m_fin);
    const bool rec_mode = gridDim.z > 1;   // un-normalised records for prefill_merge_kernel
    const float inv = (l_tot > 0.f && !aborted) ? (rec_mode ? 1.0f : 1.0f / l_tot) : 0.f;
    const bool have = nt > 0 && !aborted;
    if (rec_mode && ch == 0 && row0 + r < p.n_q) {
      // header of this row's record; natural-log units like every record of the library
      float *rec = p.records + (((size_t)(row0 + r) * p.n_head + head) * gridDim.z + blockIdx.z) * kRec;
      const bool some = have && l_tot > 0.f;
      rec[0] = some ? m_fin * 0.6931471805599453f : -INFINITY;
      rec[1] = some ? l_tot : 0.f;
    }
    const uint32_t stg = sQ + ch * (kPfM * 256);
    uint8_t *gstg = gQ + ch * (kPfM * 256);
    for (int cc = 0; cc < 2; ++cc) {
      const int c = 2 * cc + ch;
      uint32_t o[2][32];
      if (have) {
        tmem_ld32(lane_addr + kTmemO + 64 * c, o[0]);
        tmem_ld32(lane_addr + kTmemO + 64 * c + 32, o[1]);
        tmem_wait_ld();
      }
#pragma unroll
      for (int q = 0; q < 16; ++q) {
        const int hq = q >> 3, iq = (q & 7) * 4;
        uint32_t w[4];
#pragma unroll
        for (int e = 0; e < 4; ++e)
          w[e] = have ? __float_as_uint(__uint_as_float(o[hq][iq + e]) * inv) : 0u;
        sts128(stg + r * 256 + ((q ^ (r & 15)) << 4), w[0], w[1], w[2], w[3]);
      }
      asm volatile("bar.sync %0, 128;" ::"r"(3 + ch) : "memory");
      if (threadIdx.x == 0) RD_PF_TRACE(1, 47, 2 + cc);   // round cc staged
      // 128 threads: 8 rows x 16 chunks per pass
      if (rec_mode) {
#pragma unroll 8
        for (int pass = 0; pass < kPfM / 8; ++pass) {
          const int rr = pass * 8 + (gt >> 4), q = gt & 15;
          const int gr = row0 + rr;
          if (gr < p.n_q) {
            // a record's values start 8 bytes into a 16-byte line: two 8-byte stores
            const float4 v = *reinterpret_cast<const float4 *>(gstg + rr * 256 + ((q ^ (rr & 15)) << 4));
            float2 *dst = reinterpret_cast<float2 *>(
                p.records + (((size_t)gr * p.n_head + head) * gridDim.z + blockIdx.z) * kRec + 2 + 64 * c + 4 * q);
            dst[0] = make_float2(v.x, v.y);
            dst[1] = make_float2(v.z, v.w);
          }
        }
      } else if (p.gate == nullptr) {
#pragma unroll 8
        for (int pass = 0; pass < kPfM / 8; ++pass) {
          const int rr = pass * 8 + (gt >> 4), q = gt & 15;
          const int gr = row0 + rr;
          if (gr < p.n_q)
            *reinterpret_cast<float4 *>(p.out + ((size_t)gr * p.n_head + head) * kHeadDim + 64 * c + 4 * q) =
                *reinterpret_cast<const float4 *>(gstg + rr * 256 + ((q ^ (rr & 15)) << 4));
        }
      } else {
        // the gate values of 4 passes are requested together before any store (out and gate
        // may alias as far as the compiler knows, so it would otherwise wait for every load
        // behind the previous store)
        for (int p0 = 0; p0 < kPfM / 8; p0 += 4) {
          float4 gv[4];
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            const int rr = (p0 + k) * 8 + (gt >> 4), gr = row0 + rr;
            gv[k] = make_float4(0.f, 0.f, 0.f, 0.f);
            if (gr < p.n_q)
              gv[k] = *reinterpret_cast<const float4 *>(p.gate + ((size_t)gr * p.n_head + head) * kHeadDim +
                                                        64 * c + 4 * (gt & 15));
          }
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            const int rr = (p0 + k) * 8 + (gt >> 4), q = gt & 15;
            const int gr = row0 + rr;
            if (gr < p.n_q) {
              float4 v = *reinterpret_cast<const float4 *>(gstg + rr * 256 + ((q ^ (rr & 15)) << 4));
              // fast exp/divide: ~1e-6 relative, far inside the attention tolerance
              v.x *= __fdividef(1.0f, 1.0f + __expf(-gv[k].x));
              v.y *= __fdividef(1.0f, 1.0f + __expf(-gv[k].y));
              v.z *= __fdividef(1.0f, 1.0f + __expf(-gv[k].z));
              v.w *= __fdividef(1.0f, 1.0f + __expf(-gv[k].w));
              *reinterpret_cast<float4 *>(p.out + ((size_t)gr * p.n_head + head) * kHeadDim + 64 * c + 4 * q) = v;
            }
          }
        }
      }
      asm volatile("bar.sync %0, 128;" ::"r"(3 + ch) : "memory");
      if (threadIdx.x == 0) RD_PF_TRACE(1, 47, cc);   // round cc stored
    }
  }
  tc_fence_before();
  __syncthreads();
  if (threadIdx.x == 0) RD_PF_TRACE(0, 47, 5);   // epilogue stores done
  if (warp == 9) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(kTmemCols)
                 : "memory");
  }
}

// Combines the key-split records of a row: one warp-pair (64 threads, 4 dims each) per row
// (token, head); out = sum_z acc_z e^(m_z - M) / sum_z l_z e^(m_z - M), times sigmoid(gate)
// if given (the gate is only read). Rows whose records are all empty give zeros.
__global__ void __launch_bounds__(256)
prefill_merge_kernel(const float *__restrict__ records, float *__restrict__ out, const float *__restrict__ gate,
                     int64_t n_rows, int n_splits) {
  const int64_t row = (int64_t)blockIdx.x * 4 + (threadIdx.x >> 6);
  const int tx = threadIdx.x & 63;
  pdl_wait();   // launched under the tile kernel: its records are complete from here on
  if (row >= n_rows) return;
  const float *rec = records + (size_t)row * n_splits * kRec;
  // every load of the row is requested before the first is used (at most kPfMaxSplits
  // records): one round trip to L2 instead of one for the maxima and one per record
  float m[kPfMaxSplits], lz[kPfMaxSplits];
  float2 va[kPfMaxSplits], vb[kPfMaxSplits];
#pragma unroll
  for (int z = 0; z < kPfMaxSplits; ++z) {
    m[z] = -INFINITY;
    lz[z] = 0.f;
    va[z] = vb[z] = make_float2(0.f, 0.f);
    if (z < n_splits) {
      const float *r = rec + (size_t)z * kRec;
      m[z] = __ldcg(r);
      lz[z] = __ldcg(r + 1);
      va[z] = __ldcg(reinterpret_cast<const float2 *>(r + 2 + 4 * tx));   // a record's values start 8 bytes
      vb[z] = __ldcg(reinterpret_cast<const float2 *>(r + 4 + 4 * tx));   // into a 16-byte line
    }
  }
  float4 g = make_float4(0.f, 0.f, 0.f, 0.f);
  if (gate != nullptr) g = *reinterpret_cast<const float4 *>(gate + (size_t)row * kHeadDim + 4 * tx);
  float mm = -INFINITY;
#pragma unroll
  for (int z = 0; z < kPfMaxSplits; ++z) mm = fmaxf(mm, m[z]);
  float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
  float l = 0.f;
  if (mm != -INFINITY) {
#pragma unroll
    for (int z = 0; z < kPfMaxSplits; ++z) {
      if (m[z] == -INFINITY) continue;
      const float w = __expf(m[z] - mm);
      l = fmaf(lz[z], w, l);
      acc.x = fmaf(va[z].x, w, acc.x);
      acc.y = fmaf(va[z].y, w, acc.y);
      acc.z = fmaf(vb[z].x, w, acc.z);
      acc.w = fmaf(vb[z].y, w, acc.w);
    }
  }
  const float inv = l > 0.f ? 1.0f / l : 0.f;
  float4 o = make_float4(acc.x * inv, acc.y * inv, acc.z * inv, acc.w * inv);
  if (gate != nullptr) {
    o.x *= __fdividef(1.0f, 1.0f + __expf(-g.x));
    o.y *= __fdividef(1.0f, 1.0f + __expf(-g.y));
    o.z *= __fdividef(1.0f, 1.0f + __expf(-g.z));
    o.w *= __fdividef(1.0f, 1.0f + __expf(-g.w));
  }
  *reinterpret_cast<float4 *>(out + (size_t)row * kHeadDim + 4 * tx) = o;
}

// Query pre-pass of the rotating prefill: one block per token. (cos, sin) of pos[t] * freq[i]
// once per rotated pair (24 heads share them), then every head row: partial RoPE in f32 with
// the operation order of the K side, x scale * log2(e), rounded to f16 -- [n_q][n_head][256]
// f16, the layout the tile kernel's TMA boxes read. The tile kernel is launched directly
// after it as a programmatic dependent launch.
__global__ void __launch_bounds__(256)
q_prep_kernel(const float *__restrict__ q, const int32_t *__restrict__ pos, int n_head, int n_rot, float qscale,
              uint4 *__restrict__ q16, const float *__restrict__ k_new, const float *__restrict__ v_new,
              uint4 *__restrict__ k_dst, uint4 *__restrict__ v_dst, int nkv,
              const __grid_constant__ RopeTable tab) {
  __shared__ float2 s_cs[32];
  pdl_launch_dependents();
  const int t = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int pairs = n_rot / 2;
  // a warp has at most three head rows (n_head <= 24): requested before the table is
  // computed, so that their latency and the sincosf run side by side
  float4 pa[3], pb[3];
#pragma unroll
  for (int j = 0; j < 3; ++j) {
    const int head = warp + 8 * j;
    pa[j] = pb[j] = make_float4(0.f, 0.f, 0.f, 0.f);
    if (head < n_head) {
      const float4 *src = reinterpret_cast<const float4 *>(q + ((size_t)t * n_head + head) * kHeadDim);
      pa[j] = src[2 * lane];
      pb[j] = src[2 * lane + 1];
    }
  }
  // ... and, with a fused append, the warp's K or V row of the token (2 * nkv <= 8 rows)
  float4 ka = make_float4(0.f, 0.f, 0.f, 0.f), kb = ka;
  if (k_new != nullptr && warp < 2 * nkv) {
    const float4 *src = reinterpret_cast<const float4 *>((warp < nkv ? k_new : v_new) +
                                                         ((size_t)t * nkv + (warp < nkv ? warp : warp - nkv)) * kHeadDim);
    ka = src[2 * lane];
    kb = src[2 * lane + 1];
  }
  if ((int)threadIdx.x < pairs) {
    float c, s;
    sincosf((float)pos[t] * tab.f[threadIdx.x], &s, &c);
    s_cs[threadIdx.x] = make_float2(c, s);
  }
  __syncthreads();
  // lanes 0..(n_rot/8 - 1) hold the rotated dims; dims d and d + n_rot/2 sit in lanes l and
  // l ^ (n_rot/16) at the same element index
  const int half_lanes = n_rot / 16;
  const bool rot = lane < 2 * half_lanes, lo = lane < half_lanes;
#pragma unroll
  for (int j = 0; j < 3; ++j) {
    const int head = warp + 8 * j;
    if (head >= n_head) break;
    const size_t row = (size_t)t * n_head + head;
    const float4 a = pa[j], b = pb[j];
    float v[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const float other = __shfl_xor_sync(0xffffffffu, v[i], half_lanes);
      if (rot) {
        const float2 cs = s_cs[8 * (lo ? lane : lane - half_lanes) + i];
        v[i] = lo ? __fsub_rn(__fmul_rn(v[i], cs.x), __fmul_rn(other, cs.y))
                  : __fadd_rn(__fmul_rn(other, cs.y), __fmul_rn(v[i], cs.x));
      }
    }
    q16[row * 32 + lane] = make_uint4(pack_h2(v[0] * qscale, v[1] * qscale), pack_h2(v[2] * qscale, v[3] * qscale),
                                      pack_h2(v[4] * qscale, v[5] * qscale), pack_h2(v[6] * qscale, v[7] * qscale));
  }
  // Fused append (k_new != nullptr): the token's K rows, rotated with the same (cos, sin) and
  // the operation order of kv_append_kernel, and its V rows, rounded to f16 into cache row t
  // -- the bytes rd_kv_append stores for f16 caches.
  if (k_new == nullptr || warp >= 2 * nkv) return;
  {
    const int r = warp;
    const bool is_k = r < nkv;
    const size_t row = (size_t)t * nkv + (is_k ? r : r - nkv);
    float v[8] = {ka.x, ka.y, ka.z, ka.w, kb.x, kb.y, kb.z, kb.w};
    if (is_k) {
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const float other = __shfl_xor_sync(0xffffffffu, v[i], half_lanes);
        if (rot) {
          const float2 cs = s_cs[8 * (lo ? lane : lane - half_lanes) + i];
          v[i] = lo ? __fsub_rn(__fmul_rn(v[i], cs.x), __fmul_rn(other, cs.y))
                    : __fadd_rn(__fmul_rn(other, cs.y), __fmul_rn(v[i], cs.x));
        }
      }
    }
    (is_k ? k_dst : v_dst)[row * 32 + lane] =
        make_uint4(pack_h2(v[0], v[1]), pack_h2(v[2], v[3]), pack_h2(v[4], v[5]), pack_h2(v[6], v[7]));
  }
}
size_t prefill_rope_bytes(int n_q, int n_head) { return (size_t)n_q * n_head * kHeadDim * 2; }

// Key splits that fill the GPU, picked with a three-constant cost model measured on B200:
// a key tile costs a CTA about 2 us, a CTA's prologue + epilogue about 9 us (the query
// tile is converted and the result written whatever the key count), and the records cost
// about 0.5 ns each (written by the tile kernel, read by the merge pass). Splitting pays only when the waves it saves outweigh the fixed
// costs it multiplies: 512 tokens x 24 heads gain from about 8192 keys upwards (3 splits:
// 96 -> 288 CTAs = two full waves of 148 SMs), shorter prefixes do not.
int prefill_splits(int n_q, int keys_total, int n_head, int sms) {
  const int ctas = ((n_q + kPfM - 1) / kPfM) * n_head;
  const int tiles = (keys_total + kPfN - 1) / kPfN;
#ifdef RD_TIMING_SWITCHES
  if (const char *e = getenv("RD_PF_SPLITS")) {   // timing builds: force a split count
    const int z = atoi(e);
    if (z >= 1 && z <= kPfMaxSplits && z <= tiles) return z;
  }
#endif
  auto cost = [&](int z) {
    const double waves = (double)((ctas * z + sms - 1) / sms);
    return waves * ((double)tiles / z * 2.0 + 9.0) + (z > 1 ? 0.0005 * n_q * n_head * z : 0.0);
  };
  int best = 1;
  double best_cost = cost(1) * 0.92;   // a split must win clearly to be worth its records
  for (int z = 2; z <= kPfMaxSplits && tiles / z >= 8; ++z) {
    if (cost(z) < best_cost) {
      best_cost = cost(z);
      best = z;
    }
  }
  return best;
}
size_t prefill_record_bytes(int n_q, int n_head, int splits) {
  return splits > 1 ? (size_t)n_q * n_head * splits * kRec * sizeof(float) : 0;
}

int launch_prefill(const float *q, const void *k, const void *v, float *out, const float *gate,
                   const int32_t *pos, int n_q, int keys_total, int n_head, int n_head_kv, float scale,
                   int n_rot, float freq_base, DeviceStatus *status, float *records, int n_splits,
                   void *q16, const float *k_new, const float *v_new, void *k_dst, void *v_dst,
                   cudaStream_t st) {
  PrefillArgs a;
  memset(&a, 0, sizeof(a));
  int rc = encode_f16_tmap(&a.tm_k, k, n_head_kv, keys_total, kPfN);
  if (rc != RD_OK) return rc;
  rc = encode_f16_tmap(&a.tm_v, v, n_head_kv, keys_total, kPfVUnitKeys);
  if (rc != RD_OK) return rc;
  a.q = q;
  a.out = out;
  a.gate = gate;
  a.pos = pos;
  a.n_q = n_q;
  a.n_head = n_head;
  a.nkv = n_head_kv;
  a.qscale = scale * 1.4426950408889634f;
  const bool prepass = n_rot > 0 || k_new != nullptr;   // rotation and / or fused append
  a.q16 = prepass ? 1 : 0;
  a.kv_wait = k_new != nullptr ? 1 : 0;
  if (prepass) {
    if (q16 == nullptr) return RD_ERR_WORKSPACE;
    if ((rc = encode_f16_tmap(&a.tm_q, q16, n_head, n_q, kPfM)) != RD_OK) return rc;
  }
  a.status = status;
  a.debug = 0;
#ifdef RD_TIMING_SWITCHES
  if (const char *e = getenv("RD_PREFILL_DEBUG")) a.debug = atoi(e);
#endif
  static bool attr_set[32] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return RD_ERR_CUDA;
  if (dev < 0 || dev >= 32 || !attr_set[dev]) {
    if (cudaFuncSetAttribute(prefill_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             kPfSmemBytes) != cudaSuccess)
      return RD_ERR_CUDA;
    if (dev >= 0 && dev < 32) attr_set[dev] = true;
  }
  if (n_splits < 1 || records == nullptr) n_splits = 1;
  a.records = records;
  const dim3 grid((unsigned)((n_q + kPfM - 1) / kPfM), (unsigned)n_head, (unsigned)n_splits);
  if (prepass) {
    q_prep_kernel<<<(unsigned)n_q, 256, 0, st>>>(q, pos, n_head, n_rot, a.qscale, (uint4 *)q16, k_new, v_new,
                                                (uint4 *)k_dst, (uint4 *)v_dst, n_head_kv,
                                                make_rope_table(n_rot, freq_base));
    if (cudaGetLastError() != cudaSuccess) return RD_ERR_CUDA;
    // the tile kernel may start while that pass runs; it waits for it (griddepcontrol)
    // before it loads its Q tile
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = dim3(kPfThreads);
    cfg.dynamicSmemBytes = kPfSmemBytes;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    if (cudaLaunchKernelEx(&cfg, prefill_kernel, a) != cudaSuccess) return RD_ERR_CUDA;
  } else {
    prefill_kernel<<<grid, kPfThreads, kPfSmemBytes, st>>>(a);
    if (cudaGetLastError() != cudaSuccess) return RD_ERR_CUDA;
  }
  if (n_splits > 1) {
    const int64_t n_rows = (int64_t)n_q * n_head;
    if (n_splits > kPfMaxSplits) return RD_ERR_SHAPE;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)((n_rows + 3) / 4));
    cfg.blockDim = dim3(256);
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    if (cudaLaunchKernelEx(&cfg, prefill_merge_kernel, (const float *)records, out, gate, n_rows, n_splits) !=
        cudaSuccess)
      return RD_ERR_CUDA;
  }
  return RD_OK;
}

}  // namespace rd

#ifdef RD_PF_TRACING
extern "C" int rd_debug_pf_trace(unsigned long long *host_dst) {
  return cudaMemcpyFromSymbol(host_dst, g_pf_trace, sizeof(g_pf_trace)) == cudaSuccess ? 0 : -1;
}
#endif
