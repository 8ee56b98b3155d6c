// Causal prefill attention on the 5th-generation tensor cores (tcgen05 + TMEM + TMA).
//
// Replaces attn_fa2_prefill_kernel (include/rdna4/attn_fa2.cuh:30-169 of the reference)
// for f16 K/V caches. One CTA owns a tile of 128 query tokens of ONE query head. Tensor
// memory (512 columns x 128 lanes, lane = query row) holds everything the tensor core
// reads or writes except K and V:
//   columns   0..255  O, the f32 output accumulator
//   columns 256..383  Q as f16 pairs (the A operand of S = Q K^T, read from TMEM)
//   columns 384..511  two score buffers of 64 f32 columns; the f16 P of a tile is
//                     written over the first 32 columns of its buffer (the A operand of
//                     O += P V, read from TMEM)
//
//   prologue   the 128 x 256 f32 query rows are loaded coalesced into a staging area,
//              each thread takes its row: optional partial RoPE, scale*log2(e), f16,
//              tcgen05.st into the Q columns;
//   per 64-key tile j (K and V on separate 2-stage TMA rings, sub-tiles of
//              [64 keys][64 dims], hardware 128B swizzle, one producer warp each):
//     MMA warp   S = Q K_j^T         16 x tcgen05.mma M128 N64  K16 (A in TMEM, B K-major)
//     8 warps    two threads per query row, 32 score columns each (row max exchanged
//                through shared memory): tcgen05.ld the scores, causal mask
//                (key <= pos[r]), running max with LAZY rescale (the reference point
//                only moves when a row's max grows by more than 2^8, so P stays below 256
//                in f16 and O in TMEM is rarely touched), P -> f16 pairs, tcgen05.st
//     MMA warp   O += P V_j           4 x tcgen05.mma M128 N256 K16 (A in TMEM, B = V
//                                     MN-major)
//   epilogue   O / l (times sigmoid(gate) if asked) through a swizzled staging tile to
//              coalesced f32 stores.
//
// Scores are double-buffered: the tensor core computes S of tile j+1 while the softmax
// warps work on tile j. The tensor pipe executes in issue order, which is what makes the
// in-place P safe: S of tile j+2 is issued after P V of tile j.
//
// Synchronisation is mbarriers only (TMA transaction counts, tcgen05.commit); every wait
// is bounded and a timeout unwinds the CTA (TMEM is always freed). No cluster launch, no
// multicast.
#include <stdlib.h>
#include <string.h>

#include "rd_common.cuh"
#include "rd_internal.h"

namespace rd {

constexpr int kPfM = 128;                 // query rows per CTA
constexpr int kPfN = 64;                  // keys per tile
constexpr int kPfStages = 2;
constexpr int kPfQBytes = kPfM * kHeadDim * 2;             // staging (prologue, epilogue): 65536
constexpr int kPfKVStageBytes = 2 * kPfN * kHeadDim * 2;   // K + V tile: 65536
// 192 KB of dynamic shared memory (one CTA per SM: TMEM is allocated whole)
constexpr int kPfSmemBytes = kPfQBytes + kPfStages * kPfKVStageBytes;
constexpr int kPfThreads = 384;           // 8 softmax warps, K TMA, S MMA, V TMA, PV MMA warps
constexpr uint32_t kTmemCols = 512;
constexpr uint32_t kTmemO = 0;            // columns [0, 256): output accumulator
constexpr uint32_t kTmemQ = 256;          // columns [256, 384): the query tile as f16 pairs
constexpr uint32_t kTmemS = 384;          // columns [384, 512): two score buffers of 64; the
                                          // f16 P of a tile overwrites its first 32 columns
constexpr float kLazyThreshold = 8.0f;    // log2 units

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
  int n_rot;             // 0: the queries are already rotated
  float freq_base;
  RopeTable rope;        // host-computed frequencies of the n_rot/2 <= 32 pairs
  int debug;             // timing experiments only (bit mask), 0 in production
  DeviceStatus *status;
};

// ---- tcgen05 wrappers -------------------------------------------------------------
__device__ __forceinline__ void tc_fence_before() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar)
               : "memory");
}
// D[tmem] (+)= A[tmem] * B[smem]: the A operand lives in tensor memory (rows = lanes, two
// f16 per 32-bit column), B behind a shared-memory descriptor.
__device__ __forceinline__ void tc_mma_f16_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc,
                                              uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
      :
      : "r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Shared-memory matrix descriptor, 128-byte swizzle, descriptor version 1 (sm_100).
__device__ __forceinline__ uint64_t smem_desc(uint32_t addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
  return (uint64_t)((addr >> 4) & 0x3FFFu) | ((uint64_t)((lbo_bytes >> 4) & 0x3FFFu) << 16) |
         ((uint64_t)((sbo_bytes >> 4) & 0x3FFFu) << 32) | (1ull << 46) | (2ull << 61);
}
// Instruction descriptor, kind::f16: f32 accumulate, f16 A and B.
__host__ __device__ constexpr uint32_t idesc_f16(int m, int n, bool b_mn_major) {
  return (1u << 4) | (b_mn_major ? (1u << 16) : 0u) | ((uint32_t)(n >> 3) << 17) |
         ((uint32_t)(m >> 4) << 24);
}
#define RD_LD64_REGS(r)                                                                         \
  "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),  \
  "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]),       \
  "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]),     \
  "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]),     \
  "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
// 32 lanes x 32 consecutive columns: thread i gets lane base+i, registers = columns.
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,"
      "%25,%26,%27,%28,%29,%30,%31}, [%32];"
      : RD_LD64_REGS(r)
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,"
      "%26,%27,%28,%29,%30,%31,%32};"
      :
      : "r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]),
        "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]),
        "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]),
        "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]),
        "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
      "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"
      :
      : "r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]),
        "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]),
        "r"(r[15])
      : "memory");
}
__device__ __forceinline__ void tmem_wait_ld() {
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_wait_st() {
  asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void sts128(uint32_t addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
  asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(addr), "r"(a), "r"(b), "r"(c), "r"(d)
               : "memory");
}

// Barrier slots (8 bytes each) at the start of the aligned shared-memory block.
// K and V tiles travel on separate rings: a K stage is free as soon as its S MMAs are
// done (long before the tile's P V), so K loads run two tiles ahead.
enum { kBarVFull = 0, kBarVFree = 2, kBarS = 4, kBarP = 6, kBarQ = 8, kBarKFull = 9, kBarKFree = 11,
       kBarX = 13, kBarCount = 15 };

// Build with -DRD_PREFILL_TRACE to accumulate clock64() spans of the per-tile phases of
// one softmax thread and of the MMA thread of CTA (0,0) (development aid, off by default).
#ifdef RD_PREFILL_TRACE
__device__ unsigned long long g_pf_trace[32];
#define RD_TR_DECL long long tr_t = clock64(); unsigned long long tr_acc[12] = {}
#define RD_TR(i) do { const long long tr_n = clock64(); tr_acc[i] += (unsigned long long)(tr_n - tr_t); tr_t = tr_n; } while (0)
#define RD_TR_OUT(base, n) do { if (blockIdx.x == 0 && blockIdx.y == 0) for (int tr_i = 0; tr_i < (n); ++tr_i) g_pf_trace[(base) + tr_i] = tr_acc[tr_i]; } while (0)
#else
#define RD_TR_DECL
#define RD_TR(i)
#define RD_TR_OUT(base, n)
#endif

__global__ void __launch_bounds__(kPfThreads, 1) prefill_kernel(const __grid_constant__ PrefillArgs p) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  __shared__ __align__(8) unsigned long long s_bars[kBarCount];
  __shared__ uint32_t s_tmem_base;
  __shared__ int s_maxpos;
  __shared__ int s_abort;
  __shared__ float s_freq[64];  // RoPE frequencies of the n_rot/2 pairs
  __shared__ float s_mx[2][2][kPfM];   // [tile parity][column half][row]: partial row maxima

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
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
  const uint32_t sKV = sQ + kPfQBytes;                    // stage s: K at +0, V at +32 KB
  uint8_t *gQ = smem_raw + (base - smem_u32(smem_raw));   // generic pointer to sQ
  const uint32_t bars = smem_u32(s_bars);

  if (threadIdx.x == 0) {
    s_maxpos = -1;
    s_abort = 0;
    for (int i = 0; i < kPfStages; ++i) {
      mbar_init(bars + 8 * (kBarVFull + i), 1);
      mbar_init(bars + 8 * (kBarVFree + i), 1);
      mbar_init(bars + 8 * (kBarKFull + i), 1);
      mbar_init(bars + 8 * (kBarKFree + i), 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(bars + 8 * (kBarS + i), 1);
      mbar_init(bars + 8 * (kBarP + i), 8);   // one elected lane per softmax warp
      mbar_init(bars + 8 * (kBarX + i), 8);
    }
    mbar_init(bars + 8 * kBarQ, 8);          // one per prologue warp
    fence_barrier_init();
  }
  if (p.n_rot > 0 && (int)threadIdx.x >= 64 && (int)threadIdx.x < 64 + p.n_rot / 2)
    s_freq[threadIdx.x - 64] = p.rope.f[threadIdx.x - 64];
  if (warp == 9) {  // TMEM: 512 columns for this CTA (one CTA per SM: no contention)
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                     smem_u32(&s_tmem_base)),
                 "r"(kTmemCols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  __syncthreads();

  // ---- positions of this tile's rows; the last key any of them attends ----
  int my_pos = -1;
  if (threadIdx.x < 2 * kPfM) {
    const int r = row0 + (threadIdx.x & (kPfM - 1));
    if (r < p.n_q) my_pos = p.pos[r];
  }
  if (threadIdx.x < kPfM) {
    int mx = my_pos;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mx = max(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    if (lane == 0) atomicMax(&s_maxpos, mx);
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = s_tmem_base;
  const int maxpos = s_maxpos;
  const int nt = maxpos >= 0 ? maxpos / kPfN + 1 : 0;  // key tiles this CTA walks

  // ---- prologue: Q rows -> f16 pairs in tensor memory (the A operand of S = Q K^T) ----
  // Two passes of two 64-dim chunks: all 8 warps load the chunks coalesced into a staging
  // area ([128 rows][64 floats] per chunk, 16-byte piece q of row r at q ^ (r & 15)), then
  // warps 0-3 take the even chunk and warps 4-7 the odd one: thread = row (= TMEM lane)
  // reads its 64 values, rotates them (chunk 0 holds all n_rot <= 64 rotated dims),
  // scales by scale*log2(e), packs and stores 32 columns with tcgen05.st.
  if (warp < 8) {
    const int r = threadIdx.x & (kPfM - 1), half_id = threadIdx.x >> 7;   // row, chunk parity
    const int gr_me = row0 + r;
    const float fpos = gr_me < p.n_q ? (float)p.pos[gr_me] : 0.f;
    const uint32_t lane_addr = tmem + ((uint32_t)((warp & 3) * 32) << 16);
#pragma unroll 1
    for (int pass = 0; pass < 2; ++pass) {
      // 2 chunks x 128 rows x 16 pieces = 4096 pieces of 16 bytes, 16 per thread
#pragma unroll 4
      for (int i = 0; i < 16; ++i) {
        const int idx = i * 256 + (int)threadIdx.x;
        const int cpar = idx >> 11, rr = (idx >> 4) & (kPfM - 1), q = idx & 15;
        const int gr = row0 + rr;
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        if (gr < p.n_q)
          v = *(reinterpret_cast<const float4 *>(p.q + ((size_t)gr * p.n_head + head) * kHeadDim +
                                                 64 * (2 * pass + cpar)) + q);
        sts128(sQ + cpar * (kPfM * 256) + rr * 256 + ((q ^ (rr & 15)) << 4), __float_as_uint(v.x),
               __float_as_uint(v.y), __float_as_uint(v.z), __float_as_uint(v.w));
      }
      asm volatile("bar.sync 2, 256;" ::: "memory");
      float x[64];
#pragma unroll
      for (int q = 0; q < 16; ++q) {
        const float4 v = *reinterpret_cast<const float4 *>(gQ + half_id * (kPfM * 256) + r * 256 +
                                                           ((q ^ (r & 15)) << 4));
        x[4 * q] = v.x; x[4 * q + 1] = v.y; x[4 * q + 2] = v.z; x[4 * q + 3] = v.w;
      }
      if (pass == 0 && half_id == 0 && p.n_rot > 0) {
        const int half = p.n_rot / 2;   // 8, 16, 24 or 32 pairs: (i, i + half)
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          if (i < half) {
            float c, sn;
            sincosf(fpos * s_freq[i], &sn, &c);
            // the partner index is a compile-time constant only for half == 32
            const float x0 = x[i];
            float x1 = 0.f;
#pragma unroll
            for (int k = 8; k <= 32; k += 8)
              if (half == k) x1 = x[i + k];
            const float y0 = __fsub_rn(__fmul_rn(x0, c), __fmul_rn(x1, sn));
            const float y1 = __fadd_rn(__fmul_rn(x0, sn), __fmul_rn(x1, c));
            x[i] = y0;
#pragma unroll
            for (int k = 8; k <= 32; k += 8)
              if (half == k) x[i + k] = y1;
          }
        }
      }
      uint32_t w[32];
#pragma unroll
      for (int i = 0; i < 32; ++i) w[i] = pack_h2(x[2 * i] * p.qscale, x[2 * i + 1] * p.qscale);
      tmem_st32(lane_addr + kTmemQ + 32 * (2 * pass + half_id), w);
      asm volatile("bar.sync 2, 256;" ::: "memory");   // staging free for the next pass
    }
    tmem_wait_st();
    tc_fence_before();
    __syncwarp();
    if (lane == 0) mbar_arrive(bars + 8 * kBarQ);  // the MMA warp waits for all 8 warps; TMA already runs
  }

  float l_run = 0.f;                 // softmax threads: row sum
  float m_ref = -1.0e30f;            //                  reference maximum (log2 units)

  if (warp == 8 || warp == 10) {
    // =============================== TMA producers =================================
    // warp 8 feeds the K ring, warp 10 the V ring. They are separate warps on purpose:
    // two lanes of one warp waiting on different barriers hold each other up (a lane
    // parked in try_wait parks the warp).
    if (lane == 0) {
      const bool is_k = warp == 8;
      const CUtensorMap *tm = is_k ? &p.tm_k : &p.tm_v;
      const int b_full = is_k ? kBarKFull : kBarVFull, b_free = is_k ? kBarKFree : kBarVFree;
      for (int j = 0; j < nt; ++j) {
        const int st = j & 1;
        if (j >= kPfStages && !mbar_wait(bars + 8 * (b_free + st), ((j >> 1) - 1) & 1, p.status, 11)) {
          s_abort = 1;
          break;
        }
        if (*(volatile int *)&s_abort) break;
        const uint32_t full = bars + 8 * (b_full + st);
        if (p.debug & 32) {
          mbar_arrive(full);
          continue;
        }
        mbar_expect_tx(full, kPfKVStageBytes / 2);
        const uint32_t dst = sKV + st * kPfKVStageBytes + (is_k ? 0 : kPfKVStageBytes / 2);
#pragma unroll
        for (int c = 0; c < 4; ++c)  // four [64 keys][64 dims] sub-tiles
          tma_load_2d(dst + c * (kPfN * 128), tm, kvh * kHeadDim + 64 * c, j * kPfN, full);
      }
    }
  } else if (warp == 9) {
    // ============================ MMA issuer: S = Q K^T =============================
    // The two contractions are issued by two threads (this one and warp 11): issuing a
    // tcgen05.mma costs the issuing thread tens of cycles whatever its size, and with
    // one thread the 16 small S MMAs and the 4 P V MMAs of a tile queue up behind each
    // other's waits.
    if (lane == 0) {
      constexpr uint32_t idesc_s = idesc_f16(kPfM, kPfN, false);
      // Descriptors differ only in the 16-byte-granular start address (low 14 bits, and
      // every address here is below 256 KB), so each one is a base plus a constant.
      const uint64_t dk = smem_desc(sKV, 16, 1024);
      RD_TR_DECL;
      bool ok = mbar_wait(bars + 8 * kBarQ, 0, p.status, 18);  // Q tile stored by warps 0-7
      tc_fence_after();
      for (int j = 0; j < nt && ok; ++j) {
        const int st = j & 1;
        RD_TR(0);
        if (!mbar_wait(bars + 8 * (kBarKFull + st), (j >> 1) & 1, p.status, 12)) { ok = false; break; }
        RD_TR(4);
        // score buffer st still holds P(j-2) until P V of tile j-2 has read it
        if (j >= 2 && !mbar_wait(bars + 8 * (kBarVFree + st), ((j - 2) >> 1) & 1, p.status, 15)) {
          ok = false;
          break;
        }
        RD_TR(1);
        tc_fence_after();
        // S(j) into score buffer j&1: A = Q from TMEM (16 dims = 8 columns per step),
        // B = K tile K-major, 8-row groups 1 KB apart
        const uint64_t dks = dk + (uint64_t)((st * kPfKVStageBytes) >> 4);
        const uint32_t d_s = tmem + kTmemS + 64 * st;
        if (!(p.debug & 8)) {
#pragma unroll
          for (int kk = 0; kk < 16; ++kk) {
            const uint64_t b = dks + (uint64_t)(((kk >> 2) * (kPfN * 128) + (kk & 3) * 32) >> 4);
            tc_mma_f16_ts(d_s, tmem + kTmemQ + 8 * kk, b, idesc_s, kk > 0);
          }
        }
        RD_TR(5);
        tc_commit(bars + 8 * (kBarS + st));
        tc_commit(bars + 8 * (kBarKFree + st));  // the K stage can be refilled
        RD_TR(6);
      }
      RD_TR_OUT(16, 7);
      if (!ok) s_abort = 1;
    }
  } else if (warp == 11) {
    // ============================ MMA issuer: O += P V ==============================
    if (lane == 0) {
      constexpr uint32_t idesc_o = idesc_f16(kPfM, kHeadDim, true);
      const uint64_t dv = smem_desc(sKV + kPfKVStageBytes / 2, kPfN * 128, 1024);
      bool ok = true;
      for (int j = 0; j < nt && ok; ++j) {
        const int st = j & 1;
        if (!mbar_wait(bars + 8 * (kBarP + st), (j >> 1) & 1, p.status, 13) ||
            !mbar_wait(bars + 8 * (kBarVFull + st), (j >> 1) & 1, p.status, 19)) {
          ok = false;
          break;
        }
        tc_fence_after();
        // A = P(j) from TMEM (16 keys = 8 columns per step), B = V MN-major: 64-dim groups
        // 8 KB apart (LBO), 8-key groups 1 KB apart (SBO); 4 steps of 16 keys = 2 KB each
        const uint64_t dvs = dv + (uint64_t)((st * kPfKVStageBytes) >> 4);
        const uint32_t a_p = tmem + kTmemS + 64 * st;
        if (!(p.debug & 4)) {
#pragma unroll
          for (int kk = 0; kk < 4; ++kk)
            tc_mma_f16_ts(tmem + kTmemO, a_p + 8 * kk, dvs + (uint64_t)((kk * 2048) >> 4), idesc_o,
                          (j > 0 || kk > 0) ? 1u : 0u);
        }
        tc_commit(bars + 8 * (kBarVFree + st));  // V stage and score buffer reusable, O settled
      }
      if (!ok) s_abort = 1;
    }
  } else {
    // ================== softmax: thread = (row r, 32-column half ch) ==================
    const int r = threadIdx.x & (kPfM - 1), ch = threadIdx.x >> 7;
    const uint32_t lane_addr = tmem + ((uint32_t)((warp & 3) * 32) << 16);
    bool ok = true;
    RD_TR_DECL;
    for (int j = 0; j < nt && ok; ++j) {
      const int st = j & 1;
      if (!mbar_wait(bars + 8 * (kBarS + st), (j >> 1) & 1, p.status, 14)) { ok = false; break; }
      RD_TR(0);
      tc_fence_after();
      uint32_t sraw[32];
      tmem_ld32(lane_addr + kTmemS + 64 * st + 32 * ch, sraw);
      tmem_wait_ld();
      RD_TR(1);
      const int key0 = j * kPfN + 32 * ch;
      // only tiles that reach past some row's last key need the causal mask
      if (__any_sync(0xffffffffu, key0 + 31 > my_pos)) {
#pragma unroll
        for (int i = 0; i < 32; ++i)
          if (key0 + i > my_pos) sraw[i] = 0xff800000u;  // -inf
      }
      float mx[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
      for (int i = 0; i < 32; ++i) mx[i & 3] = fmaxf(mx[i & 3], __uint_as_float(sraw[i]));
      float mt = fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3]));
      s_mx[st][ch][r] = mt;
      RD_TR(2);
      // exchange through an mbarrier (bounded wait) rather than bar.sync: a thread that
      // gave up on a wait must not leave the others parked on a hardware barrier
      // (this exchange also orders both halves' score loads before either half
      // overwrites the buffer with P)
      __syncwarp();
      if (lane == 0) mbar_arrive(bars + 8 * (kBarX + st));
      if (!mbar_wait(bars + 8 * (kBarX + st), (j >> 1) & 1, p.status, 20)) { ok = false; break; }
      mt = fmaxf(mt, s_mx[st][ch ^ 1][r]);   // both halves now agree on the row maximum
      RD_TR(3);
      RD_TR(4);
      const bool grow = mt > m_ref + kLazyThreshold;
      if (__any_sync(0xffffffffu, grow)) {
        const float m_new = fmaxf(m_ref, mt);
        const float f = ex2(m_ref - m_new);   // 1 for rows that keep their reference
        m_ref = m_new;
        l_run *= f;
        if (j > 0) {  // O holds data only after the first P V; and P V of tile j-1 must be done
          if (!mbar_wait(bars + 8 * (kBarVFree + ((j - 1) & 1)), ((j - 1) >> 1) & 1, p.status, 17)) {
            ok = false;
            break;
          }
          tc_fence_after();
#pragma unroll 1
          for (int c = 0; c < kHeadDim / 64; ++c) {   // this half's 128 output columns
            uint32_t o[32];
            const uint32_t col = kTmemO + 128 * ch + 32 * c;
            tmem_ld32(lane_addr + col, o);
            tmem_wait_ld();
#pragma unroll
            for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * f);
            tmem_st32(lane_addr + col, o);
          }
          tmem_wait_st();
        }
      }
      RD_TR(5);
      // P = 2^(s - m_ref) as f16 pairs, written over the score buffer: keys 32ch..32ch+31
      // of row r become columns 16ch..16ch+15 (the A operand of P V, read from TMEM)
      float ls[4] = {0.f, 0.f, 0.f, 0.f};
      uint32_t pw[16];
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        const float p0 = (p.debug & 1) ? __uint_as_float(sraw[2 * i]) : ex2(__uint_as_float(sraw[2 * i]) - m_ref);
        const float p1 = (p.debug & 1) ? __uint_as_float(sraw[2 * i + 1]) : ex2(__uint_as_float(sraw[2 * i + 1]) - m_ref);
        ls[i & 3] += p0 + p1;
        pw[i] = pack_h2(p0, p1);
      }
      tmem_st16(lane_addr + kTmemS + 64 * st + 16 * ch, pw);
      l_run += (ls[0] + ls[1]) + (ls[2] + ls[3]);
      RD_TR(6);
      tmem_wait_st();
      tc_fence_before();
      RD_TR(7);
      __syncwarp();
      if (lane == 0) mbar_arrive(bars + 8 * (kBarP + st));
      RD_TR(8);
    }
#ifdef RD_PREFILL_TRACE
    if (threadIdx.x == 0) RD_TR_OUT(0, 9);
    if (threadIdx.x == 0 && blockIdx.x == 0 && blockIdx.y == 0) g_pf_trace[15] = (unsigned long long)nt;
#endif
    if (ok && nt > 0 &&
        !mbar_wait(bars + 8 * (kBarVFree + ((nt - 1) & 1)), ((nt - 1) >> 1) & 1, p.status, 16))
      ok = false;
    if (!ok) s_abort = 1;
    tc_fence_after();
  }

  __syncthreads();
  const bool aborted = s_abort != 0;
  // the two column halves of a row add their partial sums (s_mx is free now)
  if (warp < 8) s_mx[0][threadIdx.x >> 7][threadIdx.x & (kPfM - 1)] = l_run;
  __syncthreads();

  // ---- epilogue: O / l (x sigmoid(gate)) -> global, 64 columns at a time ----
  // staging tile [128 rows][64 floats] aliases the Q region; 16-byte chunk q of row r is
  // stored at q ^ (r & 15), so both the row-wise writes and the coalesced reads are
  // conflict-free.
  if (warp < 8) {
    // warpgroup ch stores output columns [64*(2c+ch), +64), c = 0..1, through its own
    // staging tile and named barrier
    const int r = threadIdx.x & (kPfM - 1), ch = threadIdx.x >> 7, gt = threadIdx.x & (kPfM - 1);
    const uint32_t lane_addr = tmem + ((uint32_t)((warp & 3) * 32) << 16);
    const float l_tot = s_mx[0][0][r] + s_mx[0][1][r];
    const float inv = (l_tot > 0.f && !aborted) ? 1.0f / l_tot : 0.f;
    const bool have = nt > 0 && !aborted;
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
      // 128 threads: 8 rows x 16 chunks per pass
#pragma unroll 8
      for (int pass = 0; pass < kPfM / 8; ++pass) {
        const int rr = pass * 8 + (gt >> 4), q = gt & 15;
        const int gr = row0 + rr;
        if (gr < p.n_q) {
          float4 v = *reinterpret_cast<const float4 *>(gstg + rr * 256 + ((q ^ (rr & 15)) << 4));
          const size_t off = ((size_t)gr * p.n_head + head) * kHeadDim + 64 * c + 4 * q;
          if (p.gate != nullptr) {
            const float4 g = *reinterpret_cast<const float4 *>(p.gate + off);
            // fast exp/divide: ~1e-6 relative, far inside the attention tolerance
            v.x *= __fdividef(1.0f, 1.0f + __expf(-g.x));
            v.y *= __fdividef(1.0f, 1.0f + __expf(-g.y));
            v.z *= __fdividef(1.0f, 1.0f + __expf(-g.z));
            v.w *= __fdividef(1.0f, 1.0f + __expf(-g.w));
          }
          *reinterpret_cast<float4 *>(p.out + off) = v;
        }
      }
      asm volatile("bar.sync %0, 128;" ::"r"(3 + ch) : "memory");
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 9) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(kTmemCols)
                 : "memory");
  }
}

int launch_prefill(const float *q, const void *k, const void *v, float *out, const float *gate,
                   const int32_t *pos, int n_q, int keys_total, int n_head, int n_head_kv, float scale,
                   int n_rot, float freq_base, DeviceStatus *status, cudaStream_t st) {
  PrefillArgs a;
  memset(&a, 0, sizeof(a));
  int rc = encode_f16_tmap(&a.tm_k, k, n_head_kv, keys_total, kPfN);
  if (rc != RD_OK) return rc;
  rc = encode_f16_tmap(&a.tm_v, v, n_head_kv, keys_total, kPfN);
  if (rc != RD_OK) return rc;
  a.q = q;
  a.out = out;
  a.gate = gate;
  a.pos = pos;
  a.n_q = n_q;
  a.n_head = n_head;
  a.nkv = n_head_kv;
  a.qscale = scale * 1.4426950408889634f;
  a.n_rot = n_rot;
  a.freq_base = freq_base;
  a.rope = make_rope_table(n_rot, freq_base);
  a.status = status;
  {
    const char *e = getenv("RD_PREFILL_DEBUG");
    a.debug = e ? atoi(e) : 0;
  }
  static bool attr_set[32] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return RD_ERR_CUDA;
  if (dev < 0 || dev >= 32 || !attr_set[dev]) {
    if (cudaFuncSetAttribute(prefill_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             kPfSmemBytes) != cudaSuccess)
      return RD_ERR_CUDA;
    if (dev >= 0 && dev < 32) attr_set[dev] = true;
  }
  const dim3 grid((unsigned)((n_q + kPfM - 1) / kPfM), (unsigned)n_head);
  prefill_kernel<<<grid, kPfThreads, kPfSmemBytes, st>>>(a);
  return cudaGetLastError() == cudaSuccess ? RD_OK : RD_ERR_CUDA;
}

}  // namespace rd

#ifdef RD_PREFILL_TRACE
extern "C" int rd_prefill_trace(unsigned long long *out32) {
  return cudaMemcpyFromSymbol(out32, rd::g_pf_trace, sizeof(rd::g_pf_trace)) == cudaSuccess ? 0 : -6;
}
#endif
