// Split-KV decode attention with both contractions on the 5th-generation tensor cores:
// the quantized K / V blocks are dequantized in registers by the same fragment loaders as
// decode_kernel (rd_decode.cuh), but the fragments are stored into TENSOR MEMORY as the A
// operand of tcgen05.mma instead of feeding mma.sync, the accumulators (scores and O) live in
// tensor memory, and the query block / the softmax weights are the B operands in shared
// memory. Same contract as decode_kernel: CTA s owns a contiguous run of 16-key slots and
// writes one partial record (m, l, acc[256]) per query head (include/rdna4/attn.cuh:445-560).
//
// Why: on sm_100 the legacy mma.sync path costs about a third of decode_kernel's key loop
// (33 MMAs per 16 keys x kv head that the other pipes do not hide) and pins 96 registers per
// thread for accumulators and query fragments. Here one elected thread issues 16 tcgen05.mma
// per 16-key slot for all four kv heads together.
//
// Geometry (n_head_kv == 4, 6 query heads per kv head, head_dim 256):
//   * 8 warps = 2 teams x 4 warps; warp (team, q) owns kv head q and -- because warp w can
//     only touch tensor-memory lanes 32 (w % 4) .. + 31 -- lane quarter q. Teams take the
//     CTA's slots in turn (team t: slots t, t + 2, ...), each through its own ring.
//   * Q K^T: M = 128 rows = 4 quarters x 32 lanes; in quarter q, lanes 0-15 hold the slot's 16
//     keys of kv head q for dims "half 0" (fragment units n = 0..7) and lanes 16-31 the same
//     keys for "half 1" (n = 8..15); K = 16 per MMA, 8 MMAs j = 0..7 over 8 columns each.
//     The two halves need different query dims, so B carries both: N = 64 columns
//     = (half, kv head q', head h) -> n = 32 half + 8 q' + h, and the lanes of half x read
//     their partial score from columns 32 x + 8 q .. + 5; the two partials of a key meet
//     with one shuffle.
//   * P V: M = 128 rows = (kv head q, 32 dims of slice s), 8 slices, K = the slot's 16 keys,
//     N = 32 columns = (kv head q', head h): only the diagonal blocks q' = q mean anything,
//     which keeps every lane quarter private to its kv head. O = 8 slices x 32 columns.
//   * tensor memory (512 columns): O 0..255; team t: operand staging 64 columns (K, then V
//     of the same slot once the score MMAs are done) and 64 score columns.
//   * softmax with a lazy reference per head (moves only when a score exceeds it by 2^8,
//     O in tensor memory rescaled then); the two teams' warps of a quarter share the
//     reference and take their slots' softmax strictly in slot order, and the P V batches
//     are issued in slot order, so every sum has a fixed order.
#pragma once
#include "rd_decode.cuh"
#include "rd_tc.cuh"

namespace rd {

constexpr int kTcTeams = 2;
constexpr int kTcComputeThreads = kTcTeams * 4 * 32;
constexpr int kTcThreads = kTcComputeThreads + 32;   // + the warp that issues the MMAs
constexpr uint32_t kTcColsO = 0;                 // 8 slices x 32 columns
constexpr uint32_t kTcColsTeam = 256;            // team t: + 128 t
constexpr uint32_t kTcStage = 0, kTcScore = 64;  // inside a team's 128 columns
constexpr int kTcQBytes = 8 * 2048;              // B of Q K^T: 8 MMAs x [64 n][16 k] f16
constexpr int kTcPBytes = 1024;                  // B of P V: [16 k][32 n] f16, per team
// front of the dynamic shared memory: barriers and counters (512 bytes), Q, P x 2
constexpr int kTcRingOffset = 512 + kTcQBytes + kTcTeams * kTcPBytes;
static_assert(kTcRingOffset % 128 == 0, "ring must start 128-byte aligned");

__host__ __device__ constexpr int tc_ring_depth(int kt, int vt) {
  const int d = (kSmemBudget - kTcRingOffset) / (kTcTeams * slot_bytes(kt, vt, 4));
  return d > kMaxStages ? kMaxStages : d;
}
// The tensor-memory kernel serves block-quantized K and V (small rows: one tensor-map box
// per slot) when every team gets a ring of at least three slots.
__host__ __device__ constexpr bool tc_decode_usable(int kt, int vt) {
  return kt >= RD_KV_Q8_0 && vt >= RD_KV_Q8_0 && tc_ring_depth(kt, vt) >= 3;
}

// spin on a shared-memory word until it reaches `want`; gives up (returns false) after
// about a second or as soon as the CTA is unwinding
__device__ __forceinline__ bool tc_wait_seq(const volatile int *word, int want, const volatile int *abort_flag) {
  for (uint32_t i = 0; i < (64u << 20); ++i) {
    if (*word >= want) return true;
    if ((i & 255u) == 255u && *abort_flag) return false;
  }
  return false;
}

template <int KT, int VT>
__global__ void __launch_bounds__(kTcThreads, 1) decode_tc_kernel(const __grid_constant__ DecodeKernelArgs p) {
  constexpr int RK = row_bytes(KT), RV = row_bytes(VT);
  constexpr int PK = 4 * RK + 16, PV = 4 * RV + 16;   // key pitch in a slot (4 kv heads + pad)
  constexpr uint32_t SLOT = (uint32_t)kSlotKeys * (PK + PV);
  constexpr uint32_t V_OFF = kSlotKeys * PK;
  using KL = KLoad<KT>;
  using VL = VLoad<VT>;
  constexpr unsigned FULL = 0xffffffffu;
  constexpr float kNegBig = -1.0e30f;

  extern __shared__ __align__(128) uint8_t smem[];
  __shared__ int s_abort, s_seq_sm[4];
  __shared__ uint32_t s_tmem_base;
  __shared__ float s_mref[4][8];                        // lazy softmax reference per (kv head, head)
  __shared__ float s_red[kTcTeams][4][16];              // epilogue: per (team, kv head): 6 maxima, 6 sums
  pdl_launch_dependents();
  if (threadIdx.x == 0 && p.k_tmap) asm volatile("prefetch.tensormap [%0];" ::"l"(&p.tm_k) : "memory");
  if (threadIdx.x == 32 && p.v_tmap) asm volatile("prefetch.tensormap [%0];" ::"l"(&p.tm_v) : "memory");

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, tq = lane & 3;
  const int team = warp >> 2, q = warp & 3;             // q = kv head = tensor-memory lane quarter
  const int D = p.depth;
  const uint32_t sbase = smem_u32(smem);
  // barriers: full[team * D + d], then score-ready and PV-done per team
  const uint32_t bar_full = sbase;                               // 16 x 8 bytes
  const uint32_t bar_s = sbase + 8 * 16, bar_pv = bar_s + 8 * kTcTeams;
  const uint32_t bar_k = bar_pv + 8 * kTcTeams, bar_p = bar_k + 8 * kTcTeams;   // K staged / P and V staged
  const uint32_t cnt0 = sbase + 192, nfill0 = cnt0 + 64, sid0 = nfill0 + 64;   // 16 x 4 bytes each
  const uint32_t sQ = sbase + 512, sP = sQ + kTcQBytes + team * kTcPBytes;
  const uint32_t ring0 = sbase + kTcRingOffset;
  const uint32_t my_ring = ring0 + team * (uint32_t)p.group_bytes;
  volatile int *abort_flag = &s_abort;

  if (threadIdx.x == 0) {
    s_abort = 0;
    for (int i = 0; i < 4; ++i) s_seq_sm[i] = 0;
    for (int i = 0; i < kTcTeams * D; ++i) {
      mbar_init(bar_full + 8 * i, 1);
      sts32(cnt0 + 4 * i, 0u);
      sts32(nfill0 + 4 * i, 0u);
    }
    for (int i = 0; i < kTcTeams; ++i) {
      mbar_init(bar_s + 8 * i, 1);
      mbar_init(bar_pv + 8 * i, 1);
      mbar_init(bar_k + 8 * i, 4);   // one arrival per warp of the team
      mbar_init(bar_p + 8 * i, 4);
    }
    fence_barrier_init();
  }
  if (threadIdx.x < 32) s_mref[threadIdx.x >> 3][threadIdx.x & 7] = kNegBig;
  if (warp == 0) {   // all 512 columns: one CTA per SM, nobody to share with
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&s_tmem_base)),
                 "r"(512u)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  pdl_wait();   // everything below reads what earlier kernels of the stream wrote

  const int s = blockIdx.x, S = gridDim.x;
  const int t_last = p.t, key_begin = p.key_begin;
  float *rec0 = p.partial + (size_t)s * kRec;
  const int n_keys = t_last >= key_begin ? t_last - key_begin + 1 : 0;
  const int slots_total = (n_keys + kSlotKeys - 1) / kSlotKeys;
  const int c_b = (int)(((int64_t)slots_total * s) / S);
  const int c_e = (int)(((int64_t)slots_total * (s + 1)) / S);
  const int n_slots = c_e - c_b;
  const int key0 = key_begin + c_b * kSlotKeys;

  // ---- B operand of Q K^T: for MMA j, tile [n = 32 half + 8 q' + h][kk], K-major core
  // matrices (8 n x 8 kk, 128 bytes): kk-th contraction element of fragment unit 8 half + j
  // is dim KL::dim(kk >> 2, 8 half + j, kk & 3); columns h = 6, 7 are zero.
  {
    const float qmul = p.qscale * KL::kUnscale;
    for (int e = threadIdx.x; e < 8 * 64 * 16; e += kTcThreads) {
      const int j = e >> 10, n = (e >> 4) & 63, kk = e & 15;
      const int half = n >> 5, qq = (n >> 3) & 3, h = n & 7;
      float v = 0.f;
      if (h < kGroup) v = p.q[(size_t)(qq * kGroup + h) * kHeadDim + KL::dim(kk >> 2, 8 * half + j, kk & 3)] * qmul;
      const uint32_t addr = sQ + j * 2048 + (n >> 3) * 256 + (kk >> 3) * 128 + (n & 7) * 16 + (kk & 7) * 2;
      asm volatile("st.shared.u16 [%0], %1;" ::"r"(addr), "h"(__half_as_ushort(__float2half_rn(v))) : "memory");
    }
    fence_proxy_async();   // generic-proxy writes -> visible to the tensor core's async proxy
  }

  // Loads this team's next slot for ring position d, or completes the position empty
  // (slot number -1) once the team's slots have run out. Warp-collective.
  auto fill = [&](int ft, int d) {
    const int pos = ft * D + d;
    const uint32_t bar = bar_full + 8 * pos;
    const uint32_t sk = ring0 + ft * (uint32_t)p.group_bytes + d * SLOT, sv = sk + V_OFF;
    int c = 0;
    if (lane == 0) {
      const uint32_t lap = lds32(nfill0 + 4 * pos);
      c = ft + kTcTeams * ((int)lap * D + d);
      if (c >= n_slots) c = -1;
      sts32(sid0 + 4 * pos, (uint32_t)c);
      sts32(nfill0 + 4 * pos, lap + 1u);
      if (c < 0)
        mbar_arrive(bar);
      else
        mbar_expect_tx(bar, kSlotKeys * (PK + PV));   // a box counts its zero-filled padding too
    }
    c = __shfl_sync(FULL, c, 0);
    if (c < 0) return;
    const int row0 = key0 + c * kSlotKeys;
    if (lane == 0) tma_load_2d(sk, &p.tm_k, 0, row0, bar);
    if (lane == 16) tma_load_2d(sv, &p.tm_v, 0, row0, bar);
  };

  tc_fence_before();
  __syncthreads();   // barriers, tensor memory, the Q operand are in place
  tc_fence_after();
  const uint32_t tmem = s_tmem_base;
  const uint32_t lane_addr = tmem + ((uint32_t)(32 * q) << 16);
  const uint32_t t_stage = kTcColsTeam + 128 * team + kTcStage, t_score = kTcColsTeam + 128 * team + kTcScore;
  if (warp == 0)
    for (int ft = 0; ft < kTcTeams; ++ft) fill(ft, 0);
  if (warp < 8)
    for (int x = 1; x < D; ++x)
      if ((x & 3) == q) fill(team, x);

  // ---- per-thread softmax state: lanes 0-15 of a warp own the slot's 16 keys ----
  float run[kGroup], lsum[kGroup], lref[kGroup];
#pragma unroll
  for (int h = 0; h < kGroup; ++h) {
    run[h] = kNegBig;
    lsum[h] = 0.f;
    lref[h] = kNegBig;
  }
  constexpr uint32_t idesc_s = idesc_f16(128, 64, false);   // scores: B K-major
  constexpr uint32_t idesc_o = idesc_f16(128, 32, true);    // output: B (= P) MN-major
  const uint64_t qdesc = smem_desc_plain(sQ, 128, 256);
  const uint64_t pdesc = smem_desc_plain(sP, 128, 256);
  const uint32_t k_row = (uint32_t)g * PK + q * RK;
  const uint32_t v_row = (uint32_t)(2 * tq) * PV + q * RV;
#ifdef RD_TIMING_SWITCHES
  long long tw[10] = {0, 0, 0, 0, 0, 0, 0, 0, 0, 0};
  long long tprev = clock64();
  const long long tloop0 = tprev;
#define RD_TCT(i)                      \
  {                                    \
    const long long tn_ = clock64();   \
    tw[i] += tn_ - tprev;              \
    tprev = tn_;                       \
  }
#else
#define RD_TCT(i)
#endif
  const int max_iters = n_slots / kTcTeams + 2;   // a team's slots, and the empty position that ends them
  if (warp == 8) {
    // ========================= the MMA issuer (one thread) =========================
    // Fixed order: scores of slot c, then P V of slot c - 1. Scores only wait for the
    // team's K fragments (whose columns the P V of slot c - 2, issued two steps back, has
    // released by then); the P V batches follow each other in slot order, so every output
    // sum has a fixed order and the first batch initialises O.
    if (lane == 0) {
      for (int c = 0; c <= n_slots; ++c) {
        if (c < n_slots) {
          const int t = c & 1, il = c >> 1;
          if (!*abort_flag && !mbar_wait(bar_k + 8 * t, il & 1, p.status, 35)) s_abort = 1;
          tc_fence_after();
          const uint32_t stg = kTcColsTeam + 128 * t + kTcStage, scr = kTcColsTeam + 128 * t + kTcScore;
#pragma unroll
          for (int j = 0; j < 8; ++j)
            tc_mma_f16_ts(tmem + scr, tmem + stg + 8 * j, qdesc + (uint64_t)(j * (2048 >> 4)), idesc_s, j > 0);
          tc_commit(bar_s + 8 * t);
        }
        if (c >= 1) {
          const int t = (c - 1) & 1, il = (c - 1) >> 1;
          if (!*abort_flag && !mbar_wait(bar_p + 8 * t, il & 1, p.status, 36)) s_abort = 1;
          tc_fence_after();
          const uint32_t stg = kTcColsTeam + 128 * t + kTcStage;
          const uint64_t pd = smem_desc_plain(sQ + kTcQBytes + t * kTcPBytes, 128, 256);
#pragma unroll
          for (int sl = 0; sl < 8; ++sl)
            tc_mma_f16_ts(tmem + kTcColsO + 32 * sl, tmem + stg + 8 * sl, pd, idesc_o, c - 1 > 0);
          tc_commit(bar_pv + 8 * t);
        }
      }
    }
  } else

  {
  int d = 0;         // ring position of the next slot to consume
  uint32_t ph = 0;   // and the parity its full barrier completes with
  for (int i = 0; i < max_iters; ++i) {
    const int pos = team * D + d;
    if (!*abort_flag && !mbar_wait(bar_full + 8 * pos, ph, p.status, 2)) s_abort = 1;
    const int c = (int)lds32(sid0 + 4 * pos);   // the CTA's slot number held here; the same for the team's warps
    if (c < 0) break;
    RD_TCT(0);   // waiting for the slot
    const uint32_t sk = my_ring + d * SLOT, sv = sk + V_OFF;
    const int kfirst = key0 + c * kSlotKeys;

    // (1) K fragments (unit n goes to lane half n >> 3, columns 8 (n & 7)) ...
    {
      uint32_t kf[16][4];
      KL::run(sk + k_row, sk + k_row + 8 * PK, tq, [&](int n, uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3) {
        kf[n][0] = a0, kf[n][1] = a2, kf[n][2] = a1, kf[n][3] = a3;
      });
      RD_TCT(1);   // K dequantization
      // (2) ... into the staging columns, once the P V batch of this team's previous slot
      // has read them
      if (i > 0 && !*abort_flag && !mbar_wait(bar_pv + 8 * team, (i - 1) & 1, p.status, 31)) s_abort = 1;
      tc_fence_after();
      RD_TCT(2);   // waiting for the previous P V
#pragma unroll
      for (int b = 0; b < 4; ++b) {
        uint32_t r[16];
#pragma unroll
        for (int u = 0; u < 4; ++u)
#pragma unroll
          for (int e = 0; e < 4; ++e) r[4 * u + e] = kf[4 * b + u][e];
        tmem_st_16x256b_x4(lane_addr + ((uint32_t)(16 * (b >> 1)) << 16) + t_stage + 32 * (b & 1), r);
      }
      tmem_wait_st();
      tc_fence_before();
    }
    RD_TCT(3);   // K stores
    __syncwarp();
    if (lane == 0) mbar_arrive(bar_k + 8 * team);   // the issuer starts the score MMAs after the fourth
    RD_TCT(4);
    // (3) V fragments into registers while the score MMAs run; then the slot can go back
    uint32_t vf[16][4];
    {
      uint32_t rows[4];
      const uint32_t r0 = sv + v_row;
      rows[0] = r0, rows[1] = r0 + PV, rows[2] = r0 + 8 * PV, rows[3] = r0 + 9 * PV;
      VL::run(rows, g, [&](int m, uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3) {
        vf[m][0] = a0, vf[m][1] = a2, vf[m][2] = a1, vf[m][3] = a3;
      });
    }
    __syncwarp();
    {
      uint32_t last = 0;
      if (lane == 0) last = atom_add_acq_rel_shared(cnt0 + 4 * pos, 1u) == 3u;
      last = __shfl_sync(FULL, last, 0);
      if (last) {
        if (lane == 0) sts32(cnt0 + 4 * pos, 0u);
        fill(team, d);
      }
    }
    RD_TCT(5);   // V dequantization, slot hand-back
    // (4) scores of this warp's keys; the staging columns are free again: V goes in
    if (!*abort_flag && !mbar_wait(bar_s + 8 * team, i & 1, p.status, 32)) s_abort = 1;
    tc_fence_after();
    RD_TCT(6);   // waiting for the scores
#pragma unroll
    for (int b = 0; b < 4; ++b) {   // unit m: lane half m & 1, columns 8 (m >> 1)
      uint32_t r[16];
#pragma unroll
      for (int u = 0; u < 4; ++u)
#pragma unroll
        for (int e = 0; e < 4; ++e) r[4 * u + e] = vf[2 * (4 * (b & 1) + u) + (b >> 1)][e];
      tmem_st_16x256b_x4(lane_addr + ((uint32_t)(16 * (b >> 1)) << 16) + t_stage + 32 * (b & 1), r);
    }
    float sc[kGroup];
    {
      uint32_t s0[8], s1[8];
      tmem_ld8(lane_addr + t_score + 8 * q, s0);
      tmem_ld8(lane_addr + t_score + 32 + 8 * q, s1);
      tmem_wait_ld();
      const bool dead = kfirst + (lane & 15) > t_last;   // key beyond the last attended one
#pragma unroll
      for (int h = 0; h < kGroup; ++h) {
        const float mine = __uint_as_float(lane < 16 ? s0[h] : s1[h]);
        const float both = mine + __shfl_xor_sync(FULL, mine, 16);
        sc[h] = dead ? -INFINITY : both;
        run[h] = fmaxf(run[h], sc[h]);
      }
    }
    RD_TCT(7);   // V stores, score loads
    // (5) softmax against the quarter's shared reference, in slot order across the teams
    if (!tc_wait_seq(&s_seq_sm[q], c, abort_flag)) s_abort = 1;
    RD_TCT(8);   // waiting for the quarter's turn
    float mr[kGroup];
    bool grow = false;
#pragma unroll
    for (int h = 0; h < kGroup; ++h) {
      mr[h] = *reinterpret_cast<volatile float *>(&s_mref[q][h]);
      grow |= sc[h] > mr[h] + kRefSlack;
    }
    if (__any_sync(FULL, grow)) {
      // move the references to the column maxima and rescale O (rare: once or twice per CTA)
      float cf[kGroup];
#pragma unroll
      for (int h = 0; h < kGroup; ++h) {
        float nm = sc[h];
#pragma unroll
        for (int o = 1; o < 16; o <<= 1) nm = fmaxf(nm, __shfl_xor_sync(FULL, nm, o));
        nm = fmaxf(nm, mr[h]);
        cf[h] = ex2(mr[h] - nm);
        mr[h] = nm;
      }
      if (c > 0) {   // every P V batch up to slot c - 1 (they run in slot order) must have landed
        if (!*abort_flag && !mbar_wait(bar_pv + 8 * ((c - 1) & 1), ((c - 1) >> 1) & 1, p.status, 33)) s_abort = 1;
        tc_fence_after();
#pragma unroll 1
        for (int sl = 0; sl < 8; ++sl) {
          uint32_t o[8];
          tmem_ld8(lane_addr + kTcColsO + 32 * sl + 8 * q, o);
          tmem_wait_ld();
#pragma unroll
          for (int h = 0; h < kGroup; ++h) o[h] = __float_as_uint(__uint_as_float(o[h]) * cf[h]);
          tmem_st8(lane_addr + kTcColsO + 32 * sl + 8 * q, o);
        }
      }
      if (lane == 0) {
#pragma unroll
        for (int h = 0; h < kGroup; ++h) *reinterpret_cast<volatile float *>(&s_mref[q][h]) = mr[h];
      }
    }
    {
      float pr[kGroup];
#pragma unroll
      for (int h = 0; h < kGroup; ++h) {
        pr[h] = ex2(sc[h] - mr[h]);
        if (lane < 16) {
          if (lref[h] != mr[h]) {   // this thread's sum is still relative to an older reference
            lsum[h] *= ex2(lref[h] - mr[h]);
            lref[h] = mr[h];
          }
          lsum[h] += pr[h];
        }
      }
      if (lane < 16) {
        // row kk of the B operand: contraction element kk of the V fragments is key
        // 2 (kk >> 2) + (kk & 1) + 8 ((kk >> 1) & 1)
        const int r = lane, kk = 4 * ((r & 7) >> 1) + (r & 1) + 2 * (r >> 3);
        sts128(sP + q * 256 + (kk >> 3) * 128 + (kk & 7) * 16, pack_h2(pr[0], pr[1]), pack_h2(pr[2], pr[3]),
               pack_h2(pr[4], pr[5]), 0u);
      }
    }
    fence_proxy_async();   // P: generic-proxy writes -> the tensor core's async proxy
    tmem_wait_st();        // V fragments (and a rescaled O) are in tensor memory
    tc_fence_before();
    __syncwarp();
    if (lane == 0) {
      __threadfence_block();
      *reinterpret_cast<volatile int *>(&s_seq_sm[q]) = c + 1;   // the quarter's next slot may take its turn
    }
    if (lane == 0) mbar_arrive(bar_p + 8 * team);   // P and the V fragments of this warp are in place
    RD_TCT(9);   // softmax, P
    if (++d == D) {
      d = 0;
      ph ^= 1;
    }
  }
  }

  // ---- epilogue ----
  __syncthreads();   // both teams are out of their loops
  {
    // the last P V batch of either team has landed
    for (int t = 0; t < kTcTeams; ++t) {
      const int n_t = (n_slots - t + kTcTeams - 1) / kTcTeams;
      if (n_t > 0 && !*abort_flag && !mbar_wait(bar_pv + 8 * t, (n_t - 1) & 1, p.status, 34)) s_abort = 1;
    }
    tc_fence_after();
  }
  // softmax statistics of kv head q: the 16 key lanes of the warp, then the two teams
  float mfin[kGroup];
  if (warp < 8) {
#pragma unroll
  for (int h = 0; h < kGroup; ++h) {
    mfin[h] = *reinterpret_cast<volatile float *>(&s_mref[q][h]);
    float l = lane < 16 ? lsum[h] : 0.f;
    if (lane < 16 && lref[h] != mfin[h]) l *= ex2(lref[h] - mfin[h]);   // 0 stays 0
    float m = run[h];
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      l += __shfl_xor_sync(FULL, l, o);
      m = fmaxf(m, __shfl_xor_sync(FULL, m, o));
    }
    if (lane == 0) {
      s_red[team][q][h] = m;
      s_red[team][q][8 + h] = l;
    }
  }
  }
  __syncthreads();
  const bool aborted = s_abort != 0;
  if (aborted && threadIdx.x == 0) {
    // Unwinding after a bounded wait ran out: give copies still in flight one more bounded
    // chance to land before the CTA (and its shared memory) goes away.
    for (int i = 0; i < kTcTeams * D; ++i) {
      const uint32_t nf = lds32(nfill0 + 4 * i);
      const int cc = (int)lds32(sid0 + 4 * i);
      if (nf > 0 && cc >= 0) mbar_wait(bar_full + 8 * i, (nf - 1) & 1, nullptr, 0);
    }
  }
  __syncthreads();
  // O -> planes [head][dim] over the ring (dim d at 33 (d >> 5) + (d & 31), heads kPlaneHead
  // floats apart); team t moves slices 4 t .. 4 t + 3. Row L of quarter q in slice sl is dim
  // VL::dim(L & 7, 2 sl + (L >> 4), (L >> 3) & 1) of kv head q.
  float *plane = reinterpret_cast<float *>(smem + kTcRingOffset);
  if (n_slots > 0 && !aborted && warp < 8) {
#pragma unroll 1
    for (int k = 0; k < 4; ++k) {
      const int sl = 4 * team + k;
      uint32_t o[8];
      tmem_ld8(lane_addr + kTcColsO + 32 * sl + 8 * q, o);
      tmem_wait_ld();
      const int dim = VL::dim(lane & 7, 2 * sl + (lane >> 4), (lane >> 3) & 1);
      const int a = 33 * (dim >> 5) + (dim & 31);
#pragma unroll
      for (int h = 0; h < kGroup; ++h) plane[(q * kGroup + h) * kPlaneHead + a] = __uint_as_float(o[h]);
    }
  }
  tc_fence_before();
  __syncthreads();
  {
    const size_t head_stride = (size_t)S * kRec;
    const bool wide = (reinterpret_cast<uintptr_t>(rec0) & 7) == 0;
    for (int idx = threadIdx.x; idx < 4 * kGroup * (kHeadDim / 2); idx += kTcThreads) {
      const int hd = idx >> 7, dd = 2 * (idx & 127);
      const int qq = hd / kGroup, h = hd % kGroup;
      // record: m = the true maximum, l and acc brought from the lazy reference to it
      const float mt = fmaxf(s_red[0][qq][h], s_red[1][qq][h]);
      const float mrf = *reinterpret_cast<volatile float *>(&s_mref[qq][h]);
      const bool empty = aborted || n_slots == 0 || mt <= 0.5f * kNegBig;
      const float f = empty ? 0.f : ex2(mrf - mt);
      const int off = hd * kPlaneHead + 33 * (dd >> 5) + (dd & 31);
      const float a0 = empty ? 0.f : plane[off] * f * VL::kUnscale;
      const float a1 = empty ? 0.f : plane[off + 1] * f * VL::kUnscale;
      float *rec = rec0 + hd * head_stride;
      if (dd == 0) {
        rec[0] = empty ? -INFINITY : mt * 0.6931471805599453f;   // natural log
        rec[1] = empty ? 0.f : (s_red[0][qq][8 + h] + s_red[1][qq][8 + h]) * f;
      }
      if (wide) {
        *reinterpret_cast<float2 *>(rec + 2 + dd) = make_float2(a0, a1);
      } else {
        rec[2 + dd] = a0;
        rec[3 + dd] = a1;
      }
    }
  }
#ifdef RD_TIMING_SWITCHES
  if ((p.debug & 32) && threadIdx.x == 0) {   // overwrite the first record with this warp's clock sums
    unsigned *o = reinterpret_cast<unsigned *>(rec0 + 2);
    for (int i = 0; i < 10; ++i) o[i] = (unsigned)tw[i];
    o[10] = (unsigned)(clock64() - tloop0);
    o[11] = (unsigned)n_slots;
  }
#endif
  __syncthreads();
  if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512u) : "memory");
}

// Host side: launches the tensor-memory kernel for one token of one sequence.
template <int KT, int VT>
int launch_decode_tc(const DecodeKernelArgs &k0, int n_splits, cudaStream_t st) {
  DecodeKernelArgs k = k0;
  k.depth = tc_ring_depth(KT, VT);
  k.group_bytes = k.depth * slot_bytes(KT, VT, 4);
  const size_t smem = kTcRingOffset + (size_t)kTcTeams * k.group_bytes;
  static bool attr_set[8] = {false, false, false, false, false, false, false, false};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return RD_ERR_CUDA;
  if (dev < 0 || dev >= 8 || !attr_set[dev]) {
    if (cudaFuncSetAttribute(decode_tc_kernel<KT, VT>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBudget) !=
        cudaSuccess)
      return RD_ERR_CUDA;
    if (dev >= 0 && dev < 8) attr_set[dev] = true;
  }
  return launch_pdl(2, decode_tc_kernel<KT, VT>, dim3((unsigned)n_splits), dim3(kTcThreads), smem, st, k) ==
                 cudaSuccess
             ? RD_OK
             : RD_ERR_CUDA;
}

#undef RD_TCT

}  // namespace rd
