// Device side of the context-sharded exchange that more than one kernel uses: the
// exchange-buffer header, the epoch-tagged 8-byte words, and the PUSH half (reduce this
// rank's split records of one (head, dim quarter) to one record part and store it into
// every rank's buffer). See rd_shard.cu for the protocol.
#pragma once
#include "rd_common.cuh"
#include "rd_internal.h"

namespace rd {

constexpr int kPushDims = 64;
constexpr int kQuarters = kHeadDim / kPushDims;

struct XHeader {
  uint32_t epoch;          // calls completed on this rank
  uint32_t merge_count;    // CTAs of the running merge that are done
  uint32_t push_count[2];  // by call parity: decode CTAs of a fused decode+push launch whose
                           // records are written (zeroed again by that call's merge)
};
static_assert(sizeof(XHeader) <= kShardHeaderBytes, "exchange header");

__device__ __forceinline__ uint2 *xwords(unsigned char *xbuf) {
  return reinterpret_cast<uint2 *>(xbuf + kShardHeaderBytes);
}
// One (value, epoch) word = one aligned 8-byte scalar access: single-copy atomic by the
// memory model, so a reader never pairs a fresh epoch with a stale value.
__device__ __forceinline__ void st_word_sys(uint2 *p, float v, uint32_t epoch) {
  const unsigned long long w = ((unsigned long long)epoch << 32) | (unsigned long long)__float_as_uint(v);
  asm volatile("st.relaxed.sys.global.b64 [%0], %1;" ::"l"(p), "l"(w) : "memory");
}
__device__ __forceinline__ uint2 ld_word_sys(const uint2 *p) {
  unsigned long long w;
  asm volatile("ld.relaxed.sys.global.b64 %0, [%1];" : "=l"(w) : "l"(p) : "memory");
  return make_uint2((uint32_t)w, (uint32_t)(w >> 32));
}

// PUSH of one (head row, dim quarter) by NG groups of 64 threads (thread = (group ty, dim
// tx)): group ty walks records ty, ty + NG, ... with four loads in flight and a local
// log-sum-exp, the groups meet in shared memory (s_acc [NG][64], s_l / s_gm [NG]), and the
// first group stores the part [m, l, 64 values] into every rank's buffer as (value, epoch)
// words. `partial` holds this rank's records [n_head][n_in][258]. All NG * 64 threads must
// call it (it synchronises them with the given named barrier).
template <int NG>
__device__ __forceinline__ void shard_push_part(const float *partial, int n_in, int n_head, int row,
                                                int quarter, int tx, int ty, const ShardPeers &g,
                                                uint32_t epoch, float (*s_acc)[kPushDims], float *s_l,
                                                float *s_gm, int bar_id) {
  const int d = quarter * kPushDims + tx;
  const int par = epoch & 1;
  const size_t rstride = (size_t)n_head * kQuarters * kXPart;
  const size_t part0 = (size_t)par * g.world * rstride + ((size_t)row * kQuarters + quarter) * kXPart;
  const float *base = partial + (size_t)row * n_in * kRec;
  float mloc = -INFINITY, acc = 0.f, ll = 0.f;
  for (int s0 = ty; s0 < n_in; s0 += 4 * NG) {
    float m4[4], a4[4], l4[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const int sidx = s0 + k * NG;
      m4[k] = -INFINITY;
      a4[k] = l4[k] = 0.f;
      if (sidx < n_in) {
        const float *rec = base + (size_t)sidx * kRec;
        m4[k] = __ldcg(rec);
        a4[k] = __ldcg(rec + 2 + d);
        if (tx == 0) l4[k] = __ldcg(rec + 1);
      }
    }
    const float mb = fmaxf(fmaxf(mloc, fmaxf(m4[0], m4[1])), fmaxf(m4[2], m4[3]));
    if (mb != -INFINITY) {
      const float f = expf(mloc - mb);
      acc *= f;
      ll *= f;
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        if (m4[k] != -INFINITY) {
          const float w = expf(m4[k] - mb);
          acc = fmaf(a4[k], w, acc);
          ll = fmaf(l4[k], w, ll);
        }
      }
      mloc = mb;
    }
  }
  s_acc[ty][tx] = acc;
  if (tx == 0) {
    s_l[ty] = ll;
    s_gm[ty] = mloc;
  }
  asm volatile("bar.sync %0, %1;" ::"r"(bar_id), "r"(NG * kPushDims) : "memory");
  if (ty == 0) {
    float mm = -INFINITY;
#pragma unroll
    for (int i = 0; i < NG; ++i) mm = fmaxf(mm, s_gm[i]);
    float a = 0.f, l = 0.f;
#pragma unroll
    for (int i = 0; i < NG; ++i) {
      if (s_gm[i] != -INFINITY) {
        const float w = expf(s_gm[i] - mm);
        a = fmaf(s_acc[i][tx], w, a);
        l = fmaf(s_l[i], w, l);
      }
    }
    // every quarter carries its own copy of (m, l): part layout [m, l, 64 values]
    const size_t mine = part0 + (size_t)g.rank * rstride;
    for (int r = 0; r < g.world; ++r) {
      uint2 *rec = xwords(g.x[r]) + mine;
      st_word_sys(rec + 2 + tx, a, epoch);
      if (tx == 0) {
        st_word_sys(rec, mm, epoch);
        st_word_sys(rec + 1, l, epoch);
      }
    }
  }
  asm volatile("bar.sync %0, %1;" ::"r"(bar_id), "r"(NG * kPushDims) : "memory");   // the arrays may be reused
}

// MERGE of one (head row, dim quarter) by 64 threads (tx = dim of the quarter; whole warps):
// waits (bounded) for every rank's part of this call in the LOCAL buffer, combines them and
// writes the output quarter, with the optional fused sigmoid gate (sigmoid stored back).
__device__ __forceinline__ void shard_merge_part(float *out, float *gate, int n_head, int row, int quarter,
                                                 int tx, const ShardPeers &g, uint32_t epoch,
                                                 DeviceStatus *status) {
  const int d = quarter * kPushDims + tx;
  const int par = epoch & 1;
  // word index of part (parity, source rank r, head row, quarter): + r * rstride
  const size_t rstride = (size_t)n_head * kQuarters * kXPart;
  const size_t part0 = (size_t)par * g.world * rstride + ((size_t)row * kQuarters + quarter) * kXPart;
  const uint2 *recs = xwords(g.x[g.rank]) + part0;
  // the gate value does not depend on the exchange: requested before the waits
  float *gp = gate != nullptr ? gate + (size_t)row * kHeadDim + d : nullptr;
  const float gv = gp != nullptr ? *gp : 0.f;
  bool ok = true;
  float m_r[kShardMaxWorld], l_r[kShardMaxWorld], a_r[kShardMaxWorld];
  // Every round requests all 3 * world words back to back (one round trip to L2 for the
  // lot, not one per word) and repeats until each carries this call's epoch, or the time
  // limit passes (the clock is read every 64 rounds: it costs as much as a round).
#pragma unroll
  for (int r = 0; r < kShardMaxWorld; ++r) {
    m_r[r] = -INFINITY;
    l_r[r] = a_r[r] = 0.f;
  }
  unsigned long long t0 = 0;
  unsigned polls = 0;
  for (;;) {
    uint2 w_m[kShardMaxWorld], w_l[kShardMaxWorld], w_a[kShardMaxWorld];
#pragma unroll
    for (int r = 0; r < kShardMaxWorld; ++r) {
      if (r < g.world) {
        const uint2 *rec = recs + r * rstride;
        w_m[r] = ld_word_sys(rec);
        w_l[r] = ld_word_sys(rec + 1);
        w_a[r] = ld_word_sys(rec + 2 + tx);
      }
    }
    bool all = true;
#pragma unroll
    for (int r = 0; r < kShardMaxWorld; ++r) {
      if (r < g.world) {
        all = all && w_m[r].y == epoch && w_l[r].y == epoch && w_a[r].y == epoch;
        m_r[r] = __uint_as_float(w_m[r].x);
        l_r[r] = __uint_as_float(w_l[r].x);
        a_r[r] = __uint_as_float(w_a[r].x);
      }
    }
    if (all) break;
    if ((++polls & 63u) == 0) {
      if (t0 == 0) t0 = global_ns();
      else if (global_ns() - t0 > g.wait_ns) {
        ok = false;
        break;
      }
    }
  }
  ok = __all_sync(0xffffffffu, ok);
  if (!ok && tx == 0 && status != nullptr && atomicExch(&status->timeout_flag, 1) == 0)
    status->where = 100 + g.rank;   // some rank never pushed: zeros, reported
  float mm = -INFINITY;
#pragma unroll
  for (int r = 0; r < kShardMaxWorld; ++r) mm = fmaxf(mm, m_r[r]);
  float a = 0.f, l = 0.f;
  if (mm != -INFINITY) {
#pragma unroll
    for (int r = 0; r < kShardMaxWorld; ++r) {
      const float w = expf(m_r[r] - mm);   // 0 for an empty part (m = -inf)
      if (w > 0.f) {
        a = fmaf(a_r[r], w, a);
        l = fmaf(l_r[r], w, l);
      }
    }
  }
  float o = (ok && mm != -INFINITY && l > 0.f) ? a / l : 0.f;
  if (gp != nullptr) {
    const float sg = __fdiv_rn(1.0f, 1.0f + expf(-gv));
    *gp = sg;
    o *= sg;
  }
  out[(size_t)row * kHeadDim + d] = o;
}

// PUSH of one (head row, dim quarter) inside another kernel's epilogue, shaped for latency:
// NT threads = NT / 16 groups of 16, thread (group ty, tx) owns dims 4 tx .. 4 tx + 3 of the
// quarter and its group's records ty, ty + NG, ... -- all of them requested before the
// first is used, so the walk over a launch's ~150 records is ONE round trip to L2. Scratch:
// s_acc [NG][64] floats, s_l [NG], s_gm [NG]. All NT threads call it.
// xv != nullptr folds one more key in as a record of its own (m = x_score in natural-log
// units, l = 1, acc = the key's stored V row xv of type xvt): the newest position's row,
// which the same launch has just stored and none of its CTAs attended.
template <int NT>
__device__ __forceinline__ void shard_push_part_wide(const float *partial, int n_in, int n_head, int row,
                                                     int quarter, const ShardPeers &g, uint32_t epoch,
                                                     float *s_acc, float *s_l, float *s_gm, int bar_id,
                                                     float x_prod = 0.f, float x_scale = 0.f,
                                                     const uint8_t *xv = nullptr, int xvt = 0) {
  constexpr int NG = NT / 16;
  constexpr int kBatch = 8;
  // The extra key's score = x_scale * (sum of every thread's x_prod): the caller has
  // requested the products' operands just before this call, so their round trip runs with
  // the one of the records; the warps' sums meet in s_xp (behind s_gm) at the barrier below.
  float *s_xp = s_gm + NG;
  // the extra key's value, requested with the records instead of after their reduction
  float x_val = 0.f;
  if (xv != nullptr && threadIdx.x < kPushDims) x_val = load_cache_value(xv, xvt, quarter * kPushDims + threadIdx.x);
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
  const float *base = partial + (size_t)row * n_in * kRec;
  float mloc = -INFINITY, ll = 0.f;
  float acc[4] = {0.f, 0.f, 0.f, 0.f};
  for (int s0 = ty; s0 < n_in; s0 += kBatch * NG) {
    float m8[kBatch], l8[kBatch];
    float2 lo[kBatch], hi[kBatch];
#pragma unroll
    for (int k = 0; k < kBatch; ++k) {
      const int sidx = s0 + k * NG;
      m8[k] = -INFINITY;
      l8[k] = 0.f;
      lo[k] = hi[k] = make_float2(0.f, 0.f);
      if (sidx < n_in) {
        const float *rec = base + (size_t)sidx * kRec;
        m8[k] = __ldcg(rec);
        l8[k] = __ldcg(rec + 1);
        // a record starts 8 bytes into a 16-byte line (258 floats per record): two 8-byte loads
        const float2 *a2 = reinterpret_cast<const float2 *>(rec + 2 + quarter * kPushDims + 4 * tx);
        lo[k] = __ldcg(a2);
        hi[k] = __ldcg(a2 + 1);
      }
    }
    float mb = mloc;
#pragma unroll
    for (int k = 0; k < kBatch; ++k) mb = fmaxf(mb, m8[k]);
    if (mb != -INFINITY) {
      const float f = expf(mloc - mb);
      ll *= f;
#pragma unroll
      for (int j = 0; j < 4; ++j) acc[j] *= f;
#pragma unroll
      for (int k = 0; k < kBatch; ++k) {
        if (m8[k] != -INFINITY) {
          const float w = expf(m8[k] - mb);
          ll = fmaf(l8[k], w, ll);
          acc[0] = fmaf(lo[k].x, w, acc[0]);
          acc[1] = fmaf(lo[k].y, w, acc[1]);
          acc[2] = fmaf(hi[k].x, w, acc[2]);
          acc[3] = fmaf(hi[k].y, w, acc[3]);
        }
      }
      mloc = mb;
    }
  }
#pragma unroll
  for (int j = 0; j < 4; ++j) s_acc[ty * kPushDims + 4 * tx + j] = acc[j];
  if (tx == 0) {
    s_l[ty] = ll;
    s_gm[ty] = mloc;
  }
  if (xv != nullptr) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) x_prod += __shfl_xor_sync(0xffffffffu, x_prod, o);
    if ((threadIdx.x & 31) == 0) s_xp[threadIdx.x >> 5] = x_prod;
  }
  asm volatile("bar.sync %0, %1;" ::"r"(bar_id), "r"(NT) : "memory");
  if (threadIdx.x < kPushDims) {
    const int dx = threadIdx.x;
    float mm = -INFINITY;
    for (int i = 0; i < NG; ++i) mm = fmaxf(mm, s_gm[i]);
    float a = 0.f, l = 0.f;
    for (int i = 0; i < NG; ++i) {
      if (s_gm[i] != -INFINITY) {
        const float w = expf(s_gm[i] - mm);
        a = fmaf(s_acc[i * kPushDims + dx], w, a);
        l = fmaf(s_l[i], w, l);
      }
    }
    if (xv != nullptr) {
      float x_score = 0.f;
      for (int i = 0; i < NT / 32; ++i) x_score += s_xp[i];
      x_score *= x_scale;
      const float mx = fmaxf(mm, x_score);
      const float f = mm == -INFINITY ? 0.f : expf(mm - mx), w = expf(x_score - mx);
      a = fmaf(x_val, w, a * f);
      l = fmaf(l, f, w);
      mm = mx;
    }
    const int par = epoch & 1;
    const size_t rstride = (size_t)n_head * kQuarters * kXPart;
    const size_t mine = (size_t)par * g.world * rstride + ((size_t)row * kQuarters + quarter) * kXPart +
                        (size_t)g.rank * rstride;
    for (int r = 0; r < g.world; ++r) {
      uint2 *rec = xwords(g.x[r]) + mine;
      st_word_sys(rec + 2 + dx, a, epoch);
      if (dx == 0) {
        st_word_sys(rec, mm, epoch);
        st_word_sys(rec + 1, l, epoch);
      }
    }
  }
  asm volatile("bar.sync %0, %1;" ::"r"(bar_id), "r"(NT) : "memory");   // the scratch may be reused
}

}  // namespace rd
