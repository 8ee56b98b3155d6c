// Context-sharded decode: the exchange of per-shard attention records fused into the
// merge kernels, over peer-mapped memory (NVLink stores), instead of a library
// all-gather between two merges. (The reference is single-GPU; the record format and
// the merge are attn_merge_kernel's, include/rdna4/attn.cuh:563-590.)
//
// Every rank owns an exchange buffer that all ranks can address:
//   header   epoch, arrival counter
//   records  [parity][source rank][head][dim quarter][2 + 64] 8-byte words, each word =
//            (f32 value, epoch it belongs to): m, l and 64 accumulator values
// One sharded attention call on rank r is two launches on r's stream:
//   1. the split-KV decode kernel over r's slice of the keys -> S records per head in
//      the caller's workspace (rd_decode.cuh);
//   2. shard_exchange_kernel<PUSH, MERGE>: CTA (head, quarter) reduces the S records to
//      one and STORES ITS QUARTER INTO EVERY RANK'S buffer, every value as one 8-byte
//      (value, epoch) store; the same CTA then reads the `world` parts from its own
//      buffer, each thread spinning (bounded) on its own words until they carry this
//      call's epoch, and merges them into its quarter of the output (optional fused
//      sigmoid gate). The last CTA to finish advances the local epoch.
// Tagging every word with the epoch (the low-latency protocol of collective libraries)
// needs no flag, no fence and no barrier between data and flag: an 8-byte store arrives
// whole, so a word that shows the epoch IS the value. Measured on two B200s, a system
// fence plus separate flags cost 5-7 us per call more.
// A CTA waits only after it has pushed, and only for pushes, so no rank can block
// another; a rank can run at most one call ahead of the slowest one (its next merge
// needs that rank's next push), which is why two parities of records are enough. The
// epoch lives in device memory, not in a launch argument, so the same launches can be
// replayed from a CUDA graph. The two halves also exist as separate launches (PUSH only,
// MERGE only) for callers that compute the records themselves.
#include "rd_common.cuh"
#include "rd_internal.h"

namespace rd {

constexpr int kPushDims = 64;
constexpr int kPushGroups = 16;
constexpr int kQuarters = kHeadDim / kPushDims;

struct XHeader {
  uint32_t epoch;        // calls completed on this rank
  uint32_t merge_count;  // CTAs of the running merge that are done
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
__device__ __forceinline__ unsigned long long global_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}
// Spins until the word carries `epoch`; false when wait_ns ran out first. The clock is
// only consulted every 64 polls: reading it costs as much as a poll.
__device__ __forceinline__ bool wait_word(const uint2 *p, uint32_t epoch, unsigned long long wait_ns,
                                          float &value) {
  uint2 w = ld_word_sys(p);
  if (w.y != epoch) {
    const unsigned long long t0 = global_ns();
    unsigned polls = 0;
    do {
      if ((++polls & 63u) == 0 && global_ns() - t0 > wait_ns) return false;
      w = ld_word_sys(p);
    } while (w.y != epoch);
  }
  value = __uint_as_float(w.x);
  return true;
}

// grid (n_head, 4 dim quarters), 1024 threads = 16 record groups x 64 dims. CTA (head,
// quarter) handles that quarter of the head's record in both halves:
//   PUSH : this rank's n_in split records -> one record part, stored into every rank's
//          buffer as (value, epoch) words;
//   MERGE: every thread of the first two warps waits (bounded) for its words of all
//          ranks' parts, combines them into the output quarter, and the CTA counts
//          towards the epoch advance.
// A CTA never waits before it has pushed, so ranks cannot block one another.
template <bool PUSH, bool MERGE>
__global__ void __launch_bounds__(kPushDims *kPushGroups)
shard_exchange_kernel(const float *__restrict__ partial, int n_in, float *__restrict__ out,
                      float *__restrict__ gate, int n_head, ShardPeers g, DeviceStatus *status) {
  __shared__ float s_l[kPushGroups];
  __shared__ float s_gm[kPushGroups];
  __shared__ float s_acc[kPushGroups][kPushDims];

  const int row = blockIdx.x, quarter = blockIdx.y;
  const int tx = threadIdx.x % kPushDims, ty = threadIdx.x / kPushDims;
  const int d = quarter * kPushDims + tx;
  XHeader *me = reinterpret_cast<XHeader *>(g.x[g.rank]);
  const uint32_t epoch = *reinterpret_cast<volatile uint32_t *>(&me->epoch) + 1;
  const int par = epoch & 1;
  // word index of part (parity, source rank r, head row, quarter): + r * rstride
  const size_t rstride = (size_t)n_head * kQuarters * kXPart;
  const size_t part0 = (size_t)par * g.world * rstride + ((size_t)row * kQuarters + quarter) * kXPart;

  if (PUSH) {
    // one pass, as in merge_kernel: group ty walks records ty, ty+16, ... with four loads
    // in flight and a local log-sum-exp; the 16 groups meet in shared memory
    const float *base = partial + (size_t)row * n_in * kRec;
    float mloc = -INFINITY, acc = 0.f, ll = 0.f;
    for (int s0 = ty; s0 < n_in; s0 += 4 * kPushGroups) {
      float m4[4], a4[4], l4[4];
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const int sidx = s0 + k * kPushGroups;
        m4[k] = -INFINITY;
        a4[k] = l4[k] = 0.f;
        if (sidx < n_in) {
          const float *rec = base + (size_t)sidx * kRec;
          m4[k] = rec[0];
          a4[k] = rec[2 + d];
          if (tx == 0) l4[k] = rec[1];
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
    __syncthreads();
    if (ty == 0) {
      float mm = -INFINITY;
#pragma unroll
      for (int i = 0; i < kPushGroups; ++i) mm = fmaxf(mm, s_gm[i]);
      float a = 0.f, l = 0.f;
#pragma unroll
      for (int i = 0; i < kPushGroups; ++i) {
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
  }

  if (MERGE) {
    if (ty == 0) {
      const uint2 *recs = xwords(g.x[g.rank]) + part0;
      bool ok = true;
      float m_r[kShardMaxWorld], l_r[kShardMaxWorld], a_r[kShardMaxWorld];
#pragma unroll
      for (int r = 0; r < kShardMaxWorld; ++r) {
        m_r[r] = -INFINITY;
        l_r[r] = a_r[r] = 0.f;
        if (r < g.world && ok) {
          const uint2 *rec = recs + r * rstride;
          ok = wait_word(rec, epoch, g.wait_ns, m_r[r]) && wait_word(rec + 1, epoch, g.wait_ns, l_r[r]) &&
               wait_word(rec + 2 + tx, epoch, g.wait_ns, a_r[r]);
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
      if (gate != nullptr) {
        float *gp = gate + (size_t)row * kHeadDim + d;
        const float sg = __fdiv_rn(1.0f, 1.0f + expf(-*gp));
        *gp = sg;
        o *= sg;
      }
      out[(size_t)row * kHeadDim + d] = o;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      const uint32_t prev = atomicAdd(&me->merge_count, 1u);
      if (prev == gridDim.x * gridDim.y - 1) {
        me->merge_count = 0;
        me->epoch = epoch;  // every CTA read the old value before it arrived here
      }
    }
  }
}

int launch_shard_push(const float *partial, int n_in, int n_head, const ShardPeers &g,
                      cudaStream_t st) {
  const dim3 grid((unsigned)n_head, kQuarters);
  shard_exchange_kernel<true, false>
      <<<grid, kPushDims * kPushGroups, 0, st>>>(partial, n_in, nullptr, nullptr, n_head, g, nullptr);
  return cudaGetLastError() == cudaSuccess ? RD_OK : RD_ERR_CUDA;
}

int launch_shard_merge(float *out, float *gate, int n_head, const ShardPeers &g,
                       DeviceStatus *status, cudaStream_t st) {
  const dim3 grid((unsigned)n_head, kQuarters);
  shard_exchange_kernel<false, true>
      <<<grid, kPushDims * kPushGroups, 0, st>>>(nullptr, 0, out, gate, n_head, g, status);
  return cudaGetLastError() == cudaSuccess ? RD_OK : RD_ERR_CUDA;
}

int launch_shard_exchange(const float *partial, int n_in, float *out, float *gate, int n_head,
                          const ShardPeers &g, DeviceStatus *status, cudaStream_t st) {
  const dim3 grid((unsigned)n_head, kQuarters);
  shard_exchange_kernel<true, true>
      <<<grid, kPushDims * kPushGroups, 0, st>>>(partial, n_in, out, gate, n_head, g, status);
  return cudaGetLastError() == cudaSuccess ? RD_OK : RD_ERR_CUDA;
}

}  // namespace rd
