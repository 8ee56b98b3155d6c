// Context-sharded decode: the exchange of per-shard attention records fused into the
// merge kernels, over peer-mapped memory (NVLink stores), instead of a library
// all-gather between two merges. (The reference is single-GPU; the record format and
// the merge are attn_merge_kernel's, include/rdna4/attn.cuh:563-590.)
//
// Every rank owns an exchange buffer that all ranks can address:
//   header   epoch, arrival counter, flag[parity][source rank][head][dim quarter]
//   records  [parity][source rank][head][dim quarter][2 + 64] f32 (m, l, 64 acc values)
// One sharded attention call on rank r is two launches on r's stream:
//   1. the split-KV decode kernel over r's slice of the keys -> S records per head in
//      the caller's workspace (rd_decode.cuh);
//   2. shard_exchange_kernel<PUSH, MERGE>: CTA (head, quarter) reduces the S records to
//      one, STORES ITS QUARTER INTO EVERY RANK'S buffer and then the call's epoch into
//      that rank's flag (release, system scope); the same CTA then waits (bounded) until
//      the local flags of all ranks show this epoch and merges the `world` records into
//      its quarter of the output (optional fused sigmoid gate). The last CTA to finish
//      advances the local epoch.
// A CTA waits only after it has pushed, and only for pushes, so no rank can block
// another; a rank can run at most one call ahead of the slowest one (its next merge
// needs that rank's next push), which is why two parities of records and flags are
// enough. The epoch lives in device memory, not in a launch argument, so the same
// launches can be replayed from a CUDA graph. The two halves also exist as separate
// launches (PUSH only, MERGE only) for callers that compute the records themselves.
#include "rd_common.cuh"
#include "rd_internal.h"

namespace rd {

constexpr int kPushDims = 64;
constexpr int kPushGroups = 16;
constexpr int kQuarters = kHeadDim / kPushDims;

struct XHeader {
  uint32_t epoch;        // calls completed on this rank
  uint32_t merge_count;  // CTAs of the running merge that are done
  uint32_t pad_[62];
  // [parity][source rank][head * 4 + dim quarter]: the epoch whose record part has landed
  uint32_t flag[2][kShardMaxWorld][kShardMaxHeads * kQuarters];
};
static_assert(sizeof(XHeader) <= kShardHeaderBytes, "exchange header");

__device__ __forceinline__ float *xrecords(unsigned char *xbuf) {
  return reinterpret_cast<float *>(xbuf + kShardHeaderBytes);
}
// Polls use a relaxed system-scope load; one acquire fence after the last poll orders
// the record reads behind it (an acquire load per poll costs a fence per poll).
__device__ __forceinline__ uint32_t ld_relaxed_sys(const uint32_t *p) {
  uint32_t v;
  asm volatile("ld.relaxed.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void fence_acq_rel_sys() {
  asm volatile("fence.acq_rel.sys;" ::: "memory");
}
__device__ __forceinline__ unsigned long long global_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}

// grid (n_head, 4 dim quarters), 1024 threads = 16 record groups x 64 dims. CTA (head,
// quarter) handles that quarter of the head's record in both halves:
//   PUSH : this rank's n_in split records -> one record, stored into every rank's buffer,
//          then the epoch into every rank's flag for (this rank, head, quarter);
//   MERGE: wait (bounded) for all ranks' flags of (head, quarter), combine the `world`
//          records into the output quarter, count the CTA towards the epoch advance.
// A CTA never waits before it has pushed, so ranks cannot block one another.
template <bool PUSH, bool MERGE>
__global__ void __launch_bounds__(kPushDims *kPushGroups)
shard_exchange_kernel(const float *__restrict__ partial, int n_in, float *__restrict__ out,
                      float *__restrict__ gate, int n_head, ShardPeers g, DeviceStatus *status) {
  __shared__ float s_l[kPushGroups];
  __shared__ float s_acc[kPushGroups][kPushDims];
  __shared__ float s_mm;
  __shared__ int s_ok;

  const int row = blockIdx.x, quarter = blockIdx.y;
  const int tx = threadIdx.x % kPushDims, ty = threadIdx.x / kPushDims;
  const int d = quarter * kPushDims + tx;
  XHeader *me = reinterpret_cast<XHeader *>(g.x[g.rank]);
  const uint32_t epoch = *reinterpret_cast<volatile uint32_t *>(&me->epoch) + 1;
  const int par = epoch & 1;
  const int fidx = row * kQuarters + quarter;

  if (PUSH) {
    const float *base = partial + (size_t)row * n_in * kRec;
    float mx = -INFINITY;
    for (int s = threadIdx.x; s < n_in; s += blockDim.x) mx = fmaxf(mx, base[(size_t)s * kRec]);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    if ((threadIdx.x & 31) == 0) s_acc[0][threadIdx.x >> 5] = mx;
    __syncthreads();
    if (threadIdx.x == 0) {
      float m = -INFINITY;
      for (int i = 0; i < (int)(blockDim.x >> 5); ++i) m = fmaxf(m, s_acc[0][i]);
      s_mm = m;
    }
    __syncthreads();
    const float mm = s_mm;
    __syncthreads();

    float acc = 0.f, ll = 0.f;
    if (mm != -INFINITY) {
      for (int s = ty; s < n_in; s += kPushGroups) {
        const float *rec = base + (size_t)s * kRec;
        const float w = expf(rec[0] - mm);
        if (w > 0.f) {
          acc = fmaf(rec[2 + d], w, acc);
          if (tx == 0) ll = fmaf(rec[1], w, ll);
        }
      }
    }
    s_acc[ty][tx] = acc;
    if (tx == 0) s_l[ty] = ll;
    __syncthreads();
    if (ty == 0) {
      float a = 0.f, l = 0.f;
#pragma unroll
      for (int i = 0; i < kPushGroups; ++i) {
        a += s_acc[i][tx];
        l += s_l[i];
      }
      // every quarter carries its own copy of (m, l): slot layout [quarter][2 + 64]
      const size_t slot =
          ((((size_t)par * g.world + g.rank) * n_head + row) * kQuarters + quarter) * kXPart;
      for (int r = 0; r < g.world; ++r) {
        float *rec = xrecords(g.x[r]) + slot;
        rec[2 + tx] = a;
        if (tx == 0) {
          rec[0] = mm;
          rec[1] = l;
        }
      }
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      // The barrier above ordered the CTA's record stores before this thread; one
      // system-scope fence then covers all of them (release is cumulative), and the
      // flags can go out as plain system-scope stores behind it.
      __threadfence_system();
      for (int r = 0; r < g.world; ++r)
        asm volatile("st.relaxed.sys.global.u32 [%0], %1;" ::"l"(
                         &reinterpret_cast<XHeader *>(g.x[r])->flag[par][g.rank][fidx]),
                     "r"(epoch)
                     : "memory");
    }
  }

  if (MERGE) {
    if (threadIdx.x < 32) {
      bool ok = true;
      if ((int)threadIdx.x < g.world) {
        const uint32_t *f = &me->flag[par][threadIdx.x][fidx];
        const unsigned long long t0 = global_ns();
        unsigned polls = 0;
        while ((int32_t)(ld_relaxed_sys(f) - epoch) < 0) {
          // the clock is only consulted now and then: reading it costs as much as a poll
          if ((++polls & 63u) == 0 && global_ns() - t0 > g.wait_ns) {  // that rank never pushed
            ok = false;
            break;
          }
        }
        fence_acq_rel_sys();
      }
      ok = __all_sync(0xffffffffu, ok);
      if (threadIdx.x == 0) {
        s_ok = ok ? 1 : 0;
        if (!ok && status != nullptr && atomicExch(&status->timeout_flag, 1) == 0)
          status->where = 100 + g.rank;
      }
    }
    __syncthreads();
    if (ty == 0) {
      float o = 0.f;
      if (s_ok) {
        const float *recs = xrecords(g.x[g.rank]) +
                            (((size_t)par * g.world * n_head + row) * kQuarters + quarter) * kXPart;
        const size_t rstride = (size_t)n_head * kQuarters * kXPart;
        float mm = -INFINITY;
        for (int r = 0; r < g.world; ++r) mm = fmaxf(mm, __ldcg(recs + r * rstride));
        float a = 0.f, l = 0.f;
        if (mm != -INFINITY) {
          for (int r = 0; r < g.world; ++r) {
            const float *rec = recs + r * rstride;
            const float w = expf(__ldcg(rec) - mm);
            if (w > 0.f) {
              a = fmaf(__ldcg(rec + 2 + tx), w, a);
              l = fmaf(__ldcg(rec + 1), w, l);
            }
          }
        }
        o = (mm != -INFINITY && l > 0.f) ? a / l : 0.f;
      }
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
