// Context-sharded decode: the exchange of per-shard attention records fused into the
// merge kernels, over peer-mapped memory (NVLink stores), instead of a library
// all-gather between two merges. (The reference is single-GPU; the record format and
// the merge are attn_merge_kernel's, include/rdna4/attn.cuh:563-590.)
//
// Every rank owns an exchange buffer that all ranks can address:
//   header   epoch, arrival counters, flag[parity][source rank]
//   records  [parity][source rank][head][258] f32
// One sharded attention call on rank r is three launches on r's stream:
//   1. the split-KV decode kernel over r's slice of the keys -> S records per head in
//      the caller's workspace (rd_decode.cuh);
//   2. shard_push_kernel: S records -> one record per head, STORED INTO EVERY RANK'S
//      buffer at [parity][r][head]; the last CTA then writes the call's epoch into
//      flag[parity][r] of every rank (release, system scope);
//   3. shard_merge_kernel: waits (bounded) until the local flags of all ranks show this
//      epoch, merges the `world` records per head into the output (optional fused
//      sigmoid gate), and its last CTA advances the local epoch.
// Kernel 3 of a rank only waits for kernels 2 of the other ranks, which never wait for
// anything, so no rank can block another; a rank can run at most one call ahead of the
// slowest one (its next merge needs that rank's next push), which is why two parities
// of records and flags are enough. The epoch lives in device memory, not in a launch
// argument, so the same three launches can be replayed from a CUDA graph.
#include "rd_common.cuh"
#include "rd_internal.h"

namespace rd {

constexpr int kPushDims = 64;
constexpr int kPushGroups = 16;

struct XHeader {
  uint32_t epoch;        // calls completed on this rank
  uint32_t push_count;   // CTAs of the running push kernel that have stored their part
  uint32_t merge_count;  // CTAs of the running merge kernel that are done
  uint32_t pad_[61];
  uint32_t flag[2][kShardMaxWorld][8];  // [parity][source rank], 32 bytes apart
};
static_assert(sizeof(XHeader) <= kShardHeaderBytes, "exchange header");

__device__ __forceinline__ float *xrecords(unsigned char *xbuf) {
  return reinterpret_cast<float *>(xbuf + kShardHeaderBytes);
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t *p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_sys(uint32_t *p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned long long global_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}

// grid (n_head, 4 dim quarters), 1024 threads: 16 record groups x 64 dims.
__global__ void __launch_bounds__(kPushDims *kPushGroups)
shard_push_kernel(const float *__restrict__ partial, int n_in, int n_head, ShardPeers g) {
  __shared__ float s_l[kPushGroups];
  __shared__ float s_acc[kPushGroups][kPushDims];
  __shared__ float s_mm;

  const int row = blockIdx.x, quarter = blockIdx.y;
  const int tx = threadIdx.x % kPushDims, ty = threadIdx.x / kPushDims;
  const float *base = partial + (size_t)row * n_in * kRec;
  XHeader *me = reinterpret_cast<XHeader *>(g.x[g.rank]);
  const uint32_t epoch = *reinterpret_cast<volatile uint32_t *>(&me->epoch) + 1;
  const int par = epoch & 1;

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
        acc = fmaf(rec[2 + quarter * kPushDims + tx], w, acc);
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
    const int d = quarter * kPushDims + tx;
    const size_t slot = (((size_t)par * g.world + g.rank) * n_head + row) * kRec;
    for (int r = 0; r < g.world; ++r) {
      float *rec = xrecords(g.x[r]) + slot;
      rec[2 + d] = a;
      if (d == 0) {
        rec[0] = mm;
        rec[1] = l;
      }
    }
    __threadfence_system();  // this thread's stores are ordered before the arrival below
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    const uint32_t prev = atomicAdd(&me->push_count, 1u);
    if (prev == gridDim.x * gridDim.y - 1) {
      // every CTA has stored and fenced: publish the epoch to all ranks
      me->push_count = 0;
      __threadfence_system();
      for (int r = 0; r < g.world; ++r)
        st_release_sys(&reinterpret_cast<XHeader *>(g.x[r])->flag[par][g.rank][0], epoch);
    }
  }
}

// grid (n_head), 256 threads: one output dim per thread, `world` records per head.
__global__ void __launch_bounds__(kHeadDim)
shard_merge_kernel(float *__restrict__ out, float *__restrict__ gate, int n_head, ShardPeers g,
                   DeviceStatus *status) {
  __shared__ int s_ok;
  XHeader *me = reinterpret_cast<XHeader *>(g.x[g.rank]);
  const uint32_t epoch = *reinterpret_cast<volatile uint32_t *>(&me->epoch) + 1;
  const int par = epoch & 1;
  if (threadIdx.x < 32) {
    bool ok = true;
    if ((int)threadIdx.x < g.world) {
      const uint32_t *f = &me->flag[par][threadIdx.x][0];
      const unsigned long long t0 = global_ns();
      while ((int32_t)(ld_acquire_sys(f) - epoch) < 0) {
        if (global_ns() - t0 > g.wait_ns) {  // the rank never pushed: give up, report
          ok = false;
          break;
        }
        __nanosleep(100);
      }
    }
    ok = __all_sync(0xffffffffu, ok);
    if (threadIdx.x == 0) {
      s_ok = ok ? 1 : 0;
      if (!ok && status != nullptr && atomicExch(&status->timeout_flag, 1) == 0)
        status->where = 100 + g.rank;
    }
  }
  __syncthreads();
  const int row = blockIdx.x, d = threadIdx.x;
  float o = 0.f;
  if (s_ok) {
    const float *recs = xrecords(g.x[g.rank]) + (size_t)par * g.world * n_head * kRec;
    float mm = -INFINITY;
    for (int r = 0; r < g.world; ++r)
      mm = fmaxf(mm, __ldcg(recs + ((size_t)r * n_head + row) * kRec));
    float a = 0.f, l = 0.f;
    if (mm != -INFINITY) {
      for (int r = 0; r < g.world; ++r) {
        const float *rec = recs + ((size_t)r * n_head + row) * kRec;
        const float w = expf(__ldcg(rec) - mm);
        if (w > 0.f) {
          a = fmaf(__ldcg(rec + 2 + d), w, a);
          l = fmaf(__ldcg(rec + 1), w, l);
        }
      }
    }
    o = (mm != -INFINITY && l > 0.f) ? a / l : 0.f;
  }
  float *op = out + (size_t)row * kHeadDim + d;
  if (gate != nullptr) {
    float *gp = gate + (size_t)row * kHeadDim + d;
    const float sg = __fdiv_rn(1.0f, 1.0f + expf(-*gp));
    *gp = sg;
    o *= sg;
  }
  *op = o;
  __syncthreads();
  if (threadIdx.x == 0) {
    const uint32_t prev = atomicAdd(&me->merge_count, 1u);
    if (prev == gridDim.x - 1) {
      me->merge_count = 0;
      me->epoch = epoch;  // every CTA read the old value before it arrived here
    }
  }
}

int launch_shard_push(const float *partial, int n_in, int n_head, const ShardPeers &g,
                      cudaStream_t st) {
  const dim3 grid((unsigned)n_head, kHeadDim / kPushDims);
  shard_push_kernel<<<grid, kPushDims * kPushGroups, 0, st>>>(partial, n_in, n_head, g);
  return cudaGetLastError() == cudaSuccess ? RD_OK : RD_ERR_CUDA;
}

int launch_shard_merge(float *out, float *gate, int n_head, const ShardPeers &g,
                       DeviceStatus *status, cudaStream_t st) {
  shard_merge_kernel<<<(unsigned)n_head, kHeadDim, 0, st>>>(out, gate, n_head, g, status);
  return cudaGetLastError() == cudaSuccess ? RD_OK : RD_ERR_CUDA;
}

}  // namespace rd
