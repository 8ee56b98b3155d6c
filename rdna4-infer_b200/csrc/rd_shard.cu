// Context-sharded decode: the exchange of per-shard attention records fused into the
// merge kernels, over peer-mapped memory (NVLink stores), instead of a library
// all-gather between two merges. (The reference is single-GPU; the record format and
// the merge are attn_merge_kernel's, include/rdna4/attn.cuh:563-590.)
//
// Every rank owns an exchange buffer that all ranks can address:
//   header   epoch, arrival counter
//   records  [parity][source rank][head][dim quarter][2 + 64] 8-byte words, each word =
//            (f32 value, epoch it belongs to): m, l and 64 accumulator values
// One sharded attention call on rank r is ONE launch on r's stream (rd_attn_decode_sharded):
// the split-KV decode kernel over r's slice of the keys writes S records per head into the
// caller's workspace (rd_decode.cuh); every CTA then reports in, and the launch's first
// n_head * 4 CTAs take one (head, dim quarter) each: wait (bounded) for all CTAs, reduce the
// S records to one part, STORE IT INTO EVERY RANK'S buffer, every value as one 8-byte
// (value, epoch) store, then read the `world` parts from their own buffer, each thread
// spinning (bounded) on its own words until they carry this call's epoch, and merge them
// into the output quarter (optional fused sigmoid gate). The last of them advances the local
// epoch. The same two halves exist as the kernel below for callers that compute the
// records themselves: shard_exchange_kernel<PUSH, MERGE>, grid (head, quarter).
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
#include "rd_shard.cuh"

namespace rd {

constexpr int kPushGroups = 16;

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
  XHeader *me = reinterpret_cast<XHeader *>(g.x[g.rank]);
  const uint32_t epoch = *reinterpret_cast<volatile uint32_t *>(&me->epoch) + 1;
  const int par = epoch & 1;
  if (PUSH)
    shard_push_part<kPushGroups>(partial, n_in, n_head, row, quarter, tx, ty, g, epoch, s_acc, s_l, s_gm, 1);

  if (MERGE) {
    if (ty == 0) shard_merge_part(out, gate, n_head, row, quarter, tx, g, epoch, status);
    __syncthreads();
    if (threadIdx.x == 0) {
      const uint32_t prev = atomicAdd(&me->merge_count, 1u);
      if (prev == gridDim.x * gridDim.y - 1) {
        me->merge_count = 0;
        me->push_count[par] = 0;  // arrival counter of a fused decode + push launch of this call
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
