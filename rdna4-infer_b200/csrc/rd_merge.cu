// Log-sum-exp merge of split-KV partial records (replaces attn_merge_kernel and
// attn_merge_batch_kernel, include/rdna4/attn.cuh:563-590,795-827).
//
//   mm = max_s m_s;  out = sum_s acc_s * e^(m_s - mm) / sum_s l_s * e^(m_s - mm)
//
// A row whose records are all empty (m = -inf) gives zeros, never NaN. The reference
// runs one 32-lane warp per head over at most 16 records; here a head can have one
// record per SM, so a CTA owns (row, 64-dim quarter) and spreads the records over 16
// thread groups: 4 * n_rows CTAs of 1024 threads keep the read of the partial buffer
// wide enough to stay off the critical path of a ~25 us decode step.
#include "rd_common.cuh"
#include "rd_internal.h"

namespace rd {

constexpr int kMergeDims = 64;    // dims per CTA
constexpr int kMergeGroups = 16;  // record groups per CTA

// MODE 0: normalised output (optionally gated). MODE 1: un-normalised record out.
// MODE 3: like 0, plus one more key -- the newest position's row, still only in the cache
// -- attended here as one more record (m = scale * q.k, l = 1, acc = v).
// MODE 2: like 0, but row = (sequence, token, head) and the record block, split count,
// output and gate come from the sequence's descriptor (rows_per_seq = q_len * n_head).
template <int MODE>
__global__ void __launch_bounds__(kMergeDims *kMergeGroups, MODE == 2 ? 2 : 1)
merge_kernel(const float *__restrict__ partial, float *__restrict__ out, int n_in, int n_out,
             float *__restrict__ gate, const DecodeSeq *__restrict__ seqs, int rows_per_seq,
             const ExtraKey xk) {
  __shared__ float s_l[kMergeGroups];
  __shared__ float s_gm[kMergeGroups];
  __shared__ float s_acc[kMergeGroups][kMergeDims];
  pdl_launch_dependents();
  pdl_wait();

  const int row = blockIdx.x;
  const int quarter = blockIdx.y;
  const int j = MODE == 1 ? blockIdx.z : 0;  // output record index
  const int tx = threadIdx.x % kMergeDims, ty = threadIdx.x / kMergeDims;
  const int lo = MODE == 1 ? (int)(((int64_t)n_in * j) / n_out) : 0;
  int hi = MODE == 1 ? (int)(((int64_t)n_in * (j + 1)) / n_out) : n_in;
  const float *base = partial + (size_t)row * n_in * kRec;
  int out_row = row;
  if (MODE == 2) {
    const DecodeSeq &d = seqs[row / rows_per_seq];
    out_row = row % rows_per_seq;
    n_in = d.n_splits;
    base = partial + ((size_t)d.rec_base + (size_t)out_row * n_in) * kRec;
    out = d.out;
    gate = d.gate;
    hi = n_in;
  }

  // One pass: group ty walks records lo+ty, lo+ty+16, ... and keeps a local log-sum-exp
  // (m, l, acc); the 16 groups are then combined through shared memory. An empty record
  // (m = -inf) weighs nothing and whatever its body holds is never used. A batch is ten
  // records per group -- the 148 records of a full-GPU decode in ONE round trip to L2 (four
  // per batch took three) -- and the first batch is requested before anything else, the
  // gate value with it.
  // (the many-sequence launch has thousands of CTAs with a handful of records each: there
  // a small batch keeps the registers low enough for two CTAs per SM)
  constexpr int kBatch = MODE == 2 ? 4 : 10;
  float mB[kBatch], aB[kBatch], lB[kBatch];
  auto request = [&](int s0) {
#pragma unroll
    for (int k = 0; k < kBatch; ++k) {
      const int s = s0 + k * kMergeGroups;
      mB[k] = -INFINITY;
      aB[k] = lB[k] = 0.f;
      if (s < hi) {
        const float *rec = base + (size_t)s * kRec;
        mB[k] = rec[0];
        aB[k] = rec[2 + quarter * kMergeDims + tx];
        if (tx == 0) lB[k] = rec[1];
      }
    }
  };
  request(lo + ty);
  float gate_in = 0.f;
  if (MODE != 1 && gate != nullptr && ty == 0) gate_in = gate[(size_t)out_row * kHeadDim + quarter * kMergeDims + tx];

  // MODE 3: the score of the extra key, by the first 256 threads (one dim each)
  float x_score = -INFINITY;
  const uint8_t *x_vrow = nullptr;
  if (MODE == 3) {
    __shared__ float s_dot[8];
    const int kvh = row / kGroup;
    float prod = 0.f;
    if (threadIdx.x < kHeadDim)
      prod = xk.q[(size_t)row * kHeadDim + threadIdx.x] *
             load_cache_value(xk.k_row + (size_t)kvh * merge_row_bytes(xk.kt), xk.kt, threadIdx.x);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) prod += __shfl_xor_sync(0xffffffffu, prod, o);
    if (threadIdx.x < kHeadDim && (threadIdx.x & 31) == 0) s_dot[threadIdx.x >> 5] = prod;
    __syncthreads();
    float dot = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) dot += s_dot[i];
    x_score = dot * xk.scale;
    x_vrow = xk.v_row + (size_t)kvh * merge_row_bytes(xk.vt);
  }

  // (its value for this thread's dim: requested here, used after the groups have met)
  float x_val = 0.f;
  if (MODE == 3 && ty == 0) x_val = load_cache_value(x_vrow, xk.vt, quarter * kMergeDims + tx);

  float mloc = -INFINITY, acc = 0.f, ll = 0.f;
  for (int s0 = lo + ty; s0 < hi; s0 += kBatch * kMergeGroups) {
    if (s0 != lo + ty) request(s0);
    float mb = mloc;
#pragma unroll
    for (int k = 0; k < kBatch; ++k) mb = fmaxf(mb, mB[k]);
    if (mb != -INFINITY) {
      const float f = expf(mloc - mb);   // 0 while nothing has been accumulated
      acc *= f;
      ll *= f;
#pragma unroll
      for (int k = 0; k < kBatch; ++k) {
        if (mB[k] != -INFINITY) {
          const float w = expf(mB[k] - mb);
          acc = fmaf(aB[k], w, acc);
          ll = fmaf(lB[k], w, ll);
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
    float mm = MODE == 3 ? x_score : -INFINITY;
#pragma unroll
    for (int i = 0; i < kMergeGroups; ++i) mm = fmaxf(mm, s_gm[i]);
    float a = 0.f, l = 0.f;
#pragma unroll
    for (int i = 0; i < kMergeGroups; ++i) {
      if (s_gm[i] != -INFINITY) {
        const float w = expf(s_gm[i] - mm);
        a = fmaf(s_acc[i][tx], w, a);
        l = fmaf(s_l[i], w, l);
      }
    }
    const int d = quarter * kMergeDims + tx;
    if (MODE == 3) {
      const float w = expf(x_score - mm);
      a = fmaf(x_val, w, a);
      l += w;
    }
    if (MODE != 1) {
      float o = (mm != -INFINITY && l > 0.f) ? a / l : 0.f;
      float *op = out + (size_t)out_row * kHeadDim + d;
      if (gate != nullptr) {
        float *gp = gate + (size_t)out_row * kHeadDim + d;
        const float sg = __fdiv_rn(1.0f, 1.0f + expf(-gate_in));
        *gp = sg;
        o *= sg;
      }
      *op = o;
    } else {
      float *rec = out + ((size_t)row * n_out + j) * kRec;
      rec[2 + d] = a;
      if (d == 0) {
        rec[0] = mm;
        rec[1] = l;
      }
    }
  }
}

int launch_merge(const float *partial, float *out, int n_rows, int n_splits, float *gate,
                 cudaStream_t st) {
  if (n_rows == 0) return RD_OK;
  const dim3 grid((unsigned)n_rows, kHeadDim / kMergeDims, 1);
  return launch_pdl(4, merge_kernel<0>, grid, dim3(kMergeDims * kMergeGroups), 0, st, partial, out, n_splits,
                    1, gate, nullptr, 1, ExtraKey{}) == cudaSuccess
             ? RD_OK
             : RD_ERR_CUDA;
}

int launch_merge_extra(const float *partial, float *out, int n_rows, int n_splits, float *gate,
                       const ExtraKey &x, cudaStream_t st) {
  if (n_rows == 0) return RD_OK;
  const dim3 grid((unsigned)n_rows, kHeadDim / kMergeDims, 1);
  return launch_pdl(4, merge_kernel<3>, grid, dim3(kMergeDims * kMergeGroups), 0, st, partial, out, n_splits,
                    1, gate, nullptr, 1, x) == cudaSuccess
             ? RD_OK
             : RD_ERR_CUDA;
}

int launch_merge_records(const float *partial, float *records, int n_rows, int n_in, int n_out,
                         cudaStream_t st) {
  if (n_rows == 0) return RD_OK;
  const dim3 grid((unsigned)n_rows, kHeadDim / kMergeDims, (unsigned)n_out);
  return launch_pdl(4, merge_kernel<1>, grid, dim3(kMergeDims * kMergeGroups), 0, st, partial, records, n_in,
                    n_out, nullptr, nullptr, 1, ExtraKey{}) == cudaSuccess
             ? RD_OK
             : RD_ERR_CUDA;
}

int launch_merge_multi(const DecodeSeq *dev_seqs, const float *records, int n_seq, int q_len,
                       int n_head, cudaStream_t st) {
  const int rows = n_seq * q_len * n_head;
  if (rows == 0) return RD_OK;
  const dim3 grid((unsigned)rows, kHeadDim / kMergeDims, 1);
  return launch_pdl(4, merge_kernel<2>, grid, dim3(kMergeDims * kMergeGroups), 0, st, records, nullptr, 0, 1,
                    nullptr, dev_seqs, q_len * n_head, ExtraKey{}) == cudaSuccess
             ? RD_OK
             : RD_ERR_CUDA;
}

}  // namespace rd
