// Shared device/host helpers of the sm_100a attention / KV-cache library.
#pragma once
#include <math.h>
#include <stdlib.h>
#include <cuda.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "rd_attn.h"

namespace rd {

constexpr int kHeadDim = 256;   // the only head size built (reference model: qwen35)
constexpr int kGroup = 6;       // query heads per KV head
constexpr int kRec = 2 + kHeadDim;  // floats in one partial record (m, l, acc[256])

// Bytes of one stored row of kHeadDim elements; include/rdna4/kv.h:155-169.
__host__ __device__ constexpr int row_bytes(int type) {
  return type == RD_KV_F32   ? kHeadDim * 4
         : type == RD_KV_F16 ? kHeadDim * 2
         : type == RD_KV_Q8_0 ? 8 * 34
         : type == RD_KV_Q4_0 ? 8 * 18
         : type == RD_KV_Q5_0 ? 8 * 22
         : type == RD_KV_Q4_1 ? 8 * 20
                              : 0;
}

// Status word written by kernels that give up on a bounded wait. Lives at the start
// of the workspace; sticky until read by rd_device_status().
// RoPE frequencies base^(-2p/n_rot) of the first pairs, computed on the host in double
// and rounded once (the reference calls f32 powf, attn.cuh:39; a one-ulp difference moves
// theta by milliradians at position 131000) and passed by value: a double pow per CTA
// on the device costs microseconds. Pairs beyond kRopeTablePairs fall back to the
// device computation.
constexpr int kRopeTablePairs = 64;
struct RopeTable {
  float f[kRopeTablePairs];
};
inline RopeTable make_rope_table(int n_rot, float freq_base) {
  RopeTable t;
  for (int p = 0; p < kRopeTablePairs; ++p) {
    const float e = -2.0f * (float)p / (float)n_rot;
    t.f[p] = n_rot > 0 && p < n_rot / 2 ? (float)pow((double)freq_base, (double)e) : 0.f;
  }
  return t;
}

struct DeviceStatus {
  int timeout_flag;   // non-zero: some wait ran out
  int where;          // site id of the first wait that ran out
  int pad[2];
};

// ---- decode tile geometry (shared by the kernel and the host-side split planning)
// A CTA of the decode kernel runs G key groups of four warps (one per kv head); group gi
// streams 16-key slots through its own ring of D shared-memory slots.
constexpr int kMaxStages = 8;            // ring depth per key group
constexpr int kMaxGroups = 3;
constexpr int kMaxPos = 24;              // ring positions of a CTA, all groups together
constexpr int kSmemBudget = 225 * 1024;  // dynamic, per CTA, of the 227 KB an sm_100 CTA may use
constexpr int kSlotKeys = 16;            // keys per ring slot = rows of one MMA tile

// Bytes of one key in a shared-memory tile: the n_head_kv rows plus 16 bytes, which
// makes the per-lane row walks of every loader above bank-conflict-free for
// n_head_kv == 4 (pitch = 16 or 80 bytes mod 128).
__host__ __device__ constexpr int key_pitch(int type, int nkv) { return nkv * row_bytes(type) + 16; }

// Shared memory in front of the ring: the slots' mbarriers and counters (512 bytes),
// then the query fragments of the CTA's token: a 256-entry dim -> slot table (512
// bytes) and 144 bytes per (head, quad lane) for up to 24 heads.
constexpr int kBarBytes = 512;
constexpr int kFragPitch = 144;
constexpr int kQStageBytes = 512 + 4 * kGroup * 4 * kFragPitch;   // n_head_kv <= 4
constexpr int kRingOffset = kBarBytes + kQStageBytes;             // multiple of 128
static_assert(kRingOffset % 128 == 0, "ring must start 128-byte aligned");

__host__ __device__ constexpr int slot_bytes(int kt, int vt, int nkv) {
  return kSlotKeys * (key_pitch(kt, nkv) + key_pitch(vt, nkv));
}
// Key groups per CTA: as many (up to 3) as leave every group a ring of at least two
// slots -- more resident warps hide the dequantize -> MMA latency better, and two slots
// per group keep one load in flight while the other slot is consumed.
__host__ __device__ constexpr int key_groups(int kt, int vt) {
  return 3 * 2 * slot_bytes(kt, vt, 4) <= kSmemBudget - kRingOffset   ? 3
         : 2 * 2 * slot_bytes(kt, vt, 4) <= kSmemBudget - kRingOffset ? 2
                                                                      : 1;
}
// Ring depth per group for n_head_kv kv heads (0: one slot does not fit).
__host__ __device__ constexpr int ring_depth(int kt, int vt, int nkv) {
  const int d = (kSmemBudget - kRingOffset) / (key_groups(kt, vt) * slot_bytes(kt, vt, nkv));
  const int cap = kMaxPos / key_groups(kt, vt) < kMaxStages ? kMaxPos / key_groups(kt, vt) : kMaxStages;
  return d > cap ? cap : d;
}

// ---- programmatic dependent launch ---------------------------------------------
// The hot kernels of a layer step (append, decode, merge) are launched with the
// programmatic-stream-serialization attribute: the next kernel of the stream may be
// scheduled while this one still runs, so its launch latency and its memory-independent
// set-up overlap this kernel's tail. Every such kernel calls pdl_launch_dependents() first
// (the kernel after it may start launching) and pdl_wait() before its first access to
// global memory (the kernel before it has completed and its writes are visible).
__device__ __forceinline__ void pdl_launch_dependents() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

inline int pdl_mask() {
#ifdef RD_TIMING_SWITCHES
  static const int m = [] {
    const char *e = getenv("RD_PDL");
    return e ? atoi(e) : 2;
  }();
  return m;
#else
  return 2;   // measured: only the decode kernel gains as a dependent launch
#endif
}
template <class... KArgs, class... Args>
inline cudaError_t launch_pdl(int which, void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                              cudaStream_t st, Args &&...args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = (pdl_mask() & which) ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

// ---- PTX helpers ---------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void *p) {
  return (uint32_t)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ uint32_t lds32(uint32_t addr) {
  uint32_t v;
  asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr));
  return v;
}
__device__ __forceinline__ uint4 lds128(uint32_t addr) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "r"(addr));
  return v;
}
__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
  uint32_t r;
  asm("prmt.b32 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(sel));
  return r;
}
// (a & b) | c in one LOP3 (immLut 0xEA).
__device__ __forceinline__ uint32_t and_or(uint32_t a, uint32_t b, uint32_t c) {
  uint32_t r;
  asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(r) : "r"(a), "r"(b), "r"(c));
  return r;
}
// half2 fma on raw 32-bit registers.
__device__ __forceinline__ uint32_t hfma2(uint32_t a, uint32_t b, uint32_t c) {
  uint32_t r;
  asm("fma.rn.f16x2 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(c));
  return r;
}
__device__ __forceinline__ uint32_t hmul2(uint32_t a, uint32_t b) {
  uint32_t r;
  asm("mul.rn.f16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
  return r;
}
__device__ __forceinline__ uint32_t hsub2(uint32_t a, uint32_t b) {
  uint32_t r;
  asm("sub.rn.f16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
  return r;
}
__device__ __forceinline__ uint32_t pack_h2(float lo, float hi) {
  uint32_t r;
  asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
  return r;
}
__device__ __forceinline__ float ex2(float x) {
  float r;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x));
  return r;
}
// Packed pairs of f32 (sm_100 add.f32x2 / fma.rn.f32x2: two lanes per instruction).
__device__ __forceinline__ unsigned long long f2_pack(float lo, float hi) {
  unsigned long long r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
  return r;
}
__device__ __forceinline__ void f2_unpack(unsigned long long v, float &lo, float &hi) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ unsigned long long f2_add(unsigned long long a, unsigned long long b) {
  unsigned long long r;
  asm("add.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
  return r;
}
__device__ __forceinline__ float max3(float a, float b, float c) {
  float r;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(a), "f"(b), "f"(c));
  return r;
}
// D = A(16x16, row) * B(16x8, col) + D, f16 inputs, f32 accumulate.
__device__ __forceinline__ void mma16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                         uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
// Warp-wide transpose of an 8x8 matrix of b16 held in mma fragment layout.
__device__ __forceinline__ uint32_t movmatrix_trans(uint32_t a) {
  uint32_t r;
  asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(r) : "r"(a));
  return r;
}

// ---- mbarrier / bulk copy ------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded wait: gives up once kWaitNs of wall-clock time have passed (the clock is read
// every 256 polls), records the site in `status` and returns false so the caller can
// unwind without leaving the GPU spinning.
constexpr unsigned long long kWaitNs = 2000000000ull;
__device__ __forceinline__ unsigned long long global_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ bool mbar_test_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, DeviceStatus *status,
                                          int site) {
  // a short burst of non-suspending polls first: most waits in a running pipeline are
  // satisfied within a few hundred cycles, and try_wait may park the thread for longer
#ifndef RD_POLL_BURST
#define RD_POLL_BURST 128
#endif
  for (int i = 0; i < RD_POLL_BURST; ++i) {
    if (mbar_test_wait(bar, parity)) return true;
  }
  const unsigned long long t0 = global_ns();
  for (uint32_t i = 1;; ++i) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((i & 255u) == 0 && global_ns() - t0 > kWaitNs) break;
  }
  if (status != nullptr && atomicExch(&status->timeout_flag, 1) == 0) status->where = site;
  return false;
}
// global -> shared bulk copy (TMA engine, no tensor map): 16-byte aligned both sides,
// size a multiple of 16; completion is signalled on `bar` by byte count.
__device__ __forceinline__ void bulk_g2s(uint32_t dst_smem, const void *src, uint32_t bytes,
                                         uint32_t bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::
          "r"(dst_smem),
      "l"(src), "r"(bytes), "r"(bar)
      : "memory");
}
// global -> shared 2-D tile copy through a tensor map: box rows land densely in shared
// memory (128-byte aligned), rows outside the tensor are filled with zeros. x is in
// elements of the map's data type and must keep x * element size a multiple of 16.
__device__ __forceinline__ void tma_load_2d(uint32_t dst_smem, const CUtensorMap *map, int x, int y,
                                            uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, "
      "{%2, %3}], [%4];" ::"r"(dst_smem),
      "l"(map), "r"(x), "r"(y), "r"(bar)
      : "memory");
}
__device__ __forceinline__ void fence_barrier_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void fence_proxy_async() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

// ---- fp16 storage conversion, include/rdna4/fp16.h:37-57 ----------------------
// Round-to-nearest-even like the hardware conversion, except that NaN becomes a
// signed infinity (the reference's bit routine has no NaN case).
__device__ __forceinline__ uint16_t f32_to_f16_bits(float f) {
  if (f != f) return (uint16_t)(((__float_as_uint(f) >> 16) & 0x8000u) | 0x7c00u);
  return __half_as_ushort(__float2half_rn(f));
}
__device__ __forceinline__ float f16_bits_to_f32(uint16_t h) {
  return __half2float(__ushort_as_half(h));
}

// One stored value of a cache row (kv_load, include/rdna4/kv.h:174-229), type chosen at run
// time: used for the single newest key that a merge or an exchange folds in.
__device__ __forceinline__ float load_cache_value(const uint8_t *row, int type, int d) {
  const int b = d >> 5, j = d & 31;
  auto h2f = [](const uint8_t *p) { return __half2float(__ushort_as_half(*reinterpret_cast<const unsigned short *>(p))); };
  switch (type) {
    case RD_KV_F32: return reinterpret_cast<const float *>(row)[d];
    case RD_KV_F16: return h2f(row + 2 * d);
    case RD_KV_Q8_0: {
      const uint8_t *blk = row + 34 * b;
      return __fmul_rn(h2f(blk), (float)(int8_t)blk[2 + j]);
    }
    case RD_KV_Q4_0: {
      const uint8_t *blk = row + 18 * b;
      const int byte = blk[2 + (j & 15)];
      return __fmul_rn(h2f(blk), (float)((j < 16 ? (byte & 15) : (byte >> 4)) - 8));
    }
    case RD_KV_Q5_0: {
      const uint8_t *blk = row + 22 * b;
      const int byte = blk[6 + (j & 15)];
      const int hi = (blk[2 + (j >> 3)] >> (j & 7)) & 1;
      return __fmul_rn(h2f(blk), (float)(((j < 16 ? (byte & 15) : (byte >> 4)) | (hi << 4)) - 16));
    }
    default: {  // RD_KV_Q4_1
      const uint8_t *blk = row + 20 * b;
      const int byte = blk[4 + (j & 15)];
      return __fadd_rn(__fmul_rn(h2f(blk), (float)(j < 16 ? (byte & 15) : (byte >> 4))), h2f(blk + 2));
    }
  }
}
__host__ __device__ constexpr int merge_row_bytes(int type) {
  return type == RD_KV_F32 ? 1024 : type == RD_KV_F16 ? 512 : type == RD_KV_Q8_0 ? 272 : type == RD_KV_Q4_0 ? 144
         : type == RD_KV_Q5_0 ? 176 : 160;
}


}  // namespace rd
