// Host-only stand-in for the HIP runtime header, used ONLY to compile the
// reference project's attention / KV headers with g++ so that their kernels can
// be executed on the CPU as the parity pin of the oracle (see ../../ref_driver.cpp).
// It declares just enough of the device vocabulary for those headers to parse:
// qualifiers become no-ops, the thread/block indices are globals that the fiber
// scheduler in the driver sets before it resumes a simulated thread, and the two
// warp/block synchronisation primitives call back into that scheduler.
#pragma once
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>

#define __global__
#define __device__
#define __host__
#define __forceinline__ inline
#define __shared__ static

struct rdshim_dim3 {
  unsigned x, y, z;
  constexpr rdshim_dim3(unsigned x_ = 1, unsigned y_ = 1, unsigned z_ = 1) : x(x_), y(y_), z(z_) {}
};
typedef rdshim_dim3 dim3;
struct uint4 {
  unsigned x, y, z, w;
};

extern rdshim_dim3 threadIdx, blockIdx, blockDim, gridDim;

typedef void *hipStream_t;
typedef int hipError_t;
static const hipError_t hipSuccess = 0;
inline hipError_t hipGetLastError() { return hipSuccess; }

// Implemented by the driver's fiber scheduler.
void rdshim_syncthreads();
float rdshim_shfl_xor(float v, int lane_mask);
#define __syncthreads() rdshim_syncthreads()
#define __shfl_xor_sync(mask, v, off) rdshim_shfl_xor((v), (off))

// Device math the reference's other kernels in the same headers name.
inline float rsqrtf(float x) { return 1.0f / sqrtf(x); }
