// Stand-in for the HIP runtime header that lets nvcc compile the reference project's
// attention / KV headers UNMODIFIED for sm_100a (see ../../ref_gpu_driver.cu): the handful
// of runtime names those headers use are mapped onto their CUDA equivalents. Used only
// to build oracle/_ref/librd_ref_gpu.so, the "reference kernels on the same GPU"
// cross-check and timing row -- never part of the product library.
#pragma once
#include <cuda_runtime.h>

typedef cudaStream_t hipStream_t;
typedef cudaError_t hipError_t;
#define hipSuccess cudaSuccess
#define hipGetLastError cudaGetLastError
#if defined(__CUDA_ARCH__)
#define __HIP_DEVICE_COMPILE__ 1
#endif
// The reference's "unknown enum" branch traps on the device. It is unreachable with the
// six valid KV types, and nothing here may ever fault a GPU, so it compiles to nothing.
#define __builtin_trap() ((void)0)
