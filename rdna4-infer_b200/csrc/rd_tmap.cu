// Host-side construction of TMA tensor maps for KV-cache tiles. The driver's encoder
// is reached through cudaGetDriverEntryPoint, so the library links against the CUDA
// runtime only.
#include <mutex>

#include "rd_common.cuh"
#include "rd_internal.h"

namespace rd {

namespace {
typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *,
                                  const cuuint64_t *, const cuuint64_t *, const cuuint32_t *,
                                  const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn g_encode = nullptr;
std::once_flag g_once;

void resolve() {
  void *fn = nullptr;
  cudaDriverEntryPointQueryResult q;
  if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q) == cudaSuccess &&
      q == cudaDriverEntryPointSuccess)
    g_encode = (EncodeTiledFn)fn;
}
}  // namespace

int encode_kv_tmap(void *tmap_out, const void *base, int type, int n_head_kv, int64_t n_rows,
                   int tile_rows) {
  std::call_once(g_once, resolve);
  if (g_encode == nullptr) return RD_ERR_CUDA;
  // One key = the n_head_kv stored rows, contiguous: viewed as u64 elements. The box is
  // two elements (16 bytes) wider than the key; those columns lie outside the tensor and
  // are zero-filled, which gives every key of the shared-memory tile a pitch of
  // key bytes + 16 -- the bank-conflict-free layout the fragment loaders want.
  const int key_bytes = n_head_kv * row_bytes(type);
  if (key_bytes == 0 || key_bytes % 16 != 0 || key_bytes / 8 + 2 > 256 || tile_rows > 256 ||
      n_rows < 1)
    return RD_ERR_SHAPE;
  if (((uintptr_t)base & 15) != 0) return RD_ERR_ALIGN;
  const cuuint64_t dims[2] = {(cuuint64_t)(key_bytes / 8), (cuuint64_t)n_rows};
  const cuuint64_t strides[1] = {(cuuint64_t)key_bytes};  // bytes between keys
  const cuuint32_t box[2] = {(cuuint32_t)(key_bytes / 8 + 2), (cuuint32_t)tile_rows};
  const cuuint32_t estr[2] = {1, 1};
  const CUresult r = g_encode((CUtensorMap *)tmap_out, CU_TENSOR_MAP_DATA_TYPE_UINT64, 2,
                              const_cast<void *>(base), dims, strides, box, estr,
                              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
                              CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? RD_OK : RD_ERR_CUDA;
}


int encode_f16_tmap(void *tmap_out, const void *base, int n_head_kv, int64_t n_rows, int tile_rows) {
  std::call_once(g_once, resolve);
  if (g_encode == nullptr) return RD_ERR_CUDA;
  if (n_rows < 1 || tile_rows > 256) return RD_ERR_SHAPE;
  if (((uintptr_t)base & 15) != 0) return RD_ERR_ALIGN;
  const cuuint64_t dims[2] = {(cuuint64_t)n_head_kv * kHeadDim, (cuuint64_t)n_rows};
  const cuuint64_t strides[1] = {(cuuint64_t)n_head_kv * kHeadDim * 2};
  const cuuint32_t box[2] = {64, (cuuint32_t)tile_rows};  // 64 halves = one 128-byte swizzle row
  const cuuint32_t estr[2] = {1, 1};
  const CUresult r = g_encode((CUtensorMap *)tmap_out, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2,
                              const_cast<void *>(base), dims, strides, box, estr,
                              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                              CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? RD_OK : RD_ERR_CUDA;
}

}  // namespace rd
