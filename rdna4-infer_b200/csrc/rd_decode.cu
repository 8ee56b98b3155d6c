// Type dispatch of the split-KV decode kernel (instantiations live in
// rd_decode_k_*.cu so that they compile in parallel).
#include "rd_common.cuh"
#include "rd_internal.h"

namespace rd {

int launch_decode_k_f32(int vt, const DecodeArgs &a, cudaStream_t st);
int launch_decode_k_f16(int vt, const DecodeArgs &a, cudaStream_t st);
int launch_decode_k_q8_0(int vt, const DecodeArgs &a, cudaStream_t st);
int launch_decode_k_q4_0(int vt, const DecodeArgs &a, cudaStream_t st);
int launch_decode_k_q5_0(int vt, const DecodeArgs &a, cudaStream_t st);
int launch_decode_k_q4_1(int vt, const DecodeArgs &a, cudaStream_t st);

int launch_decode_multi_k_f32(int vt, const MultiDecodeArgs &a, cudaStream_t st);
int launch_decode_multi_k_f16(int vt, const MultiDecodeArgs &a, cudaStream_t st);
int launch_decode_multi_k_q8_0(int vt, const MultiDecodeArgs &a, cudaStream_t st);
int launch_decode_multi_k_q4_0(int vt, const MultiDecodeArgs &a, cudaStream_t st);
int launch_decode_multi_k_q5_0(int vt, const MultiDecodeArgs &a, cudaStream_t st);
int launch_decode_multi_k_q4_1(int vt, const MultiDecodeArgs &a, cudaStream_t st);

int launch_decode_multi(int kt, int vt, const MultiDecodeArgs &a, cudaStream_t st) {
  switch (kt) {
    case RD_KV_F32: return launch_decode_multi_k_f32(vt, a, st);
    case RD_KV_F16: return launch_decode_multi_k_f16(vt, a, st);
    case RD_KV_Q8_0: return launch_decode_multi_k_q8_0(vt, a, st);
    case RD_KV_Q4_0: return launch_decode_multi_k_q4_0(vt, a, st);
    case RD_KV_Q5_0: return launch_decode_multi_k_q5_0(vt, a, st);
    case RD_KV_Q4_1: return launch_decode_multi_k_q4_1(vt, a, st);
    default: return RD_ERR_UNSUPPORTED;
  }
}

int launch_decode(int kt, int vt, const DecodeArgs &a, cudaStream_t st) {
  switch (kt) {
    case RD_KV_F32: return launch_decode_k_f32(vt, a, st);
    case RD_KV_F16: return launch_decode_k_f16(vt, a, st);
    case RD_KV_Q8_0: return launch_decode_k_q8_0(vt, a, st);
    case RD_KV_Q4_0: return launch_decode_k_q4_0(vt, a, st);
    case RD_KV_Q5_0: return launch_decode_k_q5_0(vt, a, st);
    case RD_KV_Q4_1: return launch_decode_k_q4_1(vt, a, st);
    default: return RD_ERR_UNSUPPORTED;
  }
}

int decode_tile_keys(int kt, int vt) { return 16 * key_groups(kt, vt); }

}  // namespace rd
