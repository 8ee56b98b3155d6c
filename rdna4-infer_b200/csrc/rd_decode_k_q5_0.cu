// Decode-attention kernels whose K cache is q5_0, one instantiation per V type.
#include "rd_decode.cuh"

namespace rd {
int launch_decode_k_q5_0(int vt, const DecodeArgs &a, cudaStream_t st) {
  switch (vt) {
    case RD_KV_F32: return launch_decode_typed<RD_KV_Q5_0, RD_KV_F32>(a, st);
    case RD_KV_F16: return launch_decode_typed<RD_KV_Q5_0, RD_KV_F16>(a, st);
    case RD_KV_Q8_0: return launch_decode_typed<RD_KV_Q5_0, RD_KV_Q8_0>(a, st);
    case RD_KV_Q4_0: return launch_decode_typed<RD_KV_Q5_0, RD_KV_Q4_0>(a, st);
    case RD_KV_Q5_0: return launch_decode_typed<RD_KV_Q5_0, RD_KV_Q5_0>(a, st);
    case RD_KV_Q4_1: return launch_decode_typed<RD_KV_Q5_0, RD_KV_Q4_1>(a, st);
    default: return RD_ERR_UNSUPPORTED;
  }
}
int launch_decode_multi_k_q5_0(int vt, const MultiDecodeArgs &a, cudaStream_t st) {
  switch (vt) {
    case RD_KV_F32: return multi_decode_typed<RD_KV_Q5_0, RD_KV_F32>(a, st);
    case RD_KV_F16: return multi_decode_typed<RD_KV_Q5_0, RD_KV_F16>(a, st);
    case RD_KV_Q8_0: return multi_decode_typed<RD_KV_Q5_0, RD_KV_Q8_0>(a, st);
    case RD_KV_Q4_0: return multi_decode_typed<RD_KV_Q5_0, RD_KV_Q4_0>(a, st);
    case RD_KV_Q5_0: return multi_decode_typed<RD_KV_Q5_0, RD_KV_Q5_0>(a, st);
    case RD_KV_Q4_1: return multi_decode_typed<RD_KV_Q5_0, RD_KV_Q4_1>(a, st);
    default: return RD_ERR_UNSUPPORTED;
  }
}
}  // namespace rd
