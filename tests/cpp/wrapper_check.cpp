// Compiles a caller written against the reference's names (namespace rdna4, KvType,
// *_launch returning bool) against include/rdna4/ and checks the host-side behaviour
// that needs no GPU: tables, byte budgets, and that bad arguments return false.
#include <cstdio>

#include "rdna4/attn.cuh"
#include "rdna4/attn_fa2.cuh"

#define CHECK(c)                                     \
  do {                                               \
    if (!(c)) {                                      \
      std::printf("FAILED line %d: %s\n", __LINE__, #c); \
      return 1;                                      \
    }                                                \
  } while (0)

int main() {
  using namespace rdna4;
  KvType t = KvType::F32;
  CHECK(kv_type_parse("q4_0", &t) == nullptr && t == KvType::Q4_0);
  CHECK(kv_type_parse("q5_1", &t) != nullptr);  // a name llama.cpp has and the engine does not
  CHECK(kv_type_parse("", &t) != nullptr);
  CHECK(kv_row_bytes(KvType::Q4_0, 256) == 144 && kv_row_bytes(KvType::Q8_0, 256) == 272);
  CHECK(kv_row_bytes(KvType::Q5_0, 256) == 176 && kv_row_bytes(KvType::Q4_1, 256) == 160);
  CHECK(kv_row_bytes(KvType::F16, 256) == 512 && kv_row_bytes(KvType::F32, 256) == 1024);
  CHECK(kv_bytes_per_elem(KvType::Q4_0) == 18.0 / 32.0);
  CHECK(attn_partial_bytes(24, 256, 16) == 396288);
  CHECK(attn_split_wpb(4) == 16 && attn_split_wpb(8) == 8 && attn_split_wpb(16) == 16);
  // 131072-token cache budgets: 16 layers x 4 kv heads
  auto per_tok = [](KvType k, KvType v) { return 16ull * 4 * (kv_row_bytes(k, 256) + kv_row_bytes(v, 256)); };
  CHECK(131072ull * per_tok(KvType::F16, KvType::F16) == 8589934592ull);
  CHECK(131072ull * per_tok(KvType::Q4_0, KvType::Q4_0) == 2415919104ull);
  // launchers refuse bad arguments on the host and report false
  CHECK(!attn_launch(nullptr, nullptr, nullptr, nullptr, 3, 24, 4, 256, 0.0625f, t, t));
  CHECK(!attn_launch_split(nullptr, nullptr, nullptr, nullptr, nullptr, 3, 24, 4, 256, 0.0625f,
                           KvType::F16, KvType::F16, 0));
  CHECK(!kv_store_row_launch<KvType::Q8_0>(nullptr, nullptr, 33));
  CHECK(!kv_store_row_launch((KvType)99, nullptr, nullptr, 64));
  CHECK(!kv_fill_launch((KvType)99, nullptr, 4, 256, 1));
  CHECK(fa2_prefill_usable(KvType::F16, KvType::F16, 512, 2048, 24, 4, 256));
  CHECK(!fa2_prefill_usable(KvType::Q8_0, KvType::F16, 512, 2048, 24, 4, 256));
  std::printf("wrapper check OK\n");
  return 0;
}
