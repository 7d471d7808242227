// Host check of the tensor-map cache with a counting stand-in for the driver's encoder.
// Prints "calls_off calls_on hit_equal miss_differs"; the Python test asserts on them.
#include <stdio.h>
#include <string.h>

#include "tmap_cache.h"

static int g_calls = 0;

static CUresult fake_encode(CUtensorMap* map, CUtensorMapDataType, cuuint32_t, void* ptr,
                            const cuuint64_t* dims, const cuuint64_t* strides, const cuuint32_t* box,
                            const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                            CUtensorMapL2promotion, CUtensorMapFloatOOBfill) {
  ++g_calls;
  memset(map, 0, sizeof(*map));
  unsigned long long sig = (unsigned long long)(size_t)ptr ^ (dims[0] * 3) ^ (dims[1] * 5) ^
                           (dims[2] * 7) ^ (strides[0] * 11) ^ (strides[1] * 13) ^
                           (box[0] * 17ull) ^ (box[1] * 19ull) ^ ((unsigned long long)g_calls << 48);
  memcpy(map, &sig, sizeof(sig));
  return CUDA_SUCCESS;
}

int main() {
  CUtensorMap a, b, c;
  cuuint64_t dims[3] = {768, 768, 4}, strides[2] = {1536, 1179648};
  cuuint32_t box[3] = {64, 128, 1};
  void* p = (void*)0x7f0000001000ull;
  for (int i = 0; i < 3; ++i) dion::encode_bf16_3d(fake_encode, &a, p, dims, strides, box);
  const int calls_same = g_calls;                 // 3 without the cache, 1 with it
  dion::encode_bf16_3d(fake_encode, &b, p, dims, strides, box);
  const int hit_equal = memcmp(&a, &b, sizeof(a)) == 0;
  cuuint32_t box2[3] = {64, 64, 1};
  dion::encode_bf16_3d(fake_encode, &c, p, dims, strides, box2);      // other box: must miss
  const int miss_differs = memcmp(&a, &c, sizeof(a)) != 0;
  const int before = g_calls;
  void* q = (void*)0x7f0000002000ull;
  dion::encode_bf16_3d(fake_encode, &c, q, dims, strides, box);       // other address: must miss
  const int other_ptr_encoded = g_calls == before + 1;
  printf("%d %d %d %d %d\n", calls_same, g_calls, hit_equal, miss_differs, other_ptr_encoded);
  return 0;
}
