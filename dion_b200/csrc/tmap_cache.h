// Host-side cache of encoded TMA tensor maps (opt-in: DION_B200_TMAP_CACHE=1).
//
// Every GEMM launch needs up to four 3-D bf16 tensor maps; an eager Newton-Schulz loop encodes 60
// per call although only about 14 distinct ones occur, and with the caching allocator the same
// buffers come back step after step.  An encoded map is a pure function of (address, extents,
// strides, box) for the fixed element type / swizzle / promotion used in this library, so a map
// found under the same key can be reused.  The table is direct-mapped (a colliding key simply
// replaces the slot) and guarded by a mutex because the library entry points may be called from
// several host threads.
#pragma once

#include <cuda.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#include <mutex>

namespace dion {

struct TmapKey {
  uint64_t ptr;
  uint64_t dims[3];
  uint64_t strides[2];
  uint32_t box[3];
  uint32_t pad;
};

struct TmapSlot {
  TmapKey key;
  CUtensorMap map;
  int used;
};

constexpr int kTmapSlots = 512;

inline bool tmap_cache_enabled() {
  static const bool on = [] {
    const char* v = getenv("DION_B200_TMAP_CACHE");
    return v != nullptr && v[0] == '1';
  }();
  return on;
}

inline uint64_t tmap_hash(const TmapKey& k) {
  const uint64_t* w = reinterpret_cast<const uint64_t*>(&k);
  uint64_t h = 0x9E3779B97F4A7C15ull;
  for (size_t i = 0; i < sizeof(TmapKey) / 8; ++i) {
    h ^= w[i] + 0x9E3779B97F4A7C15ull + (h << 6) + (h >> 2);
  }
  return h ^ (h >> 29);
}

// Encodes (or fetches) the 3-D bf16 map with 128-byte swizzle used throughout this library.
// `enc` is the driver's cuTensorMapEncodeTiled.  Returns 0, or -2 when the driver rejects the map.
template <typename EncodeFn>
inline int encode_bf16_3d(EncodeFn enc, CUtensorMap* map, const void* ptr, const cuuint64_t dims[3],
                          const cuuint64_t strides[2], const cuuint32_t box[3]) {
  static std::mutex mu;
  static TmapSlot slots[kTmapSlots];  // zero-initialised: used == 0
  const bool cached = tmap_cache_enabled();
  TmapKey key;
  TmapSlot* slot = nullptr;
  if (cached) {
    memset(&key, 0, sizeof(key));
    key.ptr = reinterpret_cast<uint64_t>(ptr);
    for (int i = 0; i < 3; ++i) { key.dims[i] = dims[i]; key.box[i] = box[i]; }
    key.strides[0] = strides[0];
    key.strides[1] = strides[1];
    slot = &slots[tmap_hash(key) % kTmapSlots];
    std::lock_guard<std::mutex> guard(mu);
    if (slot->used && memcmp(&slot->key, &key, sizeof(key)) == 0) {
      memcpy(map, &slot->map, sizeof(CUtensorMap));
      return 0;
    }
  }
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(ptr), dims, strides,
                   box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return -2;
  if (cached) {
    std::lock_guard<std::mutex> guard(mu);
    slot->key = key;
    memcpy(&slot->map, map, sizeof(CUtensorMap));
    slot->used = 1;
  }
  return 0;
}

}  // namespace dion
