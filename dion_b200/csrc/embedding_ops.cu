// Backward of the token embedding for sm_100a: the weight gradient GW[v] = sum of the rows of DY
// whose token id is v, written exactly once per row (zeros where the id does not occur), with a
// result that does not depend on scheduling.  It replaces what the reference gets from the stock
// dense embedding backward under its compiler (models/gpt_model.py:298-307: `nn.Embedding`), which
// zero-fills the [V, C] gradient and scatters into it with atomics.
//
// Four launches, no host synchronisation, scratch supplied by the caller:
//   1. keys[i] = id (V for ids outside [0, V)), vals[i] = i as 32-bit integers;
//   2. a stable radix sort of the (key, position) pairs over just the bits an id needs
//      (CUB's device-wide sort; 16 bits for a 50 K vocabulary instead of the 64 of a sort of the
//      id tensor itself), so that every id's positions are consecutive and ascending;
//   3. starts[v] = first sorted index whose key is >= v, one thread per v (binary search) - the
//      run of row v is [starts[v], starts[v+1]);
//   4. one warp per row of GW sums the run in fp32 in position order, or writes zeros.  Runs
//      longer than kEmbLongRun are split into contiguous segments over the block's warps and the
//      partial sums added in segment order: real token streams have ids that occur thousands of
//      times per batch, and one warp walking such a run alone would decide the kernel's duration.
#include <cub/device/device_radix_sort.cuh>

#include "common.cuh"

namespace dion {

enum : int { DT_F32 = 0, DT_BF16 = 1 };

// 8 consecutive elements as floats (callers guarantee 8-element alignment).
__device__ __forceinline__ void emb_load8(const void* p, int dt, long long i, float (&v)[8]) {
  if (dt == DT_F32) {
    const float4* q = reinterpret_cast<const float4*>(reinterpret_cast<const float*>(p) + i);
    const float4 a = q[0], b = q[1];
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
  } else {
    const uint4 u = *reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(p) + i);
    const float2 a = unpack_bf16x2(u.x), b = unpack_bf16x2(u.y), c = unpack_bf16x2(u.z),
                 d = unpack_bf16x2(u.w);
    v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y; v[4] = c.x; v[5] = c.y; v[6] = d.x; v[7] = d.y;
  }
}

__global__ void __launch_bounds__(256)
emb_keys_kernel(const long long* __restrict__ ids, int* __restrict__ keys, int* __restrict__ vals,
                int n, int V) {
  const int i = blockIdx.x * 256 + threadIdx.x;
  if (i >= n) return;
  const long long t = ids[i];
  keys[i] = (t >= 0 && t < V) ? static_cast<int>(t) : V;
  vals[i] = i;
}

__global__ void __launch_bounds__(256)
emb_starts_kernel(const int* __restrict__ sorted, int* __restrict__ starts, int n, int V) {
  const int v = blockIdx.x * 256 + threadIdx.x;
  if (v > V) return;
  int lo = 0, hi = n;                      // first index with sorted[idx] >= v
  while (lo < hi) {
    const int mid = (lo + hi) >> 1;
    if (sorted[mid] < v) lo = mid + 1; else hi = mid;
  }
  starts[v] = lo;
}

constexpr int kEmbWarps = 8;
constexpr int kEmbLongRun = 64;

// acc += the rows perm[j] of DY for j in [j0, j1), columns [c8*8, c8*8+8), four loads in flight.
__device__ __forceinline__ void emb_sum_run(const void* __restrict__ DY, int dy_dt,
                                            const int* __restrict__ perm, int j0, int j1, int C,
                                            int c8, float (&acc)[8]) {
  int j = j0;
  for (; j + 4 <= j1; j += 4) {
    float v[4][8];
#pragma unroll
    for (int u = 0; u < 4; ++u) emb_load8(DY, dy_dt, (long long)perm[j + u] * C + c8 * 8, v[u]);
#pragma unroll
    for (int u = 0; u < 4; ++u)
#pragma unroll
      for (int e = 0; e < 8; ++e) acc[e] += v[u][e];
  }
  for (; j < j1; ++j) {
    float v[8];
    emb_load8(DY, dy_dt, (long long)perm[j] * C + c8 * 8, v);
#pragma unroll
    for (int e = 0; e < 8; ++e) acc[e] += v[e];
  }
}

__global__ void __launch_bounds__(kEmbWarps * 32)
embedding_bwd_kernel(const int* __restrict__ starts, const int* __restrict__ perm,
                     const void* __restrict__ DY, int dy_dt, float* __restrict__ GW, int C,
                     int V) {
  extern __shared__ __align__(16) float emb_part[];          // [kEmbWarps][C]
  __shared__ int run_lo[kEmbWarps], run_hi[kEmbWarps];
  const int w = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int C8 = C / 8;
  // Every block walks whole groups of kEmbWarps rows so that its barriers stay uniform.
  for (int base = blockIdx.x * kEmbWarps; base < V; base += gridDim.x * kEmbWarps) {
    const int v = base + w;
    int s = 0, e = 0;
    if (v < V) { s = starts[v]; e = starts[v + 1]; }
    if (lane == 0) { run_lo[w] = s; run_hi[w] = e; }
    if (v < V && e - s <= kEmbLongRun) {
      for (int c8 = lane; c8 < C8; c8 += 32) {
        float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        emb_sum_run(DY, dy_dt, perm, s, e, C, c8, acc);
        float4* q = reinterpret_cast<float4*>(GW + (long long)v * C + c8 * 8);
        q[0] = make_float4(acc[0], acc[1], acc[2], acc[3]);
        q[1] = make_float4(acc[4], acc[5], acc[6], acc[7]);
      }
    }
    __syncthreads();
    for (int ww = 0; ww < kEmbWarps; ++ww) {
      const int ls = run_lo[ww], le = run_hi[ww];
      if (le - ls <= kEmbLongRun) continue;                  // same decision in every thread
      const int seg = (le - ls + kEmbWarps - 1) / kEmbWarps;
      int j0 = ls + w * seg, j1 = j0 + seg;
      if (j0 > le) j0 = le;
      if (j1 > le) j1 = le;
      for (int c8 = lane; c8 < C8; c8 += 32) {
        float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        emb_sum_run(DY, dy_dt, perm, j0, j1, C, c8, acc);
#pragma unroll
        for (int q = 0; q < 8; ++q) emb_part[(size_t)w * C + c8 * 8 + q] = acc[q];
      }
      __syncthreads();
      for (int c = threadIdx.x; c < C; c += kEmbWarps * 32) {
        float t = 0.f;
#pragma unroll
        for (int q = 0; q < kEmbWarps; ++q) t += emb_part[(size_t)q * C + c];
        GW[(long long)(base + ww) * C + c] = t;
      }
      __syncthreads();
    }
    __syncthreads();                                          // run_lo / run_hi are rewritten next
  }
}

static inline int key_bits(long long V) {   // bits needed for the values 0 .. V
  int b = 1;
  while ((1LL << b) <= V) ++b;
  return b;
}

}  // namespace dion

using namespace dion;
static inline cudaStream_t S(void* s) { return static_cast<cudaStream_t>(s); }

// Bytes of temporary storage the sort of n (key, position) pairs needs.
DION_EXPORT long long dion_embedding_sort_bytes(long long n, long long V) {
  if (n <= 0) return 0;
  size_t bytes = 0;
  const int* kin = nullptr;
  int* kout = nullptr;
  if (cub::DeviceRadixSort::SortPairs(nullptr, bytes, kin, kout, kin, kout, static_cast<int>(n), 0,
                                      key_bits(V)) != cudaSuccess)
    return -1;
  return static_cast<long long>(bytes);
}

// ids: int64 [n].  DY: [n, C] fp32 or bf16 (dy_dt).  GW: fp32 [V, C], needs no initialisation.
// Scratch: keys, vals int32 [2n] each (unsorted then sorted halves), starts int32 [V+1], temp of
// at least dion_embedding_sort_bytes(n, V) bytes.  Limits: n, V < 2^31; 8*C*4 bytes of shared
// memory (C <= 7168); C a multiple of 8.
DION_EXPORT int dion_embedding_bwd(const void* ids, const void* DY, int dy_dt, float* GW,
                                   long long n, int C, long long V, int* keys, int* vals,
                                   int* starts, void* temp, long long temp_bytes, void* stream) {
  if (V <= 0) return 0;
  if (C % 8 || n < 0 || n >= (1LL << 31) - 256 || V >= (1LL << 31) - 256) return -2;
  const size_t smem = (size_t)kEmbWarps * C * sizeof(float);
  if (smem > 224 * 1024) return -2;
  const int ni = static_cast<int>(n), Vi = static_cast<int>(V);
  if (ni > 0) {
    emb_keys_kernel<<<(ni + 255) / 256, 256, 0, S(stream)>>>(static_cast<const long long*>(ids),
                                                            keys, vals, ni, Vi);
    size_t bytes = static_cast<size_t>(temp_bytes);
    if (cub::DeviceRadixSort::SortPairs(temp, bytes, keys, keys + ni, vals, vals + ni, ni, 0,
                                        key_bits(V), S(stream)) != cudaSuccess)
      return -4;
  }
  emb_starts_kernel<<<(Vi + 1 + 255) / 256, 256, 0, S(stream)>>>(keys + ni, starts, ni, Vi);
  if (smem > 48 * 1024 &&
      cudaFuncSetAttribute(embedding_bwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                           (int)smem) != cudaSuccess)
    return -3;
  const int groups = (Vi + kEmbWarps - 1) / kEmbWarps;
  const int cap = 148 * 8;
  embedding_bwd_kernel<<<groups < cap ? groups : cap, kEmbWarps * 32, smem, S(stream)>>>(
      starts, vals + ni, DY, dy_dt, GW, C, Vi);
  return cudaGetLastError() == cudaSuccess ? 0 : -1;
}
