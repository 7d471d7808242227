// Implementation of the allocation-free entry point declared in no_alloc.h.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdio.h>

#include "no_alloc.h"

namespace {

constexpr int kThreads = 256;
constexpr int kChunk = 4096;
constexpr int kMaxDevices = 64;

// Scratch that lives in the module: one accumulator per matrix.  In host code this name is only
// a stand-in for the symbol; its device address is looked up once per GPU below.
static __device__ __align__(256) float g_sumsq_scratch[DION_NOALLOC_MAX_MATRICES];

static float* g_scratch_addr[kMaxDevices] = {nullptr};

__global__ void __launch_bounds__(kThreads)
sumsq_kernel(const __nv_bfloat16* X, long long numel, float* acc) {
  __shared__ float red[kThreads / 32];
  const int t = blockIdx.y;
  const __nv_bfloat16* x = X + (long long)t * numel;
  const long long base = (long long)blockIdx.x * kChunk;
  const long long end = (base + kChunk < numel) ? base + kChunk : numel;
  float s = 0.f;
  for (long long i = base + threadIdx.x; i < end; i += kThreads) {
    const float f = __bfloat162float(x[i]);
    s += f * f;
  }
  for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = s;
  __syncthreads();
  if (threadIdx.x < 32) {
    float v = threadIdx.x < kThreads / 32 ? red[threadIdx.x] : 0.f;
    for (int o = 4; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    if (threadIdx.x == 0) atomicAdd(&acc[t], v);
  }
}

__global__ void finalize_kernel(const float* acc, float* scale, int n, float mult, float eps) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) scale[i] = 1.f / (sqrtf(acc[i]) * mult + eps);
}

}  // namespace

extern "C" __attribute__((visibility("default")))
int dion_frobenius_scale_noalloc(const void* X, int n, long long numel, float mult, float eps,
                                 float* scale_out, void* stream) {
  if (X == nullptr || scale_out == nullptr || n <= 0 || numel <= 0) {
    fprintf(stderr, "dion_frobenius_scale_noalloc: bad arguments (null pointer or size <= 0)\n");
    return DION_NOALLOC_ERR_BAD_ARGS;
  }
  if (n > DION_NOALLOC_MAX_MATRICES) {
    fprintf(stderr,
            "dion_frobenius_scale_noalloc: n = %d matrices exceeds the built-in scratch of %d; "
            "split the batch\n", n, DION_NOALLOC_MAX_MATRICES);
    return DION_NOALLOC_ERR_TOO_LARGE;
  }
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices)
    return DION_NOALLOC_ERR_LAUNCH;
  float* scratch = g_scratch_addr[dev];
  if (scratch == nullptr) {
    // First call on this GPU: resolve the device address of the module's array.
    void* p = nullptr;
    const cudaError_t e = cudaGetSymbolAddress(&p, g_sumsq_scratch);
    if (e != cudaSuccess || p == nullptr) {
      fprintf(stderr, "dion_frobenius_scale_noalloc: cudaGetSymbolAddress failed: %s\n",
              cudaGetErrorString(e));
      return DION_NOALLOC_ERR_LAUNCH;
    }
    scratch = static_cast<float*>(p);
    g_scratch_addr[dev] = scratch;
  }
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  // The array keeps whatever the previous call left in it: clear the part used now.
  if (cudaMemsetAsync(scratch, 0, sizeof(float) * (size_t)n, s) != cudaSuccess)
    return DION_NOALLOC_ERR_LAUNCH;
  dim3 grid((unsigned)((numel + kChunk - 1) / kChunk), (unsigned)n);
  if (grid.y > 65535u) {  // gridDim.y limit; n <= 16384 keeps us below it
    return DION_NOALLOC_ERR_TOO_LARGE;
  }
  sumsq_kernel<<<grid, kThreads, 0, s>>>(static_cast<const __nv_bfloat16*>(X), numel, scratch);
  finalize_kernel<<<(n + 127) / 128, 128, 0, s>>>(scratch, scale_out, n, mult, eps);
  return cudaGetLastError() == cudaSuccess ? DION_NOALLOC_OK : DION_NOALLOC_ERR_LAUNCH;
}
