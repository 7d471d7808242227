// Flag protocol for exchanges over peer-mapped (symmetric) memory on NVLink / NVSwitch.
//
// Data moves with ordinary stores issued by compute kernels straight into the destination GPU's
// buffer (the momentum kernel writes its bf16 output into the owners' receive buffers; the last
// Newton-Schulz GEMM writes result rows into the owners' return buffers).  These small kernels
// only publish and await that movement:
//
//   bump_seq      ++*seq                         start of an exchange round
//   signal_peers  flag[slot] on every peer = *seq   after the stores of the preceding kernels
//   wait_flags    spin until flags[i] >= *seq + delta for all i, bounded
//
// The sequence number lives in device memory, so a captured CUDA graph replays the protocol
// with fresh numbers.  Every wait is bounded: after about a second it stores an error code in
// the status word and returns, so a peer that never arrives cannot hang the GPU.
#include "common.cuh"

namespace dion {

__device__ __forceinline__ int ld_acquire_sys_i32(const int* p) {
  int v;
  asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_sys_i32(int* p, int v) {
  asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

constexpr unsigned kMaxFlagPolls = 1u << 22;

__global__ void bump_seq_kernel(int* seq) {
  if (threadIdx.x == 0 && blockIdx.x == 0) *seq += 1;
}

// peer_flags: device array of n_peers addresses (int64), each the base of that peer's flag array.
__global__ void signal_peers_kernel(const long long* peer_flags, int n_peers, int slot,
                                    const int* seq) {
  const int d = threadIdx.x;
  if (d >= n_peers) return;
  __threadfence_system();  // stores of earlier kernels on this stream are ordered before the flag
  st_release_sys_i32(reinterpret_cast<int*>(peer_flags[d]) + slot, *seq);
}

__global__ void wait_flags_kernel(const int* flags, int n, const int* seq, int delta, int* status) {
  const int i = threadIdx.x;
  if (i >= n) return;
  const int want = *seq + delta;
  for (unsigned k = 0; k < kMaxFlagPolls; ++k) {
    if (ld_acquire_sys_i32(flags + i) >= want) return;
    __nanosleep(64);
  }
  atomicExch(status, kStatusTimeoutPeer);
}

// scale[b] = 1 / (sqrt(sum_s partials[b*n_src + s]) * mult + eps); optionally clears partials.
__global__ void scale_from_partials_kernel(float* partials, int n_mats, int n_src, float mult,
                                           float eps, float* scale, int clear) {
  const int b = blockIdx.x * blockDim.x + threadIdx.x;
  if (b >= n_mats) return;
  float ss = 0.f;
  for (int s = 0; s < n_src; ++s) {
    ss += partials[(long long)b * n_src + s];
    if (clear) partials[(long long)b * n_src + s] = 0.f;
  }
  scale[b] = 1.f / (sqrtf(ss) * mult + eps);
}

}  // namespace dion

using namespace dion;
static inline cudaStream_t S(void* s) { return static_cast<cudaStream_t>(s); }
static inline int rc() { return cudaGetLastError() == cudaSuccess ? 0 : -1; }

DION_EXPORT int dion_bump_seq(int* seq, void* stream) {
  bump_seq_kernel<<<1, 32, 0, S(stream)>>>(seq);
  return rc();
}
DION_EXPORT int dion_signal_peers(const void* peer_flags, int n_peers, int slot, const int* seq,
                                  void* stream) {
  if (n_peers <= 0) return 0;
  if (n_peers > 1024) return -2;
  signal_peers_kernel<<<1, ((n_peers + 31) / 32) * 32, 0, S(stream)>>>(
      static_cast<const long long*>(peer_flags), n_peers, slot, seq);
  return rc();
}
DION_EXPORT int dion_wait_flags(const int* flags, int n, const int* seq, int delta, int* status,
                                void* stream) {
  if (n <= 0) return 0;
  if (n > 1024) return -2;
  wait_flags_kernel<<<1, ((n + 31) / 32) * 32, 0, S(stream)>>>(flags, n, seq, delta, status);
  return rc();
}
DION_EXPORT int dion_scale_from_partials(float* partials, int n_mats, int n_src, float mult,
                                         float eps, float* scale, int clear, void* stream) {
  if (n_mats <= 0) return 0;
  scale_from_partials_kernel<<<(n_mats + 127) / 128, 128, 0, S(stream)>>>(partials, n_mats, n_src,
                                                                          mult, eps, scale, clear);
  return rc();
}
