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
  if (flag_wait_bounded(flags + i, want)) return;
  report_peer_timeout(status, i, want, ld_acquire_sys_i32(flags + i));
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

// ---------------------------------------------------------------------------------------------
// All-reduce (sum, optionally scaled) of a symmetric buffer, two-shot: this rank reduces the
// slice [rank*per, (rank+1)*per) of 16-byte vectors over all ranks and writes the result into
// every rank's buffer.  Two forms:
//   multimem: one `multimem.ld_reduce` per vector (the NVSwitch adds the ranks' copies) and one
//             `multimem.st` (the switch replicates the store), on the multicast address;
//   peer    : plain loads from every peer's copy and plain stores to every peer's copy.
// dt: 0 = fp32, 1 = bf16 (accumulated in fp32).
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ float4 mm_ld_reduce_f32(const void* mc) {
  float4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0, %1, %2, %3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
               : "l"(mc)
               : "memory");
  return v;
}
__device__ __forceinline__ uint4 mm_ld_reduce_bf16(const void* mc) {
  uint4 v;
  asm volatile(
      "multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0, %1, %2, %3}, [%4];"
      : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
      : "l"(mc)
      : "memory");
  return v;
}
__device__ __forceinline__ void mm_st_b32x4(void* mc, uint4 v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(mc),
               "f"(__uint_as_float(v.x)), "f"(__uint_as_float(v.y)), "f"(__uint_as_float(v.z)),
               "f"(__uint_as_float(v.w))
               : "memory");
}
__device__ __forceinline__ uint4 scale_vec(uint4 v, int dt, float scale) {
  if (scale == 1.f) return v;
  if (dt == 0) {
    v.x = __float_as_uint(__uint_as_float(v.x) * scale);
    v.y = __float_as_uint(__uint_as_float(v.y) * scale);
    v.z = __float_as_uint(__uint_as_float(v.z) * scale);
    v.w = __float_as_uint(__uint_as_float(v.w) * scale);
  } else {
    uint32_t* w = &v.x;
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      float2 f = unpack_bf16x2(w[e]);
      w[e] = pack_bf16x2(f.x * scale, f.y * scale);
    }
  }
  return v;
}

// The flag barriers are part of the kernel (one launch per all-reduce).  Block 0 tells every peer that
// this rank's input is in place (the kernel runs after its producers in stream order); every
// block waits (bounded) for all peers' inputs, reduces its share of this rank's slice and
// writes it everywhere; the block that finishes last publishes "slice written" to the peers,
// waits (bounded) for theirs and advances the sequence number.  Blocks never wait for each
// other, only for other GPUs.
struct AllReduceArgs {
  char* mc_base;                 // multicast address of the data (0 = use peer_bases)
  const long long* peer_bases;   // [world] data base addresses
  const long long* peer_in;      // [world] base of each peer's "input ready" flags
  const long long* peer_out;     // [world] base of each peer's "slice written" flags
  const int* flags_in;           // local flags, one per source rank
  const int* flags_out;
  int* seq;
  unsigned* counter;
  int* status;
  long long vec_begin, vec_end;
  int world, rank, dt;
  float scale;
  int gather;                    // 1: all-gather (push this rank's slice to everyone), 0: reduce
};

__global__ void __launch_bounds__(256)
allreduce_fused_kernel(const AllReduceArgs a) {
  __shared__ int s_ok;
  __shared__ int s_last;
  const int seq = *a.seq + 1;
  if (threadIdx.x == 0) s_ok = 1;
  __syncthreads();
  if (blockIdx.x == 0 && threadIdx.x < a.world) {
    __threadfence_system();
    st_release_sys_i32(reinterpret_cast<int*>(a.peer_in[threadIdx.x]) + a.rank, seq);
  }
  if (threadIdx.x < a.world) {
    const bool got = flag_wait_bounded(a.flags_in + threadIdx.x, seq);
    if (!got) {
      report_peer_timeout(a.status, threadIdx.x, seq, ld_acquire_sys_i32(a.flags_in + threadIdx.x));
      s_ok = 0;
    }
  }
  __syncthreads();
  if (s_ok && a.gather) {
    // All-gather: this rank's slice already lies in its own copy; replicate it.
    const char* own = reinterpret_cast<const char*>(a.peer_bases[a.rank]);
    for (long long i = a.vec_begin + (long long)blockIdx.x * 256 + threadIdx.x; i < a.vec_end;
         i += (long long)gridDim.x * 256) {
      const uint4 v = *reinterpret_cast<const uint4*>(own + i * 16);
      if (a.mc_base != nullptr) {
        mm_st_b32x4(a.mc_base + i * 16, v);   // the switch delivers it to every rank
      } else {
        for (int r = 0; r < a.world; ++r)
          if (r != a.rank)
            *reinterpret_cast<uint4*>(reinterpret_cast<char*>(a.peer_bases[r]) + i * 16) = v;
      }
    }
  } else if (s_ok) {
    for (long long i = a.vec_begin + (long long)blockIdx.x * 256 + threadIdx.x; i < a.vec_end;
         i += (long long)gridDim.x * 256) {
      if (a.mc_base != nullptr) {
        char* p = a.mc_base + i * 16;
        uint4 v;
        if (a.dt == 0) {
          const float4 f = mm_ld_reduce_f32(p);
          v = make_uint4(__float_as_uint(f.x), __float_as_uint(f.y), __float_as_uint(f.z),
                         __float_as_uint(f.w));
        } else {
          v = mm_ld_reduce_bf16(p);
        }
        mm_st_b32x4(p, scale_vec(v, a.dt, a.scale));
      } else {
        float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        for (int r = 0; r < a.world; ++r) {
          const uint4 u = *reinterpret_cast<const uint4*>(
              reinterpret_cast<const char*>(a.peer_bases[r]) + i * 16);
          if (a.dt == 0) {
            acc[0] += __uint_as_float(u.x); acc[1] += __uint_as_float(u.y);
            acc[2] += __uint_as_float(u.z); acc[3] += __uint_as_float(u.w);
          } else {
            const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const float2 f = unpack_bf16x2(w[e]);
              acc[2 * e] += f.x; acc[2 * e + 1] += f.y;
            }
          }
        }
        uint4 out;
        if (a.dt == 0) {
          out = make_uint4(__float_as_uint(acc[0] * a.scale), __float_as_uint(acc[1] * a.scale),
                           __float_as_uint(acc[2] * a.scale), __float_as_uint(acc[3] * a.scale));
        } else {
          out = make_uint4(pack_bf16x2(acc[0] * a.scale, acc[1] * a.scale),
                           pack_bf16x2(acc[2] * a.scale, acc[3] * a.scale),
                           pack_bf16x2(acc[4] * a.scale, acc[5] * a.scale),
                           pack_bf16x2(acc[6] * a.scale, acc[7] * a.scale));
        }
        for (int r = 0; r < a.world; ++r)
          *reinterpret_cast<uint4*>(reinterpret_cast<char*>(a.peer_bases[r]) + i * 16) = out;
      }
    }
  }
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) s_last = (atomicAdd(a.counter, 1u) == gridDim.x - 1) ? 1 : 0;
  __syncthreads();
  if (!s_last) return;
  __threadfence_system();
  if (threadIdx.x < a.world) {
    st_release_sys_i32(reinterpret_cast<int*>(a.peer_out[threadIdx.x]) + a.rank, seq);
    const bool got = flag_wait_bounded(a.flags_out + threadIdx.x, seq);
    if (!got)
      report_peer_timeout(a.status, threadIdx.x, seq,
                          ld_acquire_sys_i32(a.flags_out + threadIdx.x));
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    *a.counter = 0u;
    *a.seq = seq;
  }
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

// In-place all-reduce (gather = 0) or all-gather (gather = 1: [vec_begin, vec_end) is this rank's
// slice) of 16-byte vectors of a symmetric buffer in one launch (see allreduce_fused_kernel).  `seq` and `counter` are device words owned by the workspace.
DION_EXPORT int dion_allreduce_fused(void* mc_base, const void* peer_bases, const void* peer_in,
                                     const void* peer_out, const int* flags_in,
                                     const int* flags_out, int* seq, unsigned* counter,
                                     int* status, int world, int rank, long long vec_begin,
                                     long long vec_end, int dt, float scale, int gather,
                                     int num_blocks, void* stream) {
  if (world <= 0 || world > 256 || (dt != 0 && dt != 1)) return -2;
  long long n = vec_end > vec_begin ? vec_end - vec_begin : 0;
  long long need = (n + 255) / 256;
  int blocks = (int)(need < (long long)num_blocks ? need : (long long)num_blocks);
  if (blocks < 1) blocks = 1;  // an empty slice still takes part in the barriers
  AllReduceArgs a;
  a.mc_base = static_cast<char*>(mc_base);
  a.peer_bases = static_cast<const long long*>(peer_bases);
  a.peer_in = static_cast<const long long*>(peer_in);
  a.peer_out = static_cast<const long long*>(peer_out);
  a.flags_in = flags_in; a.flags_out = flags_out;
  a.seq = seq; a.counter = counter; a.status = status;
  a.vec_begin = vec_begin; a.vec_end = vec_end > vec_begin ? vec_end : vec_begin;
  a.world = world; a.rank = rank; a.dt = dt; a.scale = scale; a.gather = gather;
  allreduce_fused_kernel<<<blocks, 256, 0, S(stream)>>>(a);
  return rc();
}
