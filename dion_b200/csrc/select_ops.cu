// Dion2 / NorDion2 sub-matrix selection on sm_100a.
//
//   1. slice_norms : M += G (optional) fused with the L1 norm of every row or column of M
//   2. topk_select : exact top-k of the slice norms per matrix (radix select on the float bits,
//                    ties broken by lowest index so the result is deterministic), writing the
//                    selected indices and an inverse map (slice -> position or -1)
//   3. gather_ef   : copy the selected slices to a dense bf16 matrix and scale them in M by the
//                    error-feedback factor
//
// Together these replace the reference's compiled dion2_pre_orthogonalize
// (dion/dion2.py:437-547: foreach add, stacked norm, torch.topk, gather, per-parameter scatter_).
#include "common.cuh"

namespace dion {

enum : int { DT_F32 = 0, DT_BF16 = 1 };

__device__ __forceinline__ float ldv(const void* p, int dt, long long i) {
  return dt == DT_F32 ? reinterpret_cast<const float*>(p)[i]
                      : __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p)[i]);
}
__device__ __forceinline__ void stv(void* p, int dt, long long i, float v) {
  if (dt == DT_F32) reinterpret_cast<float*>(p)[i] = v;
  else reinterpret_cast<__nv_bfloat16*>(p)[i] = __float2bfloat16_rn(v);
}
__device__ __forceinline__ float rnd(float v, int dt) {
  return dt == DT_F32 ? v : __bfloat162float(__float2bfloat16_rn(v));
}

// 8 consecutive elements as floats / back (16-byte accesses for bf16, 2 x 16 for fp32).
__device__ __forceinline__ void ld8v(const void* p, int dt, long long i, float (&v)[8]) {
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
__device__ __forceinline__ void st8v(void* p, int dt, long long i, const float (&v)[8]) {
  if (dt == DT_F32) {
    float4* q = reinterpret_cast<float4*>(reinterpret_cast<float*>(p) + i);
    q[0] = make_float4(v[0], v[1], v[2], v[3]);
    q[1] = make_float4(v[4], v[5], v[6], v[7]);
  } else {
    *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(p) + i) =
        make_uint4(pack_bf16x2(v[0], v[1]), pack_bf16x2(v[2], v[3]), pack_bf16x2(v[4], v[5]),
                   pack_bf16x2(v[6], v[7]));
  }
}
__device__ __forceinline__ bool aligned16(const void* p) {
  return (reinterpret_cast<uintptr_t>(p) & 15) == 0;
}

// ptrs: device array [2][n] of int64 = G pointers (may be 0) then M pointers.
// Row selection: one warp per row; 8 elements per lane per step when the row length is a
// multiple of 8 and the buffers are 16-byte aligned.
__global__ void __launch_bounds__(256)
row_norms_kernel(const long long* ptrs, int n, int rows, int cols, int g_dt, int m_dt,
                 float* norms) {
  const long long wid = (long long)blockIdx.x * 8 + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (wid >= (long long)n * rows) return;
  const int t = (int)(wid / rows), r = (int)(wid - (long long)t * rows);
  const void* G = reinterpret_cast<const void*>(ptrs[t]);
  void* M = reinterpret_cast<void*>(ptrs[n + t]);
  const long long off = (long long)r * cols;
  float s = 0.f;
  if ((cols & 7) == 0 && aligned16(M) && (G == nullptr || aligned16(G))) {
    for (int c = lane * 8; c < cols; c += 256) {
      float m[8];
      ld8v(M, m_dt, off + c, m);
      if (G) {
        float g[8];
        ld8v(G, g_dt, off + c, g);
#pragma unroll
        for (int e = 0; e < 8; ++e) m[e] = rnd(m[e] + rnd(g[e], m_dt), m_dt);
        st8v(M, m_dt, off + c, m);
      }
#pragma unroll
      for (int e = 0; e < 8; ++e) s += fabsf(m[e]);
    }
  } else {
    for (int c = lane; c < cols; c += 32) {
      float m = ldv(M, m_dt, off + c);
      if (G) {
        m = rnd(m + rnd(ldv(G, g_dt, off + c), m_dt), m_dt);
        stv(M, m_dt, off + c, m);
      }
      s += fabsf(m);
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
  if (lane == 0) norms[wid] = s;
}

// Column selection: thread = column, block covers 64 columns x a strip of rows; partial column
// sums are accumulated with atomics into norms (zeroed by the caller).
constexpr int kColStrip = 128;
__global__ void __launch_bounds__(256)
col_norms_kernel(const long long* ptrs, int n, int rows, int cols, int g_dt, int m_dt,
                 float* norms) {
  const int t = blockIdx.z;
  const int c = blockIdx.x * 64 + (threadIdx.x & 63);
  const int rlane = threadIdx.x >> 6;  // 0..3
  const int r0 = blockIdx.y * kColStrip;
  const int r1 = min(rows, r0 + kColStrip);
  if (c >= cols) return;
  const void* G = reinterpret_cast<const void*>(ptrs[t]);
  void* M = reinterpret_cast<void*>(ptrs[n + t]);
  float s = 0.f;
  for (int r = r0 + rlane; r < r1; r += 4) {
    const long long e = (long long)r * cols + c;
    float m = ldv(M, m_dt, e);
    if (G) {
      m = rnd(m + rnd(ldv(G, g_dt, e), m_dt), m_dt);
      stv(M, m_dt, e, m);
    }
    s += fabsf(m);
  }
  atomicAdd(&norms[(long long)t * cols + c], s);
}

// Same for row lengths that are multiples of 8 and 16-byte aligned buffers: a thread owns 8
// adjacent columns; 256 threads = 32 column groups (256 columns) x 8 row lanes; the row lanes
// are combined in shared memory before one atomic per column.
__global__ void __launch_bounds__(256)
col_norms_vec_kernel(const long long* ptrs, int n, int rows, int cols, int g_dt, int m_dt,
                     float* norms) {
  __shared__ float part[8][256 + 8];
  const int t = blockIdx.z;
  const int cg = threadIdx.x & 31, rlane = threadIdx.x >> 5;
  const int c = blockIdx.x * 256 + cg * 8;
  const int r0 = blockIdx.y * kColStrip;
  const int r1 = min(rows, r0 + kColStrip);
  const void* G = reinterpret_cast<const void*>(ptrs[t]);
  void* M = reinterpret_cast<void*>(ptrs[n + t]);
  float s[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  const bool vec = aligned16(M) && (G == nullptr || aligned16(G));
  if (c < cols) {
    for (int r = r0 + rlane; r < r1; r += 8) {
      const long long e = (long long)r * cols + c;
      float m[8];
      if (vec) {
        ld8v(M, m_dt, e, m);
        if (G) {
          float g[8];
          ld8v(G, g_dt, e, g);
#pragma unroll
          for (int q = 0; q < 8; ++q) m[q] = rnd(m[q] + rnd(g[q], m_dt), m_dt);
          st8v(M, m_dt, e, m);
        }
      } else {  // a matrix that starts off a 16-byte boundary
#pragma unroll
        for (int q = 0; q < 8; ++q) {
          m[q] = ldv(M, m_dt, e + q);
          if (G) {
            m[q] = rnd(m[q] + rnd(ldv(G, g_dt, e + q), m_dt), m_dt);
            stv(M, m_dt, e + q, m[q]);
          }
        }
      }
#pragma unroll
      for (int q = 0; q < 8; ++q) s[q] += fabsf(m[q]);
    }
  }
#pragma unroll
  for (int q = 0; q < 8; ++q) part[rlane][cg * 8 + q] = s[q];
  __syncthreads();
  const int col = blockIdx.x * 256 + threadIdx.x;
  if (col < cols) {
    float tot = 0.f;
#pragma unroll
    for (int l = 0; l < 8; ++l) tot += part[l][threadIdx.x];
    atomicAdd(&norms[(long long)t * cols + col], tot);
  }
}

// ---------------------------------------------------------------------------------------------
// Exact top-k per matrix.  One block of 1024 threads per matrix; norms are non-negative, so the
// float bit pattern orders like an unsigned integer.
// ---------------------------------------------------------------------------------------------
constexpr int kSelThreads = 1024;

__device__ __forceinline__ int block_exclusive_scan(int v, int* total, int* warp_sums) {
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  int x = v;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    int y = __shfl_up_sync(0xffffffffu, x, o);
    if (lane >= o) x += y;
  }
  __syncthreads();
  if (lane == 31) warp_sums[w] = x;
  __syncthreads();
  if (w == 0) {
    int s = warp_sums[lane];
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      int y = __shfl_up_sync(0xffffffffu, s, o);
      if (lane >= o) s += y;
    }
    warp_sums[lane] = s;
  }
  __syncthreads();
  const int warp_off = (w == 0) ? 0 : warp_sums[w - 1];
  *total = warp_sums[31];
  return warp_off + x - v;
}

__global__ void __launch_bounds__(kSelThreads)
topk_select_kernel(const float* norms, int num, int k, long long* idx_out, int* map_out) {
  __shared__ int hist[256];
  __shared__ int warp_sums[32];
  __shared__ uint32_t s_prefix;
  __shared__ int s_remaining;
  const int t = blockIdx.x;
  const uint32_t* keys = reinterpret_cast<const uint32_t*>(norms + (long long)t * num);
  long long* idx = idx_out + (long long)t * k;
  int* map = map_out + (long long)t * num;

  if (threadIdx.x == 0) { s_prefix = 0; s_remaining = k; }
  __syncthreads();
  // Radix select: after the loop s_prefix is the key of the k-th largest element.
  for (int shift = 24; shift >= 0; shift -= 8) {
    if (threadIdx.x < 256) hist[threadIdx.x] = 0;
    __syncthreads();
    const uint32_t prefix = s_prefix;
    const uint32_t hi_mask = (shift == 24) ? 0u : (0xFFFFFFFFu << (shift + 8));
    for (int i = threadIdx.x; i < num; i += kSelThreads) {
      const uint32_t key = keys[i];
      if ((key & hi_mask) == prefix) atomicAdd(&hist[(key >> shift) & 255], 1);
    }
    __syncthreads();
    if (threadIdx.x < 32) {
      // Find the bin that holds the rem-th largest key, walking from bin 255 down: every lane
      // owns eight bins, a suffix sum over the lanes tells each how many keys lie in the bins
      // above its own, and the one lane whose bins contain the target finishes the walk.
      const int lane = threadIdx.x;
      int h[8], mine = 0;
#pragma unroll
      for (int j = 0; j < 8; ++j) { h[j] = hist[lane * 8 + j]; mine += h[j]; }
      int incl = mine;                       // sum over lanes >= this one
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int y = __shfl_down_sync(0xffffffffu, incl, o);
        if (lane + o < 32) incl += y;
      }
      const int above = incl - mine;
      const int rem0 = s_remaining;
      const bool here = above < rem0 && rem0 <= incl;
      // No lane qualifies only if fewer than rem keys match the prefix, which the counts of the
      // previous digit exclude; lane 0 then settles on bin 0 as a serial walk would.
      const unsigned who = __ballot_sync(0xffffffffu, here);
      if (here || (who == 0u && lane == 0)) {
        int rem = rem0 - above, b = lane * 8;
        if (here) {
#pragma unroll
          for (int j = 7; j >= 0; --j) {
            if (h[j] >= rem) { b = lane * 8 + j; break; }
            rem -= h[j];
          }
        }
        s_prefix = prefix | ((uint32_t)b << shift);
        s_remaining = rem;
      }
    }
    __syncthreads();
  }
  const uint32_t thr = s_prefix;
  // s_remaining = how many elements equal to thr are taken (lowest indices first).
  const int take_eq = s_remaining;
  const int n_gt = k - take_eq;
  int run_gt = 0, run_eq = 0;
  for (int base = 0; base < num; base += kSelThreads) {
    const int i = base + threadIdx.x;
    uint32_t key = 0;
    const bool in = i < num;
    if (in) key = keys[i];
    const int f_gt = (in && key > thr) ? 1 : 0;
    const int f_eq = (in && key == thr) ? 1 : 0;
    int tot_gt, tot_eq;
    const int p_gt = block_exclusive_scan(f_gt, &tot_gt, warp_sums);
    __syncthreads();
    const int p_eq = block_exclusive_scan(f_eq, &tot_eq, warp_sums);
    __syncthreads();
    if (in) {
      int pos = -1;
      if (f_gt) pos = run_gt + p_gt;
      else if (f_eq && run_eq + p_eq < take_eq) pos = n_gt + run_eq + p_eq;
      map[i] = pos;
      if (pos >= 0) idx[pos] = i;
    }
    run_gt += tot_gt;
    run_eq += tot_eq;
  }
}

// Row gather + error feedback.  grid = (k, n); U[t][j][:] = bf16(M[t][idx[j]][:]);
// M[t][idx[j]][:] *= ef (skipped when ef_apply == 0).  M pointers from ptrs[n + t].
// With u_ptrs the destination of matrix t is u_ptrs[t] (possibly another GPU's peer-mapped
// memory) instead of U + t*u_stride; with ss_ptrs the sum of squares of the bf16 values of each
// gathered row is added to *ss_ptrs[t].
__global__ void __launch_bounds__(256)
gather_rows_kernel(const long long* ptrs, int n, int cols, int m_dt, const long long* idx, int k,
                   __nv_bfloat16* U, long long u_stride, float ef, int ef_apply,
                   const long long* u_ptrs, const long long* ss_ptrs) {
  __shared__ float red[8];
  const int j = blockIdx.x, t = blockIdx.y;
  void* M = reinterpret_cast<void*>(ptrs[n + t]);
  const long long r = idx[(long long)t * k + j];
  const long long off = r * cols;
  __nv_bfloat16* base = u_ptrs ? reinterpret_cast<__nv_bfloat16*>(u_ptrs[t])
                               : U + (long long)t * u_stride;
  __nv_bfloat16* u = base + (long long)j * cols;
  float acc = 0.f;
  if ((cols & 7) == 0 && aligned16(M) && aligned16(u)) {
    for (int c = threadIdx.x * 8; c < cols; c += 256 * 8) {
      float m[8], o[8];
      ld8v(M, m_dt, off + c, m);
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        o[e] = __bfloat162float(__float2bfloat16_rn(m[e]));
        acc += o[e] * o[e];
      }
      st8v(u, DT_BF16, c, o);
      if (ef_apply) {
#pragma unroll
        for (int e = 0; e < 8; ++e) m[e] *= ef;
        st8v(M, m_dt, off + c, m);
      }
    }
  } else {
    for (int c = threadIdx.x; c < cols; c += 256) {
      const float m = ldv(M, m_dt, off + c);
      const __nv_bfloat16 b = __float2bfloat16_rn(m);
      u[c] = b;
      const float f = __bfloat162float(b);
      acc += f * f;
      if (ef_apply) stv(M, m_dt, off + c, m * ef);
    }
  }
  if (ss_ptrs) {
    for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = acc;
    __syncthreads();
    if (threadIdx.x == 0) {
      float s = 0.f;
      for (int w = 0; w < 8; ++w) s += red[w];
      atomicAdd(reinterpret_cast<float*>(ss_ptrs[t]), s);
    }
  }
}

// Column gather: U[t][r][j] = bf16(M[t][r][idx[j]]); M *= ef at the selected columns.
// grid = (ceil(rows/8), n); 256 threads = 8 rows x 32 column lanes.
__global__ void __launch_bounds__(256)
gather_cols_kernel(const long long* ptrs, int n, int rows, int cols, int m_dt,
                   const long long* idx, int k, __nv_bfloat16* U, long long u_stride, float ef,
                   int ef_apply) {
  const int t = blockIdx.y;
  const int r = blockIdx.x * 8 + (threadIdx.x >> 5);
  if (r >= rows) return;
  void* M = reinterpret_cast<void*>(ptrs[n + t]);
  const long long* id = idx + (long long)t * k;
  __nv_bfloat16* u = U + (long long)t * u_stride + (long long)r * k;
  for (int j = threadIdx.x & 31; j < k; j += 32) {
    const long long e = (long long)r * cols + id[j];
    const float m = ldv(M, m_dt, e);
    u[j] = __float2bfloat16_rn(m);
    if (ef_apply) stv(M, m_dt, e, m * ef);
  }
}

// Scatter rows of a dense bf16 [n][k][cols] into zero-initialised [n][rows][cols] (global scope).
__global__ void __launch_bounds__(256)
scatter_rows_kernel(const __nv_bfloat16* src, const long long* idx, int k, int cols,
                    __nv_bfloat16* dst, int rows) {
  const int j = blockIdx.x, t = blockIdx.y;
  const long long r = idx[(long long)t * k + j];
  const __nv_bfloat16* s = src + ((long long)t * k + j) * cols;
  __nv_bfloat16* d = dst + ((long long)t * rows + r) * cols;
  for (int c = threadIdx.x; c < cols; c += 256) d[c] = s[c];
}

}  // namespace dion

using namespace dion;
static inline cudaStream_t S(void* s) { return static_cast<cudaStream_t>(s); }
static inline int rc() { return cudaGetLastError() == cudaSuccess ? 0 : -1; }

// norms must hold n*rows (select_rows) or n*cols floats; for column selection it must be zeroed.
DION_EXPORT int dion_slice_norms(const void* ptrs, int n, int rows, int cols, int g_dt, int m_dt,
                                 int select_rows, float* norms, void* stream) {
  if (n <= 0 || rows <= 0 || cols <= 0) return 0;
  if (select_rows) {
    const long long warps = (long long)n * rows;
    row_norms_kernel<<<(unsigned)((warps + 7) / 8), 256, 0, S(stream)>>>(
        static_cast<const long long*>(ptrs), n, rows, cols, g_dt, m_dt, norms);
  } else {
    if ((cols & 7) == 0) {
      dim3 grid((cols + 255) / 256, (rows + kColStrip - 1) / kColStrip, n);
      col_norms_vec_kernel<<<grid, 256, 0, S(stream)>>>(static_cast<const long long*>(ptrs), n,
                                                        rows, cols, g_dt, m_dt, norms);
    } else {
      dim3 grid((cols + 63) / 64, (rows + kColStrip - 1) / kColStrip, n);
      col_norms_kernel<<<grid, 256, 0, S(stream)>>>(static_cast<const long long*>(ptrs), n, rows,
                                                    cols, g_dt, m_dt, norms);
    }
  }
  return rc();
}

DION_EXPORT int dion_topk_select(const float* norms, int n, int num, int k, long long* idx,
                                 int* map, void* stream) {
  if (n <= 0 || num <= 0) return 0;
  if (k <= 0 || k > num) return -2;
  topk_select_kernel<<<n, kSelThreads, 0, S(stream)>>>(norms, num, k, idx, map);
  return rc();
}

DION_EXPORT int dion_gather_ef(const void* ptrs, int n, int rows, int cols, int m_dt,
                               const long long* idx, int k, int select_rows, void* U,
                               long long u_stride, float ef, int ef_apply, const void* u_ptrs,
                               const void* ss_ptrs, void* stream) {
  if (n <= 0 || k <= 0) return 0;
  if (select_rows) {
    dim3 grid(k, n);
    gather_rows_kernel<<<grid, 256, 0, S(stream)>>>(
        static_cast<const long long*>(ptrs), n, cols, m_dt, idx, k,
        static_cast<__nv_bfloat16*>(U), u_stride, ef, ef_apply,
        static_cast<const long long*>(u_ptrs), static_cast<const long long*>(ss_ptrs));
  } else {
    if (u_ptrs != nullptr || ss_ptrs != nullptr) return -3;
    dim3 grid((rows + 7) / 8, n);
    gather_cols_kernel<<<grid, 256, 0, S(stream)>>>(static_cast<const long long*>(ptrs), n, rows,
                                                    cols, m_dt, idx, k,
                                                    static_cast<__nv_bfloat16*>(U), u_stride, ef,
                                                    ef_apply);
  }
  return rc();
}

DION_EXPORT int dion_scatter_rows(const void* src, const long long* idx, int n, int k, int cols,
                                  void* dst, int rows, void* stream) {
  if (n <= 0 || k <= 0) return 0;
  dim3 grid(k, n);
  scatter_rows_kernel<<<grid, 256, 0, S(stream)>>>(static_cast<const __nv_bfloat16*>(src), idx, k,
                                                   cols, static_cast<__nv_bfloat16*>(dst), rows);
  return rc();
}
