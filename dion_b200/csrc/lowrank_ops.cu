// Batched dense factorizations for Dion's randomized Cholesky-QR (fp32, sm_100a):
//
//   dion_qr_r_factor   : R (upper triangular, r x r) of a batch of k x r matrices, k >= r,
//                        by Householder reflections;
//   dion_cholesky_upper: upper Cholesky factor of a batch of r x r symmetric matrices.
//
// They stand in for the per-matrix cuSOLVER calls behind torch.linalg.qr / cholesky_ex in the
// reference's orthogonalize() (dion/dion.py:1265-1308), which run one matrix after the other.
// Here one CTA owns one matrix and all matrices of a batch run at once.  A warp owns one column
// and keeps it in registers (rows lane, lane+32, ...).  Columns are processed in panels of 16:
// a panel's columns first receive every earlier panel's transformations (no synchronization,
// the earlier reflectors / factor columns are read back from global memory through L1), then the
// panel is factored column by column, each finished column being handed to the later warps of the
// panel through shared memory.
#include "common.cuh"

namespace dion {

constexpr int kLrThreads = 512;
constexpr int kPanel = kLrThreads / 32;   // 16 columns per panel
constexpr int kTilePitch = kPanel + 1;

__device__ __forceinline__ float warp_sum_f(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// Shared memory: tile[k][17] staging of a 16-column block | vs[2][k] published column |
// prev[16][k] reflectors of an earlier panel.
template <int KPL>
__global__ void __launch_bounds__(kLrThreads)
qr_r_kernel(const float* __restrict__ A, float* V, float* tau_g, float* __restrict__ R, int k,
            int r) {
  extern __shared__ float lr_smem[];
  float* tile = lr_smem;
  float* vs = lr_smem + (size_t)k * kTilePitch;
  float* prev = vs + 2 * (size_t)k;          // [16][k] reflectors of an earlier panel
  __shared__ float tau_s[2];
  __shared__ float prev_tau[kPanel];
  const int n = blockIdx.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const float* An = A + (size_t)n * k * r;
  float* Vn = V + (size_t)n * r * k;
  float* tn = tau_g + (size_t)n * r;
  float* Rn = R + (size_t)n * r * r;

  for (int c0 = 0; c0 < r; c0 += kPanel) {
    const int c = c0 + warp;
    const bool active = c < r;
    // Stage the block of columns [c0, c0+16) with row-contiguous reads.
    for (int e = threadIdx.x; e < k * kPanel; e += kLrThreads) {
      const int i = e / kPanel, cc = e - i * kPanel;
      tile[i * kTilePitch + cc] = (c0 + cc < r) ? An[(size_t)i * r + c0 + cc] : 0.f;
    }
    __syncthreads();
    float x[KPL];
#pragma unroll
    for (int t = 0; t < KPL; ++t) {
      const int i = lane + 32 * t;
      x[t] = (i < k) ? tile[i * kTilePitch + warp] : 0.f;
    }
    // Reflectors of earlier panels, 16 at a time through shared memory (all threads fetch them
    // with row-contiguous reads; every warp then applies them to its column).
    for (int jb = 0; jb < c0; jb += kPanel) {
      for (int e = threadIdx.x; e < kPanel * k; e += kLrThreads) prev[e] = Vn[(size_t)jb * k + e];
      if (threadIdx.x < kPanel) prev_tau[threadIdx.x] = tn[jb + threadIdx.x];
      __syncthreads();
      if (active) {
#pragma unroll 1
        for (int j = 0; j < kPanel; ++j) {
          const float* vj = prev + (size_t)j * k;
          float v[KPL];
          float dot = 0.f;
#pragma unroll
          for (int t = 0; t < KPL; ++t) {
            const int i = lane + 32 * t;
            v[t] = (i < k) ? vj[i] : 0.f;
            dot += v[t] * x[t];
          }
          dot = warp_sum_f(dot) * prev_tau[j];
#pragma unroll
          for (int t = 0; t < KPL; ++t) x[t] -= dot * v[t];
        }
      }
      __syncthreads();
    }
    // Factor the panel.
    for (int jj = 0; jj < kPanel; ++jj) {
      const int cj = c0 + jj;
      if (cj >= r) break;  // uniform over the block
      float* vbuf = vs + (size_t)(jj & 1) * k;
      if (warp == jj) {
        float nrm2 = 0.f, xd = 0.f;
#pragma unroll
        for (int t = 0; t < KPL; ++t) {
          const int i = lane + 32 * t;
          if (i >= cj && i < k) nrm2 += x[t] * x[t];
          if (i == cj) xd = x[t];
        }
        nrm2 = warp_sum_f(nrm2);
        xd = warp_sum_f(xd);  // only one lane contributed
        const float nrm = sqrtf(nrm2);
        const float alpha = (xd >= 0.f) ? -nrm : nrm;
        const float vd = xd - alpha;
        const float vtv = nrm2 - xd * xd + vd * vd;
        const float tau = (vtv > 0.f) ? 2.f / vtv : 0.f;
#pragma unroll
        for (int t = 0; t < KPL; ++t) {
          const int i = lane + 32 * t;
          if (i < k) {
            const float vi = (i < cj) ? 0.f : (i == cj ? vd : x[t]);
            vbuf[i] = vi;
            Vn[(size_t)cj * k + i] = vi;
            if (i == cj) x[t] = alpha;
            else if (i > cj) x[t] = 0.f;
          }
        }
        if (lane == 0) {
          tau_s[jj & 1] = tau;
          tn[cj] = tau;
        }
      }
      __syncthreads();
      if (warp > jj && active) {
        const float tau = tau_s[jj & 1];
        float v[KPL];
        float dot = 0.f;
#pragma unroll
        for (int t = 0; t < KPL; ++t) {
          const int i = lane + 32 * t;
          v[t] = (i < k) ? vbuf[i] : 0.f;
          dot += v[t] * x[t];
        }
        dot = warp_sum_f(dot) * tau;
#pragma unroll
        for (int t = 0; t < KPL; ++t) x[t] -= dot * v[t];
      }
      // vbuf alternates, and the warp that writes it next has passed the barrier above after
      // every reader of the previous use: one barrier per column is enough.
    }
    // The later panels read this panel's reflectors from global memory.
    __threadfence_block();
    __syncthreads();
    // Write the finished columns of R (rows <= column index) through the staging tile.
#pragma unroll
    for (int t = 0; t < KPL; ++t) {
      const int i = lane + 32 * t;
      if (i < k) tile[i * kTilePitch + warp] = x[t];
    }
    __syncthreads();
    const int rows_out = min(r, c0 + kPanel);
    for (int e = threadIdx.x; e < rows_out * kPanel; e += kLrThreads) {
      const int i = e / kPanel, cc = e - i * kPanel;
      if (c0 + cc < r) Rn[(size_t)i * r + c0 + cc] = (i <= c0 + cc) ? tile[i * kTilePitch + cc] : 0.f;
    }
    // Rows below the panel's last column are zero in R.
    for (int e = threadIdx.x; e < (r - rows_out) * kPanel; e += kLrThreads) {
      const int i = rows_out + e / kPanel, cc = e % kPanel;
      if (c0 + cc < r) Rn[(size_t)i * r + c0 + cc] = 0.f;
    }
    __syncthreads();
  }
}

// Upper Cholesky factor U (G = U^T U).  Row j of U is column j of the lower factor, so the rows
// already written to U serve as the earlier columns.  A non-positive pivot yields NaNs in the
// rest of that matrix (as LAPACK's info > 0 would signal); the caller screens for NaNs.
template <int KPL>
__global__ void __launch_bounds__(kLrThreads)
cholesky_upper_kernel(const float* __restrict__ G, float* U, int r) {
  extern __shared__ float lr_smem[];
  float* vs = lr_smem;            // [2][r]
  float* prev = lr_smem + 2 * (size_t)r;  // [16][r] earlier columns
  const int n = blockIdx.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const float* Gn = G + (size_t)n * r * r;
  float* Un = U + (size_t)n * r * r;
  for (int c0 = 0; c0 < r; c0 += kPanel) {
    const int c = c0 + warp;
    const bool active = c < r;
    float x[KPL];
    // Column c of the symmetric input equals its row c: contiguous reads.
#pragma unroll
    for (int t = 0; t < KPL; ++t) {
      const int i = lane + 32 * t;
      x[t] = (active && i < r && i >= c) ? Gn[(size_t)c * r + i] : 0.f;
    }
    // Earlier columns of the factor, 16 at a time through shared memory.
    for (int jb = 0; jb < c0; jb += kPanel) {
      for (int e = threadIdx.x; e < kPanel * r; e += kLrThreads) prev[e] = Un[(size_t)jb * r + e];
      __syncthreads();
      if (active) {
#pragma unroll 2
        for (int j = 0; j < kPanel; ++j) {
          const float* lj = prev + (size_t)j * r;
          const float ljc = lj[c];
#pragma unroll
          for (int t = 0; t < KPL; ++t) {
            const int i = lane + 32 * t;
            if (i < r && i >= c) x[t] -= lj[i] * ljc;
          }
        }
      }
      __syncthreads();
    }
    for (int jj = 0; jj < kPanel; ++jj) {
      const int cj = c0 + jj;
      if (cj >= r) break;
      float* vbuf = vs + (size_t)(jj & 1) * r;
      if (warp == jj) {
        float d = 0.f;
#pragma unroll
        for (int t = 0; t < KPL; ++t)
          if (lane + 32 * t == cj) d = x[t];
        d = warp_sum_f(d);
        const float piv = sqrtf(d);  // NaN for a negative pivot
        const float inv = 1.f / piv;
#pragma unroll
        for (int t = 0; t < KPL; ++t) {
          const int i = lane + 32 * t;
          if (i < r) {
            const float li = (i < cj) ? 0.f : (i == cj ? piv : x[t] * inv);
            vbuf[i] = li;
            Un[(size_t)cj * r + i] = li;
          }
        }
      }
      __syncthreads();
      if (warp > jj && active) {
        const float ljc = vbuf[c];
#pragma unroll
        for (int t = 0; t < KPL; ++t) {
          const int i = lane + 32 * t;
          if (i < r && i >= c) x[t] -= vbuf[i] * ljc;
        }
      }
    }
    __threadfence_block();
    __syncthreads();
  }
}


// ---------------------------------------------------------------------------------------------
// Inverse of upper-triangular matrices (fp32), one CTA per matrix, r <= 1024.
//
// The randomized Cholesky-QR needs P R^-1 twice per step.  With R^-1 in hand that product is an
// ordinary tall GEMM for the tensor cores (lowrank_gemm_sm100.cu) instead of a triangular solve,
// which the reference leaves to cuBLAS trsm (dion/dion.py:1290-1300).
//
// The matrix is cut into 32 x 32 blocks (padded with the identity), warp I owns block row I.
// First every warp inverts its diagonal block (lane l solves for column l by back substitution,
// the column in registers) and keeps it in shared memory.  Then the block super-diagonals are
// filled one after the other: X[I,J] = -inv(U[I,I]) * sum_{K=I+1..J} U[I,K] X[K,J], where every
// X[K,J] on the right lies on an earlier super-diagonal of block column J.  Blocks of one
// super-diagonal are independent (one per warp); a block barrier separates the super-diagonals.
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ float triu_elem(const float* __restrict__ U, int r, int i, int k) {
  if (i < r && k < r) return __ldg(U + (size_t)i * r + k);
  return i == k ? 1.f : 0.f;
}

template <int kMaxThreads>
__global__ void __launch_bounds__(kMaxThreads)
triu_inverse_kernel(const float* __restrict__ Uall, float* Xall, int r) {
  extern __shared__ float ti_smem[];            // [NB][32][32] inverses of the diagonal blocks
  const int NB = blockDim.x >> 5;
  const int I = threadIdx.x >> 5, l = threadIdx.x & 31;
  const float* U = Uall + (size_t)blockIdx.x * r * r;
  float* X = Xall + (size_t)blockIdx.x * r * r;
  float* Ys = ti_smem + (size_t)I * 1024;
  const bool fast = (r & 3) == 0 && (reinterpret_cast<uintptr_t>(U) & 15) == 0;
  const int i0 = I * 32;

  // ---- diagonal block: lane l solves U[I,I] y = e_l ----
  {
    // Stage the block so that row reads below are shared-memory broadcasts.
    for (int i = 0; i < 32; ++i) Ys[i * 32 + l] = triu_elem(U, r, i0 + i, i0 + l);
    __syncwarp();
    float y[32];
#pragma unroll
    for (int i = 31; i >= 0; --i) {
      float s = (i == l) ? 1.f : 0.f;
#pragma unroll
      for (int k = i + 1; k < 32; ++k) s -= Ys[i * 32 + k] * y[k];
      y[i] = s / Ys[i * 32 + i];
    }
    __syncwarp();
#pragma unroll
    for (int i = 0; i < 32; ++i) {
      Ys[i * 32 + l] = y[i];
      if (i0 + i < r && i0 + l < r) X[(size_t)(i0 + i) * r + i0 + l] = y[i];
    }
    // Blocks below the diagonal are zero.
    for (int J = 0; J < I; ++J)
      for (int i = 0; i < 32; ++i)
        if (i0 + i < r) X[(size_t)(i0 + i) * r + J * 32 + l] = 0.f;
  }

  for (int d = 1; d < NB; ++d) {
    __syncthreads();   // the previous super-diagonal (and the diagonal blocks) are in memory
    if (I >= NB - d) continue;
    const int J = I + d, j0 = J * 32;
    float acc[32];
#pragma unroll
    for (int i = 0; i < 32; ++i) acc[i] = 0.f;
    for (int K = I + 1; K <= J; ++K) {
      const int k0 = K * 32;
      float xk[32];
#pragma unroll
      for (int k = 0; k < 32; ++k)
        xk[k] = (k0 + k < r && j0 + l < r) ? X[(size_t)(k0 + k) * r + j0 + l] : 0.f;
      if (fast && k0 + 32 <= r && i0 + 32 <= r) {
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          const float4* urow = reinterpret_cast<const float4*>(U + (size_t)(i0 + i) * r + k0);
#pragma unroll
          for (int q = 0; q < 8; ++q) {
            const float4 u = __ldg(urow + q);
            acc[i] += u.x * xk[q * 4] + u.y * xk[q * 4 + 1] + u.z * xk[q * 4 + 2] +
                      u.w * xk[q * 4 + 3];
          }
        }
      } else {
#pragma unroll
        for (int i = 0; i < 32; ++i) {
#pragma unroll 4
          for (int k = 0; k < 32; ++k) {
            const float u = (i0 + i < r && k0 + k < r) ? __ldg(U + (size_t)(i0 + i) * r + k0 + k)
                                                       : 0.f;
            acc[i] += u * xk[k];
          }
        }
      }
    }
    // X[I,J] = -inv(U[I,I]) * acc
#pragma unroll
    for (int i = 0; i < 32; ++i) {
      float s = 0.f;
      const float4* yrow = reinterpret_cast<const float4*>(Ys + i * 32);
#pragma unroll
      for (int q = 0; q < 8; ++q) {
        const float4 yv = yrow[q];
        s += yv.x * acc[q * 4] + yv.y * acc[q * 4 + 1] + yv.z * acc[q * 4 + 2] +
             yv.w * acc[q * 4 + 3];
      }
      if (i0 + i < r && j0 + l < r) X[(size_t)(i0 + i) * r + j0 + l] = -s;
    }
  }
}


// ---------------------------------------------------------------------------------------------
// Gaussian sketch: out[i] = std * N(0,1), a pure function of (seed, i) - Philox4x32-10 with the
// element index / 4 as counter and Box-Muller on the four outputs - so every replica that derives
// the same seed generates the same sketch without any communication and without a generator
// state (the reference draws it from the framework generator, dion/dion.py:1218-1260).
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ void philox4x32_10(uint32_t c0, uint32_t c1, uint32_t c2, uint32_t c3,
                                              uint32_t k0, uint32_t k1, uint32_t (&out)[4]) {
#pragma unroll
  for (int round = 0; round < 10; ++round) {
    const uint32_t hi0 = __umulhi(0xD2511F53u, c0), lo0 = 0xD2511F53u * c0;
    const uint32_t hi1 = __umulhi(0xCD9E8D57u, c2), lo1 = 0xCD9E8D57u * c2;
    c0 = hi1 ^ c1 ^ k0;
    c1 = lo1;
    c2 = hi0 ^ c3 ^ k1;
    c3 = lo0;
    k0 += 0x9E3779B9u;
    k1 += 0xBB67AE85u;
  }
  out[0] = c0; out[1] = c1; out[2] = c2; out[3] = c3;
}

template <typename T>
__global__ void __launch_bounds__(256)
philox_normal_kernel(T* out, long long n, unsigned long long seed, float std_dev) {
  const long long q = (long long)blockIdx.x * blockDim.x + threadIdx.x;   // group of 4 elements
  const long long i = q * 4;
  if (i >= n) return;
  uint32_t r[4];
  philox4x32_10((uint32_t)q, (uint32_t)(q >> 32), 0u, 0u, (uint32_t)seed, (uint32_t)(seed >> 32),
                r);
  // uniforms in (0, 1]: never zero, so the logarithm is finite
  const float u0 = ((float)(r[0] >> 8) + 1.0f) * (1.0f / 16777216.0f);
  const float u1 = ((float)(r[1] >> 8) + 1.0f) * (1.0f / 16777216.0f);
  const float u2 = ((float)(r[2] >> 8) + 1.0f) * (1.0f / 16777216.0f);
  const float u3 = ((float)(r[3] >> 8) + 1.0f) * (1.0f / 16777216.0f);
  const float ra = std_dev * sqrtf(-2.0f * __logf(u0));
  const float rb = std_dev * sqrtf(-2.0f * __logf(u2));
  float sa, ca, sb, cb;
  __sincosf(6.283185307179586f * u1, &sa, &ca);
  __sincosf(6.283185307179586f * u3, &sb, &cb);
  const float v[4] = {ra * ca, ra * sa, rb * cb, rb * sb};
#pragma unroll
  for (int k = 0; k < 4; ++k)
    if (i + k < n) out[i + k] = static_cast<T>(v[k]);
}

}  // namespace dion

using namespace dion;
static inline cudaStream_t S(void* s) { return static_cast<cudaStream_t>(s); }

template <int KPL>
static int launch_qr(const float* A, float* V, float* tau, float* R, int n, int k, int r,
                     cudaStream_t s) {
  const size_t smem = ((size_t)k * kTilePitch + 2 * (size_t)k + (size_t)kPanel * k) * sizeof(float);
  if (cudaFuncSetAttribute(qr_r_kernel<KPL>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                           (int)smem) != cudaSuccess)
    return -3;
  qr_r_kernel<KPL><<<n, kLrThreads, smem, s>>>(A, V, tau, R, k, r);
  return cudaGetLastError() == cudaSuccess ? 0 : -1;
}

// A: [n][k][r] fp32 (dense).  V: scratch [n][r][k], tau: scratch [n][r], R: out [n][r][r].
// Limits: r <= k <= 1024.
DION_EXPORT int dion_qr_r_factor(const void* A, void* V, void* tau, void* R, int n, int k, int r,
                                 void* stream) {
  if (n <= 0 || r <= 0) return 0;
  if (k < r || k > 1024) return -2;
  const float* a = static_cast<const float*>(A);
  float* v = static_cast<float*>(V);
  float* t = static_cast<float*>(tau);
  float* rr = static_cast<float*>(R);
  if (k <= 256) return launch_qr<8>(a, v, t, rr, n, k, r, S(stream));
  if (k <= 512) return launch_qr<16>(a, v, t, rr, n, k, r, S(stream));
  if (k <= 768) return launch_qr<24>(a, v, t, rr, n, k, r, S(stream));
  return launch_qr<32>(a, v, t, rr, n, k, r, S(stream));
}

template <int KPL>
static int launch_chol(const float* G, float* U, int n, int r, cudaStream_t s) {
  const size_t smem = (2 + kPanel) * (size_t)r * sizeof(float);
  if (cudaFuncSetAttribute(cholesky_upper_kernel<KPL>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                           (int)smem) != cudaSuccess)
    return -3;
  cholesky_upper_kernel<KPL><<<n, kLrThreads, smem, s>>>(G, U, r);
  return cudaGetLastError() == cudaSuccess ? 0 : -1;
}

// G: [n][r][r] fp32 symmetric (only the upper triangle of each row is read), U: out [n][r][r].
// Limit: r <= 1024.
DION_EXPORT int dion_cholesky_upper(const void* G, void* U, int n, int r, void* stream) {
  if (n <= 0 || r <= 0) return 0;
  if (r > 1024) return -2;
  const float* g = static_cast<const float*>(G);
  float* u = static_cast<float*>(U);
  if (r <= 256) return launch_chol<8>(g, u, n, r, S(stream));
  if (r <= 512) return launch_chol<16>(g, u, n, r, S(stream));
  if (r <= 768) return launch_chol<24>(g, u, n, r, S(stream));
  return launch_chol<32>(g, u, n, r, S(stream));
}

// X[b] = U[b]^-1 for a batch of upper-triangular r x r fp32 matrices (r <= 1024); the strictly
// lower triangle of X is written as zero.  X must not alias U.
DION_EXPORT int dion_triu_inverse(const void* U, void* X, int n, int r, void* stream) {
  if (n <= 0 || r <= 0) return 0;
  if (r > 1024 || U == X) return -2;
  const int nb = (r + 31) / 32;
  const int smem = nb * 4096;
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(dion::triu_inverse_kernel<512>,
                             cudaFuncAttributeMaxDynamicSharedMemorySize, 16 * 4096) != cudaSuccess ||
        cudaFuncSetAttribute(dion::triu_inverse_kernel<1024>,
                             cudaFuncAttributeMaxDynamicSharedMemorySize, 32 * 4096) != cudaSuccess)
      return -3;
    configured = true;
  }
  const float* u = static_cast<const float*>(U);
  float* x = static_cast<float*>(X);
  if (nb <= 16)   // up to 512 threads: twice the registers per thread
    dion::triu_inverse_kernel<512><<<n, nb * 32, smem, S(stream)>>>(u, x, r);
  else
    dion::triu_inverse_kernel<1024><<<n, nb * 32, smem, S(stream)>>>(u, x, r);
  return cudaGetLastError() == cudaSuccess ? 0 : -1;
}

// out[i] = std_dev * N(0,1) from (seed, i); dt: 0 = fp32, 1 = bf16.
DION_EXPORT int dion_philox_normal(void* out, long long n, unsigned long long seed, float std_dev,
                                   int dt, void* stream) {
  if (n <= 0) return 0;
  const long long groups = (n + 3) / 4;
  const unsigned blocks = (unsigned)((groups + 255) / 256);
  if (dt == 0)
    dion::philox_normal_kernel<float><<<blocks, 256, 0, S(stream)>>>(
        static_cast<float*>(out), n, seed, std_dev);
  else
    dion::philox_normal_kernel<__nv_bfloat16><<<blocks, 256, 0, S(stream)>>>(
        static_cast<__nv_bfloat16*>(out), n, seed, std_dev);
  return cudaGetLastError() == cudaSuccess ? 0 : -1;
}
