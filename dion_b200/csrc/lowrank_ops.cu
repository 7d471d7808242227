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
// Inverse of upper-triangular matrices (fp32), r <= 1024.
//
// The randomized Cholesky-QR needs P R^-1 twice per step.  With R^-1 in hand that product is an
// ordinary tall GEMM for the tensor cores (lowrank_gemm_sm100.cu) instead of a triangular solve,
// which the reference leaves to cuBLAS trsm (dion/dion.py:1290-1300).
//
// The matrix is cut into 32 x 32 blocks (padded with the identity).  Block column J of the
// inverse depends on U and on itself only: X[J,J] = inv(U[J,J]) and, going up,
//     X[I,J] = -inv(U[I,I]) * sum_{K=I+1..J} U[I,K] X[K,J].
// Kernel 1 inverts the diagonal blocks (one warp each: lane l solves for column l by back
// substitution, the column in registers) and clears the blocks below the diagonal.  Kernel 2
// runs one CTA of 8 or 16 warps per block column: as soon as X[K,J] is known, every warp adds
// U[I,K] X[K,J] to the sums of the block rows I < K it owns, then the owner of row K-1 finishes
// X[K-1,J] and publishes it through shared memory.  All block columns of all matrices
// run side by side, so a batch of a few matrices still fills the GPU.
// ---------------------------------------------------------------------------------------------
// r is a multiple of 32 here (the host pads other sizes with the identity).
__global__ void __launch_bounds__(32)
triu_diag_inverse_kernel(const float* __restrict__ Uall, float* Xall, int r) {
  __shared__ float D[32 * 32];
  const int I = blockIdx.x, l = threadIdx.x;
  const float* U = Uall + (size_t)blockIdx.y * r * r;
  float* X = Xall + (size_t)blockIdx.y * r * r;
  const int i0 = I * 32;
  for (int i = 0; i < 32; ++i) D[i * 32 + l] = __ldg(U + (size_t)(i0 + i) * r + i0 + l);
  __syncwarp();
  float y[32];
#pragma unroll
  for (int i = 31; i >= 0; --i) {
    float s = (i == l) ? 1.f : 0.f;
#pragma unroll
    for (int k = i + 1; k < 32; ++k) s -= D[i * 32 + k] * y[k];
    y[i] = s / D[i * 32 + i];
  }
#pragma unroll
  for (int i = 0; i < 32; ++i) X[(size_t)(i0 + i) * r + i0 + l] = y[i];
  for (int J = 0; J < I; ++J)     // blocks below the diagonal are zero
    for (int i = 0; i < 32; ++i) X[(size_t)(i0 + i) * r + J * 32 + l] = 0.f;
}

constexpr int kBlkPitch = 36;   // floats per staged block row (16-byte aligned rows)

// acc[i] += sum_k A[i0+i, k0+k] * xk[k] for a 32 x 32 block of the row-major matrix A.  The warp
// first stages the block in its own shared-memory buffer with 32 independent coalesced loads per
// lane (one round trip to L2 instead of a chain of dependent broadcast loads), then multiplies
// from shared memory (16-byte broadcasts).
__device__ __forceinline__ void block_mac(const float* A, int r, int i0, int k0, float* stage,
                                          int lane, const float (&xk)[32], float (&acc)[32]) {
  float tmp[32];
#pragma unroll
  for (int i = 0; i < 32; ++i) tmp[i] = A[(size_t)(i0 + i) * r + k0 + lane];
  __syncwarp();                      // earlier reads of the buffer are done
#pragma unroll
  for (int i = 0; i < 32; ++i) stage[i * kBlkPitch + lane] = tmp[i];
  __syncwarp();
#pragma unroll
  for (int i = 0; i < 32; ++i) {
    const float4* row = reinterpret_cast<const float4*>(stage + i * kBlkPitch);
#pragma unroll
    for (int q = 0; q < 8; ++q) {
      const float4 u = row[q];
      acc[i] += u.x * xk[q * 4] + u.y * xk[q * 4 + 1] + u.z * xk[q * 4 + 2] + u.w * xk[q * 4 + 3];
    }
  }
}

// WARPS x ROWS >= number of block rows: block row I belongs to warp I % WARPS, slot I / WARPS.
// Dynamic shared memory: one 32 x kBlkPitch staging block per warp.
template <int WARPS, int ROWS>
__global__ void __launch_bounds__(WARPS * 32, 1)
triu_column_kernel(const float* __restrict__ Uall, float* Xall, int r) {
  extern __shared__ __align__(16) float tc_smem[];
  __shared__ float Xs[32 * 33];                 // X[K,J], row k at Xs[k*33 ..]
  const int J = blockIdx.x;
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
  float* stage = tc_smem + (size_t)w * 32 * kBlkPitch;
  const float* U = Uall + (size_t)blockIdx.y * r * r;
  float* X = Xall + (size_t)blockIdx.y * r * r;
  const int j0 = J * 32;
  float acc[ROWS][32];
#pragma unroll
  for (int s = 0; s < ROWS; ++s)
#pragma unroll
    for (int i = 0; i < 32; ++i) acc[s][i] = 0.f;

  // X[J,J] was written by the diagonal kernel.
  for (int e = threadIdx.x; e < 1024; e += WARPS * 32) {
    const int k = e >> 5, c = e & 31;
    Xs[k * 33 + c] = X[(size_t)(j0 + k) * r + j0 + c];
  }
  __syncthreads();

  for (int K = J; K >= 1; --K) {
    float xk[32];
#pragma unroll
    for (int k = 0; k < 32; ++k) xk[k] = Xs[k * 33 + l];
    // sums of my block rows I < K
#pragma unroll
    for (int s = 0; s < ROWS; ++s) {
      const int I = s * WARPS + w;
      if (I < K) block_mac(U, r, I * 32, K * 32, stage, l, xk, acc[s]);
    }
    __syncthreads();                             // everybody has read X[K,J]
    const int In = K - 1;                        // next block to finish
    if (In % WARPS == w) {
      // X[In,J] = -inv(U[In,In]) * acc, the inverse read from the diagonal block of X
#pragma unroll
      for (int k = 0; k < 32; ++k) xk[k] = 0.f;  // reused as the output column
#pragma unroll
      for (int s = 0; s < ROWS; ++s)
        if (s == In / WARPS) block_mac(X, r, In * 32, In * 32, stage, l, acc[s], xk);
#pragma unroll
      for (int i = 0; i < 32; ++i) {
        const float v = -xk[i];
        Xs[i * 33 + l] = v;
        X[(size_t)(In * 32 + i) * r + j0 + l] = v;
      }
    }
    __syncthreads();
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


// ---------------------------------------------------------------------------------------------
// Clean-up of the power-iteration factors and the new Q, two launches for a whole batch
// (reference: fix_all_zero_or_nan, local_column_sum_sq, column_normalize and update_Q_matrix_,
// dion/dion.py:1414-1558, a dozen element-wise passes over tensors as large as P and R).
//
//   fix_factor_kernel   X <- all-zero momentum ? fallback (or 0) : nan_to_num(X)   in place, and
//                       optionally the column sums of squares of the result (fp32, atomics)
//   normalize_q_kernel  Q = R / (sqrt(colsq) + eps), written to a stack and, where given, straight
//                       into the per-parameter state tensors
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ float nan_to_num_f(float v) {
  if (v != v) return 0.f;
  if (v == INFINITY) return 3.4028234663852886e38f;
  if (v == -INFINITY) return -3.4028234663852886e38f;
  return v;
}
template <typename T> __device__ __forceinline__ float to_f(T v);
template <> __device__ __forceinline__ float to_f<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f<__nv_bfloat16>(__nv_bfloat16 v) {
  return __bfloat162float(v);
}
template <typename T> __device__ __forceinline__ T from_f(float v);
template <> __device__ __forceinline__ float from_f<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f<__nv_bfloat16>(float v) {
  return __float2bfloat16_rn(v);
}

constexpr int kFixRows = 32;   // rows per block

// X: [batch, rows, cols]; fallback (optional): same shape; sumsq[b] == 0 marks an all-zero
// momentum; colsq (optional): [batch, cols], pre-zeroed.  grid = (ceil(rows/32), batch).
template <typename T>
__global__ void __launch_bounds__(256)
fix_factor_kernel(T* X, const T* fallback, const float* sumsq, int rows, int cols, float* colsq) {
  const int b = blockIdx.y;
  const int r0 = blockIdx.x * kFixRows;
  const int r1 = min(rows, r0 + kFixRows);
  const bool zero = sumsq[b] == 0.f;
  T* x = X + (size_t)b * rows * cols;
  const T* f = fallback ? fallback + (size_t)b * rows * cols : nullptr;
  for (int c = threadIdx.x; c < cols; c += 256) {
    float s = 0.f;
#pragma unroll 8
    for (int r = r0; r < r1; ++r) {
      const size_t e = (size_t)r * cols + c;
      float v;
      if (zero) v = f ? to_f<T>(f[e]) : 0.f;
      else v = nan_to_num_f(to_f<T>(x[e]));
      const T t = from_f<T>(v);
      x[e] = t;
      const float w = to_f<T>(t);
      s += w * w;
    }
    if (colsq) atomicAdd(colsq + (size_t)b * cols + c, s);
  }
}

// q_ptrs (optional): one address per matrix (0 = skip) of a [rows, cols] tensor of dtype q_dt.
template <typename T>
__global__ void __launch_bounds__(256)
normalize_q_kernel(const T* R, const float* colsq, float eps, T* Qstack, const long long* q_ptrs,
                   int q_dt, int rows, int cols) {
  const int b = blockIdx.y;
  const int r0 = blockIdx.x * kFixRows;
  const int r1 = min(rows, r0 + kFixRows);
  const T* x = R + (size_t)b * rows * cols;
  T* q = Qstack + (size_t)b * rows * cols;
  void* state = q_ptrs ? reinterpret_cast<void*>(q_ptrs[b]) : nullptr;
  for (int c = threadIdx.x; c < cols; c += 256) {
    const float inv = 1.f / (sqrtf(colsq[(size_t)b * cols + c]) + eps);
#pragma unroll 8
    for (int r = r0; r < r1; ++r) {
      const size_t e = (size_t)r * cols + c;
      const T t = from_f<T>(to_f<T>(x[e]) * inv);
      q[e] = t;
      if (state) {
        if (q_dt == 0) static_cast<float*>(state)[e] = to_f<T>(t);
        else static_cast<__nv_bfloat16*>(state)[e] = __float2bfloat16_rn(to_f<T>(t));
      }
    }
  }
}


// ---------------------------------------------------------------------------------------------
// Blocked upper Cholesky factor (fp32), one CTA of 16 warps per matrix, r a multiple of 32 up to
// 1024:  G = U^T U.  Right-looking over 32 x 32 blocks, all in the output buffer (which starts as
// a copy of the upper blocks of G):
//   for every block row k:  warp 0 factors the diagonal block in registers (lane l owns column
//                           l; the row being eliminated travels by shuffles) and inverts the
//                           factor;
//                           block row:  U[k,j] = inv(U[k,k])^T G[k,j]          one block per warp
//                           trailing:   G[i,j] -= U[k,i]^T U[k,j], k < i <= j  one block per warp
// Every product is a 32 x 32 x 32 block operation with the left factor staged in the warp's own
// shared-memory buffer and the right factor's column in registers.  A non-positive pivot gives
// NaN, which propagates (the caller's clean-up turns the update into a no-op), as
// torch.linalg.cholesky_ex does not raise either.
// ---------------------------------------------------------------------------------------------
// Copy the 32 x 32 block A[m0.., a0..] of a row-major matrix into the warp's staging buffer
// (32 independent coalesced loads per lane).
__device__ __forceinline__ void stage_block(const float* A, int r, int m0, int a0, float* stage,
                                            int lane) {
  float tmp[32];
#pragma unroll
  for (int m = 0; m < 32; ++m) tmp[m] = A[(size_t)(m0 + m) * r + a0 + lane];
  __syncwarp();
#pragma unroll
  for (int m = 0; m < 32; ++m) stage[m * kBlkPitch + lane] = tmp[m];
  __syncwarp();
}

// acc[a] += sum_m S[m][a] * xm[m]  (S^T times a column) for a staged block S: one row of S per
// m, read as 16-byte broadcasts.
__device__ __forceinline__ void mac_t_staged(const float* stage, const float (&xm)[32],
                                             float (&acc)[32]) {
#pragma unroll
  for (int m = 0; m < 32; ++m) {
    const float4* row = reinterpret_cast<const float4*>(stage + m * kBlkPitch);
    const float x = xm[m];
#pragma unroll
    for (int q = 0; q < 8; ++q) {
      const float4 u = row[q];
      acc[q * 4] += u.x * x;
      acc[q * 4 + 1] += u.y * x;
      acc[q * 4 + 2] += u.z * x;
      acc[q * 4 + 3] += u.w * x;
    }
  }
}

constexpr int kCholWarps = 16;

__global__ void __launch_bounds__(kCholWarps * 32, 1)
cholesky_blocked_kernel(const float* __restrict__ Gall, float* Uall, int r) {
  extern __shared__ __align__(16) float cb_smem[];
  __shared__ __align__(16) float Yk[32 * kBlkPitch];   // inv(U[k,k]), row-major
  const int NB = r >> 5;
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
  float* stage = cb_smem + (size_t)w * 32 * kBlkPitch;
  const float* G = Gall + (size_t)blockIdx.x * r * r;
  float* U = Uall + (size_t)blockIdx.x * r * r;

  // U <- upper blocks of G, zero below.
  for (int e = threadIdx.x; e < r * (r / 4); e += kCholWarps * 32) {
    const int row = e / (r / 4), c4 = e - row * (r / 4);
    const int col = c4 * 4;
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
    if ((col >> 5) >= (row >> 5)) v = *reinterpret_cast<const float4*>(G + (size_t)row * r + col);
    *reinterpret_cast<float4*>(U + (size_t)row * r + col) = v;
  }
  __syncthreads();

  for (int k = 0; k < NB; ++k) {
    const int k0 = k * 32;
    if (w == 0) {
      // ---- factor the diagonal block: lane l owns column l (a[i] = element (i, l)) ----
      float a[32];
#pragma unroll
      for (int i = 0; i < 32; ++i) a[i] = U[(size_t)(k0 + i) * r + k0 + l];
#pragma unroll
      for (int j = 0; j < 32; ++j) {
        const float piv = sqrtf(__shfl_sync(0xffffffffu, a[j], j));   // NaN if not positive
        const float rj = (l >= j) ? a[j] / piv : 0.f;                 // row j of the factor
        a[j] = rj;
#pragma unroll
        for (int i = j + 1; i < 32; ++i) {
          const float rji = __shfl_sync(0xffffffffu, rj, i);
          a[i] -= rji * rj;                                           // meaningful for l >= i
        }
      }
      // write the factor (zero below the diagonal) and stage it for the inversion
#pragma unroll
      for (int i = 0; i < 32; ++i) {
        const float v = (l >= i) ? a[i] : 0.f;
        U[(size_t)(k0 + i) * r + k0 + l] = v;
        stage[i * kBlkPitch + l] = v;
      }
      __syncwarp();
      // ---- invert it: lane l solves R y = e_l by back substitution ----
      float y[32];
      const float* vs = stage;
#pragma unroll
      for (int i = 31; i >= 0; --i) {
        float sacc = (i == l) ? 1.f : 0.f;
#pragma unroll
        for (int m = i + 1; m < 32; ++m) sacc -= vs[i * kBlkPitch + m] * y[m];
        y[i] = sacc / vs[i * kBlkPitch + i];
      }
#pragma unroll
      for (int i = 0; i < 32; ++i) Yk[i * kBlkPitch + l] = y[i];
    }
    __syncthreads();
    // ---- block row: U[k,j] = Yk^T G[k,j] for j > k ----
    for (int j = k + 1 + w; j < NB; j += kCholWarps) {
      const int j0 = j * 32;
      // Without this the 1024 loop-invariant reads of Yk are hoisted out of the loop and spilled.
      asm volatile("" ::: "memory");
      float g[32], acc[32];
#pragma unroll
      for (int m = 0; m < 32; ++m) {
        g[m] = U[(size_t)(k0 + m) * r + j0 + l];
        acc[m] = 0.f;
      }
      mac_t_staged(Yk, g, acc);          // acc[a] = sum_m Yk[m][a] * g[m]
#pragma unroll
      for (int a = 0; a < 32; ++a) U[(size_t)(k0 + a) * r + j0 + l] = acc[a];
    }
    __syncthreads();
    // ---- trailing update: G[i,j] -= U[k,i]^T U[k,j] for k < i <= j ----
    const int nt = NB - k - 1;              // trailing blocks per side
    const int total = nt * (nt + 1) / 2;
    for (int t = w; t < total; t += kCholWarps) {
      // t -> (ii, jj) with ii <= jj over the upper triangle, row by row
      int ii = 0, rem = t;
      while (rem >= nt - ii) { rem -= nt - ii; ++ii; }
      const int i = k + 1 + ii, j = i + rem;
      const int i0 = i * 32, j0 = j * 32;
      stage_block(U, r, k0, i0, stage, l);       // U[k,i]
      float xm[32], acc[32];
#pragma unroll
      for (int m = 0; m < 32; ++m) {
        xm[m] = U[(size_t)(k0 + m) * r + j0 + l];
        acc[m] = 0.f;
      }
      mac_t_staged(stage, xm, acc);
#pragma unroll
      for (int a = 0; a < 32; ++a) U[(size_t)(i0 + a) * r + j0 + l] -= acc[a];
    }
    __syncthreads();
  }
}

// ---------------------------------------------------------------------------------------------
// Panel step of a blocked Householder QR (compact WY form).  One CTA per matrix factors the
// 32-column panel A[j:, j:j+32] in shared memory and leaves
//   * the panel's part of R (upper triangle of its top 32 rows) in A,
//   * V  [kk, 32]: the reflectors, unit lower trapezoidal (kk = k - j rows),
//   * VT [kk, 32] = V T^T, with T the 32 x 32 upper-triangular factor of
//     H_0 ... H_31 = I - V T V^T,
// so that the caller updates the columns to the right of the panel with two products on the
// tensor cores:  W = V^T A[j:, j+32:],  A[j:, j+32:] -= VT W.
// Within a column, lane = panel column: the dot products of column c with the columns to its
// right are taken by all warps over interleaved rows, reduced through shared memory, and the
// rank-one update follows; two block barriers per column.
// ---------------------------------------------------------------------------------------------
constexpr int kQpWarps = 16;
constexpr int kQpPitch = 33;

// Reflector entry (i, a) of the panel held in P: zero above the diagonal, one on it.
__device__ __forceinline__ float qp_v(const float* P, int i, int a) {
  return i > a ? P[i * kQpPitch + a] : (i == a ? 1.f : 0.f);
}

__global__ void __launch_bounds__(kQpWarps * 32, 1)
qr_panel_kernel(float* Aall, long long strideA, int ld, int k, int j, float* Vall, float* VTall,
                float* Vlo_all, float* VTlo_all) {
  extern __shared__ __align__(16) float qp_smem[];
  const int kk = k - j;
  float* P = qp_smem;                               // [kk][33]
  float* part = P + (size_t)kk * kQpPitch;          // [16][32]
  float* wv = part + kQpWarps * 32;                 // [32]  w of the current column
  float* taus = wv + 32;                            // [32]
  float* sc = taus + 32;                            // [32]  1 / (alpha - beta) per column
  float* G = sc + 32;                               // [32][33]  V^T V (strictly upper part used)
  float* T = G + 32 * kQpPitch;                     // [32][33]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  float* A = Aall + (size_t)blockIdx.x * strideA + (size_t)j * ld + j;
  float* V = Vall + (size_t)blockIdx.x * k * 32;
  float* VT = VTall + (size_t)blockIdx.x * k * 32;
  float* Vlo = Vlo_all + (size_t)blockIdx.x * k * 32;
  float* VTlo = VTlo_all + (size_t)blockIdx.x * k * 32;

  for (int i = warp; i < kk; i += kQpWarps) P[i * kQpPitch + lane] = A[(size_t)i * ld + lane];
  for (int e = threadIdx.x; e < 32 * kQpPitch; e += kQpWarps * 32) G[e] = 0.f;
  __syncthreads();

  // Dot products of column 0 with every column, over the rows below the diagonal.
  {
    float acc = 0.f;
    for (int i = 1 + warp; i < kk; i += kQpWarps)
      acc += P[i * kQpPitch] * P[i * kQpPitch + lane];
    part[warp * 32 + lane] = acc;
  }
  __syncthreads();

  for (int c = 0; c < 32; ++c) {
    // part holds d[lane] = sum_{i > c} P[i][c] * P[i][lane]  (lane = c: the squared tail norm)
    if (warp == 0) {
      float d = 0.f;
#pragma unroll
      for (int q = 0; q < kQpWarps; ++q) d += part[q * 32 + lane];
      const float sigma = __shfl_sync(0xffffffffu, d, c);
      const float alpha = P[c * kQpPitch + c];
      float tau = 0.f, scale = 0.f, rcc = alpha;    // tail already zero: H = I (as LAPACK's larfg)
      if (sigma > 0.f) {
        const float beta = -copysignf(sqrtf(alpha * alpha + sigma), alpha);
        tau = (beta - alpha) / beta;
        scale = 1.f / (alpha - beta);
        rcc = beta;
      }
      // w[lane] = tau * v^T A[:, lane] with v = (1, scale * tail)
      const float w = lane > c ? tau * (P[c * kQpPitch + lane] + scale * d) : 0.f;
      wv[lane] = w;
      if (lane > c) P[c * kQpPitch + lane] -= w;    // row c: v_c = 1
      if (lane == c) {
        taus[c] = tau;
        sc[c] = scale;
        P[c * kQpPitch + c] = rcc;
      }
    }
    __syncthreads();
    // Rank-one update of the rows below the diagonal (the reflector's tail stays unscaled in P
    // until the loop is over, so no lane writes what another reads), and in the same pass the
    // dot products for the next column, whose updated entry arrives by a shuffle from its lane.
    const float ws = wv[lane] * sc[c];
    const int cn = (c + 1) & 31;
    float a0 = 0.f, a1 = 0.f;
    int i = c + 1 + warp;
    for (; i + kQpWarps < kk; i += 2 * kQpWarps) {
      float* p0 = P + i * kQpPitch;
      float* p1 = p0 + kQpWarps * kQpPitch;
      const float x0 = p0[c], x1 = p1[c];
      float v0 = p0[lane], v1 = p1[lane];
      if (lane > c) {
        v0 -= x0 * ws;
        v1 -= x1 * ws;
        p0[lane] = v0;
        p1[lane] = v1;
      }
      const float n0 = __shfl_sync(0xffffffffu, v0, cn), n1 = __shfl_sync(0xffffffffu, v1, cn);
      if (i > c + 1) a0 += n0 * v0;
      a1 += n1 * v1;
    }
    if (i < kk) {
      float* p0 = P + i * kQpPitch;
      const float x0 = p0[c];
      float v0 = p0[lane];
      if (lane > c) {
        v0 -= x0 * ws;
        p0[lane] = v0;
      }
      const float n0 = __shfl_sync(0xffffffffu, v0, cn);
      if (i > c + 1) a0 += n0 * v0;
    }
    part[warp * 32 + lane] = a0 + a1;   // read by warp 0 only after the next barrier
    __syncthreads();
  }
  // scale the reflector tails: V[i][a] = P[i][a] * sc[a] for i > a
  {
    const float scl = sc[lane];
    for (int i = 1 + warp; i < kk; i += kQpWarps)
      if (i > lane) P[i * kQpPitch + lane] *= scl;
  }
  __syncthreads();

  // G[a][lane] = sum_i V[i][a] V[i][lane]
  {
    float g[32];
#pragma unroll
    for (int a = 0; a < 32; ++a) g[a] = 0.f;
    for (int i = warp; i < kk; i += kQpWarps) {
      const float vc = qp_v(P, i, lane);
      if (i < 32) {
#pragma unroll
        for (int a = 0; a < 32; ++a) g[a] += qp_v(P, i, a) * vc;
      } else {
#pragma unroll
        for (int a = 0; a < 32; ++a) g[a] += P[i * kQpPitch + a] * vc;
      }
    }
#pragma unroll
    for (int a = 0; a < 32; ++a) atomicAdd(&G[a * kQpPitch + lane], g[a]);
  }
  __syncthreads();
  // T by columns (lane = row a):  T[a][c] = -tau_c * sum_{b = a}^{c-1} T[a][b] G[b][c],  T[c][c] = tau_c
  if (warp == 0) {
    float t[32];
#pragma unroll
    for (int c = 0; c < 32; ++c) {
      float sacc = 0.f;
#pragma unroll
      for (int b = 0; b < 32; ++b)
        if (b < c) sacc += (b >= lane ? t[b] : 0.f) * G[b * kQpPitch + c];
      const float tc = taus[c];
      t[c] = lane < c ? -tc * sacc : (lane == c ? tc : 0.f);
      T[lane * kQpPitch + c] = t[c];
    }
  }
  __syncthreads();
  // V and VT = V T^T to global memory (lane = column a; row a of T in registers)
  {
    float trow[32];
#pragma unroll
    for (int c = 0; c < 32; ++c) trow[c] = T[lane * kQpPitch + c];
    for (int i = warp; i < kk; i += kQpWarps) {
      float acc = 0.f;
      if (i < 32) {
#pragma unroll
        for (int c = 0; c < 32; ++c) acc += qp_v(P, i, c) * trow[c];
      } else {
#pragma unroll
        for (int c = 0; c < 32; ++c) acc += P[i * kQpPitch + c] * trow[c];
      }
      const float vv = qp_v(P, i, lane);
      V[(size_t)(j + i) * 32 + lane] = vv;
      VT[(size_t)(j + i) * 32 + lane] = acc;
      // what a tf32 instruction does not see of them (second and third segment of the products)
      Vlo[(size_t)(j + i) * 32 + lane] = vv - __uint_as_float(__float_as_uint(vv) & 0xFFFFE000u);
      VTlo[(size_t)(j + i) * 32 + lane] = acc - __uint_as_float(__float_as_uint(acc) & 0xFFFFE000u);
    }
  }
  // the panel's part of R back into A (reflectors are not kept there)
  for (int i = warp; i < 32 && i < kk; i += kQpWarps)
    if (lane >= i) A[(size_t)i * ld + lane] = P[i * kQpPitch + lane];
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
  if ((r & 31) == 0 && r >= 64 && G != U && (reinterpret_cast<uintptr_t>(G) & 15) == 0 &&
      (reinterpret_cast<uintptr_t>(U) & 15) == 0) {
    // blocked kernel (the column-by-column kernel below serves the remaining sizes)
    static bool configured = false;
    constexpr int kStage = dion::kCholWarps * 32 * dion::kBlkPitch * 4;
    if (!configured) {
      if (cudaFuncSetAttribute(dion::cholesky_blocked_kernel,
                               cudaFuncAttributeMaxDynamicSharedMemorySize, kStage) != cudaSuccess)
        return -3;
      configured = true;
    }
    dion::cholesky_blocked_kernel<<<n, dion::kCholWarps * 32, kStage, S(stream)>>>(g, u, r);
    return cudaGetLastError() == cudaSuccess ? 0 : -1;
  }
  if (r <= 256) return launch_chol<8>(g, u, n, r, S(stream));
  if (r <= 512) return launch_chol<16>(g, u, n, r, S(stream));
  if (r <= 768) return launch_chol<24>(g, u, n, r, S(stream));
  return launch_chol<32>(g, u, n, r, S(stream));
}

// X[b] = U[b]^-1 for a batch of upper-triangular r x r fp32 matrices, r a multiple of 32 up to
// 1024, 16-byte aligned; the strictly lower triangle of X is written as zero.  X must not alias U.
DION_EXPORT int dion_triu_inverse(const void* U, void* X, int n, int r, void* stream) {
  if (n <= 0 || r <= 0) return 0;
  if (r > 1024 || (r & 31) || U == X || (reinterpret_cast<uintptr_t>(U) & 15) ||
      (reinterpret_cast<uintptr_t>(X) & 15))
    return -2;
  const int nb = r / 32;
  const float* u = static_cast<const float*>(U);
  float* x = static_cast<float*>(X);
  dim3 grid(nb, n);
  dion::triu_diag_inverse_kernel<<<grid, 32, 0, S(stream)>>>(u, x, r);
  static bool configured = false;
  constexpr int kStage16 = 16 * 32 * dion::kBlkPitch * 4;   // 72 KB
  if (!configured) {
    if (cudaFuncSetAttribute(dion::triu_column_kernel<16, 1>,
                             cudaFuncAttributeMaxDynamicSharedMemorySize, kStage16) != cudaSuccess ||
        cudaFuncSetAttribute(dion::triu_column_kernel<16, 2>,
                             cudaFuncAttributeMaxDynamicSharedMemorySize, kStage16) != cudaSuccess)
      return -3;
    configured = true;
  }
  if (nb <= 8)
    dion::triu_column_kernel<8, 1><<<grid, 256, kStage16 / 2, S(stream)>>>(u, x, r);
  else if (nb <= 16)
    dion::triu_column_kernel<16, 1><<<grid, 512, kStage16, S(stream)>>>(u, x, r);
  else
    dion::triu_column_kernel<16, 2><<<grid, 512, kStage16, S(stream)>>>(u, x, r);
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

// dt: 0 = fp32, 1 = bf16 (X, fallback).  See fix_factor_kernel.
DION_EXPORT int dion_fix_factor(void* X, const void* fallback, const float* sumsq, int batch,
                                int rows, int cols, float* colsq, int dt, void* stream) {
  if (batch <= 0 || rows <= 0 || cols <= 0) return 0;
  dim3 grid((rows + dion::kFixRows - 1) / dion::kFixRows, batch);
  if (dt == 0)
    dion::fix_factor_kernel<float><<<grid, 256, 0, S(stream)>>>(
        static_cast<float*>(X), static_cast<const float*>(fallback), sumsq, rows, cols, colsq);
  else
    dion::fix_factor_kernel<__nv_bfloat16><<<grid, 256, 0, S(stream)>>>(
        static_cast<__nv_bfloat16*>(X), static_cast<const __nv_bfloat16*>(fallback), sumsq, rows,
        cols, colsq);
  return cudaGetLastError() == cudaSuccess ? 0 : -1;
}

DION_EXPORT int dion_normalize_q(const void* R, const float* colsq, float eps, void* Qstack,
                                 const void* q_ptrs, int q_dt, int batch, int rows, int cols,
                                 int dt, void* stream) {
  if (batch <= 0 || rows <= 0 || cols <= 0) return 0;
  dim3 grid((rows + dion::kFixRows - 1) / dion::kFixRows, batch);
  if (dt == 0)
    dion::normalize_q_kernel<float><<<grid, 256, 0, S(stream)>>>(
        static_cast<const float*>(R), colsq, eps, static_cast<float*>(Qstack),
        static_cast<const long long*>(q_ptrs), q_dt, rows, cols);
  else
    dion::normalize_q_kernel<__nv_bfloat16><<<grid, 256, 0, S(stream)>>>(
        static_cast<const __nv_bfloat16*>(R), colsq, eps, static_cast<__nv_bfloat16*>(Qstack),
        static_cast<const long long*>(q_ptrs), q_dt, rows, cols);
  return cudaGetLastError() == cudaSuccess ? 0 : -1;
}

// One panel step of the blocked QR on every matrix of A [n][k][ld-pitched rows] (fp32, in
// place): columns j .. j+31, rows j .. k-1.  V, VT and their tf32 remainders Vlo, VTlo:
// [n][k][32] (rows j.. written).
// Limits: j a multiple of 32, j + 32 <= min(k, columns), (k - j) * 33 * 4 bytes + 17 KB of
// shared memory (k - j <= 1580).
DION_EXPORT int dion_qr_panel(void* A, long long strideA, int ld, int n, int k, int j, void* V,
                              void* VT, void* Vlo, void* VTlo, void* stream) {
  if (n <= 0) return 0;
  if (j < 0 || (j & 31) || j + 32 > k || j + 32 > ld) return -2;
  const size_t smem = ((size_t)(k - j) * kQpPitch + kQpWarps * 32 + 96 + 2 * 32 * kQpPitch) *
                      sizeof(float);
  if (smem > 226 * 1024) return -2;
  if (cudaFuncSetAttribute(dion::qr_panel_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                           (int)smem) != cudaSuccess)
    return -3;
  dion::qr_panel_kernel<<<n, kQpWarps * 32, smem, S(stream)>>>(
      static_cast<float*>(A), strideA, ld, k, j, static_cast<float*>(V), static_cast<float*>(VT),
      static_cast<float*>(Vlo), static_cast<float*>(VTlo));
  return cudaGetLastError() == cudaSuccess ? 0 : -1;
}
