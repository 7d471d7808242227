// Fused element-wise kernels of the GPT block and the loss, forward and backward, for sm_100a.
// They take the place of what the reference gets from tracing its model with a compiler
// (models/gpt_model.py:82-124, 171-179, 195-200):
//   * residual add + RMS norm (fp32 residual stream in, bf16 normalised activations out) and its
//     backward, which also folds in the residual-gradient accumulation and the bf16 cast;
//   * rotary embedding + QK RMS norm;
//   * ReLU^2;
//   * cross entropy that reads bf16 logits once and leaves its gradient in their place.
// All of them are bandwidth-bound: 128-bit accesses, fp32 arithmetic, one pass over the data
// (rows are held in registers between the reduction and the write).
#include "common.cuh"

namespace dion {

enum : int { DT_F32 = 0, DT_BF16 = 1 };

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// 8 consecutive elements as floats (callers guarantee 8-element alignment).
__device__ __forceinline__ void load8(const void* p, int dt, long long i, float (&v)[8]) {
  if (dt == DT_F32) {
    const float4* q = reinterpret_cast<const float4*>(reinterpret_cast<const float*>(p) + i);
    float4 a = q[0], b = q[1];
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
  } else {
    uint4 u = *reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(p) + i);
    float2 a = unpack_bf16x2(u.x), b = unpack_bf16x2(u.y), c = unpack_bf16x2(u.z),
           d = unpack_bf16x2(u.w);
    v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y; v[4] = c.x; v[5] = c.y; v[6] = d.x; v[7] = d.y;
  }
}
__device__ __forceinline__ void store8(void* p, int dt, long long i, const float (&v)[8]) {
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

// ---------------------------------------------------------------------------------------------
// (residual add +) RMS norm.  One warp per row.  VPL = 8-element vectors per lane; rows with
// D <= 256*VPL columns stay in registers between the reduction and the store.
//   x_new = X + DELTA (DELTA optional);  Y = x_new * rsqrt(mean(x_new^2) + eps)
// XOUT (optional) receives x_new in X's dtype.
// ---------------------------------------------------------------------------------------------
template <int VPL>
__global__ void __launch_bounds__(256)
rmsnorm_fwd_kernel(const void* X, int x_dt, const void* DELTA, int d_dt, void* XOUT, void* Y,
                   int y_dt, float* rstd, long long rows, int D, float eps) {
  const long long row = (long long)blockIdx.x * 8 + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (row >= rows) return;
  const long long base = row * D;
  const int nvec = D / 8;
  float v[VPL][8];
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < VPL; ++i) {
    const int j = lane + 32 * i;
    if (j < nvec) {
      load8(X, x_dt, base + j * 8, v[i]);
      if (DELTA) {
        float d[8];
        load8(DELTA, d_dt, base + j * 8, d);
#pragma unroll
        for (int e = 0; e < 8; ++e) v[i][e] += d[e];
        if (XOUT) store8(XOUT, x_dt, base + j * 8, v[i]);
      }
#pragma unroll
      for (int e = 0; e < 8; ++e) ss += v[i][e] * v[i][e];
    }
  }
  ss = warp_sum(ss);
  const float r = rsqrtf(ss / (float)D + eps);
  if (lane == 0) rstd[row] = r;
#pragma unroll
  for (int i = 0; i < VPL; ++i) {
    const int j = lane + 32 * i;
    if (j < nvec) {
#pragma unroll
      for (int e = 0; e < 8; ++e) v[i][e] *= r;
      store8(Y, y_dt, base + j * 8, v[i]);
    }
  }
}

// dx = (GX) + r * (dy - xhat * mean(dy * xhat)),  xhat = x * r.
// GX (optional, X's dtype) is the gradient arriving through the residual connection; DX2
// (optional, bf16) receives a second copy of dx for the bf16 branch that produced DELTA.
template <int VPL>
__global__ void __launch_bounds__(256)
rmsnorm_bwd_kernel(const void* X, int x_dt, const void* DY, int dy_dt, const float* rstd,
                   const void* GX, void* DX, void* DX2, long long rows, int D) {
  const long long row = (long long)blockIdx.x * 8 + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (row >= rows) return;
  const long long base = row * D;
  const int nvec = D / 8;
  const float r = rstd[row];
  float x[VPL][8], g[VPL][8], gx[VPL][8];
  float dot = 0.f;
  // All loads of the row (x, dy and the residual-path gradient) are issued before the first use,
  // so one memory latency covers them.
#pragma unroll
  for (int i = 0; i < VPL; ++i) {
    const int j = lane + 32 * i;
    if (j < nvec) {
      load8(X, x_dt, base + j * 8, x[i]);
      load8(DY, dy_dt, base + j * 8, g[i]);
      if (GX) load8(GX, x_dt, base + j * 8, gx[i]);
    }
  }
#pragma unroll
  for (int i = 0; i < VPL; ++i) {
    const int j = lane + 32 * i;
    if (j < nvec) {
#pragma unroll
      for (int e = 0; e < 8; ++e) dot += g[i][e] * x[i][e];
    }
  }
  dot = warp_sum(dot) * r / (float)D;  // mean(dy * xhat)
#pragma unroll
  for (int i = 0; i < VPL; ++i) {
    const int j = lane + 32 * i;
    if (j < nvec) {
      float o[8];
#pragma unroll
      for (int e = 0; e < 8; ++e) o[e] = r * (g[i][e] - x[i][e] * r * dot);
      if (GX) {
#pragma unroll
        for (int e = 0; e < 8; ++e) o[e] += gx[i][e];
      }
      store8(DX, x_dt, base + j * 8, o);
      if (DX2) store8(DX2, DT_BF16, base + j * 8, o);
    }
  }
}

// ---------------------------------------------------------------------------------------------
// RoPE + RMS norm over head_dim for q and k.  Inputs are [B*T, H, D] bf16 with a row stride (so
// slices of a fused projection can be read in place), cos/sin are [T, D/2] bf16, outputs are
// contiguous.  D/16 threads share one head vector: each holds 8 elements of the first half and
// the 8 elements they are rotated with.
// ---------------------------------------------------------------------------------------------
template <int D>
__global__ void __launch_bounds__(256)
rope_qknorm_fwd_kernel(const __nv_bfloat16* Q, const __nv_bfloat16* K, long long in_row_stride,
                       const __nv_bfloat16* COS, const __nv_bfloat16* SIN, __nv_bfloat16* QO,
                       __nv_bfloat16* KO, float* rstd, long long n_vec, int T, int H, float eps) {
  constexpr int HALF = D / 2, TPV = D / 16;
  const long long gid = (long long)blockIdx.x * 256 + threadIdx.x;
  const long long w_raw = gid / TPV;
  const int sub = (int)(gid % TPV);
  const bool valid = w_raw < 2 * n_vec;  // no early exit: the shuffles below need whole warps
  const long long w = valid ? w_raw : 0;
  const bool is_k = w >= n_vec;
  const long long vec = is_k ? w - n_vec : w;
  const long long bt = vec / H;
  const int h = (int)(vec - bt * H);
  const int t = (int)(bt % T);
  const __nv_bfloat16* x = (is_k ? K : Q) + bt * in_row_stride + (long long)h * D;
  __nv_bfloat16* y = (is_k ? KO : QO) + vec * D;
  float x1[8], x2[8], c[8], s[8], y1[8], y2[8];
  load8(x, DT_BF16, sub * 8, x1);
  load8(x, DT_BF16, HALF + sub * 8, x2);
  load8(COS, DT_BF16, (long long)t * HALF + sub * 8, c);
  load8(SIN, DT_BF16, (long long)t * HALF + sub * 8, s);
  float ss = 0.f;
#pragma unroll
  for (int e = 0; e < 8; ++e) {
    y1[e] = x1[e] * c[e] + x2[e] * s[e];
    y2[e] = x2[e] * c[e] - x1[e] * s[e];
    ss += y1[e] * y1[e] + y2[e] * y2[e];
  }
#pragma unroll
  for (int o = TPV / 2; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
  const float r = rsqrtf(ss / (float)D + eps);
  if (!valid) return;
  if (sub == 0) rstd[w] = r;
#pragma unroll
  for (int e = 0; e < 8; ++e) { y1[e] *= r; y2[e] *= r; }
  store8(y, DT_BF16, sub * 8, y1);
  store8(y, DT_BF16, HALF + sub * 8, y2);
}

template <int D>
__global__ void __launch_bounds__(256)
rope_qknorm_bwd_kernel(const __nv_bfloat16* Q, const __nv_bfloat16* K, long long in_row_stride,
                       const __nv_bfloat16* COS, const __nv_bfloat16* SIN,
                       const __nv_bfloat16* DQO, const __nv_bfloat16* DKO, const float* rstd,
                       __nv_bfloat16* DQ, __nv_bfloat16* DK, long long out_row_stride,
                       const __nv_bfloat16* DVI, long long dvi_row_stride, __nv_bfloat16* DVO,
                       long long n_vec, int T, int H) {
  constexpr int HALF = D / 2, TPV = D / 16;
  const long long gid = (long long)blockIdx.x * 256 + threadIdx.x;
  const long long w_raw = gid / TPV;
  const int sub = (int)(gid % TPV);
  const bool valid = w_raw < 2 * n_vec;  // no early exit: the shuffles below need whole warps
  // Optional third section: copy the gradient of v (dense) beside dq and dk (strided rows).
  const bool is_v = DVI != nullptr && w_raw >= 2 * n_vec && w_raw < 3 * n_vec;
  const long long w = valid ? w_raw : 0;
  const bool is_k = w >= n_vec;
  const long long vec = is_k ? w - n_vec : w;
  const long long bt = vec / H;
  const int h = (int)(vec - bt * H);
  const int t = (int)(bt % T);
  const __nv_bfloat16* x = (is_k ? K : Q) + bt * in_row_stride + (long long)h * D;
  const __nv_bfloat16* g = (is_k ? DKO : DQO) + vec * D;
  __nv_bfloat16* dx = (is_k ? DK : DQ) + bt * out_row_stride + (long long)h * D;
  const float r = rstd[w];
  float x1[8], x2[8], c[8], s[8], y1[8], y2[8], g1[8], g2[8];
  load8(x, DT_BF16, sub * 8, x1);
  load8(x, DT_BF16, HALF + sub * 8, x2);
  load8(COS, DT_BF16, (long long)t * HALF + sub * 8, c);
  load8(SIN, DT_BF16, (long long)t * HALF + sub * 8, s);
  load8(g, DT_BF16, sub * 8, g1);
  load8(g, DT_BF16, HALF + sub * 8, g2);
  float dot = 0.f;
#pragma unroll
  for (int e = 0; e < 8; ++e) {
    y1[e] = x1[e] * c[e] + x2[e] * s[e];
    y2[e] = x2[e] * c[e] - x1[e] * s[e];
    dot += g1[e] * y1[e] + g2[e] * y2[e];
  }
#pragma unroll
  for (int o = TPV / 2; o > 0; o >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
  if (is_v) {
    const long long vv = w_raw - 2 * n_vec;
    const long long vbt = vv / H;
    const int vh = (int)(vv - vbt * H);
    const uint4* src = reinterpret_cast<const uint4*>(DVI + vbt * dvi_row_stride + (long long)vh * D);
    uint4* dst = reinterpret_cast<uint4*>(DVO + vbt * out_row_stride + (long long)vh * D);
    dst[sub] = src[sub];
    dst[HALF / 8 + sub] = src[HALF / 8 + sub];
    return;
  }
  if (!valid) return;
  dot = dot * r / (float)D;
  float o1[8], o2[8];
#pragma unroll
  for (int e = 0; e < 8; ++e) {
    const float d1 = r * (g1[e] - y1[e] * r * dot);  // gradient w.r.t. the rotated vector
    const float d2 = r * (g2[e] - y2[e] * r * dot);
    o1[e] = d1 * c[e] - d2 * s[e];
    o2[e] = d1 * s[e] + d2 * c[e];
  }
  store8(dx, DT_BF16, sub * 8, o1);
  store8(dx, DT_BF16, HALF + sub * 8, o2);
}

// ---------------------------------------------------------------------------------------------
// ReLU^2
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
relu2_fwd_kernel(const void* X, void* Y, int dt, long long n8) {
  for (long long i = (long long)blockIdx.x * 256 + threadIdx.x; i < n8;
       i += (long long)gridDim.x * 256) {
    float v[8];
    load8(X, dt, i * 8, v);
#pragma unroll
    for (int e = 0; e < 8; ++e) { const float r = fmaxf(v[e], 0.f); v[e] = r * r; }
    store8(Y, dt, i * 8, v);
  }
}
__global__ void __launch_bounds__(256)
relu2_bwd_kernel(const void* X, const void* DY, void* DX, int dt, long long n8) {
  for (long long i = (long long)blockIdx.x * 256 + threadIdx.x; i < n8;
       i += (long long)gridDim.x * 256) {
    float x[8], g[8];
    load8(X, dt, i * 8, x);
    load8(DY, dt, i * 8, g);
#pragma unroll
    for (int e = 0; e < 8; ++e) g[e] = 2.f * fmaxf(x[e], 0.f) * g[e];
    store8(DX, dt, i * 8, g);
  }
}

// ---------------------------------------------------------------------------------------------
// Cross entropy.  One block per row: online max / sum-of-exponentials in one read, then the
// gradient (softmax - onehot) / count is written over the logits in a second sweep that is served
// from L2.
// ---------------------------------------------------------------------------------------------
__global__ void ce_count_kernel(const long long* tgt, long long n, int ignore_index, float* count) {
  float c = 0.f;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n;
       i += (long long)gridDim.x * blockDim.x)
    c += (tgt[i] != ignore_index) ? 1.f : 0.f;
  c = warp_sum(c);
  if ((threadIdx.x & 31) == 0 && c != 0.f) atomicAdd(count, c);
}

constexpr int kCeThreads = 512;
constexpr float kLog2e = 1.4426950408889634f;
__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// One block per row.  Pass 1: online (max, sum of exp) over 8-element vectors; pass 2 (optional):
// d(loss)/d(logits) = (softmax - onehot) / count written over the logits.  The exponentials are
// taken in base 2 on pre-scaled arguments (one FFMA + one EX2 each); the dtype is a template
// parameter and the target column is patched per vector, not compared per element, because the
// kernel is bound by instruction issue and the special-function unit, not by memory.
template <int DT>
__global__ void __launch_bounds__(kCeThreads)
ce_fwd_bwd_kernel(void* L, const long long* tgt, long long n, int V, long long ld,
                  int ignore_index, float* losses, const float* count, int write_grad) {
  __shared__ float s_m[kCeThreads / 32], s_s[kCeThreads / 32];
  __shared__ float s_lse2;
  const long long row = blockIdx.x;
  const long long base = row * ld;
  const long long target = tgt[row];
  const int nvec = V / 8;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (target == ignore_index) {
    if (threadIdx.x == 0) losses[row] = 0.f;
    if (write_grad) {
      float z[8] = {0, 0, 0, 0, 0, 0, 0, 0};
      for (int j = threadIdx.x; j < nvec; j += kCeThreads) store8(L, DT, base + j * 8, z);
    }
    return;
  }
  // m, s in the base-2 domain: m = max(x) * log2(e), s = sum 2^(x*log2e - m).
  float m = -INFINITY, s = 0.f;
  for (int j = threadIdx.x; j < nvec; j += kCeThreads) {
    float v[8];
    load8(L, DT, base + j * 8, v);
    float vm = v[0];
#pragma unroll
    for (int e = 1; e < 8; ++e) vm = fmaxf(vm, v[e]);
    const float nm = fmaxf(m, vm * kLog2e);
    float acc = 0.f;
#pragma unroll
    for (int e = 0; e < 8; ++e) acc += fast_exp2(fmaf(v[e], kLog2e, -nm));
    s = s * fast_exp2(m - nm) + acc;
    m = nm;
  }
  const float wm = warp_max(m);
  s = warp_sum(m == -INFINITY ? 0.f : s * fast_exp2(m - wm));
  if (lane == 0) { s_m[warp] = wm; s_s[warp] = s; }
  __syncthreads();
  if (warp == 0) {
    float mm = lane < kCeThreads / 32 ? s_m[lane] : -INFINITY;
    float ssum = lane < kCeThreads / 32 ? s_s[lane] : 0.f;
    const float bm = warp_max(mm);
    ssum = warp_sum(mm == -INFINITY ? 0.f : ssum * fast_exp2(mm - bm));
    if (lane == 0) s_lse2 = bm + log2f(ssum);   // log2 of the sum of exp(x)
  }
  __syncthreads();
  const float lse2 = s_lse2;
  if (threadIdx.x == 0) {
    const float xt = DT == DT_F32
                         ? reinterpret_cast<const float*>(L)[base + target]
                         : __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(L)[base + target]);
    losses[row] = lse2 * 0.6931471805599453f - xt;
  }
  if (!write_grad) return;
  __syncthreads();  // the target logit has been read before it is overwritten
  const float inv = 1.f / fmaxf(*count, 1.f);
  const int tj = (int)(target >> 3), te = (int)(target & 7);
  for (int j = threadIdx.x; j < nvec; j += kCeThreads) {
    float v[8];
    load8(L, DT, base + j * 8, v);
#pragma unroll
    for (int e = 0; e < 8; ++e) v[e] = fast_exp2(fmaf(v[e], kLog2e, -lse2)) * inv;
    if (j == tj) {
#pragma unroll
      for (int e = 0; e < 8; ++e)
        if (e == te) v[e] -= inv;
    }
    store8(L, DT, base + j * 8, v);
  }
}

// x *= *scale unless *scale == 1 (every block exits at once in the common case).
__global__ void __launch_bounds__(256)
scale_unless_one_kernel(void* X, int dt, long long n8, const float* scale) {
  const float s = *scale;
  if (s == 1.f) return;
  for (long long i = (long long)blockIdx.x * 256 + threadIdx.x; i < n8;
       i += (long long)gridDim.x * 256) {
    float v[8];
    load8(X, dt, i * 8, v);
#pragma unroll
    for (int e = 0; e < 8; ++e) v[e] *= s;
    store8(X, dt, i * 8, v);
  }
}

}  // namespace dion

using namespace dion;
static inline cudaStream_t S(void* s) { return static_cast<cudaStream_t>(s); }
static inline int rc() { return cudaGetLastError() == cudaSuccess ? 0 : -1; }
static inline unsigned grid_for(long long n8) {
  long long b = (n8 + 255) / 256;
  return (unsigned)(b < 148 * 16 ? (b > 0 ? b : 1) : 148 * 16);
}

#define DION_VPL_DISPATCH(D_, CALL)                              \
  if ((D_) <= 256) { constexpr int VPL = 1; CALL; }              \
  else if ((D_) <= 512) { constexpr int VPL = 2; CALL; }         \
  else if ((D_) <= 768) { constexpr int VPL = 3; CALL; }         \
  else if ((D_) <= 1024) { constexpr int VPL = 4; CALL; }        \
  else if ((D_) <= 2048) { constexpr int VPL = 8; CALL; }        \
  else if ((D_) <= 4096) { constexpr int VPL = 16; CALL; }       \
  else return -3;

// Y = rmsnorm(X + DELTA); DELTA and XOUT may be null (plain RMS norm).  D % 8 == 0, D <= 4096.
DION_EXPORT int dion_rmsnorm_fwd(const void* X, int x_dt, const void* DELTA, int d_dt, void* XOUT,
                                 void* Y, int y_dt, float* rstd, long long rows, int D, float eps,
                                 void* stream) {
  if (rows <= 0) return 0;
  if (D % 8) return -2;
  const unsigned grid = (unsigned)((rows + 7) / 8);
  DION_VPL_DISPATCH(D, (rmsnorm_fwd_kernel<VPL><<<grid, 256, 0, S(stream)>>>(
                           X, x_dt, DELTA, d_dt, XOUT, Y, y_dt, rstd, rows, D, eps)))
  return rc();
}
// DX = GX + rmsnorm_backward(DY); GX and DX2 (bf16 copy of DX) may be null.
DION_EXPORT int dion_rmsnorm_bwd(const void* X, int x_dt, const void* DY, int dy_dt,
                                 const float* rstd, const void* GX, void* DX, void* DX2,
                                 long long rows, int D, void* stream) {
  if (rows <= 0) return 0;
  if (D % 8) return -2;
  const unsigned grid = (unsigned)((rows + 7) / 8);
  DION_VPL_DISPATCH(D, (rmsnorm_bwd_kernel<VPL><<<grid, 256, 0, S(stream)>>>(
                           X, x_dt, DY, dy_dt, rstd, GX, DX, DX2, rows, D)))
  return rc();
}

#define DION_ROPE_DISPATCH(D_, CALL) \
  switch (D_) {                      \
    case 32: { constexpr int DD = 32; CALL; break; }   \
    case 64: { constexpr int DD = 64; CALL; break; }   \
    case 128: { constexpr int DD = 128; CALL; break; } \
    case 256: { constexpr int DD = 256; CALL; break; } \
    default: return -2;              \
  }

DION_EXPORT int dion_rope_qknorm_fwd(const void* Q, const void* K, long long in_row_stride,
                                     const void* COS, const void* SIN, void* QO, void* KO,
                                     float* rstd, int B, int T, int H, int D, float eps,
                                     void* stream) {
  const long long n_vec = (long long)B * T * H;
  if (n_vec <= 0) return 0;
  if (in_row_stride % 8) return -2;
  const long long threads = 2 * n_vec * (D / 16);
  const unsigned grid = (unsigned)((threads + 255) / 256);
  typedef const __nv_bfloat16* CP;
  typedef __nv_bfloat16* P;
  DION_ROPE_DISPATCH(D, (rope_qknorm_fwd_kernel<DD><<<grid, 256, 0, S(stream)>>>(
                            (CP)Q, (CP)K, in_row_stride, (CP)COS, (CP)SIN, (P)QO, (P)KO, rstd,
                            n_vec, T, H, eps)))
  return rc();
}
DION_EXPORT int dion_rope_qknorm_bwd(const void* Q, const void* K, long long in_row_stride,
                                     const void* COS, const void* SIN, const void* DQO,
                                     const void* DKO, const float* rstd, void* DQ, void* DK,
                                     long long out_row_stride, const void* DVI,
                                     long long dvi_row_stride, void* DVO, int B, int T, int H,
                                     int D, void* stream) {
  const long long n_vec = (long long)B * T * H;
  if (n_vec <= 0) return 0;
  if (in_row_stride % 8 || out_row_stride % 8) return -2;
  if (DVI != nullptr && (dvi_row_stride % 8 || dvi_row_stride < (long long)H * D)) return -2;
  if (DVI != nullptr && ((reinterpret_cast<uintptr_t>(DVI) | reinterpret_cast<uintptr_t>(DVO)) & 15))
    return -2;
  const long long threads = (DVI != nullptr ? 3 : 2) * n_vec * (D / 16);
  const unsigned grid = (unsigned)((threads + 255) / 256);
  typedef const __nv_bfloat16* CP;
  typedef __nv_bfloat16* P;
  DION_ROPE_DISPATCH(D, (rope_qknorm_bwd_kernel<DD><<<grid, 256, 0, S(stream)>>>(
                            (CP)Q, (CP)K, in_row_stride, (CP)COS, (CP)SIN, (CP)DQO, (CP)DKO, rstd,
                            (P)DQ, (P)DK, out_row_stride, (CP)DVI, dvi_row_stride, (P)DVO, n_vec,
                            T, H)))
  return rc();
}

DION_EXPORT int dion_relu2_fwd(const void* X, void* Y, int dt, long long n, void* stream) {
  if (n <= 0) return 0;
  relu2_fwd_kernel<<<grid_for(n / 8), 256, 0, S(stream)>>>(X, Y, dt, n / 8);
  return rc();
}
DION_EXPORT int dion_relu2_bwd(const void* X, const void* DY, void* DX, int dt, long long n,
                               void* stream) {
  if (n <= 0) return 0;
  relu2_bwd_kernel<<<grid_for(n / 8), 256, 0, S(stream)>>>(X, DY, DX, dt, n / 8);
  return rc();
}

DION_EXPORT int dion_ce_count(const void* tgt, long long n, int ignore_index, float* count,
                              void* stream) {
  if (n <= 0) return 0;
  const long long blocks = (n + 1023) / 1024;
  ce_count_kernel<<<(unsigned)(blocks < 256 ? blocks : 256), 1024, 0, S(stream)>>>(
      static_cast<const long long*>(tgt), n, ignore_index, count);
  return rc();
}
DION_EXPORT int dion_ce_fwd_bwd(void* L, int dt, const void* tgt, long long n, int V, long long ld,
                                int ignore_index, float* losses, const float* count,
                                int write_grad, void* stream) {
  if (n <= 0) return 0;
  if (V % 8 || ld % 8) return -2;
  if (dt == DT_F32)
    ce_fwd_bwd_kernel<DT_F32><<<(unsigned)n, kCeThreads, 0, S(stream)>>>(
        L, static_cast<const long long*>(tgt), n, V, ld, ignore_index, losses, count, write_grad);
  else
    ce_fwd_bwd_kernel<DT_BF16><<<(unsigned)n, kCeThreads, 0, S(stream)>>>(
        L, static_cast<const long long*>(tgt), n, V, ld, ignore_index, losses, count, write_grad);
  return rc();
}
DION_EXPORT int dion_scale_unless_one(void* X, int dt, long long n, const float* scale,
                                      void* stream) {
  if (n <= 0) return 0;
  scale_unless_one_kernel<<<grid_for(n / 8), 256, 0, S(stream)>>>(X, dt, n / 8, scale);
  return rc();
}
