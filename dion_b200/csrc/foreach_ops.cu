// Multi-tensor ("foreach") optimizer kernels for sm_100a.
//
// One launch updates every tensor of a parameter bucket.  The tensors are described by a device
// table of int64: [n, chunk_prefix[n+1], numel[n], ptr_0[n], ptr_1[n], ...]; a block looks up
// its tensor by binary search over chunk_prefix.  Hyper-parameters that a scheduler may change
// (lr, weight decay) are read through device pointers so that a captured CUDA graph sees the
// live value.
//
// These replace the reference's torch.compile'd foreach helpers (dion/muon.py:283-347,
// dion/scalar_opts.py:121-308, dion/dion2.py:666-740, dion/normuon.py:344-399) and the ATen
// fused AdamW it calls.
#include "common.cuh"

namespace dion {

constexpr int kChunk = 4096;    // elements per block
constexpr int kThreads = 256;
static_assert(kChunk == kThreads * 16, "the vector paths read 16 elements per thread and chunk");

enum : int { DT_F32 = 0, DT_BF16 = 1 };

struct Table {
  const long long* raw;
  __device__ __forceinline__ int n() const { return (int)raw[0]; }
  __device__ __forceinline__ const long long* prefix() const { return raw + 1; }
  __device__ __forceinline__ long long numel(int t) const { return raw[1 + (n() + 1) + t]; }
  __device__ __forceinline__ void* ptr(int which, int t) const {
    return reinterpret_cast<void*>(raw[1 + (n() + 1) + n() * (1 + which) + t]);
  }
};

__device__ __forceinline__ int find_tensor(const Table& tb, long long chunk) {
  const long long* pre = tb.prefix();
  int lo = 0, hi = tb.n();
  while (hi - lo > 1) {
    int mid = (lo + hi) >> 1;
    if (pre[mid] <= chunk) lo = mid; else hi = mid;
  }
  return lo;
}

__device__ __forceinline__ float ld(const void* p, int dt, long long i) {
  return dt == DT_F32 ? reinterpret_cast<const float*>(p)[i]
                      : __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p)[i]);
}
__device__ __forceinline__ void st(void* p, int dt, long long i, float v) {
  if (dt == DT_F32) reinterpret_cast<float*>(p)[i] = v;
  else reinterpret_cast<__nv_bfloat16*>(p)[i] = __float2bfloat16_rn(v);
}
__device__ __forceinline__ float round_to(float v, int dt) {
  return dt == DT_F32 ? v : __bfloat162float(__float2bfloat16_rn(v));
}

// 4-wide access.  `vec` says that the pointer is 16-byte (fp32) / 8-byte (bf16) aligned.
__device__ __forceinline__ void ld4(const void* p, int dt, long long i, bool vec, float (&v)[4]) {
  if (vec) {
    if (dt == DT_F32) {
      float4 f = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(p) + i);
      v[0] = f.x; v[1] = f.y; v[2] = f.z; v[3] = f.w;
    } else {
      uint2 u = *reinterpret_cast<const uint2*>(reinterpret_cast<const __nv_bfloat16*>(p) + i);
      float2 a = unpack_bf16x2(u.x), b = unpack_bf16x2(u.y);
      v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y;
    }
  } else {
#pragma unroll
    for (int k = 0; k < 4; ++k) v[k] = ld(p, dt, i + k);
  }
}
__device__ __forceinline__ void st4(void* p, int dt, long long i, bool vec, const float (&v)[4]) {
  if (vec) {
    if (dt == DT_F32) {
      *reinterpret_cast<float4*>(reinterpret_cast<float*>(p) + i) =
          make_float4(v[0], v[1], v[2], v[3]);
    } else {
      *reinterpret_cast<uint2*>(reinterpret_cast<__nv_bfloat16*>(p) + i) =
          make_uint2(pack_bf16x2(v[0], v[1]), pack_bf16x2(v[2], v[3]));
    }
  } else {
#pragma unroll
    for (int k = 0; k < 4; ++k) st(p, dt, i + k, v[k]);
  }
}
__device__ __forceinline__ bool aligned4(const void* p, int dt) {
  return (reinterpret_cast<uintptr_t>(p) & (dt == DT_F32 ? 15 : 7)) == 0;
}

// 8 bf16 elements (16 bytes) at once.
__device__ __forceinline__ void ld8b(const void* p, long long i, float (&v)[8]) {
  const uint4 u = *reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(p) + i);
  const float2 a = unpack_bf16x2(u.x), b = unpack_bf16x2(u.y), c = unpack_bf16x2(u.z),
               d = unpack_bf16x2(u.w);
  v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y; v[4] = c.x; v[5] = c.y; v[6] = d.x; v[7] = d.y;
}
__device__ __forceinline__ void st8b(void* p, long long i, const float (&v)[8]) {
  *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(p) + i) =
      make_uint4(pack_bf16x2(v[0], v[1]), pack_bf16x2(v[2], v[3]), pack_bf16x2(v[4], v[5]),
                 pack_bf16x2(v[6], v[7]));
}
__device__ __forceinline__ bool aligned16(const void* p) {
  return (reinterpret_cast<uintptr_t>(p) & 15) == 0;
}

__device__ __forceinline__ float block_sum(float v) {
  __shared__ float red[kThreads / 32];
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  __syncthreads();
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
  __syncthreads();
  float s = 0.f;
  if (threadIdx.x < kThreads / 32) s = red[threadIdx.x];
  if (threadIdx.x < 32) {
#pragma unroll
    for (int o = 4; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
  }
  return s;  // valid in thread 0
}

// Iterates the 4-element groups of this block's chunk: f(i, count) with count in 1..4.
#define DION_CHUNK_LOOP(tb, ...)                                                        \
  const int t = find_tensor(tb, blockIdx.x);                                            \
  const long long numel = tb.numel(t);                                                  \
  const long long base = ((long long)blockIdx.x - tb.prefix()[t]) * kChunk;             \
  const long long end = (base + kChunk < numel) ? base + kChunk : numel;                \
  for (long long i = base + (long long)threadIdx.x * 4; i < end; i += kThreads * 4) {   \
    const bool full = (i + 4 <= end);                                                   \
    __VA_ARGS__                                                                         \
  }

// ---------------------------------------------------------------------------------------------
// Muon pre-orthogonalize: M = mu*M + G;  U = nesterov ? mu*M + G : M;  U -> bf16 (+ sum of u^2).
// Table pointers: 0=G, 1=M, 2=U(bf16 out).  sumsq (optional): one float per tensor.
// With add_only != 0 computes M += G and U = M (Dion2's accumulate step).
// u_cols > 0: every tensor is a [rows, u_cols] matrix whose U goes into a wider matrix with row
// pitch u_ld (a column block of an assembled matrix, possibly in a peer's memory): element i is
// stored at (i / u_cols) * u_ld + i % u_cols.  u_cols must be a multiple of 8.
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(kThreads)
muon_pre_kernel(const long long* raw, int g_dt, int m_dt, float mu, int nesterov, int add_only,
                float* sumsq, int sumsq_in_table, long long u_cols, long long u_ld) {
  Table tb{raw};
  auto u_index = [&](long long i) -> long long {
    if (u_cols <= 0) return i;
    const long long row = i / u_cols;
    return row * u_ld + (i - row * u_cols);
  };
  float acc = 0.f;
  const void* G;
  void* M;
  void* U;
  {
    const int t0 = find_tensor(tb, blockIdx.x);
    G = tb.ptr(0, t0); M = tb.ptr(1, t0); U = tb.ptr(2, t0);
  }
  const bool vg = aligned4(G, g_dt), vm = aligned4(M, m_dt), vu = aligned4(U, DT_BF16);
  // All-bf16, 16-byte aligned tensors whose size is a multiple of 8: 16-byte accesses, and the
  // loads of both halves of the chunk are issued before either is used.
  if (g_dt == DT_BF16 && m_dt == DT_BF16 && aligned16(G) && aligned16(M) &&
      (U == nullptr || aligned16(U))) {
    const int t = find_tensor(tb, blockIdx.x);
    const long long numel = tb.numel(t);
    if ((numel & 7) == 0) {
      const long long base = ((long long)blockIdx.x - tb.prefix()[t]) * kChunk;
      const long long end = (base + kChunk < numel) ? base + kChunk : numel;
      const long long i0 = base + (long long)threadIdx.x * 8;
      const long long i1 = i0 + kThreads * 8;
      float g0[8], m0[8], g1[8], m1[8];
      const bool h0 = i0 < end, h1 = i1 < end;
      if (h0) { ld8b(G, i0, g0); ld8b(M, i0, m0); }
      if (h1) { ld8b(G, i1, g1); ld8b(M, i1, m1); }
      auto body = [&](float (&g)[8], float (&m)[8], long long i) {
        float u[8];
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          const float gk = g[k];
          float mk = add_only ? (m[k] + gk) : (mu * m[k] + gk);
          mk = round_to(mk, DT_BF16);
          m[k] = mk;
          float uk = (nesterov && !add_only) ? (mu * mk + gk) : mk;
          uk = round_to(uk, DT_BF16);
          u[k] = uk;
          acc += uk * uk;
        }
        st8b(M, i, m);
        if (U) st8b(U, u_index(i), u);
      };
      if (h0) body(g0, m0, i0);
      if (h1) body(g1, m1, i1);
      if (sumsq) {
        const float s = block_sum(acc);
        if (threadIdx.x == 0) atomicAdd(&sumsq[t], s);
      } else if (sumsq_in_table) {
        float* target = reinterpret_cast<float*>(tb.ptr(3, t));
        const float s = block_sum(acc);
        if (threadIdx.x == 0 && target != nullptr) atomicAdd(target, s);
      }
      return;
    }
  }
  DION_CHUNK_LOOP(tb, {
    float g[4], m[4], u[4];
    if (full) {
      ld4(G, g_dt, i, vg, g);
      ld4(M, m_dt, i, vm, m);
    } else {
      for (int k = 0; k < 4; ++k) {
        g[k] = (i + k < end) ? ld(G, g_dt, i + k) : 0.f;
        m[k] = (i + k < end) ? ld(M, m_dt, i + k) : 0.f;
      }
    }
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float gk = round_to(g[k], m_dt);  // the reference casts G to M's dtype first
      float mk = add_only ? (m[k] + gk) : (mu * m[k] + gk);
      mk = round_to(mk, m_dt);
      m[k] = mk;
      float uk = (nesterov && !add_only) ? (mu * mk + gk) : mk;
      uk = round_to(round_to(uk, m_dt), DT_BF16);
      u[k] = uk;
      if (full || i + k < end) acc += uk * uk;
    }
    if (full) {
      st4(M, m_dt, i, vm, m);
      if (U) st4(U, DT_BF16, u_index(i), vu, u);
    } else {
      for (int k = 0; k < 4 && i + k < end; ++k) {
        st(M, m_dt, i + k, m[k]);
        if (U) st(U, DT_BF16, u_index(i + k), u[k]);
      }
    }
  })
  if (sumsq) {
    const float s = block_sum(acc);
    if (threadIdx.x == 0) atomicAdd(&sumsq[t], s);
  } else if (sumsq_in_table) {
    // table pointer 3: where this tensor's partial sum is accumulated (may be peer memory)
    float* target = reinterpret_cast<float*>(tb.ptr(3, t));
    const float s = block_sum(acc);
    if (threadIdx.x == 0 && target != nullptr) atomicAdd(target, s);
  }
}

// ---------------------------------------------------------------------------------------------
// Post-orthogonalize apply: X = X*(1 - lr*wd) - lr*ratio*rescale_t * U * rowscale[r]
// (cautious: decay only where X*U >= 0).  Table pointers: 0=X, 1=U(bf16), 2=rowscale (optional,
// fp32 per row, NorMuon), cols in numel2.  `rescale` (optional) is one float per tensor.
// ---------------------------------------------------------------------------------------------
struct ApplyArgs {
  const float* lr;
  const float* wd_ptr;
  float wd;
  float ratio;      // adjusted_lr / lr
  int cautious;
  int x_dt;
  int cols;         // row length (for rowscale); 0 = unused
  const float* normU2;    // NorMuon: per-tensor ||U||^2 and ||U/denom||^2
  const float* normNew2;
  // U of tensor t was stored into this GPU's memory by rank t / per_rank, which then raised
  // wait_flags[t / per_rank] to *seq_ptr (optional).
  const int* wait_flags;
  const int* seq_ptr;
  int per_rank;
  int* status;
};

__device__ __forceinline__ bool wait_flag_block(const int* flag, int want) {
  __shared__ int ok;
  if (threadIdx.x == 0) {
    ok = flag_wait_bounded(flag, want) ? 1 : 0;
  }
  __syncthreads();
  return ok != 0;
}

__global__ void __launch_bounds__(kThreads)
muon_post_kernel(const long long* raw, const ApplyArgs a) {
  Table tb{raw};
  if (a.wait_flags) {
    // An earlier kernel of this step (or this kernel's wait below) gave up on a peer: the update
    // buffer may be incomplete, so the weights are left exactly as they are.
    if (status_is_set(a.status)) return;
    const int t0 = find_tensor(tb, blockIdx.x);
    const int src = t0 / a.per_rank;
    if (!wait_flag_block(a.wait_flags + src, *a.seq_ptr)) {
      if (threadIdx.x == 0) report_peer_timeout(a.status, src, *a.seq_ptr, a.wait_flags[src]);
      return;
    }
  }
  const float lr = *a.lr;
  const float wd = a.wd_ptr ? *a.wd_ptr : a.wd;
  const float decay = 1.f - lr * wd;
  const float coeff = lr * wd;
  float step = lr * a.ratio;
  void* X; const void* U; const float* rs;
  int tt;
  {
    tt = find_tensor(tb, blockIdx.x);
    X = tb.ptr(0, tt); U = tb.ptr(1, tt); rs = reinterpret_cast<const float*>(tb.ptr(2, tt));
  }
  if (a.normU2) {
    const float nu = sqrtf(a.normU2[tt]);
    const float nn = fmaxf(sqrtf(a.normNew2[tt]), 1e-8f);
    step *= nu / nn;
  }
  const bool vx = aligned4(X, a.x_dt), vu = aligned4(U, DT_BF16);
  if (a.x_dt == DT_BF16 && aligned16(X) && aligned16(U) && (rs == nullptr || (a.cols & 7) == 0)) {
    const long long numel = tb.numel(tt);
    if ((numel & 7) == 0) {
      const long long base = ((long long)blockIdx.x - tb.prefix()[tt]) * kChunk;
      const long long end = (base + kChunk < numel) ? base + kChunk : numel;
      const long long i0 = base + (long long)threadIdx.x * 8;
      const long long i1 = i0 + kThreads * 8;
      float x0[8], u0[8], x1[8], u1[8];
      const bool h0 = i0 < end, h1 = i1 < end;
      if (h0) { ld8b(X, i0, x0); ld8b(U, i0, u0); }
      if (h1) { ld8b(X, i1, x1); ld8b(U, i1, u1); }
      auto body = [&](float (&x)[8], float (&u)[8], long long i) {
        const float rsv = rs ? rs[i / a.cols] : 1.f;
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          const float uk = u[k] * rsv;
          float xk = x[k];
          if (a.cautious) {
            const float prod = xk * uk;
            xk = (prod >= 0.f) ? (xk - xk * coeff) : xk;
          } else {
            xk = xk * decay;
          }
          x[k] = xk - step * uk;
        }
        st8b(X, i, x);
      };
      if (h0) body(x0, u0, i0);
      if (h1) body(x1, u1, i1);
      return;
    }
  }
  DION_CHUNK_LOOP(tb, {
    float x[4], u[4];
    if (full) {
      ld4(X, a.x_dt, i, vx, x);
      ld4(U, DT_BF16, i, vu, u);
    } else {
      for (int k = 0; k < 4; ++k) {
        x[k] = (i + k < end) ? ld(X, a.x_dt, i + k) : 0.f;
        u[k] = (i + k < end) ? ld(U, DT_BF16, i + k) : 0.f;
      }
    }
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      float uk = u[k];
      if (rs) uk *= rs[(i + k) / a.cols];
      float xk = x[k];
      if (a.cautious) {
        const float prod = xk * uk;
        xk = (prod >= 0.f) ? (xk - xk * coeff) : xk;
      } else {
        xk = xk * decay;
      }
      x[k] = xk - step * uk;
    }
    if (full) st4(X, a.x_dt, i, vx, x);
    else for (int k = 0; k < 4 && i + k < end; ++k) st(X, a.x_dt, i + k, x[k]);
  })
}

// ---------------------------------------------------------------------------------------------
// AdamW.  Table pointers: 0=X, 1=G, 2=M, 3=V, 4=step (fp32 scalar per tensor, already advanced).
// Matches ATen's fused AdamW arithmetic: decoupled decay first, lerp for the first moment,
// bias corrections evaluated in double.
// ---------------------------------------------------------------------------------------------
struct AdamArgs {
  const float* lr;
  const float* wd_ptr;
  float wd;
  float beta1, beta2, eps;
  int cautious;
  int x_dt, g_dt, m_dt, v_dt;
  float fixed_step;  // used when the table carries no step pointers (legacy scalar step)
  int has_step;
};

__global__ void adamw_inc_steps_kernel(const long long* raw) {
  Table tb{raw};
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < tb.n()) {
    float* s = reinterpret_cast<float*>(tb.ptr(4, i));
    // Several parameters may share one step tensor: advance each distinct tensor once.
    bool first = true;
    for (int j = 0; j < i; ++j)
      if (tb.ptr(4, j) == s) { first = false; break; }
    if (first) *s += 1.f;
  }
}

__global__ void __launch_bounds__(kThreads)
adamw_kernel(const long long* raw, const AdamArgs a) {
  Table tb{raw};
  void* X; const void* G; void* M; void* V;
  float stepf;
  {
    const int t0 = find_tensor(tb, blockIdx.x);
    X = tb.ptr(0, t0); G = tb.ptr(1, t0); M = tb.ptr(2, t0); V = tb.ptr(3, t0);
    stepf = a.has_step ? *reinterpret_cast<const float*>(tb.ptr(4, t0)) : a.fixed_step;
  }
  const double lr = (double)*a.lr;
  const float wd = a.wd_ptr ? *a.wd_ptr : a.wd;
  const double bc1 = 1.0 - pow((double)a.beta1, (double)stepf);
  const double bc2 = 1.0 - pow((double)a.beta2, (double)stepf);
  const float step_size = (float)(lr / bc1);
  const float bc2_sqrt = (float)sqrt(bc2);
  const float lrf = (float)lr;
  const float w1 = 1.f - a.beta1;
  const bool vx = aligned4(X, a.x_dt), vg = aligned4(G, a.g_dt), vm = aligned4(M, a.m_dt),
             vv = aligned4(V, a.v_dt);
  DION_CHUNK_LOOP(tb, {
    float x[4], g[4], m[4], v[4];
    if (full) {
      ld4(X, a.x_dt, i, vx, x); ld4(G, a.g_dt, i, vg, g);
      ld4(M, a.m_dt, i, vm, m); ld4(V, a.v_dt, i, vv, v);
    } else {
      for (int k = 0; k < 4; ++k) {
        const bool in = i + k < end;
        x[k] = in ? ld(X, a.x_dt, i + k) : 0.f; g[k] = in ? ld(G, a.g_dt, i + k) : 0.f;
        m[k] = in ? ld(M, a.m_dt, i + k) : 0.f; v[k] = in ? ld(V, a.v_dt, i + k) : 0.f;
      }
    }
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float gk = g[k];
      const float mk = m[k] + w1 * (gk - m[k]);
      const float vk = a.beta2 * v[k] + (1.f - a.beta2) * gk * gk;
      float xk = x[k];
      const bool decay_here = !a.cautious || (mk * xk >= 0.f);
      if (decay_here) xk -= lrf * wd * xk;
      const float denom = sqrtf(vk) / bc2_sqrt + a.eps;
      xk -= step_size * mk / denom;
      x[k] = xk; m[k] = mk; v[k] = vk;
    }
    if (full) {
      st4(X, a.x_dt, i, vx, x); st4(M, a.m_dt, i, vm, m); st4(V, a.v_dt, i, vv, v);
    } else {
      for (int k = 0; k < 4 && i + k < end; ++k) {
        st(X, a.x_dt, i + k, x[k]); st(M, a.m_dt, i + k, m[k]); st(V, a.v_dt, i + k, v[k]);
      }
    }
  })
}

// ---------------------------------------------------------------------------------------------
// Lion.  Table pointers: 0=X, 1=G, 2=M.
// ---------------------------------------------------------------------------------------------
struct LionArgs {
  const float* lr;
  const float* wd_ptr;
  float wd;
  float beta1, beta2;
  int cautious;
  int x_dt, g_dt, m_dt;
};

__global__ void __launch_bounds__(kThreads)
lion_kernel(const long long* raw, const LionArgs a) {
  Table tb{raw};
  void* X; const void* G; void* M;
  {
    const int t0 = find_tensor(tb, blockIdx.x);
    X = tb.ptr(0, t0); G = tb.ptr(1, t0); M = tb.ptr(2, t0);
  }
  const float lr = *a.lr;
  const float wd = a.wd_ptr ? *a.wd_ptr : a.wd;
  const float decay = 1.f - lr * wd, coeff = lr * wd;
  const bool vx = aligned4(X, a.x_dt), vg = aligned4(G, a.g_dt), vm = aligned4(M, a.m_dt);
  DION_CHUNK_LOOP(tb, {
    float x[4], g[4], m[4];
    if (full) {
      ld4(X, a.x_dt, i, vx, x); ld4(G, a.g_dt, i, vg, g); ld4(M, a.m_dt, i, vm, m);
    } else {
      for (int k = 0; k < 4; ++k) {
        const bool in = i + k < end;
        x[k] = in ? ld(X, a.x_dt, i + k) : 0.f; g[k] = in ? ld(G, a.g_dt, i + k) : 0.f;
        m[k] = in ? ld(M, a.m_dt, i + k) : 0.f;
      }
    }
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float gk = round_to(g[k], a.m_dt);
      const float d = gk - m[k];
      const float c = m[k] + (1.f - a.beta1) * d;
      const float u = (c > 0.f) ? 1.f : ((c < 0.f) ? -1.f : 0.f);
      m[k] = m[k] + (1.f - a.beta2) * d;
      float xk = x[k];
      if (a.cautious) xk = (u * xk >= 0.f) ? (xk - xk * coeff) : xk;
      else xk *= decay;
      x[k] = xk - lr * u;
    }
    if (full) { st4(X, a.x_dt, i, vx, x); st4(M, a.m_dt, i, vm, m); }
    else for (int k = 0; k < 4 && i + k < end; ++k) {
      st(X, a.x_dt, i + k, x[k]); st(M, a.m_dt, i + k, m[k]);
    }
  })
}

// ---------------------------------------------------------------------------------------------
// Dion2 post-update: x = a*x - b*u[map] with a single rounding, all parameters in one launch.
// Table pointers: 0=X, 1=U (bf16, [k,cols] for row selection / [rows,k] for column selection),
// 2=map (int32; per row for select_rows, per column otherwise; -1 = not selected).
// ---------------------------------------------------------------------------------------------
struct Dion2PostArgs {
  const float* lr;
  const float* wd_ptr;
  float wd;
  float ratio;
  int x_dt;
  int cols;         // row length of X
  int k;            // number of selected slices (row length of U when selecting columns)
  int select_rows;
  const float* normU2;    // optional NorDion2 rescale (per tensor)
  const float* normNew2;
  // As in ApplyArgs: U of tensor t was stored here by rank t / per_rank (optional).
  const int* wait_flags;
  const int* seq_ptr;
  int per_rank;
  int* status;
};

__global__ void __launch_bounds__(kThreads)
dion2_post_kernel(const long long* raw, const Dion2PostArgs a) {
  Table tb{raw};
  if (a.wait_flags) {
    if (status_is_set(a.status)) return;  // see muon_post_kernel
    const int t0 = find_tensor(tb, blockIdx.x);
    const int src = t0 / a.per_rank;
    if (!wait_flag_block(a.wait_flags + src, *a.seq_ptr)) {
      if (threadIdx.x == 0) report_peer_timeout(a.status, src, *a.seq_ptr, a.wait_flags[src]);
      return;
    }
  }
  void* X; const __nv_bfloat16* U; const int* map; const float* rs;
  int tt;
  {
    tt = find_tensor(tb, blockIdx.x);
    X = tb.ptr(0, tt);
    U = reinterpret_cast<const __nv_bfloat16*>(tb.ptr(1, tt));
    map = reinterpret_cast<const int*>(tb.ptr(2, tt));
    rs = reinterpret_cast<const float*>(tb.ptr(3, tt));
  }
  const float lr = *a.lr;
  const float wd = a.wd_ptr ? *a.wd_ptr : a.wd;
  const float ca = 1.f - lr * wd;
  float cb = lr * a.ratio;
  if (a.normU2) cb *= sqrtf(a.normU2[tt]) / fmaxf(sqrtf(a.normNew2[tt]), 1e-8f);
  const bool vx = aligned4(X, a.x_dt);
  const bool vu = aligned4(U, DT_BF16);
  // With a row length that is a multiple of 4 every 4-element group lies in one row: one
  // division and one map lookup per group, and U is read 4 wide.
  const bool row_groups = (a.cols & 3) == 0;
  const bool vmap = (reinterpret_cast<uintptr_t>(map) & 15) == 0;
  DION_CHUNK_LOOP(tb, {
    float x[4];
    if (full) ld4(X, a.x_dt, i, vx, x);
    else for (int k = 0; k < 4; ++k) x[k] = (i + k < end) ? ld(X, a.x_dt, i + k) : 0.f;
    if (row_groups && full) {
      const int r = (int)(i / a.cols), c = (int)(i - (long long)r * a.cols);
      float u[4] = {0.f, 0.f, 0.f, 0.f};
      if (a.select_rows) {
        const int j = map[r];
        if (j >= 0) {
          ld4(U, DT_BF16, (long long)j * a.cols + c, vu, u);
          if (rs) {
            const float s = rs[j];
#pragma unroll
            for (int k = 0; k < 4; ++k) u[k] *= s;
          }
        }
      } else {
        int js[4];
        if (vmap) {
          const int4 jj = *reinterpret_cast<const int4*>(map + c);
          js[0] = jj.x; js[1] = jj.y; js[2] = jj.z; js[3] = jj.w;
        } else {
#pragma unroll
          for (int k = 0; k < 4; ++k) js[k] = map[c + k];
        }
        const __nv_bfloat16* urow = U + (long long)r * a.k;
#pragma unroll
        for (int k = 0; k < 4; ++k)
          if (js[k] >= 0) u[k] = __bfloat162float(urow[js[k]]);
      }
#pragma unroll
      for (int k = 0; k < 4; ++k) x[k] = ca * x[k] - cb * u[k];
    } else {
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const long long e = i + k;
        if (e >= end) break;
        const int r = (int)(e / a.cols), c = (int)(e - (long long)r * a.cols);
        float u = 0.f;
        if (a.select_rows) {
          const int j = map[r];
          if (j >= 0) { u = __bfloat162float(U[(long long)j * a.cols + c]); if (rs) u *= rs[j]; }
        } else {
          const int j = map[c];
          if (j >= 0) u = __bfloat162float(U[(long long)r * a.k + j]);
        }
        x[k] = ca * x[k] - cb * u;
      }
    }
    if (full) st4(X, a.x_dt, i, vx, x);
    else for (int k = 0; k < 4 && i + k < end; ++k) st(X, a.x_dt, i + k, x[k]);
  })
}

// ---------------------------------------------------------------------------------------------
// Dion2 with global selection scope: the update U comes back full-size and exactly zero off the
// selected slices (orthonormal slices have unit norm, so "selected" == "has a non-zero").
//   pass 1  flags[t][slice] = 1 for every slice of U_t that holds a non-zero
//   pass 2  X = (1 - lr*wd)*X - lr*ratio*U ;  M[selected slices] *= ef_decay
// Table pointers: 0=X, 1=M, 2=U(bf16).  Replaces the per-parameter compiled function
// dion/dion2.py:621-659 of the reference with two launches for all parameters.
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(kThreads)
slice_flags_kernel(const long long* raw, int cols, int select_rows, int num_select, int* flags) {
  Table tb{raw};
  const __nv_bfloat16* U;
  {
    const int t0 = find_tensor(tb, blockIdx.x);
    U = reinterpret_cast<const __nv_bfloat16*>(tb.ptr(2, t0));
  }
  const bool vu = aligned4(U, DT_BF16);
  DION_CHUNK_LOOP(tb, {
    float u[4];
    if (full) ld4(U, DT_BF16, i, vu, u);
    else for (int k = 0; k < 4; ++k) u[k] = (i + k < end) ? ld(U, DT_BF16, i + k) : 0.f;
    int* f = flags + (long long)t * num_select;
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      if (u[k] != 0.f) {   // every writer stores the same value: the race is benign
        const long long e = i + k;
        const int r = (int)(e / cols);
        f[select_rows ? r : (int)(e - (long long)r * cols)] = 1;
      }
    }
  })
}

struct MaskedPostArgs {
  const float* lr;
  const float* wd_ptr;
  float wd, ratio, ef_decay;
  int x_dt, m_dt, cols, select_rows, num_select;
  const int* flags;
};

__global__ void __launch_bounds__(kThreads)
dion2_post_masked_kernel(const long long* raw, const MaskedPostArgs a) {
  Table tb{raw};
  void* X; void* M; const __nv_bfloat16* U;
  {
    const int t0 = find_tensor(tb, blockIdx.x);
    X = tb.ptr(0, t0); M = tb.ptr(1, t0);
    U = reinterpret_cast<const __nv_bfloat16*>(tb.ptr(2, t0));
  }
  const float lr = *a.lr;
  const float wd = a.wd_ptr ? *a.wd_ptr : a.wd;
  const float ca = 1.f - lr * wd, cb = lr * a.ratio;
  const bool vx = aligned4(X, a.x_dt), vm = aligned4(M, a.m_dt), vu = aligned4(U, DT_BF16);
  DION_CHUNK_LOOP(tb, {
    const int* f = a.flags + (long long)t * a.num_select;
    float x[4], m[4], u[4];
    if (full) {
      ld4(X, a.x_dt, i, vx, x); ld4(M, a.m_dt, i, vm, m); ld4(U, DT_BF16, i, vu, u);
    } else {
      for (int k = 0; k < 4; ++k) {
        const bool in = i + k < end;
        x[k] = in ? ld(X, a.x_dt, i + k) : 0.f;
        m[k] = in ? ld(M, a.m_dt, i + k) : 0.f;
        u[k] = in ? ld(U, DT_BF16, i + k) : 0.f;
      }
    }
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const long long e = i + k;
      if (e < end) {
        const int r = (int)(e / a.cols);
        const int slice = a.select_rows ? r : (int)(e - (long long)r * a.cols);
        if (f[slice]) m[k] *= a.ef_decay;
      }
      x[k] = ca * x[k] - cb * u[k];
    }
    if (full) {
      st4(X, a.x_dt, i, vx, x); st4(M, a.m_dt, i, vm, m);
    } else {
      for (int k = 0; k < 4 && i + k < end; ++k) {
        st(X, a.x_dt, i + k, x[k]); st(M, a.m_dt, i + k, m[k]);
      }
    }
  })
}

// ---------------------------------------------------------------------------------------------
// NorMuon row statistics over a stacked bf16 update U[n_mats][rows][cols]:
//   rowms = mean(u^2); V = lerp(V, rowms, 1-beta2); rinv[r] = 1/(sqrt(V)+1e-8);
//   normU2[t] += sum(u^2); normNew2[t] += sum(u^2)*rinv^2.
// V pointers come from the table (pointer 0, dtype v_dt, one value per row); `vmap` (optional,
// pointer 1, int64 per U-row) redirects U-row j to V-row vmap[j] (NorDion2 selected rows).
// One warp per row.
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ float sumsq8(const uint4 q) {
  const uint32_t w[4] = {q.x, q.y, q.z, q.w};
  float s = 0.f;
#pragma unroll
  for (int e = 0; e < 4; ++e) { const float2 f = unpack_bf16x2(w[e]); s += f.x * f.x + f.y * f.y; }
  return s;
}

__global__ void __launch_bounds__(kThreads)
normuon_rowstats_kernel(const long long* raw, const __nv_bfloat16* U, int rows, int cols, int v_dt,
                        float beta2, float* rinv, float* normU2, float* normNew2, int n_mats,
                        const int* guard_status) {
  // U came from other GPUs and a wait on them gave up: keep the second-moment state as it is.
  if (status_is_set(guard_status)) return;
  constexpr int kWarps = kThreads / 32;
  __shared__ int s_t[kWarps];
  __shared__ float s_u2[kWarps], s_n2[kWarps];
  Table tb{raw};
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long row_global = (long long)blockIdx.x * kWarps + warp;
  int t = -1;
  float su = 0.f, sn = 0.f;
  if (row_global < (long long)n_mats * rows) {
    t = (int)(row_global / rows);
    const int r = (int)(row_global - (long long)t * rows);
    const __nv_bfloat16* u = U + row_global * cols;
    float s = 0.f;
    if ((cols & 7) == 0 && (reinterpret_cast<uintptr_t>(u) & 15) == 0) {
      // Four independent 16-byte loads per lane are issued before any is consumed: a warp keeps
      // 2 KB in flight, which is what hides the DRAM latency at one warp per row.
      for (int c0 = lane * 8; c0 < cols; c0 += 4 * 256) {
        uint4 q[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int c = c0 + j * 256;
          q[j] = c < cols ? __ldg(reinterpret_cast<const uint4*>(u + c)) : make_uint4(0, 0, 0, 0);
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) s += sumsq8(q[j]);
      }
    } else {
      for (int c = lane; c < cols; c += 32) { float f = __bfloat162float(u[c]); s += f * f; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    if (lane == 0) {
      void* V = tb.ptr(0, t);
      const long long* vmap = reinterpret_cast<const long long*>(tb.ptr(1, t));
      const long long vr = vmap ? vmap[r] : r;
      const float ms = s / (float)cols;
      float v = ld(V, v_dt, vr);
      v = v + (1.f - beta2) * (ms - v);
      const float vst = round_to(v, v_dt);
      st(V, v_dt, vr, vst);
      const float inv = 1.f / (sqrtf(v) + 1e-8f);
      rinv[row_global] = inv;
      su = s;
      sn = s * inv * inv;
    }
  }
  if (lane == 0) { s_t[warp] = t; s_u2[warp] = su; s_n2[warp] = sn; }
  __syncthreads();
  if (threadIdx.x == 0) {
    // One pair of atomics per run of rows of the same matrix (usually one per block) instead of
    // one per row: thousands of rows add into the same two words per matrix.
    int ct = s_t[0];
    float au = s_u2[0], an = s_n2[0];
    for (int w = 1; w < kWarps; ++w) {
      if (s_t[w] == ct) { au += s_u2[w]; an += s_n2[w]; continue; }
      if (ct >= 0) { atomicAdd(&normU2[ct], au); atomicAdd(&normNew2[ct], an); }
      ct = s_t[w]; au = s_u2[w]; an = s_n2[w];
    }
    if (ct >= 0) { atomicAdd(&normU2[ct], au); atomicAdd(&normNew2[ct], an); }
  }
}

// sum of squares per matrix of a contiguous bf16 batch [n][numel] -> out[n] (atomic accumulate)
__global__ void __launch_bounds__(kThreads)
sumsq_kernel(const __nv_bfloat16* X, long long numel, float* out) {
  const int t = blockIdx.y;
  const __nv_bfloat16* x = X + (long long)t * numel;
  float acc = 0.f;
  const long long base = (long long)blockIdx.x * kChunk;
  const long long end = (base + kChunk < numel) ? base + kChunk : numel;
  if ((numel & 7) == 0 && (reinterpret_cast<uintptr_t>(X) & 15) == 0) {
    // kChunk = 16 elements per thread: two 16-byte loads, both issued before use
    const long long i0 = base + (long long)threadIdx.x * 8, i1 = i0 + kThreads * 8;
    const uint4 z = make_uint4(0, 0, 0, 0);
    const uint4 q0 = i0 < end ? __ldg(reinterpret_cast<const uint4*>(x + i0)) : z;
    const uint4 q1 = i1 < end ? __ldg(reinterpret_cast<const uint4*>(x + i1)) : z;
    acc = sumsq8(q0) + sumsq8(q1);
  } else {
    for (long long i = base + threadIdx.x; i < end; i += kThreads) {
      const float f = __bfloat162float(x[i]);
      acc += f * f;
    }
  }
  const float s = block_sum(acc);
  if (threadIdx.x == 0) atomicAdd(&out[t], s);
}

// scale[t] = 1 / (sqrt(sumsq[t]) * mult + eps)
__global__ void finalize_scale_kernel(const float* sumsq, float* scale, int n, float mult,
                                      float eps) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) scale[i] = 1.f / (sqrtf(sumsq[i]) * mult + eps);
}

// ---------------------------------------------------------------------------------------------
// AOL rescaling of a Newton-Schulz input (reference: dion/newton_schulz_triton.py:601-612, seven
// element-wise library passes there): s_i = rsqrt(max(sum_j |A_ij|, eps)) from the Gram matrix
// A = X X^T, then X <- diag(s) X and A <- diag(s) A diag(s).  Two launches: one warp per row of A
// for the scales, one warp per row of X or A for the in-place rescale (16-byte accesses; m and n
// multiples of 8).
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
aol_rowscale_kernel(const __nv_bfloat16* __restrict__ A, int m, long long rows, float eps,
                    float* __restrict__ s) {
  const long long row = (long long)blockIdx.x * 8 + (threadIdx.x >> 5);
  if (row >= rows) return;
  const int lane = threadIdx.x & 31;
  const uint4* p = reinterpret_cast<const uint4*>(A + row * m);
  float acc = 0.f;
  for (int c = lane; c < m / 8; c += 32) {
    const uint4 q = __ldg(p + c);
    const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float2 f = unpack_bf16x2(w[e]);
      acc += fabsf(f.x) + fabsf(f.y);
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  if (lane == 0) s[row] = rsqrtf(fmaxf(acc, eps));
}

__global__ void __launch_bounds__(256)
aol_apply_kernel(__nv_bfloat16* X, int n, __nv_bfloat16* A, int m, long long rows,
                 const float* __restrict__ s) {
  long long row = (long long)blockIdx.x * 8 + (threadIdx.x >> 5);
  if (row >= 2 * rows) return;
  const int lane = threadIdx.x & 31;
  const bool gram = row >= rows;          // second half of the grid: rows of A
  if (gram) row -= rows;
  const float si = s[row];
  const float* sj = s + (row / m) * m;    // scales of this matrix's columns
  uint4* p = reinterpret_cast<uint4*>(gram ? A + row * m : X + row * n);
  const int vecs = (gram ? m : n) / 8;
  for (int c = lane; c < vecs; c += 32) {
    uint4 q = p[c];
    uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      float2 f = unpack_bf16x2(w[e]);
      const float c0 = gram ? si * sj[c * 8 + e * 2] : si;
      const float c1 = gram ? si * sj[c * 8 + e * 2 + 1] : si;
      w[e] = pack_bf16x2(f.x * c0, f.y * c1);
    }
    p[c] = make_uint4(w[0], w[1], w[2], w[3]);
  }
}

}  // namespace dion

using namespace dion;

static inline cudaStream_t S(void* s) { return static_cast<cudaStream_t>(s); }
static inline int rc() { return cudaGetLastError() == cudaSuccess ? 0 : -1; }

DION_EXPORT int dion_muon_pre(const void* table, long long n_chunks, int g_dt, int m_dt, float mu,
                              int nesterov, int add_only, float* sumsq, int sumsq_in_table,
                              long long u_cols, long long u_ld, void* stream) {
  if (n_chunks <= 0) return 0;
  if (u_cols > 0 && ((u_cols & 7) || (u_ld & 7) || u_ld < u_cols)) return -2;
  muon_pre_kernel<<<(unsigned)n_chunks, kThreads, 0, S(stream)>>>(
      static_cast<const long long*>(table), g_dt, m_dt, mu, nesterov, add_only, sumsq,
      sumsq_in_table, u_cols, u_ld);
  return rc();
}

DION_EXPORT int dion_muon_post(const void* table, long long n_chunks, const float* lr,
                               const float* wd_ptr, float wd, float ratio, int cautious, int x_dt,
                               int cols, const float* normU2, const float* normNew2,
                               const int* wait_flags, const int* seq_ptr, int per_rank,
                               int* status, void* stream) {
  if (n_chunks <= 0) return 0;
  ApplyArgs a{lr, wd_ptr, wd, ratio, cautious, x_dt, cols, normU2, normNew2,
              wait_flags, seq_ptr, per_rank > 0 ? per_rank : 1, status};
  muon_post_kernel<<<(unsigned)n_chunks, kThreads, 0, S(stream)>>>(
      static_cast<const long long*>(table), a);
  return rc();
}

DION_EXPORT int dion_adamw(const void* table, long long n_chunks, int n_tensors, const float* lr,
                           const float* wd_ptr, float wd, float beta1, float beta2, float eps,
                           int cautious, int x_dt, int g_dt, int m_dt, int v_dt, int has_step,
                           float fixed_step, void* stream) {
  if (n_chunks <= 0) return 0;
  if (has_step) {
    adamw_inc_steps_kernel<<<(n_tensors + 127) / 128, 128, 0, S(stream)>>>(
        static_cast<const long long*>(table));
  }
  AdamArgs a{lr, wd_ptr, wd, beta1, beta2, eps, cautious, x_dt, g_dt, m_dt, v_dt, fixed_step,
             has_step};
  adamw_kernel<<<(unsigned)n_chunks, kThreads, 0, S(stream)>>>(
      static_cast<const long long*>(table), a);
  return rc();
}

DION_EXPORT int dion_lion(const void* table, long long n_chunks, const float* lr,
                          const float* wd_ptr, float wd, float beta1, float beta2, int cautious,
                          int x_dt, int g_dt, int m_dt, void* stream) {
  if (n_chunks <= 0) return 0;
  LionArgs a{lr, wd_ptr, wd, beta1, beta2, cautious, x_dt, g_dt, m_dt};
  lion_kernel<<<(unsigned)n_chunks, kThreads, 0, S(stream)>>>(static_cast<const long long*>(table),
                                                             a);
  return rc();
}

DION_EXPORT int dion_dion2_post(const void* table, long long n_chunks, const float* lr,
                                const float* wd_ptr, float wd, float ratio, int x_dt, int cols,
                                int k, int select_rows, const float* normU2, const float* normNew2,
                                const int* wait_flags, const int* seq_ptr, int per_rank,
                                int* status, void* stream) {
  if (n_chunks <= 0) return 0;
  Dion2PostArgs a{lr, wd_ptr, wd, ratio, x_dt, cols, k, select_rows, normU2, normNew2,
                  wait_flags, seq_ptr, per_rank > 0 ? per_rank : 1, status};
  dion2_post_kernel<<<(unsigned)n_chunks, kThreads, 0, S(stream)>>>(
      static_cast<const long long*>(table), a);
  return rc();
}

// `flags` is an int32 array [n_tensors, num_select] that this call zeroes and fills.
DION_EXPORT int dion_dion2_post_masked(const void* table, long long n_chunks, int n_tensors,
                                       const float* lr, const float* wd_ptr, float wd, float ratio,
                                       float ef_decay, int x_dt, int m_dt, int cols,
                                       int select_rows, int num_select, int* flags, void* stream) {
  if (n_chunks <= 0) return 0;
  if (cudaMemsetAsync(flags, 0, sizeof(int) * (size_t)n_tensors * num_select, S(stream)) !=
      cudaSuccess)
    return -1;
  slice_flags_kernel<<<(unsigned)n_chunks, kThreads, 0, S(stream)>>>(
      static_cast<const long long*>(table), cols, select_rows, num_select, flags);
  MaskedPostArgs a{lr, wd_ptr, wd, ratio, ef_decay, x_dt, m_dt, cols, select_rows, num_select,
                   flags};
  dion2_post_masked_kernel<<<(unsigned)n_chunks, kThreads, 0, S(stream)>>>(
      static_cast<const long long*>(table), a);
  return rc();
}

DION_EXPORT int dion_normuon_rowstats(const void* table, const void* U, int n_mats, int rows,
                                      int cols, int v_dt, float beta2, float* rinv, float* normU2,
                                      float* normNew2, const int* guard_status, void* stream) {
  const long long total_rows = (long long)n_mats * rows;
  if (total_rows <= 0) return 0;
  const int wpb = kThreads / 32;
  normuon_rowstats_kernel<<<(unsigned)((total_rows + wpb - 1) / wpb), kThreads, 0, S(stream)>>>(
      static_cast<const long long*>(table), static_cast<const __nv_bfloat16*>(U), rows, cols, v_dt,
      beta2, rinv, normU2, normNew2, n_mats, guard_status);
  return rc();
}

DION_EXPORT int dion_sumsq(const void* X, int n, long long numel, float* out, void* stream) {
  if (n <= 0 || numel <= 0) return 0;
  dim3 grid((unsigned)((numel + kChunk - 1) / kChunk), (unsigned)n);
  sumsq_kernel<<<grid, kThreads, 0, S(stream)>>>(static_cast<const __nv_bfloat16*>(X), numel, out);
  return rc();
}

DION_EXPORT int dion_finalize_scale(const float* sumsq, float* scale, int n, float mult, float eps,
                                    void* stream) {
  if (n <= 0) return 0;
  finalize_scale_kernel<<<(n + 127) / 128, 128, 0, S(stream)>>>(sumsq, scale, n, mult, eps);
  return rc();
}

// X: bf16 [B, m, n], A: bf16 [B, m, m] (the Gram matrix of X), s: fp32 scratch [B*m].  In place.
DION_EXPORT int dion_aol_rescale(void* X, void* A, float* s, long long batch, int m, int n,
                                 float eps, void* stream) {
  if (batch <= 0 || m <= 0) return 0;
  if ((m & 7) || (n & 7)) return -2;
  const long long rows = batch * m;
  aol_rowscale_kernel<<<(unsigned)((rows + 7) / 8), 256, 0, S(stream)>>>(
      static_cast<const __nv_bfloat16*>(A), m, rows, eps, s);
  aol_apply_kernel<<<(unsigned)((2 * rows + 7) / 8), 256, 0, S(stream)>>>(
      static_cast<__nv_bfloat16*>(X), n, static_cast<__nv_bfloat16*>(A), m, rows, s);
  return rc();
}
