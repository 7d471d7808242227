// Whole Newton-Schulz iteration of small matrices in ONE launch on sm_100a.
//
// For a batch whose GEMMs have fewer tiles than the GPU has SMs, the 15 launches of a
// five-iteration loop (Gram, polynomial, update per iteration) cost more in launch latency,
// pipeline fill and drain than in arithmetic.  This kernel runs all of them back to back:
//
//     for every (a, b, c):   A  = s^2 X X^T   (X^T X for tall X)      symmetric, half the tiles
//                            B  = b A + c A A                           symmetric
//                            X' = s (a X + B X)   (X B for tall X)
//
// with the input scale s applied in the first iteration only, X and X' ping-ponging between two
// buffers.  The phases are the same tcgen05 GEMMs as in ns_gemm_sm100.cu (128 x 128 tiles, TMA
// producer warp, one MMA thread, four epilogue warps, TMEM accumulators) and are separated by a
// grid-wide barrier: the CTAs are launched cooperatively (all resident), count themselves in on
// a global counter and spin, bounded, until everybody has arrived.  A phase reads what the
// previous one wrote through L2 only: operand tiles by TMA after a proxy fence, the epilogue's
// D operand with ld.global.cg.
//
// The reference has no counterpart; its drivers launch three kernels per iteration
// (dion/newton_schulz_triton.py:526-568).
#include "common.cuh"

namespace dion {

constexpr int PBM = 128, PBN = 128, PBK = 64;
constexpr int kPThreads = 192;
constexpr int kPStages = 6;
constexpr int kPStageBytes = (PBM + PBN) * PBK * 2;   // 32 KB
constexpr int kPDynBytes = kPStages * kPStageBytes + 1024;
constexpr int kMaxPhases = 24;   // eight iterations; keeps the launch parameters under 4 KB

// One GEMM of the loop.  Buffers and tensor maps are referred to by index.
struct Phase {
  int map_a, map_b;      // tensor maps of the operands
  int a_mn, b_mn;        // operand given as [K, rows] (rows contiguous) instead of [rows, K]
  int M, N, K;
  int sym;               // compute tiles on or above the diagonal, mirror the rest
  int d_buf, c_buf;      // buffer indices of the addend (-1: none) and of the output
  float alpha, beta;
  int alpha_pow, beta_pow;   // powers of the per-matrix input scale (first iteration)
  int tiles_per_mat;
  int tile_ofs;          // offset of this phase's (tile_m, tile_n) list in `tiles`
};

struct PersistArgs {
  CUtensorMap maps[8];
  Phase ph[kMaxPhases];
  int n_phases;
  int batch;
  __nv_bfloat16* buf[4];       // X, Xalt, A, Bm
  long long ld[4], stride[4];
  const int2* tiles;
  const float* scale;          // one fp32 per matrix or nullptr
  unsigned int* counter;       // grid barrier, zero at launch; left at zero
  int* status;
};

__device__ __forceinline__ float ipow_p(float s, int p) {
  float r = 1.f;
  for (int i = 0; i < p; ++i) r *= s;
  return r;
}

__device__ __forceinline__ unsigned ld_acquire_gpu_u32(const unsigned* p) {
  unsigned v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

__device__ __forceinline__ uint4 ld_cg_u4(const void* p) {
  uint4 v;
  asm volatile("ld.global.cg.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p)
               : "memory");
  return v;
}
__device__ __forceinline__ float ld_cg_bf16(const __nv_bfloat16* p) {
  unsigned short v;
  asm volatile("ld.global.cg.u16 %0, [%1];" : "=h"(v) : "l"(p) : "memory");
  return __bfloat162float(__ushort_as_bfloat16(v));
}

// Barrier over the four epilogue warps (named barrier 1).
__device__ __forceinline__ void epi_sync() {
  asm volatile("barrier.cta.sync.aligned 1, 128;" ::: "memory");
}

__global__ void __launch_bounds__(kPThreads, 1)
ns_persistent_kernel(const __grid_constant__ PersistArgs p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  __shared__ __align__(8) uint64_t full_bar[kPStages];
  __shared__ __align__(8) uint64_t empty_bar[kPStages];
  __shared__ __align__(8) uint64_t tfull_bar[2];
  __shared__ __align__(8) uint64_t tempty_bar[2];
  __shared__ __align__(8) uint64_t phase_bar;   // "the grid has finished the previous phase"
  __shared__ uint32_t tmem_base_slot;
  __shared__ int grid_ok;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  constexpr uint32_t kTmemCols = 2 * PBN;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kPStages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tfull_bar[a], 1);
      mbar_init(&tempty_bar[a], 4);
    }
    mbar_init(&phase_bar, 1);
    grid_ok = 1;
    fence_barrier_init();
    fence_proxy_async();
    for (int m = 0; m < 8; ++m) prefetch_tmap(&p.maps[m]);
  }
  if (warp == 1) {
    tmem_alloc(&tmem_base_slot, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_base_slot;

  if (warp == 0) {
    // ------------------------------ TMA producer ------------------------------
    if (lane == 0) {
      uint32_t stage = 0, phase = 0;
      bool ok = true;
      for (int ph = 0; ph < p.n_phases && ok; ++ph) {
        const Phase& g = p.ph[ph];
        if (ph > 0) {
          // operands of this phase were written by the previous one, possibly on other SMs
          if (!mbar_wait_bounded(&phase_bar, (ph - 1) & 1)) {
            atomicExch(p.status, kStatusTimeoutEmpty);
            break;
          }
          asm volatile("fence.proxy.async;" ::: "memory");
        }
        const int num_kb = (g.K + PBK - 1) / PBK;
        const int total = g.tiles_per_mat * p.batch;
        const CUtensorMap* ma = &p.maps[g.map_a];
        const CUtensorMap* mb = &p.maps[g.map_b];
        for (int t = blockIdx.x; t < total && ok; t += gridDim.x) {
          const int b = t / g.tiles_per_mat;
          const int2 tt = p.tiles[g.tile_ofs + t - b * g.tiles_per_mat];
          for (int kb = 0; kb < num_kb; ++kb) {
            if (!mbar_wait_bounded(&empty_bar[stage], phase ^ 1)) {
              atomicExch(p.status, kStatusTimeoutEmpty);
              ok = false;
              break;
            }
            uint8_t* sa = smem + stage * kPStageBytes;
            uint8_t* sb = sa + PBM * PBK * 2;
            mbar_expect_tx(&full_bar[stage], kPStageBytes);
            if (!g.a_mn) {
              tma_load_3d(sa, ma, &full_bar[stage], kb * PBK, tt.x * PBM, b);
            } else {
#pragma unroll
              for (int c = 0; c < PBM / 64; ++c)
                tma_load_3d(sa + c * (PBK * 128), ma, &full_bar[stage], tt.x * PBM + c * 64,
                            kb * PBK, b);
            }
            if (!g.b_mn) {
              tma_load_3d(sb, mb, &full_bar[stage], kb * PBK, tt.y * PBN, b);
            } else {
#pragma unroll
              for (int c = 0; c < PBN / 64; ++c)
                tma_load_3d(sb + c * (PBK * 128), mb, &full_bar[stage], tt.y * PBN + c * 64,
                            kb * PBK, b);
            }
            if (++stage == kPStages) {
              stage = 0;
              phase ^= 1;
            }
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer --------------------------------
    if (lane == 0) {
      uint32_t stage = 0, phase = 0;
      uint32_t aslot = 0, aphase = 0;
      bool ok = true;
      for (int ph = 0; ph < p.n_phases && ok; ++ph) {
        const Phase& g = p.ph[ph];
        const int num_kb = (g.K + PBK - 1) / PBK;
        const int total = g.tiles_per_mat * p.batch;
        const uint32_t idesc = make_idesc_bf16(PBM, PBN, g.a_mn, g.b_mn);
        for (int t = blockIdx.x; t < total && ok; t += gridDim.x) {
          if (!mbar_wait_bounded(&tempty_bar[aslot], aphase ^ 1)) {
            atomicExch(p.status, kStatusTimeoutTmemEmpty);
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t d_tmem = tmem_base + aslot * PBN;
          for (int kb = 0; kb < num_kb; ++kb) {
            if (!mbar_wait_bounded(&full_bar[stage], phase)) {
              atomicExch(p.status, kStatusTimeoutFull);
              ok = false;
              break;
            }
            tc_fence_after();
            const uint32_t sa = smem_u32(smem + stage * kPStageBytes);
            const uint32_t sb = sa + PBM * PBK * 2;
#pragma unroll
            for (int k = 0; k < PBK / 16; ++k) {
              const uint64_t da = g.a_mn ? make_smem_desc(sa + k * 2048, PBK * 128, 1024)
                                         : make_smem_desc(sa + k * 32, 16, 1024);
              const uint64_t db = g.b_mn ? make_smem_desc(sb + k * 2048, PBK * 128, 1024)
                                         : make_smem_desc(sb + k * 32, 16, 1024);
              tc_mma_bf16(d_tmem, da, db, idesc, (kb | k) != 0 ? 1u : 0u);
            }
            tc_commit(&empty_bar[stage]);
            if (++stage == kPStages) {
              stage = 0;
              phase ^= 1;
            }
          }
          if (!ok) break;
          tc_commit(&tfull_bar[aslot]);
          aslot ^= 1;
          if (aslot == 0) aphase ^= 1;
        }
      }
    }
  } else {
    // ------------------------------ epilogue ----------------------------------
    const int lane_grp = warp & 3;
    const int row_in_tile = lane_grp * 32 + lane;
    const bool leader = (warp == 2 && lane == 0);
    uint32_t aslot = 0, aphase = 0;
    bool ok = true;
    for (int ph = 0; ph < p.n_phases; ++ph) {
      const Phase& g = p.ph[ph];
      const int total = g.tiles_per_mat * p.batch;
      const long long ldc = p.ld[g.c_buf], sc_ = p.stride[g.c_buf];
      const long long ldd = g.d_buf >= 0 ? p.ld[g.d_buf] : 0;
      const long long sd_ = g.d_buf >= 0 ? p.stride[g.d_buf] : 0;
      for (int t = blockIdx.x; t < total && ok; t += gridDim.x) {
        const int b = t / g.tiles_per_mat;
        const int2 tt = p.tiles[g.tile_ofs + t - b * g.tiles_per_mat];
        if (!mbar_wait_bounded(&tfull_bar[aslot], aphase)) {
          if (lane == 0) atomicExch(p.status, kStatusTimeoutTmemFull);
          ok = false;
          break;
        }
        tc_fence_after();
        float s = 1.f;
        if (p.scale != nullptr && (g.alpha_pow | g.beta_pow)) s = p.scale[b];
        const float alpha = g.alpha * ipow_p(s, g.alpha_pow);
        const float beta = g.beta * ipow_p(s, g.beta_pow);
        const int r = tt.x * PBM + row_in_tile;
        const int warp_row0 = tt.x * PBM + lane_grp * 32;
        const bool row_ok = r < g.M;
        __nv_bfloat16* Cb = p.buf[g.c_buf] + (long long)b * sc_;
        __nv_bfloat16* Crow = Cb + (long long)r * ldc;
        const __nv_bfloat16* Drow =
            g.d_buf >= 0 ? p.buf[g.d_buf] + (long long)b * sd_ + (long long)r * ldd : nullptr;
#pragma unroll 1
        for (int ch = 0; ch < PBN / 32; ++ch) {
          const int c0 = tt.y * PBN + ch * 32;
          if (c0 >= g.N) continue;
          if (g.sym && c0 + 31 < warp_row0) continue;   // wholly below the diagonal
          float v[32];
          tmem_ld_32x32(tmem_base + (static_cast<uint32_t>(lane_grp * 32) << 16) + aslot * PBN +
                            ch * 32,
                        v);
          tmem_ld_wait();
          if (!row_ok) continue;
          const bool full = c0 + 32 <= g.N;
          if (Drow != nullptr) {
            if (full) {
#pragma unroll
              for (int q = 0; q < 4; ++q) {
                const uint4 u = ld_cg_u4(Drow + c0 + q * 8);
                const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                  const float2 f = unpack_bf16x2(w[e]);
                  v[q * 8 + e * 2] = alpha * v[q * 8 + e * 2] + beta * f.x;
                  v[q * 8 + e * 2 + 1] = alpha * v[q * 8 + e * 2 + 1] + beta * f.y;
                }
              }
            } else {
#pragma unroll
              for (int j = 0; j < 32; ++j)
                v[j] = alpha * v[j] + (c0 + j < g.N ? beta * ld_cg_bf16(Drow + c0 + j) : 0.f);
            }
          } else {
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] *= alpha;
          }
          uint32_t pk[16];
#pragma unroll
          for (int j = 0; j < 16; ++j) pk[j] = pack_bf16x2(v[2 * j], v[2 * j + 1]);
          if (full && (!g.sym || c0 >= r)) {
            uint4* cp = reinterpret_cast<uint4*>(Crow + c0);
#pragma unroll
            for (int q = 0; q < 4; ++q)
              cp[q] = make_uint4(pk[q * 4], pk[q * 4 + 1], pk[q * 4 + 2], pk[q * 4 + 3]);
          } else {
#pragma unroll
            for (int j = 0; j < 32; ++j) {
              const int c = c0 + j;
              if (c < g.N && (!g.sym || c >= r)) {
                const uint32_t w = pk[j >> 1];
                reinterpret_cast<uint16_t*>(Crow)[c] = (j & 1) ? (w >> 16) : (w & 0xFFFF);
              }
            }
          }
          if (g.sym) {
#pragma unroll
            for (int j = 0; j < 32; ++j) {
              const int c = c0 + j;
              if (c > r && c < g.N) {
                const uint32_t w = pk[j >> 1];
                reinterpret_cast<uint16_t*>(Cb)[(long long)c * ldc + r] =
                    (j & 1) ? (w >> 16) : (w & 0xFFFF);
              }
            }
          }
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&tempty_bar[aslot]);
        aslot ^= 1;
        if (aslot == 0) aphase ^= 1;
      }
      // ---- end of phase: grid-wide barrier (skipped after the last phase) ----
      if (ph + 1 < p.n_phases) {
        // this thread's stores (generic proxy) are ordered before the TMA reads (async proxy)
        // that other CTAs issue after the barrier
        asm volatile("fence.proxy.async;" ::: "memory");
        epi_sync();                        // every epilogue thread of this CTA has stored
        if (leader) {
          __threadfence();
          atomicAdd(p.counter, 1u);
          const unsigned want = gridDim.x * (unsigned)(ph + 1);
          WaitBudget budget;
          bool arrived = true;
          while (ld_acquire_gpu_u32(p.counter) < want) {
            if (budget.spent()) {
              arrived = false;
              break;
            }
            __nanosleep(32);
          }
          if (!arrived) {
            atomicExch(p.status, kStatusTimeoutGrid);
            grid_ok = 0;
          }
          mbar_arrive(&phase_bar);          // lets the TMA producer start the next phase
        }
        epi_sync();
        if (!grid_ok) ok = false;
        if (!ok) break;
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
  // Leave the barrier counter at zero for the next launch: the last CTA to pass resets it.
  if (threadIdx.x == 0) {
    __threadfence();
    const unsigned done = atomicAdd(p.counter + 1, 1u);
    if (done == gridDim.x - 1) {
      p.counter[0] = 0u;
      p.counter[1] = 0u;
    }
  }
}

// ---------------------------------------------------------------------------------------------
// Host side
// ---------------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFnP)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                   const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                   const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                   CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFnP get_encode_fn_p() {
  static EncodeTiledFnP fn = nullptr;
  if (fn) return fn;
  void* sym = nullptr;
  cudaDriverEntryPointQueryResult qres;
  if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &qres) !=
          cudaSuccess ||
      qres != cudaDriverEntryPointSuccess)
    return nullptr;
  fn = reinterpret_cast<EncodeTiledFnP>(sym);
  return fn;
}

// bf16 [batch, rows, cols] (cols contiguous), box {box_cols, box_rows, 1}, 128-byte swizzle.
static int make_map_p(CUtensorMap* map, const void* ptr, int batch, int rows, int cols,
                      int box_cols, int box_rows) {
  EncodeTiledFnP enc = get_encode_fn_p();
  if (!enc) return -1;
  cuuint64_t dims[3] = {(cuuint64_t)cols, (cuuint64_t)rows, (cuuint64_t)batch};
  cuuint64_t strides[2] = {(cuuint64_t)cols * 2, (cuuint64_t)rows * cols * 2};
  cuuint32_t box[3] = {(cuuint32_t)box_cols, (cuuint32_t)box_rows, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(ptr), dims, strides,
                   box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : -2;
}

}  // namespace dion

// All iterations (a, b, c) = coeffs[3*i .. 3*i+2] of the Newton-Schulz loop on the dense bf16 batch
// X [batch, m, n] in one cooperative launch.  Xalt [batch, m, n], A and Bm [batch, g, g]
// (g = min(m, n)) are work buffers; `counter` points to two zero-initialised unsigned ints in
// device memory that the kernel leaves at zero.  tiles_all: (tile_m, tile_n) pairs in units of
// 128 x 128, first the n_tiles_gg tiles on or above the diagonal of the symmetric g x g products,
// then the n_tiles_mn tiles of the m x n update.  The result lies in Xalt when `iters` is odd, else in X.  Returns 0 on success,
// -20 when the grid cannot be co-resident (the caller then uses the per-GEMM launches).
DION_EXPORT int dion_ns_persistent(void* X, void* Xalt, void* A, void* Bm, int batch, int m, int n,
                                   const float* coeffs, int iters, const float* scale,
                                   const void* tiles_all, int n_tiles_gg, int n_tiles_mn,
                                   unsigned int* counter, int num_sms, int* status,
                                   void* stream) {
  using namespace dion;
  if (batch <= 0 || m <= 0 || n <= 0 || iters <= 0) return 0;
  if (3 * iters > kMaxPhases) return -10;
  if ((m & 7) || (n & 7)) return -10;
  for (void* ptr : {X, Xalt, A, Bm})
    if (reinterpret_cast<uintptr_t>(ptr) & 15) return -10;
  const int tall = m > n;
  const int g = tall ? n : m;
  PersistArgs a;
  // maps: 0 X K-major, 1 X MN-major, 2 Xalt K-major, 3 Xalt MN-major, 4 A K-major, 5 Bm K-major
  if (make_map_p(&a.maps[0], X, batch, m, n, PBK, PBM) != 0) return -12;
  if (make_map_p(&a.maps[1], X, batch, m, n, 64, PBK) != 0) return -12;
  if (make_map_p(&a.maps[2], Xalt, batch, m, n, PBK, PBM) != 0) return -12;
  if (make_map_p(&a.maps[3], Xalt, batch, m, n, 64, PBK) != 0) return -12;
  if (make_map_p(&a.maps[4], A, batch, g, g, PBK, PBM) != 0) return -12;
  if (make_map_p(&a.maps[5], Bm, batch, g, g, PBK, PBM) != 0) return -12;
  a.maps[6] = a.maps[0];
  a.maps[7] = a.maps[0];
  a.buf[0] = static_cast<__nv_bfloat16*>(X);
  a.buf[1] = static_cast<__nv_bfloat16*>(Xalt);
  a.buf[2] = static_cast<__nv_bfloat16*>(A);
  a.buf[3] = static_cast<__nv_bfloat16*>(Bm);
  a.ld[0] = a.ld[1] = n;
  a.stride[0] = a.stride[1] = (long long)m * n;
  a.ld[2] = a.ld[3] = g;
  a.stride[2] = a.stride[3] = (long long)g * g;
  a.batch = batch;
  a.tiles = static_cast<const int2*>(tiles_all);
  a.scale = scale;
  a.counter = counter;
  a.status = status;
  a.n_phases = 3 * iters;
  int max_tiles = 0;
  for (int it = 0; it < iters; ++it) {
    const float ca = coeffs[3 * it], cb = coeffs[3 * it + 1], cc = coeffs[3 * it + 2];
    const int cur = it & 1, nxt = cur ^ 1;   // buffer index of X / X'
    const int p2 = (it == 0 && scale) ? 2 : 0, p1 = (it == 0 && scale) ? 1 : 0;
    Phase& gram = a.ph[3 * it];
    gram = Phase{};
    if (!tall) {  // X [g, K=n] against itself
      gram.map_a = gram.map_b = cur == 0 ? 0 : 2;
      gram.a_mn = gram.b_mn = 0;
      gram.K = n;
    } else {      // X read as [K=m, g] on both sides
      gram.map_a = gram.map_b = cur == 0 ? 1 : 3;
      gram.a_mn = gram.b_mn = 1;
      gram.K = m;
    }
    gram.M = gram.N = g;
    gram.sym = 1;
    gram.d_buf = -1;
    gram.c_buf = 2;
    gram.alpha = 1.f; gram.beta = 0.f; gram.alpha_pow = p2; gram.beta_pow = 0;
    gram.tiles_per_mat = n_tiles_gg; gram.tile_ofs = 0;
    Phase& poly = a.ph[3 * it + 1];
    poly = Phase{};
    poly.map_a = poly.map_b = 4;
    poly.M = poly.N = poly.K = g;
    poly.sym = 1;
    poly.d_buf = 2; poly.c_buf = 3;
    poly.alpha = cc; poly.beta = cb;
    poly.tiles_per_mat = n_tiles_gg; poly.tile_ofs = 0;
    Phase& upd = a.ph[3 * it + 2];
    upd = Phase{};
    if (!tall) {  // X' = a X + B X, X given as [K, N]
      upd.map_a = 5; upd.a_mn = 0;
      upd.map_b = cur == 0 ? 1 : 3; upd.b_mn = 1;
    } else {      // X' = a X + X B, B symmetric: given as [N, K]
      upd.map_a = cur == 0 ? 0 : 2; upd.a_mn = 0;
      upd.map_b = 5; upd.b_mn = 0;
    }
    upd.M = m; upd.N = n; upd.K = g;
    upd.sym = 0;
    upd.d_buf = cur; upd.c_buf = nxt;
    upd.alpha = 1.f; upd.beta = ca; upd.alpha_pow = p1; upd.beta_pow = p1;
    upd.tiles_per_mat = n_tiles_mn; upd.tile_ofs = n_tiles_gg;
    const int tg = n_tiles_gg * batch, tm = n_tiles_mn * batch;
    if (tg > max_tiles) max_tiles = tg;
    if (tm > max_tiles) max_tiles = tm;
  }
  static bool configured = false;
  static int max_blocks = 0;
  if (!configured) {
    if (cudaFuncSetAttribute(ns_persistent_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             kPDynBytes) != cudaSuccess)
      return -3;
    int per_sm = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, ns_persistent_kernel, kPThreads,
                                                      kPDynBytes) != cudaSuccess || per_sm < 1)
      return -20;
    max_blocks = per_sm * num_sms;
    configured = true;
  }
  int grid = max_tiles < num_sms ? max_tiles : num_sms;
  if (grid > max_blocks) grid = max_blocks;
  if (grid <= 0) return 0;
  void* kargs[] = {&a};
  cudaError_t e = cudaLaunchCooperativeKernel(reinterpret_cast<void*>(ns_persistent_kernel),
                                              dim3(grid), dim3(kPThreads), kargs, kPDynBytes,
                                              static_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) {
    cudaGetLastError();
    return e == cudaErrorCooperativeLaunchTooLarge ? -20 : -4;
  }
  return 0;
}
