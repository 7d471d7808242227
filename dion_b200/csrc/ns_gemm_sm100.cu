// Batched bf16 GEMM for the Newton-Schulz family on sm_100a:
//
//     C[b] = alpha * s_b^pa * A[b] * op(B[b]) + beta * s_b^pb * D[b]
//
// A is [M,K] K-contiguous.  B is either [N,K] K-contiguous ("NT") or [K,N]
// N-contiguous ("NN", read as an MN-major tcgen05 operand, so that
// X' = a*X + B*X needs no transposed copy of X).  With `sym` only the tiles that
// touch the upper triangle are computed and every element above the diagonal is
// also stored at its mirrored position, so the output is exactly symmetric and
// costs about half the MMA work.  This is the role played by the three Triton
// kernels in the reference (dion/newton_schulz_triton.py:83-157, 201-287, 379-447)
// and by cuBLAS baddbmm in its drivers (:557-563).
//
// Structure: persistent CTAs, one per SM.  Warp 0 feeds a multi-stage shared
// memory ring with TMA (128-byte swizzle, no multicast); warp 1 issues
// tcgen05.mma (128xBNx16, fp32 accumulators in TMEM, two accumulator slots);
// warps 2-5 drain TMEM with tcgen05.ld, apply the epilogue and store.  While the
// epilogue drains slot k the MMA warp already fills slot k^1.
#include "common.cuh"
#include "tmap_cache.h"

namespace dion {

constexpr int BM = 128;
constexpr int BK = 64;
constexpr int kNumThreads = 192;

struct GemmArgs {
  int batch, M, N, K;
  const __nv_bfloat16* D;
  long long ldd, strideD;
  __nv_bfloat16* C;
  long long ldc, strideC;
  __nv_bfloat16* CT;  // optional transposed copy of C ([N,M] per batch)
  long long ldct, strideCT;
  float* Cf;  // optional fp32 output instead of C (same ld/stride in elements)
  float alpha, beta;
  const float* scale;  // optional per-batch scalar
  int alpha_pow, beta_pow;
  int sym;
  const int2* tiles;  // (tile_m, tile_n) pairs of one matrix
  int tiles_per_mat;
  int total_tiles;
  int* status;
  // ---- optional coupling to other GPUs (all-to-all fused into the kernel) ----
  // Rows [s*rows_per_src, (s+1)*rows_per_src) of the gated operands were written into this GPU's
  // memory by rank s, which then set wait_flags[s] to the current sequence number.  The TMA
  // producer polls the flags of the sources a tile needs before it loads the tile.
  const int* wait_flags;
  const int* seq_ptr;
  int n_src;
  int rows_per_src;
  int wait_a, wait_b, wait_k;
  // scale = 1 / (sqrt(sum_s scale_partials[b*n_src + s]) * scale_mult + scale_eps): the
  // Frobenius norm assembled from per-source partial sums that travel with the data.
  const float* scale_partials;
  float scale_mult, scale_eps;
  // Output rows scattered to their owners: row r of batch b is stored at
  // remote_c[r / rows_per_dst] + ((remote_slot + b) * rows_per_dst + r % rows_per_dst) * ldc.
  long long remote_c[8];
  int rows_per_dst;
  int remote_slot;
  // cols_per_dst > 0: the output is split by columns instead: element (r, c) of matrix b goes to
  // remote_c[c / cols_per_dst] + ((remote_slot + b) * M + r) * cols_per_dst + c % cols_per_dst
  // (cols_per_dst a multiple of 32, so a 32-column chunk has one destination).
  int cols_per_dst;
};

__device__ __forceinline__ int ld_acquire_sys(const int* p) {
  int v;
  asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ float ld_volatile_f32(const float* p) {
  float v;
  asm volatile("ld.volatile.global.f32 %0, [%1];" : "=f"(v) : "l"(p) : "memory");
  return v;
}
// Waits until flag >= seq; false once the wait budget is spent.
__device__ __forceinline__ bool wait_flag_bounded(const int* flag, int seq) {
  return flag_wait_bounded(flag, seq);
}

template <int BN>
struct SmemLayout {
  static constexpr int kABytes = BM * BK * 2;
  static constexpr int kBBytes = BN * BK * 2;
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kStages = (BN == 256) ? 4 : 6;
  static constexpr int kDynBytes = kStages * kStageBytes + 1024;  // + alignment slack
};

__device__ __forceinline__ float ipow(float s, int p) {
  float r = 1.f;
  for (int i = 0; i < p; ++i) r *= s;
  return r;
}

template <int BN, bool A_MN, bool B_MN>
__global__ void __launch_bounds__(kNumThreads, 1)
ns_gemm_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
               const GemmArgs p) {
  using L = SmemLayout<BN>;
  constexpr int kStages = L::kStages;
  constexpr uint32_t kTmemCols = 2 * BN;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  __shared__ __align__(8) uint64_t full_bar[kStages];
  __shared__ __align__(8) uint64_t empty_bar[kStages];
  __shared__ __align__(8) uint64_t tfull_bar[2];
  __shared__ __align__(8) uint64_t tempty_bar[2];
  __shared__ uint32_t tmem_base_slot;
  __shared__ int abort_flag;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int num_kb = (p.K + BK - 1) / BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tfull_bar[a], 1);
      mbar_init(&tempty_bar[a], 4);  // one arrival per epilogue warp
    }
    abort_flag = 0;
    fence_barrier_init();
    fence_proxy_async();
    prefetch_tmap(&map_a);
    prefetch_tmap(&map_b);
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
      uint32_t ready_mask = 0;
      const int seq = p.wait_flags ? *p.seq_ptr : 0;
      for (int t = blockIdx.x; t < p.total_tiles && ok; t += gridDim.x) {
        const int b = t / p.tiles_per_mat;
        const int2 tt = p.tiles[t - b * p.tiles_per_mat];
        if (p.wait_flags) {
          // Gate this tile on the arrival of the source ranks that own its operand rows.
          for (int op = 0; op < 2 && ok; ++op) {
            if (op == 0 ? !p.wait_a : !p.wait_b) continue;
            const int lim = op == 0 ? p.M : p.N;
            const int r0 = op == 0 ? tt.x * BM : tt.y * BN;
            int r1 = r0 + (op == 0 ? BM : BN) - 1;
            if (r1 > lim - 1) r1 = lim - 1;
            if (r0 > r1) continue;
            for (int src = r0 / p.rows_per_src; src <= r1 / p.rows_per_src && src < p.n_src; ++src) {
              if (ready_mask & (1u << src)) continue;
              if (!wait_flag_bounded(p.wait_flags + src, seq)) {
                report_peer_timeout(p.status, src, seq, ld_acquire_sys(p.wait_flags + src));
                abort_flag = 1;
                ok = false;
                break;
              }
              ready_mask |= 1u << src;
            }
          }
          if (!ok) break;
          // peer stores (generic proxy) must be visible to the TMA reads (async proxy)
          asm volatile("fence.proxy.async;" ::: "memory");
        }
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait_bounded(&empty_bar[stage], phase ^ 1)) {
            atomicExch(p.status, kStatusTimeoutEmpty);
            abort_flag = 1;
            ok = false;
            break;
          }
          uint8_t* sa = smem + stage * L::kStageBytes;
          uint8_t* sb = sa + L::kABytes;
          mbar_expect_tx(&full_bar[stage], L::kStageBytes);
          if (p.wait_flags && p.wait_k) {
            // K-slab gating: rows [kb*BK, +BK) of the MN-major operands come from these sources.
            int k1 = kb * BK + BK - 1;
            if (k1 > p.K - 1) k1 = p.K - 1;
            for (int src = (kb * BK) / p.rows_per_src; src <= k1 / p.rows_per_src && src < p.n_src;
                 ++src) {
              if (ready_mask & (1u << src)) continue;
              if (!wait_flag_bounded(p.wait_flags + src, seq)) {
                report_peer_timeout(p.status, src, seq, ld_acquire_sys(p.wait_flags + src));
                abort_flag = 1;
                ok = false;
                break;
              }
              ready_mask |= 1u << src;
              asm volatile("fence.proxy.async;" ::: "memory");
            }
            if (!ok) break;
          }
          if (!A_MN) {
            tma_load_3d(sa, &map_a, &full_bar[stage], kb * BK, tt.x * BM, b);
          } else {
#pragma unroll
            for (int c = 0; c < BM / 64; ++c)
              tma_load_3d(sa + c * (BK * 128), &map_a, &full_bar[stage], tt.x * BM + c * 64,
                          kb * BK, b);
          }
          if (!B_MN) {
            tma_load_3d(sb, &map_b, &full_bar[stage], kb * BK, tt.y * BN, b);
          } else {
#pragma unroll
            for (int c = 0; c < BN / 64; ++c)
              tma_load_3d(sb + c * (BK * 128), &map_b, &full_bar[stage], tt.y * BN + c * 64,
                          kb * BK, b);
          }
          if (++stage == kStages) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer --------------------------------
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc_bf16(BM, BN, A_MN ? 1 : 0, B_MN ? 1 : 0);
      uint32_t stage = 0, phase = 0;
      uint32_t aslot = 0, aphase = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < p.total_tiles && ok; t += gridDim.x) {
        if (!mbar_wait_bounded(&tempty_bar[aslot], aphase ^ 1)) {
          atomicExch(p.status, kStatusTimeoutTmemEmpty);
          abort_flag = 1;
          break;
        }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + aslot * BN;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait_bounded(&full_bar[stage], phase)) {
            atomicExch(p.status, kStatusTimeoutFull);
            abort_flag = 1;
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + stage * L::kStageBytes);
          const uint32_t sb = sa + L::kABytes;
#pragma unroll
          for (int k = 0; k < BK / 16; ++k) {
            const uint64_t da = A_MN ? make_smem_desc(sa + k * 2048, BK * 128, 1024)
                                     : make_smem_desc(sa + k * 32, 16, 1024);
            const uint64_t db = B_MN ? make_smem_desc(sb + k * 2048, BK * 128, 1024)
                                     : make_smem_desc(sb + k * 32, 16, 1024);
            tc_mma_bf16(d_tmem, da, db, idesc, (kb | k) != 0 ? 1u : 0u);
          }
          tc_commit(&empty_bar[stage]);
          if (++stage == kStages) {
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
  } else {
    // ------------------------------ epilogue ----------------------------------
    const int lane_grp = warp & 3;  // TMEM lanes [32*lane_grp, +32) belong to this warp
    const int row_in_tile = lane_grp * 32 + lane;
    uint32_t aslot = 0, aphase = 0;
    bool all_sources_ready = false;
    for (int t = blockIdx.x; t < p.total_tiles; t += gridDim.x) {
      const int b = t / p.tiles_per_mat;
      const int2 tt = p.tiles[t - b * p.tiles_per_mat];
      if (!mbar_wait_bounded(&tfull_bar[aslot], aphase)) {
        if (lane == 0) atomicExch(p.status, kStatusTimeoutTmemFull);
        break;
      }
      tc_fence_after();
      float sc = 1.f;
      if (p.scale != nullptr) sc = p.scale[b];
      if (p.scale_partials != nullptr) {
        // The norm needs every source's partial sum: wait for all of them once.
        if (!all_sources_ready) {
          bool fine = true;
          if (lane == 0) {
            const int seq = *p.seq_ptr;
            int src = 0;
            for (; src < p.n_src && fine; ++src)
              fine = wait_flag_bounded(p.wait_flags + src, seq);
            if (!fine)
              report_peer_timeout(p.status, src - 1, seq, ld_acquire_sys(p.wait_flags + src - 1));
          }
          fine = __shfl_sync(0xffffffffu, fine ? 1 : 0, 0) != 0;
          if (!fine) break;
          all_sources_ready = true;
        }
        float ss = 0.f;
        for (int src = 0; src < p.n_src; ++src)
          ss += ld_volatile_f32(p.scale_partials + (long long)b * p.n_src + src);
        sc = 1.f / (sqrtf(ss) * p.scale_mult + p.scale_eps);
      }
      const float alpha = p.alpha * ipow(sc, p.alpha_pow);
      const float beta = p.beta * ipow(sc, p.beta_pow);
      const int r = tt.x * BM + row_in_tile;
      const int warp_row0 = tt.x * BM + lane_grp * 32;
      const bool row_ok = r < p.M;
      const __nv_bfloat16* Drow =
          p.D ? p.D + (long long)b * p.strideD + (long long)r * p.ldd : nullptr;
      __nv_bfloat16* Crow = p.C ? p.C + (long long)b * p.strideC + (long long)r * p.ldc : nullptr;
      if (p.remote_c[0] != 0 && row_ok && p.cols_per_dst == 0) {
        const int dst = r / p.rows_per_dst;
        Crow = reinterpret_cast<__nv_bfloat16*>(p.remote_c[dst]) +
               ((long long)(p.remote_slot + b) * p.rows_per_dst + (r - dst * p.rows_per_dst)) *
                   p.ldc;
      }
      float* Cfrow = p.Cf ? p.Cf + (long long)b * p.strideC + (long long)r * p.ldc : nullptr;
      __nv_bfloat16* Cb = p.C ? p.C + (long long)b * p.strideC : nullptr;
      float* Cfb = p.Cf ? p.Cf + (long long)b * p.strideC : nullptr;
      __nv_bfloat16* CTb = p.CT ? p.CT + (long long)b * p.strideCT : nullptr;
      const bool vec_ok = ((p.ldc & 7) == 0) && p.Cf == nullptr &&
                          (p.remote_c[0] != 0
                               ? true
                               : (((p.strideC & 7) == 0) &&
                                  ((reinterpret_cast<uintptr_t>(p.C) & 15) == 0)));
      const bool dvec_ok = p.D && ((p.ldd & 7) == 0) && ((p.strideD & 7) == 0) &&
                           ((reinterpret_cast<uintptr_t>(p.D) & 15) == 0);

#pragma unroll 1
      for (int ch = 0; ch < BN / 32; ++ch) {
        const int c0 = tt.y * BN + ch * 32;
        // Warp-uniform skips: chunk outside the matrix, or wholly below the diagonal.
        if (c0 >= p.N) continue;
        if (p.sym && c0 + 31 < warp_row0) continue;
        float v[32];
        tmem_ld_32x32(tmem_base + (static_cast<uint32_t>(lane_grp * 32) << 16) + aslot * BN +
                          ch * 32,
                      v);
        tmem_ld_wait();
        if (!row_ok) continue;
        if (p.cols_per_dst > 0) {
          // Column split: this chunk's destination; biased so that Crow[c] is element (r, c).
          const int dst = c0 / p.cols_per_dst;
          Crow = reinterpret_cast<__nv_bfloat16*>(p.remote_c[dst]) +
                 ((long long)(p.remote_slot + b) * p.M + r) * p.cols_per_dst -
                 (long long)dst * p.cols_per_dst;
        }

        // acc*alpha + beta*D
        if (p.D) {
          if (dvec_ok && c0 + 32 <= p.N) {
            const uint4* dp = reinterpret_cast<const uint4*>(Drow + c0);
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              uint4 u = __ldg(dp + q);
              const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                float2 f = unpack_bf16x2(w[e]);
                v[q * 8 + e * 2] = alpha * v[q * 8 + e * 2] + beta * f.x;
                v[q * 8 + e * 2 + 1] = alpha * v[q * 8 + e * 2 + 1] + beta * f.y;
              }
            }
          } else {
#pragma unroll
            for (int j = 0; j < 32; ++j) {
              const int c = c0 + j;
              const float d = (c < p.N) ? __bfloat162float(Drow[c]) : 0.f;
              v[j] = alpha * v[j] + beta * d;
            }
          }
        } else {
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] *= alpha;
        }

        if (Cfrow) {
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            const int c = c0 + j;
            if (c < p.N && (!p.sym || c >= r)) Cfrow[c] = v[j];
            if (p.sym && c > r && c < p.N) Cfb[(long long)c * p.ldc + r] = v[j];
          }
          continue;
        }

        // Round once; the direct and the mirrored store use the same bf16 value.
        uint32_t pk[16];
#pragma unroll
        for (int j = 0; j < 16; ++j) pk[j] = pack_bf16x2(v[2 * j], v[2 * j + 1]);

        const bool full_chunk = (c0 + 32 <= p.N) && (!p.sym || c0 >= r);
        if (vec_ok && full_chunk) {
          uint4* cp = reinterpret_cast<uint4*>(Crow + c0);
#pragma unroll
          for (int q = 0; q < 4; ++q)
            cp[q] = make_uint4(pk[q * 4], pk[q * 4 + 1], pk[q * 4 + 2], pk[q * 4 + 3]);
        } else {
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            const int c = c0 + j;
            if (c < p.N && (!p.sym || c >= r)) {
              const uint32_t w = pk[j >> 1];
              const uint16_t h = (j & 1) ? (w >> 16) : (w & 0xFFFF);
              reinterpret_cast<uint16_t*>(Crow)[c] = h;
            }
          }
        }
        if (p.sym) {
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            const int c = c0 + j;
            if (c > r && c < p.N) {
              const uint32_t w = pk[j >> 1];
              const uint16_t h = (j & 1) ? (w >> 16) : (w & 0xFFFF);
              reinterpret_cast<uint16_t*>(Cb)[(long long)c * p.ldc + r] = h;
            }
          }
        }
        if (CTb) {
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            const int c = c0 + j;
            if (c < p.N) {
              const uint32_t w = pk[j >> 1];
              const uint16_t h = (j & 1) ? (w >> 16) : (w & 0xFFFF);
              reinterpret_cast<uint16_t*>(CTb)[(long long)c * p.ldct + r] = h;
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
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

// ---------------------------------------------------------------------------------------------
// Host side
// ---------------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (fn) return fn;
  void* sym = nullptr;
  cudaDriverEntryPointQueryResult qres;
  if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &qres) !=
          cudaSuccess ||
      qres != cudaDriverEntryPointSuccess)
    return nullptr;
  fn = reinterpret_cast<EncodeTiledFn>(sym);
  return fn;
}

// 3-D map over a [batch, rows, cols] bf16 tensor (cols contiguous) with a {box_cols, box_rows, 1}
// box and 128-byte swizzle.
static int make_map_3d(CUtensorMap* map, const void* ptr, int batch, int rows, int cols,
                       long long ld, long long batch_stride, int box_cols, int box_rows) {
  EncodeTiledFn enc = get_encode_fn();
  if (!enc) return -1;
  cuuint64_t dims[3] = {(cuuint64_t)cols, (cuuint64_t)rows, (cuuint64_t)batch};
  cuuint64_t strides[2] = {(cuuint64_t)ld * 2, (cuuint64_t)batch_stride * 2};
  if (batch == 1) strides[1] = (cuuint64_t)ld * 2 * (cuuint64_t)rows;
  cuuint32_t box[3] = {(cuuint32_t)box_cols, (cuuint32_t)box_rows, 1};
  return encode_bf16_3d(enc, map, ptr, dims, strides, box);  // cached when opted in
}

template <int BN, bool A_MN, bool B_MN>
static int launch(const CUtensorMap& ma, const CUtensorMap& mb, const GemmArgs& args, int num_sms,
                  cudaStream_t stream) {
  using L = SmemLayout<BN>;
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(ns_gemm_kernel<BN, A_MN, B_MN>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             L::kDynBytes) != cudaSuccess)
      return -3;
    configured = true;
  }
  int grid = args.total_tiles < num_sms ? args.total_tiles : num_sms;
  if (grid <= 0) return 0;
  ns_gemm_kernel<BN, A_MN, B_MN><<<grid, kNumThreads, L::kDynBytes, stream>>>(ma, mb, args);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

}  // namespace dion

// C[b] = alpha*s^pa * A[b] op(B[b]) + beta*s^pb * D[b].  All matrix pointers are bf16 device
// pointers; lda/ldb/... are in elements.  `b_mn` selects B given as [K,N] (N contiguous).
// `tiles` is a device array of (tile_m, tile_n) pairs in units of (128, bn).  Returns 0 on a
// successful launch.  Requirements: K-contiguous leading dimensions and batch strides that are
// multiples of 8 elements and 16-byte aligned base pointers for A and B.
// Optional cross-GPU coupling of one launch; see the matching fields of GemmArgs.
struct DionGemmExtra {
  const int* wait_flags;
  const int* seq_ptr;
  int n_src, rows_per_src, wait_a, wait_b, wait_k;
  const float* scale_partials;
  float scale_mult, scale_eps;
  long long remote_c[8];
  int rows_per_dst, remote_slot;
  int cols_per_dst;
};

DION_EXPORT int dion_ns_gemm_ex(const void* A, long long lda, long long strideA, int a_mn,
                                const void* B, long long ldb, long long strideB, int b_mn, void* C,
                                long long ldc,
                                long long strideC, const void* D, long long ldd, long long strideD,
                                void* CT, long long ldct, long long strideCT, void* Cf, int batch,
                                int M, int N, int K, float alpha, float beta, const float* scale,
                                int alpha_pow, int beta_pow, int sym, const void* tiles,
                                int tiles_per_mat, int bn, int num_sms, int* status, void* stream,
                                const DionGemmExtra* ex) {
  using namespace dion;
  if (batch <= 0 || M <= 0 || N <= 0 || K <= 0) return 0;
  if ((lda & 7) || (ldb & 7) || (strideA & 7) || (strideB & 7) ||
      (reinterpret_cast<uintptr_t>(A) & 15) || (reinterpret_cast<uintptr_t>(B) & 15))
    return -10;
  if (bn != 128 && bn != 256) return -11;
  CUtensorMap ma, mb;
  if (!a_mn) {
    if (make_map_3d(&ma, A, batch, M, K, lda, strideA, BK, BM) != 0) return -12;
  } else {
    if (make_map_3d(&ma, A, batch, K, M, lda, strideA, 64, BK) != 0) return -12;
  }
  if (!b_mn) {
    if (make_map_3d(&mb, B, batch, N, K, ldb, strideB, BK, bn) != 0) return -13;
  } else {
    if (make_map_3d(&mb, B, batch, K, N, ldb, strideB, 64, BK) != 0) return -13;
  }
  GemmArgs a;
  a.batch = batch; a.M = M; a.N = N; a.K = K;
  a.D = static_cast<const __nv_bfloat16*>(D); a.ldd = ldd; a.strideD = strideD;
  a.C = static_cast<__nv_bfloat16*>(C); a.ldc = ldc; a.strideC = strideC;
  a.CT = static_cast<__nv_bfloat16*>(CT); a.ldct = ldct; a.strideCT = strideCT;
  a.Cf = static_cast<float*>(Cf);
  if (a.Cf) a.C = nullptr;
  a.alpha = alpha; a.beta = beta; a.scale = scale; a.alpha_pow = alpha_pow; a.beta_pow = beta_pow;
  a.sym = sym;
  a.tiles = static_cast<const int2*>(tiles); a.tiles_per_mat = tiles_per_mat;
  a.total_tiles = tiles_per_mat * batch;
  a.status = status;
  a.wait_flags = nullptr; a.seq_ptr = nullptr; a.n_src = 0; a.rows_per_src = 1;
  a.wait_a = a.wait_b = a.wait_k = 0;
  a.scale_partials = nullptr; a.scale_mult = 1.f; a.scale_eps = 0.f;
  for (int i = 0; i < 8; ++i) a.remote_c[i] = 0;
  a.rows_per_dst = 1; a.remote_slot = 0; a.cols_per_dst = 0;
  if (ex != nullptr) {
    if (ex->n_src > 8 || ex->n_src < 0) return -14;
    if (ex->remote_c[0] != 0 && (sym || CT != nullptr || Cf != nullptr)) return -15;
    if ((ex->wait_flags != nullptr || ex->scale_partials != nullptr) &&
        (ex->seq_ptr == nullptr || ex->rows_per_src <= 0))
      return -16;
    a.wait_flags = ex->wait_flags; a.seq_ptr = ex->seq_ptr; a.n_src = ex->n_src;
    a.rows_per_src = ex->rows_per_src; a.wait_a = ex->wait_a; a.wait_b = ex->wait_b;
    a.wait_k = ex->wait_k;
    a.scale_partials = ex->scale_partials; a.scale_mult = ex->scale_mult;
    a.scale_eps = ex->scale_eps;
    for (int i = 0; i < 8; ++i) a.remote_c[i] = ex->remote_c[i];
    a.rows_per_dst = ex->rows_per_dst > 0 ? ex->rows_per_dst : 1;
    a.remote_slot = ex->remote_slot;
    if (ex->cols_per_dst < 0 || (ex->cols_per_dst & 31)) return -16;
    a.cols_per_dst = ex->remote_c[0] != 0 ? ex->cols_per_dst : 0;
  }
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int mode = (a_mn ? 2 : 0) | (b_mn ? 1 : 0);
  if (bn == 256) {
    switch (mode) {
      case 0: return launch<256, false, false>(ma, mb, a, num_sms, s);
      case 1: return launch<256, false, true>(ma, mb, a, num_sms, s);
      case 2: return launch<256, true, false>(ma, mb, a, num_sms, s);
      default: return launch<256, true, true>(ma, mb, a, num_sms, s);
    }
  }
  switch (mode) {
    case 0: return launch<128, false, false>(ma, mb, a, num_sms, s);
    case 1: return launch<128, false, true>(ma, mb, a, num_sms, s);
    case 2: return launch<128, true, false>(ma, mb, a, num_sms, s);
    default: return launch<128, true, true>(ma, mb, a, num_sms, s);
  }
}

DION_EXPORT int dion_ns_gemm(const void* A, long long lda, long long strideA, const void* B,
                             long long ldb, long long strideB, int b_mn, void* C, long long ldc,
                             long long strideC, const void* D, long long ldd, long long strideD,
                             void* CT, long long ldct, long long strideCT, void* Cf, int batch,
                             int M, int N, int K, float alpha, float beta, const float* scale,
                             int alpha_pow, int beta_pow, int sym, const void* tiles,
                             int tiles_per_mat, int bn, int num_sms, int* status, void* stream) {
  return dion_ns_gemm_ex(A, lda, strideA, 0, B, ldb, strideB, b_mn, C, ldc, strideC, D, ldd, strideD,
                         CT, ldct, strideCT, Cf, batch, M, N, K, alpha, beta, scale, alpha_pow,
                         beta_pow, sym, tiles, tiles_per_mat, bn, num_sms, status, stream, nullptr);
}
