// Two-CTA (cta_group::2) variant of the Newton-Schulz GEMM for sm_100a:
//
//     C[b] = alpha * s_b^pa * A[b] * op(B[b]) + beta * s_b^pb * D[b]
//
// A pair of CTAs on neighbouring SMs (a cluster of two) computes one 256x256 output tile with
// tcgen05.mma.cta_group::2 (UMMA 256x256x16).  Each CTA stages only its own 128 rows of A and its
// own 128 of the 256 columns of B per 64-wide K slab (32 KB instead of the 48 KB a lone CTA needs
// for a 128x256 tile), which takes the shared-memory traffic per MMA cycle below the SM's
// bandwidth - the limit the single-CTA kernel in ns_gemm_sm100.cu runs into.  Loads are plain TMA
// (cp.async.bulk.tensor with .cta_group::2 so that both CTAs' transfers complete on the leader's
// barrier; no multicast).  The leader CTA's MMA thread issues the instructions for the pair and
// releases stages / publishes accumulators in both CTAs with a cluster-multicast tcgen05.commit.
// Each CTA drains its own half (128 TMEM lanes) of the accumulator in its epilogue warps, 64 columns
// at a time through shared memory: D arrives by TMA (prefetched two sub-tiles ahead), each thread
// combines its row in place in the 128-byte-swizzled buffer, and the buffer leaves by TMA store.
// In symmetric mode only tiles on or above the diagonal are computed; an off-diagonal tile also
// writes a transposed copy of each sub-tile that a second TMA store places at the mirrored
// position, so both halves of the output are written with full-width bursts.
//
// Operand layouts and the epilogue arithmetic are the same as in the single-CTA kernel.  All waits
// are bounded; the epilogue threads meet at a barrier that also ANDs their wait results, so a
// timeout makes all of them leave together.
#include "common.cuh"
#include "tmap_cache.h"

namespace dion {

constexpr int BM2 = 128;   // rows per CTA (256 per pair)
constexpr int BN2 = 256;   // columns per pair (128 loaded by each CTA)
constexpr int BK2 = 64;
constexpr int kThreads2 = 192;
constexpr int kStagesSym = 5;     // symmetric mode also stages transposed sub-tiles
constexpr int kStagesPlain = 6;
constexpr int kABytes2 = BM2 * BK2 * 2;          // 16 KB
constexpr int kBBytes2 = (BN2 / 2) * BK2 * 2;    // 16 KB
constexpr int kStageBytes2 = kABytes2 + kBBytes2;
constexpr int kSubCols = 64;                       // epilogue sub-tile: 128 rows x 64 columns
constexpr int kEpiBufs = 2;
constexpr int kEpiBufBytes = BM2 * kSubCols * 2;    // 16 KB: two 64 x 64 boxes of bf16
// stages | kEpiBufs D/C buffers | kEpiBufs transposed buffers (symmetric mode) | alignment slack
constexpr int dyn_bytes2(int stages, bool sym) {
  return stages * kStageBytes2 + (sym ? 2 : 1) * kEpiBufs * kEpiBufBytes + 1024;
}
constexpr uint32_t kTmemCols2 = 2 * BN2;

// Epilogue forms: C = alpha*acc + beta*D | relu(alpha*acc)^2 | alpha*acc * 2*sqrt(D).
enum : int { kEpiAxpby = 0, kEpiRelu2 = 1, kEpiMul2Sqrt = 2 };

struct Gemm2Args {
  int batch, M, N, K;
  const __nv_bfloat16* D;
  long long ldd, strideD;
  __nv_bfloat16* C;
  long long ldc, strideC;
  float alpha, beta;
  const float* scale;
  int alpha_pow, beta_pow;
  int sym;
  const int2* tiles;  // (tile_m, tile_n) in units of 256 x 256
  int tiles_per_mat;
  int total_tiles;
  int* status;
  int epi;      // kEpi*
  // ---- optional coupling to other GPUs (same meaning as in GemmArgs of ns_gemm_sm100.cu) ----
  // Gating: rows [s*rows_per_src, (s+1)*rows_per_src) of the gated operands were stored into
  // this GPU's memory by rank s, which then raised wait_flags[s] to *seq_ptr.
  const int* wait_flags;
  const int* seq_ptr;
  int n_src;
  int rows_per_src;
  int wait_a, wait_b, wait_k;
  // scale = 1 / (sqrt(sum_s scale_partials[b*n_src + s]) * scale_mult + scale_eps)
  const float* scale_partials;
  float scale_mult, scale_eps;
  // Output rows go to their owners instead of C: row r of matrix b is stored at
  // remote_c[r / rows_per_dst] + ((remote_slot + b) * rows_per_dst + r % rows_per_dst) * ldc.
  long long remote_c[8];
  int rows_per_dst;
  int remote_slot;
  // cols_per_dst > 0: split by columns instead: element (r, c) of matrix b goes to
  // remote_c[c / cols_per_dst] + ((remote_slot + b) * M + r) * cols_per_dst + c % cols_per_dst
  // (a multiple of 8 columns, so a 16-byte piece has one destination).
  int cols_per_dst;
};

__device__ __forceinline__ int ld_acquire_sys2(const int* p) {
  int v;
  asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ float ld_volatile_f32_2(const float* p) {
  float v;
  asm volatile("ld.volatile.global.f32 %0, [%1];" : "=f"(v) : "l"(p) : "memory");
  return v;
}
// Barrier over the 128 epilogue threads without a predicate (barrier 2).
__device__ __forceinline__ void epi_barrier_plain() {
  asm volatile("barrier.cta.sync.aligned 2, 128;" ::: "memory");
}

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ uint32_t cluster_id_x() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%clusterid.x;" : "=r"(r));
  return r;
}
__device__ __forceinline__ uint32_t num_clusters_x() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%nclusterid.x;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// shared::cluster address of `local_addr` (a shared::cta address) in the CTA with rank `rank`.
__device__ __forceinline__ uint32_t map_to_cta(uint32_t local_addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local_addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr)
               : "memory");
}
// TMA load whose completion is counted on a barrier that may live in the peer CTA of the pair.
__device__ __forceinline__ void tma_load_3d_pair(void* smem_dst, const CUtensorMap* map,
                                                 uint32_t bar_cluster_addr, int x, int y, int z) {
  asm volatile(
      "cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes "
      "[%0], [%1, {%3, %4, %5}], [%2];" ::"r"(smem_u32(smem_dst)),
      "l"(reinterpret_cast<uint64_t>(map)), "r"(bar_cluster_addr), "r"(x), "r"(y), "r"(z)
      : "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t* smem_result, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                   smem_u32(smem_result)),
               "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols)
               : "memory");
}
// Arrives on the barrier at the same shared-memory offset in both CTAs of the pair once all
// tcgen05.mma issued so far have completed.
__device__ __forceinline__ void tc_commit_pair(uint64_t* bar) {
  const uint16_t mask = 3;
  asm volatile(
      "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 "
      "[%0], %1;" ::"r"(smem_u32(bar)),
      "h"(mask)
      : "memory");
}
__device__ __forceinline__ void tc_mma_bf16_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                                 uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n"
      "}\n" ::"r"(d_tmem),
      "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}

// Bounded wait with cluster-scope acquire (the arrivals come from both CTAs of the pair).
__device__ __forceinline__ bool mbar_wait_bounded_cluster(uint64_t* bar, uint32_t parity) {
  WaitBudget budget;
  for (;;) {
    uint32_t ok;
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n"
        "selp.u32 %0, 1, 0, p;\n"
        "}\n"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    if (ok) return true;
    if (budget.spent()) return false;
  }
}

// TMA store of one box from shared memory (bulk-group completion).
__device__ __forceinline__ void tma_store_3d(const CUtensorMap* map, const void* smem_src, int x,
                                             int y, int z) {
  asm volatile(
      "cp.async.bulk.tensor.3d.global.shared::cta.bulk_group [%0, {%2, %3, %4}], [%1];" ::"l"(
          reinterpret_cast<uint64_t>(map)),
      "r"(smem_u32(smem_src)), "r"(x), "r"(y), "r"(z)
      : "memory");
}
__device__ __forceinline__ void bulk_commit_group() {
  asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}
__device__ __forceinline__ void bulk_wait_group_read_all() {
  asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
}
__device__ __forceinline__ void bulk_wait_group_all() {
  asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
}
// Barrier over the 128 epilogue threads (barrier 1) that also ANDs a predicate.
__device__ __forceinline__ bool epi_barrier_and(bool mine) {
  uint32_t out;
  asm volatile(
      "{\n"
      ".reg .pred p, q;\n"
      "setp.ne.u32 q, %1, 0;\n"
      "barrier.cta.red.and.pred.aligned p, 1, 128, q;\n"
      "selp.u32 %0, 1, 0, p;\n"
      "}\n"
      : "=r"(out)
      : "r"((uint32_t)mine)
      : "memory");
  return out != 0;
}

__device__ __forceinline__ float ipow2(float s, int p) {
  float r = 1.f;
  for (int i = 0; i < p; ++i) r *= s;
  return r;
}

template <bool A_MN, bool B_MN, int kStages2>
__global__ void __launch_bounds__(kThreads2, 1)
ns_gemm2_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                const __grid_constant__ CUtensorMap map_c, const __grid_constant__ CUtensorMap map_d,
                const Gemm2Args p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  __shared__ __align__(8) uint64_t full_bar[kStages2];    // used in the leader CTA
  __shared__ __align__(8) uint64_t empty_bar[kStages2];   // one copy per CTA
  __shared__ __align__(8) uint64_t tfull_bar[2];          // one copy per CTA
  __shared__ __align__(8) uint64_t tempty_bar[2];         // used in the leader CTA
  __shared__ __align__(8) uint64_t dfull_bar[kEpiBufs];   // D sub-tiles, one copy per CTA
  __shared__ uint32_t tmem_base_slot;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t cta = cluster_ctarank();  // 0 = leader
  const int num_kb = (p.K + BK2 - 1) / BK2;
  const int first_tile = (int)cluster_id_x();
  const int tile_step = (int)num_clusters_x();

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages2; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tfull_bar[a], 1);
      mbar_init(&tempty_bar[a], 8);  // four epilogue warps in each CTA of the pair
    }
    for (int a = 0; a < kEpiBufs; ++a) mbar_init(&dfull_bar[a], 1);
    fence_barrier_init();
    fence_proxy_async();
    prefetch_tmap(&map_a);
    prefetch_tmap(&map_b);
    prefetch_tmap(&map_c);
    if (p.D) prefetch_tmap(&map_d);
  }
  if (warp == 1) {
    tmem_alloc_pair(&tmem_base_slot, kTmemCols2);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // barriers of both CTAs are initialised before anyone signals them
  tc_fence_after();
  const uint32_t tmem_base = tmem_base_slot;

  if (warp == 0) {
    // ------------------------------ TMA producer (both CTAs) ------------------------------
    if (lane == 0) {
      uint32_t stage = 0, phase = 0;
      bool ok = true;
      uint32_t ready_mask = 0;
      const int seq = p.wait_flags ? *p.seq_ptr : 0;
      // Waits (bounded) until every source rank owning rows [r0, r1] has delivered.
      auto sources_ready = [&](int r0, int r1) -> bool {
        for (int src = r0 / p.rows_per_src; src <= r1 / p.rows_per_src && src < p.n_src; ++src) {
          if (ready_mask & (1u << src)) continue;
          if (!flag_wait_bounded(p.wait_flags + src, seq)) {
            report_peer_timeout(p.status, src, seq, ld_acquire_sys2(p.wait_flags + src));
            return false;
          }
          ready_mask |= 1u << src;
          // peer stores (generic proxy) must be visible to the TMA reads (async proxy)
          asm volatile("fence.proxy.async;" ::: "memory");
        }
        return true;
      };
      for (int t = first_tile; t < p.total_tiles && ok; t += tile_step) {
        const int b = t / p.tiles_per_mat;
        const int2 tt = p.tiles[t - b * p.tiles_per_mat];
        const int row0 = tt.x * 256 + (int)cta * BM2;          // this CTA's rows of A
        const int col0 = tt.y * BN2 + (int)cta * (BN2 / 2);    // this CTA's columns of B
        if (p.wait_flags) {
          // Gate this CTA's share of the tile on the ranks that own its operand rows.
          if (p.wait_a && row0 < p.M) {
            const int r1 = row0 + BM2 - 1 < p.M ? row0 + BM2 - 1 : p.M - 1;
            ok = sources_ready(row0, r1);
          }
          if (ok && p.wait_b && col0 < p.N) {
            const int r1 = col0 + BN2 / 2 - 1 < p.N ? col0 + BN2 / 2 - 1 : p.N - 1;
            ok = sources_ready(col0, r1);
          }
          if (!ok) break;
        }
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait_bounded(&empty_bar[stage], phase ^ 1)) {
            atomicExch(p.status, kStatusTimeoutEmpty);
            ok = false;
            break;
          }
          if (p.wait_flags && p.wait_k) {
            // K-slab gating: rows [kb*BK2, +BK2) of MN-major operands belong to these sources.
            const int k1 = kb * BK2 + BK2 - 1 < p.K ? kb * BK2 + BK2 - 1 : p.K - 1;
            if (!sources_ready(kb * BK2, k1)) {
              ok = false;
              break;
            }
          }
          uint8_t* sa = smem + stage * kStageBytes2;
          uint8_t* sb = sa + kABytes2;
          const uint32_t bar = map_to_cta(smem_u32(&full_bar[stage]), 0);
          if (cta == 0) mbar_expect_tx(&full_bar[stage], 2 * kStageBytes2);
          if (!A_MN) {
            tma_load_3d_pair(sa, &map_a, bar, kb * BK2, row0, b);
          } else {
#pragma unroll
            for (int c = 0; c < BM2 / 64; ++c)
              tma_load_3d_pair(sa + c * (BK2 * 128), &map_a, bar, row0 + c * 64, kb * BK2, b);
          }
          if (!B_MN) {
            tma_load_3d_pair(sb, &map_b, bar, kb * BK2, col0, b);
          } else {
#pragma unroll
            for (int c = 0; c < (BN2 / 2) / 64; ++c)
              tma_load_3d_pair(sb + c * (BK2 * 128), &map_b, bar, col0 + c * 64, kb * BK2, b);
          }
          if (++stage == kStages2) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer (leader CTA only) --------------------------
    if (lane == 0 && cta == 0) {
      constexpr uint32_t idesc = make_idesc_bf16(256, BN2, A_MN ? 1 : 0, B_MN ? 1 : 0);
      uint32_t stage = 0, phase = 0;
      uint32_t aslot = 0, aphase = 0;
      bool ok = true;
      for (int t = first_tile; t < p.total_tiles && ok; t += tile_step) {
        if (!mbar_wait_bounded_cluster(&tempty_bar[aslot], aphase ^ 1)) {
          atomicExch(p.status, kStatusTimeoutTmemEmpty);
          break;
        }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + aslot * BN2;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait_bounded_cluster(&full_bar[stage], phase)) {
            atomicExch(p.status, kStatusTimeoutFull);
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + stage * kStageBytes2);
          const uint32_t sb = sa + kABytes2;
#pragma unroll
          for (int k = 0; k < BK2 / 16; ++k) {
            const uint64_t da = A_MN ? make_smem_desc(sa + k * 2048, BK2 * 128, 1024)
                                     : make_smem_desc(sa + k * 32, 16, 1024);
            const uint64_t db = B_MN ? make_smem_desc(sb + k * 2048, BK2 * 128, 1024)
                                     : make_smem_desc(sb + k * 32, 16, 1024);
            tc_mma_bf16_pair(d_tmem, da, db, idesc, (kb | k) != 0 ? 1u : 0u);
          }
          tc_commit_pair(&empty_bar[stage]);
          if (++stage == kStages2) {
            stage = 0;
            phase ^= 1;
          }
        }
        if (!ok) break;
        tc_commit_pair(&tfull_bar[aslot]);
        aslot ^= 1;
        if (aslot == 0) aphase ^= 1;
      }
    }
  } else {
    // ------------------------------ epilogue (both CTAs) ----------------------------------
    // The 128 x 256 half-tile of this CTA is drained in sub-tiles of 64 columns.  D arrives by
    // TMA into a shared-memory buffer (prefetched two sub-tiles ahead), each thread combines
    // its row in place, and the buffer leaves by TMA store; with `sym`, off-diagonal tiles also
    // write a transposed copy that a second TMA store places at the mirrored position.
    const int lane_grp = warp & 3;
    const int row_in_tile = lane_grp * 32 + lane;
    const bool elected = (warp == 2 && lane == 0);
    const bool has_d = p.D != nullptr;
    const int epi = p.epi;
    const uint32_t row_off = (uint32_t)(row_in_tile >> 6) * 8192u + (uint32_t)(row_in_tile & 63) * 128u;
    const uint32_t row_sw = (uint32_t)(row_in_tile & 7);
    uint8_t* dc_base = smem + kStages2 * kStageBytes2;
    uint8_t* t_base = dc_base + kEpiBufs * kEpiBufBytes;

    // Iterator over the sub-tiles this pair will process, in order (used for the D prefetch).
    int pf_t = first_tile, pf_s = 0;
    auto pf_valid = [&]() { return pf_t < p.total_tiles; };
    auto pf_coords = [&](int& b, int& r0, int& c0) {
      b = pf_t / p.tiles_per_mat;
      const int2 tt = p.tiles[pf_t - b * p.tiles_per_mat];
      r0 = tt.x * 256 + (int)cta * BM2;
      c0 = tt.y * BN2 + pf_s * kSubCols;
    };
    auto pf_advance = [&]() {
      const int b = pf_t / p.tiles_per_mat;
      const int2 tt = p.tiles[pf_t - b * p.tiles_per_mat];
      ++pf_s;
      if (pf_s >= 4 || tt.y * BN2 + pf_s * kSubCols >= p.N) {
        pf_s = 0;
        pf_t += tile_step;
      }
    };
    uint32_t d_issued = 0;  // D sub-tiles requested so far (elected thread)
    auto issue_d = [&](uint32_t g) {
      d_issued = g + 1;
      int b, r0, c0;
      pf_coords(b, r0, c0);
      const uint32_t buf = g % kEpiBufs;
      uint8_t* dst = dc_base + buf * kEpiBufBytes;
      mbar_expect_tx(&dfull_bar[buf], kEpiBufBytes);
      tma_load_3d(dst, &map_d, &dfull_bar[buf], c0, r0, b);
      tma_load_3d(dst + 8192, &map_d, &dfull_bar[buf], c0, r0 + 64, b);
    };
    if (elected && has_d) {
      for (uint32_t g0 = 0; g0 < 2 && pf_valid(); ++g0) {
        issue_d(g0);
        pf_advance();
      }
    }

    uint32_t aslot = 0, aphase = 0;
    uint32_t g = 0;  // running sub-tile count
    bool ok = true;
    bool all_sources_ready = false;
    const bool remote = p.remote_c[0] != 0;
    const int epi_tid = (warp - 2) * 32 + lane;   // 0..127
    for (int t = first_tile; t < p.total_tiles && ok; t += tile_step) {
      const int b = t / p.tiles_per_mat;
      const int2 tt = p.tiles[t - b * p.tiles_per_mat];
      bool mine_ok = __all_sync(0xffffffffu, mbar_wait_bounded(&tfull_bar[aslot], aphase));
      if (!mine_ok && lane == 0) atomicExch(p.status, kStatusTimeoutTmemFull);
      tc_fence_after();
      float sc = 1.f;
      if (p.scale != nullptr) sc = p.scale[b];
      if (p.scale_partials != nullptr && mine_ok) {
        // The norm needs every source's partial sum: wait for all of them once.
        if (!all_sources_ready) {
          int fine = 1;
          if (lane == 0) {
            const int seq = *p.seq_ptr;
            for (int src = 0; src < p.n_src && fine; ++src) {
              if (!flag_wait_bounded(p.wait_flags + src, seq)) {
                report_peer_timeout(p.status, src, seq, ld_acquire_sys2(p.wait_flags + src));
                fine = 0;
              }
            }
          }
          fine = __shfl_sync(0xffffffffu, fine, 0);
          if (!fine) mine_ok = false;
          all_sources_ready = true;
        }
        float ss = 0.f;
        for (int src = 0; src < p.n_src; ++src)
          ss += ld_volatile_f32_2(p.scale_partials + (long long)b * p.n_src + src);
        sc = 1.f / (sqrtf(ss) * p.scale_mult + p.scale_eps);
      }
      const float alpha = p.alpha * ipow2(sc, p.alpha_pow);
      const float beta = p.beta * ipow2(sc, p.beta_pow);
      const int row0 = tt.x * 256 + (int)cta * BM2;
      const bool mirror = p.sym && tt.y > tt.x;
      int nsub = (p.N - tt.y * BN2 + kSubCols - 1) / kSubCols;
      nsub = nsub > 4 ? 4 : nsub;
#pragma unroll 1
      for (int s = 0; s < nsub; ++s, ++g) {
        const int c0 = tt.y * BN2 + s * kSubCols;
        const uint32_t buf = g % kEpiBufs;
        uint8_t* dc = dc_base + buf * kEpiBufBytes;
        uint8_t* tb = t_base + buf * kEpiBufBytes;
        if (has_d && mine_ok) {
          mine_ok = __all_sync(0xffffffffu,
                               mbar_wait_bounded(&dfull_bar[buf], (g / kEpiBufs) & 1));
          if (!mine_ok && lane == 0) atomicExch(p.status, kStatusTimeoutFull);
        }
        if (mine_ok) {
          float v[kSubCols];
          const uint32_t taddr = tmem_base + (static_cast<uint32_t>(lane_grp * 32) << 16) +
                                 aslot * BN2 + s * kSubCols;
          tmem_ld_32x32(taddr, v);
          tmem_ld_32x32(taddr + 32, v + 32);
          tmem_ld_wait();
          if (s == nsub - 1) {
            // Last read of this accumulator: hand the TMEM slot back to the MMA thread.
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(map_to_cta(smem_u32(&tempty_bar[aslot]), 0));
          }
          uint8_t* rowp = dc + row_off;
#pragma unroll
          for (int j = 0; j < kSubCols / 8; ++j) {
            uint4* cell = reinterpret_cast<uint4*>(rowp + (((uint32_t)j ^ row_sw) << 4));
            float* vj = v + j * 8;
            if (has_d) {
              const uint4 u = *cell;
              const uint32_t w[4] = {u.x, u.y, u.z, u.w};
              if (epi == kEpiMul2Sqrt) {
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                  const float2 f = unpack_bf16x2(w[e]);
                  vj[2 * e] = alpha * vj[2 * e] * (2.f * sqrtf(f.x));
                  vj[2 * e + 1] = alpha * vj[2 * e + 1] * (2.f * sqrtf(f.y));
                }
              } else {
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                  const float2 f = unpack_bf16x2(w[e]);
                  vj[2 * e] = alpha * vj[2 * e] + beta * f.x;
                  vj[2 * e + 1] = alpha * vj[2 * e + 1] + beta * f.y;
                }
              }
            } else if (epi == kEpiRelu2) {
#pragma unroll
              for (int e = 0; e < 8; ++e) {
                const float t = fmaxf(alpha * vj[e], 0.f);
                vj[e] = t * t;
              }
            } else {
#pragma unroll
              for (int e = 0; e < 8; ++e) vj[e] *= alpha;
            }
            uint32_t pk[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) pk[e] = pack_bf16x2(vj[2 * e], vj[2 * e + 1]);
            *cell = make_uint4(pk[0], pk[1], pk[2], pk[3]);
            if (mirror) {
              // Transposed copy: element (row, c0 + c) goes to row c, column `row` of two
              // 64 x 64 boxes (128-byte swizzled like every other buffer).
              const uint32_t tcol = (uint32_t)(row_in_tile >> 6) * 8192u +
                                    ((uint32_t)(row_in_tile & 7) << 1);
              const uint32_t tchunk = (uint32_t)(row_in_tile & 63) >> 3;
#pragma unroll
              for (int e = 0; e < 8; ++e) {
                const uint32_t c = (uint32_t)(j * 8 + e);
                const uint32_t w = pk[e >> 1];
                const uint16_t h = (e & 1) ? (uint16_t)(w >> 16) : (uint16_t)(w & 0xFFFF);
                *reinterpret_cast<uint16_t*>(tb + tcol + c * 128u + ((tchunk ^ (c & 7)) << 4)) = h;
              }
            }
          }
          fence_proxy_async();
        }
        // Every epilogue thread reaches this barrier (all waits above are bounded); it also
        // tells whether any of them gave up.
        ok = epi_barrier_and(mine_ok);
        if (!ok) break;
        if (remote) {
          // Rows leave for the ranks that own them: 16-byte stores over NVLink, eight
          // consecutive threads per 128-byte row segment of the (swizzled) sub-tile.
          const int chunk = epi_tid & 7;
          if (c0 + chunk * 8 < p.N) {
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              const int rr = (epi_tid >> 3) + 16 * i;     // row of the 128-row half-tile
              const int grow = row0 + rr;
              if (grow < p.M) {
                const uint8_t* src = dc + (uint32_t)(rr >> 6) * 8192u + (uint32_t)(rr & 63) * 128u +
                                     (((uint32_t)chunk ^ (uint32_t)(rr & 7)) << 4);
                __nv_bfloat16* out;
                if (p.cols_per_dst > 0) {
                  const int col = c0 + chunk * 8;
                  const int dst = col / p.cols_per_dst;
                  out = reinterpret_cast<__nv_bfloat16*>(p.remote_c[dst]) +
                        ((long long)(p.remote_slot + b) * p.M + grow) * p.cols_per_dst +
                        (col - dst * p.cols_per_dst);
                } else {
                  const int dst = grow / p.rows_per_dst;
                  out = reinterpret_cast<__nv_bfloat16*>(p.remote_c[dst]) +
                        ((long long)(p.remote_slot + b) * p.rows_per_dst +
                         (grow - dst * p.rows_per_dst)) * p.ldc + c0 + chunk * 8;
                }
                *reinterpret_cast<uint4*>(out) = *reinterpret_cast<const uint4*>(src);
              }
            }
          }
          epi_barrier_plain();   // the buffer has been read: it may take the next D sub-tile
          if (elected && has_d && pf_valid()) {
            issue_d(g + 2);
            pf_advance();
          }
          continue;
        }
        if (elected) {
          if (row0 < p.M) tma_store_3d(&map_c, dc, c0, row0, b);
          if (row0 + 64 < p.M) tma_store_3d(&map_c, dc + 8192, c0, row0 + 64, b);
          if (mirror) {
            if (row0 < p.N) tma_store_3d(&map_c, tb, row0, c0, b);
            if (row0 + 64 < p.N) tma_store_3d(&map_c, tb + 8192, row0 + 64, c0, b);
          }
          bulk_commit_group();
          // Once the stores have read their buffers, these are free for sub-tile g+2.
          bulk_wait_group_read_all();
          if (has_d && pf_valid()) {
            issue_d(g + 2);
            pf_advance();
          }
        }
      }
      aslot ^= 1;
      if (aslot == 0) aphase ^= 1;
    }
    if (elected) {
      bulk_wait_group_all();
      // After a timeout: let the D copies still in flight land before the CTA exits.
      if (!ok)
        for (uint32_t x = g; x < d_issued; ++x)
          mbar_wait_bounded(&dfull_bar[x % kEpiBufs], (x / kEpiBufs) & 1);
    }
  }

  // Nobody leaves while the peer may still read this CTA's shared memory or signal its barriers.
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, kTmemCols2);
  }
}

}  // namespace dion

// ---------------------------------------------------------------------------------------------
// Host side
// ---------------------------------------------------------------------------------------------
namespace dion {

typedef CUresult (*EncodeTiledFn2)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                   const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                   const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                   CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn2 get_encode_fn2() {
  static EncodeTiledFn2 fn = nullptr;
  if (fn) return fn;
  void* sym = nullptr;
  cudaDriverEntryPointQueryResult qres;
  if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &qres) !=
          cudaSuccess ||
      qres != cudaDriverEntryPointSuccess)
    return nullptr;
  fn = reinterpret_cast<EncodeTiledFn2>(sym);
  return fn;
}

static int make_map2(CUtensorMap* map, const void* ptr, int batch, int rows, int cols,
                     long long ld, long long batch_stride, int box_cols, int box_rows) {
  EncodeTiledFn2 enc = get_encode_fn2();
  if (!enc) return -1;
  cuuint64_t dims[3] = {(cuuint64_t)cols, (cuuint64_t)rows, (cuuint64_t)batch};
  cuuint64_t strides[2] = {(cuuint64_t)ld * 2, (cuuint64_t)batch_stride * 2};
  if (batch == 1) strides[1] = (cuuint64_t)ld * 2 * (cuuint64_t)rows;
  cuuint32_t box[3] = {(cuuint32_t)box_cols, (cuuint32_t)box_rows, 1};
  return encode_bf16_3d(enc, map, ptr, dims, strides, box);  // cached when opted in
}

template <bool A_MN, bool B_MN, int STAGES>
static int launch2(const CUtensorMap& ma, const CUtensorMap& mb, const CUtensorMap& mc,
                   const CUtensorMap& md, const Gemm2Args& args, cudaStream_t stream) {
  static bool configured = false;
  static int max_clusters = 0;
  auto kernel = ns_gemm2_kernel<A_MN, B_MN, STAGES>;
  constexpr int kDynBytes2 = dyn_bytes2(STAGES, STAGES == kStagesSym);
  if (!configured) {
    if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kDynBytes2) !=
        cudaSuccess)
      return -3;
    cudaLaunchConfig_t probe = {};
    probe.gridDim = dim3(2 * 74, 1, 1);
    probe.blockDim = dim3(kThreads2, 1, 1);
    probe.dynamicSmemBytes = kDynBytes2;
    cudaLaunchAttribute pattr[1];
    pattr[0].id = cudaLaunchAttributeClusterDimension;
    pattr[0].val.clusterDim.x = 2;
    pattr[0].val.clusterDim.y = 1;
    pattr[0].val.clusterDim.z = 1;
    probe.attrs = pattr;
    probe.numAttrs = 1;
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, kernel, &probe) != cudaSuccess || n <= 0) {
      cudaGetLastError();
      return -5;
    }
    max_clusters = n;
    configured = true;
  }
  int clusters = args.total_tiles < max_clusters ? args.total_tiles : max_clusters;
  if (clusters <= 0) return 0;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(2 * clusters, 1, 1);
  cfg.blockDim = dim3(kThreads2, 1, 1);
  cfg.dynamicSmemBytes = kDynBytes2;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  if (cudaLaunchKernelEx(&cfg, kernel, ma, mb, mc, md, args) != cudaSuccess) {
    cudaGetLastError();
    return -4;
  }
  return 0;
}

}  // namespace dion

// Optional cross-GPU coupling of one launch; see the matching fields of Gemm2Args (the layout is
// shared with DionGemmExtra of ns_gemm_sm100.cu so that one host structure serves both kernels).
struct DionGemm2Extra {
  const int* wait_flags;
  const int* seq_ptr;
  int n_src, rows_per_src, wait_a, wait_b, wait_k;
  const float* scale_partials;
  float scale_mult, scale_eps;
  long long remote_c[8];
  int rows_per_dst, remote_slot;
  int cols_per_dst;
};

// Same contract as dion_ns_gemm_ex (ns_gemm_sm100.cu) for the features it has: bf16 output,
// optional D, per-batch scale, symmetric mode, gating on peer flags, norm from partial sums and
// rows stored to their owners (then C may be null); `tiles` holds (tile_m, tile_n) pairs in units
// of 256 x 256.
DION_EXPORT int dion_ns_gemm2_ex(const void* A, long long lda, long long strideA, int a_mn,
                                 const void* B, long long ldb, long long strideB, int b_mn, void* C,
                                 long long ldc, long long strideC, const void* D, long long ldd,
                                 long long strideD, int batch, int M, int N, int K, float alpha,
                                 float beta, const float* scale, int alpha_pow, int beta_pow,
                                 int sym, const void* tiles, int tiles_per_mat, int epi,
                                 int* status, void* stream, const DionGemm2Extra* ex) {
  using namespace dion;
  if (batch <= 0 || M <= 0 || N <= 0 || K <= 0) return 0;
  const bool remote = ex != nullptr && ex->remote_c[0] != 0;
  if ((lda & 7) || (ldb & 7) || (strideA & 7) || (strideB & 7) ||
      (reinterpret_cast<uintptr_t>(A) & 15) || (reinterpret_cast<uintptr_t>(B) & 15) ||
      (C == nullptr && !remote))
    return -10;
  CUtensorMap ma, mb;
  if (!a_mn) {
    if (make_map2(&ma, A, batch, M, K, lda, strideA, BK2, BM2) != 0) return -12;
  } else {
    if (make_map2(&ma, A, batch, K, M, lda, strideA, 64, BK2) != 0) return -12;
  }
  if (!b_mn) {
    if (make_map2(&mb, B, batch, N, K, ldb, strideB, BK2, BN2 / 2) != 0) return -13;
  } else {
    if (make_map2(&mb, B, batch, K, N, ldb, strideB, 64, BK2) != 0) return -13;
  }
  // C leaves (and D arrives) through TMA in 64 x 64 boxes.
  if (C && ((ldc & 7) || (strideC & 7) || (reinterpret_cast<uintptr_t>(C) & 15))) return -11;
  if (D && ((ldd & 7) || (strideD & 7) || (reinterpret_cast<uintptr_t>(D) & 15))) return -11;
  if (remote && (sym || (ldc & 7) || (N & 7) || (D == nullptr && C == nullptr))) return -15;
  CUtensorMap mc, md;
  // A map needs some valid tensor even where the kernel never uses it (no D / remote output).
  const void* c_for_map = C ? C : D;
  if (make_map2(&mc, c_for_map, batch, M, N, C ? ldc : ldd, C ? strideC : strideD, kSubCols,
                64) != 0)
    return -14;
  if (make_map2(&md, D ? D : C, batch, M, N, D ? ldd : ldc, D ? strideD : strideC, kSubCols,
                64) != 0)
    return -14;
  Gemm2Args a;
  a.batch = batch; a.M = M; a.N = N; a.K = K;
  a.D = static_cast<const __nv_bfloat16*>(D); a.ldd = ldd; a.strideD = strideD;
  a.C = static_cast<__nv_bfloat16*>(C); a.ldc = ldc; a.strideC = strideC;
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
    if (ex->cols_per_dst < 0 || (ex->cols_per_dst & 7)) return -16;
    a.cols_per_dst = ex->remote_c[0] != 0 ? ex->cols_per_dst : 0;
  }
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  a.epi = epi;
  if (epi == kEpiMul2Sqrt && D == nullptr) return -16;
  if (epi == kEpiRelu2 && D != nullptr) return -16;
  const int mode = (a_mn ? 2 : 0) | (b_mn ? 1 : 0);
  if (sym) {
    switch (mode) {
      case 0: return launch2<false, false, kStagesSym>(ma, mb, mc, md, a, s);
      case 1: return launch2<false, true, kStagesSym>(ma, mb, mc, md, a, s);
      case 2: return launch2<true, false, kStagesSym>(ma, mb, mc, md, a, s);
      default: return launch2<true, true, kStagesSym>(ma, mb, mc, md, a, s);
    }
  }
  switch (mode) {
    case 0: return launch2<false, false, kStagesPlain>(ma, mb, mc, md, a, s);
    case 1: return launch2<false, true, kStagesPlain>(ma, mb, mc, md, a, s);
    case 2: return launch2<true, false, kStagesPlain>(ma, mb, mc, md, a, s);
    default: return launch2<true, true, kStagesPlain>(ma, mb, mc, md, a, s);
  }
}

DION_EXPORT int dion_ns_gemm2(const void* A, long long lda, long long strideA, int a_mn,
                              const void* B, long long ldb, long long strideB, int b_mn, void* C,
                              long long ldc, long long strideC, const void* D, long long ldd,
                              long long strideD, int batch, int M, int N, int K, float alpha,
                              float beta, const float* scale, int alpha_pow, int beta_pow, int sym,
                              const void* tiles, int tiles_per_mat, int epi, int* status,
                              void* stream) {
  return dion_ns_gemm2_ex(A, lda, strideA, a_mn, B, ldb, strideB, b_mn, C, ldc, strideC, D, ldd,
                          strideD, batch, M, N, K, alpha, beta, scale, alpha_pow, beta_pow, sym,
                          tiles, tiles_per_mat, epi, status, stream, nullptr);
}

// Whole Newton-Schulz iteration from one host call: for every coefficient triple (a, b, c)
//   A  = s^2 * X X^T            (wide / square; X^T X for tall matrices), symmetric
//   B  = b * A + c * A A        symmetric
//   X' = s * (a * X + B X)      (X B for tall matrices)
// with the input scale s applied in the first iteration only, ping-ponging between the buffers
// X and Xalt.  All operands are dense [batch, rows, cols] bf16.  The result of the last
// iteration lies in Xalt when `iters` is odd, else in X.  This only saves the host the 3 * iters
// trips through the Python front end; the launches are the same as issued one by one.
DION_EXPORT int dion_ns_iterate2(void* X, void* Xalt, void* A, void* Bm, int batch, int m, int n,
                                 const float* coeffs, int iters, const float* scale,
                                 const void* tiles_gg, int n_tiles_gg, const void* tiles_mn,
                                 int n_tiles_mn, int* status, void* stream) {
  const int tall = m > n;
  const int g = tall ? n : m;
  const long long sx = (long long)m * n, sg = (long long)g * g;
  void* cur = X;
  void* nxt = Xalt;
  for (int it = 0; it < iters; ++it) {
    const float a = coeffs[3 * it], b = coeffs[3 * it + 1], c = coeffs[3 * it + 2];
    const float* sc = (it == 0) ? scale : nullptr;
    const int p2 = sc ? 2 : 0, p1 = sc ? 1 : 0;
    // Gram matrix: wide X [g, K=n] against itself; tall X read as [K=m, g] on both sides.
    int rc = dion_ns_gemm2(cur, n, sx, tall, cur, n, sx, tall, A, g, sg, nullptr, 0, 0, batch, g, g,
                           tall ? m : n, 1.f, 0.f, sc, p2, 0, 1, tiles_gg, n_tiles_gg, 0, status,
                           stream);
    if (rc != 0) return rc;
    rc = dion_ns_gemm2(A, g, sg, 0, A, g, sg, 0, Bm, g, sg, A, g, sg, batch, g, g, g, c, b, nullptr,
                       0, 0, 1, tiles_gg, n_tiles_gg, 0, status, stream);
    if (rc != 0) return rc;
    if (tall) {  // X' = a X + X B, B symmetric: given as [N, K]
      rc = dion_ns_gemm2(cur, n, sx, 0, Bm, g, sg, 0, nxt, n, sx, cur, n, sx, batch, m, n, g, 1.f, a,
                         sc, p1, p1, 0, tiles_mn, n_tiles_mn, 0, status, stream);
    } else {     // X' = a X + B X, X given as [K, N]
      rc = dion_ns_gemm2(Bm, g, sg, 0, cur, n, sx, 1, nxt, n, sx, cur, n, sx, batch, m, n, g, 1.f, a,
                         sc, p1, p1, 0, tiles_mn, n_tiles_mn, 0, status, stream);
    }
    if (rc != 0) return rc;
    void* t = cur; cur = nxt; nxt = t;
  }
  return 0;
}
