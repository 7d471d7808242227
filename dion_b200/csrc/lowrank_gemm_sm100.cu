// Batched GEMM for the low-rank (Dion) path on sm_100a, fp32 or bf16 operands:
//
//     C[b] = alpha * sum_s A_s[b] * op(B_s[b]) + beta * D[b]          s = 0 .. nseg-1
//
// fp32 operands are multiplied on the tensor cores as tf32 (tcgen05.mma.kind::tf32, fp32
// accumulators in TMEM); bf16 operands with kind::f16.  Either operand may be K-major ([rows, K],
// K contiguous) or MN-major ([K, rows], rows contiguous), so M, M^T, Q and P of the power
// iteration (P = M Q, R = M^T P) and of the rank-r updates (M -= c P R^T, X = bX - a P Q^T) are
// all read in place from their row-major storage.  C and D are fp32 or bf16, D may be C itself
// (in-place update of momentum / weights), and C may be given as a table of per-matrix pointers
// (the weights of a model are separate allocations).
//
// Up to three K segments accumulate into the same tile.  That is how a product is computed at
// (nearly) fp32 accuracy from tf32 instructions: with x = hi + lo (hi = the tf32 part the
// instruction sees, lo = the remainder, prepared by split_lo_kernel),
//     A B ~= A_hi B_hi + A_lo B_hi + A_hi B_lo  =  segments (A, B), (A_lo, B), (A, B_lo)
// (the instruction itself ignores the low mantissa bits of the operands it is given, so A and B
// stand for their own hi parts).  The triangular solves of the randomized Cholesky-QR use this form.
//
// This replaces cuBLAS bmm / addmm / trsm in the reference's dion/dion.py:797-869, 1218-1305,
// 1491-1527.  Structure as in ns_gemm_sm100.cu: persistent CTAs, warp 0 = TMA producer (128-byte
// swizzle, no multicast), warp 1 = MMA issuer, then four epilogue warps per kEpiGroups; every wait is bounded.
#include <string.h>

#include "common.cuh"

namespace dion {

constexpr int LBM = 128;          // tile rows
constexpr int kEpiGroups = 1;      // epilogue warps per TMEM lane quarter: each takes every
                                   // kEpiGroups-th 32-column chunk
constexpr int kRing = 4;           // tile numbers in flight between the producer and the others
constexpr int kEpiPitch = 33;      // floats per row of an epilogue warp's 32 x 32 staging block
constexpr int kLrThreads = 64 + 128 * kEpiGroups;
constexpr int kRowBytes = 128;    // one swizzle row = one K slab of a K-major operand row

struct LrGemmArgs {
  int batch, M, N, K;       // K: extent of one segment
  int nseg;
  void* C;                  // base of a strided batch, or nullptr when c_table is used
  long long ldc, strideC;
  const long long* c_table; // optional: one output pointer per matrix
  const void* D;            // optional addend (may alias C)
  long long ldd, strideD;
  const long long* d_table;
  int c_dt, d_dt;           // 0 = fp32, 1 = bf16
  float alpha, beta;
  int tiles_n;              // column tiles per matrix
  int tiles_per_mat;
  int total_tiles;
  int* status;
  // Optional dynamic tile order: sched[0] hands out tile numbers, sched[1] counts finished CTAs
  // (the last one zeroes both, so launches that follow one another on a stream can share the
  // pair).  CTAs that start late - their SM was still held by another stream's kernel - then
  // find the tiles taken instead of making everybody wait for their fixed share.
  int* sched;
  // How the result leaves (fp32 C only for the last two):
  //   kOutStore      plain store into C / c_table[b]
  //   kOutReduce     red.add into C / c_table[b]: with c_table[b] pointing into the buffer of
  //                  the rank that owns matrix b (peer-mapped memory), every rank's launch adds
  //                  its contribution there - a reduce-scatter over the batch carried by the
  //                  epilogue
  //   kOutBroadcast  store into each of n_targets buffers at matrix slot (slot0 + b): an
  //                  all-gather carried by the epilogue
  int out_mode;
  long long targets[8];
  int n_targets;
  int slot0;
  // Optional: column sums of squares of the stored values, accumulated per matrix into
  // colsq[b * N + c] (fp32, pre-zeroed).
  float* colsq;
};

enum : int { kOutStore = 0, kOutReduce = 1, kOutBroadcast = 2 };

struct LrMaps {
  CUtensorMap a[3];
  CUtensorMap b[3];
};

__host__ __device__ constexpr uint32_t make_idesc(int fmt, int m, int n, int a_mn, int b_mn) {
  return (1u << 4)                                   // D format: fp32
         | (static_cast<uint32_t>(fmt) << 7)         // A format: 1 = bf16, 2 = tf32
         | (static_cast<uint32_t>(fmt) << 10)        // B format
         | (static_cast<uint32_t>(a_mn) << 15)
         | (static_cast<uint32_t>(b_mn) << 16)
         | (static_cast<uint32_t>(n >> 3) << 17)
         | (static_cast<uint32_t>(m >> 4) << 24);
}

// Shared-memory descriptor of an MN-major operand.  16-bit elements use the plain 128-byte
// swizzle (16-byte chunks XORed with the row, 8-row atoms 1024 bytes apart).  For 32-bit (tf32)
// elements the tensor core only accepts the "128-byte swizzle with 32-byte atoms" layout: 32-byte
// chunks XORed with the row, 4-row atoms 512 bytes apart - the layout TMA produces with
// CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B.  `lead_bytes` is the distance between consecutive
// 128-byte-wide blocks along MN.
template <int EB>
__device__ __forceinline__ uint64_t make_mn_desc(uint32_t saddr, uint32_t lead_bytes) {
  if constexpr (EB == 4) {
    uint64_t d = 0;
    d |= static_cast<uint64_t>((saddr & 0x3FFFF) >> 4);
    d |= static_cast<uint64_t>((lead_bytes >> 4) & 0x3FFF) << 16;
    d |= static_cast<uint64_t>((512u >> 4) & 0x3FFF) << 32;
    d |= static_cast<uint64_t>(1) << 46;  // descriptor version for sm_100
    d |= static_cast<uint64_t>(1) << 61;  // SWIZZLE_128B with 32-byte atoms
    return d;
  } else {
    return make_smem_desc(saddr, lead_bytes, 1024);
  }
}

template <int EB>
__device__ __forceinline__ void tc_mma(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                       uint32_t idesc, uint32_t accumulate) {
  if constexpr (EB == 4) {
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n"
        "}\n" ::"r"(d_tmem),
        "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
  } else {
    tc_mma_bf16(d_tmem, a_desc, b_desc, idesc, accumulate);
  }
}

__device__ __forceinline__ void red_add_f32x4(float* p, float4 v) {
  asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(p), "f"(v.x), "f"(v.y),
               "f"(v.z), "f"(v.w)
               : "memory");
}

// EB: bytes per operand element (4: fp32 read as tf32, 2: bf16).  BN: tile columns.
template <int EB, int BN, bool A_MN, bool B_MN>
__global__ void __launch_bounds__(kLrThreads, 1)
lr_gemm_kernel(const __grid_constant__ LrMaps maps, const LrGemmArgs p) {
  constexpr int BK = kRowBytes / EB;          // K elements per stage (64 bf16 / 32 fp32)
  constexpr int UK = 32 / EB;                 // K elements per instruction (16 / 8)
  constexpr int kABytes = LBM * kRowBytes;    // 16 KB
  constexpr int kBBytes = BN * kRowBytes;
  constexpr int kStageBytes = kABytes + kBBytes;
  constexpr int kStages = (BN == 256) ? 4 : 6;
  constexpr int kBoxElems = kRowBytes / EB;   // MN elements per box of an MN-major operand
  constexpr int kBoxBytes = BK * kRowBytes;   // one MN-major box: BK rows of 128 bytes
  constexpr int kStepMN = UK * kRowBytes;     // MN-major advance per instruction
  constexpr uint32_t kTmemCols = 2 * BN;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  __shared__ __align__(8) uint64_t full_bar[kStages];
  __shared__ __align__(8) uint64_t empty_bar[kStages];
  __shared__ __align__(8) uint64_t tfull_bar[2];
  __shared__ __align__(8) uint64_t tempty_bar[2];
  __shared__ uint32_t tmem_base_slot;
  __shared__ float epi_stage[4 * kEpiGroups][32 * kEpiPitch];
  __shared__ __align__(8) uint64_t ring_full[kRing];
  __shared__ __align__(8) uint64_t ring_empty[kRing];
  __shared__ int tile_ring[kRing];

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
      mbar_init(&tempty_bar[a], 4 * kEpiGroups);
    }
    for (int q = 0; q < kRing; ++q) {
      mbar_init(&ring_full[q], 1);
      mbar_init(&ring_empty[q], 1 + 4 * kEpiGroups);   // MMA thread + one lane per epilogue warp
    }
    fence_barrier_init();
    fence_proxy_async();
    for (int s = 0; s < p.nseg; ++s) {
      prefetch_tmap(&maps.a[s]);
      prefetch_tmap(&maps.b[s]);
    }
  }
  if (warp == 1) {
    tmem_alloc(&tmem_base_slot, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_base_slot;

  // Tile hand-out.  The producer thread decides the it-th tile of this CTA (its fixed share, or
  // the next number of the device counter) and posts it in a small ring; -1 ends the kernel.
  auto post_tile = [&](int it) -> int {
    const int slot = it & (kRing - 1);
    const uint32_t ph = (static_cast<uint32_t>(it) / kRing) & 1u;
    int t = -1;
    if (mbar_wait_bounded(&ring_empty[slot], ph ^ 1u)) {
      t = p.sched ? atomicAdd(p.sched, 1) : static_cast<int>(blockIdx.x + it * gridDim.x);
      if (t >= p.total_tiles) t = -1;
    } else {
      atomicExch(p.status, kStatusTimeoutEmpty);
    }
    tile_ring[slot] = t;
    mbar_arrive(&ring_full[slot]);
    return t;
  };
  // The other roles read it: the MMA thread alone (`whole_warp` false), or the 32 lanes of an
  // epilogue warp together, of which one (`arrive`) hands the slot back once all have read.
  auto take_tile = [&](int it, bool arrive, bool whole_warp) -> int {
    const int slot = it & (kRing - 1);
    const uint32_t ph = (static_cast<uint32_t>(it) / kRing) & 1u;
    if (!mbar_wait_bounded(&ring_full[slot], ph)) {
      if (arrive) atomicExch(p.status, kStatusTimeoutFull);
      return -1;
    }
    const int t = tile_ring[slot];
    if (whole_warp) __syncwarp();
    if (arrive) mbar_arrive(&ring_empty[slot]);
    return t;
  };

  if (warp == 0) {
    // ------------------------------ TMA producer ------------------------------
    if (lane == 0) {
      uint32_t stage = 0, phase = 0;
      bool ok = true;
      for (int it = 0; ok; ++it) {
        const int t = post_tile(it);
        if (t < 0) break;
        const int b = t / p.tiles_per_mat;
        const int rem = t - b * p.tiles_per_mat;
        const int tm = rem / p.tiles_n, tn = rem - tm * p.tiles_n;
        for (int seg = 0; seg < p.nseg && ok; ++seg) {
          const CUtensorMap* ma = &maps.a[seg];
          const CUtensorMap* mb = &maps.b[seg];
          for (int kb = 0; kb < num_kb; ++kb) {
            if (!mbar_wait_bounded(&empty_bar[stage], phase ^ 1)) {
              atomicExch(p.status, kStatusTimeoutEmpty);
              ok = false;
              break;
            }
            uint8_t* sa = smem + stage * kStageBytes;
            uint8_t* sb = sa + kABytes;
            mbar_expect_tx(&full_bar[stage], kStageBytes);
            if (!A_MN) {
              tma_load_3d(sa, ma, &full_bar[stage], kb * BK, tm * LBM, b);
            } else {
#pragma unroll
              for (int c = 0; c < LBM / kBoxElems; ++c)
                tma_load_3d(sa + c * kBoxBytes, ma, &full_bar[stage], tm * LBM + c * kBoxElems,
                            kb * BK, b);
            }
            if (!B_MN) {
              tma_load_3d(sb, mb, &full_bar[stage], kb * BK, tn * BN, b);
            } else {
#pragma unroll
              for (int c = 0; c < BN / kBoxElems; ++c)
                tma_load_3d(sb + c * kBoxBytes, mb, &full_bar[stage], tn * BN + c * kBoxElems,
                            kb * BK, b);
            }
            if (++stage == kStages) {
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
      constexpr uint32_t idesc = make_idesc(EB == 4 ? 2 : 1, LBM, BN, A_MN ? 1 : 0, B_MN ? 1 : 0);
      uint32_t stage = 0, phase = 0;
      uint32_t aslot = 0, aphase = 0;
      bool ok = true;
      const int total_kb = num_kb * p.nseg;
      for (int it = 0; ok; ++it) {
        if (take_tile(it, true, false) < 0) break;
        if (!mbar_wait_bounded(&tempty_bar[aslot], aphase ^ 1)) {
          atomicExch(p.status, kStatusTimeoutTmemEmpty);
          break;
        }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + aslot * BN;
        for (int kb = 0; kb < total_kb; ++kb) {
          if (!mbar_wait_bounded(&full_bar[stage], phase)) {
            atomicExch(p.status, kStatusTimeoutFull);
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + stage * kStageBytes);
          const uint32_t sb = sa + kABytes;
#pragma unroll
          for (int k = 0; k < BK / UK; ++k) {
            const uint64_t da = A_MN ? make_mn_desc<EB>(sa + k * kStepMN, kBoxBytes)
                                     : make_smem_desc(sa + k * 32, 16, 1024);
            const uint64_t db = B_MN ? make_mn_desc<EB>(sb + k * kStepMN, kBoxBytes)
                                     : make_smem_desc(sb + k * 32, 16, 1024);
            tc_mma<EB>(d_tmem, da, db, idesc, (kb | k) != 0 ? 1u : 0u);
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
    const int lane_grp = warp & 3;     // TMEM lanes this warp may read: 32 * (warp % 4) ...
    const int epi_grp = (warp - 2) >> 2;
    const int row_in_tile = lane_grp * 32 + lane;
    uint32_t aslot = 0, aphase = 0;
    for (int it = 0;; ++it) {
      const int t = take_tile(it, lane == 0, true);
      if (t < 0) break;
      const int b = t / p.tiles_per_mat;
      const int rem = t - b * p.tiles_per_mat;
      const int tm = rem / p.tiles_n, tn = rem - tm * p.tiles_n;
      const int r = tm * LBM + row_in_tile;
      const bool row_ok = r < p.M;
      char* Cb = p.c_table ? reinterpret_cast<char*>(p.c_table[b])
                           : (p.C ? static_cast<char*>(p.C) +
                                        (long long)b * p.strideC * (p.c_dt ? 2 : 4)
                                  : nullptr);
      const char* Db = p.d_table ? reinterpret_cast<const char*>(p.d_table[b])
                                 : (p.D ? static_cast<const char*>(p.D) +
                                              (long long)b * p.strideD * (p.d_dt ? 2 : 4)
                                        : nullptr);
      const bool c_vec = (p.ldc & 7) == 0 && (reinterpret_cast<uintptr_t>(Cb) & 15) == 0 &&
                         (p.c_table != nullptr || (p.strideC & 7) == 0);
      const bool d_vec = Db != nullptr && (p.ldd & 7) == 0 &&
                         (reinterpret_cast<uintptr_t>(Db) & 15) == 0 &&
                         (p.d_table != nullptr || (p.strideD & 7) == 0);
      if (Db != nullptr && row_ok && epi_grp == 0) {
        // While the tensor cores still work on this tile, pull this thread's row of D towards
        // L2: with K as short as a rank the epilogue is the longer half of a tile, and most of
        // it used to be the DRAM latency of one D chunk after the other.
        const int esz = p.d_dt ? 2 : 4;
        const char* drow = Db + ((long long)r * p.ldd + (long long)tn * BN) * esz;
        const int cols_here = (p.N - tn * BN) < BN ? (p.N - tn * BN) : BN;
        for (int off = 0; off < cols_here * esz; off += 128)
          asm volatile("prefetch.global.L2 [%0];" ::"l"(drow + off));
      }
      if (!mbar_wait_bounded(&tfull_bar[aslot], aphase)) {
        if (lane == 0) atomicExch(p.status, kStatusTimeoutTmemFull);
        break;
      }
      tc_fence_after();
#pragma unroll 1
      for (int ch = epi_grp; ch < BN / 32; ch += kEpiGroups) {
        const int c0 = tn * BN + ch * 32;
        if (c0 >= p.N) continue;  // warp-uniform
        const bool full = c0 + 32 <= p.N;
        // The vector form of D is requested before the accumulator is read, so that both are
        // in flight together (fp32: eight 16-byte pieces; bf16: four, carried as raw bits).
        if (p.out_mode == kOutStore && p.colsq == nullptr && c_vec && full &&
            (Db == nullptr || (d_vec && p.d_dt == p.c_dt))) {
          // Plain store, possibly in place over D.  A thread of the accumulator owns a row, so
          // row-wise accesses would touch 32 different lines per instruction, 16 bytes of each:
          // request slots between L1 and L2, not bytes, then bound the kernel.  The block is
          // turned through shared memory instead: per instruction the warp covers four rows of
          // 128 bytes (fp32; eight rows of 64 bytes for bf16), whole lines or sectors, and all
          // loads of D are issued before the accumulator is read.
          float* st = epi_stage[warp - 2];
          const int wrow0 = tm * LBM + lane_grp * 32;
          if (p.c_dt == 0) {
            const int rsub = lane >> 3, cq = (lane & 7) * 4;
            float4 d[8];
            if (Db != nullptr) {
#pragma unroll
              for (int it = 0; it < 8; ++it) {
                const int rr = wrow0 + it * 4 + rsub;
                if (rr < p.M)
                  d[it] = *reinterpret_cast<const float4*>(
                      reinterpret_cast<const float*>(Db) + (long long)rr * p.ldd + c0 + cq);
              }
            }
            float v[32];
            tmem_ld_32x32(tmem_base + (static_cast<uint32_t>(lane_grp * 32) << 16) + aslot * BN +
                              ch * 32,
                          v);
            tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 32; ++j) st[lane * kEpiPitch + j] = p.alpha * v[j];
            __syncwarp();
#pragma unroll
            for (int it = 0; it < 8; ++it) {
              const int rl = it * 4 + rsub;
              const int rr = wrow0 + rl;
              if (rr < p.M) {
                const float* sp = st + rl * kEpiPitch + cq;
                float4 x = make_float4(sp[0], sp[1], sp[2], sp[3]);
                if (Db != nullptr) {
                  x.x += p.beta * d[it].x;
                  x.y += p.beta * d[it].y;
                  x.z += p.beta * d[it].z;
                  x.w += p.beta * d[it].w;
                }
                *reinterpret_cast<float4*>(reinterpret_cast<float*>(Cb) + (long long)rr * p.ldc +
                                           c0 + cq) = x;
              }
            }
          } else {
            const int rsub = lane >> 2, cq = (lane & 3) * 8;
            uint4 d[4];
            if (Db != nullptr) {
#pragma unroll
              for (int it = 0; it < 4; ++it) {
                const int rr = wrow0 + it * 8 + rsub;
                if (rr < p.M)
                  d[it] = *reinterpret_cast<const uint4*>(
                      reinterpret_cast<const __nv_bfloat16*>(Db) + (long long)rr * p.ldd + c0 + cq);
              }
            }
            float v[32];
            tmem_ld_32x32(tmem_base + (static_cast<uint32_t>(lane_grp * 32) << 16) + aslot * BN +
                              ch * 32,
                          v);
            tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 32; ++j) st[lane * kEpiPitch + j] = p.alpha * v[j];
            __syncwarp();
#pragma unroll
            for (int it = 0; it < 4; ++it) {
              const int rl = it * 8 + rsub;
              const int rr = wrow0 + rl;
              if (rr < p.M) {
                const float* sp = st + rl * kEpiPitch + cq;
                float x[8];
#pragma unroll
                for (int e = 0; e < 8; ++e) x[e] = sp[e];
                if (Db != nullptr) {
                  const uint32_t w[4] = {d[it].x, d[it].y, d[it].z, d[it].w};
#pragma unroll
                  for (int e = 0; e < 4; ++e) {
                    const float2 f = unpack_bf16x2(w[e]);
                    x[2 * e] += p.beta * f.x;
                    x[2 * e + 1] += p.beta * f.y;
                  }
                }
                *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(Cb) +
                                          (long long)rr * p.ldc + c0 + cq) =
                    make_uint4(pack_bf16x2(x[0], x[1]), pack_bf16x2(x[2], x[3]),
                               pack_bf16x2(x[4], x[5]), pack_bf16x2(x[6], x[7]));
              }
            }
          }
          __syncwarp();     // the staging block is reused by the next chunk
          continue;
        }
        float4 dpre[8];
        const bool pre = row_ok && d_vec && full;
        if (pre) {
          if (p.d_dt == 0) {
            const float4* dp = reinterpret_cast<const float4*>(
                reinterpret_cast<const float*>(Db) + (long long)r * p.ldd + c0);
#pragma unroll
            for (int q = 0; q < 8; ++q) dpre[q] = dp[q];
          } else {
            const float4* dp = reinterpret_cast<const float4*>(
                reinterpret_cast<const __nv_bfloat16*>(Db) + (long long)r * p.ldd + c0);
#pragma unroll
            for (int q = 0; q < 4; ++q) dpre[q] = dp[q];
          }
        }
        float v[32];
        tmem_ld_32x32(tmem_base + (static_cast<uint32_t>(lane_grp * 32) << 16) + aslot * BN +
                          ch * 32,
                      v);
        tmem_ld_wait();
        if (row_ok) {
          // ---- combine with D ----
          if (Db != nullptr) {
            if (p.d_dt == 0) {
              const float* drow = reinterpret_cast<const float*>(Db) + (long long)r * p.ldd + c0;
              if (pre) {
#pragma unroll
                for (int q = 0; q < 8; ++q) {
                  const float4 d = dpre[q];
                  v[q * 4] = p.alpha * v[q * 4] + p.beta * d.x;
                  v[q * 4 + 1] = p.alpha * v[q * 4 + 1] + p.beta * d.y;
                  v[q * 4 + 2] = p.alpha * v[q * 4 + 2] + p.beta * d.z;
                  v[q * 4 + 3] = p.alpha * v[q * 4 + 3] + p.beta * d.w;
                }
              } else {
#pragma unroll
                for (int j = 0; j < 32; ++j)
                  v[j] = p.alpha * v[j] + (c0 + j < p.N ? p.beta * drow[j] : 0.f);
              }
            } else {
              const __nv_bfloat16* drow =
                  reinterpret_cast<const __nv_bfloat16*>(Db) + (long long)r * p.ldd + c0;
              if (pre) {
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                  const uint4 u = make_uint4(__float_as_uint(dpre[q].x), __float_as_uint(dpre[q].y),
                                             __float_as_uint(dpre[q].z), __float_as_uint(dpre[q].w));
                  const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
                  for (int e = 0; e < 4; ++e) {
                    const float2 f = unpack_bf16x2(w[e]);
                    v[q * 8 + e * 2] = p.alpha * v[q * 8 + e * 2] + p.beta * f.x;
                    v[q * 8 + e * 2 + 1] = p.alpha * v[q * 8 + e * 2 + 1] + p.beta * f.y;
                  }
                }
              } else {
#pragma unroll
                for (int j = 0; j < 32; ++j)
                  v[j] = p.alpha * v[j] +
                         (c0 + j < p.N ? p.beta * __bfloat162float(drow[j]) : 0.f);
              }
            }
          } else {
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] *= p.alpha;
          }
          // ---- store / reduce ----
          if (p.out_mode == kOutReduce) {
            float* crow = reinterpret_cast<float*>(Cb) + (long long)r * p.ldc + c0;
            if (c_vec && full) {
#pragma unroll
              for (int q = 0; q < 8; ++q)
                red_add_f32x4(crow + q * 4,
                              make_float4(v[q * 4], v[q * 4 + 1], v[q * 4 + 2], v[q * 4 + 3]));
            } else {
#pragma unroll
              for (int j = 0; j < 32; ++j)
                if (c0 + j < p.N) atomicAdd(crow + j, v[j]);
            }
          } else if (p.out_mode == kOutBroadcast) {
            for (int tgt = 0; tgt < p.n_targets; ++tgt) {
              float* crow = reinterpret_cast<float*>(p.targets[tgt]) +
                            (long long)(p.slot0 + b) * p.strideC + (long long)r * p.ldc + c0;
              if ((p.ldc & 3) == 0 && (p.strideC & 3) == 0 && full) {
#pragma unroll
                for (int q = 0; q < 8; ++q)
                  *reinterpret_cast<float4*>(crow + q * 4) =
                      make_float4(v[q * 4], v[q * 4 + 1], v[q * 4 + 2], v[q * 4 + 3]);
              } else {
#pragma unroll
                for (int j = 0; j < 32; ++j)
                  if (c0 + j < p.N) crow[j] = v[j];
              }
            }
          } else if (p.c_dt == 0) {
            float* crow = reinterpret_cast<float*>(Cb) + (long long)r * p.ldc + c0;
            if (c_vec && full) {
#pragma unroll
              for (int q = 0; q < 8; ++q)
                *reinterpret_cast<float4*>(crow + q * 4) =
                    make_float4(v[q * 4], v[q * 4 + 1], v[q * 4 + 2], v[q * 4 + 3]);
            } else {
#pragma unroll
              for (int j = 0; j < 32; ++j)
                if (c0 + j < p.N) crow[j] = v[j];
            }
          } else {
            __nv_bfloat16* crow = reinterpret_cast<__nv_bfloat16*>(Cb) + (long long)r * p.ldc + c0;
            if (c_vec && full) {
#pragma unroll
              for (int q = 0; q < 4; ++q)
                *reinterpret_cast<uint4*>(crow + q * 8) =
                    make_uint4(pack_bf16x2(v[q * 8], v[q * 8 + 1]),
                               pack_bf16x2(v[q * 8 + 2], v[q * 8 + 3]),
                               pack_bf16x2(v[q * 8 + 4], v[q * 8 + 5]),
                               pack_bf16x2(v[q * 8 + 6], v[q * 8 + 7]));
            } else {
#pragma unroll
              for (int j = 0; j < 32; ++j)
                if (c0 + j < p.N) crow[j] = __float2bfloat16(v[j]);
            }
          }
        }
        if (p.colsq != nullptr) {
          // Column sums of squares over the 32 rows of this warp: lane j ends up with column j.
          // (Rows beyond M contribute zero.)  Values are taken as stored (bf16-rounded if so).
          float mine = 0.f;
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            float x = row_ok ? v[j] : 0.f;
            if (p.c_dt == 1) x = __bfloat162float(__float2bfloat16(x));
            float s = x * x;
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
            if (lane == j) mine = s;
          }
          if (c0 + lane < p.N) atomicAdd(p.colsq + (long long)b * p.N + c0 + lane, mine);
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
  if (threadIdx.x == 0 && p.sched != nullptr) {
    // Every CTA has drawn its last number by now; the last one to get here rewinds the pair.
    __threadfence();
    if (atomicAdd(p.sched + 1, 1) == static_cast<int>(gridDim.x) - 1) {
      p.sched[0] = 0;
      __threadfence();
      p.sched[1] = 0;
    }
  }
}

// lo = x - tf32_part(x): what a tf32 instruction does not see of x (it reads sign, exponent and
// the upper 10 mantissa bits).
__global__ void split_lo_kernel(const float* __restrict__ x, float* __restrict__ lo, long long n) {
  const long long i = ((long long)blockIdx.x * blockDim.x + threadIdx.x) * 4;
  if (i + 3 < n && (reinterpret_cast<uintptr_t>(x) & 15) == 0 &&
      (reinterpret_cast<uintptr_t>(lo) & 15) == 0) {
    const float4 a = *reinterpret_cast<const float4*>(x + i);
    float4 o;
    o.x = a.x - __uint_as_float(__float_as_uint(a.x) & 0xFFFFE000u);
    o.y = a.y - __uint_as_float(__float_as_uint(a.y) & 0xFFFFE000u);
    o.z = a.z - __uint_as_float(__float_as_uint(a.z) & 0xFFFFE000u);
    o.w = a.w - __uint_as_float(__float_as_uint(a.w) & 0xFFFFE000u);
    *reinterpret_cast<float4*>(lo + i) = o;
  } else {
    for (long long k = i; k < n && k < i + 4; ++k)
      lo[k] = x[k] - __uint_as_float(__float_as_uint(x[k]) & 0xFFFFE000u);
  }
}

// The same for a batch of `rows` x `cols` matrices read through a strided view (row pitch ld_x,
// batch pitch bs_x; cols, pitches and bases multiples of 4 elements / 16 bytes); lo is dense.
__global__ void split_lo_view_kernel(const float* __restrict__ x, long long ld_x, long long bs_x,
                                     float* __restrict__ lo, long long total4, int rows,
                                     int cols4) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total4) return;
  const long long row_all = i / cols4;
  const int c = static_cast<int>(i - row_all * cols4) * 4;
  const long long b = row_all / rows;
  const long long row = row_all - b * rows;
  const float4 a = *reinterpret_cast<const float4*>(x + b * bs_x + row * ld_x + c);
  float4 o;
  o.x = a.x - __uint_as_float(__float_as_uint(a.x) & 0xFFFFE000u);
  o.y = a.y - __uint_as_float(__float_as_uint(a.y) & 0xFFFFE000u);
  o.z = a.z - __uint_as_float(__float_as_uint(a.z) & 0xFFFFE000u);
  o.w = a.w - __uint_as_float(__float_as_uint(a.w) & 0xFFFFE000u);
  *reinterpret_cast<float4*>(lo + i * 4) = o;
}

// ---------------------------------------------------------------------------------------------
// Host side
// ---------------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFnLr)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                    const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                    const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                    CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFnLr get_encode_fn_lr() {
  static EncodeTiledFnLr fn = nullptr;
  if (fn) return fn;
  void* sym = nullptr;
  cudaDriverEntryPointQueryResult qres;
  if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &qres) !=
          cudaSuccess ||
      qres != cudaDriverEntryPointSuccess)
    return nullptr;
  fn = reinterpret_cast<EncodeTiledFnLr>(sym);
  return fn;
}

// 3-D map over [batch, rows, cols] (cols contiguous) of 2- or 4-byte elements, box
// {box_cols, box_rows, 1}, 128-byte swizzle (box_cols * elem_bytes == 128); `atom32` selects the
// variant with 32-byte atoms that MN-major tf32 operands need (see make_mn_desc).
static int make_map_lr(CUtensorMap* map, const void* ptr, int eb, int batch, int rows, int cols,
                       long long ld, long long batch_stride, int box_cols, int box_rows,
                       bool atom32 = false) {
  EncodeTiledFnLr enc = get_encode_fn_lr();
  if (!enc) return -1;
  cuuint64_t dims[3] = {(cuuint64_t)cols, (cuuint64_t)rows, (cuuint64_t)batch};
  cuuint64_t strides[2] = {(cuuint64_t)ld * eb, (cuuint64_t)batch_stride * eb};
  if (batch == 1) strides[1] = (cuuint64_t)ld * eb * (cuuint64_t)rows;
  cuuint32_t box[3] = {(cuuint32_t)box_cols, (cuuint32_t)box_rows, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = enc(map, eb == 4 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16,
                   3, const_cast<void*>(ptr), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE,
                   atom32 ? CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B : CU_TENSOR_MAP_SWIZZLE_128B,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : -2;
}

template <int EB, int BN, bool A_MN, bool B_MN>
static int launch_lr(const LrMaps& maps, const LrGemmArgs& args, int num_sms, cudaStream_t stream) {
  constexpr int kStages = (BN == 256) ? 4 : 6;
  constexpr int kDyn = kStages * (LBM * kRowBytes + BN * kRowBytes) + 1024;
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(lr_gemm_kernel<EB, BN, A_MN, B_MN>,
                             cudaFuncAttributeMaxDynamicSharedMemorySize, kDyn) != cudaSuccess)
      return -3;
    configured = true;
  }
  const int grid = args.total_tiles < num_sms ? args.total_tiles : num_sms;
  if (grid <= 0) return 0;
  lr_gemm_kernel<EB, BN, A_MN, B_MN><<<grid, kLrThreads, kDyn, stream>>>(maps, args);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

template <int EB, int BN>
static int dispatch_lr(int a_mn, int b_mn, const LrMaps& maps, const LrGemmArgs& a, int num_sms,
                       cudaStream_t s) {
  switch ((a_mn ? 2 : 0) | (b_mn ? 1 : 0)) {
    case 0: return launch_lr<EB, BN, false, false>(maps, a, num_sms, s);
    case 1: return launch_lr<EB, BN, false, true>(maps, a, num_sms, s);
    case 2: return launch_lr<EB, BN, true, false>(maps, a, num_sms, s);
    default: return launch_lr<EB, BN, true, true>(maps, a, num_sms, s);
  }
}

}  // namespace dion

// One operand of a segment: base pointer, leading dimension and batch stride in elements.
struct DionLrOperand {
  const void* ptr;
  long long ld, stride;
};

// Everything beyond the plain strided-batch case.
struct DionLrExtra {
  const long long* c_table;   // per-matrix output pointers (C must then be null)
  const long long* d_table;   // per-matrix addend pointers
  int out_mode;               // 0 store, 1 red.add into C / c_table[b], 2 store to all targets
  long long targets[8];       // mode 2: bases of fp32 buffers [slots, M, N] (ldc, strideC apply)
  int n_targets;
  int slot0;                  // mode 2: matrix b goes to slot slot0 + b
  float* colsq;               // [batch, N] column sums of squares of the result
  int* sched;                 // optional: two zeroed ints for the dynamic tile order (see LrGemmArgs)
};

// C[b] = alpha * sum_s A_s[b] op(B_s[b]) + beta * D[b].
//   elem_bytes   4: fp32 operands multiplied as tf32; 2: bf16 operands.
//   a_mn / b_mn  0: operand given as [rows, K] with K contiguous; 1: as [K, rows], rows contiguous.
//   c_dt / d_dt  0: fp32, 1: bf16.  ldc/strideC (ldd/strideD) in elements.
// Operand pointers must be 16-byte aligned with leading dimensions and batch strides that are
// multiples of 16 bytes (TMA).  Returns 0 on a successful launch.
DION_EXPORT int dion_lr_gemm(int elem_bytes, int nseg, const DionLrOperand* A,
                             const DionLrOperand* B, int a_mn, int b_mn, void* C, long long ldc,
                             long long strideC, int c_dt, const void* D, long long ldd,
                             long long strideD, int d_dt, int batch, int M, int N, int K,
                             float alpha, float beta, int bn, int num_sms, int* status,
                             void* stream, const DionLrExtra* ex) {
  using namespace dion;
  if (batch <= 0 || M <= 0 || N <= 0 || K <= 0) return 0;
  if (elem_bytes != 2 && elem_bytes != 4) return -10;
  if (nseg < 1 || nseg > 3) return -10;
  if (bn != 128 && bn != 256) return -11;
  const int per16 = 16 / elem_bytes;
  LrMaps maps;
  memset(&maps, 0, sizeof(maps));
  const int bk = kRowBytes / elem_bytes;
  const int box_mn = kRowBytes / elem_bytes;
  for (int s = 0; s < nseg; ++s) {
    const DionLrOperand& a = A[s];
    const DionLrOperand& b = B[s];
    if ((a.ld % per16) || (b.ld % per16) || (a.stride % per16) || (b.stride % per16) ||
        (reinterpret_cast<uintptr_t>(a.ptr) & 15) || (reinterpret_cast<uintptr_t>(b.ptr) & 15))
      return -12;
    int rc;
    if (!a_mn) rc = make_map_lr(&maps.a[s], a.ptr, elem_bytes, batch, M, K, a.ld, a.stride, bk, LBM);
    else rc = make_map_lr(&maps.a[s], a.ptr, elem_bytes, batch, K, M, a.ld, a.stride, box_mn, bk,
                          elem_bytes == 4);
    if (rc != 0) return -13;
    if (!b_mn) rc = make_map_lr(&maps.b[s], b.ptr, elem_bytes, batch, N, K, b.ld, b.stride, bk, bn);
    else rc = make_map_lr(&maps.b[s], b.ptr, elem_bytes, batch, K, N, b.ld, b.stride, box_mn, bk,
                          elem_bytes == 4);
    if (rc != 0) return -14;
  }
  LrGemmArgs g;
  memset(&g, 0, sizeof(g));
  g.batch = batch; g.M = M; g.N = N; g.K = K; g.nseg = nseg;
  g.C = C; g.ldc = ldc; g.strideC = strideC; g.c_dt = c_dt;
  g.D = D; g.ldd = ldd; g.strideD = strideD; g.d_dt = d_dt;
  g.alpha = alpha; g.beta = beta;
  g.tiles_n = (N + bn - 1) / bn;
  g.tiles_per_mat = ((M + LBM - 1) / LBM) * g.tiles_n;
  g.total_tiles = g.tiles_per_mat * batch;
  g.status = status;
  if (ex != nullptr) {
    g.c_table = ex->c_table;
    g.d_table = ex->d_table;
    g.out_mode = ex->out_mode;
    g.n_targets = ex->n_targets;
    g.slot0 = ex->slot0;
    for (int i = 0; i < 8; ++i) g.targets[i] = ex->targets[i];
    g.colsq = ex->colsq;
    g.sched = ex->sched;
    if (g.out_mode < 0 || g.out_mode > 2 || g.n_targets < 0 || g.n_targets > 8) return -15;
    if (g.out_mode != 0 && c_dt != 0) return -15;
    if (g.out_mode == 2 && g.n_targets == 0) return -15;
  }
  if (g.c_table == nullptr && g.C == nullptr && g.out_mode != 2) return -16;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (elem_bytes == 4) {
    return bn == 256 ? dispatch_lr<4, 256>(a_mn, b_mn, maps, g, num_sms, s)
                     : dispatch_lr<4, 128>(a_mn, b_mn, maps, g, num_sms, s);
  }
  return bn == 256 ? dispatch_lr<2, 256>(a_mn, b_mn, maps, g, num_sms, s)
                   : dispatch_lr<2, 128>(a_mn, b_mn, maps, g, num_sms, s);
}

DION_EXPORT int dion_split_lo(const float* x, float* lo, long long n, void* stream) {
  if (n <= 0) return 0;
  const long long threads = (n + 3) / 4;
  dion::split_lo_kernel<<<(unsigned)((threads + 255) / 256), 256, 0,
                          static_cast<cudaStream_t>(stream)>>>(x, lo, n);
  return cudaGetLastError() == cudaSuccess ? 0 : -1;
}

DION_EXPORT int dion_split_lo_view(const float* x, long long ld_x, long long bs_x, float* lo,
                                   long long batch, int rows, int cols, void* stream) {
  if (batch <= 0 || rows <= 0 || cols <= 0) return 0;
  if ((cols & 3) || (ld_x & 3) || (bs_x & 3) || (reinterpret_cast<uintptr_t>(x) & 15) ||
      (reinterpret_cast<uintptr_t>(lo) & 15))
    return -2;
  const long long total4 = batch * rows * (cols / 4);
  dion::split_lo_view_kernel<<<(unsigned)((total4 + 255) / 256), 256, 0,
                               static_cast<cudaStream_t>(stream)>>>(x, ld_x, bs_x, lo, total4, rows,
                                                                    cols / 4);
  return cudaGetLastError() == cudaSuccess ? 0 : -1;
}
