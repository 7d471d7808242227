// Shared device helpers for the sm_100a kernels: mbarrier, TMA, tcgen05 and
// bounded-wait primitives, written as inline PTX.
//
// Every spin-wait in this library goes through bounded_* helpers: a wait that
// runs out of polls records a code in a global status word and lets the caller
// unwind (free TMEM, return) instead of spinning forever.
#pragma once
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#ifndef DION_EXPORT
#define DION_EXPORT extern "C" __attribute__((visibility("default")))
#endif

namespace dion {

// Status codes written to the global status word (0 = ok).
enum : int {
  kStatusOk = 0,
  kStatusTimeoutFull = 1,       // consumer waited for a TMA stage that never landed
  kStatusTimeoutEmpty = 2,      // producer waited for a stage that was never released
  kStatusTimeoutTmemFull = 3,   // epilogue waited for an accumulator that never completed
  kStatusTimeoutTmemEmpty = 4,  // MMA issuer waited for an accumulator that was never drained
  kStatusTimeoutPeer = 5,       // wait on a flag written by another GPU ran out
  kStatusBadArgs = 6,
  kStatusTimeoutGrid = 7,       // a grid-wide barrier inside a persistent kernel was not completed
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}

__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)),
               "r"(bytes)
               : "memory");
}

__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
      "selp.u32 %0, 1, 0, p;\n"
      "}\n"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}

// ---- bounded waits ------------------------------------------------------------------------
// Every spin in this library gives up after a time budget measured on the GPU's nanosecond
// timer (the same for on-chip barriers and for flags written by other GPUs), records a code in
// the status word and lets the caller unwind.  The budget is a per-library device variable that
// the host may change with dion_set_wait_budget_ns() on the device that is current; the Python
// loader does so when DION_B200_WAIT_BUDGET_MS is set.
__device__ unsigned long long g_wait_budget_ns = 2000000000ull;  // 2 s

__device__ __forceinline__ unsigned long long global_timer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

// Polls that run before the clock is consulted at all (the common case ends well inside them).
constexpr uint32_t kFreePolls = 2048;
// The timer is read once per this many further polls.
constexpr uint32_t kPollsPerClockRead = 64;

struct WaitBudget {
  unsigned long long t0 = 0;
  uint32_t polls = 0;
  // Call after every unsuccessful poll; true once the budget is spent.
  __device__ __forceinline__ bool spent() {
    ++polls;
    if (polls < kFreePolls) return false;
    if (polls == kFreePolls) {
      t0 = global_timer_ns();
      return false;
    }
    if ((polls & (kPollsPerClockRead - 1)) != 0) return false;
    return global_timer_ns() - t0 > g_wait_budget_ns;
  }
};

// Waits for the barrier phase; returns false once the time budget is spent.
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t* bar, uint32_t parity) {
  WaitBudget budget;
  for (;;) {
    if (mbar_try_wait(bar, parity)) return true;
    if (budget.spent()) return false;
  }
}

// status[0] = error code, [1] = index of the flag (source rank) that did not arrive,
// [2] = sequence number waited for, [3] = value found.  The first reporter wins.
__device__ __forceinline__ void report_peer_timeout(int* status, int who, int want, int found) {
  if (status != nullptr && atomicCAS(status, 0, kStatusTimeoutPeer) == 0) {
    status[1] = who;
    status[2] = want;
    status[3] = found;
  }
}

// True when a kernel has already recorded an error in the status word.
__device__ __forceinline__ bool status_is_set(const int* status) {
  if (status == nullptr) return false;
  int v;
  asm volatile("ld.volatile.global.s32 %0, [%1];" : "=r"(v) : "l"(status) : "memory");
  return v != 0;
}

// Waits until *flag >= want (flag written by another GPU, or by the host); false on timeout.
__device__ __forceinline__ bool flag_wait_bounded(const int* flag, int want) {
  WaitBudget budget;
  for (;;) {
    int v;
    asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(flag) : "memory");
    if (v >= want) return true;
    if (budget.spent()) return false;
    __nanosleep(64);
  }
}

__device__ __forceinline__ void fence_barrier_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void fence_proxy_async() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

// ---- TMA (tiled, no multicast) ------------------------------------------------------------
__device__ __forceinline__ void tma_load_3d(void* smem_dst, const CUtensorMap* map, uint64_t* bar,
                                            int x, int y, int z) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes "
      "[%0], [%1, {%3, %4, %5}], [%2];" ::"r"(smem_u32(smem_dst)),
      "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(x), "r"(y), "r"(z)
      : "memory");
}

__device__ __forceinline__ void prefetch_tmap(const CUtensorMap* map) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(map)) : "memory");
}

// ---- tcgen05 ------------------------------------------------------------------------------
__device__ __forceinline__ void tmem_alloc(uint32_t* smem_result, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                   smem_u32(smem_result)),
               "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tc_fence_before() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
// Arrives on the mbarrier once all tcgen05.mma issued so far by this thread have completed.
__device__ __forceinline__ void tc_commit(uint64_t* bar) {
  asm volatile(
      "tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
          smem_u32(bar))
      : "memory");
}
// D[tmem] (+)= A[smem] * B[smem], bf16 inputs, fp32 accumulate.
__device__ __forceinline__ void tc_mma_bf16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                            uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n"
      "}\n" ::"r"(d_tmem),
      "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}

// 32 lanes x 32 consecutive fp32 columns: thread i of the warp receives lane (base+i).
__device__ __forceinline__ void tmem_ld_32x32(uint32_t taddr, float* v) {
  uint32_t* r = reinterpret_cast<uint32_t*>(v);
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]),
        "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
        "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() {
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// Shared-memory matrix descriptor for tcgen05.mma, 128-byte swizzle.
//   K-major operand : rows of 64 bf16 (128 B) stacked densely; 8-row groups 1024 B apart.
//   MN-major operand: 64 MN-elements (128 B) per K-row, 8 K-rows per 1024-B atom (stride_bytes),
//                     next 64 MN-elements `lead_bytes` further on.
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t saddr, uint32_t lead_bytes,
                                                   uint32_t stride_bytes) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((saddr & 0x3FFFF) >> 4);
  d |= static_cast<uint64_t>((lead_bytes >> 4) & 0x3FFF) << 16;
  d |= static_cast<uint64_t>((stride_bytes >> 4) & 0x3FFF) << 32;
  d |= static_cast<uint64_t>(1) << 46;  // descriptor version for sm_100
  d |= static_cast<uint64_t>(2) << 61;  // SWIZZLE_128B
  return d;
}

// Instruction descriptor for kind::f16 with bf16 operands and fp32 accumulation.
__host__ __device__ constexpr uint32_t make_idesc_bf16(int m, int n, int a_mn_major,
                                                       int b_mn_major) {
  return (1u << 4)                                   // D format: fp32
         | (1u << 7)                                 // A format: bf16
         | (1u << 10)                                // B format: bf16
         | (static_cast<uint32_t>(a_mn_major) << 15) // A major
         | (static_cast<uint32_t>(b_mn_major) << 16) // B major
         | (static_cast<uint32_t>(n >> 3) << 17)     // N / 8
         | (static_cast<uint32_t>(m >> 4) << 24);    // M / 16
}

__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}
__device__ __forceinline__ float2 unpack_bf16x2(uint32_t u) {
  __nv_bfloat162 v = *reinterpret_cast<__nv_bfloat162*>(&u);
  return __bfloat1622float2(v);
}

}  // namespace dion

// One definition per library (each .cu includes this header once).
DION_EXPORT int dion_set_wait_budget_ns(unsigned long long ns) {
  return cudaMemcpyToSymbol(dion::g_wait_budget_ns, &ns, sizeof(ns)) == cudaSuccess ? 0 : -1;
}
