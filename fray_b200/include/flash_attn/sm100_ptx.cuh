#pragma once
// Thin inline-PTX wrappers for the Blackwell (sm_100a) features the attention kernels use:
// mbarriers with bounded waits, TMA tensor copies, tensor memory (TMEM) management,
// tcgen05 MMA issue/commit and TMEM load/store. Nothing here depends on CUTLASS/CuTe.
//
// Every wait in this file is bounded: when a barrier does not flip within
// kWaitLimitCycles the waiter records a site code in `fray_attn_status`, raises the
// CTA-wide abort flag and returns, so a protocol error ends as a wrong answer plus a
// status word instead of a hung GPU.

#include <cuda.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

// 16-bit operand type of this translation unit: fp16 by default, bf16 when bf16_operands.cuh was
// included first (the JIT does that for bf16 tensors; every built library has one operand type).
#ifdef FRAY_ATTN_BF16
#include <cuda_bf16.h>
#endif

namespace fray {
#ifdef FRAY_ATTN_BF16
using operand_t = __nv_bfloat16;
static constexpr int kOperandIsBf16 = 1;
#else
using operand_t = __half;
static constexpr int kOperandIsBf16 = 0;
#endif

namespace sm100 {

// Sticky device status: [0] = first failing site code (0 = healthy), [1] = block x,
// [2] = block y, [3] = extra. A non-zero [0] makes later CTAs return at entry.
__device__ int fray_attn_status[4] = {0, 0, 0, 0};

// Cycle budget of one wait.  A translation unit may define FRAY_WAIT_LIMIT_CYCLES before including this
// file (the wait-timeout test does, to make a wait run out in a millisecond).
#ifndef FRAY_WAIT_LIMIT_CYCLES
#define FRAY_WAIT_LIMIT_CYCLES 400000000LL  // ~0.2 s at 1.9 GHz
#endif
static constexpr long long kWaitLimitCycles = FRAY_WAIT_LIMIT_CYCLES;

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}


// ---------------------------------------------------------------- mbarrier
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void fence_barrier_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
// Orders generic-proxy shared-memory writes before later async-proxy (TMA / MMA) reads.
__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
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
      "selp.b32 %0, 1, 0, p;\n"
      "}\n"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}

__device__ __noinline__ void report_timeout(volatile uint32_t* abort_flag, uint32_t site, uint32_t extra) {
  *abort_flag = 1;
  if (atomicCAS(&fray_attn_status[0], 0, static_cast<int>(site)) == 0) {
    fray_attn_status[1] = blockIdx.x;
    fray_attn_status[2] = blockIdx.y;
    fray_attn_status[3] = static_cast<int>(extra);
  }
}

// Waits for the phase with the given parity to complete. Returns early (without the
// barrier having flipped) when the CTA abort flag is up or the cycle limit is hit.
__device__ __forceinline__ void mbar_wait(uint64_t* bar, uint32_t parity, volatile uint32_t* abort_flag,
                                          uint32_t site, uint32_t extra = 0) {
  if (mbar_try_wait(bar, parity)) return;
  const long long t0 = clock64();
  uint32_t polls = 0;
  while (!mbar_try_wait(bar, parity)) {
    if ((++polls & 31u) == 0u) {
      if (*abort_flag) return;
      if (clock64() - t0 > kWaitLimitCycles) {
        report_timeout(abort_flag, site, extra);
        return;
      }
    }
  }
}


// Same contract as mbar_wait, but polls with the non-blocking test_wait instead of the suspending
// try_wait.  A suspended waiter was measured to resume a few hundred cycles after the barrier
// flips; on the hand-overs that sit on the critical path (scores ready, probabilities ready) a
// polling waiter reacts within a shared-memory round trip at the price of a few issue slots.
__device__ __forceinline__ bool mbar_test_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n"
      "selp.b32 %0, 1, 0, p;\n"
      "}\n"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
__device__ __forceinline__ void mbar_wait_spin(uint64_t* bar, uint32_t parity, volatile uint32_t* abort_flag,
                                               uint32_t site, uint32_t extra = 0) {
  if (mbar_test_wait(bar, parity)) return;
  const long long t0 = clock64();
  uint32_t polls = 0;
  while (!mbar_test_wait(bar, parity)) {
    if ((++polls & 255u) == 0u) {
      if (*abort_flag) return;
      if (clock64() - t0 > kWaitLimitCycles) {
        report_timeout(abort_flag, site, extra);
        return;
      }
    }
  }
}

// ---------------------------------------------------------------- CTA pairs (clusters of two)
// Rank of this CTA inside its cluster (0 for a kernel launched without clusters).
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// Shared-memory address of the same object in the CTA of rank `cta` of this cluster.
__device__ __forceinline__ uint32_t mapa_shared(uint32_t smem_addr, uint32_t cta) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr), "r"(cta));
  return r;
}
__device__ __forceinline__ uint32_t ld_shared_cluster_u32(uint32_t cluster_addr) {
  uint32_t v;
  asm volatile("ld.shared::cluster.u32 %0, [%1];" : "=r"(v) : "r"(cluster_addr) : "memory");
  return v;
}
// All threads of both CTAs meet; memory operations before it are visible cluster-wide after it.
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\nbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// Arrive on an mbarrier named by a cluster-wide address (this CTA's or the peer's).  Plain CTA-scope
// release: what these arrivals hand over lives in tensor memory (ordered by the tcgen05 fences around
// them) or was written by the copy engine (ordered by its own byte-count completion), never in generic
// memory of the other CTA; a cluster-scope release was measured to cost ~700 cycles per arrival.
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}

// ---------------------------------------------------------------- TMA
__device__ __forceinline__ void prefetch_tensormap(const CUtensorMap* m) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(m)) : "memory");
}

// 4-D tiled load global -> shared (this CTA), completion counted in bytes on `bar`.
__device__ __forceinline__ void tma_load_4d(void* smem_dst, const CUtensorMap* map, uint64_t* bar, int c0,
                                            int c1, int c2, int c3) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4, %5, %6}], [%2];"
      :
      : "r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(c0), "r"(c1),
        "r"(c2), "r"(c3)
      : "memory");
}

// The same copy issued by a CTA of a pair: the data lands in this CTA's shared memory, the byte
// count is signalled on `bar_cluster_addr`, a cluster-wide mbarrier address that may name the
// peer CTA's barrier (the pair's leader collects the arrivals of both halves of an operand).
// No multicast: each CTA fetches exactly the half it holds.
__device__ __forceinline__ void tma_load_4d_pair(void* smem_dst, const CUtensorMap* map, uint32_t bar_cluster_addr,
                                                 int c0, int c1, int c2, int c3) {
  asm volatile(
      "cp.async.bulk.tensor.4d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4, %5, %6}], [%2];"
      :
      : "r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar_cluster_addr), "r"(c0), "r"(c1),
        "r"(c2), "r"(c3)
      : "memory");
}

// 4-D tiled store shared -> global, tracked by the issuing thread's bulk group.
__device__ __forceinline__ void tma_store_4d(const CUtensorMap* map, const void* smem_src, int c0, int c1,
                                             int c2, int c3) {
  asm volatile(
      "cp.async.bulk.tensor.4d.global.shared::cta.bulk_group"
      " [%0, {%2, %3, %4, %5}], [%1];"
      :
      : "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(smem_src)), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
      : "memory");
}
__device__ __forceinline__ void tma_store_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
__device__ __forceinline__ void tma_store_wait_read() {
  asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
}

// ---------------------------------------------------------------- TMEM management
__device__ __forceinline__ void tmem_alloc(uint32_t* slot_in_smem, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(slot_in_smem)),
               "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before_sync() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after_sync() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// ---------------------------------------------------------------- MMA descriptors
// Shared-memory operand descriptor, 128-byte swizzle, tile base 1024-byte aligned.
//   bits [0,14)  start address >> 4        bits [16,30) leading byte offset >> 4
//   bits [32,46) stride byte offset >> 4   bits [46,48) version = 1
//   bits [61,64) layout type, 2 = SWIZZLE_128B
__host__ __device__ constexpr uint64_t smem_desc_sw128(uint32_t lbo_bytes, uint32_t sbo_bytes) {
  return (static_cast<uint64_t>((lbo_bytes >> 4) & 0x3FFF) << 16) |
         (static_cast<uint64_t>((sbo_bytes >> 4) & 0x3FFF) << 32) | (1ull << 46) | (2ull << 61);
}
__device__ __forceinline__ uint64_t smem_desc_at(uint64_t desc_template, uint32_t smem_addr) {
  return desc_template | static_cast<uint64_t>((smem_addr & 0x3FFFF) >> 4);
}

// Instruction descriptor for kind::f16 with fp16 A/B and fp32 accumulation.
//   bits [4,6) D format (1 = f32), [7,10) A format (0 = f16, 1 = bf16), [10,13) B format,
//   bit 15 A major (1 = MN), bit 16 B major (1 = MN), [17,23) N >> 3, [24,29) M >> 4.
__host__ __device__ constexpr uint32_t idesc_f16_f32(int m, int n, bool a_mn_major, bool b_mn_major) {
  return (1u << 4) | (static_cast<uint32_t>(kOperandIsBf16) << 7) | (static_cast<uint32_t>(kOperandIsBf16) << 10) |
         (static_cast<uint32_t>(a_mn_major) << 15) | (static_cast<uint32_t>(b_mn_major) << 16) |
         (static_cast<uint32_t>(n >> 3) << 17) | (static_cast<uint32_t>(m >> 4) << 24);
}

// D[tmem] (+)= A[smem] * B[smem]
__device__ __forceinline__ void mma_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                       uint32_t accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n"
      "}\n"
      :
      : "r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// D[tmem] (+)= A[tmem] * B[smem]
__device__ __forceinline__ void mma_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc,
                                       uint32_t accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n"
      "}\n"
      :
      : "r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Split-descriptor forms: the shared-memory descriptors are passed as (low, high) 32-bit halves
// and joined inside the instruction block.  Only the low half (the start address) changes from
// one K step to the next, so an unrolled issue sequence needs one 32-bit value per operand and
// step instead of a 64-bit pair, which keeps the issuing warp inside a small register budget.
__device__ __forceinline__ void mma_ss_elect_lohi(uint32_t d_tmem, uint32_t a_lo, uint32_t a_hi, uint32_t b_lo,
                                                  uint32_t b_hi, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p, e;\n"
      ".reg .b64 da, db;\n"
      "mov.b64 da, {%1, %2};\n"
      "mov.b64 db, {%3, %4};\n"
      "elect.sync _|e, 0xffffffff;\n"
      "setp.ne.b32 p, %6, 0;\n"
      "@e tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %5, p;\n"
      "}\n"
      :
      : "r"(d_tmem), "r"(a_lo), "r"(a_hi), "r"(b_lo), "r"(b_hi), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void mma_ts_elect_lohi(uint32_t d_tmem, uint32_t a_tmem, uint32_t b_lo, uint32_t b_hi,
                                                  uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p, e;\n"
      ".reg .b64 db;\n"
      "mov.b64 db, {%2, %3};\n"
      "elect.sync _|e, 0xffffffff;\n"
      "setp.ne.b32 p, %5, 0;\n"
      "@e tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], db, %4, p;\n"
      "}\n"
      :
      : "r"(d_tmem), "r"(a_tmem), "r"(b_lo), "r"(b_hi), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void mma_commit_elect(uint64_t* bar) {
  asm volatile(
      "{\n"
      ".reg .pred e;\n"
      "elect.sync _|e, 0xffffffff;\n"
      "@e tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n"
      "}\n" ::"r"(smem_u32(bar))
      : "memory");
}

// CTA-pair forms (cta_group::2): issued by one thread of the pair's leader (even rank).  The product
// has M = 256 rows, 128 per CTA; each CTA supplies its own rows of A (shared memory or tensor memory at
// the same addresses in both CTAs) and one half of B along N; each CTA's tensor memory receives its 128
// rows of D.
template <int CTAS>
__device__ __forceinline__ void mma_ss_elect_g(uint32_t d_tmem, uint32_t a_lo, uint32_t a_hi, uint32_t b_lo,
                                               uint32_t b_hi, uint32_t idesc, uint32_t accumulate) {
  if constexpr (CTAS == 1) {
    mma_ss_elect_lohi(d_tmem, a_lo, a_hi, b_lo, b_hi, idesc, accumulate);
  } else {
    asm volatile(
        "{\n"
        ".reg .pred p, e;\n"
        ".reg .b64 da, db;\n"
        "mov.b64 da, {%1, %2};\n"
        "mov.b64 db, {%3, %4};\n"
        "elect.sync _|e, 0xffffffff;\n"
        "setp.ne.b32 p, %6, 0;\n"
        "@e tcgen05.mma.cta_group::2.kind::f16 [%0], da, db, %5, p;\n"
        "}\n"
        :
        : "r"(d_tmem), "r"(a_lo), "r"(a_hi), "r"(b_lo), "r"(b_hi), "r"(idesc), "r"(accumulate)
        : "memory");
  }
}
template <int CTAS>
__device__ __forceinline__ void mma_ts_elect_g(uint32_t d_tmem, uint32_t a_tmem, uint32_t b_lo, uint32_t b_hi,
                                               uint32_t idesc, uint32_t accumulate) {
  if constexpr (CTAS == 1) {
    mma_ts_elect_lohi(d_tmem, a_tmem, b_lo, b_hi, idesc, accumulate);
  } else {
    asm volatile(
        "{\n"
        ".reg .pred p, e;\n"
        ".reg .b64 db;\n"
        "mov.b64 db, {%2, %3};\n"
        "elect.sync _|e, 0xffffffff;\n"
        "setp.ne.b32 p, %5, 0;\n"
        "@e tcgen05.mma.cta_group::2.kind::f16 [%0], [%1], db, %4, p;\n"
        "}\n"
        :
        : "r"(d_tmem), "r"(a_tmem), "r"(b_lo), "r"(b_hi), "r"(idesc), "r"(accumulate)
        : "memory");
  }
}
// Arrives once on `bar` (the barrier at this shared-memory offset in BOTH CTAs of a pair when CTAS == 2)
// when every MMA issued so far by the elected thread has completed.
template <int CTAS>
__device__ __forceinline__ void mma_commit_elect_g(uint64_t* bar) {
  if constexpr (CTAS == 1) {
    mma_commit_elect(bar);
  } else {
    asm volatile(
        "{\n"
        ".reg .pred e;\n"
        ".reg .b16 m;\n"
        "mov.b16 m, 3;\n"
        "elect.sync _|e, 0xffffffff;\n"
        "@e tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], m;\n"
        "}\n" ::"r"(smem_u32(bar))
        : "memory");
  }
}


// Arrives once on `bar` when every MMA issued so far by this thread has completed.
__device__ __forceinline__ void mma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
               : "memory");
}

// ---------------------------------------------------------------- TMEM load / store




// Each lane of the warp writes 16 consecutive 32-bit columns of its own TMEM lane.
__device__ __forceinline__ void tmem_st_x16(uint32_t taddr, const uint32_t (&r)[16]) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x16.b32 [%16], {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15};"
               :
               : "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(taddr)
               : "memory");
}

// Each lane of the warp reads 32 consecutive 32-bit columns of its own TMEM lane.
__device__ __forceinline__ void tmem_ld_x16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
               : "r"(taddr)
               : "memory");
}
__device__ __forceinline__ void tmem_ld_x32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
               : "r"(taddr)
               : "memory");
}

// Each lane of the warp writes 32 consecutive 32-bit columns of its own TMEM lane.
__device__ __forceinline__ void tmem_st_x32(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x32.b32 [%32], {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31};"
               :
               : "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31]), "r"(taddr)
               : "memory");
}



// ---------------------------------------------------------------- small math helpers
__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float max3(float a, float b, float c) {
  float r;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(a), "f"(b), "f"(c));
  return r;
}
// Two-lane packed fp32 arithmetic (one issue slot for two elements).
__device__ __forceinline__ uint64_t pack_f32x2(float lo, float hi) {
  uint64_t r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
  return r;
}
__device__ __forceinline__ void unpack_f32x2(uint64_t v, float& lo, float& hi) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ uint64_t fma_f32x2(uint64_t a, uint64_t b, uint64_t c) {
  uint64_t r;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
  return r;
}
__device__ __forceinline__ uint64_t add_f32x2(uint64_t a, uint64_t b) {
  uint64_t r;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
  return r;
}
// 2^x for two values on the FMA/ALU pipes instead of the special-function unit: round x to the
// nearest integer n with the 1.5*2^23 trick, evaluate a cubic for 2^(x-n) on [-0.5, 0.5]
// (max relative error 7.5e-5, below fp16 rounding) and add n to the exponent field.
// Inputs are clamped at -120 so the exponent arithmetic cannot wrap (-inf included).
__device__ __forceinline__ float ex2_poly(float x) {
  x = fmaxf(x, -120.f);
  const float t = x + 12582912.f;          // low mantissa bits now hold round(x)
  const float f = x - (t - 12582912.f);    // in [-0.5, 0.5]
  float q = fmaf(0.0551716685f, f, 0.2426111251f);
  q = fmaf(q, f, 0.6932609677f);
  q = fmaf(q, f, 0.9999280572f);
  return __uint_as_float(__float_as_uint(q) + (__float_as_uint(t) << 23));
}
// 2^x for a packed pair on the FMA/ALU pipes: the same cubic as ex2_poly with the additions and the
// Horner steps as packed f32x2 instructions (one issue slot per pair), the clamp and the exponent
// insertion per element.
__device__ __forceinline__ uint64_t ex2_poly_f32x2(uint64_t x2) {
  float x0, x1;
  unpack_f32x2(x2, x0, x1);
  x0 = fmaxf(x0, -120.f);
  x1 = fmaxf(x1, -120.f);
  const uint64_t xc = pack_f32x2(x0, x1);
  const uint64_t magic = pack_f32x2(12582912.f, 12582912.f);
  const uint64_t neg_magic = pack_f32x2(-12582912.f, -12582912.f);
  const uint64_t t = add_f32x2(xc, magic);                 // low mantissa bits hold round(x)
  const uint64_t r = add_f32x2(t, neg_magic);              // round(x) as a float
  const uint64_t f = fma_f32x2(r, pack_f32x2(-1.f, -1.f), xc);  // x - round(x) in [-0.5, 0.5]
  uint64_t q = fma_f32x2(pack_f32x2(0.0551716685f, 0.0551716685f), f, pack_f32x2(0.2426111251f, 0.2426111251f));
  q = fma_f32x2(q, f, pack_f32x2(0.6932609677f, 0.6932609677f));
  q = fma_f32x2(q, f, pack_f32x2(0.9999280572f, 0.9999280572f));
  float q0, q1, t0, t1;
  unpack_f32x2(q, q0, q1);
  unpack_f32x2(t, t0, t1);
  const uint32_t e0 = __float_as_uint(q0) + (__float_as_uint(t0) << 23);
  const uint32_t e1 = __float_as_uint(q1) + (__float_as_uint(t1) << 23);
  return pack_f32x2(__uint_as_float(e0), __uint_as_float(e1));
}
// Two fp32 values rounded to nearest into a pair of the 16-bit operand type (fp16, or bf16 in a
// bf16 build), low element first.
__device__ __forceinline__ uint32_t pack_half2(float lo, float hi) {
  uint32_t r;
#ifdef FRAY_ATTN_BF16
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
#else
  asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
#endif
  return r;
}

}  // namespace sm100
}  // namespace fray
