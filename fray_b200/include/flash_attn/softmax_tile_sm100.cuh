#pragma once
// Pieces shared by the warp-specialised attention kernels: register budgets, named barriers, the
// timeline macros, the softmax step of the two-tile kernel (a softmax thread owns one query row of a
// 128-key score tile that sits in tensor memory, turns it into 16-bit probabilities in place, handing
// them to the MMA warp chunk by chunk, and updates the row's running state) and the tile epilogue.
//
// Arithmetic restated from the reference (fray/include/flash_attn/softmax.cuh:24-67): base-2
// exponentials with the softmax scale folded in, row sum taken from the unrounded fp32 values,
// P rounded to fp16 for the P.V product.  Difference: the exponent offset is moved lazily (see
// kRescaleThreshold) instead of on every tile; O and l always share the offset, so O/l is unchanged.

#include "sm100_ptx.cuh"

namespace fray {
namespace sm100 {

template <int N>
__device__ __forceinline__ void set_max_regs_inc() {
  asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(N));
}
template <int N>
__device__ __forceinline__ void set_max_regs_dec() {
  asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(N));
}
__device__ __forceinline__ void named_barrier_sync(int id, int threads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}

// Waits on the critical path (scores ready, probabilities ready) use the plain suspending form: polling
// reacted no faster in measurements and executed ~30 % more instructions, which costs clock under the
// power cap, and try_wait with a short suspend-time hint (10 or 30 ns) measured 1 % slower.
#define FRAY_CRIT_WAIT mbar_wait

// Optional role timeline for bring-up and tuning: with -DFRAY_ATTN_TRACE one thread per role of
// CTA (0,0) stamps clock64 into a shared-memory table indexed by (event, tile, iteration < 40);
// the table is copied to a device buffer at the end and read back with fray_attn_trace_read.
// Compiled out by default.
#ifndef FRAY_TRACE_ROW
#define FRAY_TRACE_ROW 0  // which row's thread stamps the softmax events
#endif
#ifdef FRAY_ATTN_TRACE
static constexpr int kTraceEvents = 12, kTraceIters = 40;
static constexpr int kTraceWords = kTraceEvents * 2 * kTraceIters;
__device__ unsigned int fray_attn_trace_buf[kTraceWords];
#define FRAY_TRACE(event, tile, iter)                                                              \
  do {                                                                                             \
    if (trace_on && (iter) < kTraceIters)                                                          \
      trace_sm[((event) * 2 + (tile)) * kTraceIters + (iter)] = static_cast<unsigned int>(clock64()); \
  } while (0)
// Wall-clock stamp (nanoseconds, low 32 bits) beside a cycle stamp: the two together give the SM clock the
// kernel really ran at.
#define FRAY_TRACE_NS(event, tile, iter)                                                           \
  do {                                                                                             \
    if (trace_on) {                                                                                \
      unsigned long long ns_;                                                                      \
      asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(ns_));                                      \
      trace_sm[((event) * 2 + (tile)) * kTraceIters + (iter)] = static_cast<unsigned int>(ns_);    \
    }                                                                                              \
  } while (0)
inline int read_attn_trace(unsigned int* out, int max_words) {
  const int n = max_words < kTraceWords ? max_words : kTraceWords;
  if (cudaMemcpyFromSymbol(out, fray_attn_trace_buf, sizeof(unsigned int) * n) != cudaSuccess) return -1;
  return n;
}
#else
#define FRAY_TRACE(event, tile, iter) do { } while (0)
#define FRAY_TRACE_NS(event, tile, iter) do { } while (0)
#endif

// Timeline stamps inside the softmax step (compiled in with -DFRAY_ATTN_TRACE only): `tr` points at
// this step's slot of event 0 in the caller's table, or is null; event e lives e*80 words further.
#ifdef FRAY_ATTN_TRACE
#define FRAY_SM_TRACE(tr, e) do { if ((tr) != nullptr) (tr)[(e) * 80] = static_cast<unsigned int>(clock64()); } while (0)
#else
#define FRAY_SM_TRACE(tr, e) do { } while (0)
#endif

// Lazy-rescale threshold in the scaled base-2 domain: offsets move only when the max grew by > 2^8.
static constexpr float kRescaleThreshold = 8.0f;

// t_s        tensor-memory address of this thread's lane at column 0 of the S tile (P overwrites it)
// p_bar      PCHUNKS consecutive mbarriers, arrival count 4 (one per warp of the group): chunk q of P stored
// rescale_o  called by every thread with the factor its row of O has to be multiplied by before this
//            step's P.V (1 when the offset stays; not called on the first tile of a row): the two-tile
//            kernel publishes it to its correction group, the one-tile kernel rescales O on the spot
// first_tile no running state yet: the tile max becomes the offset
// SMALL_STORES  P is computed and stored in pieces of 32 keys (16 columns) instead of 64: fewer values live at a
//            time; in the two-tile kernel measured +1 to +3.5 % at head dim 64 and -0.3 % at 128 (it chooses by
//            head dim), in the one-tile kernel -1 to -2 % (it does not use it)
// MASK       some key of the tile is past seq_len or above the causal diagonal (two instantiations: the
//            masking code costs the unmasked steps several per cent even when it is branched around)
// The whole row is pulled into registers at once, the row max uses three-input max instructions, the
// scaling and the row sum packed f32x2 arithmetic (one issue slot per pair).  Every exponential goes
// to the special-function unit: a share by polynomial on the FMA pipe was measured slower here (the
// chain softmax -> P.V -> next S bounds this kernel, not the unit).
template <int BN, int PCHUNKS, bool MASK, bool SMALL_STORES, class Rescale>
__device__ __forceinline__ void softmax_tile_with(uint32_t t_s, uint64_t* p_bar, Rescale&& rescale_o, bool first_tile, int kv0,
                                                  int row, int seq_len, int causal, float scale_log2, int lane, float& m_ref,
                                                  float& l_run, unsigned int* tr = nullptr) {
  static_assert(BN == 128, "written for 128-key tiles");
  static_assert(PCHUNKS == 4 || PCHUNKS == 2, "P is handed over in 4 chunks of 32 keys or 2 of 64");
  static_assert(!SMALL_STORES || PCHUNKS == 2, "the 32-key pieces are written for two hand-over chunks");
  uint32_t sa[64], sb[64];
  tmem_ld_x32(t_s, reinterpret_cast<uint32_t(&)[32]>(sa[0]));
  tmem_ld_x32(t_s + 32, reinterpret_cast<uint32_t(&)[32]>(sa[32]));
  tmem_ld_x32(t_s + 64, reinterpret_cast<uint32_t(&)[32]>(sb[0]));
  tmem_ld_x32(t_s + 96, reinterpret_cast<uint32_t(&)[32]>(sb[32]));
  tmem_wait_ld();
  FRAY_SM_TRACE(tr, 1);
  if constexpr (MASK) {
#pragma unroll
    for (int c = 0; c < 64; ++c) {
      const int kv = kv0 + c;
      if (kv >= seq_len || (causal && kv > row)) sa[c] = __float_as_uint(-INFINITY);
      if (kv + 64 >= seq_len || (causal && kv + 64 > row)) sb[c] = __float_as_uint(-INFINITY);
    }
  }
  float mx0 = -INFINITY, mx1 = -INFINITY, mx2 = -INFINITY, mx3 = -INFINITY;
#pragma unroll
  for (int c = 0; c < 64; c += 4) {
    mx0 = max3(mx0, __uint_as_float(sa[c + 0]), __uint_as_float(sb[c + 0]));
    mx1 = max3(mx1, __uint_as_float(sa[c + 1]), __uint_as_float(sb[c + 1]));
    mx2 = max3(mx2, __uint_as_float(sa[c + 2]), __uint_as_float(sb[c + 2]));
    mx3 = max3(mx3, __uint_as_float(sa[c + 3]), __uint_as_float(sb[c + 3]));
  }
  const float m_new = fmaxf(fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3)), m_ref);
  if (first_tile) {
    m_ref = m_new;
  } else {
    float alpha = 1.f;
    if ((m_new - m_ref) * scale_log2 > kRescaleThreshold) {
      alpha = ex2_approx((m_ref - m_new) * scale_log2);
      l_run *= alpha;
      m_ref = m_new;
    }
    rescale_o(alpha);
  }
  FRAY_SM_TRACE(tr, 2);
  const float neg_m = (m_ref == -INFINITY) ? 0.f : -m_ref * scale_log2;
  uint64_t rsp0 = 0ull, rsp1 = 0ull;
  const uint64_t scale2 = pack_f32x2(scale_log2, scale_log2), neg_m2 = pack_f32x2(neg_m, neg_m);
  // One chunk of KEYS keys: exponentials, row sum from the unrounded values, 16-bit rounding, store as
  // chunk q of P.  The hand-over of a chunk (wait for the store, fence, arrive) is issued after the NEXT
  // chunk's arithmetic: the store's latency then hides under that arithmetic, and only the last chunk's
  // wait sits in the step.
  // keys per compute / store call: a hand-over chunk, or 32 with SMALL_STORES (two calls per chunk)
  constexpr int KEYS = SMALL_STORES ? 32 : BN / PCHUNKS;
  auto compute = [&](const uint32_t (&h)[64], int off, uint32_t (&pk)[KEYS / 2]) {
#pragma unroll
    for (int c = 0; c < KEYS; c += 8) {
      uint64_t p[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const uint64_t x = fma_f32x2(pack_f32x2(__uint_as_float(h[off + c + 2 * e]), __uint_as_float(h[off + c + 2 * e + 1])), scale2, neg_m2);
        float x0, x1;
        unpack_f32x2(x, x0, x1);
        p[e] = pack_f32x2(ex2_approx(x0), ex2_approx(x1));
      }
      rsp0 = add_f32x2(rsp0, add_f32x2(p[0], p[2]));
      rsp1 = add_f32x2(rsp1, add_f32x2(p[1], p[3]));
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        float p0, p1;
        unpack_f32x2(p[e], p0, p1);
        pk[(c >> 1) + e] = pack_half2(p0, p1);
      }
    }
  };
  auto store = [&](const uint32_t (&pk)[KEYS / 2], int q) {
    if constexpr (KEYS == 32) {
      tmem_st_x16(t_s + q * 16, pk);
    } else {
      tmem_st_x32(t_s + q * 32, pk);
    }
  };
  auto hand_over = [&](int q) {  // every store issued so far has landed: chunk q may be consumed
    tmem_wait_st();
    tc_fence_before_sync();
    __syncwarp();
    if (lane == 0) mbar_arrive(p_bar + q);
  };
  uint32_t pa[KEYS / 2], pb[KEYS / 2];
  if constexpr (PCHUNKS == 4 && !SMALL_STORES) {
    compute(sa, 0, pa);
    store(pa, 0);
    compute(sa, 32, pb);
    hand_over(0);
    store(pb, 1);
    compute(sb, 0, pa);
    hand_over(1);
    store(pa, 2);
    compute(sb, 32, pb);
    hand_over(2);
    store(pb, 3);
    hand_over(3);
  } else if constexpr (SMALL_STORES) {
    compute(sa, 0, pa);
    store(pa, 0);
    compute(sa, 32, pb);
    store(pb, 1);
    FRAY_SM_TRACE(tr, 3);
    compute(sb, 0, pa);
    FRAY_SM_TRACE(tr, 9);
    hand_over(0);
    FRAY_SM_TRACE(tr, 10);
    store(pa, 2);
    compute(sb, 32, pb);
    store(pb, 3);
    FRAY_SM_TRACE(tr, 11);
    hand_over(1);
  } else {
    compute(sa, 0, pa);
    FRAY_SM_TRACE(tr, 3);
    store(pa, 0);
    compute(sb, 0, pb);
    FRAY_SM_TRACE(tr, 9);
    hand_over(0);
    FRAY_SM_TRACE(tr, 10);
    store(pb, 1);
    FRAY_SM_TRACE(tr, 11);
    hand_over(1);
  }
  float r0, r1, r2, r3;
  unpack_f32x2(rsp0, r0, r1);
  unpack_f32x2(rsp1, r2, r3);
  l_run += (r0 + r1) + (r2 + r3);
}


// The step with the factor handed to a correction group: alpha_slot receives this row's factor, corr_bar
// (arrival count 4, one per warp) tells the group that the slots of this step are filled.
template <int BN, int PCHUNKS, bool MASK, bool SMALL_STORES = false>
__device__ __forceinline__ void softmax_tile(uint32_t t_s, uint64_t* p_bar, uint64_t* corr_bar, float* alpha_slot,
                                             bool first_tile, int kv0, int row, int seq_len, int causal, float scale_log2,
                                             int lane, float& m_ref, float& l_run, unsigned int* tr = nullptr) {
  softmax_tile_with<BN, PCHUNKS, MASK, SMALL_STORES>(
      t_s, p_bar,
      [&](float alpha) {
        *alpha_slot = alpha;
        __syncwarp();
        if (lane == 0) mbar_arrive(corr_bar);
      },
      first_tile, kv0, row, seq_len, causal, scale_log2, lane, m_ref, l_run, tr);
}

// Epilogue of one query tile, run by the 128 threads that own its rows (thread r = row r, reading its
// own tensor-memory lane): O / l -> 16-bit -> shared memory (the tile's dead Q buffer, 128B-swizzled)
// -> TMA store, and the row's log-sum-exp when asked for.  t_o includes the thread's lane offset; m is
// the row's final exponent offset in score units; barrier_id names a 128-thread barrier of the group.
// The thread with r == 0 issues and commits the store; it must wait for the store's reads of shared
// memory (tma_store_wait_read) before the CTA ends.
template <class Cfg, int D>
__device__ __forceinline__ void epilogue_tile(uint32_t t_o, uint8_t* o_tile, int r, float l, float m,
                                              const CUtensorMap* tm_o, int row0, int h, int b, int num_heads,
                                              int seq_len, float scale_log2, float* lse, int barrier_id) {
  const float inv_l = l > 0.f ? 1.f / l : 1.f;
#pragma unroll
  for (int c = 0; c < D / 32; ++c) {
    uint32_t orr[32];
    tmem_ld_x32(t_o + c * 32, orr);
    tmem_wait_ld();
    uint8_t* panel_row = o_tile + (c >> 1) * Cfg::kQPanelBytes + r * 128;
#pragma unroll
    for (int x = 0; x < 32; x += 8) {
      uint4 v4;
      v4.x = pack_half2(__uint_as_float(orr[x + 0]) * inv_l, __uint_as_float(orr[x + 1]) * inv_l);
      v4.y = pack_half2(__uint_as_float(orr[x + 2]) * inv_l, __uint_as_float(orr[x + 3]) * inv_l);
      v4.z = pack_half2(__uint_as_float(orr[x + 4]) * inv_l, __uint_as_float(orr[x + 5]) * inv_l);
      v4.w = pack_half2(__uint_as_float(orr[x + 6]) * inv_l, __uint_as_float(orr[x + 7]) * inv_l);
      const int chunk = (c & 1) * 4 + (x >> 3);  // 16-byte chunk inside the 128-byte row
      *reinterpret_cast<uint4*>(panel_row + ((chunk ^ (r & 7)) << 4)) = v4;
    }
  }
  fence_proxy_async_smem();
  named_barrier_sync(barrier_id, 128);
  if (r == 0) {
#pragma unroll
    for (int p = 0; p < Cfg::kPanels; ++p) tma_store_4d(tm_o, o_tile + p * Cfg::kQPanelBytes, p * 64, row0, h, b);
    tma_store_commit();
  }
  if (lse != nullptr && row0 + r < seq_len) {
    // log-sum-exp of the scaled scores in natural units: offset plus log of the row sum (written
    // after the tile is on its way: nothing waits for this)
    lse[(static_cast<size_t>(b) * num_heads + h) * seq_len + row0 + r] =
        l > 0.f ? (m * scale_log2 + log2f(l)) * 0.69314718055994531f : -INFINITY;
  }
}

}  // namespace sm100
}  // namespace fray
