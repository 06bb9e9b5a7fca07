#pragma once
// One softmax step of the warp-specialised attention kernels: a softmax thread owns one query
// row of a 128-key score tile that sits in tensor memory, turns it into fp16 probabilities in
// place (handing them to the MMA warp chunk by chunk) and updates the row's running state.
//
// Arithmetic restated from the reference (fray/include/flash_attn/softmax.cuh:24-67): base-2
// exponentials with the softmax scale folded in, row sum taken from the unrounded fp32 values,
// P rounded to fp16 for the P.V product.  Difference: the exponent offset is moved lazily (see
// kRescaleThreshold) instead of on every tile; O and l always share the offset, so O/l is unchanged.

#include "sm100_ptx.cuh"

namespace fray {
namespace sm100 {

// Compile-time integer tag for generic lambdas.
template <int V>
struct SmInt {
  static constexpr int value = V;
};

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

// Waits on the critical path (scores ready, probabilities ready).  The suspending form is the
// default: polling (-DFRAY_POLLING_WAITS) reacted no faster in measurements and executed ~30 % more
// instructions, which costs clock under the power cap.
#ifdef FRAY_POLLING_WAITS
#define FRAY_CRIT_WAIT mbar_wait_spin
#else
#define FRAY_CRIT_WAIT mbar_wait
#endif

// Whether the two softmax groups take turns on the special-function unit (-DFRAY_SFU_TURNS=0/1).
#ifndef FRAY_SFU_TURNS
#define FRAY_SFU_TURNS 0  // measured slower than letting the groups overlap freely
#endif
static constexpr bool kSfuTurns = FRAY_SFU_TURNS != 0;

// Whether the first copies of a CTA are issued during set-up, before the roles separate
// (-DFRAY_EARLY_COPIES=0/1).  Measured on one box: +3 % for the whole-tile kernel on short causal
// CTAs, nothing on the headline shape, -4 % for the half-step kernel; off.
#ifndef FRAY_EARLY_COPIES
#define FRAY_EARLY_COPIES 0
#endif
static constexpr bool kEarlyCopies = FRAY_EARLY_COPIES != 0;

// Timeline stamps inside the softmax step (compiled in with -DFRAY_ATTN_TRACE only): `tr` points at
// this step's slot of event 0 in the caller's table, or is null; event e lives e*80 words further.
#ifdef FRAY_ATTN_TRACE
#define FRAY_SM_TRACE(tr, e) do { if ((tr) != nullptr) (tr)[(e) * 80] = static_cast<unsigned int>(clock64()); } while (0)
#else
#define FRAY_SM_TRACE(tr, e) do { } while (0)
#endif

// Lazy-rescale threshold in the scaled base-2 domain: offsets move only when the max grew by > 2^8.
static constexpr float kRescaleThreshold = 8.0f;
// P is handed to the MMA warp in this many column chunks (one mbarrier each, one arrival per warp).
static constexpr int kSoftmaxPChunks = 4;
// Value of the POLY tuning key that selects packed fp16 exponentials.
static constexpr int kExpPackedHalf = 16;

// t_s        tensor-memory address of this thread's lane at column 0 of the S tile (P overwrites it)
// p_bar      kSoftmaxPChunks consecutive mbarriers, arrival count 4 (one per warp of the group)
// corr_bar   mbarrier (count 4) telling the correction group that alpha_slot holds this step's factor
// alpha_slot where this row's rescale factor is published (skipped on the first tile of a row)
// my_turn / other_turn  when not null, the special-function work of the two softmax groups is
//            serialised: this group waits on my_turn (phase parity turn_parity) before its first
//            exponential and arrives on other_turn (count 4, one arrival per warp) after its last.
//            The two groups need the unit for as long as the tensor pipe needs for both tiles, so
//            letting them overlap freely only stretches both; taking turns keeps one tile in its
//            exponentials while the other owns the tensor pipe.
// first_tile no running state yet: the tile max becomes the offset, nothing is published
// need_mask  some key of the tile is past seq_len or above the causal diagonal
// POLY       exponential mode: 0..4 = of every 4 element pairs, how many take the polynomial exp2
//            instead of the fp32 special-function instruction; kExpPackedHalf (16) = the scaled
//            scores are rounded to fp16 first and two exponentials are taken per instruction
//            (ex2.approx.f16x2), the fp16 results being P itself; the row sum is then gathered in
//            fp16 groups of 8 before it joins the fp32 total.  P is rounded to fp16 for the P.V
//            product in every mode; the packed mode also rounds the exponent argument, which costs
//            about 2x in calc_diff (1e-7 instead of 4e-8, against a bound of 1e-5) and halves the
//            special-function work, the scarcest resource of this kernel.
template <int BN, int POLY>
__device__ __forceinline__ void softmax_tile(uint32_t t_s, uint64_t* p_bar, uint64_t* corr_bar, float* alpha_slot,
                                             bool first_tile, bool need_mask, int kv0, int row, int seq_len, int causal,
                                             float scale_log2, int lane, float& m_ref, float& l_run,
                                             uint64_t* my_turn, uint64_t* other_turn, uint32_t turn_parity,
                                             volatile uint32_t* abort_flag) {
  static_assert(BN == 128, "written for 128-key tiles");
  static_assert(POLY != kExpPackedHalf || !kOperandIsBf16, "the packed exponentials produce fp16");
  constexpr int kChunkCols = BN / kSoftmaxPChunks;  // 32 keys per chunk -> 16 packed fp16 columns

  // Register diet: the row is handled as two 64-key halves.  Both are loaded once for the row
  // max; only the first stays in registers for its exponentials, and the second is fetched from
  // tensor memory again afterwards (a ~100-cycle load) instead of being held.  With 128 live
  // score registers the scheduler had too little room to overlap the dependent FFMA -> MUFU ->
  // FADD/convert chains and the loop ran well below the special-function unit's rate.
  auto load_half = [&](uint32_t (&h)[64], int half) {
    tmem_ld_x32(t_s + half * 64, reinterpret_cast<uint32_t(&)[32]>(h[0]));
    tmem_ld_x32(t_s + half * 64 + 32, reinterpret_cast<uint32_t(&)[32]>(h[32]));
  };
  auto mask_half = [&](uint32_t (&h)[64], int half) {
#pragma unroll
    for (int c = 0; c < 64; ++c) {
      const int kv = kv0 + half * 64 + c;
      if (kv >= seq_len || (causal && kv > row)) h[c] = __float_as_uint(-INFINITY);
    }
  };

  uint32_t sa[64];
  float mx[8];
#pragma unroll
  for (int q = 0; q < 8; ++q) mx[q] = -INFINITY;
  {
    uint32_t sb[64];
    load_half(sa, 0);
    load_half(sb, 1);
    tmem_wait_ld();
    if (need_mask) {
      mask_half(sa, 0);
      mask_half(sb, 1);
    }
#pragma unroll
    for (int c = 0; c < 64; c += 8) {
#pragma unroll
      for (int q = 0; q < 8; ++q) mx[q] = fmaxf(mx[q], fmaxf(__uint_as_float(sa[c + q]), __uint_as_float(sb[c + q])));
    }
  }
  const float m_new = fmaxf(
      fmaxf(fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3])), fmaxf(fmaxf(mx[4], mx[5]), fmaxf(mx[6], mx[7]))), m_ref);
  if (first_tile) {
    m_ref = m_new;
  } else {
    float alpha = 1.f;
    if ((m_new - m_ref) * scale_log2 > kRescaleThreshold) {
      alpha = ex2_approx((m_ref - m_new) * scale_log2);
      l_run *= alpha;
      m_ref = m_new;
    }
    *alpha_slot = alpha;
    __syncwarp();
    if (lane == 0) mbar_arrive(corr_bar);
  }
  const float neg_m = (m_ref == -INFINITY) ? 0.f : -m_ref * scale_log2;

  if constexpr (POLY == kExpPackedHalf) {
    // Packed mode: one chunk of 32 keys at a time, exponentials, row sum and the store together.
    uint32_t acc[8];
#pragma unroll
    for (int q = 0; q < 8; ++q) acc[q] = 0u;  // +0.0 twice
    auto chunk16 = [&](const uint32_t (&h)[64], int off, int q) {
      uint32_t pk[kChunkCols / 2];
#pragma unroll
      for (int c = 0; c < kChunkCols; c += 2) {
        const float x0 = fmaf(__uint_as_float(h[off + c]), scale_log2, neg_m);
        const float x1 = fmaf(__uint_as_float(h[off + c + 1]), scale_log2, neg_m);
        const uint32_t p = ex2_approx_f16x2(pack_half2(x0, x1));
        acc[(c >> 1) & 7] = add_f16x2(acc[(c >> 1) & 7], p);  // 8 terms of at most 2^8 each per slot
        pk[c >> 1] = p;
      }
      tmem_st_x16(t_s + q * (kChunkCols / 2), pk);
      tmem_wait_st();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(p_bar + q);
    };
    uint32_t sb2[64];
    load_half(sb2, 1);  // second half again; it sits at columns [64,128), clear of chunks 0 and 1
    chunk16(sa, 0, 0);
    chunk16(sa, 32, 1);
    tmem_wait_ld();
    if (need_mask) mask_half(sb2, 1);
    chunk16(sb2, 0, 2);
    chunk16(sb2, 32, 3);
    float r0 = 0.f, r1 = 0.f;
#pragma unroll
    for (int q = 0; q < 8; ++q) {
      float lo, hi;
      unpack_half2(acc[q], lo, hi);
      r0 += lo;
      r1 += hi;
    }
    l_run += r0 + r1;
    return;
  }

  float rs0 = 0.f, rs1 = 0.f, rs2 = 0.f, rs3 = 0.f;
  // h[...] <- exp2(S*c - m*c) for one 64-key half, in place.
  auto exp_half = [&](uint32_t (&h)[64]) {
#pragma unroll
    for (int c = 0; c < 64; c += 2) {
      const float x0 = fmaf(__uint_as_float(h[c]), scale_log2, neg_m);
      const float x1 = fmaf(__uint_as_float(h[c + 1]), scale_log2, neg_m);
      float p0, p1;
      if (((c >> 1) & 3) < POLY) {
        ex2_poly_pair(x0, x1, p0, p1);
      } else {
        p0 = ex2_approx(x0);
        p1 = ex2_approx(x1);
      }
      h[c] = __float_as_uint(p0);
      h[c + 1] = __float_as_uint(p1);
    }
  };
  // Round 32 keys to fp16, add them to the row sum, store them to tensor memory as chunk q and
  // hand the chunk to the MMA warp once the store has landed.
  auto store_publish = [&](const uint32_t (&h)[64], int off, int q) {
    uint32_t pk[kChunkCols / 2];
#pragma unroll
    for (int c = 0; c < kChunkCols; c += 4) {
      const float p0 = __uint_as_float(h[off + c]), p1 = __uint_as_float(h[off + c + 1]);
      const float p2 = __uint_as_float(h[off + c + 2]), p3 = __uint_as_float(h[off + c + 3]);
      rs0 += p0;
      rs1 += p1;
      rs2 += p2;
      rs3 += p3;
      pk[c >> 1] = pack_half2(p0, p1);
      pk[(c >> 1) + 1] = pack_half2(p2, p3);
    }
    tmem_st_x16(t_s + q * (kChunkCols / 2), pk);
    tmem_wait_st();
    tc_fence_before_sync();
    __syncwarp();
    if (lane == 0) mbar_arrive(p_bar + q);
  };

  uint32_t sb2[64];
  load_half(sb2, 1);  // second half again; it sits at columns [64,128), clear of the P chunks below
  if (my_turn != nullptr) FRAY_CRIT_WAIT(my_turn, turn_parity, abort_flag, 0xA01, kv0);
  exp_half(sa);
  store_publish(sa, 0, 0);
  store_publish(sa, 32, 1);
  tmem_wait_ld();
  if (need_mask) mask_half(sb2, 1);
  exp_half(sb2);
  if (other_turn != nullptr) {
    // all exponentials of this tile have been issued: the other group may start its own
    __syncwarp();
    if (lane == 0) mbar_arrive(other_turn);
  }
  store_publish(sb2, 0, 2);
  store_publish(sb2, 32, 3);
  l_run += (rs0 + rs1) + (rs2 + rs3);
}


// The same step with TWO threads per query row (threads of two warpgroups that share the row's 32
// tensor-memory lanes).  This thread owns keys [KEY0, KEY0 + NKEYS) of the tile; the first part
// (KEY0 == 0) takes its exponentials from the special-function unit, the second part may take them
// from the polynomial (USE_POLY).  The unit delivers 16 exponentials per clock and SM, which for a
// 128 x 128 tile is exactly the time the tensor pipe needs for the tile's two products, so a softmax
// that uses nothing else can never hide behind the tensor work.  A warp that mixes both kinds of
// exponential stalls on the unit's queue with its polynomial work still unissued behind it; giving
// the two kinds to two warps of the same scheduler lets them overlap: one warp is bound by the
// unit, the other by instruction issue.
//
// The two threads of a row must agree on the exponent offset, so each publishes the max of its
// part in shared memory (xchg_mine / xchg_other, double-buffered by the caller over the step
// parity) and both meet on the named barrier pair_barrier (256 threads: the two warpgroups of the
// tile).  That barrier also orders the P stores of the second part (which land in columns below
// 64) behind the first part's loads of the scores that sit there.  Both threads keep the same
// m_ref; each keeps the partial row sum of its own keys (the caller adds the two at the end).
// on_alpha(alpha) is called on every step but a row's first with the factor by which the running
// state shrinks (1 when the offset stays): the caller publishes it or applies it to O.
//
// P is handed over in pieces of 32 keys (16 where a part begins or ends on an odd multiple of 16);
// piece n of this part arrives on p_bar[CHUNK0 + n].
template <int BN, int KEY0, int NKEYS, bool USE_POLY, int CHUNK0, class AlphaFn>
__device__ __forceinline__ void softmax_part_tile(uint32_t t_s, uint64_t* p_bar, AlphaFn&& on_alpha, float* xchg_mine,
                                                  const float* xchg_other, int pair_barrier, bool first_tile,
                                                  bool need_mask, int kv0, int row, int seq_len, int causal,
                                                  float scale_log2, int lane, float& m_ref, float& l_run,
                                                  unsigned int* tr = nullptr) {
  static_assert(BN == 128, "written for 128-key tiles");
  static_assert(KEY0 % 16 == 0 && NKEYS % 16 == 0 && NKEYS >= 32 && KEY0 + NKEYS <= BN, "parts are multiples of 16 keys");
  uint32_t sc[NKEYS];
  {
    constexpr int kFull = NKEYS / 32 * 32;
#pragma unroll
    for (int c = 0; c < kFull; c += 32) tmem_ld_x32(t_s + KEY0 + c, reinterpret_cast<uint32_t(&)[32]>(sc[c]));
    if constexpr (NKEYS % 32 == 16) tmem_ld_x16(t_s + KEY0 + kFull, reinterpret_cast<uint32_t(&)[16]>(sc[kFull]));
  }
  tmem_wait_ld();
  FRAY_SM_TRACE(tr, 1);
  if (need_mask) {
#pragma unroll
    for (int c = 0; c < NKEYS; ++c) {
      const int kv = kv0 + KEY0 + c;
      if (kv >= seq_len || (causal && kv > row)) sc[c] = __float_as_uint(-INFINITY);
    }
  }
  float mx[8];
#pragma unroll
  for (int q = 0; q < 8; ++q) mx[q] = __uint_as_float(sc[q]);
#pragma unroll
  for (int c = 8; c < NKEYS; c += 8) {
#pragma unroll
    for (int q = 0; q < 8; ++q) mx[q] = fmaxf(mx[q], __uint_as_float(sc[c + q]));
  }
  const float m_part =
      fmaxf(fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3])), fmaxf(fmaxf(mx[4], mx[5]), fmaxf(mx[6], mx[7])));
  *xchg_mine = m_part;
  FRAY_SM_TRACE(tr, 3);
  named_barrier_sync(pair_barrier, 256);
  FRAY_SM_TRACE(tr, 2);
  const float m_new = fmaxf(fmaxf(m_part, *xchg_other), m_ref);
  if (first_tile) {
    m_ref = m_new;
  } else {
    float alpha = 1.f;
    if ((m_new - m_ref) * scale_log2 > kRescaleThreshold) {
      alpha = ex2_approx((m_ref - m_new) * scale_log2);
      l_run *= alpha;
      m_ref = m_new;
    }
    on_alpha(alpha);
  }
  const float neg_m = (m_ref == -INFINITY) ? 0.f : -m_ref * scale_log2;

  float rs0 = 0.f, rs1 = 0.f, rs2 = 0.f, rs3 = 0.f;
  // One piece of KEYS keys starting at offset OFF of this part: exponentials, row sum, fp16
  // packing, store to the P columns, hand-over.
  auto piece = [&](auto off_tag, auto keys_tag, int n) {
    constexpr int OFF = decltype(off_tag)::value;
    constexpr int KEYS = decltype(keys_tag)::value;
    uint32_t pk[KEYS / 2];
#pragma unroll
    for (int c = 0; c < KEYS; c += 4) {
      const int e = OFF + c;
      const float x0 = fmaf(__uint_as_float(sc[e]), scale_log2, neg_m);
      const float x1 = fmaf(__uint_as_float(sc[e + 1]), scale_log2, neg_m);
      const float x2 = fmaf(__uint_as_float(sc[e + 2]), scale_log2, neg_m);
      const float x3 = fmaf(__uint_as_float(sc[e + 3]), scale_log2, neg_m);
      float p0, p1, p2, p3;
      if constexpr (USE_POLY) {
        p0 = ex2_poly(x0);
        p1 = ex2_poly(x1);
        p2 = ex2_poly(x2);
        p3 = ex2_poly(x3);
      } else {
        p0 = ex2_approx(x0);
        p1 = ex2_approx(x1);
        p2 = ex2_approx(x2);
        p3 = ex2_approx(x3);
      }
      rs0 += p0;
      rs1 += p1;
      rs2 += p2;
      rs3 += p3;
      pk[c >> 1] = pack_half2(p0, p1);
      pk[(c >> 1) + 1] = pack_half2(p2, p3);
    }
    if constexpr (KEYS == 32) {
      tmem_st_x16(t_s + (KEY0 + OFF) / 2, pk);
    } else {
      tmem_st_x8(t_s + (KEY0 + OFF) / 2, pk);
    }
    tmem_wait_st();
    tc_fence_before_sync();
    __syncwarp();
    if (lane == 0) mbar_arrive(p_bar + CHUNK0 + n);
    if (n == 0) FRAY_SM_TRACE(tr, 9);
  };
  using I0 = SmInt<0>;
  using I16 = SmInt<16>;
  using I32 = SmInt<32>;
  if constexpr (KEY0 % 32 == 16) {
    // 16-key piece first, then 32-key pieces
    piece(I0{}, I16{}, 0);
    if constexpr (NKEYS >= 48) piece(I16{}, I32{}, 1);
    if constexpr (NKEYS >= 80) piece(SmInt<48>{}, I32{}, 2);
    if constexpr (NKEYS >= 112) piece(SmInt<80>{}, I32{}, 3);
  } else {
    piece(I0{}, I32{}, 0);
    if constexpr (NKEYS >= 64) piece(I32{}, I32{}, 1);
    if constexpr (NKEYS >= 96) piece(SmInt<64>{}, I32{}, 2);
    if constexpr (NKEYS == 128) piece(SmInt<96>{}, I32{}, 3);
    if constexpr (NKEYS % 32 == 16) piece(SmInt<NKEYS - 16>{}, I16{}, NKEYS / 32);
  }
  l_run += (rs0 + rs1) + (rs2 + rs3);
}


// One softmax step over a 64-key score tile (one thread per row), for the kernel that pipelines
// half tiles: the scores sit in 64 tensor-memory columns starting at t_s, P (fp16) overwrites the
// first 32 of them and is handed over in one piece (p_bar, one arrival per warp): the P.V product of
// a step is not what the group waits for next, so an early first chunk buys nothing and a second
// hand-over costs the group and the MMA warp a barrier round trip each.  Same arithmetic as softmax_tile: base-2 exponentials, lazy offset, row sum from the
// unrounded values.  alpha is published on every step but a row's first.
//
// my_turn / other_turn (both or neither null): the two softmax groups of a CTA take turns on the
// exponentials.  Their warps share the schedulers, and a step is two kinds of work: loads, row max
// and hand-over, which leave the special-function unit idle, and the exponentials, which saturate
// it.  Two groups that run their steps in phase compete for the unit and then leave it idle
// together; kept in anti-phase, one group's exponentials cover the other's remaining work.  The
// group waits on my_turn (phase parity turn_parity) before its first exponential and arrives on
// other_turn (count 4, one arrival per warp) after its last.
__device__ __forceinline__ void softmax_half_step(uint32_t t_s, uint64_t* p_bar, uint64_t* corr_bar, float* alpha_slot,
                                                  bool first_tile, bool need_mask, int kv0, int row, int seq_len,
                                                  int causal, float scale_log2, int lane, float& m_ref, float& l_run,
                                                  uint64_t* my_turn, uint64_t* other_turn, uint32_t turn_parity,
                                                  volatile uint32_t* abort_flag, unsigned int* tr = nullptr) {
  uint32_t sc[64];
  tmem_ld_x32(t_s, reinterpret_cast<uint32_t(&)[32]>(sc[0]));
  tmem_ld_x32(t_s + 32, reinterpret_cast<uint32_t(&)[32]>(sc[32]));
  tmem_wait_ld();
  FRAY_SM_TRACE(tr, 1);
  if (need_mask) {
#pragma unroll
    for (int c = 0; c < 64; ++c) {
      const int kv = kv0 + c;
      if (kv >= seq_len || (causal && kv > row)) sc[c] = __float_as_uint(-INFINITY);
    }
  }
  float mx[8];
#pragma unroll
  for (int q = 0; q < 8; ++q) mx[q] = __uint_as_float(sc[q]);
#pragma unroll
  for (int c = 8; c < 64; c += 8) {
#pragma unroll
    for (int q = 0; q < 8; ++q) mx[q] = fmaxf(mx[q], __uint_as_float(sc[c + q]));
  }
  const float m_new = fmaxf(
      fmaxf(fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3])), fmaxf(fmaxf(mx[4], mx[5]), fmaxf(mx[6], mx[7]))), m_ref);
  if (first_tile) {
    m_ref = m_new;
  } else {
    float alpha = 1.f;
    if ((m_new - m_ref) * scale_log2 > kRescaleThreshold) {
      alpha = ex2_approx((m_ref - m_new) * scale_log2);
      l_run *= alpha;
      m_ref = m_new;
    }
    *alpha_slot = alpha;
    __syncwarp();
    if (lane == 0) mbar_arrive(corr_bar);
  }
  FRAY_SM_TRACE(tr, 2);
  const float neg_m = (m_ref == -INFINITY) ? 0.f : -m_ref * scale_log2;
  float rs0 = 0.f, rs1 = 0.f, rs2 = 0.f, rs3 = 0.f;
  uint32_t pk[32];
  if (my_turn != nullptr) mbar_wait(my_turn, turn_parity, abort_flag, 0xA01, kv0);
#pragma unroll
  for (int c = 0; c < 64; c += 4) {
    const float p0 = ex2_approx(fmaf(__uint_as_float(sc[c]), scale_log2, neg_m));
    const float p1 = ex2_approx(fmaf(__uint_as_float(sc[c + 1]), scale_log2, neg_m));
    const float p2 = ex2_approx(fmaf(__uint_as_float(sc[c + 2]), scale_log2, neg_m));
    const float p3 = ex2_approx(fmaf(__uint_as_float(sc[c + 3]), scale_log2, neg_m));
    rs0 += p0;
    rs1 += p1;
    rs2 += p2;
    rs3 += p3;
    pk[c >> 1] = pack_half2(p0, p1);
    pk[(c >> 1) + 1] = pack_half2(p2, p3);
  }
  if (other_turn != nullptr) {
    __syncwarp();
    if (lane == 0) mbar_arrive(other_turn);
  }
  tmem_st_x32(t_s, pk);
  tmem_wait_st();
  tc_fence_before_sync();
  __syncwarp();
  if (lane == 0) mbar_arrive(p_bar);
  FRAY_SM_TRACE(tr, 9);
  l_run += (rs0 + rs1) + (rs2 + rs3);
}

}  // namespace sm100
}  // namespace fray
