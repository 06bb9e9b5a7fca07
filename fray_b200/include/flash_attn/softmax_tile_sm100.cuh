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

// Lazy-rescale threshold in the scaled base-2 domain: offsets move only when the max grew by > 2^8.
static constexpr float kRescaleThreshold = 8.0f;
// P is handed to the MMA warp in this many column chunks (one mbarrier each, one arrival per warp).
static constexpr int kSoftmaxPChunks = 4;

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
// POLY       of every 4 element pairs, how many take the polynomial exp2 instead of MUFU
template <int BN, int POLY>
__device__ __forceinline__ void softmax_tile(uint32_t t_s, uint64_t* p_bar, uint64_t* corr_bar, float* alpha_slot,
                                             bool first_tile, bool need_mask, int kv0, int row, int seq_len, int causal,
                                             float scale_log2, int lane, float& m_ref, float& l_run,
                                             uint64_t* my_turn, uint64_t* other_turn, uint32_t turn_parity,
                                             volatile uint32_t* abort_flag) {
  static_assert(BN == 128, "written for 128-key tiles");
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

}  // namespace sm100
}  // namespace fray
