#pragma once
// Warp-specialised attention forward for sm_100a with THREE score buffers per query tile, for one
// CTA or a pair of CTAs (tcgen05 cta_group::2).
//
// A CTA owns ONE 128-row query tile of one (batch, head) slice; with CTAS == 2 a cluster of two CTAs
// owns 256 consecutive rows and every product is one M = 256 instruction issued by the pair's
// leader: each CTA holds its own rows of Q, P, S and O and only HALF of every K and V tile (K: 64 of
// the 128 keys, V: 64 of the 128 head dims), fetched by its own plain TMA copies, so the K/V
// traffic per query row is that of a 256-row tile while each CTA's tensor memory holds 128 rows.
//
//   warps 0-3   softmax group 0: KV steps 0, 2, 4, ... of the tile (thread r owns row r)
//   warps 4-7   softmax group 1: KV steps 1, 3, 5, ... of the same rows
//   warps 8-11  correction group: rescales O when the exponent offset moved; epilogue
//   warp 12     issues S(j) = Q.K_j^T          (leader CTA only when paired)
//   warp 13     TMA producer for Q and the K ring
//   warp 14     issues O += P(j).V_j           (leader CTA only when paired)
//   warp 15     TMA producer for the V ring
//
// Tensor memory (512 columns): S buffers at [0,128) [128,256) [256,384), O at [384, 384 + D).  Step j
// uses buffer j % 3; P(j) (16 bit) overwrites the first 64 columns of its buffer and is the A operand of
// O += P(j).V(j).  Why three: with two tiles and two buffers (fwd_ws_sm100.cuh) the chain
// softmax(j) -> P.V(j) -> S(j+1) -> softmax(j+1) of one tile bounds the step, because S(j+1) can only
// follow P.V(j) into the buffer P(j) occupies.  Here S(j+2) goes into the third buffer while the two
// groups work on S(j) and S(j+1), so a group finds its next scores waiting and runs its steps back
// to back; the two groups stay half a step apart and share the special-function unit evenly.
//
// The two products are issued by two warps with a ring of K tiles and a ring of V tiles of their
// own.  An issuing thread is held while the tensor pipe's short queue is full and spends a few hundred
// cycles per step on its barriers; with one issuing warp the pipe ran dry during those (measured: 2070
// cycles per step for 1024 cycles of tensor work), with two one of them always has work queued.
// S(j+3) reuses the buffer of P(j): its warp waits for P.V(j) to complete (s_free).
//
// The two groups share the row state through shared memory: the group of step j reads the offset
// m(j-1) the other group published, decides m(j) (lazily: it moves only when the row max grew by
// more than 2^8 in the scaled domain), publishes it together with the factor for O, and keeps the
// partial row sum of its own steps (rescaled when the offset moved since its last step).  The
// correction group adds the two partial sums at the end.
//
// Every barrier wait is bounded (sm100_ptx.cuh).

#include "fwd_ws_sm100.cuh"
#include "host_sm100.cuh"
#include "sm100_ptx.cuh"
#include "softmax_tile_sm100.cuh"

namespace fray {
namespace sm100 {

template <int D, int STAGES, int CTAS>
struct Ws3Cfg {
  static_assert(D == 64 || D == 128, "head dim must be 64 or 128");
  static_assert(CTAS == 1 || CTAS == 2, "one CTA or a pair");
  static_assert(CTAS == 1 || D == 128, "the paired kernel splits V into two 64-dim halves");
  static_assert(STAGES >= 4 && STAGES <= 12, "4..12 K/V buffers in total");
  static constexpr int kKStages = (STAGES + 1) / 2;        // K tiles in flight (S runs two steps ahead of P.V)
  static constexpr int kVStages = STAGES / 2;
  static constexpr int BM = 128, BN = 128;
  static constexpr int kThreads = 512;
  static constexpr int kPanels = D / 64;                   // 64-element (128-byte) column panels of Q, K, O
  static constexpr int kQPanelBytes = BM * 128;
  static constexpr int kQTileBytes = kPanels * kQPanelBytes;
  static constexpr int kKRows = BN / CTAS;                 // keys of a K tile this CTA holds
  static constexpr int kKPanelBytes = kKRows * 128;
  static constexpr int kVPanels = kPanels / CTAS;          // 64-dim panels of a V tile this CTA holds
  static constexpr int kVPanelBytes = BN * 128;
  static constexpr int kSlotBytes = kPanels * kKPanelBytes;
  static_assert(kSlotBytes == kVPanels * kVPanelBytes, "K and V halves share the ring slots");
  static constexpr int kOffQ = 0;
  static constexpr int kOffKV = kQTileBytes;
  static constexpr int kOffBars = kOffKV + STAGES * kSlotBytes;
  static constexpr int kNumBars = 1 + 2 * STAGES + 3 + 3 + 12 + 2 + 4 + 4 + 8 + 1;
  static constexpr int kOffStats = ((kOffBars + kNumBars * 8 + 16 + 127) / 128) * 128;
  static constexpr int kStatsBytes = (4 + 2 + 2 + 2) * 128 * 4;  // alpha[4], m_hand[2], l_fin[2], m_fin[2] x 128 rows
#ifdef FRAY_ATTN_TRACE
  static constexpr int kOffTrace = kOffStats + kStatsBytes;
  static constexpr int kSmemBytes = kOffTrace + 4 * 800 + 1024;
#else
  static constexpr int kSmemBytes = kOffStats + kStatsBytes + 1024;  // + alignment slack
#endif
  static_assert(kSmemBytes <= 232448, "exceeds the 227 KB shared memory of one CTA");
  static constexpr int kTmemCols = 512;
  static constexpr uint32_t kColO = 384;
  static constexpr int kRegsSoftmax = 184, kRegsCorrection = 80, kRegsOther = 64;
};

// One softmax step of one thread (= one query row) over the 128 scores at t_s.
//   p_bar       address of the first of the buffer's four "P chunk stored" barriers (cluster-wide address of the
//               leader's barriers when paired)
//   corr_bar / alpha_slot   where the factor for O of this step is published (not on a row's first step)
//   m_pub / m_other         this group's and the other group's published offsets of the row
//   hand_mine / hand_other  barriers (one arrival per warp) behind those two slots
template <int CTAS>
__device__ __forceinline__ void softmax_step3(uint32_t t_s, uint32_t p_bar, uint64_t* corr_bar, float* alpha_slot,
                                              float* m_pub, const float* m_other, uint64_t* hand_mine,
                                              uint64_t* hand_other, uint32_t hand_parity, bool first_step,
                                              bool need_mask, int kv0, int row, int seq_k, int causal,
                                              float scale_log2, int lane, float& m_mine, float& l_run,
                                              volatile uint32_t* abort_flag, int step, unsigned int* tr = nullptr) {
  auto load_half = [&](uint32_t (&h)[64], int half) {
    tmem_ld_x32(t_s + half * 64, reinterpret_cast<uint32_t(&)[32]>(h[0]));
    tmem_ld_x32(t_s + half * 64 + 32, reinterpret_cast<uint32_t(&)[32]>(h[32]));
  };
  auto mask_half = [&](uint32_t (&h)[64], int half) {
#pragma unroll
    for (int c = 0; c < 64; ++c) {
      const int kv = kv0 + half * 64 + c;
      if (kv >= seq_k || (causal && kv > row)) h[c] = __float_as_uint(-INFINITY);
    }
  };

  // The row is handled as two 64-key halves: both are loaded for the row max, the first stays in
  // registers for its exponentials and the second is fetched again afterwards.
  uint32_t sa[64];
  float mx0 = -INFINITY, mx1 = -INFINITY, mx2 = -INFINITY, mx3 = -INFINITY;
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
    for (int c = 0; c < 64; c += 4) {
      mx0 = max3(mx0, __uint_as_float(sa[c + 0]), __uint_as_float(sb[c + 0]));
      mx1 = max3(mx1, __uint_as_float(sa[c + 1]), __uint_as_float(sb[c + 1]));
      mx2 = max3(mx2, __uint_as_float(sa[c + 2]), __uint_as_float(sb[c + 2]));
      mx3 = max3(mx3, __uint_as_float(sa[c + 3]), __uint_as_float(sb[c + 3]));
    }
  }
  const float mx = fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3));
  FRAY_SM_TRACE(tr, 1);
  float m_j;
  if (first_step) {
    m_j = mx;
    *m_pub = m_j;
    __syncwarp();
    if (lane == 0) mbar_arrive(hand_mine);
  } else {
    mbar_wait(hand_other, hand_parity, abort_flag, 0x601, step);
    const float m_prev = *m_other;
    const float m_new = fmaxf(mx, m_prev);
    float alpha = 1.f;
    m_j = m_prev;
    if ((m_new - m_prev) * scale_log2 > kRescaleThreshold) {
      alpha = ex2_approx((m_prev - m_new) * scale_log2);
      m_j = m_new;
    }
    *m_pub = m_j;
    *alpha_slot = alpha;
    __syncwarp();
    if (lane == 0) {
      mbar_arrive(hand_mine);
      mbar_arrive(corr_bar);
    }
  }
  if (m_j != m_mine) {
    // the offset moved since this group's last step: bring its partial row sum along
    if (m_mine != -INFINITY) l_run *= ex2_approx((m_mine - m_j) * scale_log2);
    m_mine = m_j;
  }
  const float neg_m = (m_j == -INFINITY) ? 0.f : -m_j * scale_log2;
  FRAY_SM_TRACE(tr, 3);

  float rs0 = 0.f, rs1 = 0.f, rs2 = 0.f, rs3 = 0.f;
  auto exp_half = [&](uint32_t (&h)[64]) {
#pragma unroll
    for (int c = 0; c < 64; ++c) h[c] = __float_as_uint(ex2_approx(fmaf(__uint_as_float(h[c]), scale_log2, neg_m)));
  };
  // Round 32 keys to 16 bit, add them to the row sum, store them as chunk q of P and hand the chunk
  // to the MMA warp once the store has landed.
  auto store_publish = [&](const uint32_t (&h)[64], int off, int q) {
    uint32_t pk[16];
#pragma unroll
    for (int c = 0; c < 32; c += 4) {
      const float p0 = __uint_as_float(h[off + c]), p1 = __uint_as_float(h[off + c + 1]);
      const float p2 = __uint_as_float(h[off + c + 2]), p3 = __uint_as_float(h[off + c + 3]);
      rs0 += p0;
      rs1 += p1;
      rs2 += p2;
      rs3 += p3;
      pk[c >> 1] = pack_half2(p0, p1);
      pk[(c >> 1) + 1] = pack_half2(p2, p3);
    }
    tmem_st_x16(t_s + q * 16, pk);
    tmem_wait_st();
    tc_fence_before_sync();
    __syncwarp();
    if (lane == 0) {
      if constexpr (CTAS == 1) {
        asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(p_bar + q * 8) : "memory");
      } else {
        mbar_arrive_cluster(p_bar + q * 8);
      }
    }
  };

  uint32_t sb2[64];
  load_half(sb2, 1);  // second half again; it sits at columns [64,128), clear of the P chunks below
  exp_half(sa);
  store_publish(sa, 0, 0);
  FRAY_SM_TRACE(tr, 9);
  store_publish(sa, 32, 1);
  tmem_wait_ld();
  if (need_mask) mask_half(sb2, 1);
  exp_half(sb2);
  store_publish(sb2, 0, 2);
  store_publish(sb2, 32, 3);
  l_run += (rs0 + rs1) + (rs2 + rs3);
}

template <int D, int STAGES, int CTAS>
__global__ void __launch_bounds__(512, 1)
attn_fwd_ws3_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                    const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_o, int num_heads,
                    int seq_len, int causal, float scale_log2, int kv_group, float* lse, int seq_k) {
  using Cfg = Ws3Cfg<D, STAGES, CTAS>;
  constexpr int BN = Cfg::BN;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  uint8_t* smem = smem_raw + (((raw_addr + 1023u) & ~1023u) - raw_addr);
  uint8_t* q_smem = smem + Cfg::kOffQ;    // reused for the O tile at the end
  uint8_t* k_smem = smem + Cfg::kOffKV;                    // K ring slot s at k_smem + s * kSlotBytes
  uint8_t* v_smem = k_smem + Cfg::kKStages * Cfg::kSlotBytes;  // V ring behind it
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Cfg::kOffBars);
  uint64_t* q_full = bars;                    // [1]         producer(s) -> QK warp
  uint64_t* k_full = q_full + 1;              // [kKStages]  K producer(s) -> QK warp
  uint64_t* k_empty = k_full + Cfg::kKStages; // [kKStages]  QK warp -> K producer
  uint64_t* v_full = k_empty + Cfg::kKStages; // [kVStages]  V producer(s) -> PV warp
  uint64_t* v_empty = v_full + Cfg::kVStages; // [kVStages]  PV warp -> V producer
  uint64_t* s_full = v_empty + Cfg::kVStages; // [3]       QK warp -> softmax   (S(j) complete in buffer j % 3)
  uint64_t* s_free = s_full + 3;              // [3]       PV warp -> QK warp   (P.V(j) complete: buffer j % 3 may be overwritten)
  uint64_t* p_full = s_free + 3;              // [3][4]    softmax -> PV warp   (chunk c of P(j) stored)
  uint64_t* o_full = p_full + 12;             // [2]       PV warp -> correction (PV(j) complete, barrier j & 1)
  uint64_t* corr_ready = o_full + 2;          // [4]       softmax -> correction (factor of step j >= 1 in slot (j - 1) & 3)
  uint64_t* o_rescaled = corr_ready + 4;      // [4]       correction -> PV warp (O ready for PV(j), slot (j - 1) & 3)
  uint64_t* hand = o_rescaled + 4;            // [2][4]    softmax group g, warp w -> same warp of the other group
  uint64_t* fin = hand + 8;                   // [1]       softmax -> correction (partial row sums published)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + Cfg::kNumBars);
  volatile uint32_t* abort_flag = reinterpret_cast<volatile uint32_t*>(tmem_slot + 1);
  float* alpha_buf = reinterpret_cast<float*>(smem + Cfg::kOffStats);  // [4][128]
  float* m_hand = alpha_buf + 4 * 128;                                 // [2][128]
  float* l_fin = m_hand + 2 * 128;                                     // [2][128]
  float* m_fin = l_fin + 2 * 128;                                      // [2][128]
#ifdef FRAY_ATTN_TRACE
  unsigned int* trace_sm = reinterpret_cast<unsigned int*>(smem + Cfg::kOffTrace);
  const bool trace_on = blockIdx.x == 0 && blockIdx.y == 0;
#endif

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;
  const uint32_t rank = CTAS == 2 ? cluster_ctarank() : 0u;
  const int n_units = gridDim.x / CTAS;
  const int unit_x = blockIdx.x / CTAS;
  const int unit = causal ? (n_units - 1 - unit_x) : unit_x;  // heaviest causal tiles first
  const int m_unit0 = unit * (CTAS * Cfg::BM);
  const int m0 = m_unit0 + static_cast<int>(rank) * Cfg::BM;
  const int bh = blockIdx.y;
  const int b = bh / num_heads;
  const int h = bh - b * num_heads;
  const int h_kv = h / kv_group;

  // KV steps of this CTA (of the pair: both CTAs run the same number; the first tile of a causal pair
  // then sees one fully masked step at the end).
  int n = (seq_k + BN - 1) / BN;
  if (causal) {
    const int lim = (m_unit0 + CTAS * Cfg::BM + BN - 1) / BN;
    n = lim < n ? lim : n;
  }

  if (tid == 0) {
    FRAY_TRACE(6, 0, 0);
    *abort_flag = (*reinterpret_cast<volatile int*>(&fray_attn_status[0]) != 0) ? 2u : 0u;
    mbar_init(q_full, 1);
    for (int s = 0; s < 2 * STAGES; ++s) mbar_init(k_full + s, 1);  // k_full, k_empty, v_full, v_empty
    for (int i = 0; i < 6; ++i) mbar_init(s_full + i, 1);           // s_full, s_free
    for (int i = 0; i < 12; ++i) mbar_init(p_full + i, 4 * CTAS);  // one arrival per softmax warp of every CTA
    mbar_init(o_full, 1);
    mbar_init(o_full + 1, 1);
    for (int i = 0; i < 4; ++i) {
      mbar_init(corr_ready + i, 4);
      mbar_init(o_rescaled + i, 4 * CTAS);
    }
    for (int i = 0; i < 8; ++i) mbar_init(hand + i, 1);
    mbar_init(fin, 8);
    fence_barrier_init();
    prefetch_tensormap(&tm_q);
    prefetch_tensormap(&tm_k);
    prefetch_tensormap(&tm_v);
    prefetch_tensormap(&tm_o);
  }
  __syncthreads();
  uint32_t stop = *abort_flag;
  if constexpr (CTAS == 2) {
    // barriers of both CTAs exist before anything arrives on them; both CTAs agree on whether to run
    cluster_sync_all();
    stop |= ld_shared_cluster_u32(mapa_shared(smem_u32(const_cast<uint32_t*>(abort_flag)), rank ^ 1u));
    cluster_sync_all();  // the peer has read this CTA's flag before anything may raise it
  }
  if (stop != 0) return;  // an earlier launch left the device status raised

  if (warp == 0) {
    tmem_alloc(tmem_slot, Cfg::kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  if (tid == 0) FRAY_TRACE(6, 0, 1);

  // Barriers that softmax / correction threads of both CTAs arrive on live in the leader.
  const uint32_t p_full_addr = CTAS == 2 ? mapa_shared(smem_u32(p_full), 0) : smem_u32(p_full);
  const uint32_t o_rescaled_addr = CTAS == 2 ? mapa_shared(smem_u32(o_rescaled), 0) : smem_u32(o_rescaled);

  if (warp < 8) {
    // =============================================================== softmax groups
    set_max_regs_inc<Cfg::kRegsSoftmax>();
    const int g = warp >> 2;
    const int w = warp & 3;
    const int r = tid & 127;
    const int row = m0 + r;
    const uint32_t lane_base = static_cast<uint32_t>(w * 32) << 16;
    float m_mine = -INFINITY;  // offset this group's partial row sum refers to
    float l_run = 0.f;
    int buf = g;               // j % 3
    uint32_t s_par = 0;        // (j / 3) & 1
    for (int j = g; j < n; j += 2) {
      FRAY_CRIT_WAIT(s_full + buf, s_par, abort_flag, 0x201 + g, j);
      tc_fence_after_sync();
      if (r == FRAY_TRACE_ROW) FRAY_TRACE(0, g, j);
      const int kv0 = j * BN;
      const bool need_mask = (kv0 + BN > seq_k) || (causal && (kv0 + BN - 1 > m0));
      unsigned int* tr = nullptr;
#ifdef FRAY_ATTN_TRACE
      if (trace_on && r == FRAY_TRACE_ROW && j < kTraceIters) tr = trace_sm + g * kTraceIters + j;
#endif
      softmax_step3<CTAS>(tmem_base + buf * 128 + lane_base, p_full_addr + buf * 32, corr_ready + ((j - 1) & 3),
                          alpha_buf + ((j - 1) & 3) * 128 + r, m_hand + g * 128 + r, m_hand + (g ^ 1) * 128 + r,
                          hand + g * 4 + w, hand + (g ^ 1) * 4 + w, ((j - 1) >> 1) & 1, j == 0, need_mask, kv0, row,
                          seq_k, causal, scale_log2, lane, m_mine, l_run, abort_flag, j, tr);
      if (r == FRAY_TRACE_ROW) FRAY_TRACE(4, g, j);
      buf += 2;
      if (buf >= 3) {
        buf -= 3;
        s_par ^= 1u;
      }
    }
    l_fin[g * 128 + r] = l_run;
    m_fin[g * 128 + r] = m_mine;
    __syncwarp();
    if (lane == 0) mbar_arrive(fin);
  } else if (warp < 12) {
    // =============================================================== correction group + epilogue
    set_max_regs_dec<Cfg::kRegsCorrection>();
    const int r = tid & 127;
    const uint32_t lane_base = static_cast<uint32_t>((warp & 3) * 32) << 16;
    const uint32_t t_o = tmem_base + Cfg::kColO + lane_base;
    for (int j = 1; j < n; ++j) {
      const int k = (j - 1) & 3;  // step 0 publishes no factor: step j is the slot's ((j - 1) / 4)-th use
      mbar_wait(corr_ready + k, ((j - 1) >> 2) & 1, abort_flag, 0x301, j);
      const float alpha = alpha_buf[k * 128 + r];
      if (__any_sync(0xffffffffu, alpha != 1.f)) {
        mbar_wait(o_full + ((j - 1) & 1), ((j - 1) >> 1) & 1, abort_flag, 0x311, j);
        tc_fence_after_sync();
#pragma unroll
        for (int c = 0; c < D / 32; ++c) {
          uint32_t orr[32];
          tmem_ld_x32(t_o + c * 32, orr);
          tmem_wait_ld();
#pragma unroll
          for (int x = 0; x < 32; ++x) orr[x] = __float_as_uint(__uint_as_float(orr[x]) * alpha);
          tmem_st_x32(t_o + c * 32, orr);
        }
        tmem_wait_st();
        tc_fence_before_sync();
      }
      __syncwarp();
      if (lane == 0) {
        if constexpr (CTAS == 1) {
          mbar_arrive(o_rescaled + k);
        } else {
          mbar_arrive_cluster(o_rescaled_addr + k * 8);
        }
      }
    }
    // Epilogue: the two groups' partial row sums, each relative to the offset of that group's last
    // step, are brought to the final offset (offsets never decrease) and added.
    mbar_wait(fin, 0, abort_flag, 0x321, n);
    const float m_a = m_fin[r], m_b = m_fin[128 + r];
    const float m_f = fmaxf(m_a, m_b);
    float l = 0.f;
    if (m_a != -INFINITY) l += l_fin[r] * ex2_approx((m_a - m_f) * scale_log2);
    if (m_b != -INFINITY) l += l_fin[128 + r] * ex2_approx((m_b - m_f) * scale_log2);
    mbar_wait(o_full + ((n - 1) & 1), ((n - 1) >> 1) & 1, abort_flag, 0x331, n);
    tc_fence_after_sync();
    if (r == 0) FRAY_TRACE(6, 1, 0);
    if (m0 < seq_len) {  // warp-uniform, CTA-uniform: a pair's second tile may lie past the last query
      epilogue_tile<Cfg, D>(t_o, q_smem, r, l, m_f, &tm_o, m0, h, b, num_heads, seq_len, scale_log2, lse, 1);
      if (r == 0) {
        tma_store_wait_read();
        FRAY_TRACE(6, 1, 2);
      }
    }
  } else {
    set_max_regs_dec<Cfg::kRegsOther>();
    // With a pair, byte counts of both CTAs' copies are collected on the leader's barriers.
    auto leader_addr = [&](uint64_t* bar) { return CTAS == 2 ? mapa_shared(smem_u32(bar), 0) : smem_u32(bar); };
    if (warp == 13 && lane == 0) {
      // ============================================================= TMA producer: Q, then the K ring
      const uint32_t q_full_addr = leader_addr(q_full);
      const uint32_t k_full_addr = leader_addr(k_full);
      if (rank == 0) mbar_expect_tx(q_full, CTAS * Cfg::kQTileBytes);
#pragma unroll
      for (int p = 0; p < Cfg::kPanels; ++p) {
        if constexpr (CTAS == 1) {
          tma_load_4d(q_smem + p * Cfg::kQPanelBytes, &tm_q, q_full, p * 64, m0, h, b);
        } else {
          tma_load_4d_pair(q_smem + p * Cfg::kQPanelBytes, &tm_q, q_full_addr, p * 64, m0, h, b);
        }
      }
      int slot = 0;
      uint32_t par = 0;  // parity of the ring's current round
      for (int jj = 0; jj < n; ++jj) {
        mbar_wait(k_empty + slot, par ^ 1u, abort_flag, 0x401, jj);
        if (*abort_flag != 0) break;
        if (rank == 0) mbar_expect_tx(k_full + slot, CTAS * Cfg::kSlotBytes);
        uint8_t* dst = k_smem + slot * Cfg::kSlotBytes;
#pragma unroll
        for (int p = 0; p < Cfg::kPanels; ++p) {
          if constexpr (CTAS == 1) {
            tma_load_4d(dst + p * Cfg::kKPanelBytes, &tm_k, k_full + slot, p * 64, jj * BN, h_kv, b);
          } else {
            tma_load_4d_pair(dst + p * Cfg::kKPanelBytes, &tm_k, k_full_addr + slot * 8, p * 64,
                             jj * BN + static_cast<int>(rank) * Cfg::kKRows, h_kv, b);
          }
        }
        if (++slot == Cfg::kKStages) {
          slot = 0;
          par ^= 1u;
        }
      }
    } else if (warp == 15 && lane == 0) {
      // ============================================================= TMA producer: the V ring
      const uint32_t v_full_addr = leader_addr(v_full);
      int slot = 0;
      uint32_t par = 0;
      for (int jj = 0; jj < n; ++jj) {
        mbar_wait(v_empty + slot, par ^ 1u, abort_flag, 0x402, jj);
        if (*abort_flag != 0) break;
        if (rank == 0) mbar_expect_tx(v_full + slot, CTAS * Cfg::kSlotBytes);
        uint8_t* dst = v_smem + slot * Cfg::kSlotBytes;
#pragma unroll
        for (int p = 0; p < Cfg::kVPanels; ++p) {
          if constexpr (CTAS == 1) {
            tma_load_4d(dst + p * Cfg::kVPanelBytes, &tm_v, v_full + slot, p * 64, jj * BN, h_kv, b);
          } else {
            tma_load_4d_pair(dst + p * Cfg::kVPanelBytes, &tm_v, v_full_addr + slot * 8,
                             (static_cast<int>(rank) * Cfg::kVPanels + p) * 64, jj * BN, h_kv, b);
          }
        }
        if (++slot == Cfg::kVStages) {
          slot = 0;
          par ^= 1u;
        }
      }
    } else if (warp == 12 && rank == 0) {
      // ============================================================= S(j) = Q . K_j^T (whole warp, one elected lane issues)
      constexpr uint64_t kDescK = smem_desc_sw128(16, 1024);  // K-major operand (Q, K)
      constexpr uint32_t kDescKHi = static_cast<uint32_t>(kDescK >> 32), kDescKLo = static_cast<uint32_t>(kDescK);
      constexpr uint32_t kIdescQK = idesc_f16_f32(CTAS * Cfg::BM, BN, false, false);
      const uint32_t q_lo = kDescKLo | ((smem_u32(q_smem) & 0x3FFFF) >> 4);
      const uint32_t k_addr = smem_u32(k_smem);
      mbar_wait(q_full, 0, abort_flag, 0x511);
      int slot = 0, buf = 0;
      uint32_t par = 0, buf_par = 0;  // parities of the ring's round and of the buffer's use (jj / 3)
      for (int jj = 0; jj < n; ++jj) {
        mbar_wait(k_full + slot, par, abort_flag, 0x501, jj);
        // the buffer's previous tenant P(jj - 3) has been consumed
        if (jj >= 3) mbar_wait(s_free + buf, buf_par ^ 1u, abort_flag, 0x506, jj);
        tc_fence_after_sync();
        FRAY_TRACE(2, jj & 1, jj);
        const uint32_t k_lo = kDescKLo | (((k_addr + slot * Cfg::kSlotBytes) & 0x3FFFF) >> 4);
        const uint32_t t_s = tmem_base + buf * 128;
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint32_t qoff = ((kk >> 2) * Cfg::kQPanelBytes + (kk & 3) * 32) >> 4;
          const uint32_t koff = ((kk >> 2) * Cfg::kKPanelBytes + (kk & 3) * 32) >> 4;
          mma_ss_elect_g<CTAS>(t_s, q_lo + qoff, kDescKHi, k_lo + koff, kDescKHi, kIdescQK, kk > 0);
        }
        mma_commit_elect_g<CTAS>(s_full + buf);
        // the last ring entries are never refilled: no arrival may reach a CTA that has already left
        if (jj + Cfg::kKStages < n) mma_commit_elect_g<CTAS>(k_empty + slot);
        FRAY_TRACE(8, jj & 1, jj);
        if (++slot == Cfg::kKStages) {
          slot = 0;
          par ^= 1u;
        }
        if (++buf == 3) {
          buf = 0;
          buf_par ^= 1u;
        }
      }
    } else if (warp == 14 && rank == 0) {
      // ============================================================= O (+)= P(j) . V_j (whole warp, one elected lane issues)
      constexpr uint64_t kDescV = smem_desc_sw128(Cfg::kVPanelBytes, 1024);  // MN-major operand (V)
      constexpr uint32_t kDescVHi = static_cast<uint32_t>(kDescV >> 32), kDescVLo = static_cast<uint32_t>(kDescV);
      constexpr uint32_t kIdescPV = idesc_f16_f32(CTAS * Cfg::BM, D, false, true);
      const uint32_t v_addr = smem_u32(v_smem);
      const uint32_t t_o = tmem_base + Cfg::kColO;
      int slot = 0, buf = 0;
      uint32_t par = 0, buf_par = 0;
      for (int j = 0; j < n; ++j) {
        mbar_wait(v_full + slot, par, abort_flag, 0x502, j);
        if (j > 0) mbar_wait(o_rescaled + ((j - 1) & 3), ((j - 1) >> 2) & 1, abort_flag, 0x505, j);
        const uint32_t v_lo = kDescVLo | (((v_addr + slot * Cfg::kSlotBytes) & 0x3FFFF) >> 4);
        const uint32_t t_p = tmem_base + buf * 128;
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          FRAY_CRIT_WAIT(p_full + buf * 4 + q, buf_par, abort_flag, 0x503, j);
          tc_fence_after_sync();
          if (q == 0) FRAY_TRACE(5, j & 1, j);
#pragma unroll
          for (int s2 = 0; s2 < 2; ++s2) {
            const int kk = q * 2 + s2;
            mma_ts_elect_g<CTAS>(t_o, t_p + kk * 8, v_lo + ((kk * 2048) >> 4), kDescVHi, kIdescPV, (j > 0 || kk > 0));
          }
        }
        mma_commit_elect_g<CTAS>(o_full + (j & 1));
        if (j + 3 < n) mma_commit_elect_g<CTAS>(s_free + buf);
        if (j + Cfg::kVStages < n) mma_commit_elect_g<CTAS>(v_empty + slot);
        FRAY_TRACE(7, j & 1, j);
        if (++slot == Cfg::kVStages) {
          slot = 0;
          par ^= 1u;
        }
        if (++buf == 3) {
          buf = 0;
          buf_par ^= 1u;
        }
      }
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if constexpr (CTAS == 2) cluster_sync_all();  // neither CTA leaves while the other may still signal it
  if (warp == 0) tmem_dealloc(tmem_base, Cfg::kTmemCols);
#ifdef FRAY_ATTN_TRACE
  if (tid == 0) FRAY_TRACE(6, 0, 2);
  __syncthreads();
  if (trace_on)
    for (int w2 = tid; w2 < kTraceWords; w2 += Cfg::kThreads) fray_attn_trace_buf[w2] = trace_sm[w2];
#endif
}

// Host launcher.  Returns an AttnReturnCode.
template <int D, int STAGES, int CTAS>
inline int launch_attn_fwd_ws3(const operand_t* q, const operand_t* k, const operand_t* v, operand_t* o, const AttnShape& shp,
                               const AttnStrides (&st)[4], const AttnExtras& ex, bool causal, float scale,
                               cudaStream_t stream) {
  using Cfg = Ws3Cfg<D, STAGES, CTAS>;
  const AttnShape shp_kv{shp.B, shp.H / ex.kv_group, ex.seq_k, shp.D};
  CUtensorMap tm_q, tm_k, tm_v, tm_o;
  int rc = cached_attn_tensor_map(&tm_q, q, shp, st[0], Cfg::BM);
  if (rc != kAttnOk) return rc;
  rc = cached_attn_tensor_map(&tm_k, k, shp_kv, st[1], Cfg::kKRows);
  if (rc != kAttnOk) return rc;
  rc = cached_attn_tensor_map(&tm_v, v, shp_kv, st[2], Cfg::BN);
  if (rc != kAttnOk) return rc;
  rc = cached_attn_tensor_map(&tm_o, o, shp, st[3], Cfg::BM);
  if (rc != kAttnOk) return rc;

  auto kernel = attn_fwd_ws3_kernel<D, STAGES, CTAS>;
  rc = ensure_dynamic_smem<Cfg>(kernel, Cfg::kSmemBytes);
  if (rc != kAttnOk) return rc;

  const int tiles = (shp.S + Cfg::BM - 1) / Cfg::BM;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(((tiles + CTAS - 1) / CTAS) * CTAS, shp.B * shp.H);
  cfg.blockDim = dim3(Cfg::kThreads);
  cfg.dynamicSmemBytes = Cfg::kSmemBytes;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = CTAS;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = CTAS == 2 ? 1 : 0;
  const cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, tm_q, tm_k, tm_v, tm_o, shp.H, shp.S, causal ? 1 : 0,
                                           scale * 1.44269504088896340736f, ex.kv_group, ex.lse, ex.seq_k);
  if (e != cudaSuccess) {
    (void)cudaGetLastError();
    return kAttnLaunchFailed;
  }
  return kAttnOk;
}

}  // namespace sm100
}  // namespace fray
