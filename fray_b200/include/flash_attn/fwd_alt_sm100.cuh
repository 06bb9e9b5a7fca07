#pragma once
// Warp-specialised attention forward for sm_100a with the scores and the probabilities of a query
// tile in SEPARATE tensor-memory buffers, for one CTA or a pair of CTAs (tcgen05 cta_group::2).
//
// A CTA owns ONE 128-row query tile of one (batch, head) slice; with CTAS == 2 a cluster of two CTAs
// owns 256 consecutive rows and every product is one M = 256 instruction issued by the pair's
// leader: each CTA holds its own rows of Q, P, S and O and only HALF of every K and V tile (K: 64 of
// the 128 keys, V: 64 of the 128 head dims), fetched by its own plain TMA copies, so the K/V
// traffic per query row is that of a 256-row tile while each CTA's tensor memory holds 128 rows, and
// the operand reads of a product take 96 instead of 128 bytes of shared-memory bandwidth per clock.
//
//   warps 0-3   softmax group 0: KV steps 0, 2, 4, ... of the tile (thread r owns row r)
//   warps 4-7   softmax group 1: KV steps 1, 3, 5, ... of the same rows
//   warps 8-11  statistics group: row max and exponent offset of every step, O rescale when it moved; epilogue
//   warp 12     MMA issue (leader CTA only when paired)
//   warp 13     TMA producer for Q and the K ring (STAGES slots)
//   warp 14     TMA producer for V (three slots)
//   warp 15     idle
//
// Tensor memory (512 columns): S(j) at [0,128) or [128,256) (j & 1), P(j) (16 bit) at [256,320) or
// [320,384), O at [384, 384 + D).  In the two-tile kernel (fwd_ws_sm100.cuh) P overwrites its S, so
// S(j+1) of a tile can only follow P.V(j) and the chain softmax(j) -> P.V(j) -> S(j+1) -> softmax(j+1)
// bounds the step.  Here a softmax thread pulls its whole row of S(j) into registers first and
// releases the score buffer at once, so S(j+2) is computed while the group still works on step j
// and the group finds its next scores waiting: the two groups run their steps back to back, half a
// step apart, and share the special-function unit evenly.  P(j) goes to a buffer of its own, which
// P.V(j-2) left a whole step earlier.
//
// Issue order in the MMA warp:  S(0) S(1) | S(2) PV(0) | S(3) PV(1) | ...  The issuing thread's own time
// is the scarce resource (a satisfied barrier wait costs it ~100 cycles during which the pipe's short
// queue runs dry; two issuing warps, one per product, were measured slower still: the pipe handles
// alternating kinds of product badly), so each product waits on ONE barrier: S(j) on the one that
// collects the bytes of K_j and the arrivals of the softmax warps that released the score buffer;
// P.V(j) on the one that collects the softmax warps that stored P(j), the correction warps that made
// O ready, and the bytes of V_j.
//
// The row statistics are not the softmax groups' job: the statistics group scans S(j) for the row max as
// soon as the scores are complete, decides the step's exponent offset m(j) (lazily: it moves only when
// the row max grew by more than 2^8 in the scaled domain; the sequence lives in that group's registers,
// so nothing is exchanged between the softmax groups), rescales O when the offset moved and publishes
// m(j).  A softmax thread waits for m(j) only (which implies S(j)), pulls its row into registers, and
// spends its step on the exponentials; it keeps the partial row sum of its own steps (rescaled when the
// offset moved since its last step) and the statistics group adds the two partial sums at the end.  The
// max scan and the exponentials of a step thus run in different warps of the same schedulers, which
// gives the in-order issue three streams to interleave instead of two.
//
// Every barrier wait is bounded (sm100_ptx.cuh).

#include "host_sm100.cuh"
#include "sm100_ptx.cuh"
#include "softmax_tile_sm100.cuh"

namespace fray {
namespace sm100 {

template <int D, int STAGES, int CTAS>
struct AltCfg {
  static_assert(D == 64 || D == 128, "head dim must be 64 or 128");
  static_assert(CTAS == 1 || CTAS == 2, "one CTA or a pair");
  static_assert(CTAS == 1 || D == 128, "the paired kernel splits V into two 64-dim halves");
  static_assert(STAGES >= 2 && STAGES <= 8, "2..8 K buffers");
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
  static_assert(kSlotBytes == kVPanels * kVPanelBytes, "K and V halves have the same size");
  static constexpr int kOffQ = 0;
  static constexpr int kOffK = kQTileBytes;
  static constexpr int kOffV = kOffK + STAGES * kSlotBytes;
  static constexpr int kOffBars = kOffV + 3 * kSlotBytes;
  static constexpr int kNumBars = 1 + 2 * STAGES + 2 + 3 + 3 + 2 + 8 + 1;
  static constexpr int kOffStats = ((kOffBars + kNumBars * 8 + 16 + 127) / 128) * 128;
  static constexpr int kStatsBytes = (2 + 2 + 2) * 128 * 4;  // m_slot[2], l_fin[2], m_fin[2] x 128 rows
#ifdef FRAY_ATTN_TRACE
  static constexpr int kOffTrace = kOffStats + kStatsBytes;
  static constexpr int kSmemBytes = kOffTrace + 4 * 960 + 1024;
#else
  static constexpr int kSmemBytes = kOffStats + kStatsBytes + 1024;  // + alignment slack
#endif
  static_assert(kSmemBytes <= 232448, "exceeds the 227 KB shared memory of one CTA");
  static constexpr int kTmemCols = 512;
  static constexpr uint32_t kColP = 256, kColO = 384;
#ifndef FRAY_ALT_REGS_STATS
#define FRAY_ALT_REGS_STATS 112
#endif
  // register budgets after setmaxnreg (softmax, statistics, MMA/producer warps): their sum over the 16
  // warps is the CTA's allocation of 512 x 128 registers
  static constexpr int kRegsSoftmax = 184, kRegsCorrection = FRAY_ALT_REGS_STATS, kRegsOther = 144 - FRAY_ALT_REGS_STATS;
  static_assert(256 * kRegsSoftmax + 128 * kRegsCorrection + 128 * kRegsOther <= 512 * 128, "register budgets exceed the CTA's allocation");
  // arrivals on a "S(j) may start" barrier: the leader's K producer (with the byte count of both CTAs'
  // copies) and the softmax and statistics warps of every CTA that are done with the score buffer (step j - 2)
  static constexpr int kKFullCount = 8 * CTAS + 1;
  // arrivals on a "P.V(j) may start" barrier: softmax and statistics warps of every CTA, and the
  // leader's V producer (with the byte count of both CTAs' copies)
  static constexpr int kPvReadyCount = 8 * CTAS + 1;
};

// Share of the exponentials evaluated by polynomial on the FMA pipe (of every 4 pairs).
#ifndef FRAY_ALT_POLY
#define FRAY_ALT_POLY 1
#endif

// Barriers and slots one softmax step touches (addresses are cluster-wide where the barrier lives in the
// pair's leader).
struct SoftmaxStepIo {
  uint32_t t_s;            // tensor-memory address of this thread's lane at column 0 of S(j)
  uint32_t t_p;            // ... of P(j)
  uint32_t released_bar;   // told that S(j) is in registers (0: nothing waits for the buffer any more)
  uint32_t pv_bar;         // told that P(j) is stored
  uint64_t* p_free_bar;    // P.V(j - 2) complete: its P buffer may be overwritten (null on a group's first step)
  uint32_t p_free_parity;
  uint64_t* m_bar;         // the statistics warp of these rows has published m(j) (which implies S(j) complete)
  uint32_t m_parity;
  const float* m_slot;     // ... here
};

// Masks the scores of keys past the end of the sequence or above the causal diagonal.
template <int N>
__device__ __forceinline__ void mask_scores(uint32_t (&h)[N], int kv_first, int row, int seq_k, int causal) {
#pragma unroll
  for (int c = 0; c < N; ++c) {
    const int kv = kv_first + c;
    if (kv >= seq_k || (causal && kv > row)) h[c] = __float_as_uint(-INFINITY);
  }
}

// One softmax step of one thread (= one query row): exp2(S*c - m(j)*c) for the row's 128 scores, rounded
// to 16 bit into P(j), and the row sum of the unrounded values.  The scores are pulled into registers in
// one go and the score buffer is released right away; the rest works from registers.
// POLY of every 4 pairs of exponentials are evaluated by polynomial on the FMA pipe: a 128 x 128 tile
// needs the special-function unit (16 results per clock and SM) for exactly as long as the tensor
// pipe needs for the tile's two products, so with every exponential on the unit the softmax can
// never hide behind the tensor work.
template <int CTAS, int POLY, bool MASK>
__device__ __forceinline__ void softmax_step_alt(const SoftmaxStepIo& io, int kv0, int row, int seq_k, int causal,
                                                 float scale_log2, int lane, float& m_mine, float& l_run,
                                                 volatile uint32_t* abort_flag, int step, unsigned int* tr = nullptr) {
  static_assert(POLY >= 0 && POLY <= 2, "0, 1 or 2 of every 4 pairs by polynomial");
  FRAY_CRIT_WAIT(io.m_bar, io.m_parity, abort_flag, 0x201, step);
  const float m_j = *io.m_slot;
  tc_fence_after_sync();
  FRAY_SM_TRACE(tr, 0);
  uint32_t sa[64], sb[64];
  tmem_ld_x32(io.t_s, reinterpret_cast<uint32_t(&)[32]>(sa[0]));
  tmem_ld_x32(io.t_s + 32, reinterpret_cast<uint32_t(&)[32]>(sa[32]));
  tmem_ld_x32(io.t_s + 64, reinterpret_cast<uint32_t(&)[32]>(sb[0]));
  tmem_ld_x32(io.t_s + 96, reinterpret_cast<uint32_t(&)[32]>(sb[32]));
  tmem_wait_ld();
  tc_fence_before_sync();
  __syncwarp();
  if (lane == 0 && io.released_bar != 0) {  // this warp's part of "S(j + 2) may overwrite the scores"
    if constexpr (CTAS == 1) {
      asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(io.released_bar) : "memory");
    } else {
      mbar_arrive_cluster(io.released_bar);
    }
  }
  FRAY_SM_TRACE(tr, 1);
  // Barrier tests behind the loads, not beside them: a wait issued while tensor-memory loads are in
  // flight queues behind them (measured ~150 cycles per satisfied wait).
  // P.V(j - 2) was issued a whole step ago; that it has left the P buffer is tested here and only looked
  // at before the first store to the buffer.
  const bool p_free = io.p_free_bar == nullptr || mbar_test_wait(io.p_free_bar, io.p_free_parity);
  if constexpr (MASK) {
    mask_scores(sa, kv0, row, seq_k, causal);
    mask_scores(sb, kv0 + 64, row, seq_k, causal);
  }
  if (m_j != m_mine) {
    // the offset moved since this group's last step: bring its partial row sum along
    if (m_mine != -INFINITY) l_run *= ex2_approx((m_mine - m_j) * scale_log2);
    m_mine = m_j;
  }
  const float neg_m = (m_j == -INFINITY) ? 0.f : -m_j * scale_log2;
  FRAY_SM_TRACE(tr, 3);

  uint64_t rsp0 = 0ull, rsp1 = 0ull;  // packed partial row sums (two lanes each)
  const uint64_t scale2 = pack_f32x2(scale_log2, scale_log2), neg_m2 = pack_f32x2(neg_m, neg_m);
  // exp2(S*c - m*c) of one 64-key half, rounded to 16 bit (the row sum takes the unrounded values).
  // Packed f32x2 arithmetic: one issue slot per pair.
  auto exp_half = [&](uint32_t (&h)[64], uint32_t (&pk)[32]) {
#pragma unroll
    for (int c = 0; c < 64; c += 8) {
      uint64_t p[4];
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const uint64_t x = fma_f32x2(pack_f32x2(__uint_as_float(h[c + 2 * q]), __uint_as_float(h[c + 2 * q + 1])), scale2, neg_m2);
        if (q >= 4 - POLY) {
          p[q] = ex2_poly_f32x2(x);
        } else {
          float x0, x1;
          unpack_f32x2(x, x0, x1);
          p[q] = pack_f32x2(ex2_approx(x0), ex2_approx(x1));
        }
      }
      rsp0 = add_f32x2(rsp0, add_f32x2(p[0], p[2]));
      rsp1 = add_f32x2(rsp1, add_f32x2(p[1], p[3]));
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        float p0, p1;
        unpack_f32x2(p[q], p0, p1);
        pk[(c >> 1) + q] = pack_half2(p0, p1);
      }
    }
  };
  {
    uint32_t pk[32];
    exp_half(sa, pk);
    // first store to the P buffer: P.V(j - 2) must have read it (see above; it has, unless the other CTA
    // of a pair lags by most of a step, and then this CTA has to wait for it anyway)
    if (!p_free) mbar_wait_spin(io.p_free_bar, io.p_free_parity, abort_flag, 0x602, step);
    tmem_st_x32(io.t_p, pk);
  }
  FRAY_SM_TRACE(tr, 9);
  {
    uint32_t pk[32];
    exp_half(sb, pk);
    tmem_st_x32(io.t_p + 32, pk);
  }
  tmem_wait_st();
  tc_fence_before_sync();
  __syncwarp();
  if (lane == 0) {
    if constexpr (CTAS == 1) {
      asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(io.pv_bar) : "memory");
    } else {
      mbar_arrive_cluster(io.pv_bar);
    }
  }
  float r0, r1, r2, r3;
  unpack_f32x2(rsp0, r0, r1);
  unpack_f32x2(rsp1, r2, r3);
  l_run += (r0 + r1) + (r2 + r3);
}

template <int D, int STAGES, int CTAS>
__global__ void __launch_bounds__(512, 1)
attn_fwd_alt_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                    const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_o, int num_heads,
                    int seq_len, int causal, float scale_log2, int kv_group, float* lse, int seq_k) {
  using Cfg = AltCfg<D, STAGES, CTAS>;
  constexpr int BN = Cfg::BN;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  uint8_t* smem = smem_raw + (((raw_addr + 1023u) & ~1023u) - raw_addr);
  uint8_t* q_smem = smem + Cfg::kOffQ;  // reused for the O tile at the end
  uint8_t* k_smem = smem + Cfg::kOffK;  // K ring slot s at k_smem + s * kSlotBytes
  uint8_t* v_smem = smem + Cfg::kOffV;  // V of step j at v_smem + (j % 3) * kSlotBytes
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Cfg::kOffBars);
  uint64_t* q_full = bars;                // [1]       producer(s) -> MMA
  uint64_t* k_full = q_full + 1;          // [STAGES]  K producer(s) + softmax -> MMA: S(j) may start (slot j % STAGES)
  uint64_t* k_empty = k_full + STAGES;    // [STAGES]  MMA -> K producer
  uint64_t* s_full = k_empty + STAGES;    // [2]       MMA -> statistics: S(j) complete in buffer j & 1
  uint64_t* pv_ready = s_full + 2;        // [3]       softmax + statistics + V producer -> MMA: P.V(j) may start (j % 3)
  uint64_t* pv_done = pv_ready + 3;       // [3]       MMA -> statistics, V producer: P.V(j) complete (j % 3)
  uint64_t* p_free = pv_done + 3;         // [2]       MMA -> softmax: P.V(j) complete, its P buffer (j & 1) may be overwritten
  uint64_t* m_ready = p_free + 2;         // [2][4]    statistics warp w -> softmax warp w of group j & 1: m(j) published
  uint64_t* fin = m_ready + 8;            // [1]       softmax -> statistics: partial row sums published
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + Cfg::kNumBars);
  volatile uint32_t* abort_flag = reinterpret_cast<volatile uint32_t*>(tmem_slot + 1);
  float* m_slot = reinterpret_cast<float*>(smem + Cfg::kOffStats);     // [2][128]  m(j) of the row, slot j & 1
  float* l_fin = m_slot + 2 * 128;                                     // [2][128]
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
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(k_full + s, Cfg::kKFullCount);
      mbar_init(k_empty + s, 1);
    }
    for (int i = 0; i < 2; ++i) mbar_init(s_full + i, 1);
    for (int i = 0; i < 3; ++i) {
      mbar_init(pv_ready + i, Cfg::kPvReadyCount);
      mbar_init(pv_done + i, 1);
    }
    for (int i = 0; i < 2; ++i) mbar_init(p_free + i, 1);
    for (int i = 0; i < 8; ++i) mbar_init(m_ready + i, 1);
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

  // Barriers that threads of both CTAs arrive on live in the leader.
  auto leader_addr = [&](uint64_t* bar) { return CTAS == 2 ? mapa_shared(smem_u32(bar), 0) : smem_u32(bar); };
  auto arrive_leader = [&](uint32_t addr) {
    if constexpr (CTAS == 1) {
      asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(addr) : "memory");
    } else {
      mbar_arrive_cluster(addr);
    }
  };

  if (warp < 8) {
    // =============================================================== softmax groups
    set_max_regs_inc<Cfg::kRegsSoftmax>();
    const int g = warp >> 2;
    const int w = warp & 3;
    const int r = tid & 127;
    const int row = m0 + r;
    const uint32_t lane_base = static_cast<uint32_t>(w * 32) << 16;
    const uint32_t k_full_addr = leader_addr(k_full);
    const uint32_t pv_ready_addr = leader_addr(pv_ready);
    // both score buffers start out free: this warp's share of the arrivals S(0) and S(1) wait for
    if (lane == 0 && g < n) arrive_leader(k_full_addr + g * 8);
    SoftmaxStepIo io;
    io.t_s = tmem_base + g * 128 + lane_base;               // group g works on steps j = g (mod 2): buffer j & 1 = g
    io.t_p = tmem_base + Cfg::kColP + g * 64 + lane_base;
    io.m_bar = m_ready + g * 4 + w;
    io.m_slot = m_slot + g * 128 + r;
    float m_mine = -INFINITY;  // offset this group's partial row sum refers to
    float l_run = 0.f;
    int slot2 = (g + 2) % STAGES;  // (j + 2) % STAGES: K ring slot of the step that inherits the score buffer
    int j3 = g;                    // j % 3
    for (int j = g; j < n; j += 2) {
      const int kv0 = j * BN;
      const bool need_mask = (kv0 + BN > seq_k) || (causal && (kv0 + BN - 1 > m0));
      unsigned int* tr = nullptr;
#ifdef FRAY_ATTN_TRACE
      if (trace_on && r == FRAY_TRACE_ROW && j < kTraceIters) tr = trace_sm + g * kTraceIters + j;
#endif
      io.released_bar = (j + 2 < n) ? k_full_addr + slot2 * 8 : 0u;
      io.pv_bar = pv_ready_addr + j3 * 8;
      io.p_free_bar = (j >= 2) ? p_free + g : nullptr;   // P.V(j - 2) is the buffer's ((j - 2) / 2)-th tenant
      io.p_free_parity = ((j - 2) >> 1) & 1;
      io.m_parity = (j >> 1) & 1;
      if (need_mask) {
        softmax_step_alt<CTAS, FRAY_ALT_POLY, true>(io, kv0, row, seq_k, causal, scale_log2, lane, m_mine, l_run, abort_flag, j, tr);
      } else {
        softmax_step_alt<CTAS, FRAY_ALT_POLY, false>(io, kv0, row, seq_k, causal, scale_log2, lane, m_mine, l_run, abort_flag, j, tr);
      }
      if (r == FRAY_TRACE_ROW) FRAY_TRACE(4, g, j);
      slot2 += 2;
      if (slot2 >= STAGES) slot2 -= STAGES;
      j3 += 2;
      if (j3 >= 3) j3 -= 3;
    }
    l_fin[g * 128 + r] = l_run;
    m_fin[g * 128 + r] = m_mine;
    __syncwarp();
    if (lane == 0) mbar_arrive(fin);
  } else if (warp < 12) {
    // =============================================================== statistics group + epilogue
    set_max_regs_dec<Cfg::kRegsCorrection>();
    const int r = tid & 127;
    const int w = warp & 3;
    const int row = m0 + r;
    const uint32_t lane_base = static_cast<uint32_t>(w * 32) << 16;
    const uint32_t t_o = tmem_base + Cfg::kColO + lane_base;
    const uint32_t k_full_addr = leader_addr(k_full);
    const uint32_t pv_ready_addr = leader_addr(pv_ready);
    // both score buffers start out free: this warp's share of the arrivals S(0) and S(1) wait for
    if (lane == 0) {
      arrive_leader(k_full_addr);
      if (n > 1) arrive_leader(k_full_addr + 8);
    }
    float m_run = -INFINITY;     // m(j - 1)
    int buf = 0;                 // j % 3
    int pbuf = 2;                // (j - 1) % 3 and ((j - 1) / 3) & 1 (from j = 1)
    uint32_t ppar = 1;
    int slot2 = 2 % STAGES;      // (j + 2) % STAGES
    for (int j = 0; j < n; ++j) {
      const int g = j & 1;
      mbar_wait(s_full + g, (j >> 1) & 1, abort_flag, 0x301, j);
      tc_fence_after_sync();
      if (r == FRAY_TRACE_ROW) FRAY_TRACE(10, g, j);
      // row max of S(j), 32 columns at a time, the next load under the current chunk's arithmetic
      const int kv0 = j * BN;
      const bool need_mask = (kv0 + BN > seq_k) || (causal && (kv0 + BN - 1 > m0));
      const uint32_t t_s = tmem_base + g * 128 + lane_base;
      float mx0 = -INFINITY, mx1 = -INFINITY, mx2 = -INFINITY, mx3 = -INFINITY;
      auto max_chunk = [&](uint32_t (&h)[32], int c0) {
        if (need_mask) mask_scores(h, kv0 + c0, row, seq_k, causal);
#pragma unroll
        for (int c = 0; c < 32; c += 8) {
          mx0 = max3(mx0, __uint_as_float(h[c + 0]), __uint_as_float(h[c + 4]));
          mx1 = max3(mx1, __uint_as_float(h[c + 1]), __uint_as_float(h[c + 5]));
          mx2 = max3(mx2, __uint_as_float(h[c + 2]), __uint_as_float(h[c + 6]));
          mx3 = max3(mx3, __uint_as_float(h[c + 3]), __uint_as_float(h[c + 7]));
        }
      };
      {
        uint32_t ha[32], hb[32];
        tmem_ld_x32(t_s, ha);
        tmem_wait_ld();
        tmem_ld_x32(t_s + 32, hb);
        max_chunk(ha, 0);
        tmem_wait_ld();
        tmem_ld_x32(t_s + 64, ha);
        max_chunk(hb, 32);
        tmem_wait_ld();
        tmem_ld_x32(t_s + 96, hb);
        max_chunk(ha, 64);
        tmem_wait_ld();
        // this warp's part of "S(j + 2) may overwrite the scores"
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0 && j + 2 < n) arrive_leader(k_full_addr + slot2 * 8);
        max_chunk(hb, 96);
      }
      const float mx = fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3));
      // the step's offset: the row max on a row's first step, afterwards moved only when the max outgrew it
      float alpha = 1.f;
      float m_j = m_run;
      if (j == 0) {
        m_j = mx;
      } else {
        const float m_new = fmaxf(mx, m_run);
        if ((m_new - m_run) * scale_log2 > kRescaleThreshold) {
          alpha = ex2_approx((m_run - m_new) * scale_log2);
          m_j = m_new;
        }
      }
      m_run = m_j;
      m_slot[g * 128 + r] = m_j;
      __syncwarp();
      if (lane == 0) mbar_arrive(m_ready + g * 4 + w);
      if (r == FRAY_TRACE_ROW) FRAY_TRACE(11, g, j);
      if (__any_sync(0xffffffffu, alpha != 1.f)) {
        mbar_wait(pv_done + pbuf, ppar, abort_flag, 0x311, j);  // P.V(j - 1) complete
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
        __syncwarp();
      }
      if (lane == 0) arrive_leader(pv_ready_addr + buf * 8);  // O is ready for P.V(j)
      pbuf = buf;
      if (buf == 0) ppar ^= 1u;  // j just crossed a multiple of 3: so will j - 1 on the next turn
      if (++buf == 3) buf = 0;
      slot2 += 1;
      if (slot2 >= STAGES) slot2 -= STAGES;
    }
    // Epilogue: the two groups' partial row sums, each relative to the offset of that group's last
    // step, are brought to the final offset (offsets never decrease) and added.
    mbar_wait(fin, 0, abort_flag, 0x321, n);
    const float m_a = m_fin[r], m_b = m_fin[128 + r];
    const float m_f = m_run;
    float l = 0.f;
    if (m_a != -INFINITY) l += l_fin[r] * ex2_approx((m_a - m_f) * scale_log2);
    if (m_b != -INFINITY) l += l_fin[128 + r] * ex2_approx((m_b - m_f) * scale_log2);
    mbar_wait(pv_done + (n - 1) % 3, ((n - 1) / 3) & 1, abort_flag, 0x331, n);
    tc_fence_after_sync();
    if (r == 0) FRAY_TRACE(6, 1, 0);
    if (m0 < seq_len) {  // CTA-uniform: a pair's second tile may lie past the last query
      epilogue_tile<Cfg, D>(t_o, q_smem, r, l, m_f, &tm_o, m0, h, b, num_heads, seq_len, scale_log2, lse, 1);
      if (r == 0) {
        tma_store_wait_read();
        FRAY_TRACE(6, 1, 2);
      }
    }
  } else {
    set_max_regs_dec<Cfg::kRegsOther>();
    if (warp == 13 && lane == 0) {
      // ============================================================= TMA producer: Q, then the K ring
      // With a pair, byte counts of both CTAs' copies are collected on the leader's barriers.
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
        if (++slot == STAGES) {
          slot = 0;
          par ^= 1u;
        }
      }
    } else if (warp == 14 && lane == 0) {
      // ============================================================= TMA producer: V_j into slot j % 3
      // Its bytes are counted on the step's "P.V may start" barrier.
      const uint32_t pv_ready_addr = leader_addr(pv_ready);
      int buf = 0;
      uint32_t par = 0;  // (j / 3) & 1
      for (int j = 0; j < n; ++j) {
        if (j >= 3) mbar_wait(pv_done + buf, par ^ 1u, abort_flag, 0x402, j);  // P.V(j - 3) has left the slot
        if (*abort_flag != 0) break;
        if (rank == 0) mbar_expect_tx(pv_ready + buf, CTAS * Cfg::kSlotBytes);
        uint8_t* dst = v_smem + buf * Cfg::kSlotBytes;
#pragma unroll
        for (int p = 0; p < Cfg::kVPanels; ++p) {
          if constexpr (CTAS == 1) {
            tma_load_4d(dst + p * Cfg::kVPanelBytes, &tm_v, pv_ready + buf, p * 64, j * BN, h_kv, b);
          } else {
            tma_load_4d_pair(dst + p * Cfg::kVPanelBytes, &tm_v, pv_ready_addr + buf * 8,
                             (static_cast<int>(rank) * Cfg::kVPanels + p) * 64, j * BN, h_kv, b);
          }
        }
        if (++buf == 3) {
          buf = 0;
          par ^= 1u;
        }
      }
    } else if (warp == 12 && rank == 0) {
      // ============================================================= MMA issue (whole warp, one elected lane issues)
      constexpr uint64_t kDescK = smem_desc_sw128(16, 1024);                 // K-major operand (Q, K)
      constexpr uint64_t kDescV = smem_desc_sw128(Cfg::kVPanelBytes, 1024);  // MN-major operand (V)
      constexpr uint32_t kDescKHi = static_cast<uint32_t>(kDescK >> 32), kDescKLo = static_cast<uint32_t>(kDescK);
      constexpr uint32_t kDescVHi = static_cast<uint32_t>(kDescV >> 32), kDescVLo = static_cast<uint32_t>(kDescV);
      constexpr uint32_t kIdescQK = idesc_f16_f32(CTAS * Cfg::BM, BN, false, false);
      constexpr uint32_t kIdescPV = idesc_f16_f32(CTAS * Cfg::BM, D, false, true);
      const uint32_t q_lo = kDescKLo | ((smem_u32(q_smem) & 0x3FFFF) >> 4);
      const uint32_t k_addr = smem_u32(k_smem);
      const uint32_t v_addr = smem_u32(v_smem);
      const uint32_t t_o = tmem_base + Cfg::kColO;
      auto issue_qk = [&](int jj, int slot) __attribute__((always_inline)) {  // S(jj) = Q . K_jj^T into buffer jj & 1
        tc_fence_after_sync();
        FRAY_TRACE(2, jj & 1, jj);
        const uint32_t k_lo = kDescKLo | (((k_addr + slot * Cfg::kSlotBytes) & 0x3FFFF) >> 4);
        const uint32_t t_s = tmem_base + (jj & 1) * 128;
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint32_t qoff = ((kk >> 2) * Cfg::kQPanelBytes + (kk & 3) * 32) >> 4;
          const uint32_t koff = ((kk >> 2) * Cfg::kKPanelBytes + (kk & 3) * 32) >> 4;
          mma_ss_elect_g<CTAS>(t_s, q_lo + qoff, kDescKHi, k_lo + koff, kDescKHi, kIdescQK, kk > 0);
        }
        mma_commit_elect_g<CTAS>(s_full + (jj & 1));
        // the last ring entries are never refilled: no arrival may reach a CTA that has already left
        if (jj + STAGES < n) mma_commit_elect_g<CTAS>(k_empty + slot);
        FRAY_TRACE(8, jj & 1, jj);
      };
      auto issue_pv = [&](int j, int buf) __attribute__((always_inline)) {  // O (+)= P(j) . V_j
        tc_fence_after_sync();
        FRAY_TRACE(5, j & 1, j);
        const uint32_t v_lo = kDescVLo | (((v_addr + buf * Cfg::kSlotBytes) & 0x3FFFF) >> 4);
        const uint32_t t_p = tmem_base + Cfg::kColP + (j & 1) * 64;
#pragma unroll
        for (int kk = 0; kk < BN / 16; ++kk)
          mma_ts_elect_g<CTAS>(t_o, t_p + kk * 8, v_lo + ((kk * 2048) >> 4), kDescVHi, kIdescPV, (j > 0 || kk > 0));
        mma_commit_elect_g<CTAS>(pv_done + buf);
        mma_commit_elect_g<CTAS>(p_free + (j & 1));
        FRAY_TRACE(7, j & 1, j);
      };

      // Fixed order S(0) S(1) | S(2) PV(0) | S(3) PV(1) ...  (Issuing whichever product's barrier is ready
      // first was tried: polling two barriers without suspending took issue slots from the softmax warps
      // of the same scheduler and the suspending form reacts hundreds of cycles late; both measured slower.)
      mbar_wait(q_full, 0, abort_flag, 0x511);
      int slot = 0, buf = 0;           // jq % STAGES, jp % 3
      uint32_t k_par = 0, pv_par = 0;  // parities of the barriers those wait on
      auto next_qk = [&](int jq) __attribute__((always_inline)) {
        // K_jq has landed and both readers of S(jq - 2) hold what they need of it
        mbar_wait(k_full + slot, k_par, abort_flag, 0x501, jq);
        issue_qk(jq, slot);
        if (++slot == STAGES) {
          slot = 0;
          k_par ^= 1u;
        }
      };
      next_qk(0);
      if (n > 1) next_qk(1);
      for (int jp = 0; jp < n; ++jp) {
        if (jp + 2 < n) next_qk(jp + 2);
        FRAY_CRIT_WAIT(pv_ready + buf, pv_par, abort_flag, 0x503, jp);
        issue_pv(jp, buf);
        if (++buf == 3) {
          buf = 0;
          pv_par ^= 1u;
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
inline int launch_attn_fwd_alt(const operand_t* q, const operand_t* k, const operand_t* v, operand_t* o, const AttnShape& shp,
                               const AttnStrides (&st)[4], const AttnExtras& ex, bool causal, float scale,
                               cudaStream_t stream) {
  using Cfg = AltCfg<D, STAGES, CTAS>;
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

  auto kernel = attn_fwd_alt_kernel<D, STAGES, CTAS>;
  rc = ensure_dynamic_smem<Cfg>(kernel, Cfg::kSmemBytes, Cfg::kThreads,
                                256 * Cfg::kRegsSoftmax + 128 * Cfg::kRegsCorrection + 128 * Cfg::kRegsOther);
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
