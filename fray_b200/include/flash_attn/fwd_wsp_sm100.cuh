#pragma once
// Persistent warp-specialised attention forward for sm_100a.
//
// Same roles, tensor-memory map and per-tile pipeline as fwd_ws_sm100.cuh (two 128-row query
// tiles per CTA, softmax groups 0/1, correction group, one MMA-issue warp, one TMA producer
// warp), but one CTA per SM loops over work items - (query-tile pair, batch*head) - so that the
// tail of one item overlaps the head of the next:
//   * the producer starts loading the next item's Q tiles and first K/V tiles while the last KV
//     steps of the current item are still being consumed (Q buffers are released by the MMA warp
//     right after the item's last Q.K^T was issued);
//   * the MMA warp issues the next item's first Q.K^T for a tile directly behind that tile's last
//     P.V, so the softmax group flows from one item into the next without a bubble;
//   * the correction group's epilogue (O/l -> fp16 -> global) runs beside the next item's first
//     softmax; the first P.V of the next item waits on an "O drained" barrier.
// mbarrier phases therefore run on per-role counters that persist across items instead of the
// KV step index.
//
// Items are ordered (batch*head)-major so that CTAs running at the same time work on the same
// few heads and share their K/V through L2, and handed out round-robin (item = blockIdx.x + k *
// gridDim.x).  That static order is balanced for non-causal work; for causal work the tuner also
// has the non-persistent kernel, whose heaviest-first launch order balances better.
//
// The epilogue stores straight from registers through a small per-warp shared-memory transpose so
// that every global store instruction writes whole 64-byte row segments with 128-bit accesses.

#include "host_sm100.cuh"
#include "sm100_ptx.cuh"
#include "softmax_tile_sm100.cuh"

namespace fray {
namespace sm100 {

template <int D, int BN, int STAGES>
struct WspCfg {
  static_assert(D == 64 || D == 128, "head dim must be 64 or 128");
  static_assert(BN == 128, "the warp-specialised kernels use 128-key tiles");
  static_assert(STAGES >= 3 && STAGES <= 8, "3..8 K/V buffers");
  static constexpr int BM = 128;
  static constexpr int kThreads = 512;
  static constexpr int kPChunks = kSoftmaxPChunks;
  static constexpr int kPanels = D / 64;
  static constexpr int kQPanelBytes = BM * 128;
  static constexpr int kQTileBytes = kPanels * kQPanelBytes;
  static constexpr int kKVPanelBytes = BN * 128;
  static constexpr int kKVTileBytes = kPanels * kKVPanelBytes;
  static constexpr int kOffQ = 0;
  static constexpr int kOffKV = 2 * kQTileBytes;
  static constexpr int kOffEpi = kOffKV + STAGES * kKVTileBytes;  // 4 warps x 2 KB store-transpose scratch
  static constexpr int kOffBars = kOffEpi + 4 * 2048;
  static constexpr int kNumBars = 2 + 2 + 2 * STAGES + 2 * 6 + 2 * kPChunks;
  static constexpr int kOffStats = kOffBars + ((kNumBars * 8 + 16 + 127) / 128) * 128;  // alpha[2][128], l[2][2][128]
#ifdef FRAY_ATTN_TRACE
  static constexpr int kOffTrace = kOffStats + 6 * 128 * 4;
  static constexpr int kSmemBytes = kOffTrace + 4 * 800 + 1024;
#else
  static constexpr int kSmemBytes = kOffStats + 6 * 128 * 4 + 1024;                    // + alignment slack
#endif
  static_assert(kSmemBytes <= 232448, "exceeds the 227 KB shared memory of one CTA");
  static constexpr int kTmemCols = 512;
  static constexpr uint32_t kColS0 = 0, kColS1 = 128, kColO0 = 256, kColO1 = 384;
#ifdef FRAY_WSP_REGS_S  // tuning experiments: -DFRAY_WSP_REGS_S=.. -DFRAY_WSP_REGS_C=.. -DFRAY_WSP_REGS_O=..
  static constexpr int kRegsSoftmax = FRAY_WSP_REGS_S, kRegsCorrection = FRAY_WSP_REGS_C, kRegsOther = FRAY_WSP_REGS_O;
#else
  static constexpr int kRegsSoftmax = 168, kRegsCorrection = 96, kRegsOther = 80;
#endif
  static_assert(256 * kRegsSoftmax + 128 * kRegsCorrection + 128 * kRegsOther <= 65536, "register budgets exceed the file");
};

// Compile-time tile index handed to the generic role lambdas.
template <int I>
struct TileTag {
  static constexpr int value = I;
};

// Work item -> coordinates.  Items are numbered (batch*head)-major; within a head the pair index
// runs from the heaviest causal pair down.
struct WspItem {
  int m0, b, h, n0, n1, n_max;
};
template <int BM, int BN>
__device__ __forceinline__ WspItem wsp_decode_item(int item, int n_pairs, int num_heads, int seq_len, int causal) {
  WspItem w;
  const int bh = item / n_pairs;
  const int pidx = item - bh * n_pairs;
  const int pair = causal ? (n_pairs - 1 - pidx) : pidx;
  w.m0 = pair * (2 * BM);
  w.b = bh / num_heads;
  w.h = bh - w.b * num_heads;
  const int n_kv = (seq_len + BN - 1) / BN;
  auto tiles_for = [&](int i) {
    const int row0 = w.m0 + i * BM;
    int n = row0 < seq_len ? n_kv : 0;
    if (causal && n > 0) {
      const int lim = (row0 + BM + BN - 1) / BN;
      n = lim < n ? lim : n;
    }
    return n;
  };
  w.n0 = tiles_for(0);
  w.n1 = tiles_for(1);
  w.n_max = w.n0 > w.n1 ? w.n0 : w.n1;
  return w;
}


// ---- MMA-issue helpers of the persistent kernel.  Free functions with scalar reference parameters
// (rather than lambdas over a state struct) so that the per-tile counters stay in registers: the
// issuing warp is a serial resource and every local-memory round trip in it idles the tensor pipe.
struct WspMmaCtx {
  uint64_t* kv_full;
  uint64_t* kv_empty;
  uint64_t* q_full;
  uint64_t* q_empty;
  uint64_t* s_full;
  uint64_t* o_full;
  uint64_t* o_rescaled;
  uint64_t* o_free;
  uint64_t* p_full;
  volatile uint32_t* abort_flag;
  uint32_t q_addr, kv_addr, tmem_base;
#ifdef FRAY_ATTN_TRACE
  unsigned int* trace_sm;  // timeline table of the traced CTA, null elsewhere
#endif
};
#ifdef FRAY_ATTN_TRACE
#define WSP_TRACE(c, event, tile, iter)                                                                   \
  do {                                                                                                    \
    if ((c).trace_sm != nullptr && (iter) < kTraceIters)                                                  \
      (c).trace_sm[((event) * 2 + (tile)) * kTraceIters + (iter)] = static_cast<unsigned int>(clock64()); \
  } while (0)
#else
#define WSP_TRACE(c, event, tile, iter) do { } while (0)
#endif

// S_i = Q_i . K^T with K in ring entry t.  new_q: first use of a freshly loaded Q tile; last_user
// releases the ring entry, last_qk the Q buffer.  The tile index i is a run-time value: one copy of
// the sequence serves both tiles and every call site (the kernel is instruction-fetch sensitive).
template <class Cfg, int D, int BN, int STAGES>
__device__ __forceinline__ void wsp_issue_qk(const WspMmaCtx& c, int i, uint32_t t, bool new_q, bool last_user,
                                             bool last_qk, uint32_t& q_count) {
  constexpr uint64_t kDescK = smem_desc_sw128(16, 1024);
  constexpr uint32_t kIdescQK = idesc_f16_f32(Cfg::BM, BN, false, false);
  constexpr uint32_t kDescHi = static_cast<uint32_t>(kDescK >> 32);
  constexpr uint32_t kDescLo = static_cast<uint32_t>(kDescK);
  const int slot = t % STAGES;
  mbar_wait(c.kv_full + slot, (t / STAGES) & 1, c.abort_flag, 0x901, t);
  if (new_q) {
    mbar_wait(c.q_full + i, q_count & 1, c.abort_flag, 0x911 + i, t);
    ++q_count;
  }
  tc_fence_after_sync();
  WSP_TRACE(c, 5, i, t >> 1);  // K tile (and Q) present
  const uint32_t q_lo = kDescLo | (((c.q_addr + i * Cfg::kQTileBytes) & 0x3FFFF) >> 4);
  const uint32_t k_lo = kDescLo | (((c.kv_addr + slot * Cfg::kKVTileBytes) & 0x3FFFF) >> 4);
  const uint32_t t_s = c.tmem_base + (i == 0 ? Cfg::kColS0 : Cfg::kColS1);
#pragma unroll
  for (int kk = 0; kk < D / 16; ++kk) {
    const uint32_t qoff = ((kk >> 2) * Cfg::kQPanelBytes + (kk & 3) * 32) >> 4;
    const uint32_t koff = ((kk >> 2) * Cfg::kKVPanelBytes + (kk & 3) * 32) >> 4;
    mma_ss_elect_lohi(t_s, q_lo + qoff, kDescHi, k_lo + koff, kDescHi, kIdescQK, kk > 0);
  }
  mma_commit_elect(c.s_full + i);
  if (last_user) mma_commit_elect(c.kv_empty + slot);
  if (last_qk) mma_commit_elect(c.q_empty + i);
  WSP_TRACE(c, 7, i, t >> 1);  // S issued
}

// O_i (+)= P_i . V with V in ring entry t, chunk by chunk as P arrives.
template <class Cfg, int D, int BN, int STAGES>
__device__ __forceinline__ void wsp_issue_pv(const WspMmaCtx& c, int i, int j, uint32_t t, bool last_user,
                                             uint32_t& pv_count, uint32_t& resc_count, uint32_t items_done) {
  constexpr uint64_t kDescV = smem_desc_sw128(Cfg::kKVPanelBytes, 1024);
  constexpr uint32_t kIdescPV = idesc_f16_f32(Cfg::BM, D, false, true);
  constexpr uint32_t kDescVHi = static_cast<uint32_t>(kDescV >> 32);
  constexpr int kStepsPerChunk = (BN / 16) / Cfg::kPChunks;
  const int slot = t % STAGES;
  // A wait on an mbarrier costs this warp a shared-memory round trip (50-100 cycles) even when the
  // phase is long complete.  When this warp arrives late, everything is: test all barriers of the
  // step together first (the round trips overlap) and fall back to the one-by-one waits otherwise.
  uint64_t* b_o = j > 0 ? c.o_rescaled + i : c.o_free + i;
  const uint32_t par_o = j > 0 ? (resc_count & 1) : ((items_done - 1) & 1);
  const bool need_o = j > 0 || items_done > 0;
  bool ready = mbar_test_wait(c.kv_full + slot, (t / STAGES) & 1);  // non-blocking tests
#pragma unroll
  for (int q = 0; q < Cfg::kPChunks; ++q) ready = ready & mbar_test_wait(c.p_full + i * Cfg::kPChunks + q, pv_count & 1);
  if (need_o) ready = ready & mbar_test_wait(b_o, par_o);
  if (!ready) {
    mbar_wait(c.kv_full + slot, (t / STAGES) & 1, c.abort_flag, 0x902, t);
    if (need_o) mbar_wait(b_o, par_o, c.abort_flag, (j > 0 ? 0x905 : 0x907) + i, j);
  }
  if (j > 0) ++resc_count;
  const uint32_t v_lo = static_cast<uint32_t>(kDescV) | (((c.kv_addr + slot * Cfg::kKVTileBytes) & 0x3FFFF) >> 4);
  const uint32_t t_p = c.tmem_base + (i == 0 ? Cfg::kColS0 : Cfg::kColS1);
  const uint32_t t_o = c.tmem_base + (i == 0 ? Cfg::kColO0 : Cfg::kColO1);
  if (ready) tc_fence_after_sync();
#pragma unroll
  for (int q = 0; q < Cfg::kPChunks; ++q) {
    if (!ready) {
      FRAY_CRIT_WAIT(c.p_full + i * Cfg::kPChunks + q, pv_count & 1, c.abort_flag, 0x903 + i, j);
      tc_fence_after_sync();
    }
#pragma unroll
    for (int s2 = 0; s2 < kStepsPerChunk; ++s2) {
      const int kk = q * kStepsPerChunk + s2;
      mma_ts_elect_lohi(t_o, t_p + kk * 8, v_lo + ((kk * 2048) >> 4), kDescVHi, kIdescPV, (j > 0 || kk > 0));
    }
  }
  ++pv_count;
  mma_commit_elect(c.o_full + i);
  if (last_user) mma_commit_elect(c.kv_empty + slot);
  WSP_TRACE(c, 3, i, pv_count - 1);  // P.V issued
}

// One tile's share of KV step j of item w (j = -1: the item's lead-in, where only a first Q.K^T may
// be due).  nx is the next item of this CTA (valid when has_next).  At most one P.V and one Q.K^T are
// issued; which Q.K^T (the next step's, the item's first, or the next item's first) is decided first
// so that the sequence itself exists once.
template <class Cfg, int D, int BN, int STAGES>
__device__ __forceinline__ void wsp_tile_step(const WspMmaCtx& c, int i, const WspItem& w, const WspItem& nx,
                                              bool has_next, int j, uint32_t t_base, uint32_t t_next,
                                              uint32_t& q_count, uint32_t& pv_count, uint32_t& resc_count,
                                              uint32_t& items_done, bool& started) {
  const int n_i = i ? w.n1 : w.n0;
  if (n_i == 0) return;
  if (j >= 0 && j < n_i)
    wsp_issue_pv<Cfg, D, BN, STAGES>(c, i, j, t_base + 2 * j + 1, (i == 1) || !(j < w.n1), pv_count, resc_count,
                                     items_done);
  bool do_qk = false, new_q = false, last_user = false, last_qk = false;
  uint32_t t_qk = 0;
  if (j + 1 < n_i) {
    if (j >= 0) {
      do_qk = true;
      t_qk = t_base + 2 * (j + 1);
      last_user = (i == 1) || !(j + 1 < w.n1);
      last_qk = j + 2 == n_i;
    } else {
      if (!started) {
        do_qk = true;
        t_qk = t_base;
        new_q = true;
        last_user = (i == 1) || !(0 < w.n1);
        last_qk = n_i == 1;
      }
      started = false;
    }
  } else if (j + 1 == n_i) {
    // Tile i has finished this item.  Start it on the next item right away when the ring can hold
    // that item's K_0 beside everything the other tile still needs.
    ++items_done;
    const int nn_i = i ? nx.n1 : nx.n0;
    if (has_next && nn_i > 0 && 2 * (w.n_max - n_i) + 2 <= STAGES) {
      do_qk = true;
      t_qk = t_next;
      new_q = true;
      last_user = (i == 1) || !(0 < nx.n1);
      last_qk = nn_i == 1;
      started = true;
    }
  }
  if (do_qk) wsp_issue_qk<Cfg, D, BN, STAGES>(c, i, t_qk, new_q, last_user, last_qk, q_count);
}

template <int D, int BN, int STAGES, int POLY>
__global__ void __launch_bounds__(512, 1)
attn_fwd_wsp_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                    const __grid_constant__ CUtensorMap tm_v, operand_t* __restrict__ o_ptr, int64_t o_sb, int64_t o_sh,
                    int64_t o_ss, int num_heads, int seq_len, int causal, float scale_log2, int n_pairs, int n_items) {
  using Cfg = WspCfg<D, BN, STAGES>;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  uint8_t* smem = smem_raw + (((raw_addr + 1023u) & ~1023u) - raw_addr);
  uint8_t* q_smem = smem + Cfg::kOffQ;
  uint8_t* kv_smem = smem + Cfg::kOffKV;
  uint8_t* epi_smem = smem + Cfg::kOffEpi;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Cfg::kOffBars);
  uint64_t* q_full = bars;                      // [2] producer -> MMA
  uint64_t* q_empty = q_full + 2;               // [2] MMA -> producer (item's last Q.K^T of the tile issued and done)
  uint64_t* kv_full = q_empty + 2;              // [STAGES]
  uint64_t* kv_empty = kv_full + STAGES;        // [STAGES]
  uint64_t* s_full = kv_empty + STAGES;         // [2] MMA -> softmax i
  uint64_t* o_full = s_full + 2;                // [2] MMA -> correction (a P.V step complete)
  uint64_t* corr_ready = o_full + 2;            // [2] softmax i -> correction (alpha / final l published)
  uint64_t* o_rescaled = corr_ready + 2;        // [2] correction -> MMA (O_i ready for the next P.V step)
  uint64_t* o_free = o_rescaled + 2;            // [2] correction -> MMA (O_i of the finished item read out)
  uint64_t* p_full = o_free + 2;                // [2][kPChunks] softmax i -> MMA
  uint64_t* sfu_turn = p_full + 2 * Cfg::kPChunks;  // [2] softmax (1-i) -> softmax i: the special-function unit is yours
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + Cfg::kNumBars);
  volatile uint32_t* abort_flag = reinterpret_cast<volatile uint32_t*>(tmem_slot + 1);
  float* alpha_buf = reinterpret_cast<float*>(smem + Cfg::kOffStats);  // [2][128]
  float* l_buf = alpha_buf + 256;                                      // [item parity][2][128]

#ifdef FRAY_ATTN_TRACE
  // Role timeline (see fwd_ws_sm100.cuh); here the "iteration" is the tile's running KV-step count,
  // so the first 40 entries cover the first item and the hand-over into the second.
  unsigned int* trace_sm = reinterpret_cast<unsigned int*>(smem + Cfg::kOffTrace);
  const bool trace_on = blockIdx.x == 0;
#endif
  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;

  if (tid == 0) {
    *abort_flag = (*reinterpret_cast<volatile int*>(&fray_attn_status[0]) != 0) ? 2u : 0u;
    for (int i = 0; i < 2; ++i) {
      mbar_init(q_full + i, 1);
      mbar_init(q_empty + i, 1);
      mbar_init(s_full + i, 1);
      mbar_init(o_full + i, 1);
      mbar_init(corr_ready + i, 4);  // one arrival per warp
      mbar_init(o_rescaled + i, 4);
      mbar_init(o_free + i, 4);
      mbar_init(sfu_turn + i, 4);
      for (int c = 0; c < Cfg::kPChunks; ++c) mbar_init(p_full + i * Cfg::kPChunks + c, 4);
    }
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(kv_full + s, 1);
      mbar_init(kv_empty + s, 1);
    }
    fence_barrier_init();
    prefetch_tensormap(&tm_q);
    prefetch_tensormap(&tm_k);
    prefetch_tensormap(&tm_v);
  }
  __syncthreads();
  if (*abort_flag != 0) return;  // an earlier launch left the device status raised

  if (warp == 0) {
    tmem_alloc(tmem_slot, Cfg::kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  const int first_item = blockIdx.x;
  const int item_step = gridDim.x;

  if (warp < 8) {
    // =============================================================== softmax groups
    set_max_regs_inc<Cfg::kRegsSoftmax>();
    const int i = warp >> 2;
    const int r = tid & 127;
    const uint32_t lane_base = static_cast<uint32_t>((warp & 3) * 32) << 16;
    const uint32_t t_s = tmem_base + (i == 0 ? Cfg::kColS0 : Cfg::kColS1) + lane_base;
    uint64_t* p_bar = p_full + i * Cfg::kPChunks;
    uint32_t s_count = 0;     // S tiles consumed so far by this group (phase of s_full)
    uint32_t item_count = 0;  // items in which this tile was active (selects the l hand-over buffer)
    uint32_t turn_count = 0;  // KV steps taken under the special-function turn-taking so far

    for (int item = first_item; item < n_items; item += item_step) {
      const WspItem w = wsp_decode_item<Cfg::BM, BN>(item, n_pairs, num_heads, seq_len, causal);
      const int n_i = i ? w.n1 : w.n0;
      if (n_i == 0) continue;
      const int row0 = w.m0 + i * Cfg::BM;
      const int row = row0 + r;
      float m_ref = -INFINITY;
      float l_run = 0.f;
      for (int j = 0; j < n_i; ++j) {
        FRAY_CRIT_WAIT(s_full + i, s_count & 1, abort_flag, 0x601 + i, j);
        if (r == 0) FRAY_TRACE(0, i, s_count);
        ++s_count;
        tc_fence_after_sync();
        const int kv0 = j * BN;
        const bool need_mask = (kv0 + BN > seq_len) || (causal && (kv0 + BN - 1 > row0));
        // Steps both tiles run take turns on the special-function unit, tile 0 first.
        const bool take_turns = kSfuTurns && j < (w.n0 < w.n1 ? w.n0 : w.n1);
        softmax_tile<BN, POLY>(t_s, p_bar, corr_ready + i, alpha_buf + i * 128 + r, j == 0, need_mask, kv0, row,
                               seq_len, causal, scale_log2, lane, m_ref, l_run, take_turns ? sfu_turn + i : nullptr,
                               take_turns ? sfu_turn + (1 - i) : nullptr, (turn_count + 1 - i) & 1, abort_flag);
        if (take_turns) ++turn_count;
        if (r == 0) FRAY_TRACE(4, i, s_count - 1);
      }
      l_buf[(item_count & 1) * 256 + i * 128 + r] = l_run;
      ++item_count;
      __syncwarp();
      if (lane == 0) mbar_arrive(corr_ready + i);
    }
  } else if (warp < 12) {
    // =============================================================== correction group + epilogue
    set_max_regs_dec<Cfg::kRegsCorrection>();
    const int r = tid & 127;
    const int cw = warp & 3;
    const uint32_t lane_base = static_cast<uint32_t>(cw * 32) << 16;
    uint8_t* tr = epi_smem + cw * 2048;  // this warp's 32 rows x 64 bytes store-transpose scratch
    // per-tile counters as scalars (an indexed array would live in local memory)
    uint32_t corr_count0 = 0, corr_count1 = 0;  // corr_ready phases consumed
    uint32_t pv_base0 = 0, pv_base1 = 0;        // P.V steps of earlier items (phase base of o_full)
    uint32_t item_count0 = 0, item_count1 = 0;

    for (int item = first_item; item < n_items; item += item_step) {
      const WspItem w = wsp_decode_item<Cfg::BM, BN>(item, n_pairs, num_heads, seq_len, causal);
      for (int j = 1; j <= w.n_max; ++j) {
#pragma unroll
        for (int i = 0; i < 2; ++i) {
          const int n_i = i ? w.n1 : w.n0;
          const uint32_t t_o = tmem_base + (i == 0 ? Cfg::kColO0 : Cfg::kColO1) + lane_base;
          uint32_t& corr_count = i ? corr_count1 : corr_count0;
          uint32_t& pv_base = i ? pv_base1 : pv_base0;
          uint32_t& item_count = i ? item_count1 : item_count0;
          if (j < n_i) {
            // rescale step: O_i *= alpha before P.V step j of this tile
            mbar_wait(corr_ready + i, corr_count & 1, abort_flag, 0x701 + i, j);
            ++corr_count;
            const float alpha = alpha_buf[i * 128 + r];
            if (__any_sync(0xffffffffu, alpha != 1.f)) {
              mbar_wait(o_full + i, (pv_base + j - 1) & 1, abort_flag, 0x711 + i, j);
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
            if (lane == 0) mbar_arrive(o_rescaled + i);
          } else if (j == n_i) {
            // epilogue of tile i: O_i / l -> fp16 -> global
            mbar_wait(corr_ready + i, corr_count & 1, abort_flag, 0x721 + i, j);
            ++corr_count;
            const float l = l_buf[(item_count & 1) * 256 + i * 128 + r];
            const float inv_l = l > 0.f ? 1.f / l : 1.f;
            mbar_wait(o_full + i, (pv_base + n_i - 1) & 1, abort_flag, 0x731 + i, j);
            tc_fence_after_sync();
            if (r == 0) FRAY_TRACE(6, i, item_count);  // epilogue of this tile starts
            const int row0 = w.m0 + i * Cfg::BM + cw * 32;  // first row of this warp
            operand_t* o_base = o_ptr + static_cast<int64_t>(w.b) * o_sb + static_cast<int64_t>(w.h) * o_sh;
#pragma unroll
            for (int c = 0; c < D / 32; ++c) {
              uint32_t orr[32];
              tmem_ld_x32(t_o + c * 32, orr);
              tmem_wait_ld();
              if (c == D / 32 - 1) {
                // every row of O_i is in registers now: the next item's first P.V may overwrite it
                tc_fence_before_sync();
                __syncwarp();
                if (lane == 0) mbar_arrive(o_free + i);
              }
              // lane = row: 64 bytes (32 halves) into the transpose scratch, 16-byte pieces swizzled by row
#pragma unroll
              for (int k = 0; k < 4; ++k) {
                uint4 v4;
                v4.x = pack_half2(__uint_as_float(orr[8 * k + 0]) * inv_l, __uint_as_float(orr[8 * k + 1]) * inv_l);
                v4.y = pack_half2(__uint_as_float(orr[8 * k + 2]) * inv_l, __uint_as_float(orr[8 * k + 3]) * inv_l);
                v4.z = pack_half2(__uint_as_float(orr[8 * k + 4]) * inv_l, __uint_as_float(orr[8 * k + 5]) * inv_l);
                v4.w = pack_half2(__uint_as_float(orr[8 * k + 6]) * inv_l, __uint_as_float(orr[8 * k + 7]) * inv_l);
                *reinterpret_cast<uint4*>(tr + lane * 64 + ((k ^ ((lane >> 1) & 3)) << 4)) = v4;
              }
              __syncwarp();
              // 4 lanes per row, 8 rows per instruction: each store covers whole 64-byte row segments
#pragma unroll
              for (int g = 0; g < 4; ++g) {
                const int rr = g * 8 + (lane >> 2);
                const int k = lane & 3;
                const uint4 v4 = *reinterpret_cast<const uint4*>(tr + rr * 64 + ((k ^ ((rr >> 1) & 3)) << 4));
                const int grow = row0 + rr;
                if (grow < seq_len)
                  *reinterpret_cast<uint4*>(o_base + static_cast<int64_t>(grow) * o_ss + c * 32 + k * 8) = v4;
              }
              __syncwarp();
            }
            if (r == 0) FRAY_TRACE(9, i, item_count);  // epilogue done
            pv_base += n_i;
            ++item_count;
          }
        }
      }
    }
  } else {
    set_max_regs_dec<Cfg::kRegsOther>();
    if (warp == 13 && lane == 0) {
      // ============================================================= TMA producer
      uint32_t t = 0;                 // running K/V ring index
      uint32_t q_loaded0 = 0, q_loaded1 = 0;  // Q tiles loaded so far per tile slot
      for (int item = first_item; item < n_items; item += item_step) {
        const WspItem w = wsp_decode_item<Cfg::BM, BN>(item, n_pairs, num_heads, seq_len, causal);
        auto load_q = [&](int i) __attribute__((always_inline)) {
          if ((i ? w.n1 : w.n0) > 0) {
            uint32_t& q_loaded = i ? q_loaded1 : q_loaded0;
            if (q_loaded > 0) mbar_wait(q_empty + i, (q_loaded - 1) & 1, abort_flag, 0x801 + i, item);
            ++q_loaded;
            mbar_expect_tx(q_full + i, Cfg::kQTileBytes);
#pragma unroll
            for (int p = 0; p < Cfg::kPanels; ++p)
              tma_load_4d(q_smem + i * Cfg::kQTileBytes + p * Cfg::kQPanelBytes, &tm_q, q_full + i, p * 64,
                          w.m0 + i * Cfg::BM, w.h, w.b);
          }
        };
        load_q(0);
        for (int tt = 0; tt < 2 * w.n_max; ++tt, ++t) {
          const int slot = t % STAGES;
          mbar_wait(kv_empty + slot, ((t / STAGES) & 1) ^ 1, abort_flag, 0x811, tt);
          mbar_expect_tx(kv_full + slot, Cfg::kKVTileBytes);
          const CUtensorMap* tm = (tt & 1) ? &tm_v : &tm_k;
#pragma unroll
          for (int p = 0; p < Cfg::kPanels; ++p)
            tma_load_4d(kv_smem + slot * Cfg::kKVTileBytes + p * Cfg::kKVPanelBytes, tm, kv_full + slot, p * 64,
                        (tt >> 1) * BN, w.h, w.b);
          if (tt == 0) load_q(1);
        }
      }
    } else if (warp == 12) {
      // ============================================================= MMA issue (whole warp, one elected lane issues)
      // One warp serves both tiles in a fixed alternation (tile 0's step, tile 1's step, ...): that
      // ordering is what keeps the tiles half a step apart, one in its softmax while the other owns
      // the tensor pipe.  Per tile the order is K/V ring order - entry K_j: S_i(j) = Q_i.K_j^T, entry
      // V_j: O_i += P_i(j).V_j - and it carries over from one item to the next, so a tile's first
      // Q.K^T of the next item follows its last P.V directly.
      const WspMmaCtx ctx{kv_full, kv_empty, q_full, q_empty, s_full, o_full, o_rescaled, o_free, p_full,
                          abort_flag, smem_u32(q_smem), smem_u32(kv_smem), tmem_base
#ifdef FRAY_ATTN_TRACE
                          , trace_on ? trace_sm : nullptr
#endif
      };
      // per-tile progress, plain scalars
      uint32_t q_count0 = 0, q_count1 = 0;        // q_full phases consumed
      uint32_t pv_count0 = 0, pv_count1 = 0;      // P.V steps issued (phase of the p_full chunks)
      uint32_t resc_count0 = 0, resc_count1 = 0;  // o_rescaled phases consumed
      uint32_t items_done0 = 0, items_done1 = 0;  // items finished (phase of o_free)
      bool started0 = false, started1 = false;    // first Q.K^T already issued from the previous item's tail
      uint32_t t_base = 0;                        // ring index of the current item's K_0
      for (int item = first_item; item < n_items; item += item_step) {
        const WspItem w = wsp_decode_item<Cfg::BM, BN>(item, n_pairs, num_heads, seq_len, causal);
        const bool has_next = item + item_step < n_items;
        WspItem nx = w;
        if (has_next) nx = wsp_decode_item<Cfg::BM, BN>(item + item_step, n_pairs, num_heads, seq_len, causal);
        const uint32_t t_next = t_base + 2 * w.n_max;  // ring index of the next item's K_0
        for (int j = -1; j < w.n_max; ++j) {
#pragma unroll 1
          for (int i = 0; i < 2; ++i) {
            // per-tile progress lives in scalars; pick this tile's, run the step, put them back
            uint32_t qc = i ? q_count1 : q_count0, pc = i ? pv_count1 : pv_count0, rc = i ? resc_count1 : resc_count0;
            uint32_t dn = i ? items_done1 : items_done0;
            bool st = i ? started1 : started0;
            if (j >= 0) FRAY_TRACE(1, i, pc);  // MMA warp reaches tile i's share of step j
            wsp_tile_step<Cfg, D, BN, STAGES>(ctx, i, w, nx, has_next, j, t_base, t_next, qc, pc, rc, dn, st);
            if (j >= 0) FRAY_TRACE(2, i, pc - 1);  // ... and leaves it
            if (i) {
              q_count1 = qc, pv_count1 = pc, resc_count1 = rc, items_done1 = dn, started1 = st;
            } else {
              q_count0 = qc, pv_count0 = pc, resc_count0 = rc, items_done0 = dn, started0 = st;
            }
          }
        }
        t_base = t_next;
      }
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem_base, Cfg::kTmemCols);
#ifdef FRAY_ATTN_TRACE
  if (trace_on)
    for (int x = tid; x < kTraceWords; x += Cfg::kThreads) fray_attn_trace_buf[x] = trace_sm[x];
#endif
}

// Host launcher for the persistent kernel. Returns an AttnReturnCode.
template <int D, int BN, int STAGES, int POLY>
inline int launch_attn_fwd_wsp(const operand_t* q, const operand_t* k, const operand_t* v, operand_t* o, const AttnShape& shp,
                               const AttnStrides (&st)[4], bool causal, float scale, cudaStream_t stream) {
  using Cfg = WspCfg<D, BN, STAGES>;
  static_assert((POLY >= 0 && POLY <= 4) || POLY == kExpPackedHalf, "POLY: 0..4 polynomial pairs of 4, or 16 = packed fp16");
  CUtensorMap tm_q, tm_k, tm_v;
  int rc = cached_attn_tensor_map(&tm_q, q, shp, st[0], Cfg::BM);
  if (rc != kAttnOk) return rc;
  rc = cached_attn_tensor_map(&tm_k, k, shp, st[1], BN);
  if (rc != kAttnOk) return rc;
  rc = cached_attn_tensor_map(&tm_v, v, shp, st[2], BN);
  if (rc != kAttnOk) return rc;

  auto kernel = attn_fwd_wsp_kernel<D, BN, STAGES, POLY>;
  static int num_sms = 0;  // one process drives one GPU: query and set once
  if (num_sms == 0) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess ||
        cudaDeviceGetAttribute(&num_sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || num_sms <= 0 ||
        cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes) != cudaSuccess) {
      (void)cudaGetLastError();
      num_sms = 0;
      return kAttnSmemAttrFailed;
    }
  }
  const int n_pairs = (shp.S + 2 * Cfg::BM - 1) / (2 * Cfg::BM);
  const int64_t n_items64 = static_cast<int64_t>(n_pairs) * shp.B * shp.H;
  if (n_items64 > 0x7FFFFFFFLL) return kAttnBadShape;
  const int n_items = static_cast<int>(n_items64);
  const int grid = n_items < num_sms ? n_items : num_sms;
  kernel<<<grid, Cfg::kThreads, Cfg::kSmemBytes, stream>>>(tm_q, tm_k, tm_v, o, st[3].b, st[3].h, st[3].s, shp.H,
                                                           shp.S, causal ? 1 : 0,
                                                           scale * 1.44269504088896340736f, n_pairs, n_items);
  if (cudaGetLastError() != cudaSuccess) return kAttnLaunchFailed;
  return kAttnOk;
}

}  // namespace sm100
}  // namespace fray
