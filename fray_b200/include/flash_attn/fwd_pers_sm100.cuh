#pragma once
// Persistent form of the two-tile warp-specialised attention forward (fwd_ws_sm100.cuh) for sm_100a.
//
// The grid is one CTA per SM (or one per work item when there are fewer); a CTA walks through the work
// items blockIdx.x, blockIdx.x + gridDim.x, ...  A work item is what a CTA of the two-tile kernel
// does: two 128-row query tiles of one (batch, head) slice against all of their KV tiles.  Roles,
// tensor-memory layout, softmax step and issue order inside an item are those of the two-tile kernel;
// what changes is what happens BETWEEN items, which in the two-tile kernel is a CTA's exit and the
// next CTA's set-up (barrier initialisation, tensor-memory allocation, the latency of the very first
// copies: ~12 000 cycles per item, 9 % of an item at 4096 keys and a third of it at 1024):
//
//   * barriers, tensor memory and the K/V ring live for the whole kernel; every barrier's phase is
//     tracked by a running count instead of the step index, so the ring simply keeps turning;
//   * the producer fetches the next item's Q tiles as soon as the MMA warp's commit says that the
//     last S = Q.K^T of the current item has read them (q_free), and its K/V tiles behind the
//     current item's (three ring slots: the staging tiles take the fourth);
//   * the MMA warp issues the next item's first S of a tile right behind the current item's last
//     P.V of that tile (the slot the two-tile kernel leaves empty), so the softmax group finds scores
//     waiting when it returns from its epilogue;
//   * the epilogue has staging tiles of its own (one per query tile, behind the ring), so the Q buffers can
//     take the next item's tiles early; it hands the accumulator back (o_free: the next item's first P.V
//     of that tile waits for it) as soon as its last columns are in registers, and the TMA store of an
//     item is only waited for (its reads of the staging tile) when the next item's epilogue begins.
//     (Writing the rows straight from registers with 16-byte stores, 256 bytes apart from lane to lane,
//     took 4800 cycles per tile on the tile's critical path.)
//   * work items are numbered slice by slice and dealt round-robin; with a causal mask the direction
//     alternates from round to round, which evens out most of the causal pairs' unequal lengths without
//     a shared counter.
//
// Measured against the two-tile kernel on shapes with exactly eight items per SM: 3.5 us per item
// instead of 6.5-8.7, 2.03 us per KV step instead of 1.91-1.93 (three ring slots instead of four, and an
// SM that never idles runs at a lower clock under the board's power limit): ahead up to 2048 keys
// (+10 % at 1024, +2.5 % at 2048), behind from 4096 on (-1.7 %, -3.5 % at 8192).
//
// Every barrier wait is bounded (see sm100_ptx.cuh): a protocol error ends as a status word and a
// wrong answer, never as a hung GPU.

#include "fwd_ws_sm100.cuh"

namespace fray {
namespace sm100 {

template <int D, int BN, int STAGES>
struct PersCfg {
  using Base = WsCfg<D, BN, STAGES>;
  static constexpr int BM = Base::BM;
  static constexpr int kPChunks = Base::kPChunks;
  static constexpr int kThreads = Base::kThreads;
  static constexpr int kPanels = Base::kPanels;
  static constexpr int kQPanelBytes = Base::kQPanelBytes;
  static constexpr int kQTileBytes = Base::kQTileBytes;
  static constexpr int kKVPanelBytes = Base::kKVPanelBytes;
  static constexpr int kKVTileBytes = Base::kKVTileBytes;
  static constexpr int kOffQ = Base::kOffQ;
  static constexpr int kOffKV = Base::kOffKV;
  static constexpr int kOffStage = Base::kOffBars;                   // O staging tiles (one per query tile) behind the ring
  static constexpr int kOffBars = kOffStage + 2 * kQTileBytes;
  static constexpr int kNumBars = Base::kNumBars + 4;  // + q_free[2], o_free[2]
  static constexpr int kOffStats = kOffBars + ((kNumBars * 8 + 16 + 127) / 128) * 128;  // alpha[2][128]
  static constexpr int kSmemBytes = kOffStats + 2 * 128 * 4 + 1024;                     // + alignment slack
  static_assert(kSmemBytes <= 232448, "exceeds the 227 KB shared memory of one CTA");
  static constexpr int kTmemCols = Base::kTmemCols;
  static constexpr uint32_t kColS0 = Base::kColS0, kColS1 = Base::kColS1, kColO0 = Base::kColO0, kColO1 = Base::kColO1;
  static constexpr int kRegsSoftmax = Base::kRegsSoftmax, kRegsCorrection = Base::kRegsCorrection, kRegsOther = Base::kRegsOther;
};

// One work item: the rows [m0, m0 + 256) of slice (b, h) and the KV tiles each of its two query tiles consumes.
struct PersItem {
  int m0, b, h, h_kv, n0, n1;
};

template <int D, int BN, int STAGES>
__global__ void __launch_bounds__(512, 1)
attn_fwd_pers_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                     const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_o, int num_heads,
                     int num_bh, int seq_len, int causal, float scale_log2, int kv_group, float* lse, int seq_k, int blk) {
  using Cfg = PersCfg<D, BN, STAGES>;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  uint8_t* smem = smem_raw + (((raw_addr + 1023u) & ~1023u) - raw_addr);
  uint8_t* q_smem = smem + Cfg::kOffQ;    // tile i at q_smem + i * kQTileBytes
  uint8_t* kv_smem = smem + Cfg::kOffKV;  // ring slot s at kv_smem + s * kKVTileBytes
  uint8_t* stage_smem = smem + Cfg::kOffStage;  // O tile of query tile i at stage_smem + i * kQTileBytes
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Cfg::kOffBars);
  uint64_t* q_full = bars;                      // [2]   producer -> MMA
  uint64_t* kv_full = bars + 2;                 // [STAGES] producer -> MMA
  uint64_t* kv_empty = kv_full + STAGES;        // [STAGES] MMA -> producer
  uint64_t* s_full = kv_empty + STAGES;         // [2]   MMA -> softmax i        (S_i complete)
  uint64_t* o_full = s_full + 2;                // [2]   MMA -> correction, softmax i (a P.V of tile i complete)
  uint64_t* corr_ready = o_full + 2;            // [2]   softmax i -> correction (alpha_i published)
  uint64_t* o_rescaled = corr_ready + 2;        // [2]   correction -> MMA       (O_i ready for the next P.V)
  uint64_t* p_full = o_rescaled + 2;            // [2][kPChunks] softmax i -> MMA (chunk c of P_i stored)
  uint64_t* q_free = p_full + 2 * Cfg::kPChunks;  // [2] MMA -> producer  (the item's last S of tile i has read Q_i)
  uint64_t* o_free = q_free + 2;                // [2]   softmax i -> MMA        (the item's O_i is in registers)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + Cfg::kNumBars);
  volatile uint32_t* abort_flag = reinterpret_cast<volatile uint32_t*>(tmem_slot + 1);
  float* alpha_buf = reinterpret_cast<float*>(smem + Cfg::kOffStats);  // [2][128]

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;

  const int n_kv = (seq_k + BN - 1) / BN;                     // seq_len counts queries, seq_k keys
  const int n_pairs = (seq_len + 2 * Cfg::BM - 1) / (2 * Cfg::BM);
  const int total = n_pairs * num_bh;
  const int stride = static_cast<int>(gridDim.x);
  // Items are numbered in blocks of `blk` slices; inside a block the pairs of all its slices come heaviest
  // first (pair by pair, slice by slice).  blk = 1 is plain slice-major order: CTAs that run side by side work
  // on the same slice and share its K and V in L2, which matters more than balance as soon as K and V of the
  // slices in flight no longer sit in L2 together (4 x 32 x 4096 causal: 981 TFLOP/s with blk = 1, 917-947 with
  // 16, 847-883 with 37).  A small causal problem has the opposite trouble, one or two rounds of very unequal
  // items: with blk = all slices a single 16-head causal batch of 4096 rows runs at 690-750 instead of 525.
  // The launcher picks.  CTA c takes the positions c, G + c, 2G + c, ...; with a causal mask the direction
  // alternates from round to round (c, 2G-1-c, 2G+c, ...), which evens out most of what is left.
  auto pos = [&](int k) {
    const int c = static_cast<int>(blockIdx.x);
    return k * stride + ((causal && (k & 1)) ? stride - 1 - c : c);  // >= total: the CTA is done; grows with k
  };
  auto decode = [&](int idx) {
    PersItem it;
    const int blk_items = blk * n_pairs;
    const int blk_i = idx / blk_items;
    const int rem = idx - blk_i * blk_items;
    const int left = num_bh - blk_i * blk;
    const int ns = left < blk ? left : blk;  // slices of this block (the last block may be short)
    const int pr = rem / ns;
    const int bh = blk_i * blk + (rem - pr * ns);
    const int pair = causal ? (n_pairs - 1 - pr) : pr;
    it.m0 = pair * (2 * Cfg::BM);
    it.b = bh / num_heads;
    it.h = bh - it.b * num_heads;
    it.h_kv = it.h / kv_group;
    int n[2];
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const int row0 = it.m0 + i * Cfg::BM;
      n[i] = row0 < seq_len ? n_kv : 0;
      if (causal && n[i] > 0) {
        const int lim = (row0 + Cfg::BM + BN - 1) / BN;
        n[i] = lim < n[i] ? lim : n[i];
      }
    }
    it.n0 = n[0];
    it.n1 = n[1];
    return it;
  };

  if (tid == 0) {
    *abort_flag = (*reinterpret_cast<volatile int*>(&fray_attn_status[0]) != 0) ? 2u : 0u;
    for (int i = 0; i < 2; ++i) {
      mbar_init(q_full + i, 1);
      mbar_init(s_full + i, 1);
      for (int c = 0; c < Cfg::kPChunks; ++c) mbar_init(p_full + i * Cfg::kPChunks + c, 4);  // one arrival per warp
      mbar_init(o_full + i, 1);
      mbar_init(corr_ready + i, 4);
      mbar_init(o_rescaled + i, 4);
      mbar_init(q_free + i, 1);
      mbar_init(o_free + i, 4);
    }
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(kv_full + s, 1);
      mbar_init(kv_empty + s, 1);
    }
    fence_barrier_init();
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

  if (warp < 8) {
    // =============================================================== softmax groups
    set_max_regs_inc<Cfg::kRegsSoftmax>();
    const int i = warp >> 2;  // query tile of this group
    const int r = tid & 127;  // row inside the tile
    const uint32_t lane_base = static_cast<uint32_t>((warp & 3) * 32) << 16;
    const uint32_t t_s = tmem_base + (i == 0 ? Cfg::kColS0 : Cfg::kColS1) + lane_base;
    const uint32_t t_o = tmem_base + (i == 0 ? Cfg::kColO0 : Cfg::kColO1) + lane_base;
    uint64_t* p_bar = p_full + i * Cfg::kPChunks;
    uint32_t steps = 0;  // steps of tile i this CTA has taken so far, over all items: phase of s_full, o_full
    for (int k = 0, idx = pos(0); idx < total; idx = pos(++k)) {
      const PersItem it = decode(idx);
      const int n_i = i ? it.n1 : it.n0;
      if (n_i == 0) continue;
      const int row0 = it.m0 + i * Cfg::BM;
      const int row = row0 + r;
      float m_ref = -INFINITY;  // exponent offset currently baked into P, l and O
      float l_run = 0.f;
      for (int j = 0; j < n_i; ++j) {
        FRAY_CRIT_WAIT(s_full + i, steps & 1, abort_flag, 0x201 + i, j);
        tc_fence_after_sync();
        const int kv0 = j * BN;
        const bool need_mask = (kv0 + BN > seq_k) || (causal && (kv0 + BN - 1 > row0));
        if (need_mask) {
          softmax_tile<BN, Cfg::kPChunks, true>(t_s, p_bar, corr_ready + i, alpha_buf + i * 128 + r, j == 0, kv0, row, seq_k,
                                                causal, scale_log2, lane, m_ref, l_run);
        } else {
          softmax_tile<BN, Cfg::kPChunks, false>(t_s, p_bar, corr_ready + i, alpha_buf + i * 128 + r, j == 0, kv0, row, seq_k,
                                                 causal, scale_log2, lane, m_ref, l_run);
        }
        ++steps;
      }
      // Epilogue: wait for the item's last P.V, then O / l -> 16 bit -> this tile's staging buffer -> TMA store.
      // The store of the previous item must have read the buffer first; the accumulator is handed back
      // (o_free) as soon as its last columns are in registers.
      mbar_wait(o_full + i, (steps - 1) & 1, abort_flag, 0x331 + i, n_i);
      tc_fence_after_sync();
      if (r == 0) tma_store_wait_read();
      named_barrier_sync(4 + i, 128);
      {
        uint8_t* o_tile = stage_smem + i * Cfg::kQTileBytes;
        const float inv_l = l_run > 0.f ? 1.f / l_run : 1.f;
#pragma unroll
        for (int c = 0; c < D / 32; ++c) {
          uint32_t orr[32];
          tmem_ld_x32(t_o + c * 32, orr);
          tmem_wait_ld();
          if (c == D / 32 - 1) {
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(o_free + i);
          }
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
        named_barrier_sync(4 + i, 128);
        if (r == 0) {
#pragma unroll
          for (int p = 0; p < Cfg::kPanels; ++p) tma_store_4d(&tm_o, o_tile + p * Cfg::kQPanelBytes, p * 64, row0, it.h, it.b);
          tma_store_commit();
        }
        if (lse != nullptr && row < seq_len) {
          lse[(static_cast<size_t>(it.b) * num_heads + it.h) * seq_len + row] =
              l_run > 0.f ? (m_ref * scale_log2 + log2f(l_run)) * 0.69314718055994531f : -INFINITY;
        }
      }
    }
    if (r == 0) tma_store_wait_read();  // shared memory may go once the last copy has read it
  } else if (warp < 12) {
    // =============================================================== correction group
    set_max_regs_dec<Cfg::kRegsCorrection>();
    const int r = tid & 127;
    const uint32_t lane_base = static_cast<uint32_t>((warp & 3) * 32) << 16;
    uint32_t base0 = 0, base1 = 0;  // steps of tile 0 / 1 taken in earlier items: phase of o_full
    uint32_t cnt0 = 0, cnt1 = 0;    // rescale rounds of tile 0 / 1 so far: phase of corr_ready
    for (int k = 0, idx = pos(0); idx < total; idx = pos(++k)) {
      const PersItem it = decode(idx);
      const int n_max = it.n0 > it.n1 ? it.n0 : it.n1;
      for (int j = 1; j < n_max; ++j) {
#pragma unroll
        for (int i = 0; i < 2; ++i) {
          if (j < (i ? it.n1 : it.n0)) {
            const uint32_t cnt = i ? cnt1 : cnt0;
            mbar_wait(corr_ready + i, cnt & 1, abort_flag, 0x301 + i, j);
            const float alpha = alpha_buf[i * 128 + r];
            if (__any_sync(0xffffffffu, alpha != 1.f)) {
              mbar_wait(o_full + i, ((i ? base1 : base0) + j - 1) & 1, abort_flag, 0x311 + i, j);
              tc_fence_after_sync();
              const uint32_t t_o = tmem_base + (i == 0 ? Cfg::kColO0 : Cfg::kColO1) + lane_base;
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
            if (i) ++cnt1; else ++cnt0;
          }
        }
      }
      base0 += it.n0;
      base1 += it.n1;
    }
  } else {
    set_max_regs_dec<Cfg::kRegsOther>();
    if (warp == 13 && lane == 0) {
      // ============================================================= TMA producer
      uint32_t t_run = 0;             // K/V tiles loaded so far: ring slot and phase
      uint32_t q_cnt0 = 0, q_cnt1 = 0;  // items whose Q_0 / Q_1 this CTA has loaded
      for (int k = 0, idx = pos(0); idx < total; idx = pos(++k)) {
        const PersItem it = decode(idx);
        const int n_max = it.n0 > it.n1 ? it.n0 : it.n1;
        auto load_q = [&](int i) __attribute__((always_inline)) {
          if ((i ? it.n1 : it.n0) > 0) {
            const uint32_t cnt = i ? q_cnt1 : q_cnt0;
            // the previous tenant of the buffer has been read by its last S = Q.K^T
            if (cnt > 0) mbar_wait(q_free + i, (cnt - 1) & 1, abort_flag, 0x402 + i, idx);
            mbar_expect_tx(q_full + i, Cfg::kQTileBytes);
#pragma unroll
            for (int p = 0; p < Cfg::kPanels; ++p)
              tma_load_4d(q_smem + i * Cfg::kQTileBytes + p * Cfg::kQPanelBytes, &tm_q, q_full + i, p * 64,
                          it.m0 + i * Cfg::BM, it.h, it.b);
            if (i) ++q_cnt1; else ++q_cnt0;
          }
        };
        load_q(0);
        for (int t = 0; t < 2 * n_max; ++t) {
          const int slot = t_run % STAGES;
          const uint32_t ph = (t_run / STAGES) & 1;
          mbar_wait(kv_empty + slot, ph ^ 1, abort_flag, 0x401, t);
          if (*abort_flag != 0) break;
          mbar_expect_tx(kv_full + slot, Cfg::kKVTileBytes);
          const CUtensorMap* tm = (t & 1) ? &tm_v : &tm_k;
#pragma unroll
          for (int p = 0; p < Cfg::kPanels; ++p)
            tma_load_4d(kv_smem + slot * Cfg::kKVTileBytes + p * Cfg::kKVPanelBytes, tm, kv_full + slot, p * 64,
                        (t >> 1) * BN, it.h_kv, it.b);
          ++t_run;
          if (t == 0) load_q(1);
        }
        if (*abort_flag != 0) break;
      }
    } else if (warp == 12) {
      // ============================================================= MMA issue (whole warp, one elected lane issues)
      constexpr uint64_t kDescK = smem_desc_sw128(16, 1024);                  // K-major operand (Q, K)
      constexpr uint64_t kDescV = smem_desc_sw128(Cfg::kKVPanelBytes, 1024);  // MN-major operand (V)
      constexpr uint32_t kIdescQK = idesc_f16_f32(Cfg::BM, BN, false, false);
      constexpr uint32_t kIdescPV = idesc_f16_f32(Cfg::BM, D, false, true);
      const uint32_t q_addr = smem_u32(q_smem);
      const uint32_t kv_addr = smem_u32(kv_smem);
      uint32_t st0 = 0, st1 = 0;    // P.V products of tile 0 / 1 issued so far: phase of p_full
      uint32_t rs0 = 0, rs1 = 0;    // of those, the ones that followed a rescale round: phase of o_rescaled
      uint32_t qf0 = 0, qf1 = 0;    // items whose Q_0 / Q_1 has been waited for: phase of q_full
      uint32_t it0 = 0, it1 = 0;    // items of tile 0 / 1 whose first P.V has been issued: phase of o_free

      // S_i(j) = Q_i . K_j^T of item `it` (ring index t_abs); last_of_tile: no further S of this item reads Q_i
      auto issue_qk = [&](int i, const PersItem& it, int j, uint32_t t_abs) __attribute__((always_inline)) {
        const int slot = t_abs % STAGES;
        mbar_wait(kv_full + slot, (t_abs / STAGES) & 1, abort_flag, 0x501, j);
        tc_fence_after_sync();
        constexpr uint32_t kDescHi = static_cast<uint32_t>(kDescK >> 32);
        constexpr uint32_t kDescLo = static_cast<uint32_t>(kDescK);
        // descriptor start addresses are in 16-byte units and never carry out of the 14-bit field
        const uint32_t q_lo = kDescLo | (((q_addr + i * Cfg::kQTileBytes) & 0x3FFFF) >> 4);
        const uint32_t k_lo = kDescLo | (((kv_addr + slot * Cfg::kKVTileBytes) & 0x3FFFF) >> 4);
        const uint32_t t_s = tmem_base + (i == 0 ? Cfg::kColS0 : Cfg::kColS1);
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint32_t qoff = ((kk >> 2) * Cfg::kQPanelBytes + (kk & 3) * 32) >> 4;
          const uint32_t koff = ((kk >> 2) * Cfg::kKVPanelBytes + (kk & 3) * 32) >> 4;
          mma_ss_elect_lohi(t_s, q_lo + qoff, kDescHi, k_lo + koff, kDescHi, kIdescQK, kk > 0);
        }
        mma_commit_elect(s_full + i);
        if ((i == 1) || !(j < it.n1)) mma_commit_elect(kv_empty + slot);
        if (j + 1 == (i ? it.n1 : it.n0)) mma_commit_elect(q_free + i);
      };
      // O_i (+)= P_i(j) . V_j of item `it`, chunk by chunk as P arrives
      auto issue_pv = [&](int i, const PersItem& it, int j, uint32_t t_abs) __attribute__((always_inline)) {
        const int slot = t_abs % STAGES;
        mbar_wait(kv_full + slot, (t_abs / STAGES) & 1, abort_flag, 0x502, j);
        if (j > 0) {
          mbar_wait(o_rescaled + i, (i ? rs1 : rs0) & 1, abort_flag, 0x505 + i, j);
          if (i) ++rs1; else ++rs0;
        } else {
          // the first product of an item overwrites O: the previous item's epilogue must have read it
          const uint32_t k = i ? it1 : it0;
          if (k > 0) mbar_wait(o_free + i, (k - 1) & 1, abort_flag, 0x507 + i, j);
          if (i) ++it1; else ++it0;
        }
        constexpr uint32_t kDescVHi = static_cast<uint32_t>(kDescV >> 32);
        const uint32_t v_lo = static_cast<uint32_t>(kDescV) | (((kv_addr + slot * Cfg::kKVTileBytes) & 0x3FFFF) >> 4);
        const uint32_t t_p = tmem_base + (i == 0 ? Cfg::kColS0 : Cfg::kColS1);
        const uint32_t t_o = tmem_base + (i == 0 ? Cfg::kColO0 : Cfg::kColO1);
        const uint32_t ph = (i ? st1 : st0) & 1;
#pragma unroll
        for (int q = 0; q < Cfg::kPChunks; ++q) {
          FRAY_CRIT_WAIT(p_full + i * Cfg::kPChunks + q, ph, abort_flag, 0x503 + i, j);
          tc_fence_after_sync();
#pragma unroll
          for (int s2 = 0; s2 < 8 / Cfg::kPChunks; ++s2) {
            const int kk = (8 / Cfg::kPChunks) * q + s2;  // MMA (16 keys) inside the step
            mma_ts_elect_lohi(t_o, t_p + kk * 8, v_lo + ((kk * 2048) >> 4), kDescVHi, kIdescPV, (j > 0 || kk > 0));
          }
        }
        if (i) ++st1; else ++st0;
        mma_commit_elect(o_full + i);
        if ((i == 1) || !(j < it.n1)) mma_commit_elect(kv_empty + slot);
      };
      // first scores of tile i of item `it`: its Q tile must have landed
      auto first_qk = [&](int i, const PersItem& it, uint32_t t_abs) __attribute__((always_inline)) {
        mbar_wait(q_full + i, (i ? qf1 : qf0) & 1, abort_flag, 0x511 + i);
        if (i) ++qf1; else ++qf0;
        issue_qk(i, it, 0, t_abs);
      };

      int k = 0;
      const int idx = pos(0);
      if (idx < total) {
        PersItem cur = decode(idx);
        uint32_t t_base = 0;  // ring index of the current item's K_0
#pragma unroll 1
        for (int i = 0; i < 2; ++i)
          if ((i ? cur.n1 : cur.n0) > 0) first_qk(i, cur, t_base);
        while (true) {
          const int idx_next = pos(k + 1);
          const bool has_next = idx_next < total;
          PersItem nxt = cur;
          nxt.n0 = 0;
          nxt.n1 = 0;
          if (has_next) nxt = decode(idx_next);
          const int n_max = cur.n0 > cur.n1 ? cur.n0 : cur.n1;
          const uint32_t t_next = t_base + 2 * n_max;
          for (int j = 0; j < n_max; ++j) {
#pragma unroll 1
            for (int i = 0; i < 2; ++i) {
              const int n_i = i ? cur.n1 : cur.n0;
              if (j < n_i) {
                issue_pv(i, cur, j, t_base + 2 * j + 1);
                if (j + 1 < n_i) {
                  issue_qk(i, cur, j + 1, t_base + 2 * (j + 1));
                } else if ((i ? nxt.n1 : nxt.n0) > 0 && (i == 1 || cur.n0 == cur.n1)) {
                  first_qk(i, nxt, t_next);  // the next item's first scores, right behind this item's last P.V
                }
              }
            }
            // Tile 0 of a causal item ends one step before tile 1.  Its next first scores need the next item's
            // K_0, whose ring slot the other tile's P.V of THIS step hands back: they go behind that product.
            if (cur.n0 != cur.n1 && j + 1 == cur.n0 && nxt.n0 > 0) first_qk(0, nxt, t_next);
          }
          // a tile that had nothing to do in this item (past the last query) but has in the next
#pragma unroll 1
          for (int i = 0; i < 2; ++i)
            if ((i ? cur.n1 : cur.n0) == 0 && (i ? nxt.n1 : nxt.n0) > 0) first_qk(i, nxt, t_next);
          if (!has_next) break;
          cur = nxt;
          t_base = t_next;
          ++k;
        }
      }
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem_base, Cfg::kTmemCols);
}

// Host launcher for the persistent kernel. Returns an AttnReturnCode.
template <int D, int BN, int STAGES>
inline int launch_attn_fwd_pers(const operand_t* q, const operand_t* k, const operand_t* v, operand_t* o, const AttnShape& shp,
                                const AttnStrides (&st)[4], const AttnExtras& ex, bool causal, float scale,
                                cudaStream_t stream) {
  using Cfg = PersCfg<D, BN, STAGES>;
  const AttnShape shp_kv{shp.B, shp.H / ex.kv_group, ex.seq_k, shp.D};
  CUtensorMap tm_q, tm_k, tm_v, tm_o;
  int rc = cached_attn_tensor_map(&tm_q, q, shp, st[0], Cfg::BM);
  if (rc != kAttnOk) return rc;
  rc = cached_attn_tensor_map(&tm_k, k, shp_kv, st[1], BN);
  if (rc != kAttnOk) return rc;
  rc = cached_attn_tensor_map(&tm_v, v, shp_kv, st[2], BN);
  if (rc != kAttnOk) return rc;
  rc = cached_attn_tensor_map(&tm_o, o, shp, st[3], Cfg::BM);
  if (rc != kAttnOk) return rc;

  auto kernel = attn_fwd_pers_kernel<D, BN, STAGES>;
  rc = ensure_dynamic_smem<Cfg>(kernel, Cfg::kSmemBytes, Cfg::kThreads,
                                256 * Cfg::kRegsSoftmax + 128 * Cfg::kRegsCorrection + 128 * Cfg::kRegsOther);
  if (rc != kAttnOk) return rc;
  const int sms = device_sm_count();
  if (sms <= 0) return kAttnLaunchFailed;
  const long long items = static_cast<long long>((shp.S + 2 * Cfg::BM - 1) / (2 * Cfg::BM)) * shp.B * shp.H;
  const int grid = static_cast<int>(items < sms ? items : sms);
  // item order (see the kernel): heaviest first over all slices or slice by slice
  const int blk = heaviest_first_order(causal, shp, shp_kv) ? shp.B * shp.H : 1;
  kernel<<<grid, Cfg::kThreads, Cfg::kSmemBytes, stream>>>(tm_q, tm_k, tm_v, tm_o, shp.H, shp.B * shp.H, shp.S, causal ? 1 : 0,
                                                           scale * 1.44269504088896340736f, ex.kv_group, ex.lse, ex.seq_k, blk);
  if (cudaGetLastError() != cudaSuccess) return kAttnLaunchFailed;
  return kAttnOk;
}

}  // namespace sm100
}  // namespace fray
