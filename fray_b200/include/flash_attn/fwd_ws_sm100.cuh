#pragma once
// Warp-specialised attention forward for sm_100a.
//
// One CTA of 16 warps owns two 128-row query tiles of one (batch, head) slice:
//   warps 0-3   softmax group 0 (query tile 0; thread r owns row r)
//   warps 4-7   softmax group 1 (query tile 1)
//   warps 8-11  correction group: rescales the O accumulators when a running max moved
//               (the softmax groups write their own tiles out: O/l -> 16 bit -> shared memory -> TMA store)
//   warp 12     MMA issue for both tiles (warp-uniform code, one elected lane issues)
//   warp 13     TMA producer (Q tiles once, then K_j, V_j through a ring of STAGES buffers)
//   warps 14-15 idle (they only exist so that warps 12-15 form a full warpgroup for setmaxnreg)
//
// Tensor memory (512 columns): S0 [0,128) S1 [128,256) O0 [256,384) O1 [384,512).  P (fp16)
// overwrites the first 64 columns of its S buffer and is consumed from there as the A
// operand of the P.V product; the tensor pipe executes MMAs in issue order, so the next
// S = Q.K^T of that tile may be issued right behind it.
//
// Issue order in the MMA warp: S0(0) S1(0) | PV0(0) S0(1) PV1(0) S1(1) | PV0(1) S0(2) ...
// so that while group 0 runs the softmax of S0(j+1) the tensor cores work on PV1(j) and
// S1(j+1), and vice versa.  (One issuing warp per tile and turn-taking of the softmax groups on
// the special-function unit were both measured slower than this fixed alternation.)  P.V is
// issued in two key chunks as the softmax hands them over, so only the second half of it sits
// behind the softmax.
//
// Online softmax in base 2 with lazy rescaling: a tile's exponent offset m_ref only moves
// when the running max grew by more than 2^8 in the scaled domain; until then P may exceed
// 1 (at most 256, exact in fp16 range) and O needs no correction.  O and l always share the
// same m_ref, so the final O/l is the exact softmax up to rounding.
//
// Every barrier wait is bounded (see sm100_ptx.cuh): a protocol error ends as a status
// word and a wrong answer, never as a hung GPU.

#include "host_sm100.cuh"
#include "sm100_ptx.cuh"
#include "softmax_tile_sm100.cuh"

// The MMA warp keeps one copy of each issue sequence with the tile index as a run-time value: the kernel is
// sensitive to instruction fetch (71 KB instead of 88 KB of code measured +8 % on the short CTAs of causal
// shapes and nothing on the headline shape).

namespace fray {
namespace sm100 {

template <int D, int BN, int STAGES>
struct WsCfg {
  static_assert(D == 64 || D == 128, "head dim must be 64 or 128");
  static_assert(BN == 128, "the warp-specialised kernel uses 128-key tiles");
  static_assert(STAGES >= 2 && STAGES <= 8, "2..8 K/V buffers");
  static constexpr int BM = 128;               // rows per query tile
  // P is handed to the MMA warp in this many column chunks.  Two chunks of 64 keys measured 2 % faster than
  // four of 32: each hand-over costs the softmax thread a wait for its tensor-memory store and the MMA warp a
  // barrier round trip, and only the last chunk's product sits between the softmax and the next scores.
  static constexpr int kPChunks = 2;
  static constexpr int kSoftmaxWarps = 8;
  static constexpr int kThreads = 512;
  static constexpr int kPanels = D / 64;       // 64-element (128-byte) column panels
  static constexpr int kQPanelBytes = BM * 128;
  static constexpr int kQTileBytes = kPanels * kQPanelBytes;
  static constexpr int kKVPanelBytes = BN * 128;
  static constexpr int kKVTileBytes = kPanels * kKVPanelBytes;
  static constexpr int kOffQ = 0;
  static constexpr int kOffKV = 2 * kQTileBytes;
  static constexpr int kOffBars = kOffKV + STAGES * kKVTileBytes;
  static constexpr int kNumBars = 2 + 2 * STAGES + 2 * 4 + 2 * kPChunks;
  static constexpr int kOffStats = kOffBars + ((kNumBars * 8 + 16 + 127) / 128) * 128;  // alpha[2][128]
#ifdef FRAY_ATTN_TRACE
  static constexpr int kOffTrace = kOffStats + 2 * 128 * 4;
  static constexpr int kSmemBytes = kOffTrace + 4 * 960 + 1024;
#else
  static constexpr int kSmemBytes = kOffStats + 2 * 128 * 4 + 1024;  // + alignment slack
#endif
  static_assert(kSmemBytes <= 232448, "exceeds the 227 KB shared memory of one CTA");
  static constexpr int kTmemCols = 512;
  static constexpr uint32_t kColS0 = 0, kColS1 = 128, kColO0 = 256, kColO1 = 384;
  // register budgets after setmaxnreg (softmax, correction, MMA/producer warps; the sum over the 16 warps
  // is the CTA's allocation of 512 x 128 registers: an increase the decreases cannot cover never returns)
  static constexpr int kRegsSoftmax = 184, kRegsCorrection = 80, kRegsOther = 64;
  static_assert(256 * kRegsSoftmax + 128 * kRegsCorrection + 128 * kRegsOther <= 512 * 128, "register budgets exceed the CTA's allocation");
};


template <int D, int BN, int STAGES>
__global__ void __launch_bounds__(512, 1)
attn_fwd_ws_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                   const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_o,
                   int num_heads, int seq_len, int causal, float scale_log2, int kv_group, float* lse, int seq_k,
                   int group_slices, int num_bh) {
  using Cfg = WsCfg<D, BN, STAGES>;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  uint8_t* smem = smem_raw + (((raw_addr + 1023u) & ~1023u) - raw_addr);
  uint8_t* q_smem = smem + Cfg::kOffQ;    // tile i at q_smem + i * kQTileBytes (reused for the O tile at the end)
  uint8_t* kv_smem = smem + Cfg::kOffKV;  // ring slot s at kv_smem + s * kKVTileBytes
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Cfg::kOffBars);
  uint64_t* q_full = bars;                      // [2]   producer -> MMA
  uint64_t* kv_full = bars + 2;                 // [STAGES] producer -> MMA
  uint64_t* kv_empty = kv_full + STAGES;        // [STAGES] MMA -> producer
  uint64_t* s_full = kv_empty + STAGES;         // [2]   MMA -> softmax i        (S_i(j) complete)
  uint64_t* o_full = s_full + 2;                // [2]   MMA -> correction       (PV_i(j) complete)
  uint64_t* corr_ready = o_full + 2;            // [2]   softmax i -> correction (alpha_i(j) published)
  uint64_t* o_rescaled = corr_ready + 2;        // [2]   correction -> MMA       (O_i ready for PV_i(j))
  uint64_t* p_full = o_rescaled + 2;            // [2][kPChunks] softmax i -> MMA (chunk c of P_i(j) stored)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + Cfg::kNumBars);
  volatile uint32_t* abort_flag = reinterpret_cast<volatile uint32_t*>(tmem_slot + 1);
  float* alpha_buf = reinterpret_cast<float*>(smem + Cfg::kOffStats);  // [2][128]

#ifdef FRAY_ATTN_TRACE
  unsigned int* trace_sm = reinterpret_cast<unsigned int*>(smem + Cfg::kOffTrace);
  const bool trace_on = blockIdx.x == 0 && blockIdx.y == 0;
#endif
  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;
  // Grid order.  group_slices == 0: (tiles, slices), which runs slice by slice, so that CTAs side by side share
  // a slice's K and V in L2.  group_slices > 0: (slice inside its group, tiles, groups): the longest causal
  // tiles of all slices of a group start first, which lets first-come scheduling even out the tiles' unequal
  // lengths, while a group's K and V stay small enough to share L2 (the launcher decides, see
  // heaviest_first_group).
  const int n_x = group_slices > 0 ? gridDim.y : gridDim.x;
  const int px = group_slices > 0 ? blockIdx.y : blockIdx.x;
  const int pair = causal ? (n_x - 1 - px) : px;  // heaviest causal tiles first
  const int bh = group_slices > 0 ? static_cast<int>(blockIdx.z) * group_slices + static_cast<int>(blockIdx.x)
                                  : static_cast<int>(blockIdx.y);
  if (bh >= num_bh) return;  // padding of the last group
  const int m0 = pair * (2 * Cfg::BM);
  const int b = bh / num_heads;
  const int h = bh - b * num_heads;
  const int h_kv = h / kv_group;  // K/V head of this query head (one division per CTA, not per copy)

  // Number of KV tiles each query tile consumes (0 = tile lies past the end of the sequence).
  const int n_kv = (seq_k + BN - 1) / BN;  // seq_len counts queries, seq_k keys
  auto tiles_for = [&](int i) {
    const int row0 = m0 + i * Cfg::BM;
    int n = row0 < seq_len ? n_kv : 0;
    if (causal && n > 0) {
      const int lim = (row0 + Cfg::BM + BN - 1) / BN;
      n = lim < n ? lim : n;
    }
    return n;
  };
  const int n_t0 = tiles_for(0), n_t1 = tiles_for(1);  // scalars: an indexed array would live in local memory
  const int n_max = n_t0 > n_t1 ? n_t0 : n_t1;

  if (tid == 0) {
    FRAY_TRACE(6, 0, 0);  // CTA entry
    FRAY_TRACE_NS(6, 0, 10);
    *abort_flag = (*reinterpret_cast<volatile int*>(&fray_attn_status[0]) != 0) ? 2u : 0u;
    for (int i = 0; i < 2; ++i) {
      mbar_init(q_full + i, 1);
      mbar_init(s_full + i, 1);
      for (int c = 0; c < Cfg::kPChunks; ++c) mbar_init(p_full + i * Cfg::kPChunks + c, 4);  // one arrival per warp
      mbar_init(o_full + i, 1);
      mbar_init(corr_ready + i, 4);  // one arrival per warp: 32 lanes arriving on one barrier would serialise
      mbar_init(o_rescaled + i, 4);
    }
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(kv_full + s, 1);
      mbar_init(kv_empty + s, 1);
    }
    fence_barrier_init();
    prefetch_tensormap(&tm_o);
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
  if (tid == 0) FRAY_TRACE(6, 0, 1);  // set-up done

  // (rotating the role assignment over the warp index was measured to make no difference)
  if (warp < 8) {
    // =============================================================== softmax groups
    set_max_regs_inc<Cfg::kRegsSoftmax>();
    const int i = warp >> 2;  // query tile of this group
    const int r = tid & 127;  // row inside the tile
    const int n_i = i ? n_t1 : n_t0;
    const int row = m0 + i * Cfg::BM + r;
    const uint32_t lane_base = static_cast<uint32_t>((warp & 3) * 32) << 16;
    const uint32_t t_s = tmem_base + (i == 0 ? Cfg::kColS0 : Cfg::kColS1) + lane_base;
    uint64_t* p_bar = p_full + i * Cfg::kPChunks;
    float m_ref = -INFINITY;  // exponent offset currently baked into P, l and O
    float l_run = 0.f;
    for (int j = 0; j < n_i; ++j) {
      FRAY_CRIT_WAIT(s_full + i, j & 1, abort_flag, 0x201 + i, j);
      tc_fence_after_sync();
      if (r == FRAY_TRACE_ROW) FRAY_TRACE(0, i, j);
      const int kv0 = j * BN;
      const bool need_mask = (kv0 + BN > seq_k) || (causal && (kv0 + BN - 1 > m0 + i * Cfg::BM));
#ifdef FRAY_ATTN_TRACE
      unsigned int* tr = (trace_on && r == FRAY_TRACE_ROW && j < kTraceIters) ? trace_sm + i * kTraceIters + j : nullptr;
#else
      unsigned int* tr = nullptr;
#endif
      if (need_mask) {
        softmax_tile<BN, Cfg::kPChunks, true, D == 64>(t_s, p_bar, corr_ready + i, alpha_buf + i * 128 + r, j == 0, kv0, row, seq_k,
                                              causal, scale_log2, lane, m_ref, l_run, tr);
      } else {
        softmax_tile<BN, Cfg::kPChunks, false, D == 64>(t_s, p_bar, corr_ready + i, alpha_buf + i * 128 + r, j == 0, kv0, row, seq_k,
                                               causal, scale_log2, lane, m_ref, l_run, tr);
      }
      if (r == FRAY_TRACE_ROW) FRAY_TRACE(4, i, j);
    }
    if (n_i > 0) {
      // The group writes its own tile out: it has the row sums and offsets in registers, its threads
      // sit on the rows' tensor-memory lanes, and the two tiles' epilogues then run side by side
      // instead of one after the other in the correction group.
      mbar_wait(o_full + i, (n_i - 1) & 1, abort_flag, 0x331 + i, n_i);
      tc_fence_after_sync();
      if (r == 0) FRAY_TRACE(6, 1, i);  // last P.V of tile i complete, epilogue starts
      epilogue_tile<Cfg, D>(tmem_base + (i == 0 ? Cfg::kColO0 : Cfg::kColO1) + lane_base, q_smem + i * Cfg::kQTileBytes,
                            r, l_run, m_ref, &tm_o, m0 + i * Cfg::BM, h, b, num_heads, seq_len, scale_log2, lse, 4 + i);
      if (r == 0) {
        tma_store_wait_read();  // shared memory may go once the copy has read it; the writes finish on their own
        FRAY_TRACE(6, 1, 2 + i);
      }
    }
  } else if (warp < 12) {
    // =============================================================== correction group
    set_max_regs_dec<Cfg::kRegsCorrection>();
    const int r = tid & 127;
    const uint32_t lane_base = static_cast<uint32_t>((warp & 3) * 32) << 16;
    for (int j = 1; j < n_max; ++j) {
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        if (j < (i ? n_t1 : n_t0)) {
          const uint32_t ph = (j - 1) & 1;
          mbar_wait(corr_ready + i, ph, abort_flag, 0x301 + i, j);
          const float alpha = alpha_buf[i * 128 + r];
          if (__any_sync(0xffffffffu, alpha != 1.f)) {
            mbar_wait(o_full + i, ph, abort_flag, 0x311 + i, j);
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
        }
      }
    }
  } else {
    set_max_regs_dec<Cfg::kRegsOther>();
    if (warp == 13 && lane == 0) {
      // ============================================================= TMA producer
      // (Issuing the first copies during set-up, before tensor memory is allocated, measured -1 % on the
      // headline shape and +1.5 % on 1024-key sequences: not kept.)
      auto load_q = [&](int i) __attribute__((always_inline)) {
        if ((i ? n_t1 : n_t0) > 0) {
          mbar_expect_tx(q_full + i, Cfg::kQTileBytes);
#pragma unroll
          for (int p = 0; p < Cfg::kPanels; ++p)
            tma_load_4d(q_smem + i * Cfg::kQTileBytes + p * Cfg::kQPanelBytes, &tm_q, q_full + i, p * 64,
                        m0 + i * Cfg::BM, h, b);
        }
      };
      load_q(0);
      for (int t = 0; t < 2 * n_max; ++t) {
        const int slot = t % STAGES;
        const uint32_t ph = (t / STAGES) & 1;
        mbar_wait(kv_empty + slot, ph ^ 1, abort_flag, 0x401, t);
        if (*abort_flag != 0) break;
        mbar_expect_tx(kv_full + slot, Cfg::kKVTileBytes);
        const CUtensorMap* tm = (t & 1) ? &tm_v : &tm_k;
#pragma unroll
        for (int p = 0; p < Cfg::kPanels; ++p)
          tma_load_4d(kv_smem + slot * Cfg::kKVTileBytes + p * Cfg::kKVPanelBytes, tm, kv_full + slot, p * 64,
                      (t >> 1) * BN, h_kv, b);
        if (t == 0) load_q(1);
      }
    } else if (warp == 12) {
      // ============================================================= MMA issue (whole warp, one elected lane issues)
      // One warp serves both tiles in a fixed alternation.  That ordering is what keeps the two
      // tiles in anti-phase (one in its softmax while the other owns the tensor pipe); two
      // independent issuing warps were measured to drift into lock-step and lose the overlap.
      constexpr uint64_t kDescK = smem_desc_sw128(16, 1024);                  // K-major operand (Q, K)
      constexpr uint64_t kDescV = smem_desc_sw128(Cfg::kKVPanelBytes, 1024);  // MN-major operand (V)
      constexpr uint32_t kIdescQK = idesc_f16_f32(Cfg::BM, BN, false, false);
      constexpr uint32_t kIdescPV = idesc_f16_f32(Cfg::BM, D, false, true);
      const uint32_t q_addr = smem_u32(q_smem);
      const uint32_t kv_addr = smem_u32(kv_smem);
      const int n0 = n_t0, n1 = n_t1;

      auto issue_qk = [&](int i, int j) __attribute__((always_inline)) {  // S_i(j) = Q_i . K_j^T
        const int t = 2 * j;
        const int slot = t % STAGES;
        mbar_wait(kv_full + slot, (t / STAGES) & 1, abort_flag, 0x501, t);
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
        if ((i == 1) || !(j < n1)) mma_commit_elect(kv_empty + slot);
        FRAY_TRACE(8, i, j);
      };
      // O_i (+)= P_i(j) . V_j, chunk by chunk as P arrives.  (Waiting for the next K tile's barrier here,
      // ahead of the last chunk, to take that round trip off the path to the next S made no difference.)
      auto issue_pv = [&](int i, int j) __attribute__((always_inline)) {
        const int t = 2 * j + 1;
        const int slot = t % STAGES;
        mbar_wait(kv_full + slot, (t / STAGES) & 1, abort_flag, 0x502, t);
        if (j > 0) mbar_wait(o_rescaled + i, (j - 1) & 1, abort_flag, 0x505 + i, j);
        constexpr uint32_t kDescVHi = static_cast<uint32_t>(kDescV >> 32);
        const uint32_t v_lo = static_cast<uint32_t>(kDescV) | (((kv_addr + slot * Cfg::kKVTileBytes) & 0x3FFFF) >> 4);
        const uint32_t t_p = tmem_base + (i == 0 ? Cfg::kColS0 : Cfg::kColS1);
        const uint32_t t_o = tmem_base + (i == 0 ? Cfg::kColO0 : Cfg::kColO1);
#pragma unroll
        for (int q = 0; q < Cfg::kPChunks; ++q) {
          FRAY_CRIT_WAIT(p_full + i * Cfg::kPChunks + q, j & 1, abort_flag, 0x503 + i, j);
          tc_fence_after_sync();
          if (q == 0) FRAY_TRACE(5, i, j);
#pragma unroll
          for (int s2 = 0; s2 < 8 / Cfg::kPChunks; ++s2) {
            const int kk = (8 / Cfg::kPChunks) * q + s2;  // MMA (16 keys) inside the step
            mma_ts_elect_lohi(t_o, t_p + kk * 8, v_lo + ((kk * 2048) >> 4), kDescVHi, kIdescPV, (j > 0 || kk > 0));
          }
        }
        mma_commit_elect(o_full + i);
        if ((i == 1) || !(j < n1)) mma_commit_elect(kv_empty + slot);
        FRAY_TRACE(7, i, j);
      };

      // One copy of each issue sequence, the tile index a run-time value.
#pragma unroll 1
      for (int i = 0; i < 2; ++i) {
        if ((i ? n1 : n0) > 0) {
          mbar_wait(q_full + i, 0, abort_flag, 0x511 + i);
          issue_qk(i, 0);
        }
      }
      for (int j = 0; j < n_max; ++j) {
#pragma unroll 1
        for (int i = 0; i < 2; ++i) {
          const int n_i = i ? n1 : n0;
          if (j < n_i) {
            issue_pv(i, j);
            if (j + 1 < n_i) issue_qk(i, j + 1);
          }
        }
      }
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem_base, Cfg::kTmemCols);
#ifdef FRAY_ATTN_TRACE
  if (tid == 0) {
    FRAY_TRACE(6, 0, 2);  // CTA exit
    FRAY_TRACE_NS(6, 0, 11);
  }
  __syncthreads();
  if (trace_on)
    for (int w = tid; w < kTraceWords; w += Cfg::kThreads) fray_attn_trace_buf[w] = trace_sm[w];
#endif
}

// Host launcher for the warp-specialised kernel. Returns an AttnReturnCode.
template <int D, int BN, int STAGES>
inline int launch_attn_fwd_ws(const operand_t* q, const operand_t* k, const operand_t* v, operand_t* o, const AttnShape& shp,
                              const AttnStrides (&st)[4], const AttnExtras& ex, bool causal, float scale,
                              cudaStream_t stream) {
  using Cfg = WsCfg<D, BN, STAGES>;
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

  auto kernel = attn_fwd_ws_kernel<D, BN, STAGES>;
  rc = ensure_dynamic_smem<Cfg>(kernel, Cfg::kSmemBytes, Cfg::kThreads, 256 * Cfg::kRegsSoftmax + 128 * Cfg::kRegsCorrection + 128 * Cfg::kRegsOther);
  if (rc != kAttnOk) return rc;
  const int group_slices = heaviest_first_group(causal, shp, shp_kv);
  const unsigned n_x = (shp.S + 2 * Cfg::BM - 1) / (2 * Cfg::BM), n_bh = shp.B * shp.H;
  dim3 grid = group_slices > 0 ? dim3(group_slices, n_x, (n_bh + group_slices - 1) / group_slices) : dim3(n_x, n_bh);
  kernel<<<grid, Cfg::kThreads, Cfg::kSmemBytes, stream>>>(tm_q, tm_k, tm_v, tm_o, shp.H, shp.S, causal ? 1 : 0,
                                                           scale * 1.44269504088896340736f, ex.kv_group, ex.lse, ex.seq_k,
                                                           group_slices, static_cast<int>(n_bh));
  if (cudaGetLastError() != cudaSuccess) return kAttnLaunchFailed;
  return kAttnOk;
}

}  // namespace sm100
}  // namespace fray
