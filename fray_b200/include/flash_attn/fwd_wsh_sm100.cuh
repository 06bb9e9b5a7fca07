#pragma once
// Warp-specialised attention forward for sm_100a that pipelines HALF key tiles.
//
// Same roles, buffers and tensor-memory budget as the kernel in fwd_ws_sm100.cuh (two 128-row query
// tiles per CTA, S and O of both tiles fill the 512 columns), but a softmax step covers 64 keys and
// the 128 score columns of a tile are two buffers of 64.  In the whole-tile kernel P(j) overwrites
// S(j), so S(j+1) of a tile cannot be issued before P(j).V has read it, and a tile's chain
// S -> softmax -> P.V -> S is strictly serial; the tensor pipe and the softmax group of a tile each
// sit idle while the other works, and the two tiles only half hide that.  Here half step h uses
// buffer h & 1: S(h+2) follows P(h).V into the same buffer while the softmax works on S(h+1) in the
// other one, so the softmax group never waits for its own tile's MMAs.
//
// The price: S = Q.K^T with N = 64 reads as much of Q from shared memory per MMA as with N = 128 and
// runs at 48 instead of 32 cycles per 16 x 64 keys (shared-memory bound), so the tensor pipe needs
// 1280 instead of 1024 cycles per 128 keys of a tile; and the per-step costs of the softmax
// (barrier waits, offset decision, hand-over) are paid twice as often.
//
// A softmax group can now run up to two half steps ahead of the correction group and of the MMA
// warp's consumption of the "O rescaled" signal, so every hand-over that repeats per half step uses
// two mbarriers (and two value slots) alternating with the step parity: a single barrier could
// complete two phases before its consumer looked, and a parity wait cannot tell phase n from n+2.
//
// What double buffering does not buy: S(h+1) is issued behind P(h-1).V and so arrives most of a step
// after P(h-1) was handed over, i.e. late in softmax step h.  Taking the row max of S(h+1) inside
// step h, under the exponentials, was tried and stalled on exactly that; it would need a third buffer.
//
// Issue order in the MMA warp: S0(0) S1(0) S0(1) S1(1) | PV0(h) S0(h+2) PV1(h) S1(h+2) | ...
// K and V still arrive as 128-key tiles; half step h uses rows 64*(h&1).. of tile h >> 1.

#include "host_sm100.cuh"
#include "sm100_ptx.cuh"
#include "softmax_tile_sm100.cuh"
#include "fwd_ws_sm100.cuh"  // trace macros, WsCfg for the shared-memory layout

namespace fray {
namespace sm100 {

// Whether the two softmax groups take turns on the exponentials (-DFRAY_HALFSTEP_TURNS=0/1).
// Measured 2.5-3.5 % slower than letting them run freely, so off.
#ifndef FRAY_HALFSTEP_TURNS
#define FRAY_HALFSTEP_TURNS 0
#endif
static constexpr bool kHalfStepTurns = FRAY_HALFSTEP_TURNS != 0;

#ifndef FRAY_WSH_REGS_S
#define FRAY_WSH_REGS_S 184
#endif
#ifndef FRAY_WSH_REGS_C
#define FRAY_WSH_REGS_C 80
#endif
#ifndef FRAY_WSH_REGS_O
#define FRAY_WSH_REGS_O 64
#endif

template <int D, int STAGES>
struct WshCfg {
  static_assert(D == 64 || D == 128, "head dim must be 64 or 128");
  static_assert(STAGES >= 2 && STAGES <= 8, "2..8 K/V buffers");
  static constexpr int BM = 128;   // rows per query tile
  static constexpr int BN = 128;   // keys per K/V tile in shared memory
  static constexpr int BH = 64;    // keys per softmax step
  static constexpr int kThreads = 512;
  static constexpr int kPanels = D / 64;
  static constexpr int kQPanelBytes = BM * 128;
  static constexpr int kQTileBytes = kPanels * kQPanelBytes;
  static constexpr int kKVPanelBytes = BN * 128;
  static constexpr int kKVTileBytes = kPanels * kKVPanelBytes;
  static constexpr int kOffQ = 0;
  static constexpr int kOffKV = 2 * kQTileBytes;
  static constexpr int kOffBars = kOffKV + STAGES * kKVTileBytes;
  // q_full[2] kv_full[S] kv_empty[S] s_full[2][2] p_full[2][2] o_full[2] corr_ready[2][2] l_ready[2] o_rescaled[2][2] o_final[2]
  static constexpr int kNumBars = 2 + 2 * STAGES + 4 + 4 + 2 + 4 + 2 + 4 + 2 + 2;  // + exp_turn[2]
  static constexpr int kOffStats = kOffBars + ((kNumBars * 8 + 16 + 127) / 128) * 128;  // alpha[2][2][128], l[2][128], m[2][128]
#ifdef FRAY_ATTN_TRACE
  static constexpr int kOffTrace = kOffStats + 8 * 128 * 4;
  static constexpr int kSmemBytes = kOffTrace + 4 * 800 + 1024;
#else
  static constexpr int kSmemBytes = kOffStats + 8 * 128 * 4 + 1024;  // + alignment slack
#endif
  static_assert(kSmemBytes <= 232448, "exceeds the 227 KB shared memory of one CTA");
  static constexpr int kTmemCols = 512;
  static constexpr uint32_t kColS0 = 0, kColS1 = 128, kColO0 = 256, kColO1 = 384;
  // register budgets after setmaxnreg: 256*S + 128*C + 128*O = 512*128, the CTA's allocation at launch
  static constexpr int kRegsSoftmax = FRAY_WSH_REGS_S, kRegsCorrection = FRAY_WSH_REGS_C, kRegsOther = FRAY_WSH_REGS_O;
  static_assert(256 * kRegsSoftmax + 128 * kRegsCorrection + 128 * kRegsOther <= 65536, "register budgets exceed the CTA's allocation");
};

template <int D, int STAGES>
__global__ void __launch_bounds__(512, 1)
attn_fwd_wsh_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                    const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_o,
                    int num_heads, int seq_len, int causal, float scale_log2, int kv_group, float* lse, int seq_k) {
  using Cfg = WshCfg<D, STAGES>;
  constexpr int BN = Cfg::BN, BH = Cfg::BH;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  uint8_t* smem = smem_raw + (((raw_addr + 1023u) & ~1023u) - raw_addr);
  uint8_t* q_smem = smem + Cfg::kOffQ;
  uint8_t* kv_smem = smem + Cfg::kOffKV;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Cfg::kOffBars);
  uint64_t* q_full = bars;                  // [2]        producer -> MMA
  uint64_t* kv_full = bars + 2;             // [STAGES]   producer -> MMA
  uint64_t* kv_empty = kv_full + STAGES;    // [STAGES]   MMA -> producer
  uint64_t* s_full = kv_empty + STAGES;     // [2][2]     MMA -> softmax i   (S_i(h) complete in buffer h&1)
  uint64_t* p_full = s_full + 4;            // [2][2]     softmax i -> MMA   (P_i(h) stored in buffer h&1)
  uint64_t* o_full = p_full + 4;            // [2]        MMA -> correction  (PV_i(h) complete)
  uint64_t* corr_ready = o_full + 2;        // [2][2]     softmax i -> correction (alpha_i(h) published, barrier h&1)
  uint64_t* l_ready = corr_ready + 4;       // [2]        softmax i -> correction (final row sums published)
  uint64_t* o_rescaled = l_ready + 2;       // [2][2]     correction -> MMA  (O_i ready for PV_i(h), barrier h&1)
  // [2] MMA -> epilogue (last PV_i complete).  Not o_full: the softmax group finishes its last step
  // when PV_i of two steps earlier is complete, so o_full may be two phases short of the last one
  // when the epilogue looks, which a parity wait cannot tell from the last one itself.
  uint64_t* o_final = o_rescaled + 4;
  uint64_t* exp_turn = o_final + 2;         // [2]        softmax (1-i) -> softmax i: the exponentials are yours
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + Cfg::kNumBars);
  volatile uint32_t* abort_flag = reinterpret_cast<volatile uint32_t*>(tmem_slot + 1);
  float* alpha_buf = reinterpret_cast<float*>(smem + Cfg::kOffStats);  // [2 tiles][2 parities][128]
  float* l_buf = alpha_buf + 512;                                      // [2][128]
  float* m_buf = l_buf + 256;                                          // [2][128] final exponent offsets (for the LSE output)

#ifdef FRAY_ATTN_TRACE
  unsigned int* trace_sm = reinterpret_cast<unsigned int*>(smem + Cfg::kOffTrace);
  const bool trace_on = blockIdx.x == 0 && blockIdx.y == 0;
#endif
  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;
  const int pair = causal ? (gridDim.x - 1 - blockIdx.x) : blockIdx.x;  // heaviest causal tiles first
  const int m0 = pair * (2 * Cfg::BM);
  const int bh = blockIdx.y;
  const int b = bh / num_heads;
  const int h_idx = bh - b * num_heads;
  const int h_kv = h_idx / kv_group;  // K/V head of this query head (one division per CTA, not per copy)

  // Number of 128-key K/V tiles each query tile consumes (0 = tile lies past the end of the sequence).
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
  const int n_t0 = tiles_for(0), n_t1 = tiles_for(1);
  const int n_max = n_t0 > n_t1 ? n_t0 : n_t1;
  const int h_t0 = 2 * n_t0, h_t1 = 2 * n_t1, h_max = 2 * n_max;  // half steps

  if (tid == 0) {
    FRAY_TRACE(6, 0, 0);
    *abort_flag = (*reinterpret_cast<volatile int*>(&fray_attn_status[0]) != 0) ? 2u : 0u;
    for (int i = 0; i < 2; ++i) {
      mbar_init(q_full + i, 1);
      mbar_init(o_full + i, 1);
      mbar_init(l_ready + i, 4);  // one arrival per warp
      mbar_init(o_final + i, 1);
      mbar_init(exp_turn + i, 4);
    }
    for (int x = 0; x < 4; ++x) {
      mbar_init(corr_ready + x, 4);
      mbar_init(o_rescaled + x, 4);
    }
    for (int x = 0; x < 4; ++x) mbar_init(s_full + x, 1);
    for (int x = 0; x < 4; ++x) mbar_init(p_full + x, 4);
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(kv_full + s, 1);
      mbar_init(kv_empty + s, 1);
    }
    fence_barrier_init();
    // The first copies (Q of both tiles, K_0, V_0) go out right here, before tensor memory is
    // allocated and the roles separate, so that their latency overlaps the rest of the set-up.  The
    // producer warp continues with the third ring entry.
    if (kEarlyCopies && *abort_flag == 0 && n_max > 0) {
      auto early_q = [&](int i) {
        if ((i ? n_t1 : n_t0) > 0) {
          mbar_expect_tx(q_full + i, Cfg::kQTileBytes);
          for (int p = 0; p < Cfg::kPanels; ++p)
            tma_load_4d(q_smem + i * Cfg::kQTileBytes + p * Cfg::kQPanelBytes, &tm_q, q_full + i, p * 64,
                        m0 + i * Cfg::BM, h_idx, b);
        }
      };
      auto early_kv = [&](int t) {
        mbar_expect_tx(kv_full + t, Cfg::kKVTileBytes);
        for (int p = 0; p < Cfg::kPanels; ++p)
          tma_load_4d(kv_smem + t * Cfg::kKVTileBytes + p * Cfg::kKVPanelBytes, t ? &tm_v : &tm_k, kv_full + t, p * 64,
                      0, h_kv, b);
      };
      early_q(0);
      early_kv(0);
      early_q(1);
      early_kv(1);
    }
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
  if (tid == 0) FRAY_TRACE(6, 0, 1);

  if (warp < 8) {
    // =============================================================== softmax groups
    set_max_regs_inc<Cfg::kRegsSoftmax>();
    const int i = warp >> 2;
    const int r = tid & 127;
    const int h_i = i ? h_t1 : h_t0;
    const int row = m0 + i * Cfg::BM + r;
    const uint32_t lane_base = static_cast<uint32_t>((warp & 3) * 32) << 16;
    const uint32_t t_tile = tmem_base + (i == 0 ? Cfg::kColS0 : Cfg::kColS1) + lane_base;
    float m_ref = -INFINITY;
    float l_run = 0.f;
    const int h_both = h_t0 < h_t1 ? h_t0 : h_t1;  // half steps that both tiles run: these take turns
    auto mask_needed = [&](int h) { return (h * BH + BH > seq_k) || (causal && (h * BH + BH - 1 > m0 + i * Cfg::BM)); };
    for (int h = 0; h < h_i; ++h) {
      if (*abort_flag) break;  // a wait gave up somewhere in the CTA: stop touching tensor memory
      const int buf = h & 1;
      FRAY_CRIT_WAIT(s_full + i * 2 + buf, (h >> 1) & 1, abort_flag, 0x601 + i, h);
      tc_fence_after_sync();
      if (r == FRAY_TRACE_ROW) FRAY_TRACE(0, i, h);
      const int kv0 = h * BH;
      const bool need_mask = mask_needed(h);
      unsigned int* tr = nullptr;
#ifdef FRAY_ATTN_TRACE
      if (trace_on && r == FRAY_TRACE_ROW && h < kTraceIters) tr = trace_sm + i * kTraceIters + h;
#endif
      // Tile 0 goes first: its first wait names the parity of the phase before the barrier's first
      // one, which reads as complete; from then on each group waits for the other's previous step.
      const bool turns = kHalfStepTurns && h < h_both;
      softmax_half_step(t_tile + buf * BH, p_full + i * 2 + buf, corr_ready + i * 2 + buf,
                        alpha_buf + (i * 2 + buf) * 128 + r, h == 0, need_mask, kv0, row, seq_k, causal, scale_log2,
                        lane, m_ref, l_run, turns ? exp_turn + i : nullptr, turns ? exp_turn + (1 - i) : nullptr,
                        (h + 1 - i) & 1, abort_flag, tr);
      if (r == FRAY_TRACE_ROW) FRAY_TRACE(4, i, h);
    }
    if (h_i > 0) {
      l_buf[i * 128 + r] = l_run;
      m_buf[i * 128 + r] = m_ref;
      __syncwarp();
      if (lane == 0) mbar_arrive(l_ready + i);
    }
  } else if (warp < 12) {
    // =============================================================== correction group + epilogue
    set_max_regs_dec<Cfg::kRegsCorrection>();
    const int r = tid & 127;
    const uint32_t lane_base = static_cast<uint32_t>((warp & 3) * 32) << 16;
    for (int h = 1; h < h_max; ++h) {
      if (*abort_flag) break;
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        if (h < (i ? h_t1 : h_t0)) {
          const uint32_t use = ((h - 1) >> 1) & 1;  // parity of this use of the h&1 barriers
          mbar_wait(corr_ready + i * 2 + (h & 1), use, abort_flag, 0x701 + i, h);
          const float alpha = alpha_buf[(i * 2 + (h & 1)) * 128 + r];
          if (__any_sync(0xffffffffu, alpha != 1.f)) {
            mbar_wait(o_full + i, (h - 1) & 1, abort_flag, 0x711 + i, h);
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
          if (lane == 0) mbar_arrive(o_rescaled + i * 2 + (h & 1));
        }
      }
    }
    // Epilogue: O_i / l_i -> fp16 -> shared memory (the dead Q_i buffer, 128B-swizzled) -> TMA store.
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const int h_i = i ? h_t1 : h_t0;
      if (h_i > 0) {
        mbar_wait(l_ready + i, 0, abort_flag, 0x721 + i, h_i);
        const float l = l_buf[i * 128 + r];
        const float inv_l = l > 0.f ? 1.f / l : 1.f;
        mbar_wait(o_final + i, 0, abort_flag, 0x731 + i, h_i);
        tc_fence_after_sync();
        if (r == 0) FRAY_TRACE(6, 1, i);
        const uint32_t t_o = tmem_base + (i == 0 ? Cfg::kColO0 : Cfg::kColO1) + lane_base;
        uint8_t* o_tile = q_smem + i * Cfg::kQTileBytes;
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
        named_barrier_sync(1, 128);
        if (r == 0) {
#pragma unroll
          for (int p = 0; p < Cfg::kPanels; ++p)
            tma_store_4d(&tm_o, o_tile + p * Cfg::kQPanelBytes, p * 64, m0 + i * Cfg::BM, h_idx, b);
          tma_store_commit();
        }
        if (lse != nullptr && m0 + i * Cfg::BM + r < seq_len) {
          // log-sum-exp in natural units, written after the tile is on its way: nothing waits for this
          const float m = m_buf[i * 128 + r];
          lse[(static_cast<size_t>(b) * num_heads + h_idx) * seq_len + m0 + i * Cfg::BM + r] =
              l > 0.f ? (m * scale_log2 + log2f(l)) * 0.69314718055994531f : -INFINITY;
        }
      }
    }
    if (r == 0) {
      FRAY_TRACE(6, 1, 2);
      tma_store_wait_read();  // shared memory may go once the copies have read it; the writes finish on their own
      FRAY_TRACE(6, 1, 3);
    }
  } else {
    set_max_regs_dec<Cfg::kRegsOther>();
    if (warp == 13 && lane == 0) {
      // ============================================================= TMA producer
      // ring entries 0 and 1 and both Q tiles were issued during set-up (unless that is switched off)
      auto late_q = [&](int i) __attribute__((always_inline)) {
        if ((i ? n_t1 : n_t0) > 0) {
          mbar_expect_tx(q_full + i, Cfg::kQTileBytes);
#pragma unroll
          for (int p = 0; p < Cfg::kPanels; ++p)
            tma_load_4d(q_smem + i * Cfg::kQTileBytes + p * Cfg::kQPanelBytes, &tm_q, q_full + i, p * 64,
                        m0 + i * Cfg::BM, h_idx, b);
        }
      };
      if (!kEarlyCopies) {
        late_q(0);
      }
      for (int t = kEarlyCopies ? 2 : 0; t < 2 * n_max; ++t) {
        const int slot = t % STAGES;
        const uint32_t ph = (t / STAGES) & 1;
        mbar_wait(kv_empty + slot, ph ^ 1, abort_flag, 0x401, t);
        if (*abort_flag) break;  // issue no further copies into a CTA that is winding down
        mbar_expect_tx(kv_full + slot, Cfg::kKVTileBytes);
        const CUtensorMap* tm = (t & 1) ? &tm_v : &tm_k;
#pragma unroll
        for (int p = 0; p < Cfg::kPanels; ++p)
          tma_load_4d(kv_smem + slot * Cfg::kKVTileBytes + p * Cfg::kKVPanelBytes, tm, kv_full + slot, p * 64,
                      (t >> 1) * BN, h_kv, b);
        if (!kEarlyCopies && t == 0) late_q(1);
      }
    } else if (warp == 12) {
      // ============================================================= MMA issue (whole warp, one elected lane issues)
      constexpr uint64_t kDescK = smem_desc_sw128(16, 1024);                  // K-major operand (Q, K)
      constexpr uint64_t kDescV = smem_desc_sw128(Cfg::kKVPanelBytes, 1024);  // MN-major operand (V)
      constexpr uint32_t kIdescQK = idesc_f16_f32(Cfg::BM, BH, false, false);
      constexpr uint32_t kIdescPV = idesc_f16_f32(Cfg::BM, D, false, true);
      const uint32_t q_addr = smem_u32(q_smem);
      const uint32_t kv_addr = smem_u32(kv_smem);
      const int h0 = h_t0, h1 = h_t1;

      // A wait on an mbarrier costs this warp a shared-memory round trip (~50 cycles and more under
      // load) even when the phase is long complete, and one group of MMAs below needs up to four of
      // them.  In steady state all are complete, so they are tested together first (the round trips
      // overlap) and the bounded waits only run when one of them is not.
      auto k_slot = [&](int h) { return (2 * (h >> 1)) % STAGES; };
      auto k_par = [&](int h) { return static_cast<uint32_t>(((2 * (h >> 1)) / STAGES) & 1); };
      auto v_slot = [&](int h) { return (2 * (h >> 1) + 1) % STAGES; };
      auto v_par = [&](int h) { return static_cast<uint32_t>(((2 * (h >> 1) + 1) / STAGES) & 1); };

      // S_i(h) = Q_i . K[64 keys of half step h]^T into buffer h&1 (the K tile is known to be present)
      auto issue_qk = [&](int i, int h) __attribute__((always_inline)) {
        const int slot = k_slot(h);
        constexpr uint32_t kDescHi = static_cast<uint32_t>(kDescK >> 32);
        constexpr uint32_t kDescLo = static_cast<uint32_t>(kDescK);
        const uint32_t q_lo = kDescLo | (((q_addr + i * Cfg::kQTileBytes) & 0x3FFFF) >> 4);
        // rows 64*(h&1).. of the K tile: 64 rows of 128 bytes further inside each panel
        const uint32_t k_lo = kDescLo | (((kv_addr + slot * Cfg::kKVTileBytes + (h & 1) * (BH * 128)) & 0x3FFFF) >> 4);
        const uint32_t t_s = tmem_base + (i == 0 ? Cfg::kColS0 : Cfg::kColS1) + (h & 1) * BH;
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint32_t qoff = ((kk >> 2) * Cfg::kQPanelBytes + (kk & 3) * 32) >> 4;
          const uint32_t koff = ((kk >> 2) * Cfg::kKVPanelBytes + (kk & 3) * 32) >> 4;
          mma_ss_elect_lohi(t_s, q_lo + qoff, kDescHi, k_lo + koff, kDescHi, kIdescQK, kk > 0);
        }
        mma_commit_elect(s_full + i * 2 + (h & 1));
        // the K tile is free once the second half step of the last tile that uses it has been issued
        if ((h & 1) && ((i == 1) || !(h < h1))) mma_commit_elect(kv_empty + slot);
        FRAY_TRACE(8, i, h);
      };
      // O_i (+)= P_i(h) . V[64 keys of half step h] (V, P and the rescaled O are known to be ready)
      auto issue_pv = [&](int i, int h) __attribute__((always_inline)) {
        const int slot = v_slot(h);
        constexpr uint32_t kDescVHi = static_cast<uint32_t>(kDescV >> 32);
        const uint32_t v_lo = static_cast<uint32_t>(kDescV) | (((kv_addr + slot * Cfg::kKVTileBytes) & 0x3FFFF) >> 4);
        const uint32_t t_p = tmem_base + (i == 0 ? Cfg::kColS0 : Cfg::kColS1) + (h & 1) * BH;
        const uint32_t t_o = tmem_base + (i == 0 ? Cfg::kColO0 : Cfg::kColO1);
#pragma unroll
        for (int kk = 0; kk < BH / 16; ++kk) {
          const int kv16 = (h & 1) * 4 + kk;  // 16-key block inside the 128-key V tile
          mma_ts_elect_lohi(t_o, t_p + kk * 8, v_lo + ((kv16 * 2048) >> 4), kDescVHi, kIdescPV, (h > 0 || kk > 0));
        }
        mma_commit_elect(o_full + i);
        if (h + 1 == (i ? h1 : h0)) mma_commit_elect(o_final + i);
        if ((h & 1) && ((i == 1) || !(h < h1))) mma_commit_elect(kv_empty + slot);
        FRAY_TRACE(7, i, h);
      };
      // One group: P.V of half step h, then S of half step h+2 into the buffer that P.V frees.
      auto group = [&](int i, int h, int h_i) __attribute__((always_inline)) {
        const bool next_s = h + 2 < h_i;
        uint64_t* b_v = kv_full + v_slot(h);
        uint64_t* b_o = o_rescaled + i * 2 + (h & 1);
        uint64_t* b_p = p_full + i * 2 + (h & 1);
        uint64_t* b_k = kv_full + k_slot(h + 2);
        const uint32_t par_o = ((h - 1) >> 1) & 1, par_p = (h >> 1) & 1;
        bool ready = mbar_try_wait(b_v, v_par(h)) & mbar_try_wait(b_p, par_p);
        if (h > 0) ready = ready & mbar_try_wait(b_o, par_o);
        if (next_s) ready = ready & mbar_try_wait(b_k, k_par(h + 2));
        if (!ready) {
          mbar_wait(b_v, v_par(h), abort_flag, 0x502, h);
          if (h > 0) mbar_wait(b_o, par_o, abort_flag, 0x505 + i, h);
          FRAY_CRIT_WAIT(b_p, par_p, abort_flag, 0x503 + i, h);
        }
        tc_fence_after_sync();
        FRAY_TRACE(5, i, h);
        issue_pv(i, h);
        if (next_s) {
          if (!ready) {
            mbar_wait(b_k, k_par(h + 2), abort_flag, 0x501, h);
            tc_fence_after_sync();
          }
          issue_qk(i, h + 2);
        }
      };

      if (h0 > 0) {
        mbar_wait(q_full + 0, 0, abort_flag, 0x511);
        mbar_wait(kv_full + k_slot(0), k_par(0), abort_flag, 0x501, 0);
        tc_fence_after_sync();
        issue_qk(0, 0);
      }
      if (h1 > 0) {
        mbar_wait(q_full + 1, 0, abort_flag, 0x512);
        mbar_wait(kv_full + k_slot(0), k_par(0), abort_flag, 0x501, 0);
        tc_fence_after_sync();
        issue_qk(1, 0);
      }
      if (h0 > 1) issue_qk(0, 1);
      if (h1 > 1) issue_qk(1, 1);
      for (int h = 0; h < h_max; ++h) {
        if (*abort_flag) break;  // issue no further MMAs
        if (h < h0) group(0, h, h0);
        if (h < h1) group(1, h, h1);
      }
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem_base, Cfg::kTmemCols);
#ifdef FRAY_ATTN_TRACE
  if (tid == 0) FRAY_TRACE(6, 0, 2);
  __syncthreads();
  if (trace_on)
    for (int w = tid; w < kTraceWords; w += Cfg::kThreads) fray_attn_trace_buf[w] = trace_sm[w];
#endif
}

// Host launcher for the half-step kernel. Returns an AttnReturnCode.
template <int D, int STAGES>
inline int launch_attn_fwd_wsh(const operand_t* q, const operand_t* k, const operand_t* v, operand_t* o, const AttnShape& shp,
                               const AttnStrides (&st)[4], const AttnExtras& ex, bool causal, float scale,
                               cudaStream_t stream) {
  using Cfg = WshCfg<D, STAGES>;
  const AttnShape shp_kv{shp.B, shp.H / ex.kv_group, ex.seq_k, shp.D};
  CUtensorMap tm_q, tm_k, tm_v, tm_o;
  int rc = cached_attn_tensor_map(&tm_q, q, shp, st[0], Cfg::BM);
  if (rc != kAttnOk) return rc;
  rc = cached_attn_tensor_map(&tm_k, k, shp_kv, st[1], Cfg::BN);
  if (rc != kAttnOk) return rc;
  rc = cached_attn_tensor_map(&tm_v, v, shp_kv, st[2], Cfg::BN);
  if (rc != kAttnOk) return rc;
  rc = cached_attn_tensor_map(&tm_o, o, shp, st[3], Cfg::BM);
  if (rc != kAttnOk) return rc;

  auto kernel = attn_fwd_wsh_kernel<D, STAGES>;
  rc = ensure_dynamic_smem<Cfg>(kernel, Cfg::kSmemBytes);
  if (rc != kAttnOk) return rc;
  dim3 grid((shp.S + 2 * Cfg::BM - 1) / (2 * Cfg::BM), shp.B * shp.H);
  kernel<<<grid, Cfg::kThreads, Cfg::kSmemBytes, stream>>>(tm_q, tm_k, tm_v, tm_o, shp.H, shp.S, causal ? 1 : 0,
                                                           scale * 1.44269504088896340736f, ex.kv_group, ex.lse, ex.seq_k);
  if (cudaGetLastError() != cudaSuccess) return kAttnLaunchFailed;
  return kAttnOk;
}

}  // namespace sm100
}  // namespace fray
