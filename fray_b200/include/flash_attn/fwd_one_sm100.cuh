#pragma once
// Warp-specialised attention forward for sm_100a with ONE 128-row query tile per CTA and TWO CTAs per SM.
//
// A CTA of 8 warps owns one query tile of one (batch, head) slice:
//   warps 0-3  softmax group (thread r owns row r); it also rescales O when a row's offset moves and
//              writes the tile out at the end
//   warp 4     MMA issue (warp-uniform code, one elected lane issues)
//   warp 5     TMA producer (Q once, then K_j, V_j through a ring of STAGES buffers)
//   warps 6-7  idle (they only exist so that warps 4-7 form a full warpgroup for setmaxnreg)
//
// Tensor memory (256 columns, so two CTAs fit an SM): S [0,128), O [128, 128 + D).  P (16 bit)
// overwrites the first 64 columns of S and is consumed from there by the P.V product, as in the
// two-tile kernel (fwd_ws_sm100.cuh), and a CTA's steps form the same serial chain
// softmax(j) -> P.V(j) -> S(j+1) -> softmax(j+1).  What fills the tensor pipe and the special-function
// unit while one CTA is in the other phase is the second CTA of the SM instead of a second tile of the
// same CTA.  The two CTAs are independent launches of the hardware scheduler: when one ends the next
// starts, so a CTA's set-up, first copies and epilogue run beside the neighbour's steady state
// instead of leaving the SM idle (6-8 us per CTA of the two-tile kernel, a third of its time at 1024
// keys), and they sit half a CTA apart by themselves.
//
// There is no correction group: a softmax warp in which some row has to move its exponent offset
// (lazily: only when the row max grew by more than 2^8 in the scaled domain, which after the first KV
// tile almost never happens) waits for the previous P.V and rescales its rows of O itself.
//
// Shared memory must stay under half an SM: one Q tile and STAGES K/V buffers (2 at head dim 128: K_j
// and V_j each have a buffer of their own and the next tile is fetched as soon as the product that reads
// the buffer has completed, a full step before it is needed; up to 5 at head dim 64).
//
// Every barrier wait is bounded (see sm100_ptx.cuh): a protocol error ends as a status word and a
// wrong answer, never as a hung GPU.

#include "host_sm100.cuh"
#include "sm100_ptx.cuh"
#include "softmax_tile_sm100.cuh"

namespace fray {
namespace sm100 {

template <int D, int BN, int STAGES>
struct OneCfg {
  static_assert(D == 64 || D == 128, "head dim must be 64 or 128");
  static_assert(BN == 128, "the warp-specialised kernels use 128-key tiles");
  static_assert(STAGES >= 2 && STAGES <= 5, "2..5 K/V buffers");
  static constexpr int BM = 128;               // rows of the query tile
  static constexpr int kPChunks = 2;           // P is handed to the MMA warp in two chunks of 64 keys
  static constexpr int kThreads = 256;
  static constexpr int kPanels = D / 64;       // 64-element (128-byte) column panels
  static constexpr int kQPanelBytes = BM * 128;
  static constexpr int kQTileBytes = kPanels * kQPanelBytes;
  static constexpr int kKVPanelBytes = BN * 128;
  static constexpr int kKVTileBytes = kPanels * kKVPanelBytes;
  static constexpr int kOffQ = 0;
  static constexpr int kOffKV = kQTileBytes;
  static constexpr int kOffBars = kOffKV + STAGES * kKVTileBytes;
  static constexpr int kNumBars = 1 + 2 * STAGES + 1 + 1 + kPChunks;
  static constexpr int kSmemBytes = kOffBars + ((kNumBars * 8 + 16 + 127) / 128) * 128 + 1024;  // + alignment slack
  static_assert(2 * (kSmemBytes + 1024) <= 233472, "two CTAs must fit the 228 KB shared memory of an SM");
  static constexpr int kTmemCols = 256;
  static constexpr uint32_t kColS = 0, kColO = 128;
  // Register budgets after setmaxnreg (softmax warps, the other four).  The pool is the CTA's allocation at
  // launch, 256 threads x 128 registers (two CTAs per SM); per scheduler 2 x (184 + 72) = 512.
  static constexpr int kRegsLaunch = 128, kRegsSoftmax = 184, kRegsOther = 72;
  static_assert(128 * kRegsSoftmax + 128 * kRegsOther <= kThreads * kRegsLaunch, "register budgets exceed the CTA's allocation");
};

template <int D, int BN, int STAGES>
__global__ void __launch_bounds__(256, 2)
attn_fwd_one_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                    const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_o, int num_heads,
                    int seq_len, int causal, float scale_log2, int kv_group, float* lse, int seq_k, int heaviest_first) {
  using Cfg = OneCfg<D, BN, STAGES>;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  uint8_t* smem = smem_raw + (((raw_addr + 1023u) & ~1023u) - raw_addr);
  uint8_t* q_smem = smem + Cfg::kOffQ;    // reused for the O tile at the end
  uint8_t* kv_smem = smem + Cfg::kOffKV;  // ring slot s at kv_smem + s * kKVTileBytes
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Cfg::kOffBars);
  uint64_t* q_full = bars;                      // [1]   producer -> MMA
  uint64_t* kv_full = bars + 1;                 // [STAGES] producer -> MMA
  uint64_t* kv_empty = kv_full + STAGES;        // [STAGES] MMA -> producer
  uint64_t* s_full = kv_empty + STAGES;         // [1]   MMA -> softmax  (S(j) complete)
  uint64_t* o_full = s_full + 1;                // [1]   MMA -> softmax  (P.V(j) complete: rescale, epilogue)
  uint64_t* p_full = o_full + 1;                // [kPChunks] softmax -> MMA (chunk c of P(j) stored)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + Cfg::kNumBars);
  volatile uint32_t* abort_flag = reinterpret_cast<volatile uint32_t*>(tmem_slot + 1);

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;
  // Grid order: (tiles, slices) runs slice by slice, so that CTAs side by side share a slice's K and V in
  // L2; with heaviest_first the axes are swapped and all slices' longest causal tiles start first, which
  // balances a causal problem of few rounds of CTAs (the launcher decides, see heaviest_first_order).
  const int n_x = heaviest_first ? gridDim.y : gridDim.x;
  const int px = heaviest_first ? blockIdx.y : blockIdx.x;
  const int tile = causal ? (n_x - 1 - px) : px;  // heaviest causal tiles first
  const int m0 = tile * Cfg::BM;
  const int bh = heaviest_first ? blockIdx.x : blockIdx.y;
  const int b = bh / num_heads;
  const int h = bh - b * num_heads;
  const int h_kv = h / kv_group;

  int n = (seq_k + BN - 1) / BN;  // KV tiles this query tile consumes (seq_len counts queries, seq_k keys)
  if (causal) {
    const int lim = (m0 + Cfg::BM + BN - 1) / BN;
    n = lim < n ? lim : n;
  }

  if (tid == 0) {
    *abort_flag = (*reinterpret_cast<volatile int*>(&fray_attn_status[0]) != 0) ? 2u : 0u;
    mbar_init(q_full, 1);
    mbar_init(s_full, 1);
    mbar_init(o_full, 1);
    for (int c = 0; c < Cfg::kPChunks; ++c) mbar_init(p_full + c, 4);  // one arrival per warp
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
    // two CTAs of an SM allocate 256 columns each; the allocation waits inside the instruction until the
    // columns are there, which they are as soon as an earlier CTA of the SM has freed its own
    tmem_alloc(tmem_slot, Cfg::kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  if (warp < 4) {
    // =============================================================== softmax group
    set_max_regs_inc<Cfg::kRegsSoftmax>();
    const int r = tid;  // row inside the tile
    const int row = m0 + r;
    const uint32_t lane_base = static_cast<uint32_t>(warp * 32) << 16;
    const uint32_t t_s = tmem_base + Cfg::kColS + lane_base;
    const uint32_t t_o = tmem_base + Cfg::kColO + lane_base;
    float m_ref = -INFINITY;  // exponent offset currently baked into P, l and O
    float l_run = 0.f;
    for (int j = 0; j < n; ++j) {
      FRAY_CRIT_WAIT(s_full, j & 1, abort_flag, 0x201, j);
      tc_fence_after_sync();
      const int kv0 = j * BN;
      const bool need_mask = (kv0 + BN > seq_k) || (causal && (kv0 + BN - 1 > m0));
      // A row whose offset moves multiplies its row of O by the factor before this step's P.V is issued
      // (the MMA warp issues it only after this warp has handed P over).  Tensor-memory loads and stores
      // are warp-wide instructions: every lane takes part, rows that keep their offset multiply by one.
      auto rescale_o = [&](float alpha) {
        if (__any_sync(0xffffffffu, alpha != 1.f)) {
          mbar_wait(o_full, (j - 1) & 1, abort_flag, 0x311, j);  // the previous P.V has landed in O
          tc_fence_after_sync();
          // 16 columns at a time: the step's whole row of scores is live in registers here
#pragma unroll 1
          for (int c = 0; c < D / 16; ++c) {
            uint32_t orr[16];
            tmem_ld_x16(t_o + c * 16, orr);
            tmem_wait_ld();
#pragma unroll
            for (int x = 0; x < 16; ++x) orr[x] = __float_as_uint(__uint_as_float(orr[x]) * alpha);
            tmem_st_x16(t_o + c * 16, orr);
          }
          tmem_wait_st();
        }
      };
      if (need_mask) {
        softmax_tile_with<BN, Cfg::kPChunks, true, false>(t_s, p_full, rescale_o, j == 0, kv0, row, seq_k, causal, scale_log2, lane,
                                                   m_ref, l_run);
      } else {
        softmax_tile_with<BN, Cfg::kPChunks, false, false>(t_s, p_full, rescale_o, j == 0, kv0, row, seq_k, causal, scale_log2, lane,
                                                    m_ref, l_run);
      }
    }
    if (n > 0) {
      mbar_wait(o_full, (n - 1) & 1, abort_flag, 0x331, n);
      tc_fence_after_sync();
      epilogue_tile<Cfg, D>(t_o, q_smem, r, l_run, m_ref, &tm_o, m0, h, b, num_heads, seq_len, scale_log2, lse, 4);
      if (r == 0) tma_store_wait_read();  // shared memory may go once the copy has read it
    }
  } else {
    set_max_regs_dec<Cfg::kRegsOther>();
    if (warp == 5 && lane == 0) {
      // ============================================================= TMA producer
      if (n > 0) {
        mbar_expect_tx(q_full, Cfg::kQTileBytes);
#pragma unroll
        for (int p = 0; p < Cfg::kPanels; ++p)
          tma_load_4d(q_smem + p * Cfg::kQPanelBytes, &tm_q, q_full, p * 64, m0, h, b);
      }
      for (int t = 0; t < 2 * n; ++t) {
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
      }
    } else if (warp == 4) {
      // ============================================================= MMA issue (whole warp, one elected lane issues)
      constexpr uint64_t kDescK = smem_desc_sw128(16, 1024);                  // K-major operand (Q, K)
      constexpr uint64_t kDescV = smem_desc_sw128(Cfg::kKVPanelBytes, 1024);  // MN-major operand (V)
      constexpr uint32_t kIdescQK = idesc_f16_f32(Cfg::BM, BN, false, false);
      constexpr uint32_t kIdescPV = idesc_f16_f32(Cfg::BM, D, false, true);
      constexpr uint32_t kDescHi = static_cast<uint32_t>(kDescK >> 32);
      constexpr uint32_t kDescLo = static_cast<uint32_t>(kDescK);
      constexpr uint32_t kDescVHi = static_cast<uint32_t>(kDescV >> 32);
      const uint32_t kv_addr = smem_u32(kv_smem);
      // descriptor start addresses are in 16-byte units and never carry out of the 14-bit field
      const uint32_t q_lo = kDescLo | ((smem_u32(q_smem) & 0x3FFFF) >> 4);
      const uint32_t t_s = tmem_base + Cfg::kColS;
      const uint32_t t_o = tmem_base + Cfg::kColO;

      auto issue_qk = [&](int j) __attribute__((always_inline)) {  // S(j) = Q . K_j^T
        const int t = 2 * j;
        const int slot = t % STAGES;
        mbar_wait(kv_full + slot, (t / STAGES) & 1, abort_flag, 0x501, t);
        tc_fence_after_sync();
        const uint32_t k_lo = kDescLo | (((kv_addr + slot * Cfg::kKVTileBytes) & 0x3FFFF) >> 4);
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint32_t qoff = ((kk >> 2) * Cfg::kQPanelBytes + (kk & 3) * 32) >> 4;
          const uint32_t koff = ((kk >> 2) * Cfg::kKVPanelBytes + (kk & 3) * 32) >> 4;
          mma_ss_elect_lohi(t_s, q_lo + qoff, kDescHi, k_lo + koff, kDescHi, kIdescQK, kk > 0);
        }
        mma_commit_elect(s_full);
        mma_commit_elect(kv_empty + slot);
      };
      auto issue_pv = [&](int j) __attribute__((always_inline)) {  // O (+)= P(j) . V_j, chunk by chunk as P arrives
        const int t = 2 * j + 1;
        const int slot = t % STAGES;
        mbar_wait(kv_full + slot, (t / STAGES) & 1, abort_flag, 0x502, t);
        const uint32_t v_lo = static_cast<uint32_t>(kDescV) | (((kv_addr + slot * Cfg::kKVTileBytes) & 0x3FFFF) >> 4);
#pragma unroll
        for (int q = 0; q < Cfg::kPChunks; ++q) {
          FRAY_CRIT_WAIT(p_full + q, j & 1, abort_flag, 0x503, j);
          tc_fence_after_sync();
#pragma unroll
          for (int s2 = 0; s2 < 8 / Cfg::kPChunks; ++s2) {
            const int kk = (8 / Cfg::kPChunks) * q + s2;  // MMA (16 keys) inside the step
            mma_ts_elect_lohi(t_o, t_s + kk * 8, v_lo + ((kk * 2048) >> 4), kDescVHi, kIdescPV, (j > 0 || kk > 0));
          }
        }
        mma_commit_elect(o_full);
        mma_commit_elect(kv_empty + slot);
      };

      if (n > 0) {
        mbar_wait(q_full, 0, abort_flag, 0x511);
        issue_qk(0);
      }
      for (int j = 0; j < n; ++j) {
        issue_pv(j);
        if (j + 1 < n) issue_qk(j + 1);
      }
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem_base, Cfg::kTmemCols);
}

// Host launcher for the one-tile kernel. Returns an AttnReturnCode.
template <int D, int BN, int STAGES>
inline int launch_attn_fwd_one(const operand_t* q, const operand_t* k, const operand_t* v, operand_t* o, const AttnShape& shp,
                               const AttnStrides (&st)[4], const AttnExtras& ex, bool causal, float scale,
                               cudaStream_t stream) {
  using Cfg = OneCfg<D, BN, STAGES>;
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

  auto kernel = attn_fwd_one_kernel<D, BN, STAGES>;
  rc = ensure_dynamic_smem<Cfg>(kernel, Cfg::kSmemBytes, Cfg::kThreads, 128 * Cfg::kRegsSoftmax + 128 * Cfg::kRegsOther);
  if (rc != kAttnOk) return rc;
  const int heaviest_first = heaviest_first_order(causal, shp, shp_kv) ? 1 : 0;
  const unsigned n_x = (shp.S + Cfg::BM - 1) / (Cfg::BM), n_bh = shp.B * shp.H;
  dim3 grid(heaviest_first ? n_bh : n_x, heaviest_first ? n_x : n_bh);
  kernel<<<grid, Cfg::kThreads, Cfg::kSmemBytes, stream>>>(tm_q, tm_k, tm_v, tm_o, shp.H, shp.S, causal ? 1 : 0,
                                                           scale * 1.44269504088896340736f, ex.kv_group, ex.lse, ex.seq_k,
                                                           heaviest_first);
  if (cudaGetLastError() != cudaSuccess) return kAttnLaunchFailed;
  return kAttnOk;
}

}  // namespace sm100
}  // namespace fray
