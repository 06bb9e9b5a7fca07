#pragma once
// Warp-specialised attention forward for sm_100a.
//
// One CTA of 16 warps owns two 128-row query tiles of one (batch, head) slice:
//   warps 0-3   softmax group 0 (query tile 0; thread r owns row r)
//   warps 4-7   softmax group 1 (query tile 1)
//   warps 8-11  correction group: rescales the O accumulators when a running max moved,
//               and runs the epilogue (O/l -> fp16 -> shared memory -> TMA store)
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
// the special-function unit were both measured slower than this fixed alternation.)  P.V is issued in four key chunks as the
// softmax hands them over, so only the last quarter of it sits behind the softmax.
//
// Online softmax in base 2 with lazy rescaling: a tile's exponent offset m_ref only moves
// when the running max grew by more than 2^8 in the scaled domain; until then P may exceed
// 1 (at most 256, exact in fp16 range) and O needs no correction.  O and l always share the
// same m_ref, so the final O/l is the exact softmax up to rounding.
//
// Split-row variant (SPLIT = 2, 24 warps): each query tile gets two softmax warpgroups; the first
// works on keys [0,KA) of every tile, the second on keys [KA,128) of the same rows, with its
// exponentials on the FMA pipe when KA > 64 (see softmax_part_tile).  Warps 0-7 then serve tile 0,
// warps 8-15 tile 1, and the correction / MMA / producer warps follow.
//
// Helper variant (SPLIT = 3, 16 warps as in the plain kernel): the softmax group of a tile works on
// keys [0,KA) only, and the correction group, otherwise idle, takes keys [KA,128) of both tiles with
// its exponentials on the FMA pipe.  It runs on the same schedulers as the softmax warps, so its
// arithmetic fills the issue slots that the softmax warps leave while they wait for the
// special-function unit, and a quarter of that unit's work disappears.  The group takes part in
// the offset decision itself, so the factor for O needs no hand-over: it rescales O right there.
//
// Every barrier wait is bounded (see sm100_ptx.cuh): a protocol error ends as a status
// word and a wrong answer, never as a hung GPU.

#include "host_sm100.cuh"
#include "sm100_ptx.cuh"
#include "softmax_tile_sm100.cuh"

// Per-thread register budgets of the three kinds of warps (softmax, correction, MMA/producer), each a
// multiple of 8; 256*S + 128*C + 128*O must not exceed the 64K registers of an SM.
#ifndef FRAY_WS_REGS_S
#define FRAY_WS_REGS_S 184
#endif
#ifndef FRAY_WS_REGS_C
#define FRAY_WS_REGS_C 80
#endif
#ifndef FRAY_WS_REGS_O
#define FRAY_WS_REGS_O 64
#endif
// Helper variant: the correction group also runs a share of the softmax and needs more registers.
#ifndef FRAY_WS3_REGS_S
#define FRAY_WS3_REGS_S 168
#endif
#ifndef FRAY_WS3_REGS_C
#define FRAY_WS3_REGS_C 112
#endif
// The same for the split-row variant.  setmaxnreg only moves registers inside the CTA's own
// allocation (threads x registers at launch = 768 x 80 here, not the whole register file), and an
// increase that the decreases of the other warps cannot cover blocks for ever:
// 256*(A + B) + 128*C + 128*O <= 768*80, where the two softmax groups of a tile get A and B
// registers according to the number of keys each holds (see WsCfg).
#ifndef FRAY_WS2_REGS_C
#define FRAY_WS2_REGS_C 72
#endif
#ifndef FRAY_WS2_REGS_O
#define FRAY_WS2_REGS_O 56
#endif

// Whether the MMA warp keeps one copy of each issue sequence with the tile index as a run-time value
// (-DFRAY_COMPACT_MMA_ROLE=0/1).  The kernel shrinks from 88 to 71 KB; measured on one box: +8 % on the
// 4 x 32 x 4096 causal configuration, +2 % on 2 x 16 x 2048, nothing on the headline shape, -1.4 % on
// 1 x 32 x 16384 causal.  (In the half-step kernel, whose MMA warp is on the critical path, the same
// change cost 7 %.)
#ifndef FRAY_COMPACT_MMA_ROLE
#define FRAY_COMPACT_MMA_ROLE 1
#endif

namespace fray {
namespace sm100 {

template <int D, int BN, int STAGES, int SPLIT = 1, int KA = 64>
struct WsCfg {
  static_assert(KA == 64 || KA == 80 || KA == 96, "keys of a tile that the first softmax group of a split row takes");
  static_assert(SPLIT >= 2 || KA == 64, "KA only applies to split rows");
  static_assert(SPLIT != 3 || KA > 64, "the helper takes the smaller part");
  static_assert(SPLIT >= 1 && SPLIT <= 3, "1: one softmax thread per row; 2: two; 3: one plus the correction group as helper");
  static constexpr bool kHelper = SPLIT == 3;
  static_assert(D == 64 || D == 128, "head dim must be 64 or 128");
  static_assert(BN == 128, "the warp-specialised kernel uses 128-key tiles");
  static_assert(STAGES >= 2 && STAGES <= 8, "2..8 K/V buffers");
  static constexpr int BM = 128;               // rows per query tile
  // P is handed to the MMA warp in this many column chunks; chunk q covers chunk_steps(q) MMAs of 16 keys.
  static constexpr int kPChunks = (SPLIT >= 2 && KA == 80) ? 5 : 4;
  static constexpr int kChunksA = SPLIT == 1 ? 4 : (KA == 64 ? 2 : 3);  // chunks written by the first group
  __host__ __device__ static constexpr int chunk_steps(int q) {
    return (SPLIT >= 2 && KA == 80 && (q == 2 || q == 3)) ? 1 : 2;
  }
  static constexpr int kSoftmaxWarps = SPLIT == 2 ? 16 : 8;
  static constexpr int kThreads = 32 * (kSoftmaxWarps + 8);
  static constexpr int kPanels = D / 64;       // 64-element (128-byte) column panels
  static constexpr int kQPanelBytes = BM * 128;
  static constexpr int kQTileBytes = kPanels * kQPanelBytes;
  static constexpr int kKVPanelBytes = BN * 128;
  static constexpr int kKVTileBytes = kPanels * kKVPanelBytes;
  static constexpr int kOffQ = 0;
  static constexpr int kOffKV = 2 * kQTileBytes;
  static constexpr int kOffBars = kOffKV + STAGES * kKVTileBytes;
  static constexpr int kNumBars = 2 + 2 * STAGES + 2 * 5 + 2 * kPChunks;
  static constexpr int kOffStats = kOffBars + ((kNumBars * 8 + 16 + 127) / 128) * 128;  // alpha[2][128], l[2][128]
  static constexpr int kOffXchg = kOffStats + 6 * 128 * 4;  // (+ m[2][128]) half-row maxima [2 parities][2 tiles][2 halves][128]
  static constexpr int kXchgBytes = SPLIT >= 2 ? 2 * 2 * 2 * 128 * 4 : 0;
#ifdef FRAY_ATTN_TRACE
  static constexpr int kOffTrace = kOffXchg + kXchgBytes;
  static constexpr int kSmemBytes = kOffTrace + 4 * 800 + 1024;
#else
  static constexpr int kSmemBytes = kOffXchg + kXchgBytes + 1024;                      // + alignment slack
#endif
  static_assert(kSmemBytes <= 232448, "exceeds the 227 KB shared memory of one CTA");
  static constexpr int kTmemCols = 512;
  static constexpr uint32_t kColS0 = 0, kColS1 = 128, kColO0 = 256, kColO1 = 384;
  // register budgets after setmaxnreg (sum over 16 warps = 64K registers)
  static constexpr int kRegsSoftmax =
      SPLIT == 2 ? (KA == 64 ? 88 : KA == 80 ? 96 : 112) : SPLIT == 3 ? FRAY_WS3_REGS_S : FRAY_WS_REGS_S;
  static constexpr int kRegsSoftmaxB = SPLIT == 2 ? 176 - kRegsSoftmax : kRegsSoftmax;  // second group of a split row
  static constexpr int kRegsCorrection = SPLIT == 2 ? FRAY_WS2_REGS_C : SPLIT == 3 ? FRAY_WS3_REGS_C : FRAY_WS_REGS_C;
  static constexpr int kRegsOther = SPLIT == 2 ? FRAY_WS2_REGS_O : FRAY_WS_REGS_O;
  // Registers per thread the CTA is launched with: what __launch_bounds__(kThreads, 1) lets ptxas use.
  static constexpr int kRegsAtLaunch = (65536 / kThreads) / 8 * 8;
  static_assert(kSoftmaxWarps * 16 * (kRegsSoftmax + kRegsSoftmaxB) + 128 * kRegsCorrection + 128 * kRegsOther <=
                    kThreads * kRegsAtLaunch,
                "register budgets exceed the CTA's allocation: setmaxnreg.inc would never return");
  static_assert(kRegsCorrection <= kRegsAtLaunch && kRegsOther <= kRegsAtLaunch && kRegsSoftmax >= kRegsAtLaunch,
                "setmaxnreg.dec must not raise and .inc must not lower the count");
};


// Optional role timeline for bring-up and tuning: with -DFRAY_ATTN_TRACE one thread per role of
// CTA (0,0) stamps clock64 into a shared-memory table indexed by (event, tile, iteration < 40);
// the table is copied to a device buffer at the end and read back with fray_attn_trace_read.
// Compiled out by default.
#ifndef FRAY_TRACE_ROW
#define FRAY_TRACE_ROW 0  // which row's thread stamps the softmax events
#endif
#ifndef FRAY_TRACE_PART
#define FRAY_TRACE_PART 0  // split rows: which of the row's two threads stamps them
#endif
#ifdef FRAY_ATTN_TRACE
static constexpr int kTraceEvents = 10, kTraceIters = 40;
static constexpr int kTraceWords = kTraceEvents * 2 * kTraceIters;
__device__ unsigned int fray_attn_trace_buf[kTraceWords];
#define FRAY_TRACE(event, tile, iter)                                                              \
  do {                                                                                             \
    if (trace_on && (iter) < kTraceIters)                                                          \
      trace_sm[((event) * 2 + (tile)) * kTraceIters + (iter)] = static_cast<unsigned int>(clock64()); \
  } while (0)
inline int read_attn_trace(unsigned int* out, int max_words) {
  const int n = max_words < kTraceWords ? max_words : kTraceWords;
  if (cudaMemcpyFromSymbol(out, fray_attn_trace_buf, sizeof(unsigned int) * n) != cudaSuccess) return -1;
  return n;
}
#else
#define FRAY_TRACE(event, tile, iter) do { } while (0)
#endif


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

template <int D, int BN, int STAGES, int POLY, int SPLIT, int KA>
__global__ void __launch_bounds__(SPLIT == 2 ? 768 : 512, 1)
attn_fwd_ws_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                   const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_o,
                   int num_heads, int seq_len, int causal, float scale_log2, int kv_group, float* lse, int seq_k) {
  using Cfg = WsCfg<D, BN, STAGES, SPLIT, KA>;
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
  uint64_t* corr_ready = o_full + 2;            // [2]   softmax i -> correction (alpha_i(j) / final l published)
  uint64_t* o_rescaled = corr_ready + 2;        // [2]   correction -> MMA       (O_i ready for PV_i(j))
  uint64_t* p_full = o_rescaled + 2;            // [2][kPChunks] softmax i -> MMA (chunk c of P_i(j) stored)
  uint64_t* sfu_turn = p_full + 2 * Cfg::kPChunks;  // [2] softmax (1-i) -> softmax i: the special-function unit is yours
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + Cfg::kNumBars);
  volatile uint32_t* abort_flag = reinterpret_cast<volatile uint32_t*>(tmem_slot + 1);
  float* alpha_buf = reinterpret_cast<float*>(smem + Cfg::kOffStats);  // [2][128]
  float* l_buf = alpha_buf + 256;                                      // [2][128]
  float* m_buf = l_buf + 256;                                          // [2][128] final exponent offsets (for the LSE output)
  float* xchg = reinterpret_cast<float*>(smem + Cfg::kOffXchg);        // [2][2][2][128], split-row variant only

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
#ifdef FRAY_DEBUG_SINGLE_TILE
  const int n_t0 = tiles_for(0), n_t1 = 0;  // timing experiment: tile 1 idle (its output rows are not computed)
#else
  const int n_t0 = tiles_for(0), n_t1 = tiles_for(1);
#endif  // scalars: an indexed array would live in local memory
  const int n_max = n_t0 > n_t1 ? n_t0 : n_t1;

  if (tid == 0) {
    FRAY_TRACE(6, 0, 0);  // CTA entry
    *abort_flag = (*reinterpret_cast<volatile int*>(&fray_attn_status[0]) != 0) ? 2u : 0u;
    for (int i = 0; i < 2; ++i) {
      mbar_init(q_full + i, 1);
      mbar_init(s_full + i, 1);
      for (int c = 0; c < Cfg::kPChunks; ++c) mbar_init(p_full + i * Cfg::kPChunks + c, 4);  // one arrival per warp
      mbar_init(o_full + i, 1);
      mbar_init(corr_ready + i, 4);  // one arrival per warp: 32 lanes arriving on one barrier would serialise
      mbar_init(o_rescaled + i, 4);
      mbar_init(sfu_turn + i, 4);
    }
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
                        m0 + i * Cfg::BM, h, b);
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
  if (tid == 0) FRAY_TRACE(6, 0, 1);  // set-up done

  // (rotating the role assignment over the warp index was measured to make no difference)
  const int role = warp < Cfg::kSoftmaxWarps ? 0 : warp - Cfg::kSoftmaxWarps + 8;
  if (role < 8) {
    // =============================================================== softmax groups
    const int i = warp / (SPLIT == 2 ? 8 : 4);  // query tile of this group
    const int r = tid & 127;              // row inside the tile
    const int n_i = i ? n_t1 : n_t0;
    const int row = m0 + i * Cfg::BM + r;
    const uint32_t lane_base = static_cast<uint32_t>((warp & 3) * 32) << 16;
    const uint32_t t_s = tmem_base + (i == 0 ? Cfg::kColS0 : Cfg::kColS1) + lane_base;
    uint64_t* p_bar = p_full + i * Cfg::kPChunks;
    float m_ref = -INFINITY;  // exponent offset currently baked into P, l and O
    float l_run = 0.f;

    if constexpr (SPLIT == 1) {
      set_max_regs_inc<Cfg::kRegsSoftmax>();
      static_assert(SPLIT == 2 || Cfg::kPChunks == kSoftmaxPChunks, "softmax_tile hands P over in kSoftmaxPChunks chunks");
      const int n_both = n_t0 < n_t1 ? n_t0 : n_t1;  // KV steps that both tiles run
      for (int j = 0; j < n_i; ++j) {
        FRAY_CRIT_WAIT(s_full + i, j & 1, abort_flag, 0x201 + i, j);
        tc_fence_after_sync();
        if (r == FRAY_TRACE_ROW) FRAY_TRACE(0, i, j);

        const int kv0 = j * BN;
        const bool need_mask = (kv0 + BN > seq_k) || (causal && (kv0 + BN - 1 > m0 + i * Cfg::BM));
        // Steps both tiles run take turns on the special-function unit; tile 0 goes first (its first
        // wait uses the parity of the phase "before" the barrier's first one, which reads as complete).
        const bool take_turns = kSfuTurns && j < n_both;
        softmax_tile<BN, POLY>(t_s, p_bar, corr_ready + i, alpha_buf + i * 128 + r, j == 0, need_mask, kv0, row,
                               seq_k, causal, scale_log2, lane, m_ref, l_run, take_turns ? sfu_turn + i : nullptr,
                               take_turns ? sfu_turn + (1 - i) : nullptr, (j + 1 - i) & 1, abort_flag);
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
    } else if constexpr (SPLIT == 3) {
      // Keys [0,KA) of every step; the helper group takes the rest and owns the O rescaling.
      set_max_regs_inc<Cfg::kRegsSoftmax>();
      auto ignore_alpha = [](float) {};
      for (int j = 0; j < n_i; ++j) {
        FRAY_CRIT_WAIT(s_full + i, j & 1, abort_flag, 0x201 + i, j);
        tc_fence_after_sync();
        if (r == FRAY_TRACE_ROW) FRAY_TRACE(0, i, j);
        const int kv0 = j * BN;
        const bool need_mask = (kv0 + BN > seq_k) || (causal && (kv0 + BN - 1 > m0 + i * Cfg::BM));
        float* x = xchg + (((j & 1) * 2 + i) * 2) * 128 + r;
        unsigned int* tr = nullptr;
#ifdef FRAY_ATTN_TRACE
        if (trace_on && r == FRAY_TRACE_ROW && j < kTraceIters) tr = trace_sm + i * kTraceIters + j;
#endif
        softmax_part_tile<BN, 0, KA, false, 0>(t_s, p_bar, ignore_alpha, x, x + 128, 2 + i, j == 0, need_mask, kv0, row,
                                               seq_k, causal, scale_log2, lane, m_ref, l_run, tr);
        if (r == FRAY_TRACE_ROW) FRAY_TRACE(4, i, j);
      }
      if (n_i > 0) {
        l_buf[i * 128 + r] = l_run;  // partial sum over this group's keys; the helper adds its own
        m_buf[i * 128 + r] = m_ref;
        __syncwarp();
        if (lane == 0) mbar_arrive(corr_ready + i);
      }
    } else {
      // Two groups per tile: the first takes keys [0,KA) of every step, the second keys [KA,128).
      auto part_role = [&](auto part_tag) __attribute__((always_inline)) {
        constexpr int PART = decltype(part_tag)::value;
        for (int j = 0; j < n_i; ++j) {
          FRAY_CRIT_WAIT(s_full + i, j & 1, abort_flag, 0x201 + i, j);
          tc_fence_after_sync();
          if (r == FRAY_TRACE_ROW && PART == FRAY_TRACE_PART) FRAY_TRACE(0, i, j);
          const int kv0 = j * BN;
          const bool need_mask = (kv0 + BN > seq_k) || (causal && (kv0 + BN - 1 > m0 + i * Cfg::BM));
          float* x = xchg + (((j & 1) * 2 + i) * 2) * 128 + r;
          unsigned int* tr = nullptr;
#ifdef FRAY_ATTN_TRACE
          if (trace_on && r == FRAY_TRACE_ROW && PART == FRAY_TRACE_PART && j < kTraceIters) tr = trace_sm + i * kTraceIters + j;
#endif
          if constexpr (PART == 0) {
            auto publish_alpha = [&](float alpha) {
              alpha_buf[i * 128 + r] = alpha;
              __syncwarp();
              if (lane == 0) mbar_arrive(corr_ready + i);
            };
            softmax_part_tile<BN, 0, KA, false, 0>(t_s, p_bar, publish_alpha, x, x + 128, 2 + i, j == 0, need_mask, kv0,
                                                   row, seq_k, causal, scale_log2, lane, m_ref, l_run, tr);
          } else {
            auto ignore_alpha = [](float) {};
            softmax_part_tile<BN, KA, BN - KA, (KA > 64), Cfg::kChunksA>(t_s, p_bar, ignore_alpha, x + 128, x, 2 + i,
                                                                         j == 0, need_mask, kv0, row, seq_k, causal,
                                                                         scale_log2, lane, m_ref, l_run, tr);
          }
          if (r == FRAY_TRACE_ROW && PART == FRAY_TRACE_PART) FRAY_TRACE(4, i, j);
        }
        if (n_i > 0) {
          // the row sum is the sum of the two parts' partial sums (both carry the same offset)
          float* x = xchg + (((n_i & 1) * 2 + i) * 2) * 128 + r;
          if constexpr (PART == 1) *x = l_run;
          named_barrier_sync(2 + i, 256);
          if constexpr (PART == 0) {
            l_buf[i * 128 + r] = l_run + *x;
            m_buf[i * 128 + r] = m_ref;
            __syncwarp();
            if (lane == 0) mbar_arrive(corr_ready + i);
          }
        }
      };
      if (((warp >> 2) & 1) == 0) {
        set_max_regs_inc<Cfg::kRegsSoftmax>();
        part_role(SmInt<0>{});
      } else {
        if constexpr (Cfg::kRegsSoftmaxB >= Cfg::kRegsAtLaunch) {
          set_max_regs_inc<Cfg::kRegsSoftmaxB>();
        } else {
          set_max_regs_dec<Cfg::kRegsSoftmaxB>();
        }
        part_role(SmInt<1>{});
      }
    }
  } else if (role < 12) {
    // =============================================================== correction group + epilogue
    set_max_regs_dec<Cfg::kRegsCorrection>();
    const int r = tid & 127;
    const uint32_t lane_base = static_cast<uint32_t>((warp & 3) * 32) << 16;
    float l_help0 = 0.f, l_help1 = 0.f;  // helper variant: row sums over this group's keys
    if constexpr (Cfg::kHelper) {
      float m_help0 = -INFINITY, m_help1 = -INFINITY;
      auto helper_step = [&](auto tile_tag, int j, float& m_ref, float& l_part) __attribute__((always_inline)) {
        constexpr int i = decltype(tile_tag)::value;
        FRAY_CRIT_WAIT(s_full + i, j & 1, abort_flag, 0x341 + i, j);
        tc_fence_after_sync();
        const int kv0 = j * BN;
        const bool need_mask = (kv0 + BN > seq_k) || (causal && (kv0 + BN - 1 > m0 + i * Cfg::BM));
        const uint32_t t_s = tmem_base + (i == 0 ? Cfg::kColS0 : Cfg::kColS1) + lane_base;
        const uint32_t t_o = tmem_base + (i == 0 ? Cfg::kColO0 : Cfg::kColO1) + lane_base;
        float* x = xchg + (((j & 1) * 2 + i) * 2) * 128 + r;
        // Called on every step but the first with this step's factor: rescale O if any row of the
        // warp moved its offset, then tell the MMA warp that O may be accumulated into.
        auto rescale_o = [&](float alpha) {
          if (__any_sync(0xffffffffu, alpha != 1.f)) {
            mbar_wait(o_full + i, (j - 1) & 1, abort_flag, 0x311 + i, j);
            tc_fence_after_sync();
#pragma unroll
            for (int c = 0; c < D / 32; ++c) {
              uint32_t orr[32];
              tmem_ld_x32(t_o + c * 32, orr);
              tmem_wait_ld();
#pragma unroll
              for (int q = 0; q < 32; ++q) orr[q] = __float_as_uint(__uint_as_float(orr[q]) * alpha);
              tmem_st_x32(t_o + c * 32, orr);
            }
            tmem_wait_st();
            tc_fence_before_sync();
          }
          __syncwarp();
          if (lane == 0) mbar_arrive(o_rescaled + i);
        };
        softmax_part_tile<BN, KA, BN - KA, true, Cfg::kChunksA>(t_s, p_full + i * Cfg::kPChunks, rescale_o, x + 128, x,
                                                                 2 + i, j == 0, need_mask, kv0, m0 + i * Cfg::BM + r,
                                                                 seq_k, causal, scale_log2, lane, m_ref, l_part);
      };
      for (int j = 0; j < n_max; ++j) {
        if (j < n_t0) helper_step(SmInt<0>{}, j, m_help0, l_help0);
        if (j < n_t1) helper_step(SmInt<1>{}, j, m_help1, l_help1);
      }
    }
    for (int j = 1; j < (Cfg::kHelper ? 0 : n_max); ++j) {
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
    // Epilogue (variants with several softmax threads per row; with one thread per row the softmax
    // groups write their own tiles): row sums and offsets come through shared memory.
    if constexpr (SPLIT != 1) {
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        const int n_i = i ? n_t1 : n_t0;
        if (n_i > 0) {
          const uint32_t ph = (n_i - 1) & 1;
          // corr_ready completes once per published alpha and once for the final row sum; in the helper
          // variant only the latter happens
          mbar_wait(corr_ready + i, Cfg::kHelper ? 0u : ph, abort_flag, 0x321 + i, n_i);
          const float l = l_buf[i * 128 + r] + (Cfg::kHelper ? (i ? l_help1 : l_help0) : 0.f);
          mbar_wait(o_full + i, ph, abort_flag, 0x331 + i, n_i);
          tc_fence_after_sync();
          if (r == 0) FRAY_TRACE(6, 1, i);  // last P.V of tile i complete, epilogue starts
          epilogue_tile<Cfg, D>(tmem_base + (i == 0 ? Cfg::kColO0 : Cfg::kColO1) + lane_base,
                                q_smem + i * Cfg::kQTileBytes, r, l, m_buf[i * 128 + r], &tm_o, m0 + i * Cfg::BM, h, b,
                                num_heads, seq_len, scale_log2, lse, 1);
        }
      }
      if (r == 0) {
        FRAY_TRACE(6, 1, 2);  // stores issued
        tma_store_wait_read();  // shared memory may go once the copies have read it; the writes finish on their own
        FRAY_TRACE(6, 1, 3);
      }
    }
  } else {
    set_max_regs_dec<Cfg::kRegsOther>();
    if (role == 13 && lane == 0) {  // second warp of the last warpgroup
      // ============================================================= TMA producer
      // ring entries 0 and 1 and both Q tiles were issued during set-up (unless that is switched off)
      auto late_q = [&](int i) __attribute__((always_inline)) {
        if ((i ? n_t1 : n_t0) > 0) {
          mbar_expect_tx(q_full + i, Cfg::kQTileBytes);
#pragma unroll
          for (int p = 0; p < Cfg::kPanels; ++p)
            tma_load_4d(q_smem + i * Cfg::kQTileBytes + p * Cfg::kQPanelBytes, &tm_q, q_full + i, p * 64,
                        m0 + i * Cfg::BM, h, b);
        }
      };
      if (!kEarlyCopies) {
        late_q(0);
      }
      for (int t = kEarlyCopies ? 2 : 0; t < 2 * n_max; ++t) {
        const int slot = t % STAGES;
        const uint32_t ph = (t / STAGES) & 1;
        mbar_wait(kv_empty + slot, ph ^ 1, abort_flag, 0x401, t);
        mbar_expect_tx(kv_full + slot, Cfg::kKVTileBytes);
        const CUtensorMap* tm = (t & 1) ? &tm_v : &tm_k;
#pragma unroll
        for (int p = 0; p < Cfg::kPanels; ++p)
          tma_load_4d(kv_smem + slot * Cfg::kKVTileBytes + p * Cfg::kKVPanelBytes, tm, kv_full + slot, p * 64,
                      (t >> 1) * BN, h_kv, b);
        if (!kEarlyCopies && t == 0) late_q(1);
      }
    } else if (role == 12) {
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
        int kk = 0;  // MMA (16 keys) inside the step; a compile-time value after unrolling
#pragma unroll
        for (int q = 0; q < Cfg::kPChunks; ++q) {
          FRAY_CRIT_WAIT(p_full + i * Cfg::kPChunks + q, j & 1, abort_flag, 0x503 + i, j);
          tc_fence_after_sync();
          if (q == 0) FRAY_TRACE(5, i, j);
#pragma unroll
          for (int s2 = 0; s2 < Cfg::chunk_steps(q); ++s2, ++kk)
            mma_ts_elect_lohi(t_o, t_p + kk * 8, v_lo + ((kk * 2048) >> 4), kDescVHi, kIdescPV, (j > 0 || kk > 0));
        }
        mma_commit_elect(o_full + i);
        if ((i == 1) || !(j < n1)) mma_commit_elect(kv_empty + slot);
        FRAY_TRACE(7, i, j);
      };

      if constexpr (FRAY_COMPACT_MMA_ROLE != 0 && SPLIT == 1) {
      // One copy of each issue sequence, the tile index a run-time value: the kernels are sensitive
      // to instruction fetch, and this role's code is otherwise there once per tile and call site.
      // (One thread per row only: the 768-thread split-row variant, whose MMA warp has 56 registers,
      // stopped making progress with it - bounded waits, status 0x302 - and was left as it was.)
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
      } else {
      if (n0 > 0) {
        mbar_wait(q_full + 0, 0, abort_flag, 0x511);
        issue_qk(0, 0);
      }
      if (n1 > 0) {
        mbar_wait(q_full + 1, 0, abort_flag, 0x512);
        issue_qk(1, 0);
      }
      for (int j = 0; j < n_max; ++j) {
        if (j < n0) {
          issue_pv(0, j);
          if (j + 1 < n0) issue_qk(0, j + 1);
        }
        if (j < n1) {
          issue_pv(1, j);
          if (j + 1 < n1) issue_qk(1, j + 1);
        }
      }
      }
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem_base, Cfg::kTmemCols);
#ifdef FRAY_ATTN_TRACE
  if (tid == 0) FRAY_TRACE(6, 0, 2);  // CTA exit
  __syncthreads();
  if (trace_on)
    for (int w = tid; w < kTraceWords; w += Cfg::kThreads) fray_attn_trace_buf[w] = trace_sm[w];
#endif
}

// Host launcher for the warp-specialised kernel. Returns an AttnReturnCode.
template <int D, int BN, int STAGES, int POLY, int SPLIT = 1, int KA = 64>
inline int launch_attn_fwd_ws(const operand_t* q, const operand_t* k, const operand_t* v, operand_t* o, const AttnShape& shp,
                              const AttnStrides (&st)[4], const AttnExtras& ex, bool causal, float scale,
                              cudaStream_t stream) {
  using Cfg = WsCfg<D, BN, STAGES, SPLIT, KA>;
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

  static_assert((POLY >= 0 && POLY <= 4) || POLY == kExpPackedHalf, "POLY: 0..4 polynomial pairs of 4, or 16 = packed fp16");
  auto kernel = attn_fwd_ws_kernel<D, BN, STAGES, POLY, SPLIT, KA>;
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
