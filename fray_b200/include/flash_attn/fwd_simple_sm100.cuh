#pragma once
// Single-role attention forward for sm_100a: one CTA of 128 threads per 128-row query
// tile, thread r owns query row r. One thread issues the TMA loads and the tcgen05 MMAs;
// all threads run the base-2 online softmax out of tensor memory. Nothing overlaps - this
// variant exists as the small, easy-to-audit member of the tuning space and as the
// bring-up path for the descriptors the warp-specialised kernel shares.
//
// Arithmetic follows the reference path (fray/include/flash_attn/softmax.cuh:24-81,
// flashattn_cute.cuh:104,134,153-158): S = Q.K^T in fp32, running max m, rescale by
// exp2((m_old-m_new)*scale*log2e) every KV tile, P = exp2(S*c - m*c) summed in fp32 but
// rounded to fp16 for the P.V product, O normalised by 1/l and rounded to fp16.

#include "host_sm100.cuh"
#include "sm100_ptx.cuh"

namespace fray {
namespace sm100 {

template <int D, int BN>
struct SimpleCfg {
  static_assert(D == 64 || D == 128, "head dim must be 64 or 128");
  static_assert(BN == 64 || BN == 128, "kv tile must be 64 or 128");
  static constexpr int BM = 128;
  static constexpr int kHalves = D / 64;           // 64-element (128-byte) column panels
  static constexpr int kQPanelBytes = BM * 128;    // one panel of the Q tile
  static constexpr int kKVPanelBytes = BN * 128;   // one panel of a K or V tile
  static constexpr int kQBytes = kHalves * kQPanelBytes;
  static constexpr int kKVBytes = kHalves * kKVPanelBytes;
  static constexpr int kBarOffset = kQBytes + 2 * kKVBytes;
  static constexpr int kSmemBytes = kBarOffset + 128 + 1024;  // + barriers/flags + alignment slack
  static constexpr int kTmemCols = 256;
  static constexpr int kColS = 0;    // S (fp32) and, after the softmax, P (fp16 pairs)
  static constexpr int kColO = 128;  // O accumulator (fp32), D columns
};

template <int D, int BN>
__global__ void __launch_bounds__(128, 1)
attn_fwd_simple_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                       const __grid_constant__ CUtensorMap tm_v, operand_t* __restrict__ o_ptr, int64_t o_sb,
                       int64_t o_sh, int64_t o_ss, int num_heads, int seq_len, int causal, float scale_log2,
                       int kv_group, float* lse, int seq_k) {
  using Cfg = SimpleCfg<D, BN>;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  uint8_t* smem = smem_raw + (((raw_addr + 1023u) & ~1023u) - raw_addr);
  uint8_t* q_smem = smem;
  uint8_t* k_smem = smem + Cfg::kQBytes;
  uint8_t* v_smem = k_smem + Cfg::kKVBytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Cfg::kBarOffset);
  uint64_t* bar_q = bars + 0;
  uint64_t* bar_k = bars + 1;
  uint64_t* bar_v = bars + 2;
  uint64_t* bar_s = bars + 3;
  uint64_t* bar_o = bars + 4;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 8);
  volatile uint32_t* abort_flag = reinterpret_cast<volatile uint32_t*>(bars + 9);

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  // Causal work grows with the tile index: hand the heaviest tiles out first.
  const int m_tile = causal ? (gridDim.x - 1 - blockIdx.x) : blockIdx.x;
  const int m0 = m_tile * Cfg::BM;
  const int bh = blockIdx.y;
  const int b = bh / num_heads;
  const int h = bh - b * num_heads;
  const int h_kv = h / kv_group;  // K/V head of this query head (one division per CTA, not per copy)

  if (tid == 0) {
    *abort_flag = (*reinterpret_cast<volatile int*>(&fray_attn_status[0]) != 0) ? 2u : 0u;
    mbar_init(bar_q, 1);
    mbar_init(bar_k, 1);
    mbar_init(bar_v, 1);
    mbar_init(bar_s, 1);
    mbar_init(bar_o, 1);
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
  const uint32_t lane_base = static_cast<uint32_t>(warp * 32) << 16;
  const uint32_t t_s = tmem_base + Cfg::kColS;
  const uint32_t t_o = tmem_base + Cfg::kColO;

  int n_tiles = (seq_k + BN - 1) / BN;  // seq_len counts queries, seq_k keys
  if (causal) {
    const int lim = (m0 + Cfg::BM + BN - 1) / BN;
    n_tiles = lim < n_tiles ? lim : n_tiles;
  }

  constexpr uint64_t kDescK = smem_desc_sw128(16, 1024);                  // K-major operand (Q, K)
  constexpr uint64_t kDescV = smem_desc_sw128(Cfg::kKVPanelBytes, 1024);  // MN-major operand (V)
  constexpr uint32_t kIdescQK = idesc_f16_f32(Cfg::BM, BN, false, false);
  constexpr uint32_t kIdescPV = idesc_f16_f32(Cfg::BM, D, false, true);

  if (tid == 0) {
    mbar_expect_tx(bar_q, Cfg::kQBytes);
#pragma unroll
    for (int p = 0; p < Cfg::kHalves; ++p) tma_load_4d(q_smem + p * Cfg::kQPanelBytes, &tm_q, bar_q, p * 64, m0, h, b);
  }

  const int row = m0 + tid;
  float m_run = -INFINITY;
  float l_run = 0.f;

  for (int j = 0; j < n_tiles; ++j) {
    const uint32_t ph = static_cast<uint32_t>(j & 1);
    if (tid == 0) {
      mbar_expect_tx(bar_k, Cfg::kKVBytes);
#pragma unroll
      for (int p = 0; p < Cfg::kHalves; ++p)
        tma_load_4d(k_smem + p * Cfg::kKVPanelBytes, &tm_k, bar_k, p * 64, j * BN, h_kv, b);
      mbar_expect_tx(bar_v, Cfg::kKVBytes);
#pragma unroll
      for (int p = 0; p < Cfg::kHalves; ++p)
        tma_load_4d(v_smem + p * Cfg::kKVPanelBytes, &tm_v, bar_v, p * 64, j * BN, h_kv, b);
      if (j == 0) mbar_wait(bar_q, 0, abort_flag, 0x101);
      mbar_wait(bar_k, ph, abort_flag, 0x102, j);
      tc_fence_after_sync();
      // S = Q . K^T : D/16 MMAs of K=16, each advancing 32 bytes inside the swizzle span.
#pragma unroll
      for (int kk = 0; kk < D / 16; ++kk) {
        const uint32_t off = (kk >> 2) * Cfg::kQPanelBytes + (kk & 3) * 32;
        const uint32_t offk = (kk >> 2) * Cfg::kKVPanelBytes + (kk & 3) * 32;
        mma_ss(t_s, smem_desc_at(kDescK, smem_u32(q_smem) + off), smem_desc_at(kDescK, smem_u32(k_smem) + offk),
               kIdescQK, kk > 0);
      }
      mma_commit(bar_s);
    }

    mbar_wait(bar_s, ph, abort_flag, 0x103, j);
    tc_fence_after_sync();

    uint32_t sr[BN];
#pragma unroll
    for (int c = 0; c < BN / 32; ++c) tmem_ld_x32(t_s + lane_base + c * 32, reinterpret_cast<uint32_t(&)[32]>(sr[c * 32]));
    tmem_wait_ld();

    const int kv0 = j * BN;
    const bool need_mask = (kv0 + BN > seq_k) || (causal && (kv0 + BN - 1 > m0));
    if (need_mask) {
#pragma unroll
      for (int c = 0; c < BN; ++c) {
        const int kv = kv0 + c;
        if (kv >= seq_k || (causal && kv > row)) sr[c] = __float_as_uint(-INFINITY);
      }
    }
    float mx = -INFINITY;
#pragma unroll
    for (int c = 0; c < BN; ++c) mx = fmaxf(mx, __uint_as_float(sr[c]));
    const float m_new = fmaxf(m_run, mx);
    const float alpha = (m_new == -INFINITY) ? 0.f : ex2_approx((m_run - m_new) * scale_log2);
    const float m_sc = (m_new == -INFINITY) ? 0.f : m_new * scale_log2;
    m_run = m_new;

    uint32_t pk[BN / 2];
    float rs = 0.f;
#pragma unroll
    for (int c = 0; c < BN; c += 2) {
      const float p0 = ex2_approx(fmaf(__uint_as_float(sr[c]), scale_log2, -m_sc));
      const float p1 = ex2_approx(fmaf(__uint_as_float(sr[c + 1]), scale_log2, -m_sc));
      rs += p0 + p1;
      pk[c >> 1] = pack_half2(p0, p1);
    }
    l_run = l_run * alpha + rs;

    if (j > 0) {
#pragma unroll
      for (int c = 0; c < D / 32; ++c) {
        uint32_t orr[32];
        tmem_ld_x32(t_o + lane_base + c * 32, orr);
        tmem_wait_ld();
#pragma unroll
        for (int i = 0; i < 32; ++i) orr[i] = __float_as_uint(__uint_as_float(orr[i]) * alpha);
        tmem_st_x32(t_o + lane_base + c * 32, orr);
      }
    }
#pragma unroll
    for (int c = 0; c < BN / 64; ++c) tmem_st_x32(t_s + lane_base + c * 32, reinterpret_cast<uint32_t(&)[32]>(pk[c * 32]));
    tmem_wait_st();
    tc_fence_before_sync();
    __syncthreads();

    if (tid == 0) {
      tc_fence_after_sync();
      mbar_wait(bar_v, ph, abort_flag, 0x104, j);
      // O += P . V : P is the A operand straight from tensor memory (8 columns per K=16),
      // V is the MN-major B operand (16 kv rows = 2048 bytes per step).
#pragma unroll
      for (int kk = 0; kk < BN / 16; ++kk) {
        mma_ts(t_o, t_s + kk * 8, smem_desc_at(kDescV, smem_u32(v_smem) + kk * 2048), kIdescPV, (j > 0 || kk > 0));
      }
      mma_commit(bar_o);
    }
    mbar_wait(bar_o, ph, abort_flag, 0x105, j);
    tc_fence_after_sync();
  }

  // Epilogue: O / l -> fp16 -> global, 16 bytes per store.
  const float inv_l = l_run > 0.f ? 1.f / l_run : 1.f;
  if (lse != nullptr && row < seq_len)
    lse[(static_cast<size_t>(b) * num_heads + h) * seq_len + row] =
        l_run > 0.f ? (m_run * scale_log2 + log2f(l_run)) * 0.69314718055994531f : -INFINITY;
  operand_t* o_row = o_ptr + static_cast<int64_t>(b) * o_sb + static_cast<int64_t>(h) * o_sh +
                  static_cast<int64_t>(row) * o_ss;
#pragma unroll
  for (int c = 0; c < D / 32; ++c) {
    uint32_t orr[32];
    tmem_ld_x32(t_o + lane_base + c * 32, orr);
    tmem_wait_ld();
    if (row < seq_len) {
#pragma unroll
      for (int i = 0; i < 32; i += 8) {
        uint4 v4;
        v4.x = pack_half2(__uint_as_float(orr[i + 0]) * inv_l, __uint_as_float(orr[i + 1]) * inv_l);
        v4.y = pack_half2(__uint_as_float(orr[i + 2]) * inv_l, __uint_as_float(orr[i + 3]) * inv_l);
        v4.z = pack_half2(__uint_as_float(orr[i + 4]) * inv_l, __uint_as_float(orr[i + 5]) * inv_l);
        v4.w = pack_half2(__uint_as_float(orr[i + 6]) * inv_l, __uint_as_float(orr[i + 7]) * inv_l);
        *reinterpret_cast<uint4*>(o_row + c * 32 + i) = v4;
      }
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem_base, Cfg::kTmemCols);
}

// Host launcher for the single-role kernel. Returns an AttnReturnCode.
template <int D, int BN>
inline int launch_attn_fwd_simple(const operand_t* q, const operand_t* k, const operand_t* v, operand_t* o, const AttnShape& shp,
                                  const AttnStrides (&st)[4], const AttnExtras& ex, bool causal, float scale,
                                  cudaStream_t stream) {
  using Cfg = SimpleCfg<D, BN>;
  const AttnShape shp_kv{shp.B, shp.H / ex.kv_group, ex.seq_k, shp.D};
  CUtensorMap tm_q, tm_k, tm_v;
  int rc = cached_attn_tensor_map(&tm_q, q, shp, st[0], Cfg::BM);
  if (rc != kAttnOk) return rc;
  rc = cached_attn_tensor_map(&tm_k, k, shp_kv, st[1], BN);
  if (rc != kAttnOk) return rc;
  rc = cached_attn_tensor_map(&tm_v, v, shp_kv, st[2], BN);
  if (rc != kAttnOk) return rc;

  auto kernel = attn_fwd_simple_kernel<D, BN>;
  rc = ensure_dynamic_smem<Cfg>(kernel, Cfg::kSmemBytes);
  if (rc != kAttnOk) return rc;
  dim3 grid((shp.S + Cfg::BM - 1) / Cfg::BM, shp.B * shp.H);
  kernel<<<grid, 128, Cfg::kSmemBytes, stream>>>(tm_q, tm_k, tm_v, o, st[3].b, st[3].h, st[3].s, shp.H, shp.S,
                                                 causal ? 1 : 0, scale * 1.44269504088896340736f, ex.kv_group, ex.lse, ex.seq_k);
  if (cudaGetLastError() != cudaSuccess) return kAttnLaunchFailed;
  return kAttnOk;
}

}  // namespace sm100
}  // namespace fray
