#pragma once
// Entry points the JIT-generated `launch` bodies call for the attention forward path.
// Replaces fray::flash_attn_cute<R,C,D> (fray/include/flash_attn/flashattn_cute.cuh:166-239):
// same fp16 [B,H,S,D] operands and in-place output, plus explicit strides, an optional
// causal mask and an explicit softmax scale.

#include "fwd_simple_sm100.cuh"
#include "host_sm100.cuh"
#include "fwd_ws_sm100.cuh"
#include "fwd_wsh_sm100.cuh"
#include "fwd_ws3_sm100.cuh"

namespace fray {

// Kernel families selectable from the tuning space.
enum AttnKernelKind : int {
  kAttnSimple = 0,  // one 128-row tile per CTA, single role, no overlap
  kAttnWarpSpecialized = 1,  // two 128-row tiles per CTA, producer / MMA / softmax / correction roles
  kAttnSplitRow = 3,         // the warp-specialised kernel with two softmax threads per query row (24 warps)
  kAttnHelper = 4,           // the warp-specialised kernel whose correction group takes a share of every row
  kAttnHalfStep = 5,         // warp-specialised, softmax steps of 64 keys in two alternating score buffers per tile
  kAttnThreeBuffers = 6,     // one 128-row tile per CTA, three score buffers, two softmax groups on alternate KV steps
  kAttnPaired = 7,           // the same on a pair of CTAs (cta_group::2): 256 rows per pair, half of K and V per CTA
};

// KIND, D, BLOCK_N, STAGES, POLY are compile-time tuning keys (POLY: how many of every four
// element pairs evaluate exp2 by polynomial instead of the special-function unit; used by the
// warp-specialised kernel only); everything else is a run-time argument.  K and V have num_kv_heads heads
// (a divisor of num_heads; query head h uses K/V head h / (num_heads / num_kv_heads)) and seq_len_kv rows
// (seq_len is the number of queries); lse is null or an
// fp32 [B, H, S] array that receives the log-sum-exp of every query row.  `rc` receives an
// AttnReturnCode; a non-zero value means nothing was launched.
template <int KIND, int D, int BLOCK_N, int STAGES, int POLY = 0>
inline void flash_attn_sm100(const operand_t* q, const operand_t* k, const operand_t* v, operand_t* o, int batch_size,
                             int num_heads, int seq_len, int q_sb, int q_sh, int q_ss, int k_sb, int k_sh, int k_ss,
                             int v_sb, int v_sh, int v_ss, int o_sb, int o_sh, int o_ss, int num_kv_heads,
                             int seq_len_kv, float* lse, bool causal, float scale, cudaStream_t stream, int& rc) {
  const AttnShape shp{batch_size, num_heads, seq_len, D};
  const bool bad_shape = num_kv_heads <= 0 || num_heads % num_kv_heads != 0 || seq_len_kv <= 0;
  if (bad_shape || (reinterpret_cast<uintptr_t>(lse) & 3u) != 0) {
    rc = bad_shape ? kAttnBadShape : kAttnBadPointer;
    return;
  }
  const AttnExtras ex{num_heads / num_kv_heads, lse, seq_len_kv};
  const AttnStrides st[4] = {{q_sb, q_sh, q_ss}, {k_sb, k_sh, k_ss}, {v_sb, v_sh, v_ss}, {o_sb, o_sh, o_ss}};
  rc = validate_attn_args(q, k, v, o, shp, st);
  if (rc != kAttnOk) return;
  if constexpr (KIND == kAttnSimple) {
    rc = sm100::launch_attn_fwd_simple<D, BLOCK_N>(q, k, v, o, shp, st, ex, causal, scale, stream);
  } else if constexpr (KIND == kAttnWarpSpecialized) {
    rc = sm100::launch_attn_fwd_ws<D, BLOCK_N, STAGES, POLY>(q, k, v, o, shp, st, ex, causal, scale, stream);
  } else if constexpr (KIND == kAttnSplitRow) {
    // POLY picks how a row is divided: 0 = 64 + 64 keys, both on the special-function unit;
    // 1 = 80 + 48 and 2 = 96 + 32 keys with the smaller part on the polynomial.
    static_assert(POLY >= 0 && POLY <= 2, "split-row kernel: POLY is 0, 1 or 2");
    rc = sm100::launch_attn_fwd_ws<D, BLOCK_N, STAGES, 0, 2, (POLY == 0 ? 64 : POLY == 1 ? 80 : 96)>(
        q, k, v, o, shp, st, ex, causal, scale, stream);
  } else if constexpr (KIND == kAttnHelper) {
    // POLY picks the share: 1 = keys [80,128), 2 = keys [96,128) of every tile go to the helper.
    static_assert(POLY == 1 || POLY == 2, "helper kernel: POLY is 1 or 2");
    rc = sm100::launch_attn_fwd_ws<D, BLOCK_N, STAGES, 0, 3, (POLY == 1 ? 80 : 96)>(q, k, v, o, shp, st, ex, causal,
                                                                                 scale, stream);
  } else if constexpr (KIND == kAttnHalfStep) {
    rc = sm100::launch_attn_fwd_wsh<D, STAGES>(q, k, v, o, shp, st, ex, causal, scale, stream);
  } else if constexpr (KIND == kAttnThreeBuffers) {
    rc = sm100::launch_attn_fwd_ws3<D, STAGES, 1>(q, k, v, o, shp, st, ex, causal, scale, stream);
  } else {
    static_assert(KIND == kAttnPaired, "unknown kernel kind");
    rc = sm100::launch_attn_fwd_ws3<D, STAGES, 2>(q, k, v, o, shp, st, ex, causal, scale, stream);
  }
}

}  // namespace fray
