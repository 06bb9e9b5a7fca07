#pragma once
// Entry points the JIT-generated `launch` bodies call for the attention forward path.
// Replaces fray::flash_attn_cute<R,C,D> (fray/include/flash_attn/flashattn_cute.cuh:166-239):
// same fp16 [B,H,S,D] operands and in-place output, plus explicit strides, an optional
// causal mask and an explicit softmax scale.

#include "fwd_simple_sm100.cuh"
#include "host_sm100.cuh"
#include "fwd_ws_sm100.cuh"
#include "fwd_alt_sm100.cuh"
#include "fwd_one_sm100.cuh"
#include "fwd_pers_sm100.cuh"

namespace fray {

// Kernel families selectable from the tuning space.
enum AttnKernelKind : int {
  kAttnSimple = 0,           // one 128-row tile per CTA, single role, no overlap; two CTAs per SM
  kAttnWarpSpecialized = 1,  // two 128-row tiles per CTA, producer / MMA / softmax / correction roles
  kAttnAlternating = 2,        // one 128-row tile per CTA, scores and probabilities in separate tensor-memory buffers,
                             // two softmax groups on alternate KV steps
  kAttnPaired = 3,           // the same on a pair of CTAs (cta_group::2): 256 rows per pair, half of K and V per CTA
  kAttnOneTile = 4,          // one 128-row tile per CTA, producer / MMA / softmax roles, 256 tensor-memory columns:
                             // two CTAs per SM cover each other's start, end and softmax phases
  kAttnPersistent = 5,       // kind 1 as one CTA per SM that walks through the work items, the next item's first
                             // copies and scores behind the current item's last steps
};

// KIND, D, BLOCK_N, STAGES are compile-time tuning keys (BLOCK_N: KV tile of the single-role kernel, 128
// elsewhere; STAGES: K/V ring depth of kind 1, K ring depth of kinds 2 and 3); everything else is a
// run-time argument.  K and V have num_kv_heads heads
// (a divisor of num_heads; query head h uses K/V head h / (num_heads / num_kv_heads)) and seq_len_kv rows
// (seq_len is the number of queries); lse is null or an
// fp32 [B, H, S] array that receives the log-sum-exp of every query row.  `rc` receives an
// AttnReturnCode; a non-zero value means nothing was launched.
template <int KIND, int D, int BLOCK_N, int STAGES>
inline void flash_attn_sm100(const operand_t* q, const operand_t* k, const operand_t* v, operand_t* o, int batch_size,
                             int num_heads, int seq_len, int q_sb, int q_sh, int q_ss, int k_sb, int k_sh, int k_ss,
                             int v_sb, int v_sh, int v_ss, int o_sb, int o_sh, int o_ss, int num_kv_heads,
                             int seq_len_kv, float* lse, bool causal, float scale, cudaStream_t stream, int& rc) {
  const AttnShape shp{batch_size, num_heads, seq_len, D};
  const bool bad_shape = num_kv_heads <= 0 || num_heads % num_kv_heads != 0 || seq_len_kv <= 0 ||
                         !(scale > 0.f) || !(scale <= 3.0e38f);  // also false for NaN
  if (bad_shape || (reinterpret_cast<uintptr_t>(lse) & 3u) != 0) {
    rc = bad_shape ? kAttnBadShape : kAttnBadPointer;
    return;
  }
  const AttnExtras ex{num_heads / num_kv_heads, lse, seq_len_kv};
  const AttnStrides st[4] = {{q_sb, q_sh, q_ss}, {k_sb, k_sh, k_ss}, {v_sb, v_sh, v_ss}, {o_sb, o_sh, o_ss}};
  const AttnShape shp_kv{batch_size, num_kv_heads, seq_len_kv, D};
  rc = validate_attn_args(q, k, v, o, shp, shp_kv, st);
  if (rc != kAttnOk) return;
  if constexpr (KIND == kAttnSimple) {
    rc = sm100::launch_attn_fwd_simple<D, BLOCK_N>(q, k, v, o, shp, st, ex, causal, scale, stream);
  } else if constexpr (KIND == kAttnWarpSpecialized) {
    rc = sm100::launch_attn_fwd_ws<D, BLOCK_N, STAGES>(q, k, v, o, shp, st, ex, causal, scale, stream);
  } else if constexpr (KIND == kAttnAlternating) {
    rc = sm100::launch_attn_fwd_alt<D, STAGES, 1>(q, k, v, o, shp, st, ex, causal, scale, stream);
  } else if constexpr (KIND == kAttnOneTile) {
    rc = sm100::launch_attn_fwd_one<D, BLOCK_N, STAGES>(q, k, v, o, shp, st, ex, causal, scale, stream);
  } else if constexpr (KIND == kAttnPersistent) {
    rc = sm100::launch_attn_fwd_pers<D, BLOCK_N, STAGES>(q, k, v, o, shp, st, ex, causal, scale, stream);
  } else {
    static_assert(KIND == kAttnPaired, "unknown kernel kind");
    static_assert(D == 128, "the paired kernel is built for head dim 128");
    rc = sm100::launch_attn_fwd_alt<D, STAGES, 2>(q, k, v, o, shp, st, ex, causal, scale, stream);
  }
}

}  // namespace fray
