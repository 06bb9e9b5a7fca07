/* C ABI of one built attention kernel library (kernel.so).
 *
 * Every library produced by the JIT for `flash_attn_cute` exports the symbols below with
 * C linkage.  They replace what the reference runtime binds through ctypes
 * (fray/jit/runtime.py:30-68): a single `launch` whose prototype is generated from the
 * op's argument table (fray/jit/template.py:130-149, fray/jit_kernels/flashattn_cute.py:40).
 * All pointers are plain device or host addresses; no framework types cross the boundary.
 * The caller owns every buffer; the library allocates nothing and keeps no pointers.
 */
#ifndef FRAY_B200_ATTN_H_
#define FRAY_B200_ATTN_H_

#ifdef __cplusplus
extern "C" {
#endif

/* Queue the attention forward  O = softmax(scale * Q K^T [+ causal mask]) V  on `stream`.
 *
 * Replaces: launch(void* Q, void* K, void* V, void* O, int batch_size, int num_heads,
 *                  int seq_len, void* stream, int& __return_code)
 * generated for fray::flash_attn_cute<R,C,D> (fray/include/flash_attn/flashattn_cute.cuh:166-239).
 * Added over the reference prototype: element strides of the batch, head and sequence
 * modes of each tensor (the head-dim stride is 1), the number of K/V heads and rows, an optional
 * log-sum-exp output, the causal flag and the softmax scale, which the reference fixed to
 * contiguous / num_heads / none / false / 1/sqrt(D).
 *
 * Q, O         fp16 (bf16 in a bf16 library, see fray_attn_operand_is_bf16) device pointers, 16-byte aligned, logical shape [batch, num_heads, seq, D]
 *              where D is the head dim the library was built for (fray_attn_kernel_info).
 * K, V         the same with num_kv_heads heads and seq_len_kv rows; num_kv_heads divides
 *              num_heads and query head h reads K/V head h / (num_heads / num_kv_heads).
 *              seq_len counts the queries (rows of Q, O and Lse).  With causal != 0 query i
 *              sees keys 0..i whatever the two lengths are.
 * *_stride_*   in elements, positive multiples of 8 (ignored for modes of extent 1 of that tensor).
 * scale        positive and finite.  batch_size * num_heads is at most 65535.
 * Lse          null, or a 4-byte aligned device pointer to fp32 [batch, num_heads, seq]
 *              (contiguous) that receives log(sum_j exp(scale * q_i . k_j)) of every row.
 * stream       a cudaStream_t; the call returns once the kernel is queued.
 * __return_code receives 0 when the kernel was queued, otherwise (nothing launched):
 *              1 bad shape (a count not positive, batch * heads above 65535, num_kv_heads not a
 *              divisor of num_heads, scale not positive and finite), 2 bad pointer, 3 bad stride,
 *              5 driver entry point missing, 6 tensor map rejected, 7 shared-memory attribute
 *              failed, 8 launch failed.
 */
void launch(void* Q, void* K, void* V, void* O, int batch_size, int num_heads, int seq_len,
            int q_stride_b, int q_stride_h, int q_stride_s, int k_stride_b, int k_stride_h, int k_stride_s,
            int v_stride_b, int v_stride_h, int v_stride_s, int o_stride_b, int o_stride_h, int o_stride_s,
            int num_kv_heads, int seq_len_kv, void* Lse, bool causal, float scale, void* stream,
            int* __return_code);

/* Blocking read of the sticky device status: out4[0] is 0 when healthy, else the code of
 * the first in-kernel wait that ran out; out4[1..3] are block x, block y and an iteration
 * index.  While out4[0] != 0 later launches of this library return without computing;
 * pass clear != 0 to reset.  Returns 0 or a cudaError_t value.
 * No counterpart in the reference, which never checks device-side errors
 * (fray/jit_kernels/tuner.py:45-50 only sees the always-zero return code). */
int fray_attn_status(int* out4, int clear);

/* out4 = {kernel kind (0 single-role, 1 two query tiles per CTA, 2 one tile per CTA with two softmax
 * groups on alternate KV steps, 3 the same on a CTA pair with 2-CTA MMA, 4 one tile per CTA with two
 * CTAs per SM, 5 kind 1 as a persistent grid), head dim D, KV tile length,
 * K/V pipeline stages} this library was instantiated with - the template keys the reference keeps only in the source text
 * (fray/jit_kernels/flashattn_cute.py:32-38). */
void fray_attn_kernel_info(int* out4);

/* 1 when Q, K, V and O of this library are bf16, 0 when they are fp16 (the reference is fp16 only:
 * fray/jit_kernels/flashattn_cute.py:19 asserts torch.half).  The prototype of `launch` is the same. */
int fray_attn_operand_is_bf16(void);

#ifdef __cplusplus
}
#endif
#endif /* FRAY_B200_ATTN_H_ */
