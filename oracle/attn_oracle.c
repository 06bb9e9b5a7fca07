/* CPU oracle for the attention forward path, plain C.  TEST INFRASTRUCTURE ONLY: only
 * tests, the smoke check and the benchmark's CPU-baseline leg may load this library.
 *
 * It restates, one query row at a time, the arithmetic of the reference kernel:
 *   - S = q.k in fp32                                  (flashattn_cute.cuh:120-121)
 *   - c = scale * log2(e)                              (flashattn_cute.cuh:104)
 *   - per KV tile of `block_n` keys: m_new = max(m, max S); alpha = exp2((m - m_new) c),
 *     0 while m_new is -inf; l and O are multiplied by alpha; P = exp2(S c - m_new c);
 *     l += sum P (unrounded fp32)                      (flash_attn/softmax.cuh:24-67)
 *   - P is rounded to fp16 before O += P.V             (flashattn_cute.cuh:134-138)
 *   - O *= 1/l (1 when l <= 0), rounded to fp16        (softmax.cuh:70-81, flashattn_cute.cuh:153-158)
 * plus the causal extension (key j visible to query i iff j <= i).
 *
 * Pinning: the reference has no golden vectors for this path; this file is checked in
 * tests against torch CPU attention (the oracle of the reference's own test,
 * tests/test_flashattn_cute.py:24) and the committed fixtures under tests/golden/.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

typedef _Float16 f16;

static float h2f(uint16_t bits) { f16 h; memcpy(&h, &bits, 2); return (float)h; }
static uint16_t f2h(float x) { f16 h = (f16)x; uint16_t bits; memcpy(&bits, &h, 2); return bits; }

/* Tensors are fp16 bit patterns; strides are in elements, the D stride is 1.  Rows are
 * numbered (b*H + h)*S + i; the call handles rows [row_begin, row_end) so that a host can
 * spread one problem over threads (no OpenMP runtime is assumed).
 * Returns 0, or 1 for bad arguments. */
int fray_oracle_attn_fwd(const uint16_t* q, const uint16_t* k, const uint16_t* v, uint16_t* o, int B, int H, int S,
                         int D, const int64_t* q_st, const int64_t* k_st, const int64_t* v_st, const int64_t* o_st,
                         int causal, float scale, int block_n, long row_begin, long row_end) {
    if (B <= 0 || H <= 0 || S <= 0 || D <= 0 || block_n <= 0) return 1;
    const float c = scale * 1.44269504088896340736f;
    const long total_rows = (long)B * H * S;
    if (row_begin < 0 || row_end > total_rows || row_begin > row_end) return 1;
    {
        float* kf = (float*)malloc(sizeof(float) * (size_t)block_n * D);
        float* vf = (float*)malloc(sizeof(float) * (size_t)block_n * D);
        float* qf = (float*)malloc(sizeof(float) * D);
        float* acc = (float*)malloc(sizeof(float) * D);
        float* s = (float*)malloc(sizeof(float) * block_n);
        for (long r = row_begin; r < row_end; ++r) {
            const int i = (int)(r % S);
            const int h = (int)((r / S) % H);
            const int b = (int)(r / ((long)S * H));
            const uint16_t* qrow = q + b * q_st[0] + h * q_st[1] + i * q_st[2];
            for (int d = 0; d < D; ++d) { qf[d] = h2f(qrow[d]); acc[d] = 0.f; }
            float m = -INFINITY, l = 0.f;
            const int kv_end = causal ? (i + 1) : S;
            for (int j0 = 0; j0 < kv_end; j0 += block_n) {
                const int n = (j0 + block_n <= S ? block_n : S - j0);
                float mx = -INFINITY;
                for (int jj = 0; jj < n; ++jj) {
                    const int j = j0 + jj;
                    const uint16_t* krow = k + b * k_st[0] + h * k_st[1] + (int64_t)j * k_st[2];
                    const uint16_t* vrow = v + b * v_st[0] + h * v_st[1] + (int64_t)j * v_st[2];
                    float dot = 0.f;
                    for (int d = 0; d < D; ++d) { kf[jj * D + d] = h2f(krow[d]); vf[jj * D + d] = h2f(vrow[d]); }
                    for (int d = 0; d < D; ++d) dot += qf[d] * kf[jj * D + d];
                    s[jj] = (causal && j > i) ? -INFINITY : dot;
                    if (s[jj] > mx) mx = s[jj];
                }
                const float m_new = mx > m ? mx : m;
                const float alpha = isinf(m_new) ? 0.f : exp2f((m - m_new) * c);
                const float m_sc = isinf(m_new) ? 0.f : m_new * c;
                l *= alpha;
                for (int d = 0; d < D; ++d) acc[d] *= alpha;
                for (int jj = 0; jj < n; ++jj) {
                    const float p = exp2f(s[jj] * c - m_sc);
                    l += p;
                    const float p16 = h2f(f2h(p));
                    if (p16 != 0.f)
                        for (int d = 0; d < D; ++d) acc[d] += p16 * vf[jj * D + d];
                }
                m = m_new;
            }
            const float inv = l > 0.f ? 1.f / l : 1.f;
            uint16_t* orow = o + b * o_st[0] + h * o_st[1] + i * o_st[2];
            for (int d = 0; d < D; ++d) orow[d] = f2h(acc[d] * inv);
        }
        free(kf); free(vf); free(qf); free(acc); free(s);
    }
    return 0;
}
