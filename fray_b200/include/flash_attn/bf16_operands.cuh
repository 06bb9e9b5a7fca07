#pragma once
// Included ahead of the attention headers to build a library whose Q, K, V and O are bf16 instead of fp16
// (P is then rounded to bf16 as well; scores, row sums and the O accumulator stay fp32).
#define FRAY_ATTN_BF16 1
