"""Regenerates the golden fixtures in this directory.

The reference holds no golden vectors for the attention path (its test seeds inputs on the
CUDA device), so the fixtures are produced by the reference's own test oracle - torch
attention (tests/test_flashattn_cute.py:24) - evaluated on CPU in fp32 on the seeded inputs
of oracle.attention_ref.make_slice, and stored as fp32 .npy files.  Inputs are not stored:
they are regenerated from the seed.

    python tests/golden/make_golden.py
"""
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
from oracle import attention_ref as ref  # noqa: E402

# name -> (config index, units, S override, causal)
CASES = {
    "c1_full": (0, range(4), None, False),
    "c1_causal": (0, range(4), None, True),
    "c2_unit0_rows": (1, range(1), None, False),
    "c5_stress_unit3": (4, range(3, 4), None, False),
    "ragged_s200_causal": (0, range(2), 200, True),
}


# Cases for the extensions: grouped K/V heads (torch attention with enable_gqa) and the log-sum-exp
# output (torch.logsumexp of the scaled, masked scores).  name -> (query heads, K/V heads, S, D, causal)
EXT_CASES = {
    "gqa_h8_kv2": (8, 2, 320, 128, False),
    "gqa_h4_kv1_causal": (4, 1, 200, 64, True),
}


def ext_inputs_for(case):
    h, h_kv, S, D, causal = EXT_CASES[case]
    g = torch.Generator().manual_seed(9000 + h * 100 + h_kv)
    q = torch.randn(1, h, S, D, generator=g).half()
    k, v = (torch.randn(1, h_kv, S, D, generator=g).half() for _ in range(2))
    return q, k, v, causal


def ext_reference(q, k, v, causal):
    """(attention output, row log-sum-exp), both fp32, from torch on CPU."""
    qf, kf, vf = q.float(), k.float(), v.float()
    out = torch.nn.functional.scaled_dot_product_attention(qf, kf, vf, is_causal=causal, enable_gqa=True)
    r = q.shape[1] // k.shape[1]
    s = (qf @ kf.repeat_interleave(r, dim=1).transpose(-1, -2)) / q.shape[-1] ** 0.5
    if causal:
        s = s.masked_fill(~torch.ones(s.shape[-2:], dtype=torch.bool).tril(), float("-inf"))
    return out, torch.logsumexp(s, dim=-1)


def inputs_for(case):
    ci, units, s_override, causal = CASES[case]
    q, k, v = ref.make_inputs(ci, units)
    if s_override:
        q, k, v = (t[:, :s_override].contiguous() for t in (q, k, v))
    return q, k, v, causal


def main():
    for case in CASES:
        q, k, v, causal = inputs_for(case)
        out = torch.nn.functional.scaled_dot_product_attention(q.float(), k.float(), v.float(), is_causal=causal)
        if case == "c2_unit0_rows":
            out = out[:, ::16]  # every 16th query row keeps the file small
        np.save(os.path.join(HERE, f"{case}.npy"), out.numpy().astype(np.float32))
        print(case, tuple(out.shape))
    for case in EXT_CASES:
        q, k, v, causal = ext_inputs_for(case)
        out, lse = ext_reference(q, k, v, causal)
        np.save(os.path.join(HERE, f"{case}.npy"), out[:, :, ::4].numpy().astype(np.float32))  # every 4th row
        np.save(os.path.join(HERE, f"{case}_lse.npy"), lse.numpy().astype(np.float32))
        print(case, tuple(out.shape), tuple(lse.shape))


if __name__ == "__main__":
    main()
