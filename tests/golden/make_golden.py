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


if __name__ == "__main__":
    main()
