"""The CPU oracles agree with each other, with torch attention and with the golden fixtures."""
import importlib.util
import math
import os

import numpy as np
import pytest
import torch
import torch.nn.functional as F

from oracle import attention_ref as ref
from oracle.c_oracle import attn_fwd_c

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
_spec = importlib.util.spec_from_file_location("make_golden", os.path.join(GOLDEN, "make_golden.py"))
make_golden = importlib.util.module_from_spec(_spec)
_spec.loader.exec_module(make_golden)


@pytest.mark.parametrize("case", sorted(make_golden.CASES))
def test_oracles_match_golden(case):
    q, k, v, causal = make_golden.inputs_for(case)
    gold = torch.from_numpy(np.load(os.path.join(GOLDEN, f"{case}.npy")))
    step = 16 if case == "c2_unit0_rows" else 1
    c_out = attn_fwd_c(q.unsqueeze(0), k.unsqueeze(0), v.unsqueeze(0), causal)[0][:, ::step]
    t_out = ref.flash_fp16p(q, k, v, causal)[:, ::step]
    f32 = ref.attention_fp32(q, k, v, causal)[:, ::step]
    assert (f32 - gold).abs().max() < 1e-4                       # explicit fp32 math == torch SDPA fp32
    for out in (c_out, t_out):
        assert (out.float() - gold).abs().max() <= 1e-2          # fp16 criterion of the reference test
        assert ref.calc_diff(out, gold) <= 1e-5                  # calc_diff criterion
    assert (c_out.float() - t_out.float()).abs().max() <= 2e-3   # C and torch restatements agree


@pytest.mark.parametrize("case", sorted(make_golden.EXT_CASES))
def test_extension_oracles_match_golden(case):
    """Grouped K/V heads restated as head expansion, and the LSE reference, against the torch-made fixtures."""
    q, k, v, causal = make_golden.ext_inputs_for(case)
    gold = torch.from_numpy(np.load(os.path.join(GOLDEN, f"{case}.npy")))
    gold_lse = torch.from_numpy(np.load(os.path.join(GOLDEN, f"{case}_lse.npy")))
    ke, ve = ref.expand_kv_heads(k, v, q.shape[1])
    assert (ref.attention_fp32(q, ke, ve, causal)[:, :, ::4] - gold).abs().max() < 1e-4
    assert (ref.flash_fp16p(q, ke, ve, causal)[:, :, ::4].float() - gold).abs().max() <= 1e-2
    assert (ref.lse_fp32(q, ke, causal) - gold_lse).abs().max() < 1e-4


def test_c_oracle_matches_sdpa_fp16():
    q, k, v = ref.make_inputs(0)
    got = attn_fwd_c(q.unsqueeze(0), k.unsqueeze(0), v.unsqueeze(0))[0]
    want = ref.sdpa_cpu(q, k, v)
    assert (got.float() - want.float()).abs().max() <= 1e-3


@pytest.mark.parametrize("block_n", [32, 64, 128, 256])
def test_tile_size_does_not_change_the_answer(block_n):
    q, k, v = ref.make_inputs(0, range(2))
    a = attn_fwd_c(q.unsqueeze(0), k.unsqueeze(0), v.unsqueeze(0), True, block_n=block_n)[0]
    b = attn_fwd_c(q.unsqueeze(0), k.unsqueeze(0), v.unsqueeze(0), True, block_n=128)[0]
    assert (a.float() - b.float()).abs().max() <= 1e-3


def test_c_oracle_strided_and_scaled():
    q, k, v = ref.make_inputs(0)                       # [4, 256, 64]
    q_bshd = q.permute(1, 0, 2).contiguous()           # [S, H, D] storage
    q_view = q_bshd.permute(1, 0, 2).unsqueeze(0)      # [1, H, S, D] view, non-contiguous
    assert not q_view.is_contiguous()
    a = attn_fwd_c(q_view, k.unsqueeze(0), v.unsqueeze(0), scale=0.2)[0]
    b = ref.attention_fp32(q, k, v, scale=0.2)
    assert ref.calc_diff(a, b) <= 1e-5


def test_c_oracle_rejects_bad_row_range():
    import ctypes
    from oracle import c_oracle
    lib = c_oracle._load()
    z = (ctypes.c_int64 * 3)(1, 1, 1)
    assert lib.fray_oracle_attn_fwd(None, None, None, None, 0, 1, 1, 1, z, z, z, z, 0, ctypes.c_float(1.0), 128,
                                    ctypes.c_long(0), ctypes.c_long(0)) == 1


def test_stress_inputs_have_large_logits():
    q, k, v = ref.make_inputs(4, range(1))
    frac = (q.abs() == 16).float().mean().item()
    assert 0.005 < frac < 0.02 and q.abs().max() >= 16 and k.abs().max() >= 16
    s = (q[0].float() @ k[0].float().T) / 8.0
    assert s.max() > 60  # logits far beyond the fp16-safe exp range: rescaling must work


def test_inputs_are_reproducible_per_unit():
    a = ref.make_inputs(1, [5])[0]
    b = ref.make_inputs(1, range(4, 7))[0][1:2]
    assert torch.equal(a, b)


def test_flops_formula():
    assert ref.flops(2, 16, 2048, 128, False) == 4 * 2 * 16 * 2048 * 2048 * 128
    assert ref.flops(4, 32, 4096, 128, True) == 2 * 4 * 32 * 4096 * 4096 * 128


def test_expand_kv_heads_matches_torch_grouped_attention():
    g = torch.Generator().manual_seed(3)
    q = torch.randn(2, 6, 40, 64, generator=g)
    k, v = (torch.randn(2, 2, 40, 64, generator=g) for _ in range(2))
    ke, ve = ref.expand_kv_heads(k, v, 6)
    assert ke.shape == q.shape and torch.equal(ke[:, 4], k[:, 1]) and torch.equal(ke[:, 2], k[:, 0])
    want = F.scaled_dot_product_attention(q, k, v, enable_gqa=True)
    assert torch.allclose(ref.attention_fp32(q, ke, ve), want, atol=2e-6)


@pytest.mark.parametrize("causal", [False, True])
def test_lse_reference_against_a_direct_sum(causal):
    g = torch.Generator().manual_seed(4)
    q, k = (torch.randn(3, 17, 32, generator=g) for _ in range(2))
    got = ref.lse_fp32(q, k, causal)
    s = (q.double() @ k.double().transpose(-1, -2)) / math.sqrt(32)
    if causal:
        s = s.masked_fill(~torch.ones(17, 17, dtype=torch.bool).tril(), float("-inf"))
    want = s.exp().sum(-1).log()
    assert got.shape == (3, 17) and torch.allclose(got.double(), want, atol=1e-5)
