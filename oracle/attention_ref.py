"""CPU oracle for the attention forward path.  TEST INFRASTRUCTURE ONLY.

Only tests/, __graft_entry__.smoke() and bench.py's CPU-baseline / reference arm may
import this module; the product path never does (it has no CPU fallback).

The reference has no CPU implementation of its kernel and its own test checks the kernel
against torch attention on the same seeded inputs (tests/test_flashattn_cute.py:24,27-28),
so that is the oracle here too, in two forms:

* ``sdpa_cpu``      - torch ``scaled_dot_product_attention`` on CPU (fp16 or fp32 tensors);
* ``attention_fp32``- explicit fp32 ``softmax(q k^T * scale [+ causal mask]) v``.

``flash_fp16p`` restates the arithmetic of the reference kernel itself - base-2 online
softmax over KV tiles with P rounded to fp16 before the P.V product and the row sum taken
from the unrounded P (fray/include/flash_attn/softmax.cuh:24-81,
flashattn_cute.cuh:104,134,141) - in vectorised torch; oracle/attn_oracle.c is the same
restatement in plain C.

Pinning: the reference holds no golden vectors for this path (its inputs are seeded on
the CUDA device), so the restatements are pinned against torch SDPA - the reference's own
oracle - and against the fixtures under tests/golden/ produced by make_golden.py.
"""
import math
from typing import Dict, Tuple

import torch
import torch.nn.functional as F

# BASELINE configurations: (B, H, S, D, causal).  Index = config number - 1.
CONFIGS: Tuple[Dict, ...] = (
    dict(name="c1", B=1, H=4, S=256, D=64, causal=False),
    dict(name="c2", B=2, H=16, S=2048, D=128, causal=False),
    dict(name="c3", B=4, H=32, S=4096, D=128, causal=True),
    dict(name="c4", B=1, H=32, S=16384, D=128, causal=True),
    dict(name="c5", B=16, H=16, S=1024, D=64, causal=False, stress=True, q_transposed=True),
    dict(name="headline", B=4, H=32, S=4096, D=128, causal=False),
)


def slice_seed(cfg_index: int, bh: int) -> int:
    """Seed of the CPU generator for one (batch, head) slice; 42 is the reference test's seed."""
    return 42 * 1000 + cfg_index * 100000 + bh


def make_slice(cfg_index: int, bh: int, S: int, D: int, stress: bool = False):
    """fp16 q, k, v of shape [S, D] for one (b, h) slice, identical on any host and any GPU count."""
    g = torch.Generator(device="cpu")
    g.manual_seed(slice_seed(cfg_index, bh))
    q = torch.randn(S, D, generator=g, dtype=torch.float32)
    k = torch.randn(S, D, generator=g, dtype=torch.float32)
    v = torch.randn(S, D, generator=g, dtype=torch.float32)
    if stress:
        # large-logit stress: q,k scaled by 4 and 1 % of entries forced to +-16
        for t in (q, k):
            t.mul_(4.0)
            u = torch.rand(S, D, generator=g, dtype=torch.float32)
            t[u < 0.01] = -16.0
            t[u < 0.005] = 16.0
    return q.half(), k.half(), v.half()


def make_inputs(cfg_index: int, units=None):
    """q, k, v as [n_units, S, D] fp16 CPU tensors for the given flat (b*H+h) unit indices (default: all)."""
    cfg = CONFIGS[cfg_index]
    if units is None:
        units = range(cfg["B"] * cfg["H"])
    qs, ks, vs = [], [], []
    for bh in units:
        q, k, v = make_slice(cfg_index, bh, cfg["S"], cfg["D"], cfg.get("stress", False))
        qs.append(q), ks.append(k), vs.append(v)
    return torch.stack(qs), torch.stack(ks), torch.stack(vs)


def sdpa_cpu(q, k, v, causal=False, scale=None):
    """torch CPU attention, the oracle of the reference's own test."""
    return F.scaled_dot_product_attention(q, k, v, is_causal=causal, scale=scale)


def attention_fp32(q, k, v, causal=False, scale=None):
    """Explicit fp32 math over [..., S, D] tensors, one leading index at a time to bound memory."""
    S, D = q.shape[-2], q.shape[-1]
    scale = 1.0 / math.sqrt(D) if scale is None else scale
    qf, kf, vf = (t.reshape(-1, S, D).float() for t in (q, k, v))
    out = torch.empty_like(qf)
    mask = torch.ones(S, S, dtype=torch.bool).tril_() if causal else None
    for i in range(qf.shape[0]):
        s = (qf[i] @ kf[i].T) * scale
        if mask is not None:
            s.masked_fill_(~mask, float("-inf"))
        out[i] = torch.softmax(s, dim=-1) @ vf[i]
    return out.reshape(q.shape)


def flash_fp16p(q, k, v, causal=False, scale=None, block_n=128):
    """Tile-by-tile restatement of the kernel arithmetic (see module docstring); returns fp16."""
    S, D = q.shape[-2], q.shape[-1]
    scale = 1.0 / math.sqrt(D) if scale is None else scale
    c = scale * 1.44269504088896340736
    qf, kf, vf = (t.reshape(-1, S, D).float() for t in (q, k, v))
    n = qf.shape[0]
    m = torch.full((n, S), float("-inf"))
    l = torch.zeros(n, S)
    acc = torch.zeros(n, S, D)
    rows = torch.arange(S).view(1, S, 1)
    for j0 in range(0, S, block_n):
        j1 = min(S, j0 + block_n)
        s = qf @ kf[:, j0:j1].transpose(1, 2)
        if causal:
            cols = torch.arange(j0, j1).view(1, 1, -1)
            s = s.masked_fill(cols > rows, float("-inf"))
        m_new = torch.maximum(m, s.amax(dim=-1))
        alpha = torch.where(torch.isinf(m_new), torch.zeros_like(m_new), torch.exp2((m - m_new) * c))
        m_sc = torch.where(torch.isinf(m_new), torch.zeros_like(m_new), m_new * c)
        p = torch.exp2(s * c - m_sc.unsqueeze(-1))
        l = l * alpha + p.sum(dim=-1)
        acc = acc * alpha.unsqueeze(-1) + p.half().float() @ vf[:, j0:j1]
        m = m_new
    inv = torch.where(l > 0, 1.0 / l, torch.ones_like(l))
    return (acc * inv.unsqueeze(-1)).half().reshape(q.shape)


def expand_kv_heads(k, v, num_heads):
    """Grouped-query attention restated as plain attention: K/V head g serves query heads g*r .. g*r+r-1,
    r = num_heads / K-V heads (the mapping torch's ``enable_gqa`` and the vendored Blackwell kernels use)."""
    r = num_heads // k.shape[-3]
    return k.repeat_interleave(r, dim=-3), v.repeat_interleave(r, dim=-3)


def lse_fp32(q, k, causal=False, scale=None):
    """log(sum_j exp(scale * q_i . k_j)) over the keys row i may see, fp32, shape q.shape[:-1]."""
    S, D = q.shape[-2], q.shape[-1]
    scale = 1.0 / math.sqrt(D) if scale is None else scale
    qf, kf = (t.reshape(-1, S, D).float() for t in (q, k))
    out = torch.empty(qf.shape[0], S)
    mask = torch.ones(S, S, dtype=torch.bool).tril_() if causal else None
    for i in range(qf.shape[0]):
        s = (qf[i] @ kf[i].T) * scale
        if mask is not None:
            s.masked_fill_(~mask, float("-inf"))
        out[i] = torch.logsumexp(s, dim=-1)
    return out.reshape(q.shape[:-1])


def calc_diff(x, y):
    """Same measure as the reference's fray/utils.py:48-52."""
    x, y = x.double(), y.double()
    return float(1 - 2 * (x * y).sum() / (x * x + y * y).sum())


def flops(B, H, S, D, causal):
    """The reference's count 4*B*H*S^2*D (tests/test_flashattn_cute.py:56), halved for causal."""
    f = 4.0 * B * H * S * S * D
    return f / 2 if causal else f
