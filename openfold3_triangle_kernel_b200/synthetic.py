"""Seeded synthetic inputs and parameters for the benchmark workloads.

There is no dataset behind the hot path: every tensor is drawn from a seeded CPU generator with
the shapes and value distributions of the benchmark configurations (training crop N=384, H=4,
D=32, C=128; the pair-stack block at N=768 / 1536).  The draws follow the same order as the
generators the parity tests use, so a given seed names the same tensors everywhere.
"""
from __future__ import annotations

import math

import torch


def _gen(seed):
    return torch.Generator().manual_seed(seed)


def _xavier(g, rows, cols, dtype):
    return (torch.randn(rows, cols, generator=g) * math.sqrt(2.0 / (rows + cols))).to(dtype)


def attention_inputs(B, O, H, N, D, seed, dtype=torch.bfloat16, max_masked_fraction=0.15):
    """q, k, v ``[B,O,H,N,D]`` ~ N(0,1); pair_bias ``[B,1,H,N,N]`` ~ N(0,1); res_mask ``[B,O,1,1,N]``
    additive fp32 with -inf on a random trailing 0..max_masked_fraction of the keys of each outer row."""
    g = _gen(seed)
    q, k, v = (torch.randn(B, O, H, N, D, generator=g).to(dtype) for _ in range(3))
    bias = torch.randn(B, 1, H, N, N, generator=g).to(dtype)
    n_drop = (torch.rand(B, O, generator=g) * max_masked_fraction * N).floor().long()
    idx = torch.arange(N).view(1, 1, N)
    mask = torch.zeros(B, O, 1, 1, N)
    mask[:, :, 0, 0, :] = torch.where(idx >= (N - n_drop).unsqueeze(-1), float("-inf"), 0.0)
    return dict(q=q, k=k, v=v, pair_bias=bias, res_mask=mask)


def trimul_weights(c, seed, dtype=torch.float32):
    """Xavier-normal projection / gate matrices (fp32 masters), LayerNorm gamma = 1, beta = 0, under the
    operator's weight names (``p_in = cat[a_p, b_p]``, ``g_in = cat[a_g, b_g]``)."""
    g = _gen(seed)
    return dict(
        norm_in_weight=torch.ones(c, dtype=dtype), norm_in_bias=torch.zeros(c, dtype=dtype),
        p_in_weight=torch.cat([_xavier(g, c, c, dtype), _xavier(g, c, c, dtype)]),
        g_in_weight=torch.cat([_xavier(g, c, c, dtype), _xavier(g, c, c, dtype)]),
        norm_out_weight=torch.ones(c, dtype=dtype), norm_out_bias=torch.zeros(c, dtype=dtype),
        p_out_weight=_xavier(g, c, c, dtype), g_out_weight=_xavier(g, c, c, dtype),
    )


def trimul_inputs(B, N, C, seed, dtype=torch.bfloat16):
    """z ``[B,N,N,C]`` ~ N(0,1); pair mask 1 except a random trailing 0..10 % of the residues (rows and
    columns); weights from :func:`trimul_weights` with seed + 1000."""
    g = _gen(seed)
    z = torch.randn(B, N, N, C, generator=g).to(dtype)
    mask = torch.ones(B, N, N)
    n_drop = int(torch.randint(0, max(1, N // 10) + 1, (1,), generator=g).item())
    if n_drop:
        mask[:, N - n_drop:, :] = 0.0
        mask[:, :, N - n_drop:] = 0.0
    return dict(z=z, mask=mask, weights=trimul_weights(C, seed + 1000))


def attention_params(c_z, heads, d, seed, dtype=torch.float32):
    """Parameters of one triangle-attention module around the operator: LayerNorm, the bias
    projection ``w_z`` (c_z -> heads) and the bias-free q/k/v/gate/output Linears."""
    g = _gen(seed)
    return dict(ln_w=torch.ones(c_z, dtype=dtype), ln_b=torch.zeros(c_z, dtype=dtype),
                w_z=_xavier(g, heads, c_z, dtype),
                w_q=_xavier(g, heads * d, c_z, dtype), w_k=_xavier(g, heads * d, c_z, dtype),
                w_v=_xavier(g, heads * d, c_z, dtype), w_g=_xavier(g, heads * d, c_z, dtype),
                w_o=_xavier(g, c_z, heads * d, dtype))


def block_params(c_z, heads, d, seed, dtype=torch.float32):
    """Parameters of the pair-stack block: TriMul outgoing / incoming, attention starting / ending node."""
    return dict(tri_mul_out=trimul_weights(c_z, seed, dtype), tri_mul_in=trimul_weights(c_z, seed + 1, dtype),
                tri_att_start=attention_params(c_z, heads, d, seed + 2, dtype),
                tri_att_end=attention_params(c_z, heads, d, seed + 3, dtype))
