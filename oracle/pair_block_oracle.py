"""CPU restatement of the pair-stack part of the reference's PairBlock (test infrastructure).

Follows ``PairBlock.forward`` (openfold3/core/model/latent/base_blocks.py:433-534) with dropout
inactive and without the pair transition:

    z += TriMulOut(z, mask);  z += TriMulIn(z, mask)
    z += TriAttStart(z, mask)
    z = z^T;  z += TriAttEnd(z, mask^T, transpose_bias=True);  z = z^T

``TriangleAttention.forward`` (openfold3/core/model/layers/triangular_attention.py:245-409):
x = LayerNorm(z); mask_bias = inf * (mask - 1) as [*, I, 1, 1, J]; triangle_bias =
linear_z(x) permuted to [*, 1, H, I, J] ((2,0,1), or (2,1,0) with transpose_bias); then the gated
multi-head attention of openfold3/core/model/primitives/attention.py:347-384 (bias-free
q/k/v/g/o Linears, q scaled by D^-1/2, output gated by sigmoid(linear_g(x)), linear_o).
"""
from __future__ import annotations

import math

import torch
import torch.nn.functional as F

from .attention_oracle import attention_forward
from .trimul_oracle import trimul_forward, xavier_weights

ATT_PARAM_NAMES = ("ln_w", "ln_b", "w_z", "w_q", "w_k", "w_v", "w_g", "w_o")


def attention_params(c_z, heads, d, seed, dtype=torch.float32):
    g = torch.Generator().manual_seed(seed)

    def xn(rows, cols):
        return (torch.randn(rows, cols, generator=g) * math.sqrt(2.0 / (rows + cols))).to(dtype)

    return dict(ln_w=torch.ones(c_z, dtype=dtype), ln_b=torch.zeros(c_z, dtype=dtype), w_z=xn(heads, c_z),
                w_q=xn(heads * d, c_z), w_k=xn(heads * d, c_z), w_v=xn(heads * d, c_z), w_g=xn(heads * d, c_z),
                w_o=xn(c_z, heads * d))


def block_params(c_z, heads, d, seed, dtype=torch.float32):
    return dict(tri_mul_out=xavier_weights(c_z, seed, dtype), tri_mul_in=xavier_weights(c_z, seed + 1, dtype),
                tri_att_start=attention_params(c_z, heads, d, seed + 2, dtype),
                tri_att_end=attention_params(c_z, heads, d, seed + 3, dtype))


def triangle_attention_module(z, mask, p, heads, transpose_bias=False, inf=1e9, dtype=torch.float64):
    """z [*, I, J, C]; mask [*, I, J] (1 keeps).  Returns the update [*, I, J, C]."""
    w = {k: v.to(dtype) for k, v in p.items()}
    c = z.shape[-1]
    x = F.layer_norm(z.to(dtype), (c,), w["ln_w"], w["ln_b"], 1e-5)
    mask_bias = (inf * (mask.to(dtype) - 1))[..., :, None, None, :]
    lz = F.linear(x, w["w_z"])                                            # [*, I, J, H]
    bias = (lz.permute(*range(lz.dim() - 3), -1, -2, -3) if transpose_bias
            else lz.permute(*range(lz.dim() - 3), -1, -3, -2)).unsqueeze(-4)   # [*, 1, H, I, J]
    d = w["w_q"].shape[0] // heads

    def heads_view(t):
        return t.reshape(t.shape[:-1] + (heads, d)).transpose(-2, -3)    # [*, I, H, J, D]

    q, k, v = (heads_view(F.linear(x, w[n])) for n in ("w_q", "w_k", "w_v"))
    o, _ = attention_forward(q, k, v, bias, mask_bias, dtype=dtype)      # [*, I, J, H, D]
    gate = torch.sigmoid(F.linear(x, w["w_g"])).reshape(o.shape)
    return F.linear((o * gate).reshape(o.shape[:-2] + (heads * d,)), w["w_o"])


def pair_block_forward(z, mask, params, heads, dtype=torch.float64):
    z = z.to(dtype)
    z = z + trimul_forward(z, "outgoing", mask, params["tri_mul_out"], dtype=dtype)
    z = z + trimul_forward(z, "incoming", mask, params["tri_mul_in"], dtype=dtype)
    z = z + triangle_attention_module(z, mask, params["tri_att_start"], heads, dtype=dtype)
    z = z.transpose(-2, -3)
    z = z + triangle_attention_module(z, mask.transpose(-1, -2), params["tri_att_end"], heads, transpose_bias=True,
                                      dtype=dtype)
    return z.transpose(-2, -3)
