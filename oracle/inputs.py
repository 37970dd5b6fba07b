"""Seeded synthetic inputs for the benchmark / parity configurations
(test infrastructure).  Shapes and value distributions follow the five
workload configurations of the build's baseline description; there is no
dataset involved, every tensor is drawn from a seeded CPU generator."""
from __future__ import annotations

import torch

from .trimul_oracle import xavier_weights


def _gen(seed):
    return torch.Generator().manual_seed(seed)


def attention_inputs(B, O, H, N, D, seed, dtype=torch.bfloat16, mask_mode="trailing15", bias_scale=1.0):
    """q,k,v ``[B,O,H,N,D]``, pair_bias ``[B,1,H,N,N]``, res_mask ``[B,O,1,1,N]`` additive fp32,
    d_out = d/d(out) of mean(out^2) is left to the caller."""
    g = _gen(seed)
    q, k, v = (torch.randn(B, O, H, N, D, generator=g).to(dtype) for _ in range(3))
    bias = (torch.randn(B, 1, H, N, N, generator=g) * bias_scale).to(dtype)
    mask = torch.zeros(B, O, 1, 1, N)
    if mask_mode == "last8":
        mask[..., N - 8:] = float("-inf")
    elif mask_mode == "trailing15":
        frac = torch.rand(B, O, generator=g) * 0.15
        n_drop = (frac * N).floor().long()
        idx = torch.arange(N).view(1, 1, N)
        mask[:, :, 0, 0, :] = torch.where(idx >= (N - n_drop).unsqueeze(-1), float("-inf"), 0.0)
    elif mask_mode == "random30":
        mask[torch.rand(B, O, 1, 1, N, generator=g) < 0.3] = float("-inf")
    elif mask_mode == "none":
        pass
    else:
        raise ValueError(mask_mode)
    return dict(q=q, k=k, v=v, pair_bias=bias, res_mask=mask)


def attention_inputs_cpu_case(seed=0):
    """Config 'CPU reference': fp32, B=1, O=N=64, H=4, D=32, last 8 keys -inf."""
    return attention_inputs(1, 64, 4, 64, 32, seed, dtype=torch.float32, mask_mode="last8")


def trimul_inputs(B, N, C, seed, dtype=torch.bfloat16, mask_mode="trailing10"):
    g = _gen(seed)
    z = torch.randn(B, N, N, C, generator=g).to(dtype)
    mask = torch.ones(B, N, N)
    if mask_mode == "trailing10":
        n_drop = int(torch.randint(0, max(1, N // 10) + 1, (1,), generator=g).item())
        if n_drop:
            mask[:, N - n_drop:, :] = 0.0
            mask[:, :, N - n_drop:] = 0.0
    elif mask_mode != "none":
        raise ValueError(mask_mode)
    return dict(z=z, mask=mask, weights=xavier_weights(C, seed + 1000))


def trimul_inputs_cpu_case(seed=1):
    """Config 'CPU reference': fp32 z [1,64,64,32], gamma=1/beta=0, Xavier-normal projections."""
    return trimul_inputs(1, 64, 32, seed, dtype=torch.float32, mask_mode="none")
