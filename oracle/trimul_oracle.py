"""CPU restatement of the reference triangle multiplicative update (test infrastructure).

Follows, by file:line in the reference project:

* ``openfold3/core/model/layers/triangular_multiplicative_update.py:1262-1284``
  (``TriangleMultiplicativeUpdate.forward``, stock path): LayerNorm, gated
  a/b projections times the mask, ``_combine_projections``, output LayerNorm,
  ``linear_z``, sigmoid gate ``linear_g``.
* ``…/triangular_multiplicative_update.py:734-761`` (``_combine_projections``):
  outgoing ``x[i,j,c] = sum_k a[i,k,c] b[j,k,c]``; incoming
  ``x[i,j,c] = sum_k a[k,i,c] b[k,j,c]``.
* ``openfold3/core/model/primitives/normalization.py:28-77``: LayerNorm with
  eps 1e-5 computed in fp32 or wider.
* ``openfold3/core/config/default_linear_init_config.py:109-118``: none of the
  six Linears carries a bias.
* ``tools/aot_clean_install_smoke.py:90-134`` is the reference's own unfused
  restatement of the same equations.

Weight naming is that of the reference's fused-operator adapter
(``…/triangular_multiplicative_update.py:1592-1634``): ``p_in_weight`` is
``cat[a_p, b_p]`` ``[2C, C]``, ``g_in_weight`` is ``cat[a_g, b_g]``.

Parity pin: fixtures generated from the reference's stock modules
(``tests/golden/make_golden.py``), checked in ``tests/test_oracle_pins.py``.
"""
from __future__ import annotations

import math

import torch
import torch.nn.functional as F

WEIGHT_NAMES = (
    "norm_in_weight", "norm_in_bias", "p_in_weight", "g_in_weight",
    "norm_out_weight", "norm_out_bias", "p_out_weight", "g_out_weight",
)


def xavier_weights(c, seed, dtype=torch.float32):
    """Seeded Xavier-normal projection/gate matrices, LN gamma=1, beta=0."""
    g = torch.Generator().manual_seed(seed)

    def xn(rows, cols):
        std = math.sqrt(2.0 / (rows + cols))
        return (torch.randn(rows, cols, generator=g) * std).to(dtype)

    return dict(
        norm_in_weight=torch.ones(c, dtype=dtype), norm_in_bias=torch.zeros(c, dtype=dtype),
        p_in_weight=torch.cat([xn(c, c), xn(c, c)]), g_in_weight=torch.cat([xn(c, c), xn(c, c)]),
        norm_out_weight=torch.ones(c, dtype=dtype), norm_out_bias=torch.zeros(c, dtype=dtype),
        p_out_weight=xn(c, c), g_out_weight=xn(c, c),
    )


def trimul_forward(z, direction, mask, weights, dtype=torch.float64, eps=1e-5):
    """z ``[*B, N, N, C]``; mask ``[*B, N, N]`` or None; returns ``[*B, N, N, C]``."""
    w = {k: v.to(dtype) for k, v in weights.items()}
    c = z.shape[-1]
    zd = z.to(dtype)
    m = torch.ones(z.shape[:-1], dtype=dtype) if mask is None else mask.to(dtype)
    m = m.unsqueeze(-1)
    hid = w["p_in_weight"].shape[0] // 2  # hidden width (== c in the operator contract; the stock module allows any)
    zn = F.layer_norm(zd, (c,), w["norm_in_weight"], w["norm_in_bias"], eps)
    p = F.linear(zn, w["p_in_weight"])
    g = torch.sigmoid(F.linear(zn, w["g_in_weight"]))
    a = m * g[..., :hid] * p[..., :hid]
    b = m * g[..., hid:] * p[..., hid:]
    if direction == "outgoing":
        x = torch.einsum("...ikc,...jkc->...ijc", a, b)
    elif direction == "incoming":
        x = torch.einsum("...kic,...kjc->...ijc", a, b)
    else:
        raise ValueError(direction)
    xn = F.layer_norm(x, (hid,), w["norm_out_weight"], w["norm_out_bias"], eps)
    out = F.linear(xn, w["p_out_weight"]) * torch.sigmoid(F.linear(zn, w["g_out_weight"]))
    return out


def trimul_forward_backward(z, direction, mask, weights, d_out, dtype=torch.float64):
    """Forward and autograd backward in ``dtype``.  Returns dict(out, dz, d<weight>...)."""
    zz = z.detach().to(dtype).requires_grad_(True)
    ww = {k: v.detach().to(dtype).requires_grad_(True) for k, v in weights.items()}
    out = trimul_forward(zz, direction, mask, ww, dtype=dtype)
    out.backward(d_out.to(dtype))
    res = dict(out=out.detach(), dz=zz.grad)
    for k in WEIGHT_NAMES:
        res["d_" + k] = ww[k].grad
    return res
