"""CPU restatement of the reference triangle-attention math (test infrastructure).

Follows, by file:line in the reference project:

* ``openfold3/core/model/primitives/attention.py:176-217`` (``_attention``):
  ``softmax(q_scaled @ k^T + sum(biases)) @ v`` with the softmax in the
  compute dtype.
* ``openfold3/core/model/primitives/attention.py:365-366`` — the caller scales
  ``q`` by ``D ** -0.5`` (the fused operators take *unscaled* q and apply the
  scale themselves).
* ``openfold3/core/model/primitives/attention.py:692`` — the result is
  transposed from ``[*, O, H, N, D]`` to ``[*, O, N, H, D]``.
* ``tools/aot_numeric_smoke.py:39-48`` (``_oracle``) — the FP64 oracle used by
  the reference's acceptance gate, including the ``-inf -> -1e4`` sentinel.
  Here ``-inf`` is kept as ``-inf`` and a fully masked row is defined to give
  a zero output row and ``-inf`` log-sum-exp, which is what the reference
  kernels produce (``turbopairformer_triangle_forward.cu:1226-1227,1250-1252``).

Parity pin: ``tests/test_oracle_pins.py`` checks this file against outputs of
the reference's own stock PyTorch modules, generated in a container that has
the reference (``tests/golden/make_golden.py``) and committed as fixtures.
"""
from __future__ import annotations

import math

import torch


def attention_forward(q, k, v, pair_bias, res_mask=None, dtype=torch.float64):
    """Reference forward.

    q, k, v: ``[*B, O, H, N, D]`` (unscaled q).  pair_bias ``[*B, 1, H, N, N]``.
    res_mask additive ``[*B, O, 1, 1, N]`` or None.
    Returns ``(out [*B, O, N, H, D], lse [*B, O, H, N])`` in ``dtype``.
    """
    q, k, v = (t.to(dtype) for t in (q, k, v))
    scale = 1.0 / math.sqrt(q.shape[-1])
    s = torch.matmul(q, k.transpose(-1, -2)) * scale
    if res_mask is not None:
        s = s + res_mask.to(dtype)
    s = s + pair_bias.to(dtype)
    lse = torch.logsumexp(s, dim=-1)
    p = torch.exp(s - lse.unsqueeze(-1))
    # exp(-inf - (-inf)) is nan: a fully masked row carries no probability.
    p = torch.where(torch.isneginf(lse).unsqueeze(-1), torch.zeros_like(p), p)
    out = torch.matmul(p, v).transpose(-2, -3)
    return out, lse


def attention_forward_backward(q, k, v, pair_bias, res_mask, d_out, dtype=torch.float64):
    """Forward + analytic backward (no autograd, so -inf rows stay finite).

    Returns dict(out, lse, dq, dk, dv, dbias); dbias has pair_bias's shape
    (summed over O and over any broadcast batch dims).
    """
    qd, kd, vd = (t.to(dtype) for t in (q, k, v))
    scale = 1.0 / math.sqrt(q.shape[-1])
    s = torch.matmul(qd, kd.transpose(-1, -2)) * scale
    if res_mask is not None:
        s = s + res_mask.to(dtype)
    s = s + pair_bias.to(dtype)
    lse = torch.logsumexp(s, dim=-1)
    p = torch.exp(s - lse.unsqueeze(-1))
    p = torch.where(torch.isneginf(lse).unsqueeze(-1), torch.zeros_like(p), p)
    out_h = torch.matmul(p, vd)                       # [*B,O,H,N,D]
    do_h = d_out.to(dtype).transpose(-2, -3)          # [*B,O,H,N,D]
    dv = torch.matmul(p.transpose(-1, -2), do_h)
    dp = torch.matmul(do_h, vd.transpose(-1, -2))
    delta = (do_h * out_h).sum(-1, keepdim=True)
    ds = p * (dp - delta)
    dq = torch.matmul(ds, kd) * scale
    dk = torch.matmul(ds.transpose(-1, -2), qd) * scale
    dbias = ds.sum(dim=-4, keepdim=True)
    # reduce broadcast batch dims of pair_bias
    bshape = pair_bias.shape
    lead = dbias.dim() - len(bshape)
    if lead:
        dbias = dbias.sum(dim=tuple(range(lead)))
    for i, (have, want) in enumerate(zip(dbias.shape, bshape)):
        if have != want:
            dbias = dbias.sum(dim=i, keepdim=True)
    return dict(out=out_h.transpose(-2, -3), lse=lse, dq=dq, dk=dk, dv=dv, dbias=dbias)


def stock_bf16_forward_backward(q, k, v, pair_bias, res_mask, d_out):
    """The 'stock bf16 PyTorch' arm of the reference's acceptance envelope
    (``tools/aot_numeric_smoke.py:51-60``): bf16 matmuls, fp32 softmax,
    probabilities rounded to bf16, autograd backward.  ``-inf`` mask entries
    become -1e4 exactly as there (``:30-36``)."""
    neg = -1e4
    q_, k_, v_ = (t.detach().clone().requires_grad_(True) for t in (q, k, v))
    b_ = pair_bias.detach().clone().requires_grad_(True)
    m = res_mask.float()
    m = torch.where(torch.isinf(m), torch.full_like(m, neg), m)
    scale = 1.0 / math.sqrt(q.shape[-1])
    s = torch.matmul(q_, k_.transpose(-1, -2)).float() * scale
    s = s + m + b_.float()
    out = torch.matmul(torch.softmax(s, dim=-1).to(torch.bfloat16), v_).transpose(-2, -3)
    out.backward(d_out)
    return dict(out=out.detach(), dq=q_.grad, dk=k_.grad, dv=v_.grad, dbias=b_.grad)


def rel_l2(a, b):
    """Relative L2 error used by the reference gate (``tools/aot_numeric_smoke.py:74-75``)."""
    a, b = a.double(), b.double()
    return float((a - b).norm() / b.norm().clamp_min(1e-30))
