"""The pair-stack part of an OpenFold3 PairBlock on the B200 operators, optionally sharded
axially over the GPUs of one node.

Mirrors ``PairBlock.forward`` (openfold3/core/model/latent/base_blocks.py:433-534, dropout inactive,
pair transition excluded) and ``TriangleAttention.forward``
(openfold3/core/model/layers/triangular_attention.py:245-409): the LayerNorm and the bias-free
q/k/v/g/o/bias Linears around the attention operator run as plain bf16 torch ops; the two hot
operators are :func:`turbo_trimul` and :func:`turbo_attention` (or their axial variants).

Sharded layout (``group`` given): ``z`` is row-sharded ``[B, N/P, N, C]``.  TriMul uses
:func:`dap.axial_trimul`; starting-node attention shards its outer rows and all-gathers the
H-channel bias projection; the ending node works on ``z^T``, reached by one all-to-all
transpose of the sharded pair tensor, and is transposed back afterwards.
"""
from __future__ import annotations

import torch
import torch.distributed as dist
import torch.nn.functional as F

from . import dap
from .attention import turbo_attention
from .trimul import turbo_trimul


class _GatherRows(torch.autograd.Function):
    """all-gather along ``dim`` in forward; backward keeps this rank's slice of the incoming
    gradient (which the consumer has already summed over ranks)."""

    @staticmethod
    def forward(ctx, t, dim, group):
        ctx.dim, ctx.group = dim, group
        return dap.gather_rows(t, dim, group)

    @staticmethod
    def backward(ctx, g):
        return dap.shard_rows(g, ctx.dim, ctx.group), None, None


class _ShardedTranspose(torch.autograd.Function):
    """``[B, N/P (i), N (j), C]`` -> ``[B, N/P (j), N (i), C]`` with one all-to-all; its own inverse."""

    @staticmethod
    def forward(ctx, t, group):
        ctx.group = group
        return _sharded_transpose(t, group)

    @staticmethod
    def backward(ctx, g):
        return _sharded_transpose(g.contiguous(), ctx.group), None


def _sharded_transpose(t, group):
    P = dist.get_world_size(group)
    B, Nl, N, Cc = t.shape
    send = t.reshape(B, Nl, P, N // P, Cc).permute(2, 0, 3, 1, 4).contiguous()     # [P(dst j-block), B, Nl(j), Nl(i), C]
    recv = torch.empty_like(send)
    dist.all_to_all_single(recv, send, group=group)                                  # [P(src i-block), B, Nl(j), Nl(i), C]
    return recv.permute(1, 2, 0, 3, 4).reshape(B, N // P, N, Cc).contiguous()


def triangle_attention_update(z, mask, p, heads, transpose_bias=False, inf=1e9, group=None, attention_fn=None):
    """z ``[B, I(local), J, C]`` bf16, mask ``[B, I(local), J]``.  Returns the update, same shape as z.
    ``attention_fn`` replaces :func:`turbo_attention` (same signature; used to test the sharding
    plumbing without a GPU)."""
    c = z.shape[-1]
    x = F.layer_norm(z.float(), (c,), p["ln_w"].float(), p["ln_b"].float(), 1e-5).to(z.dtype)
    mask_bias = (inf * (mask.float() - 1))[..., :, None, None, :]
    lz = F.linear(x, p["w_z"].to(z.dtype))                               # [B, I_loc, J, H]
    if group is not None:
        lz = _GatherRows.apply(lz, 1, group)                             # [B, I, J, H]: the bias needs every row
    bias = (lz.permute(0, 3, 2, 1) if transpose_bias else lz.permute(0, 3, 1, 2)).unsqueeze(1)   # [B,1,H,N,N]
    d = p["w_q"].shape[0] // heads

    def heads_view(t):
        return t.reshape(t.shape[:-1] + (heads, d)).transpose(-2, -3)   # sequence-major view [B, I, H, J, D]

    q, k, v = (heads_view(F.linear(x, p[n].to(z.dtype))) for n in ("w_q", "w_k", "w_v"))
    if group is None:
        o = (attention_fn or turbo_attention)(q, k, v, pair_bias=bias, res_mask=mask_bias)
    else:
        o = dap.axial_attention(q, k, v, bias, mask_bias, group=group, attention_fn=attention_fn)
    gate = torch.sigmoid(F.linear(x, p["w_g"].to(z.dtype))).reshape(o.shape)
    return F.linear((o * gate).reshape(o.shape[:-2] + (heads * d,)), p["w_o"].to(z.dtype))


def pair_stack_block(z, mask, params, heads, group=None, trimul_backend=None, attention_fn=None):
    """TriMul outgoing -> TriMul incoming -> attention starting node -> attention ending node, each
    with its residual add.  ``z`` bf16 ``[B, N, N, C]`` (or the local rows ``[B, N/P, N, C]`` with
    ``group``); ``mask`` ``[B, N, N]`` (local rows likewise).  ``params`` as produced by
    ``synthetic.block_params`` (fp32 masters).  ``trimul_backend`` / ``attention_fn`` replace the
    CUDA stage back end of :func:`dap.axial_trimul` and :func:`turbo_attention` in the sharded
    path (used to test the collectives on CPU ranks); the defaults are the B200 operators."""
    if group is None:
        z = z + turbo_trimul(z, "outgoing", mask, **params["tri_mul_out"])
        z = z + turbo_trimul(z, "incoming", mask, **params["tri_mul_in"])
        z = z + triangle_attention_update(z, mask, params["tri_att_start"], heads)
        zt = z.transpose(-2, -3)
        zt = zt + triangle_attention_update(zt, mask.transpose(-1, -2), params["tri_att_end"], heads,
                                            transpose_bias=True)
        return zt.transpose(-2, -3)
    z = z + dap.axial_trimul(z, "outgoing", mask, group=group, backend=trimul_backend, **params["tri_mul_out"])
    z = z + dap.axial_trimul(z, "incoming", mask, group=group, backend=trimul_backend, **params["tri_mul_in"])
    z = z + triangle_attention_update(z, mask, params["tri_att_start"], heads, group=group, attention_fn=attention_fn)
    zt = _ShardedTranspose.apply(z, group)
    mt = _sharded_transpose(mask.unsqueeze(-1).float().contiguous(), group).squeeze(-1)
    zt = zt + triangle_attention_update(zt, mt, params["tri_att_end"], heads, transpose_bias=True, group=group,
                                        attention_fn=attention_fn)
    return _ShardedTranspose.apply(zt.contiguous(), group)
