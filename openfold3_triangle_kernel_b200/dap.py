"""Axial (DAP-style) sharding of the pair-stack operators across the GPUs of one node.

The reference only has data-parallel replicas; this module adds the partition its
north star describes, one process per GPU over ``torch.distributed`` (NCCL on GPUs, gloo
in the CPU tests):

* **Triangle attention** shards the outer rows ``O``: every (b, o) plane is independent,
  ``pair_bias`` is replicated and its gradient is summed over ranks with one all-reduce.
* **TriMul** is row-sharded for LayerNorm, projections and gating (row-local work), moves
  to a channel-sharded layout with one all-to-all for the k-contraction (each rank holds
  ``C / P`` full ``N x N`` planes of ``a`` and ``b``), and moves the result back with a
  second all-to-all for the output LayerNorm / projection / gate.  Backward mirrors it;
  weight and LayerNorm gradients are all-reduced.

The device work goes through the staged C-ABI entry points (``tpf_trimul_fwd_stages``,
``tpf_trimul_bwd_stages``, ``tpf_bmm_bf16``); the collectives are issued from Python between
them.  A ``backend`` object can replace the stage functions, which the CPU tests use to check
the sharding and collective plumbing against the unsharded oracle.
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from . import _cabi as C


# --------------------------------------------------------------------------------------
# helpers
# --------------------------------------------------------------------------------------
def _world(group):
    return dist.get_world_size(group), dist.get_rank(group)


def shard_rows(t, dim, group=None):
    """This rank's contiguous block of ``t`` along ``dim`` (extent must divide evenly)."""
    P, r = _world(group)
    n = t.shape[dim]
    if n % P:
        raise ValueError(f"extent {n} of dim {dim} is not divisible by the group size {P}")
    return t.narrow(dim, r * (n // P), n // P).contiguous()


def gather_rows(t, dim, group=None):
    """Inverse of :func:`shard_rows` (not differentiable)."""
    P, _ = _world(group)
    parts = [torch.empty_like(t) for _ in range(P)]
    dist.all_gather(parts, t.contiguous(), group=group)
    return torch.cat(parts, dim=dim)


def rows_to_channels_many(ts, group=None):
    """Each ``t`` of ``ts``: ``[B, C, N_local, N]`` (rows of this rank, all channels) ->
    ``[B, C/P, N, N]`` (all rows, channels of this rank).  ONE all-to-all moves all of them: the
    tensors travel stacked in one send buffer, so a / b (and d_a / d_b on the way back) cost one
    collective launch instead of one each."""
    P, _ = _world(group)
    B, Cc, Nl, N = ts[0].shape
    if Cc % P:
        raise ValueError(f"C={Cc} is not divisible by the group size {P}")
    K = len(ts)
    send = ts[0].new_empty((P, K, B, Cc // P, Nl, N))
    for i, t in enumerate(ts):
        send[:, i].copy_(t.reshape(B, P, Cc // P, Nl, N).permute(1, 0, 2, 3, 4))
    recv = torch.empty_like(send)
    dist.all_to_all_single(recv, send, group=group)
    return [recv[:, i].permute(1, 2, 0, 3, 4).reshape(B, Cc // P, P * Nl, N) for i in range(K)]


def channels_to_rows_many(ts, group=None):
    """Inverse of :func:`rows_to_channels_many`: each ``[B, C/P, N, N]`` -> ``[B, C, N_local, N]``."""
    P, _ = _world(group)
    B, Cl, Nf, N = ts[0].shape
    if Nf % P:
        raise ValueError(f"N={Nf} is not divisible by the group size {P}")
    K = len(ts)
    send = ts[0].new_empty((P, K, B, Cl, Nf // P, N))
    for i, t in enumerate(ts):
        send[:, i].copy_(t.reshape(B, Cl, P, Nf // P, N).permute(2, 0, 1, 3, 4))
    recv = torch.empty_like(send)
    dist.all_to_all_single(recv, send, group=group)
    return [recv[:, i].permute(1, 0, 2, 3, 4).reshape(B, P * Cl, Nf // P, N) for i in range(K)]


def rows_to_channels(t, group=None):
    """``[B, C, N_local, N]`` -> ``[B, C/P, N, N]``.  One all-to-all."""
    return rows_to_channels_many([t], group)[0]


def channels_to_rows(t, group=None):
    """Inverse of :func:`rows_to_channels`: ``[B, C/P, N, N]`` -> ``[B, C, N_local, N]``."""
    return channels_to_rows_many([t], group)[0]


class _SumGradOverRanks(torch.autograd.Function):
    """Identity in forward; all-reduce(SUM) of the gradient in backward (replicated input)."""

    @staticmethod
    def forward(ctx, t, group):
        ctx.group = group
        return t.view_as(t)

    @staticmethod
    def backward(ctx, g):
        g = g.contiguous()
        dist.all_reduce(g, op=dist.ReduceOp.SUM, group=ctx.group)
        return g, None


# --------------------------------------------------------------------------------------
# triangle attention, outer rows sharded
# --------------------------------------------------------------------------------------
def axial_attention(q, k, v, pair_bias, res_mask=None, group=None, attention_fn=None):
    """``q, k, v``: this rank's outer rows ``[*B, O/P, H, N, D]``; ``res_mask`` likewise
    ``[*B, O/P, 1, 1, N]``; ``pair_bias`` replicated ``[*B, 1, H, N, N]``.  Returns the local
    ``[*B, O/P, N, H, D]``.  The bias gradient every rank receives is the full sum over all
    outer rows, all-reduced in fp32."""
    if attention_fn is None:
        from .attention import turbo_attention as attention_fn
    # The operator returns the bias gradient in the bias dtype.  Handing it an fp32 copy of the bias (the
    # kernels round it back to the same bf16 values) keeps each rank's partial sum in fp32 through the
    # all-reduce; the single cast to the caller's dtype happens after the sum.
    wide = pair_bias if pair_bias.dtype in (torch.float32, torch.float64) else pair_bias.float()
    bias = _SumGradOverRanks.apply(wide, group)
    return attention_fn(q, k, v, pair_bias=bias, res_mask=res_mask)


# --------------------------------------------------------------------------------------
# TriMul stage back end on the C ABI
# --------------------------------------------------------------------------------------
_W_FWD = ("p_in_weight", "g_in_weight", "p_out_weight", "g_out_weight", "norm_in_weight", "norm_in_bias",
          "norm_out_weight", "norm_out_bias")
_W_BWD = ("p_in_weight", "g_in_weight", "p_out_weight", "g_out_weight", "norm_in_weight", "norm_out_weight")


class CudaTrimulStages:
    """Stage functions of the sharded TriMul on ``libtpf_b200.so``.  All tensors are bf16 / fp32 on
    one CUDA device; ``rows`` = ``N_local * N`` must be a multiple of 64."""

    def __init__(self, reuse_buffers=False):
        # reuse_buffers: keep one set of stage buffers per (shape, direction) and hand it out again on
        # the next forward.  Only for callers that finish the backward of a shape/direction before
        # they start its next forward (a benchmark loop); autograd users keep the default.
        self._reuse = bool(reuse_buffers)
        self._cache = {}

    def proj_fwd(self, z, mask, w, incoming):
        B, Nl, N, Cc = z.shape
        dev = z.device
        R = B * Nl * N
        key = (B, Nl, N, Cc, bool(incoming), dev)
        st = self._cache.get(key) if self._reuse else None
        if st is None:
            bf = lambda *s: torch.empty(s, device=dev, dtype=torch.bfloat16)  # noqa: E731
            f32 = lambda *s: torch.empty(s, device=dev, dtype=torch.float32)  # noqa: E731
            st = dict(incoming=bool(incoming), zln=bf(R, Cc), gate=bf(R, Cc), mean_in=f32(R), rstd_in=f32(R),
                      a_cm=bf(B, Cc, Nl, N), b_cm=bf(B, Cc, Nl, N),
                      x_cm=None, xln=bf(R, Cc), mean_out=f32(R), rstd_out=f32(R), out=bf(B, Nl, N, Cc))
            nbytes = max(C.load().tpf_trimul_fwd_workspace_bytes(B, N, Cc), 256)
            st["ws_f"] = torch.empty(nbytes, device=dev, dtype=torch.uint8)
            if self._reuse:
                self._cache[key] = st
        st["x_cm"] = None
        st["z"] = z.contiguous()
        st["mask"] = mask.to(torch.float32).contiguous()
        st["w"] = {k: w[k].detach().float().contiguous() for k in _W_FWD}
        self._fwd(st, 1)
        return st

    def _fwd(self, st, stages):
        z = st["z"]
        B, Nl, N, Cc = z.shape
        p = C.ptr
        x_cm = st["x_cm"] if st["x_cm"] is not None else st["a_cm"]  # unused by stage 1
        with torch.cuda.device(z.device):
            C.call("tpf_trimul_fwd_stages", p(z), p(st["mask"]), *[p(st["w"][k]) for k in _W_FWD], int(st["incoming"]),
                   B, N, Cc, p(st["out"]), p(st["zln"]), p(st["mean_in"]), p(st["rstd_in"]), p(st["a_cm"]),
                   p(st["b_cm"]), p(st["gate"]), p(x_cm), p(st["xln"]), p(st["mean_out"]), p(st["rstd_out"]),
                   p(st["ws_f"]), st["ws_f"].numel(), Nl * N, stages, C.current_stream())

    def contract(self, a, b, incoming):
        """``a, b`` ``[B, Cl, N, N]`` -> x ``[B, Cl, N, N]``."""
        B, Cl, N, _ = a.shape
        x = torch.empty_like(a)
        mn = int(bool(incoming))
        with torch.cuda.device(a.device):
            C.call("tpf_bmm_bf16", C.ptr(a), N, N * N, mn, C.ptr(b), N, N * N, mn, C.ptr(x), N, N * N, 0, N, N, N,
                   B * Cl, 0, 128, C.current_stream())
        return x

    def contract_bwd(self, dx, a, b, incoming):
        B, Cl, N, _ = a.shape
        da, db = torch.empty_like(a), torch.empty_like(a)
        s = C.current_stream
        bm = lambda A, am, Bm, bmn, D: C.call("tpf_bmm_bf16", C.ptr(A), N, N * N, am, C.ptr(Bm), N, N * N, bmn,  # noqa: E731
                                               C.ptr(D), N, N * N, 0, N, N, N, B * Cl, 0, 128, s())
        with torch.cuda.device(a.device):
            if not incoming:
                bm(dx, 0, b, 1, da)
                bm(dx, 1, a, 1, db)
            else:
                bm(b, 0, dx, 0, da)
                bm(a, 0, dx, 1, db)
        return da, db

    def out_fwd(self, st, x_cm):
        st["x_cm"] = x_cm.contiguous()
        self._fwd(st, 4)
        return st["out"]

    def _bwd(self, st, d_out, stages, dx, da, db):
        z = st["z"]
        B, Nl, N, Cc = z.shape
        dev = z.device
        p = C.ptr
        if "ws_b" not in st:
            nbytes = C.load().tpf_trimul_bwd_stages_workspace_bytes(B, Nl * N, Cc)
            st["ws_b"] = torch.empty(nbytes, device=dev, dtype=torch.uint8)
            f32 = lambda *s: torch.zeros(s, device=dev, dtype=torch.float32)  # noqa: E731
            st["grads"] = dict(p_in_weight=f32(2 * Cc, Cc), g_in_weight=f32(2 * Cc, Cc), p_out_weight=f32(Cc, Cc),
                               g_out_weight=f32(Cc, Cc), norm_in_weight=f32(Cc), norm_in_bias=f32(Cc),
                               norm_out_weight=f32(Cc), norm_out_bias=f32(Cc))
            st["d_z"] = torch.empty_like(z)
        g = st["grads"]
        with torch.cuda.device(dev):
            C.call("tpf_trimul_bwd_stages", p(d_out), p(z), p(st["mask"]), *[p(st["w"][k]) for k in _W_BWD],
                   int(st["incoming"]), B, N, Cc, p(st["out"]), p(st["zln"]), p(st["mean_in"]), p(st["rstd_in"]),
                   p(st["a_cm"]), p(st["b_cm"]), p(st["gate"]), p(st["x_cm"]), p(st["xln"]), p(st["mean_out"]),
                   p(st["rstd_out"]), p(st["d_z"]), p(g["p_in_weight"]), p(g["g_in_weight"]), p(g["p_out_weight"]),
                   p(g["g_out_weight"]), p(g["norm_in_weight"]), p(g["norm_in_bias"]), p(g["norm_out_weight"]),
                   p(g["norm_out_bias"]), p(st["ws_b"]), st["ws_b"].numel(), Nl * N, stages, p(dx), p(da), p(db),
                   C.current_stream())

    def out_bwd(self, st, d_out):
        B, Nl, N, Cc = st["z"].shape
        if st.get("dx") is None:
            st["dx"] = torch.empty(B, Cc, Nl, N, device=st["z"].device, dtype=torch.bfloat16)
        st["d_out"] = d_out.to(torch.bfloat16).contiguous()
        self._bwd(st, st["d_out"], 1, st["dx"], None, None)
        return st["dx"]

    def proj_bwd(self, st, da, db):
        self._bwd(st, st["d_out"], 4, st["dx"], da.contiguous(), db.contiguous())
        return st["d_z"], st["grads"]


# --------------------------------------------------------------------------------------
# TriMul, rows sharded
# --------------------------------------------------------------------------------------
_WNAMES = ("norm_in_weight", "norm_in_bias", "p_in_weight", "g_in_weight", "norm_out_weight", "norm_out_bias",
           "p_out_weight", "g_out_weight")


def axial_trimul_forward(z, mask, incoming, group, backend, w):
    """Forward of the row-sharded TriMul without autograd: returns ``(out, state)``; ``state`` feeds
    :func:`axial_trimul_backward`.  Collectives: one all-to-all for a and b together (rows ->
    channels), one for x (channels -> rows)."""
    st = backend.proj_fwd(z, mask, w, incoming)
    a_c, b_c = rows_to_channels_many([st["a_cm"], st["b_cm"]], group)
    x_c = backend.contract(a_c, b_c, incoming)
    x_r = channels_to_rows(x_c, group)
    out = backend.out_fwd(st, x_r)
    return out, dict(st=st, a_c=a_c, b_c=b_c, group=group, backend=backend, incoming=incoming)


def axial_trimul_backward(state, d_out):
    """Backward of :func:`axial_trimul_forward`: returns ``(d_z, grads)`` with ``grads`` a dict of fp32
    weight / LayerNorm gradients already summed over the ranks.  Collectives: one all-to-all for d_x,
    one for d_a and d_b together, one flat all-reduce of the weight gradients."""
    be, group = state["backend"], state["group"]
    dx_r = be.out_bwd(state["st"], d_out)
    dx_c = rows_to_channels(dx_r, group)
    da_c, db_c = be.contract_bwd(dx_c, state["a_c"], state["b_c"], state["incoming"])
    da_r, db_r = channels_to_rows_many([da_c, db_c], group)
    d_z, grads = be.proj_bwd(state["st"], da_r, db_r)
    # weight / LayerNorm gradients are sums over ALL pair rows: one flat all-reduce
    flat = torch.cat([grads[n].reshape(-1).float() for n in _WNAMES])
    dist.all_reduce(flat, op=dist.ReduceOp.SUM, group=group)
    outs, off = {}, 0
    for n in _WNAMES:
        k = grads[n].numel()
        outs[n] = flat[off:off + k].reshape(grads[n].shape)
        off += k
    return d_z, outs


class _AxialTriMul(torch.autograd.Function):
    @staticmethod
    def forward(ctx, z, mask, incoming, group, backend, *wlist):
        out, state = axial_trimul_forward(z, mask, incoming, group, backend, dict(zip(_WNAMES, wlist)))
        ctx.state = state
        ctx.wdtypes = [t.dtype for t in wlist]
        return out

    @staticmethod
    def backward(ctx, d_out):
        d_z, grads = axial_trimul_backward(ctx.state, d_out)
        ctx.state = None
        return (d_z, None, None, None, None, *[grads[n].to(dt) for n, dt in zip(_WNAMES, ctx.wdtypes)])


def axial_trimul(z, direction="outgoing", mask=None, *, group=None, backend=None, **weights):
    """Row-sharded triangle multiplicative update.

    ``z``: this rank's rows ``[B, N/P, N, C]`` (bf16 on the CUDA back end); ``mask`` ``[B, N/P, N]``
    or None; weights as in :func:`turbo_trimul` (all eight are required, replicated on every rank).
    Returns the local rows of the update ``[B, N/P, N, C]``.  Weight gradients come back already
    summed over ranks."""
    if direction not in ("outgoing", "incoming"):
        raise ValueError("turbo_trimul unsupported [direction]: direction must be 'outgoing' or 'incoming'")
    missing = [n for n in _WNAMES if weights.get(n) is None]
    if missing:
        raise ValueError(f"turbo_trimul unsupported [weights]: axial_trimul needs explicit weights, missing {missing}")
    if z.dim() != 4:
        raise ValueError("turbo_trimul unsupported [z_rank]: axial_trimul takes z of shape [B, N_local, N, C]")
    P, _ = _world(group)
    B, Nl, N, Cc = z.shape
    if Nl * P != N:
        raise ValueError(f"turbo_trimul unsupported [shard]: local rows {Nl} x group size {P} != N = {N}")
    if Cc % P:
        raise ValueError(f"turbo_trimul unsupported [shard]: C = {Cc} is not divisible by the group size {P}")
    if backend is None:
        if (Nl * N) % 64:
            raise ValueError("turbo_trimul unsupported [shard]: N_local * N must be a multiple of 64")
        C.load()
        backend = CudaTrimulStages()
    if mask is None:
        mask = torch.ones((B, Nl, N), device=z.device, dtype=torch.float32)
    return _AxialTriMul.apply(z, mask.detach(), direction == "incoming", group, backend,
                              *[weights[n] for n in _WNAMES])
