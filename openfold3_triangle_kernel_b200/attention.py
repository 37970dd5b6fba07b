"""``turbo_attention``: triangle attention (starting / ending node) on B200.

Operator contract (same as the reference's ``turbo_attention`` /
``turbopairformer_triangle_attention``,
openfold3/core/kernels/turbopairformer/turbopairformer_triangle_attention.py:341-472
and README.md:84-115):

* ``q, k, v``: bf16 ``[*B, O, H, N, D]``, ``1 <= D <= 64``; **unscaled** Q, the kernel
  applies ``D ** -0.5``.  Both storage orders of the reference are read in
  place: contiguous ``[*B,O,H,N,D]`` and a contiguous ``[*B,O,N,H,D]`` tensor viewed
  as ``[*B,O,H,N,D]``.
* ``pair_bias``: required, bf16 or fp32 ``[*B, 1, H, N, N]`` (prefix broadcastable).
* ``res_mask``: optional additive floating mask ``[*B, O, 1, 1, N]`` (0 keeps,
  ``-inf`` or a large negative drops); no boolean masks; never differentiated.
* returns bf16 ``[*B, O, N, H, D]``; autograd for q, k, v and pair_bias
  (the bias gradient has pair_bias's shape and dtype).

Unsupported inputs raise ``ValueError("unsupported TurboPairFormer case: ...")``
before anything is launched.  There is no fallback path: the device is reached
only through the C-ABI library.
"""
from __future__ import annotations

import math

import torch

from . import _cabi as C

_HEAD_LANES = (16, 32, 64)
_MAX_BROADCAST_PREFIX_RANK = 16
_INVOCATIONS = 0


def invocation_count() -> int:
    """Number of ``turbo_attention`` calls that reached the kernels (reference:
    ``_INVOCATIONS``, turbopairformer_triangle_attention.py:57-66)."""
    return _INVOCATIONS


# --------------------------------------------------------------------------------------
# support predicate (metadata only)
# --------------------------------------------------------------------------------------
def is_turbo_attention_supported(q, k, v, res_mask, pair_bias, *, check_device=True):
    """``(ok, reason)`` without reading tensor values.  Mirrors the order of checks of
    ``_is_turbopairformer_supported_uncached`` (…_triangle_attention.py:126-220) with
    the device requirement changed from Hopper to compute capability 10.x."""
    named = {"q": q, "k": k, "v": v, "res_mask": res_mask, "pair_bias": pair_bias}
    if any(not isinstance(t, torch.Tensor) for t in named.values()):
        return False, "all inputs must be torch.Tensor instances"
    if check_device:
        if not q.is_cuda:
            return False, "q/k/v, res_mask, and pair_bias must be CUDA tensors"
        if torch.cuda.get_device_capability(q.device)[0] != 10:
            return False, "these kernels require a Blackwell sm_100a device"
    if q.ndim < 5:
        return False, "q must have shape [*B,O,H,N,D]"
    prefix = tuple(q.shape[:-4])
    outer, heads, sequence, head_dim = q.shape[-4:]
    if not prefix or any(d <= 0 for d in prefix):
        return False, "requires a positive batch prefix"
    if outer <= 0 or sequence <= 0:
        return False, "requires positive outer and key sequence dimensions"
    if heads < 1 or head_dim < 1 or head_dim > _HEAD_LANES[-1]:
        return False, "requires H>=1 and D<=64 (pads to lanes {16,32,64})"
    for name, t in (("k", k), ("v", v)):
        if t.shape != q.shape:
            return False, f"{name} shape must match q"
    if any(t.dtype != torch.bfloat16 for t in (q, k, v)):
        return False, "q/k/v must be BF16"
    if res_mask.dtype not in (torch.float32, torch.bfloat16, torch.float16):
        return False, "res_mask must be a floating additive mask"
    if tuple(res_mask.shape[-4:]) != (outer, 1, 1, sequence):
        return False, "res_mask tail must be (O,1,1,N)"
    if tuple(pair_bias.shape[-4:]) != (1, heads, sequence, sequence):
        return False, "pair_bias tail must be (1,H,N,N)"
    if pair_bias.dtype not in (torch.bfloat16, torch.float32):
        return False, "pair_bias must be BF16 or FP32"
    if len({t.device for t in named.values()}) != 1:
        return False, "q/k/v, res_mask, and pair_bias must share one device"
    for name, t in (("res_mask", res_mask), ("pair_bias", pair_bias)):
        try:
            bp = torch.broadcast_shapes(prefix, tuple(t.shape[:-4]))
        except RuntimeError:
            return False, f"{name} prefix is not broadcastable to q prefix"
        if tuple(bp) != prefix:
            return False, f"{name} prefix must broadcast exactly to q prefix"
    if len(prefix) > _MAX_BROADCAST_PREFIX_RANK and tuple(pair_bias.shape[:-4]) != prefix:
        return False, "pair_bias broadcast supports at most 16 target-prefix dimensions"
    if res_mask.requires_grad:
        return False, "res_mask must not require gradients"
    return True, "supported"


# --------------------------------------------------------------------------------------
# custom ops (flattened batch, padded head dim): the only callers of the C ABI
# --------------------------------------------------------------------------------------
def _kernel_layout(t):
    """A [B,O,H,N,D] tensor the TMA descriptors can describe: last dim contiguous,
    16-byte aligned base and strides.  Anything else is copied once."""
    ok = t.stride(-1) == 1 and t.data_ptr() % 16 == 0 and all((s * 2) % 16 == 0 for s in t.stride()[:-1])
    return t if ok else t.contiguous()


def _prep_mask_bias(mask, bias, n):
    """mask fp32 [B,O,N] -> row pitch multiple of 4; bias bf16 [G,H,N,N] -> row pitch multiple of 8."""
    mp = (n + 3) // 4 * 4
    if mask.dtype != torch.float32 or mp != n or not mask.is_contiguous():
        m = mask.new_zeros(mask.shape[:-1] + (mp,), dtype=torch.float32)
        m[..., :n] = mask
        mask = m
    bp = (n + 7) // 8 * 8
    if bias.dtype != torch.bfloat16 or bp != n or not bias.is_contiguous():
        b = bias.new_zeros(bias.shape[:-1] + (bp,), dtype=torch.bfloat16)
        b[..., :n] = bias
        bias = b
    return mask, mp, bias, bp


@torch.library.custom_op("tpf_b200::attn_fwd", mutates_args=())
def _attn_fwd(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, mask: torch.Tensor, bias: torch.Tensor,
              scale: float) -> tuple[torch.Tensor, torch.Tensor]:
    B, O, H, N, D = q.shape
    q, k, v = (_kernel_layout(t) for t in (q, k, v))
    mask_p, mp, bias_p, bp = _prep_mask_bias(mask, bias, N)
    out = torch.empty((B, O, N, H, D), device=q.device, dtype=torch.bfloat16)
    lse = torch.empty((B, O, H, N), device=q.device, dtype=torch.float32)
    with torch.cuda.device(q.device):
        C.call("tpf_attn_fwd", C.ptr(q), C.ptr(k), C.ptr(v), C.i64_array(q.stride()[:4]),
               C.i64_array(k.stride()[:4]), C.i64_array(v.stride()[:4]), C.ptr(mask_p), mp, C.ptr(bias_p), bp,
               bias.shape[0], C.ptr(out), C.ptr(lse), B, O, H, N, D, float(scale), C.current_stream())
    return out, lse


@_attn_fwd.register_fake
def _(q, k, v, mask, bias, scale):
    B, O, H, N, D = q.shape
    return (q.new_empty((B, O, N, H, D), dtype=torch.bfloat16), q.new_empty((B, O, H, N), dtype=torch.float32))


@torch.library.custom_op("tpf_b200::attn_bwd", mutates_args=())
def _attn_bwd(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, d_out: torch.Tensor, out: torch.Tensor,
              lse: torch.Tensor, mask: torch.Tensor, bias: torch.Tensor,
              scale: float) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor]:
    B, O, H, N, D = q.shape
    G = bias.shape[0]
    q, k, v = (_kernel_layout(t) for t in (q, k, v))
    d_out = d_out.contiguous()
    out = out.contiguous()
    mask_p, mp, bias_p, bp = _prep_mask_bias(mask, bias, N)
    dq, dk, dv = (torch.empty((B, O, H, N, D), device=q.device, dtype=torch.bfloat16) for _ in range(3))
    dbias = torch.empty((G, H, N, N), device=q.device, dtype=torch.float32)
    delta = torch.empty((B, O, H, N), device=q.device, dtype=torch.float32)
    ws_bytes = C.load().tpf_attn_bwd_workspace_bytes(B, O, H, N, D, G)
    ws = torch.empty((max(ws_bytes, 256),), device=q.device, dtype=torch.uint8)
    with torch.cuda.device(q.device):
        C.call("tpf_attn_bwd", C.ptr(q), C.ptr(k), C.ptr(v), C.ptr(d_out), C.i64_array(q.stride()[:4]),
               C.i64_array(k.stride()[:4]), C.i64_array(v.stride()[:4]), C.ptr(out), C.ptr(lse), C.ptr(mask_p), mp,
               C.ptr(bias_p), bp, G, C.ptr(dq), C.ptr(dk), C.ptr(dv), C.ptr(dbias), C.ptr(delta), C.ptr(ws), ws_bytes,
               B, O, H, N, D, float(scale), C.current_stream())
    return dq, dk, dv, dbias


@_attn_bwd.register_fake
def _(q, k, v, d_out, out, lse, mask, bias, scale):
    B, O, H, N, D = q.shape
    e = lambda: q.new_empty((B, O, H, N, D), dtype=torch.bfloat16)  # noqa: E731
    return e(), e(), e(), q.new_empty((bias.shape[0], H, N, N), dtype=torch.float32)


def _attn_setup_context(ctx, inputs, output):
    q, k, v, mask, bias, scale = inputs
    out, lse = output
    ctx.save_for_backward(q, k, v, mask, bias, out, lse)
    ctx.scale = scale
    # the log-sum-exp is a by-product for callers that ask for it, not a differentiable output
    ctx.mark_non_differentiable(lse)


def _attn_backward(ctx, d_out, d_lse):
    q, k, v, mask, bias, out, lse = ctx.saved_tensors
    dq, dk, dv, dbias = torch.ops.tpf_b200.attn_bwd(q, k, v, d_out, out, lse, mask, bias, ctx.scale)
    return dq, dk, dv, None, dbias.to(bias.dtype), None


_attn_fwd.register_autograd(_attn_backward, setup_context=_attn_setup_context)


# --------------------------------------------------------------------------------------
# public operator
# --------------------------------------------------------------------------------------
def turbo_attention(q, k, v, pair_bias=None, res_mask=None, *, return_lse=False):
    """Triangle attention ``softmax(q k^T / sqrt(D) + res_mask + pair_bias) v``.

    See the module docstring for the contract.  ``return_lse=True`` additionally
    returns the fp32 log-sum-exp ``[*B, O, H, N]`` (``-inf`` for fully masked rows).
    """
    global _INVOCATIONS
    if pair_bias is None:
        raise ValueError("unsupported TurboPairFormer case: pair_bias is required (pass zeros if there is none)")
    if res_mask is None:
        if not isinstance(q, torch.Tensor) or q.ndim < 5:
            raise ValueError("unsupported TurboPairFormer case: q must have shape [*B,O,H,N,D]")
        res_mask = q.new_zeros(q.shape[:-4] + (q.shape[-4], 1, 1, q.shape[-2]), dtype=torch.float32)
    # Under torch.compile / torch.export the function is traced once on fake tensors: the metadata
    # contract is checked when it runs eagerly, and by the fake kernel and the C ABI in either case.
    if not torch.compiler.is_compiling():
        ok, reason = is_turbo_attention_supported(q, k, v, res_mask, pair_bias)
        if not ok:
            raise ValueError(f"unsupported TurboPairFormer case: {reason}")
        C.load()  # fail loudly when the native library is missing
        _INVOCATIONS += 1

    prefix = tuple(q.shape[:-4])
    O, H, N, D = (int(x) for x in q.shape[-4:])
    B = 1
    for d in prefix:
        B *= int(d)
    scale = 1.0 / math.sqrt(D)

    # head dim -> one of the compiled lanes (zero columns change nothing; the scale keeps the true D)
    lane = next(x for x in _HEAD_LANES if x >= D)
    if lane != D:
        pad = (0, lane - D)
        q, k, v = (torch.nn.functional.pad(t, pad) for t in (q, k, v))

    qf, kf, vf = (t.reshape((B,) + tuple(t.shape[-4:])) for t in (q, k, v))
    mask_f = res_mask.expand(prefix + tuple(res_mask.shape[-4:])).reshape(B, O, N).detach()

    bias_prefix = tuple(pair_bias.shape[:-4])
    if all(d == 1 for d in bias_prefix):
        bias_f = pair_bias.reshape(1, H, N, N)
    else:
        bias_f = pair_bias.expand(prefix + tuple(pair_bias.shape[-4:])).reshape(B, H, N, N)

    out, lse = torch.ops.tpf_b200.attn_fwd(qf, kf, vf, mask_f, bias_f, scale)
    if lane != D:
        out = out[..., :D]
    out = out.reshape(prefix + (O, N, H, D))
    if return_lse:
        return out, lse.reshape(prefix + (O, H, N))
    return out
