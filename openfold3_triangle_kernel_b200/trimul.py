"""``turbo_trimul``: triangle multiplicative update (outgoing / incoming) on B200.

Operator contract (reference: ``turbo_trimul`` in README.md:117-143 and
docs/openfold3-integration.md:521-526; in-tree runner
openfold3/core/kernels/turbopairformer/turbopairformer_trimul.py:887-946 and support
contract turbopairformer_trimul_support.py:153-400):

* ``z``: bf16 ``[*B, N, N, C]`` with ``C in {32, 64, 96, 128}``;
  ``direction`` is ``"outgoing"`` (default) or ``"incoming"``.
* ``mask``: optional ``[*B, N, N]`` (bool / float; 1 keeps), never differentiated.
* weights, cuEquivariance-style names (…/layers/triangular_multiplicative_update.py:1592-1634):
  ``norm_in_weight, norm_in_bias [C]``, ``p_in_weight = cat[a_p, b_p] [2C, C]``,
  ``g_in_weight = cat[a_g, b_g] [2C, C]``, ``norm_out_weight, norm_out_bias [C]``,
  ``p_out_weight [C, C]`` (linear_z), ``g_out_weight [C, C]`` (linear_g); no Linear has a
  bias, LayerNorm eps is 1e-5.  Weights are fp32 masters (rounded to bf16 inside).
  When the projection / gate matrices are omitted they are sampled per call
  (Xavier-normal) and the norms default to ones / zeros; sampled parameters get no
  gradient.
* second calling form ``turbo_trimul(module, z, mask=None)`` with an OpenFold3
  ``TriangleMultiplicativeUpdate``-like module (``linear_{a_p,a_g,b_p,b_g,g,z}``,
  ``layer_norm_{in,out}``, ``_outgoing``).
* returns bf16 ``[*B, N, N, C]``; autograd for z, the six matrices and the four norm
  vectors (first order only).

Unlike the reference (N > 100 only) any ``N >= 1`` is accepted; N that is not a multiple
of 8 is zero-padded with masked-out rows/columns and cropped again.
Unsupported inputs raise ``ValueError("... unsupported [code]: reason")``.
"""
from __future__ import annotations

import math

import torch

from . import _cabi as C

SUPPORTED_CHANNELS = (32, 64, 96, 128)
_LN_EPS = 1e-5
_WEIGHT_NAMES = ("norm_in_weight", "norm_in_bias", "p_in_weight", "g_in_weight",
                 "norm_out_weight", "norm_out_bias", "p_out_weight", "g_out_weight")


class SupportResult(tuple):
    """``(supported, code, reason)`` (reference: SupportResult, turbopairformer_trimul_support.py:52-65)."""

    def __new__(cls, supported, code, reason):
        return super().__new__(cls, (supported, code, reason))

    supported = property(lambda s: s[0])
    code = property(lambda s: s[1])
    reason = property(lambda s: s[2])


def check_trimul_support(z, direction, mask, weights, *, check_device=True) -> SupportResult:
    """Metadata-only contract check; returns the first failure."""
    if not isinstance(z, torch.Tensor):
        return SupportResult(False, "z_type", "z must be a torch.Tensor")
    if direction not in ("outgoing", "incoming"):
        return SupportResult(False, "direction", "direction must be 'outgoing' or 'incoming'")
    if z.ndim < 4:
        return SupportResult(False, "z_rank", "z must have shape [*B,N,N,C]")
    if z.dtype != torch.bfloat16:
        return SupportResult(False, "z_dtype", "z must be BF16")
    n1, n2, c = z.shape[-3:]
    if n1 != n2 or n1 < 1:
        return SupportResult(False, "z_square", "z must be square in its two residue dimensions")
    if c not in SUPPORTED_CHANNELS:
        return SupportResult(False, "channels", f"C={c} not in {SUPPORTED_CHANNELS}")
    if any(d <= 0 for d in z.shape[:-3]):
        return SupportResult(False, "batch", "batch dimensions must be positive")
    if check_device:
        if not z.is_cuda:
            return SupportResult(False, "device", "z must be a CUDA tensor")
        if torch.cuda.get_device_capability(z.device)[0] != 10:
            return SupportResult(False, "device_arch", "these kernels require a Blackwell sm_100a device")
    if mask is not None:
        if not isinstance(mask, torch.Tensor):
            return SupportResult(False, "mask_type", "mask must be a torch.Tensor")
        if mask.dtype not in (torch.bool, torch.bfloat16, torch.float32, torch.float16):
            return SupportResult(False, "mask_dtype", "mask must be bool, BF16, FP16 or FP32")
        try:
            if tuple(torch.broadcast_shapes(tuple(mask.shape), tuple(z.shape[:-1]))) != tuple(z.shape[:-1]):
                raise RuntimeError
        except RuntimeError:
            return SupportResult(False, "mask_shape", "mask must broadcast to [*B,N,N]")
        if mask.requires_grad:
            return SupportResult(False, "mask_grad", "mask must not require gradients")
    shapes = {"norm_in_weight": (c,), "norm_in_bias": (c,), "norm_out_weight": (c,), "norm_out_bias": (c,),
              "p_in_weight": (2 * c, c), "g_in_weight": (2 * c, c), "p_out_weight": (c, c), "g_out_weight": (c, c)}
    for name in _WEIGHT_NAMES:
        w = weights.get(name)
        if w is None:
            continue
        if not isinstance(w, torch.Tensor) or tuple(w.shape) != shapes[name]:
            return SupportResult(False, "weight_shape", f"{name} must have shape {shapes[name]}")
        if not w.dtype.is_floating_point:
            return SupportResult(False, "weight_dtype", f"{name} must be floating point")
        if w.device != z.device:
            return SupportResult(False, "weight_device", f"{name} must live on z's device")
    return SupportResult(True, "ok", "supported")


# --------------------------------------------------------------------------------------
# custom ops
# --------------------------------------------------------------------------------------
def _f32c(t):
    return t.detach().to(torch.float32).contiguous()


@torch.library.custom_op("tpf_b200::trimul_fwd", mutates_args=())
def _trimul_fwd(z: torch.Tensor, mask: torch.Tensor, p_in: torch.Tensor, g_in: torch.Tensor, p_out: torch.Tensor,
                g_out: torch.Tensor, nin_w: torch.Tensor, nin_b: torch.Tensor, nout_w: torch.Tensor,
                nout_b: torch.Tensor, incoming: bool) -> list[torch.Tensor]:
    B, N, _, Cc = z.shape
    R = B * N * N
    dev = z.device
    z = z.contiguous()
    mask = mask.to(torch.float32).contiguous()
    ws = [_f32c(t) for t in (p_in, g_in, p_out, g_out, nin_w, nin_b, nout_w, nout_b)]
    bf = lambda *s: torch.empty(s, device=dev, dtype=torch.bfloat16)  # noqa: E731
    f32 = lambda *s: torch.empty(s, device=dev, dtype=torch.float32)  # noqa: E731
    out, zln, gate, xln = bf(B, N, N, Cc), bf(R, Cc), bf(R, Cc), bf(R, Cc)
    a_cm, b_cm, x_cm = bf(B * Cc, N * N), bf(B * Cc, N * N), bf(B * Cc, N * N)
    mean_in, rstd_in, mean_out, rstd_out = f32(R), f32(R), f32(R), f32(R)
    nbytes = C.load().tpf_trimul_fwd_workspace_bytes(B, N, Cc)
    wsb = torch.empty((max(nbytes, 256),), device=dev, dtype=torch.uint8)
    with torch.cuda.device(dev):
        C.call("tpf_trimul_fwd", C.ptr(z), C.ptr(mask), *[C.ptr(t) for t in ws], int(incoming), B, N, Cc,
               C.ptr(out), C.ptr(zln), C.ptr(mean_in), C.ptr(rstd_in), C.ptr(a_cm), C.ptr(b_cm), C.ptr(gate),
               C.ptr(x_cm), C.ptr(xln), C.ptr(mean_out), C.ptr(rstd_out), C.ptr(wsb), nbytes, C.current_stream())
    return [out, zln, mean_in, rstd_in, a_cm, b_cm, gate, x_cm, xln, mean_out, rstd_out]


@_trimul_fwd.register_fake
def _(z, mask, p_in, g_in, p_out, g_out, nin_w, nin_b, nout_w, nout_b, incoming):
    B, N, _, Cc = z.shape
    R = B * N * N
    bf = lambda *s: z.new_empty(s, dtype=torch.bfloat16)  # noqa: E731
    f32 = lambda *s: z.new_empty(s, dtype=torch.float32)  # noqa: E731
    return [bf(B, N, N, Cc), bf(R, Cc), f32(R), f32(R), bf(B * Cc, N * N), bf(B * Cc, N * N), bf(R, Cc),
            bf(B * Cc, N * N), bf(R, Cc), f32(R), f32(R)]


@torch.library.custom_op("tpf_b200::trimul_bwd", mutates_args=())
def _trimul_bwd(d_out: torch.Tensor, z: torch.Tensor, mask: torch.Tensor, p_in: torch.Tensor, g_in: torch.Tensor,
                p_out: torch.Tensor, g_out: torch.Tensor, nin_w: torch.Tensor, nout_w: torch.Tensor, incoming: bool,
                out: torch.Tensor, zln: torch.Tensor, mean_in: torch.Tensor, rstd_in: torch.Tensor,
                a_cm: torch.Tensor, b_cm: torch.Tensor, gate: torch.Tensor, x_cm: torch.Tensor, xln: torch.Tensor,
                mean_out: torch.Tensor, rstd_out: torch.Tensor) -> list[torch.Tensor]:
    B, N, _, Cc = z.shape
    dev = z.device
    d_out = d_out.to(torch.bfloat16).contiguous()
    z = z.contiguous()
    mask = mask.to(torch.float32).contiguous()
    ws = [_f32c(t) for t in (p_in, g_in, p_out, g_out, nin_w, nout_w)]
    f32 = lambda *s: torch.empty(s, device=dev, dtype=torch.float32)  # noqa: E731
    d_z = torch.empty_like(z)
    d_p_in, d_g_in, d_p_out, d_g_out = f32(2 * Cc, Cc), f32(2 * Cc, Cc), f32(Cc, Cc), f32(Cc, Cc)
    d_nin_w, d_nin_b, d_nout_w, d_nout_b = f32(Cc), f32(Cc), f32(Cc), f32(Cc)
    nbytes = C.load().tpf_trimul_bwd_workspace_bytes(B, N, Cc)
    wsb = torch.empty((max(nbytes, 256),), device=dev, dtype=torch.uint8)
    with torch.cuda.device(dev):
        C.call("tpf_trimul_bwd", C.ptr(d_out), C.ptr(z), C.ptr(mask), *[C.ptr(t) for t in ws], int(incoming), B, N,
               Cc, C.ptr(out), C.ptr(zln), C.ptr(mean_in), C.ptr(rstd_in), C.ptr(a_cm), C.ptr(b_cm), C.ptr(gate),
               C.ptr(x_cm), C.ptr(xln), C.ptr(mean_out), C.ptr(rstd_out), C.ptr(d_z), C.ptr(d_p_in), C.ptr(d_g_in),
               C.ptr(d_p_out), C.ptr(d_g_out), C.ptr(d_nin_w), C.ptr(d_nin_b), C.ptr(d_nout_w), C.ptr(d_nout_b),
               C.ptr(wsb), nbytes, C.current_stream())
    return [d_z, d_p_in, d_g_in, d_p_out, d_g_out, d_nin_w, d_nin_b, d_nout_w, d_nout_b]


@_trimul_bwd.register_fake
def _(d_out, z, mask, p_in, g_in, p_out, g_out, nin_w, nout_w, incoming, out, zln, mean_in, rstd_in, a_cm, b_cm,
      gate, x_cm, xln, mean_out, rstd_out):
    Cc = z.shape[-1]
    f32 = lambda *s: z.new_empty(s, dtype=torch.float32)  # noqa: E731
    return [torch.empty_like(z), f32(2 * Cc, Cc), f32(2 * Cc, Cc), f32(Cc, Cc), f32(Cc, Cc), f32(Cc), f32(Cc),
            f32(Cc), f32(Cc)]


def _trimul_setup_context(ctx, inputs, output):
    z, mask, p_in, g_in, p_out, g_out, nin_w, nin_b, nout_w, nout_b, incoming = inputs
    ctx.save_for_backward(z, mask, p_in, g_in, p_out, g_out, nin_w, nout_w, *output)
    ctx.incoming = incoming
    ctx.dtypes = tuple(t.dtype for t in (p_in, g_in, p_out, g_out, nin_w, nin_b, nout_w, nout_b))
    ctx.set_materialize_grads(False)


def _trimul_backward(ctx, grads):
    d_out = grads[0]
    if d_out is None:
        return (None,) * 11
    saved = ctx.saved_tensors
    z, mask, p_in, g_in, p_out, g_out, nin_w, nout_w = saved[:8]
    res = torch.ops.tpf_b200.trimul_bwd(d_out, z, mask, p_in, g_in, p_out, g_out, nin_w, nout_w, ctx.incoming,
                                        *saved[8:])
    d_z, d_p_in, d_g_in, d_p_out, d_g_out, d_nin_w, d_nin_b, d_nout_w, d_nout_b = res
    wgrads = [g.to(dt) for g, dt in zip((d_p_in, d_g_in, d_p_out, d_g_out, d_nin_w, d_nin_b, d_nout_w, d_nout_b),
                                        ctx.dtypes)]
    return (d_z, None, *wgrads, None)


_trimul_fwd.register_autograd(_trimul_backward, setup_context=_trimul_setup_context)


# --------------------------------------------------------------------------------------
# public operator
# --------------------------------------------------------------------------------------
def sample_weights(c, device, generator=None):
    """Per-call parameters for the weight-less calling form: Xavier-normal matrices,
    unit norms (README.md:143 states they are sampled per call; the distribution is this
    build's choice)."""
    std = math.sqrt(2.0 / (c + c))
    rn = lambda r: torch.randn(r, c, device=device, generator=generator) * std  # noqa: E731
    return dict(norm_in_weight=torch.ones(c, device=device), norm_in_bias=torch.zeros(c, device=device),
                p_in_weight=rn(2 * c), g_in_weight=rn(2 * c),
                norm_out_weight=torch.ones(c, device=device), norm_out_bias=torch.zeros(c, device=device),
                p_out_weight=rn(c), g_out_weight=rn(c))


def _weights_from_module(module):
    """OpenFold3 module -> cuEq-style weights (same mapping as
    …/layers/triangular_multiplicative_update.py:1231-1256)."""
    for lin in ("linear_a_p", "linear_a_g", "linear_b_p", "linear_b_g", "linear_g", "linear_z"):
        if getattr(getattr(module, lin), "bias", None) is not None:
            raise ValueError(f"turbo_trimul unsupported [linear_bias]: {lin} must not have a bias")
    for ln in ("layer_norm_in", "layer_norm_out"):
        if abs(float(getattr(getattr(module, ln), "eps", _LN_EPS)) - _LN_EPS) > 0:
            raise ValueError(f"turbo_trimul unsupported [ln_eps]: {ln}.eps must be 1e-5")
    w = dict(
        norm_in_weight=module.layer_norm_in.weight, norm_in_bias=module.layer_norm_in.bias,
        p_in_weight=torch.cat([module.linear_a_p.weight, module.linear_b_p.weight]),
        g_in_weight=torch.cat([module.linear_a_g.weight, module.linear_b_g.weight]),
        norm_out_weight=module.layer_norm_out.weight, norm_out_bias=module.layer_norm_out.bias,
        p_out_weight=module.linear_z.weight, g_out_weight=module.linear_g.weight)
    return w, ("outgoing" if getattr(module, "_outgoing", True) else "incoming")


def turbo_trimul(z, direction="outgoing", mask=None, *, generator=None, **weights):
    """Triangle multiplicative update.  ``turbo_trimul(z, direction, mask, **weights)`` or
    ``turbo_trimul(module, z, mask)``; see the module docstring."""
    if isinstance(z, torch.nn.Module):
        module = z
        z = direction
        if isinstance(mask, str):
            raise ValueError("turbo_trimul unsupported [call_form]: use turbo_trimul(module, z, mask=None)")
        mod_weights, direction = _weights_from_module(module)
        mod_weights.update(weights)
        weights = mod_weights
    unknown = set(weights) - set(_WEIGHT_NAMES)
    if unknown:
        raise TypeError(f"turbo_trimul got unexpected keyword arguments {sorted(unknown)}")
    # Under torch.compile / torch.export the function is traced once on fake tensors: the metadata
    # contract is checked when it runs eagerly, and by the fake kernel and the C ABI in either case.
    if not torch.compiler.is_compiling():
        res = check_trimul_support(z, direction, mask, weights)
        if not res.supported:
            raise ValueError(f"turbo_trimul unsupported [{res.code}]: {res.reason}")
        C.load()

    c = int(z.shape[-1])
    n = int(z.shape[-2])
    prefix = tuple(z.shape[:-3])
    B = 1
    for d in prefix:
        B *= int(d)
    if any(weights.get(k) is None for k in ("p_in_weight", "g_in_weight", "p_out_weight", "g_out_weight")):
        sampled = sample_weights(c, z.device, generator)
        for k in _WEIGHT_NAMES:
            if weights.get(k) is None:
                weights[k] = sampled[k]
    else:
        for k, fill in (("norm_in_weight", 1.0), ("norm_in_bias", 0.0), ("norm_out_weight", 1.0),
                        ("norm_out_bias", 0.0)):
            if weights.get(k) is None:
                weights[k] = torch.full((c,), fill, device=z.device)

    zf = z.reshape(B, n, n, c)
    if mask is None:
        mask_f = torch.ones((B, n, n), device=z.device, dtype=torch.float32)
    else:
        mask_f = mask.detach().to(torch.float32).expand(prefix + (n, n)).reshape(B, n, n)
    pad = (-n) % 8
    if pad:
        zf = torch.nn.functional.pad(zf, (0, 0, 0, pad, 0, pad))
        mask_f = torch.nn.functional.pad(mask_f, (0, pad, 0, pad))
    outs = torch.ops.tpf_b200.trimul_fwd(
        zf, mask_f, weights["p_in_weight"], weights["g_in_weight"], weights["p_out_weight"], weights["g_out_weight"],
        weights["norm_in_weight"], weights["norm_in_bias"], weights["norm_out_weight"], weights["norm_out_bias"],
        direction == "incoming")
    out = outs[0]
    if pad:
        out = out[:, :n, :n, :]
    return out.reshape(prefix + (n, n, c))
