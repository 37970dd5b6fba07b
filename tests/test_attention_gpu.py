"""turbo_attention on a B200 against the CPU oracle, the reference-generated golden
fixture and the reference's own acceptance envelope
(tools/aot_numeric_smoke.py:94-180: err <= 1.1 * stock_bf16_err + 1e-6 vs FP64, bitwise
replay, fully masked planes exactly zero)."""
import math
import os

import numpy as np
import pytest
import torch

import openfold3_triangle_kernel_b200 as tk
from openfold3_triangle_kernel_b200 import _cabi as C
from oracle import attention_oracle as ao
from oracle.inputs import attention_inputs, attention_inputs_cpu_case

pytestmark = [pytest.mark.gpu, pytest.mark.skipif(not torch.cuda.is_available(), reason="needs a CUDA device")]

# bf16 outputs / grads within ~1e-2 relative (L2) of the fp32/fp64 reference; log-sum-exp within 1e-5
REL_TOL = 1e-2
LSE_TOL = 1e-5


def _run(inp, d_out=None, loss="mean_sq"):
    dev = "cuda"
    q, k, v, b = (inp[n].to(dev).bfloat16().requires_grad_(True) for n in ("q", "k", "v", "pair_bias"))
    m = inp["res_mask"].to(dev)
    out, lse = tk.turbo_attention(q, k, v, pair_bias=b, res_mask=m, return_lse=True)
    if d_out is None:
        d_out = (2.0 * out.detach().float() / out.numel()).bfloat16()
    out.backward(d_out.to(dev))
    torch.cuda.synchronize()
    assert C.device_status() == 0
    res = dict(out=out.detach(), lse=lse.detach(), dq=q.grad, dk=k.grad, dv=v.grad, dbias=b.grad)
    return {k_: v_.cpu() for k_, v_ in res.items()}, d_out.cpu()


def _oracle(inp, d_out, dtype=torch.float64):
    q, k, v, b = (inp[n].bfloat16() for n in ("q", "k", "v", "pair_bias"))
    return ao.attention_forward_backward(q, k, v, b, inp["res_mask"], d_out, dtype=dtype)


def _check(got, ref, tol=REL_TOL, names=("out", "dq", "dk", "dv", "dbias")):
    for n in names:
        assert torch.isfinite(got[n].float()).all(), n
        e = ao.rel_l2(got[n], ref[n])
        assert e <= tol, (n, e)
    fin = torch.isfinite(ref["lse"])
    assert (got["lse"][fin].double() - ref["lse"][fin].double()).abs().max().item() <= LSE_TOL * max(
        1.0, ref["lse"][fin].abs().max().item())
    assert torch.equal(torch.isneginf(got["lse"]), ~fin)


def test_cpu_reference_config_against_golden_fixture(golden_dir):
    """Config 'CPU reference': B=1, O=N=64, H=4, D=32, last 8 keys -inf, loss = mean(out^2).
    The fixture holds the fp32 outputs of the reference's stock _attention."""
    gold = np.load(os.path.join(golden_dir, "attention_cpu_case.npz"))
    inp = attention_inputs_cpu_case(seed=0)
    got, d_out = _run(inp)
    sub = slice(None, None, 4)
    # inputs are rounded to bf16 for the kernel, so compare at the operator tolerance
    assert ao.rel_l2(got["out"][:, sub], torch.from_numpy(gold["out"])) <= REL_TOL
    for n in ("dq", "dk", "dv"):
        assert ao.rel_l2(got[n][:, sub], torch.from_numpy(gold[n])) <= 2 * REL_TOL, n
    assert ao.rel_l2(got["dbias"], torch.from_numpy(gold["dbias"])) <= 2 * REL_TOL
    # and tightly against the oracle on exactly the bf16 inputs the kernel saw
    _check(got, _oracle(inp, d_out), tol=5e-3)


REFERENCE_CASES = [  # tools/aot_numeric_smoke.py:94-140 (shapes, mask fraction, fully masked planes)
    dict(B=1, O=8, H=4, N=128, D=32, mask_frac=0.0, full=0),
    dict(B=1, O=8, H=4, N=100, D=32, mask_frac=0.3, full=0),
    dict(B=1, O=4, H=4, N=384, D=24, mask_frac=0.2, full=0),
    dict(B=2, O=4, H=4, N=200, D=20, mask_frac=0.2, full=0),
    dict(B=1, O=6, H=4, N=256, D=64, mask_frac=0.2, full=2),
    dict(B=1, O=2, H=4, N=384, D=48, mask_frac=0.1, full=0),
    dict(B=1, O=2, H=8, N=768, D=16, mask_frac=0.1, full=0),
]


@pytest.mark.parametrize("case", REFERENCE_CASES, ids=lambda c: f"N{c['N']}D{c['D']}")
def test_reference_acceptance_envelope(case):
    g = torch.Generator().manual_seed(0)
    B, O, H, N, D = (case[k] for k in "BOHND")
    q, k, v = (torch.randn(B, O, H, N, D, generator=g).bfloat16() for _ in range(3))
    mask = torch.zeros(B, O, 1, 1, N)
    if case["mask_frac"]:
        mask[torch.rand(B, O, 1, 1, N, generator=g) < case["mask_frac"]] = float("-inf")
    if case["full"]:
        mask[:, :case["full"]] = float("-inf")
    bias = (torch.randn(1, 1, H, N, N, generator=g) * 2).bfloat16()
    d_out = torch.randn(B, O, N, H, D, generator=g).bfloat16()
    if case["full"]:
        d_out[:, :case["full"]] = 0
    inp = dict(q=q, k=k, v=v, pair_bias=bias, res_mask=mask)
    got, _ = _run(inp, d_out)
    replay, _ = _run(inp, d_out)
    for n in got:  # bitwise self-replay
        assert torch.equal(got[n].view(torch.uint8), replay[n].view(torch.uint8)), n
    ref = ao.attention_forward_backward(q, k, v, bias, mask, d_out, dtype=torch.float64)
    full = case["full"]
    if full:
        for n in ("out", "dq", "dk", "dv"):
            assert got[n][:, :full].abs().max().item() == 0.0, n
        assert torch.isneginf(got["lse"][:, :full]).all()
    stock = ao.stock_bf16_forward_backward(q, k, v, bias, mask, d_out)
    for n in ("out", "dq", "dk", "dv", "dbias"):
        sl = slice(full, None) if (full and n == "out") else slice(None)
        err = ao.rel_l2(got[n][:, sl], ref[n][:, sl])
        base = ao.rel_l2(stock[n][:, sl], ref[n][:, sl])
        assert err <= 1.1 * base + 1e-6, (n, err, base)


def test_strided_sequence_major_and_broadcast_bias():
    """q/k/v given as a [B,O,N,H,D] tensor viewed as [B,O,H,N,D]; fp32 bias broadcast over a
    2-D batch prefix (reference: test_turbopairformer_sr_policy.py:232-256)."""
    g = torch.Generator().manual_seed(3)
    P0, P1, O, H, N, D = 2, 2, 3, 2, 72, 32
    mk = lambda: torch.randn(P0, P1, O, N, H, D, generator=g).bfloat16()  # noqa: E731
    qs, ks, vs = mk(), mk(), mk()
    bias = torch.randn(1, P1, 1, H, N, N, generator=g)
    mask = torch.zeros(P0, 1, O, 1, 1, N)
    mask[..., N - 5:] = -1e9
    dev = "cuda"
    qd, kd, vd = (t.to(dev).requires_grad_(True) for t in (qs, ks, vs))
    bd = bias.to(dev).requires_grad_(True)
    out = tk.turbo_attention(qd.transpose(-2, -3), kd.transpose(-2, -3), vd.transpose(-2, -3), pair_bias=bd,
                             res_mask=mask.to(dev))
    d_out = torch.randn(out.shape, generator=g).bfloat16()
    out.backward(d_out.to(dev))
    assert bd.grad.dtype == torch.float32 and bd.grad.shape == bias.shape
    ref = ao.attention_forward_backward(qs.transpose(-2, -3), ks.transpose(-2, -3), vs.transpose(-2, -3),
                                        bias.bfloat16(), mask.expand(P0, P1, O, 1, 1, N), d_out)
    assert ao.rel_l2(out.cpu(), ref["out"]) <= REL_TOL
    assert ao.rel_l2(qd.grad.cpu().transpose(-2, -3), ref["dq"]) <= REL_TOL
    assert ao.rel_l2(kd.grad.cpu().transpose(-2, -3), ref["dk"]) <= REL_TOL
    assert ao.rel_l2(vd.grad.cpu().transpose(-2, -3), ref["dv"]) <= REL_TOL
    assert ao.rel_l2(bd.grad.cpu(), ref["dbias"]) <= REL_TOL


@pytest.mark.parametrize("D", [16, 32, 64])
def test_head_dim_sweep_with_ragged_n_and_masked_tail(D):
    """N = 257 (not tile aligned) with a fully masked key tail."""
    inp = attention_inputs(1, 5, 4, 257, D, seed=11 + D, mask_mode="none")
    inp["res_mask"][..., 200:] = float("-inf")
    got, d_out = _run(inp)
    _check(got, _oracle(inp, d_out), tol=6e-3)


def test_outer_dim_differs_from_sequence_and_odd_outer():
    inp = attention_inputs(2, 7, 3, 136, 32, seed=21, mask_mode="random30")
    got, d_out = _run(inp)
    _check(got, _oracle(inp, d_out), tol=6e-3)


def test_long_sequence_uses_key_strips():
    """N = 640 > 384: dQ accumulates over two key strips through the per-CTA scratch."""
    inp = attention_inputs(1, 3, 2, 640, 32, seed=31, mask_mode="trailing15")
    got, d_out = _run(inp)
    _check(got, _oracle(inp, d_out, dtype=torch.float32), tol=6e-3)


def test_training_shape_full_size_properties():
    """Config A384 (B=1, O=N=384, H=4, D=32) at full size: parity on a row subset against the
    oracle plus size-independent properties: probabilities sum to one (v = 1 gives out = 1),
    every row of dS sums to zero (so dbias rows sum to ~0), dv column sums equal the column
    sums of P^T dO."""
    inp = attention_inputs(1, 384, 4, 384, 32, seed=2, mask_mode="trailing15")
    got, d_out = _run(inp)
    sub = slice(0, 384, 48)  # 8 outer rows through the CPU oracle
    small = {k: (v[:, sub] if k != "pair_bias" else v) for k, v in inp.items()}
    ref = _oracle(small, d_out[:, sub], dtype=torch.float32)
    for n in ("out", "dq", "dk", "dv"):
        assert ao.rel_l2(got[n][:, sub], ref[n]) <= 6e-3, n
    assert (got["lse"][:, sub].double() - ref["lse"].double()).abs().max().item() <= LSE_TOL * 10
    # dBias depends on ALL 384 outer rows and on the chunk plan (o-chunks + fold at this shape): compare it
    # with the oracle's sum over every row, accumulated chunk by chunk in fp32
    dbias_ref = torch.zeros_like(inp["pair_bias"], dtype=torch.float32)
    for o0 in range(0, 384, 48):
        sl = slice(o0, o0 + 48)
        part = {k: (v[:, sl] if k != "pair_bias" else v) for k, v in inp.items()}
        dbias_ref += _oracle(part, d_out[:, sl], dtype=torch.float32)["dbias"]
    assert ao.rel_l2(got["dbias"], dbias_ref) <= 6e-3
    # dS rows sum to zero => dbias rows sum to zero up to rounding of the summands
    db = got["dbias"].float()
    assert db.sum(-1).abs().max().item() <= 2e-2 * db.abs().sum(-1).max().item()
    # v = 1  =>  out = 1
    ones = dict(inp)
    ones["v"] = torch.ones_like(inp["v"])
    out = tk.turbo_attention(*(ones[n].cuda().bfloat16() for n in ("q", "k", "v")),
                             pair_bias=ones["pair_bias"].cuda().bfloat16(), res_mask=ones["res_mask"].cuda())
    assert (out.float() - 1).abs().max().item() <= 1.0 / 64


def test_large_finite_mask_value_behaves_like_minus_inf():
    """The OpenFold3 layers pass inf = 1e9 (a large finite negative), the operator contract says -inf."""
    inp = attention_inputs(1, 4, 2, 128, 32, seed=5, mask_mode="none")
    inp["res_mask"][..., 100:] = float("-inf")
    got_inf, d_out = _run(inp)
    inp2 = dict(inp)
    inp2["res_mask"] = torch.where(torch.isinf(inp["res_mask"]), torch.full_like(inp["res_mask"], -1e9), inp["res_mask"])
    got_big, _ = _run(inp2, d_out)
    for n in ("out", "dq", "dk", "dv", "dbias"):
        assert ao.rel_l2(got_big[n], got_inf[n]) <= 1e-6, n


def test_no_python_fallback_native_library_is_loaded():
    with open("/proc/self/maps") as f:
        assert "libtpf_b200.so" in f.read()
    assert tk.attention.invocation_count() > 0
