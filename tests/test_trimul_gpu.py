"""turbo_trimul on a B200 against the CPU oracle and the reference-generated golden fixtures.
The reference itself never pins full-operator TriMul accuracy
(tools/aot_current_numeric_smoke.py:323-329); these tests are that pin."""
import os

import numpy as np
import pytest
import torch

import openfold3_triangle_kernel_b200 as tk
from openfold3_triangle_kernel_b200 import _cabi as C
from oracle import trimul_oracle as to
from oracle.attention_oracle import rel_l2
from oracle.inputs import trimul_inputs, trimul_inputs_cpu_case

pytestmark = [pytest.mark.gpu, pytest.mark.skipif(not torch.cuda.is_available(), reason="needs a CUDA device")]

# bf16 pipeline vs fp32/fp64 reference, relative L2: the output within 1e-2; gradients pass through
# five more bf16 intermediates (d_y, d_xln, d_x, d_a/d_b, d_proj) and are held to 2e-2, the bound
# the reference's own kernel-vs-stock harness uses for backward (openfold3/tests/test_kernels.py:172-174).
REL_TOL = 1e-2
GRAD_TOL = 2e-2


def _run(inp, direction, d_out=None, perturb_norms=False):
    dev = "cuda"
    z = inp["z"].to(dev).bfloat16().requires_grad_(True)
    w = {k: v.to(dev).clone().requires_grad_(True) for k, v in inp["weights"].items()}
    out = tk.turbo_trimul(z, direction, inp["mask"].to(dev) if inp["mask"] is not None else None, **w)
    if d_out is None:
        d_out = (2.0 * out.detach().float() / out.numel()).bfloat16()
    out.backward(d_out.to(dev))
    torch.cuda.synchronize()
    assert C.device_status() == 0
    res = dict(out=out.detach().cpu(), dz=z.grad.cpu())
    for k in to.WEIGHT_NAMES:
        res["d_" + k] = w[k].grad.cpu()
    return res, d_out.cpu()


def _check(got, ref, tol=REL_TOL, grad_tol=GRAD_TOL):
    for k, v in ref.items():
        assert torch.isfinite(got[k].float()).all(), k
        e = rel_l2(got[k], v)
        assert e <= (tol if k == "out" else grad_tol), (k, e)


@pytest.mark.parametrize("direction", ["outgoing", "incoming"])
def test_cpu_reference_config_against_golden_fixture(golden_dir, direction):
    """Config 'CPU reference': z [1,64,64,32], gamma = 1, beta = 0, Xavier-normal projections;
    fixture = fp32 output / gradients of the reference's stock module for loss = mean(out^2)."""
    gold = np.load(os.path.join(golden_dir, f"trimul_{direction}_cpu_case.npz"))
    inp = trimul_inputs_cpu_case(seed=1)
    got, d_out = _run(inp, direction)
    assert rel_l2(got["out"], torch.from_numpy(gold["out"])) <= REL_TOL
    assert rel_l2(got["dz"], torch.from_numpy(gold["dz"])) <= 2.5 * REL_TOL
    for n in ("p_in_weight", "g_in_weight", "p_out_weight", "g_out_weight"):
        assert rel_l2(got["d_" + n], torch.from_numpy(gold["d_" + n])) <= 2.5 * REL_TOL, n
    # tight check against the oracle fed with the bf16 z and the bf16 d_out the kernel saw
    inp_b = dict(inp, z=inp["z"].bfloat16())
    ref = to.trimul_forward_backward(inp_b["z"], direction, torch.ones(1, 64, 64), inp["weights"], d_out)
    _check(got, ref)


@pytest.mark.parametrize("C_", [32, 64, 96, 128])
@pytest.mark.parametrize("direction", ["outgoing", "incoming"])
def test_channel_sweep(C_, direction):
    inp = trimul_inputs(1, 104, C_, seed=40 + C_, mask_mode="trailing10")
    g = torch.Generator().manual_seed(C_)
    for k in ("norm_in_weight", "norm_out_weight"):
        inp["weights"][k] = 1 + 0.1 * torch.randn(C_, generator=g)
    for k in ("norm_in_bias", "norm_out_bias"):
        inp["weights"][k] = 0.1 * torch.randn(C_, generator=g)
    d_out = torch.randn(1, 104, 104, C_, generator=g).bfloat16()
    got, _ = _run(inp, direction, d_out)
    ref = to.trimul_forward_backward(inp["z"], direction, inp["mask"], inp["weights"], d_out)
    _check(got, ref)


def test_ragged_n_is_padded_and_cropped():
    inp = trimul_inputs(2, 61, 64, seed=7, mask_mode="trailing10")
    d_out = torch.randn(2, 61, 61, 64, generator=torch.Generator().manual_seed(1)).bfloat16()
    got, _ = _run(inp, "outgoing", d_out)
    ref = to.trimul_forward_backward(inp["z"], "outgoing", inp["mask"], inp["weights"], d_out)
    _check(got, ref)


def test_n257_incoming():
    inp = trimul_inputs(1, 257, 128, seed=9, mask_mode="trailing10")
    d_out = torch.randn(1, 257, 257, 128, generator=torch.Generator().manual_seed(2)).bfloat16()
    got, _ = _run(inp, "incoming", d_out)
    ref = to.trimul_forward_backward(inp["z"], "incoming", inp["mask"], inp["weights"], d_out, dtype=torch.float32)
    _check(got, ref)


@pytest.mark.parametrize("direction", ["outgoing", "incoming"])
def test_training_shape_full_size(direction):
    """Config T384: z [1,384,384,128], trailing 10 % of residues masked, loss = mean(out^2)."""
    inp = trimul_inputs(1, 384, 128, seed=3, mask_mode="trailing10")
    got, d_out = _run(inp, direction)
    ref = to.trimul_forward_backward(inp["z"], direction, inp["mask"], inp["weights"], d_out, dtype=torch.float32)
    _check(got, ref)
    # masked positions produce exactly-zero a / b, hence d_z rows of masked residues are zero
    # only through the gate path; the output itself must be finite everywhere
    assert torch.isfinite(got["out"].float()).all()


def test_bitwise_replay_and_module_calling_form():
    inp = trimul_inputs(1, 72, 64, seed=13, mask_mode="trailing10")
    d_out = torch.randn(1, 72, 72, 64, generator=torch.Generator().manual_seed(3)).bfloat16()
    a, _ = _run(inp, "incoming", d_out)
    b, _ = _run(inp, "incoming", d_out)
    for k in a:
        assert torch.equal(a[k], b[k]), k

    class Lin(torch.nn.Module):
        def __init__(self, w):
            super().__init__()
            self.weight = torch.nn.Parameter(w.clone())
            self.bias = None

    class Mod(torch.nn.Module):
        def __init__(self, w, c):
            super().__init__()
            self.linear_a_p, self.linear_b_p = Lin(w["p_in_weight"][:c]), Lin(w["p_in_weight"][c:])
            self.linear_a_g, self.linear_b_g = Lin(w["g_in_weight"][:c]), Lin(w["g_in_weight"][c:])
            self.linear_z, self.linear_g = Lin(w["p_out_weight"]), Lin(w["g_out_weight"])
            self.layer_norm_in = torch.nn.LayerNorm(c)
            self.layer_norm_out = torch.nn.LayerNorm(c)
            self._outgoing = False

    mod = Mod(inp["weights"], 64).cuda()
    z = inp["z"].cuda().bfloat16()
    out = tk.turbo_trimul(mod, z, inp["mask"].cuda())
    assert torch.equal(out.cpu(), a["out"])
    out.float().square().mean().backward()
    assert mod.linear_a_p.weight.grad is not None and mod.layer_norm_out.bias.grad is not None


def test_sampled_weights_form_runs():
    z = torch.randn(1, 64, 64, 32, device="cuda").bfloat16().requires_grad_(True)
    out = tk.turbo_trimul(z, direction="outgoing")
    out.float().square().mean().backward()
    assert out.shape == z.shape and torch.isfinite(z.grad.float()).all()
