"""Generate the golden fixtures in this folder from the reference's own stock
PyTorch modules.  Run where the reference tree is available:

    python tests/golden/make_golden.py /path/to/reference

It imports ``_attention`` (openfold3/core/model/primitives/attention.py:176-217)
and ``TriangleMultiplicationOutgoing/Incoming``
(openfold3/core/model/layers/triangular_multiplicative_update.py:1262-1284),
runs them in fp32 on seeded inputs (generators below are the same ones the
tests use to rebuild the inputs) and stores outputs and gradients.
"""
import math
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

from _ref_import import import_reference  # noqa: E402
from oracle.inputs import attention_inputs_cpu_case, trimul_inputs_cpu_case  # noqa: E402


def golden_attention(ref, path):
    inp = attention_inputs_cpu_case(seed=0)
    q, k, v, bias, mask = (inp[n] for n in ("q", "k", "v", "pair_bias", "res_mask"))
    q_, k_, v_, b_ = (t.clone().requires_grad_(True) for t in (q, k, v, bias))
    scale = 1.0 / math.sqrt(q.shape[-1])
    # caller-side scaling and final transpose as in attention.py:365-366, :692
    o = ref["_attention"](q_ * scale, k_, v_, [mask, b_]).transpose(-2, -3)
    loss = o.square().mean()
    loss.backward()
    sub = slice(None, None, 4)
    np.savez_compressed(
        path, out=o.detach()[:, sub].numpy(), dq=q_.grad[:, sub].numpy(), dk=k_.grad[:, sub].numpy(),
        dv=v_.grad[:, sub].numpy(), dbias=b_.grad.numpy(), loss=np.float64(loss.item()),
        out_sum=np.float64(o.detach().double().sum().item()))


def golden_trimul(ref, path, direction):
    inp = trimul_inputs_cpu_case(seed=1)
    c = inp["z"].shape[-1]
    cls = ref["TriangleMultiplicationOutgoing" if direction == "outgoing" else "TriangleMultiplicationIncoming"]
    mod = cls(c, c)
    w = inp["weights"]
    with torch.no_grad():
        mod.layer_norm_in.weight.copy_(w["norm_in_weight"]); mod.layer_norm_in.bias.copy_(w["norm_in_bias"])
        mod.layer_norm_out.weight.copy_(w["norm_out_weight"]); mod.layer_norm_out.bias.copy_(w["norm_out_bias"])
        mod.linear_a_p.weight.copy_(w["p_in_weight"][:c]); mod.linear_b_p.weight.copy_(w["p_in_weight"][c:])
        mod.linear_a_g.weight.copy_(w["g_in_weight"][:c]); mod.linear_b_g.weight.copy_(w["g_in_weight"][c:])
        mod.linear_z.weight.copy_(w["p_out_weight"]); mod.linear_g.weight.copy_(w["g_out_weight"])
    z = inp["z"].clone().requires_grad_(True)
    out = mod(z, mask=inp["mask"])
    loss = out.square().mean()
    loss.backward()
    np.savez_compressed(
        path, out=out.detach().numpy(), dz=z.grad.numpy(),
        d_p_in_weight=torch.cat([mod.linear_a_p.weight.grad, mod.linear_b_p.weight.grad]).numpy(),
        d_g_in_weight=torch.cat([mod.linear_a_g.weight.grad, mod.linear_b_g.weight.grad]).numpy(),
        d_p_out_weight=mod.linear_z.weight.grad.numpy(), d_g_out_weight=mod.linear_g.weight.grad.numpy(),
        d_norm_in_weight=mod.layer_norm_in.weight.grad.numpy(), d_norm_in_bias=mod.layer_norm_in.bias.grad.numpy(),
        d_norm_out_weight=mod.layer_norm_out.weight.grad.numpy(), d_norm_out_bias=mod.layer_norm_out.bias.grad.numpy(),
        loss=np.float64(loss.item()))


if __name__ == "__main__":
    ref = import_reference(sys.argv[1] if len(sys.argv) > 1 else "/root/reference")
    torch.set_num_threads(max(1, os.cpu_count() or 1))
    golden_attention(ref, os.path.join(HERE, "attention_cpu_case.npz"))
    for d in ("outgoing", "incoming"):
        golden_trimul(ref, os.path.join(HERE, f"trimul_{d}_cpu_case.npz"), d)
    print("golden fixtures written to", HERE)
