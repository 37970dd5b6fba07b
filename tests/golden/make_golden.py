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


def _load_trimul(mod, w, c):
    with torch.no_grad():
        mod.layer_norm_in.weight.copy_(w["norm_in_weight"]); mod.layer_norm_in.bias.copy_(w["norm_in_bias"])
        mod.layer_norm_out.weight.copy_(w["norm_out_weight"]); mod.layer_norm_out.bias.copy_(w["norm_out_bias"])
        mod.linear_a_p.weight.copy_(w["p_in_weight"][:c]); mod.linear_b_p.weight.copy_(w["p_in_weight"][c:])
        mod.linear_a_g.weight.copy_(w["g_in_weight"][:c]); mod.linear_b_g.weight.copy_(w["g_in_weight"][c:])
        mod.linear_z.weight.copy_(w["p_out_weight"]); mod.linear_g.weight.copy_(w["g_out_weight"])


def _load_attention(mod, p):
    with torch.no_grad():
        mod.layer_norm.weight.copy_(p["ln_w"]); mod.layer_norm.bias.copy_(p["ln_b"])
        mod.linear_z.weight.copy_(p["w_z"])
        mod.mha.linear_q.weight.copy_(p["w_q"]); mod.mha.linear_k.weight.copy_(p["w_k"])
        mod.mha.linear_v.weight.copy_(p["w_v"]); mod.mha.linear_g.weight.copy_(p["w_g"])
        mod.mha.linear_o.weight.copy_(p["w_o"])


def golden_pair_block(ref, path):
    """TriMul out -> in -> attention start -> end with residuals, composed from the reference's own
    modules exactly as PairBlock.tri_mul_out_in / tri_att_start_end do (base_blocks.py:311-431)."""
    from oracle.pair_block_oracle import block_params
    c, heads, d, n = 32, 4, 8, 24
    params = block_params(c, heads, d, seed=7)
    g = torch.Generator().manual_seed(11)
    z = torch.randn(1, n, n, c, generator=g)
    mask = torch.ones(1, n, n)
    mask[:, n - 4:, :] = 0
    mask[:, :, n - 4:] = 0
    tmo, tmi = ref["TriangleMultiplicationOutgoing"](c, c), ref["TriangleMultiplicationIncoming"](c, c)
    tas, tae = ref["TriangleAttention"](c, d, heads), ref["TriangleAttention"](c, d, heads)
    _load_trimul(tmo, params["tri_mul_out"], c); _load_trimul(tmi, params["tri_mul_in"], c)
    _load_attention(tas, params["tri_att_start"]); _load_attention(tae, params["tri_att_end"])
    with torch.no_grad():
        x = z + tmo(z, mask=mask)
        x = x + tmi(x, mask=mask)
        x = x + tas(x, mask=mask)
        x = x.transpose(-2, -3)
        x = x + tae(x, mask=mask.transpose(-1, -2), transpose_bias=True)
        x = x.transpose(-2, -3)
    np.savez_compressed(path, z=z.numpy(), mask=mask.numpy(), out=x.numpy())


def _reference_test_rng():
    """The RNG isolation + seeding of the reference's ``seeded_rng`` fixture
    (openfold3/tests/conftest.py:299-314)."""
    import contextlib
    import random

    @contextlib.contextmanager
    def ctx():
        py_state, np_state = random.getstate(), np.random.get_state()
        with torch.random.fork_rng():
            torch.manual_seed(123)
            random.seed(123)
            np.random.seed(123)
            yield
        random.setstate(py_state)
        np.random.set_state(np_state)

    return ctx()


def golden_reference_snapshots(ref, ref_root, folder):
    """Pin against the golden vectors the reference's OWN tests hold for the two stock modules:
    the ``ndarrays_regression`` snapshots of openfold3/tests/test_triangular_attention.py:27-72 and
    openfold3/tests/test_triangular_multiplicative_update.py:45-86 (c_z 128, hidden 12 / 11, 4 heads,
    batch 2, 22 residues, seed 123).  The tests' module construction and input draws are replayed
    here, the stock module's output is checked against the committed snapshot (the reference's
    tolerance: atol = rtol = 1e-4), and parameters + input + SNAPSHOT output of batch entry 0 are
    stored so that the oracle can be checked against the snapshot without the reference tree."""
    snap = os.path.join(ref_root, "openfold3", "tests", "test_data", "snapshots")
    c_z, heads, n, batch = 128, 4, 22, 2
    for starting in (True, False):
        with _reference_test_rng():
            tan = ref["TriangleAttention"](c_z, 12, heads, starting=starting)
            for prm in tan.parameters():
                torch.nn.init.normal_(prm, std=0.01)
            tan.eval()
            x = torch.rand((batch, n, n, c_z))
            with torch.no_grad():
                out = tan(x, chunk_size=None)
        gold = np.load(os.path.join(snap, "test_triangular_attention", "nvidia", f"test_shape_cpu_{starting}_.npz"))["output"]
        assert np.allclose(out.numpy(), gold, atol=1e-4, rtol=1e-4), "stock TriangleAttention does not reproduce its snapshot"
        sd = tan.state_dict()
        np.savez_compressed(
            os.path.join(folder, f"reference_snapshot_triangle_attention_{'starting' if starting else 'ending'}.npz"),
            x=x[0].numpy(), output=gold[0], ln_w=sd["layer_norm.weight"].numpy(), ln_b=sd["layer_norm.bias"].numpy(),
            w_z=sd["linear_z.weight"].numpy(), w_q=sd["mha.linear_q.weight"].numpy(), w_k=sd["mha.linear_k.weight"].numpy(),
            w_v=sd["mha.linear_v.weight"].numpy(), w_g=sd["mha.linear_g.weight"].numpy(), w_o=sd["mha.linear_o.weight"].numpy())
    with _reference_test_rng():
        tm = ref["TriangleMultiplicationOutgoing"](c_z, 11)
        for prm in tm.parameters():
            torch.nn.init.normal_(prm, std=0.01)
        tm.eval()
        x = torch.rand((batch, n, n, c_z))
        mask = torch.randint(0, 2, size=(batch, n, n))
        with torch.no_grad():
            out = tm(x, mask)
    gold = np.load(os.path.join(snap, "test_triangular_multiplicative_update", "nvidia", "test_shape_cpu_.npz"))["output"]
    assert np.allclose(out.numpy(), gold, atol=1e-4, rtol=1e-4), "stock TriangleMultiplicationOutgoing does not reproduce its snapshot"
    sd = tm.state_dict()
    np.savez_compressed(
        os.path.join(folder, "reference_snapshot_trimul_outgoing.npz"), x=x[0].numpy(), mask=mask[0].numpy(), output=gold[0],
        norm_in_weight=sd["layer_norm_in.weight"].numpy(), norm_in_bias=sd["layer_norm_in.bias"].numpy(),
        norm_out_weight=sd["layer_norm_out.weight"].numpy(), norm_out_bias=sd["layer_norm_out.bias"].numpy(),
        p_in_weight=torch.cat([sd["linear_a_p.weight"], sd["linear_b_p.weight"]]).numpy(),
        g_in_weight=torch.cat([sd["linear_a_g.weight"], sd["linear_b_g.weight"]]).numpy(),
        p_out_weight=sd["linear_z.weight"].numpy(), g_out_weight=sd["linear_g.weight"].numpy())


if __name__ == "__main__":
    if len(sys.argv) != 2:
        raise SystemExit("usage: python tests/golden/make_golden.py <path to a checkout of the reference repository>")
    ref = import_reference(sys.argv[1])
    torch.set_num_threads(max(1, os.cpu_count() or 1))
    golden_attention(ref, os.path.join(HERE, "attention_cpu_case.npz"))
    for d in ("outgoing", "incoming"):
        golden_trimul(ref, os.path.join(HERE, f"trimul_{d}_cpu_case.npz"), d)
    golden_pair_block(ref, os.path.join(HERE, "pair_block_small.npz"))
    golden_reference_snapshots(ref, sys.argv[1], HERE)
    print("golden fixtures written to", HERE)
