"""Host-side operator logic that needs no GPU: support predicates, error behaviour,
fake (meta) kernels of the custom ops."""
import pytest
import torch

import openfold3_triangle_kernel_b200 as tk
from openfold3_triangle_kernel_b200 import attention as att
from openfold3_triangle_kernel_b200 import trimul as tm


def _qkv(B=1, O=4, H=2, N=16, D=32, dtype=torch.bfloat16):
    q = torch.zeros(B, O, H, N, D, dtype=dtype)
    bias = torch.zeros(B, 1, H, N, N, dtype=torch.bfloat16)
    mask = torch.zeros(B, O, 1, 1, N)
    return q, q.clone(), q.clone(), mask, bias


@pytest.mark.parametrize("D", [1, 7, 8, 16, 24, 31, 32, 48, 64])
def test_attention_accepts_head_dims_up_to_64(D):
    q, k, v, m, b = _qkv(D=D)
    ok, reason = att.is_turbo_attention_supported(q, k, v, m, b, check_device=False)
    assert ok, reason


@pytest.mark.parametrize("D", [65, 128])
def test_attention_rejects_large_head_dims(D):
    q, k, v, m, b = _qkv(D=D)
    ok, reason = att.is_turbo_attention_supported(q, k, v, m, b, check_device=False)
    assert not ok and "D<=64" in reason


def test_attention_dtype_and_shape_rules():
    q, k, v, m, b = _qkv()
    f = lambda *a: att.is_turbo_attention_supported(*a, check_device=False)  # noqa: E731
    assert f(q, k, v, m, b.float())[0]                       # fp32 bias accepted
    assert not f(q, k, v, m, b.half())[0]                    # fp16 bias rejected
    assert not f(q.float(), k, v, m, b)[0]                   # q must be bf16
    assert not f(q, k[:, :2], v, m, b)[0]                    # k shape
    assert not f(q, k, v, m.bool(), b)[0]                    # boolean mask rejected
    assert not f(q, k, v, m[..., :8], b)[0]                  # mask tail
    assert not f(q, k, v, m, b[..., :8])[0]                  # bias tail
    assert not f(q[0], k[0], v[0], m[0], b[0])[0]            # needs a batch prefix
    m2 = m.clone().requires_grad_(True)
    assert "gradients" in f(q, k, v, m2, b)[1]
    q5 = torch.zeros(2, 3, 4, 2, 16, 32, dtype=torch.bfloat16)
    b5 = torch.zeros(1, 3, 1, 2, 16, 16, dtype=torch.bfloat16)
    m5 = torch.zeros(2, 1, 4, 1, 1, 16)
    assert f(q5, q5, q5, m5, b5)[0]                          # broadcastable prefixes
    assert not f(q5, q5, q5, m5, torch.zeros(5, 3, 1, 2, 16, 16, dtype=torch.bfloat16))[0]


def test_attention_public_call_raises_value_error_before_launch():
    q, k, v, m, b = _qkv()
    with pytest.raises(ValueError, match="unsupported TurboPairFormer case"):
        tk.turbo_attention(q, k, v, pair_bias=b, res_mask=m)   # CPU tensors
    with pytest.raises(ValueError, match="pair_bias is required"):
        tk.turbo_attention(q, k, v)


def test_trimul_support_codes():
    z = torch.zeros(1, 16, 16, 64, dtype=torch.bfloat16)
    chk = lambda *a, **k: tm.check_trimul_support(*a, check_device=False, **k)  # noqa: E731
    assert chk(z, "outgoing", None, {}).supported
    assert chk(z.float(), "outgoing", None, {}).code == "z_dtype"
    assert chk(z, "sideways", None, {}).code == "direction"
    assert chk(z[..., :48], "outgoing", None, {}).code == "channels"
    assert chk(z[:, :, :8], "outgoing", None, {}).code == "z_square"
    assert chk(z, "incoming", torch.ones(1, 16, 16, dtype=torch.bool), {}).supported
    assert chk(z, "incoming", torch.ones(1, 16, 8), {}).code == "mask_shape"
    assert chk(z, "incoming", torch.ones(1, 16, 16, dtype=torch.int32), {}).code == "mask_dtype"
    assert chk(z, "outgoing", None, {"p_in_weight": torch.zeros(64, 64)}).code == "weight_shape"
    assert chk(z, "outgoing", None, {"p_in_weight": torch.zeros(128, 64)}).supported
    for c in (32, 64, 96, 128):
        assert chk(torch.zeros(2, 3, 8, 8, c, dtype=torch.bfloat16), "outgoing", None, {}).supported


def test_trimul_public_call_errors():
    z = torch.zeros(1, 16, 16, 64, dtype=torch.bfloat16)
    with pytest.raises(ValueError, match=r"unsupported \[device\]"):
        tk.turbo_trimul(z)
    with pytest.raises(TypeError, match="unexpected keyword"):
        tk.turbo_trimul(z, linear_q=torch.zeros(1))


def test_fake_kernels_give_reference_shapes():
    from torch._subclasses.fake_tensor import FakeTensorMode
    with FakeTensorMode():
        q = torch.empty(2, 5, 4, 40, 32, dtype=torch.bfloat16)
        mask = torch.empty(2, 5, 40)
        bias = torch.empty(1, 4, 40, 40, dtype=torch.bfloat16)
        out, lse = torch.ops.tpf_b200.attn_fwd(q, q, q, mask, bias, 0.17)
        assert out.shape == (2, 5, 40, 4, 32) and out.dtype == torch.bfloat16
        assert lse.shape == (2, 5, 4, 40) and lse.dtype == torch.float32
        dq, dk, dv, db = torch.ops.tpf_b200.attn_bwd(q, q, q, out, out, lse, mask, bias, 0.17)
        assert dq.shape == q.shape and db.shape == (1, 4, 40, 40) and db.dtype == torch.float32
        z = torch.empty(2, 16, 16, 96, dtype=torch.bfloat16)
        w = lambda r: torch.empty(r, 96)  # noqa: E731
        v = torch.empty(96)
        outs = torch.ops.tpf_b200.trimul_fwd(z, torch.empty(2, 16, 16), w(192), w(192), w(96), w(96), v, v, v, v, True)
        assert len(outs) == 11 and outs[0].shape == z.shape
        assert outs[4].shape == (2 * 96, 256) and outs[2].shape == (512,)
        gr = torch.ops.tpf_b200.trimul_bwd(outs[0], z, torch.empty(2, 16, 16), w(192), w(192), w(96), w(96), v, v,
                                           True, *outs)
        assert len(gr) == 9 and gr[0].shape == z.shape and gr[1].shape == (192, 96) and gr[5].shape == (96,)


def test_module_weight_mapping():
    class Lin(torch.nn.Module):
        def __init__(self, c):
            super().__init__()
            self.weight = torch.nn.Parameter(torch.randn(c, c))
            self.bias = None

    class Mod(torch.nn.Module):
        def __init__(self, c=32):
            super().__init__()
            for n in ("a_p", "a_g", "b_p", "b_g", "g", "z"):
                setattr(self, "linear_" + n, Lin(c))
            self.layer_norm_in = torch.nn.LayerNorm(c)
            self.layer_norm_out = torch.nn.LayerNorm(c)
            self._outgoing = False

    m = Mod()
    w, direction = tm._weights_from_module(m)
    assert direction == "incoming"
    assert torch.equal(w["p_in_weight"], torch.cat([m.linear_a_p.weight, m.linear_b_p.weight]))
    assert torch.equal(w["g_in_weight"], torch.cat([m.linear_a_g.weight, m.linear_b_g.weight]))
    assert w["p_out_weight"] is m.linear_z.weight and w["g_out_weight"] is m.linear_g.weight
    m.linear_g.bias = torch.nn.Parameter(torch.zeros(32))
    with pytest.raises(ValueError, match="linear_bias"):
        tm._weights_from_module(m)


def test_synthetic_inputs_match_the_parity_generators():
    """The package's benchmark input generators draw the same tensors as the generators the parity
    tests feed to the oracle (same seed -> same workload on both arms of the benchmark)."""
    import torch
    from openfold3_triangle_kernel_b200 import synthetic
    from oracle import inputs as oi
    from oracle.pair_block_oracle import block_params

    a, b = synthetic.attention_inputs(1, 6, 2, 40, 16, seed=2), oi.attention_inputs(1, 6, 2, 40, 16, seed=2)
    assert a.keys() == b.keys() and all(torch.equal(a[k], b[k]) for k in a)
    a, b = synthetic.trimul_inputs(1, 24, 32, seed=3), oi.trimul_inputs(1, 24, 32, seed=3)
    assert torch.equal(a["z"], b["z"]) and torch.equal(a["mask"], b["mask"])
    assert all(torch.equal(a["weights"][k], b["weights"][k]) for k in b["weights"])
    a, b = synthetic.block_params(32, 2, 16, 5), block_params(32, 2, 16, 5)
    assert all(torch.equal(a[m][k], b[m][k]) for m in b for k in b[m])


def test_bench_reference_arm_line_has_the_contract_keys(monkeypatch, capsys):
    """`bench.py --impl reference` prints one JSON line with the keys the benchmark contract names;
    the CPU sample itself is stubbed here (it takes seconds of real work)."""
    import importlib
    import json
    import os
    import types

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    monkeypatch.syspath_prepend(root)
    bench = importlib.import_module("bench")
    monkeypatch.setattr(bench, "cpu_step_seconds", lambda: (2.0, 4, "stub sample"))
    bench.run_reference(types.SimpleNamespace(gpus=1, steps=3, warmup=1), rank=0)
    line = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    for key in ("impl", "metric", "value", "unit", "n_gpus", "steps", "warmup", "ms_per_step", "higher_is_better",
                "scaling", "vs_baseline", "dtype", "data", "config", "cpu_baseline", "e2e"):
        assert key in line, key
    assert line["impl"] == "reference" and line["steps_timed"] == 3 and line["ms_per_step"] == 2000.0
    assert line["e2e"]["h2d_bytes_per_step"] == 0 and line["cpu_baseline"]["kind"] == "port"
    assert line["config"]["workload"] == bench.WORKLOAD
    # ranks other than 0 print nothing
    bench.run_reference(types.SimpleNamespace(gpus=2, steps=1, warmup=0), rank=1)
    assert capsys.readouterr().out == ""
