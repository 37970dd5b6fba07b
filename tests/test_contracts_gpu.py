"""Contracts of the operators beyond numerics, on a B200:

* every entry point follows the caller's stream - a non-default stream, and two streams at once
  (reference: openfold3/tests/core/kernels/test_turbopairformer_trimul_cpp_contract.py:191-218);
* launch state is per device and safe under concurrent host threads;
* the custom ops satisfy the compiler contract the reference gates its ops with: torch.library.opcheck,
  torch.compile(fullgraph=True) equal to eager, torch.export save / load round trip
  (reference: openfold3/tests/test_turbopairformer_trimul_custom_op.py:641-900);
* the bounded wait of the kernels really gives up: a self-test kernel waits on a barrier nothing
  arrives on, returns, and tpf_device_status() reports the timeout once.
"""
import ctypes
import threading

import pytest
import torch

import openfold3_triangle_kernel_b200 as tk
from openfold3_triangle_kernel_b200 import _cabi as C
from oracle.inputs import attention_inputs, trimul_inputs

pytestmark = [pytest.mark.gpu, pytest.mark.skipif(not torch.cuda.is_available(), reason="needs a CUDA device")]


def _attention_case(dev, seed=3, O=6, N=136, D=32):
    a = attention_inputs(1, O, 4, N, D, seed=seed, mask_mode="random30")
    g = torch.Generator().manual_seed(seed)
    d_out = torch.randn(1, O, N, 4, D, generator=g).bfloat16()
    return {k: v.to(dev) for k, v in a.items()}, d_out.to(dev)


def _trimul_case(dev, seed=4, N=72, Cc=64):
    t = trimul_inputs(1, N, Cc, seed=seed, mask_mode="trailing10")
    g = torch.Generator().manual_seed(seed)
    d_out = torch.randn(1, N, N, Cc, generator=g).bfloat16()
    return dict(z=t["z"].to(dev), mask=t["mask"].to(dev), w={k: v.to(dev) for k, v in t["weights"].items()}), d_out.to(dev)


def _run_attention(a, d_out):
    q, k, v, b = (a[n].detach().clone().requires_grad_(True) for n in ("q", "k", "v", "pair_bias"))
    out = tk.turbo_attention(q, k, v, pair_bias=b, res_mask=a["res_mask"])
    out.backward(d_out)
    return [out.detach(), q.grad, k.grad, v.grad, b.grad]


def _run_trimul(t, d_out, direction):
    z = t["z"].detach().clone().requires_grad_(True)
    w = {k: v.detach().clone().requires_grad_(True) for k, v in t["w"].items()}
    out = tk.turbo_trimul(z, direction, t["mask"], **w)
    out.backward(d_out)
    return [out.detach(), z.grad] + [w[k].grad for k in sorted(w)]


def _same(xs, ys):
    return all(torch.equal(x, y) for x, y in zip(xs, ys))


# --------------------------------------------------------------------------------------------
# streams
# --------------------------------------------------------------------------------------------
def test_every_entry_point_follows_a_non_default_stream():
    dev = torch.device("cuda", 0)
    a, d_a = _attention_case(dev)
    t, d_t = _trimul_case(dev)
    ref = _run_attention(a, d_a) + _run_trimul(t, d_t, "outgoing") + _run_trimul(t, d_t, "incoming")
    torch.cuda.synchronize()
    side = torch.cuda.Stream(device=dev)
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        got = _run_attention(a, d_a) + _run_trimul(t, d_t, "outgoing") + _run_trimul(t, d_t, "incoming")
        done = torch.cuda.Event()
        done.record()
    # nothing was enqueued on the default stream: the side stream alone carries the work
    done.synchronize()
    assert _same(got, ref)
    assert C.device_status() == 0


def test_two_streams_at_once_give_the_serial_results():
    dev = torch.device("cuda", 0)
    a, d_a = _attention_case(dev, seed=7, O=24, N=200)
    t, d_t = _trimul_case(dev, seed=8, N=136, Cc=128)
    ref_a = _run_attention(a, d_a)
    ref_t = _run_trimul(t, d_t, "incoming")
    torch.cuda.synchronize()
    s1, s2 = torch.cuda.Stream(device=dev), torch.cuda.Stream(device=dev)
    got_a, got_t = [], []
    for _ in range(4):  # interleaved submission: both streams have work in flight together
        with torch.cuda.stream(s1):
            got_a.append(_run_attention(a, d_a))
        with torch.cuda.stream(s2):
            got_t.append(_run_trimul(t, d_t, "incoming"))
    s1.synchronize()
    s2.synchronize()
    assert all(_same(g, ref_a) for g in got_a)
    assert all(_same(g, ref_t) for g in got_t)
    assert C.device_status() == 0


def test_two_host_threads_call_concurrently():
    dev = torch.device("cuda", 0)
    a, d_a = _attention_case(dev, seed=9)
    t, d_t = _trimul_case(dev, seed=10)
    ref_a, ref_t = _run_attention(a, d_a), _run_trimul(t, d_t, "outgoing")
    torch.cuda.synchronize()
    results, errors = {}, []

    def work(name, fn):
        try:
            torch.cuda.set_device(dev)
            with torch.cuda.stream(torch.cuda.Stream(device=dev)):
                outs = [fn() for _ in range(6)]
                torch.cuda.current_stream().synchronize()
            results[name] = outs
        except Exception as e:  # noqa: BLE001
            errors.append((name, repr(e)))

    th = [threading.Thread(target=work, args=("a", lambda: _run_attention(a, d_a))),
          threading.Thread(target=work, args=("t", lambda: _run_trimul(t, d_t, "outgoing")))]
    for x in th:
        x.start()
    for x in th:
        x.join()
    assert not errors, errors
    assert all(_same(g, ref_a) for g in results["a"])
    assert all(_same(g, ref_t) for g in results["t"])


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_second_device_after_the_first():
    """Launch attributes and symbol addresses are per device: a process that has used cuda:0 must be able
    to use cuda:1 (large dynamic shared memory would be refused there if the attribute were cached per
    process)."""
    outs = []
    for i in (0, 1):
        dev = torch.device("cuda", i)
        a, d_a = _attention_case(dev)
        t, d_t = _trimul_case(dev)
        with torch.cuda.device(dev):
            outs.append([x.cpu() for x in _run_attention(a, d_a) + _run_trimul(t, d_t, "outgoing")])
            torch.cuda.synchronize(dev)
            assert C.device_status() == 0
    assert _same(outs[0], outs[1])


# --------------------------------------------------------------------------------------------
# compiler contract
# --------------------------------------------------------------------------------------------
def _op_inputs(dev):
    a, d_a = _attention_case(dev, O=3, N=72)
    t, d_t = _trimul_case(dev, N=40, Cc=32)
    B, O, H, N, D = a["q"].shape
    att = (a["q"], a["k"], a["v"], a["res_mask"].reshape(B, O, N).contiguous(), a["pair_bias"].reshape(1, H, N, N),
           1.0 / D ** 0.5)
    w = t["w"]
    tri = (t["z"], t["mask"], w["p_in_weight"], w["g_in_weight"], w["p_out_weight"], w["g_out_weight"],
           w["norm_in_weight"], w["norm_in_bias"], w["norm_out_weight"], w["norm_out_bias"], False)
    return att, d_a, tri, d_t


def test_custom_ops_pass_opcheck():
    dev = torch.device("cuda", 0)
    att, d_a, tri, d_t = _op_inputs(dev)
    ops = torch.ops.tpf_b200
    att_g = tuple(x.detach().clone().requires_grad_(True) if i in (0, 1, 2, 4) else x for i, x in enumerate(att))
    res = torch.library.opcheck(ops.attn_fwd.default, att_g, raise_exception=True)
    assert all(v == "SUCCESS" for v in res.values()), res
    tri_g = tuple(x.detach().clone().requires_grad_(True) if isinstance(x, torch.Tensor) and i != 1 else x
                  for i, x in enumerate(tri))
    res = torch.library.opcheck(ops.trimul_fwd.default, tri_g, raise_exception=True)
    assert all(v == "SUCCESS" for v in res.values()), res
    # the backward ops are first-order implementation details: schema, fake kernel and dispatch are checked
    # on detached inputs
    with torch.no_grad():
        out, lse = ops.attn_fwd(*att)
        saved = ops.trimul_fwd(*tri)
    bwd_tests = ("test_schema", "test_faketensor", "test_aot_dispatch_dynamic")
    res = torch.library.opcheck(ops.attn_bwd.default, (att[0], att[1], att[2], d_a, out, lse, att[3], att[4], att[5]),
                                test_utils=bwd_tests, raise_exception=True)
    assert all(v == "SUCCESS" for v in res.values()), res
    res = torch.library.opcheck(
        ops.trimul_bwd.default,
        (d_t, tri[0], tri[1], tri[2], tri[3], tri[4], tri[5], tri[6], tri[8], tri[10], *saved),
        test_utils=bwd_tests, raise_exception=True)
    assert all(v == "SUCCESS" for v in res.values()), res


class _TrimulModule(torch.nn.Module):
    def __init__(self, w, direction):
        super().__init__()
        self.direction = direction
        for k, v in w.items():
            setattr(self, k, torch.nn.Parameter(v.detach().clone()))
        self.names = sorted(w)

    def forward(self, z, mask):
        return tk.turbo_trimul(z, self.direction, mask, **{k: getattr(self, k) for k in self.names})


class _AttentionModule(torch.nn.Module):
    def forward(self, q, k, v, bias, mask):
        return tk.turbo_attention(q, k, v, pair_bias=bias, res_mask=mask)


@pytest.mark.parametrize("direction", ["outgoing", "incoming"])
def test_trimul_fullgraph_compile_equals_eager(direction):
    torch.compiler.reset()
    dev = torch.device("cuda", 0)
    t, d_t = _trimul_case(dev, N=40, Cc=32)
    eager = _TrimulModule(t["w"], direction).to(dev)
    compiled = torch.compile(_TrimulModule(t["w"], direction).to(dev), backend="aot_eager", fullgraph=True)
    outs = []
    for m in (eager, compiled):
        z = t["z"].detach().clone().requires_grad_(True)
        o = m(z, t["mask"])
        o.backward(d_t)
        mod = m._orig_mod if hasattr(m, "_orig_mod") else m
        outs.append([o.detach(), z.grad] + [getattr(mod, k).grad for k in mod.names])
    assert _same(outs[0], outs[1])


def test_attention_fullgraph_compile_equals_eager():
    torch.compiler.reset()
    dev = torch.device("cuda", 0)
    a, d_a = _attention_case(dev, O=3, N=72)
    compiled = torch.compile(_AttentionModule(), backend="aot_eager", fullgraph=True)
    outs = []
    for m in (_AttentionModule(), compiled):
        q, k, v, b = (a[n].detach().clone().requires_grad_(True) for n in ("q", "k", "v", "pair_bias"))
        o = m(q, k, v, b, a["res_mask"])
        o.backward(d_a)
        outs.append([o.detach(), q.grad, k.grad, v.grad, b.grad])
    assert _same(outs[0], outs[1])


def test_export_save_load_round_trip(tmp_path):
    dev = torch.device("cuda", 0)
    t, _ = _trimul_case(dev, N=40, Cc=32)
    mod = _TrimulModule(t["w"], "outgoing").to(dev).eval()
    exported = torch.export.export(mod, (t["z"], t["mask"]))
    targets = [str(n.target) for n in exported.graph.nodes if n.op == "call_function" and "tpf_b200" in str(n.target)]
    assert targets == ["tpf_b200.trimul_fwd.default"], targets
    path = tmp_path / "trimul.pt2"
    torch.export.save(exported, path)
    loaded = torch.export.load(path).module()
    assert torch.equal(loaded(t["z"], t["mask"]), mod(t["z"], t["mask"]))

    a, _ = _attention_case(dev, O=3, N=72)
    amod = _AttentionModule().eval()
    args = (a["q"], a["k"], a["v"], a["pair_bias"], a["res_mask"])
    exported = torch.export.export(amod, args)
    targets = [str(n.target) for n in exported.graph.nodes if n.op == "call_function" and "tpf_b200" in str(n.target)]
    assert targets == ["tpf_b200.attn_fwd.default"], targets
    path = tmp_path / "attention.pt2"
    torch.export.save(exported, path)
    assert torch.equal(torch.export.load(path).module()(*args), amod(*args))


def test_lse_is_not_differentiable():
    dev = torch.device("cuda", 0)
    a, _ = _attention_case(dev, O=2, N=64)
    q = a["q"].detach().clone().requires_grad_(True)
    out, lse = tk.turbo_attention(q, a["k"], a["v"], pair_bias=a["pair_bias"], res_mask=a["res_mask"], return_lse=True)
    assert out.requires_grad and not lse.requires_grad


# --------------------------------------------------------------------------------------------
# bounded wait
# --------------------------------------------------------------------------------------------
def test_bounded_wait_gives_up_and_reports_once():
    dev = torch.device("cuda", 0)
    torch.cuda.synchronize(dev)
    assert C.device_status() == 0
    report = torch.zeros(3, dtype=torch.int32, device=dev)
    with torch.cuda.device(dev):
        C.call("tpf_selftest_bounded_wait", C.ptr(report), C.current_stream())
        torch.cuda.synchronize(dev)        # the kernel returned by itself
    first, second, finished = (int(x) & 0xFFFFFFFF for x in report.tolist())
    assert finished == 1                   # ran to its last statement
    assert first >= 2_000_000              # the first wait lasted until the limit ...
    assert first < 200_000_000             # ... and not much longer (about a millisecond, not seconds)
    assert second < 1_000_000              # the abort flag short-circuits later waits of the CTA
    assert C.device_status() == 1          # wait timeout reported ...
    assert C.device_status() == 0          # ... once (read-and-clear)
    # the context is intact: a real operator still runs and matches its earlier result
    a, d_a = _attention_case(dev, O=2, N=64)
    assert _same(_run_attention(a, d_a), _run_attention(a, d_a))
    assert C.device_status() == 0
