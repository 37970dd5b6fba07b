"""Axial sharding on the CUDA back end: a one-rank group must reproduce the unsharded operators,
and (when two GPUs are visible) a two-rank NCCL run must reproduce the CPU oracle."""
import datetime
import os
import tempfile

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

pytestmark = [pytest.mark.gpu, pytest.mark.skipif(not torch.cuda.is_available(), reason="needs a CUDA device")]


def _case(N=128, Cc=64, seed=5):
    from oracle.inputs import trimul_inputs
    inp = trimul_inputs(1, N, Cc, seed=seed, mask_mode="trailing10")
    g = torch.Generator().manual_seed(seed)
    inp["weights"]["norm_in_weight"] = 1 + 0.1 * torch.randn(Cc, generator=g)
    inp["weights"]["norm_out_bias"] = 0.1 * torch.randn(Cc, generator=g)
    inp["d_out"] = torch.randn(1, N, N, Cc, generator=g).bfloat16()
    return inp


def _worker(rank, world, init_file, results):
    import openfold3_triangle_kernel_b200 as tk
    from openfold3_triangle_kernel_b200 import dap
    from oracle import attention_oracle as ao
    from oracle import trimul_oracle as to
    from oracle.inputs import attention_inputs
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", init_method=f"file://{init_file}", rank=rank, world_size=world, device_id=dev,
                            timeout=datetime.timedelta(seconds=120))
    try:
        inp = _case()
        for direction in ("outgoing", "incoming"):
            z = dap.shard_rows(inp["z"], 1).to(dev).requires_grad_(True)
            w = {n: t.to(dev).requires_grad_(True) for n, t in inp["weights"].items()}
            out = dap.axial_trimul(z, direction, dap.shard_rows(inp["mask"], 1).to(dev), **w)
            out.backward(dap.shard_rows(inp["d_out"], 1).to(dev))
            torch.cuda.synchronize()
            assert tk._cabi.device_status() == 0
            ref = to.trimul_forward_backward(inp["z"], direction, inp["mask"], inp["weights"], inp["d_out"])
            full = dap.gather_rows(out.detach(), 1).cpu()
            assert ao.rel_l2(full, ref["out"]) <= 1e-2, direction
            assert ao.rel_l2(dap.gather_rows(z.grad, 1).cpu(), ref["dz"]) <= 2e-2, direction
            for n in to.WEIGHT_NAMES:
                assert ao.rel_l2(w[n].grad.cpu(), ref["d_" + n]) <= 2e-2, (direction, n)
            if world == 1:  # same kernels, same order: identical to the unsharded operator
                z2 = inp["z"].to(dev).requires_grad_(True)
                o2 = tk.turbo_trimul(z2, direction, inp["mask"].to(dev), **{n: t.detach() for n, t in w.items()})
                assert torch.equal(o2, out)
        a = attention_inputs(1, 8, 4, 136, 32, seed=3, mask_mode="random30")
        d_o = torch.randn(1, 8, 136, 4, 32, generator=torch.Generator().manual_seed(1)).bfloat16()
        q, k, v = (dap.shard_rows(a[n], 1).to(dev).requires_grad_(True) for n in ("q", "k", "v"))
        b = a["pair_bias"].to(dev).requires_grad_(True)
        o = dap.axial_attention(q, k, v, b, dap.shard_rows(a["res_mask"], 1).to(dev))
        o.backward(dap.shard_rows(d_o, 1).to(dev))
        ref = ao.attention_forward_backward(a["q"], a["k"], a["v"], a["pair_bias"], a["res_mask"], d_o)
        assert ao.rel_l2(dap.gather_rows(o.detach(), 1).cpu(), ref["out"]) <= 1e-2
        assert ao.rel_l2(dap.gather_rows(q.grad, 1).cpu(), ref["dq"]) <= 1e-2
        assert ao.rel_l2(b.grad.cpu(), ref["dbias"]) <= 1e-2
        results[rank] = "ok"
    except Exception as e:  # noqa: BLE001
        import traceback
        results[rank] = "".join(traceback.format_exception(e))
    finally:
        dist.destroy_process_group()


def _run(world):
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    with tempfile.TemporaryDirectory() as d:
        mgr = mp.Manager()
        results = mgr.dict()
        mp.spawn(_worker, args=(world, os.path.join(d, "rdv"), results), nprocs=world, join=True)
        for r in range(world):
            assert results.get(r) == "ok", results.get(r)


def test_axial_one_rank_matches_unsharded_operator():
    _run(1)


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_axial_two_ranks_nccl():
    _run(2)
