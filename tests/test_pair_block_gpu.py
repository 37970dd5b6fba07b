"""Pair-stack block (TriMul out -> in -> attention start -> end with residuals; BASELINE configs 4/5 at
test size) on the B200 operators against the CPU oracle of the reference PairBlock, unsharded and
axially sharded."""
import os
import tempfile

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

pytestmark = [pytest.mark.gpu, pytest.mark.skipif(not torch.cuda.is_available(), reason="needs a CUDA device")]

N, CZ, HEADS, D = 96, 64, 4, 16


def _inputs():
    from oracle.pair_block_oracle import block_params
    g = torch.Generator().manual_seed(21)
    z = torch.randn(1, N, N, CZ, generator=g).bfloat16()
    mask = torch.ones(1, N, N)
    mask[:, N - 8:, :] = 0
    mask[:, :, N - 8:] = 0
    d_out = torch.randn(1, N, N, CZ, generator=g).bfloat16() * mask.unsqueeze(-1).bfloat16()
    return z, mask, d_out, block_params(CZ, HEADS, D, seed=9)


def _oracle(z, mask, d_out, params):
    from oracle.pair_block_oracle import pair_block_forward
    zz = z.double().requires_grad_(True)
    pp = {k: {n: t.double().requires_grad_(True) for n, t in v.items()} for k, v in params.items()}
    out = pair_block_forward(zz, mask, pp, HEADS)
    out.backward(d_out.double())
    return out.detach(), zz.grad, pp


def _rel(a, b, valid):
    a = torch.where(valid, a.double(), 0.0)
    b = torch.where(valid, b.double(), 0.0)
    return float((a - b).norm() / b.norm())


def _worker(rank, world, init_file, results):
    from openfold3_triangle_kernel_b200 import dap
    from openfold3_triangle_kernel_b200.pair_block import pair_stack_block
    from oracle.attention_oracle import rel_l2
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", init_method=f"file://{init_file}", rank=rank, world_size=world, device_id=dev)
    try:
        z, mask, d_out, params = _inputs()
        ref_out, ref_dz, ref_p = _oracle(z, mask, d_out, params)
        valid = mask.bool().unsqueeze(-1)
        pd = {k: {n: t.to(dev).requires_grad_(True) for n, t in v.items()} for k, v in params.items()}
        zl = dap.shard_rows(z, 1).to(dev).requires_grad_(True)
        out = pair_stack_block(zl, dap.shard_rows(mask, 1).to(dev), pd, HEADS, group=dist.group.WORLD)
        out.backward(dap.shard_rows(d_out, 1).to(dev))
        full = dap.gather_rows(out.detach(), 1).cpu()
        dz = dap.gather_rows(zl.grad, 1).cpu()
        assert _rel(full, ref_out, valid) <= 2e-2
        assert _rel(dz, ref_dz, valid) <= 4e-2
        # replicated parameters: every rank must hold the gradient summed over all rows
        for blk, name in (("tri_mul_out", "p_in_weight"), ("tri_mul_in", "g_out_weight")):
            assert rel_l2(pd[blk][name].grad.cpu(), ref_p[blk][name].grad) <= 4e-2, (blk, name)
        results[rank] = "ok"
    except Exception as e:  # noqa: BLE001
        import traceback
        results[rank] = "".join(traceback.format_exception(e))
    finally:
        dist.destroy_process_group()


def test_pair_block_single_gpu_matches_oracle():
    from openfold3_triangle_kernel_b200.pair_block import pair_stack_block
    from oracle.attention_oracle import rel_l2
    z, mask, d_out, params = _inputs()
    ref_out, ref_dz, ref_p = _oracle(z, mask, d_out, params)
    dev = "cuda"
    pd = {k: {n: t.to(dev).requires_grad_(True) for n, t in v.items()} for k, v in params.items()}
    zz = z.to(dev).requires_grad_(True)
    out = pair_stack_block(zz, mask.to(dev), pd, HEADS)
    out.backward(d_out.to(dev))
    valid = mask.bool().unsqueeze(-1)
    assert _rel(out.detach().cpu(), ref_out, valid) <= 2e-2
    assert _rel(zz.grad.cpu(), ref_dz, valid) <= 4e-2
    for blk in ("tri_mul_out", "tri_mul_in"):
        for name in ("p_in_weight", "g_in_weight", "p_out_weight", "g_out_weight"):
            assert rel_l2(pd[blk][name].grad.cpu(), ref_p[blk][name].grad) <= 4e-2, (blk, name)
    for blk in ("tri_att_start", "tri_att_end"):
        for name in ("w_q", "w_k", "w_v", "w_z", "w_o"):
            assert rel_l2(pd[blk][name].grad.cpu(), ref_p[blk][name].grad) <= 4e-2, (blk, name)


def _run(world):
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    with tempfile.TemporaryDirectory() as d:
        mgr = mp.Manager()
        results = mgr.dict()
        mp.spawn(_worker, args=(world, os.path.join(d, "rdv"), results), nprocs=world, join=True)
        for r in range(world):
            assert results.get(r) == "ok", results.get(r)


def test_pair_block_sharded_one_rank():
    _run(1)


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_pair_block_sharded_two_ranks():
    _run(2)
