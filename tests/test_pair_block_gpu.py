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

# (N, C_z, heads, D): a small case and the channel / head geometry of the benchmark's pair-stack block
SMALL = (96, 64, 4, 16)
BLOCK_GEOMETRY = (256, 128, 4, 32)
ATT_WEIGHTS = ("w_q", "w_k", "w_v", "w_z", "w_g", "w_o")
TRI_WEIGHTS = ("p_in_weight", "g_in_weight", "p_out_weight", "g_out_weight")


def _inputs(cfg):
    from oracle.pair_block_oracle import block_params
    N, CZ, HEADS, D = cfg
    g = torch.Generator().manual_seed(21)
    z = torch.randn(1, N, N, CZ, generator=g).bfloat16()
    mask = torch.ones(1, N, N)
    mask[:, N - 8:, :] = 0
    mask[:, :, N - 8:] = 0
    d_out = torch.randn(1, N, N, CZ, generator=g).bfloat16() * mask.unsqueeze(-1).bfloat16()
    return z, mask, d_out, block_params(CZ, HEADS, D, seed=9)


def _oracle(cfg, z, mask, d_out, params):
    """fp64 oracle for the small case, fp32 for the large one (memory); returns plain tensors."""
    from oracle.pair_block_oracle import pair_block_forward
    dt = torch.float64 if cfg[0] <= 128 else torch.float32
    zz = z.detach().clone().to(dt).requires_grad_(True)
    pp = {k: {n: t.detach().clone().to(dt).requires_grad_(True) for n, t in v.items()} for k, v in params.items()}
    out = pair_block_forward(zz, mask, pp, cfg[2], dtype=dt)
    out.backward(d_out.to(dt))
    return dict(out=out.detach(), dz=zz.grad, grads={k: {n: t.grad for n, t in v.items()} for k, v in pp.items()})


def _rel(a, b, valid):
    a = torch.where(valid, a.double(), 0.0)
    b = torch.where(valid, b.double(), 0.0)
    return float((a - b).norm() / b.norm())


def _check_weight_grads(pd, ref):
    from oracle.attention_oracle import rel_l2
    for blk in ("tri_mul_out", "tri_mul_in"):
        for name in TRI_WEIGHTS:
            assert rel_l2(pd[blk][name].grad.cpu(), ref["grads"][blk][name]) <= 4e-2, (blk, name)
    for blk in ("tri_att_start", "tri_att_end"):
        for name in ATT_WEIGHTS:
            assert rel_l2(pd[blk][name].grad.cpu(), ref["grads"][blk][name]) <= 4e-2, (blk, name)


def _worker(rank, world, init_file, ref_file, cfg, results):
    import datetime
    from openfold3_triangle_kernel_b200 import dap
    from openfold3_triangle_kernel_b200.pair_block import pair_stack_block
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", init_method=f"file://{init_file}", rank=rank, world_size=world, device_id=dev,
                            timeout=datetime.timedelta(seconds=120))
    try:
        z, mask, d_out, params = _inputs(cfg)
        ref = torch.load(ref_file)
        valid = mask.bool().unsqueeze(-1)
        pd = {k: {n: t.to(dev).requires_grad_(True) for n, t in v.items()} for k, v in params.items()}
        zl = dap.shard_rows(z, 1).to(dev).requires_grad_(True)
        out = pair_stack_block(zl, dap.shard_rows(mask, 1).to(dev), pd, cfg[2], group=dist.group.WORLD)
        out.backward(dap.shard_rows(d_out, 1).to(dev))
        full = dap.gather_rows(out.detach(), 1).cpu()
        dz = dap.gather_rows(zl.grad, 1).cpu()
        assert _rel(full, ref["out"], valid) <= 2e-2
        assert _rel(dz, ref["dz"], valid) <= 4e-2
        # TriMul weights come back summed over the ranks by the operator; the attention wrapper's Linears are
        # plain torch ops on this rank's rows, so their gradients are partial sums: add them up here
        for blk in ("tri_att_start", "tri_att_end"):
            for name in ATT_WEIGHTS:
                dist.all_reduce(pd[blk][name].grad)
        _check_weight_grads(pd, ref)
        results[rank] = "ok"
    except Exception as e:  # noqa: BLE001
        import traceback
        results[rank] = "".join(traceback.format_exception(e))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("cfg", [SMALL, BLOCK_GEOMETRY], ids=["small", "c128_h4_d32_n256"])
def test_pair_block_single_gpu_matches_oracle(cfg):
    from openfold3_triangle_kernel_b200.pair_block import pair_stack_block
    z, mask, d_out, params = _inputs(cfg)
    ref = _oracle(cfg, z, mask, d_out, params)
    dev = "cuda"
    pd = {k: {n: t.to(dev).requires_grad_(True) for n, t in v.items()} for k, v in params.items()}
    zz = z.to(dev).requires_grad_(True)
    out = pair_stack_block(zz, mask.to(dev), pd, cfg[2])
    out.backward(d_out.to(dev))
    valid = mask.bool().unsqueeze(-1)
    assert _rel(out.detach().cpu(), ref["out"], valid) <= 2e-2
    assert _rel(zz.grad.cpu(), ref["dz"], valid) <= 4e-2
    _check_weight_grads(pd, ref)


def _run(world, cfg):
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    z, mask, d_out, params = _inputs(cfg)
    with tempfile.TemporaryDirectory() as d:
        ref_file = os.path.join(d, "oracle.pt")
        torch.save(_oracle(cfg, z, mask, d_out, params), ref_file)   # computed once, read by every rank
        mgr = mp.Manager()
        results = mgr.dict()
        mp.spawn(_worker, args=(world, os.path.join(d, "rdv"), ref_file, cfg, results), nprocs=world, join=True)
        for r in range(world):
            assert results.get(r) == "ok", results.get(r)


def test_pair_block_sharded_one_rank():
    _run(1, SMALL)


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
@pytest.mark.parametrize("cfg", [SMALL, BLOCK_GEOMETRY], ids=["small", "c128_h4_d32_n256"])
def test_pair_block_sharded_two_ranks(cfg):
    _run(2, cfg)
