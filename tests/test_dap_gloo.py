"""Axial (DAP) sharding logic with world_size = 2 on CPU (gloo): row<->channel all-to-alls,
the bias-gradient all-reduce of sharded attention and the staged, row-sharded TriMul against
the unsharded oracle.  The device stage functions are replaced by a torch fp64 back end, so
only the partition / collective plumbing is under test here."""
import os
import tempfile

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp
import torch.nn.functional as F

from openfold3_triangle_kernel_b200 import dap
from oracle import attention_oracle as ao
from oracle import trimul_oracle as to

WORLD = 2


class TorchStages:
    """fp64 autograd implementation of the TriMul stage interface used by dap._AxialTriMul."""

    @torch.enable_grad()
    def proj_fwd(self, z, mask, w, incoming):
        zz = z.detach().double().requires_grad_(True)
        ww = {k: v.detach().double().requires_grad_(True) for k, v in w.items()}
        c = z.shape[-1]
        zn = F.layer_norm(zz, (c,), ww["norm_in_weight"], ww["norm_in_bias"], 1e-5)
        p = F.linear(zn, ww["p_in_weight"])
        g = torch.sigmoid(F.linear(zn, ww["g_in_weight"]))
        m = mask.double().unsqueeze(-1)
        a = (m * g[..., :c] * p[..., :c]).permute(0, 3, 1, 2)
        b = (m * g[..., c:] * p[..., c:]).permute(0, 3, 1, 2)
        return dict(zz=zz, ww=ww, zn=zn, a=a, b=b, a_cm=a.detach().contiguous(), b_cm=b.detach().contiguous())

    def contract(self, a, b, incoming):
        return torch.einsum("bcki,bckj->bcij", a, b) if incoming else torch.einsum("bcik,bcjk->bcij", a, b)

    def contract_bwd(self, dx, a, b, incoming):
        if incoming:
            return torch.einsum("bcij,bckj->bcki", dx, b), torch.einsum("bcij,bcki->bckj", dx, a)
        return torch.einsum("bcij,bcjk->bcik", dx, b), torch.einsum("bcij,bcik->bcjk", dx, a)

    @torch.enable_grad()
    def out_fwd(self, st, x_cm):
        ww = st["ww"]
        c = st["zz"].shape[-1]
        x = x_cm.detach().requires_grad_(True)
        xn = F.layer_norm(x.permute(0, 2, 3, 1), (c,), ww["norm_out_weight"], ww["norm_out_bias"], 1e-5)
        out = F.linear(xn, ww["p_out_weight"]) * torch.sigmoid(F.linear(st["zn"], ww["g_out_weight"]))
        st["x"], st["out"] = x, out
        return out.detach()

    def out_bwd(self, st, d_out):
        st["out"].backward(d_out.double(), retain_graph=True)
        return st["x"].grad

    def proj_bwd(self, st, da, db):
        torch.autograd.backward([st["a"], st["b"]], [da, db])
        return st["zz"].grad, {k: v.grad for k, v in st["ww"].items()}


def _attention_fn(q, k, v, pair_bias, res_mask):
    out, _ = ao.attention_forward(q, k, v, pair_bias, res_mask, dtype=torch.float64)
    return out


def _worker(rank, init_file, results):
    dist.init_process_group("gloo", init_method=f"file://{init_file}", rank=rank, world_size=WORLD)
    try:
        g = torch.Generator().manual_seed(0)
        # ---- layout round trip
        B, Cc, N = 2, 4, 6
        full = torch.arange(B * Cc * N * N, dtype=torch.float64).reshape(B, Cc, N, N)
        mine = dap.shard_rows(full, 2)
        ch = dap.rows_to_channels(mine)
        assert torch.equal(ch, full[:, rank * (Cc // WORLD):(rank + 1) * (Cc // WORLD)])
        assert torch.equal(dap.channels_to_rows(ch), mine)
        assert torch.equal(dap.gather_rows(mine, 2), full)

        # ---- attention: outer rows sharded, bias replicated, dbias all-reduced
        Bq, O, H, Nq, D = 1, 4, 2, 10, 8
        q, k, v = (torch.randn(Bq, O, H, Nq, D, generator=g, dtype=torch.float64) for _ in range(3))
        bias = torch.randn(Bq, 1, H, Nq, Nq, generator=g, dtype=torch.float64)
        mask = torch.zeros(Bq, O, 1, 1, Nq, dtype=torch.float64)
        mask[..., 7:] = -1e9
        d_out = torch.randn(Bq, O, Nq, H, D, generator=g, dtype=torch.float64)
        ql, kl, vl = (dap.shard_rows(t, 1).requires_grad_(True) for t in (q, k, v))
        bl = bias.clone().requires_grad_(True)
        out = dap.axial_attention(ql, kl, vl, bl, dap.shard_rows(mask, 1), attention_fn=_attention_fn)
        out.backward(dap.shard_rows(d_out, 1))
        ref = ao.attention_forward_backward(q, k, v, bias, mask, d_out)
        assert torch.allclose(dap.gather_rows(out.detach(), 1), ref["out"], atol=1e-10)
        assert torch.allclose(dap.gather_rows(ql.grad, 1), ref["dq"], atol=1e-10)
        assert torch.allclose(dap.gather_rows(kl.grad, 1), ref["dk"], atol=1e-10)
        assert torch.allclose(bl.grad, ref["dbias"], atol=1e-10)          # full sum on every rank

        # ---- TriMul: rows sharded, channel-sharded contraction, both directions
        Bt, Nt, Ct = 1, 8, 4
        z = torch.randn(Bt, Nt, Nt, Ct, generator=g, dtype=torch.float64)
        tmask = torch.ones(Bt, Nt, Nt, dtype=torch.float64)
        tmask[:, 6:, :] = 0
        tmask[:, :, 6:] = 0
        w = {n: t.double() for n, t in to.xavier_weights(Ct, 3).items()}
        w["norm_in_weight"] = 1 + 0.1 * torch.randn(Ct, generator=g, dtype=torch.float64)
        w["norm_out_bias"] = 0.1 * torch.randn(Ct, generator=g, dtype=torch.float64)
        dy = torch.randn(Bt, Nt, Nt, Ct, generator=g, dtype=torch.float64)
        for direction in ("outgoing", "incoming"):
            zl = dap.shard_rows(z, 1).requires_grad_(True)
            wl = {n: t.clone().requires_grad_(True) for n, t in w.items()}
            o = dap.axial_trimul(zl, direction, dap.shard_rows(tmask, 1), backend=TorchStages(), **wl)
            o.backward(dap.shard_rows(dy, 1))
            r = to.trimul_forward_backward(z, direction, tmask, w, dy)
            assert torch.allclose(dap.gather_rows(o.detach(), 1), r["out"], atol=1e-10), direction
            assert torch.allclose(dap.gather_rows(zl.grad, 1), r["dz"], atol=1e-10), direction
            for n in to.WEIGHT_NAMES:
                assert torch.allclose(wl[n].grad, r["d_" + n], atol=1e-10), (direction, n)

        # ---- argument errors surface before any collective
        with pytest.raises(ValueError, match="shard"):
            dap.axial_trimul(z[:, :3], "outgoing", None, backend=TorchStages(), **w)
        with pytest.raises(ValueError, match="missing"):
            dap.axial_trimul(dap.shard_rows(z, 1), "outgoing", None, backend=TorchStages())
        results[rank] = "ok"
    except Exception as e:  # noqa: BLE001
        import traceback
        results[rank] = "".join(traceback.format_exception(e))
    finally:
        dist.destroy_process_group()


def _block_worker(rank, init_file, results):
    """The whole sharded pair-stack block on two CPU ranks (fp64 stage back ends) against the
    unsharded oracle: all-gathered bias projection, all-to-all transposes for the ending node,
    TriMul all-to-alls, gradient of the local rows."""
    dist.init_process_group("gloo", init_method=f"file://{init_file}", rank=rank, world_size=WORLD)
    try:
        from openfold3_triangle_kernel_b200.pair_block import _sharded_transpose, pair_stack_block
        from oracle.pair_block_oracle import block_params, pair_block_forward

        n, c, heads, d = 8, 8, 2, 4
        g = torch.Generator().manual_seed(5)
        z = torch.randn(1, n, n, c, generator=g, dtype=torch.float64)
        mask = torch.ones(1, n, n, dtype=torch.float64)
        mask[:, 6:, :] = 0
        mask[:, :, 6:] = 0
        dy = torch.randn(1, n, n, c, generator=g, dtype=torch.float64)
        params = block_params(c, heads, d, 9, dtype=torch.float64)

        # the sharded transpose is a global transpose of the two pair axes
        zt = _sharded_transpose(dap.shard_rows(z, 1).contiguous(), dist.group.WORLD)
        assert torch.equal(dap.gather_rows(zt, 1), z.transpose(1, 2))

        zl = dap.shard_rows(z, 1).clone().requires_grad_(True)
        out = pair_stack_block(zl, dap.shard_rows(mask, 1), params, heads, group=dist.group.WORLD,
                               trimul_backend=TorchStages(), attention_fn=_attention_fn)
        out.backward(dap.shard_rows(dy, 1))

        zr = z.clone().requires_grad_(True)
        ref = pair_block_forward(zr, mask, params, heads)
        ref.backward(dy)
        valid = (mask > 0)[..., None]
        # LayerNorm of the attention wrapper runs in fp32 in the product path: fp32-level agreement
        assert torch.allclose((dap.gather_rows(out.detach(), 1) * valid), ref.detach() * valid, atol=2e-5, rtol=2e-5)
        assert torch.allclose(dap.gather_rows(zl.grad, 1) * valid, zr.grad * valid, atol=2e-4, rtol=2e-4)
        results[rank] = "ok"
    except Exception as e:  # noqa: BLE001
        import traceback
        results[rank] = "".join(traceback.format_exception(e))
    finally:
        dist.destroy_process_group()


def test_sharded_pair_block_world_size_2_gloo():
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    with tempfile.TemporaryDirectory() as d:
        init_file = os.path.join(d, "rendezvous")
        mgr = mp.Manager()
        results = mgr.dict()
        mp.spawn(_block_worker, args=(init_file, results), nprocs=WORLD, join=True)
        for r in range(WORLD):
            assert results.get(r) == "ok", results.get(r)


def test_axial_sharding_world_size_2_gloo():
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    with tempfile.TemporaryDirectory() as d:
        init_file = os.path.join(d, "rendezvous")
        mgr = mp.Manager()
        results = mgr.dict()
        mp.spawn(_worker, args=(init_file, results), nprocs=WORLD, join=True)
        for r in range(WORLD):
            assert results.get(r) == "ok", results.get(r)
