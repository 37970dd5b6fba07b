#!/usr/bin/env python
"""Benchmark of the pair-stack hot path: triangle attention fwd+bwd (B=1, O=N=384, H=4, D=32)
plus the triangle multiplicative update fwd+bwd in both directions (z [1,384,384,128]), bf16.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

One step = one pass of the hot path over one batch of seeded synthetic input.

* N = 1: the step runs on one GPU through the raw C ABI on resident buffers (`value`) and through
  the public operators with host buffers (`e2e`).
* N > 1 (launched under torch.distributed.run): the SAME step is sharded axially over the N ranks
  (strong scaling): triangle attention shards its outer rows with the pair bias replicated and the
  bias gradient all-reduced; TriMul shards pair rows for LayerNorm / projections / gating and
  moves to a channel-sharded layout by all-to-all for the k-contraction and back.  The line also
  carries `dap_parity` (not timed): rel-L2 of the gathered sharded outputs and gradients against
  the unsharded operators run on rank 0.
* Every N also times the whole pair-stack block (TriMul out -> in -> attention start -> end with
  residuals, fwd+bwd) at N = 768 and N = 1536, sharded over the ranks: `block_n768_ms`,
  `block_n1536_ms`.

Rank 0 prints ONE JSON line.  `--impl reference` times the CPU restatement of the reference's
PyTorch path (oracle/) on the host cores of this box on the full, un-scaled step.
"""
from __future__ import annotations

import argparse
import datetime
import json
import math
import os
import statistics
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

ATT = dict(B=1, O=384, H=4, N=384, D=32)
TRI = dict(B=1, N=384, C=128)
ATT_FLOPS_FWD = 4 * ATT["B"] * ATT["O"] * ATT["H"] * ATT["N"] ** 2 * ATT["D"]
ATT_FLOPS = 14 * ATT["B"] * ATT["O"] * ATT["H"] * ATT["N"] ** 2 * ATT["D"]            # fwd + 2.5 x fwd
TRI_FLOPS = 3 * (12 * TRI["N"] ** 2 * TRI["C"] ** 2 + 2 * TRI["N"] ** 3 * TRI["C"]) * TRI["B"]
TRI_BMM_FLOPS = 2 * TRI["N"] ** 3 * TRI["C"] * TRI["B"]
STEP_FLOPS = ATT_FLOPS + 2 * TRI_FLOPS
WORKLOAD = "A384 attention (B1,O384,H4,N384,D32) + T384 TriMul outgoing+incoming (z[1,384,384,128]), fwd+bwd of mean(out^2)"
METRIC = "pair_stack_hot_path_fwd_bwd_tflops"
PG_TIMEOUT_S = 180


def log(rank, msg):
    """One progress line per phase on stderr, so that a stuck phase is visible in the run's log."""
    sys.stderr.write(f"[bench rank{rank} +{time.perf_counter() - _T0:7.1f}s] {msg}\n")
    sys.stderr.flush()


_T0 = time.perf_counter()


def _peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return dict(hbm_gbs=p["hbm_gbs"], bf16_tflops=p["bf16_tflops"], source="measured")
    return dict(hbm_gbs=6650.0, bf16_tflops=1590.0, source="fallback")


def _kernel_dram_bytes():
    """Per-kernel DRAM traffic (dram__bytes_read.sum + dram__bytes_write.sum per launch) from the
    tracked ncu data file; a kernel without an entry reports traffic null."""
    path = os.path.join(ROOT, "profiles", "kernel_dram_bytes.json")
    try:
        with open(path) as f:
            return json.load(f).get("kernels", {})
    except (OSError, ValueError):
        return {}


# ------------------------------------------------------------------------------------------
# CPU arm (oracle): the full step, un-scaled
# ------------------------------------------------------------------------------------------
def cpu_step_seconds(threads=None, o_chunk=96):
    """Time the oracle on the whole A384 attention fwd+bwd (outer rows processed in chunks of
    `o_chunk` to bound memory; every row is computed) and on T384 fwd+bwd in both directions.
    Returns (seconds, cores, description)."""
    from oracle import attention_oracle as ao
    from oracle import trimul_oracle as to
    from oracle.inputs import attention_inputs, trimul_inputs
    threads = threads or os.cpu_count() or 1
    torch.set_num_threads(threads)
    a = attention_inputs(ATT["B"], ATT["O"], ATT["H"], ATT["N"], ATT["D"], seed=2, dtype=torch.float32)
    d_out = torch.randn(ATT["B"], ATT["O"], ATT["N"], ATT["H"], ATT["D"])
    t = trimul_inputs(TRI["B"], TRI["N"], TRI["C"], seed=3, dtype=torch.float32)
    d_o = torch.randn(TRI["B"], TRI["N"], TRI["N"], TRI["C"])
    t0 = time.perf_counter()
    dbias = None
    for o0 in range(0, ATT["O"], o_chunk):
        sl = slice(o0, o0 + o_chunk)
        r = ao.attention_forward_backward(a["q"][:, sl], a["k"][:, sl], a["v"][:, sl], a["pair_bias"],
                                          a["res_mask"][:, sl], d_out[:, sl], dtype=torch.float32)
        dbias = r["dbias"] if dbias is None else dbias + r["dbias"]
    for direction in ("outgoing", "incoming"):
        to.trimul_forward_backward(t["z"], direction, t["mask"], t["weights"], d_o, dtype=torch.float32)
    sec = time.perf_counter() - t0
    desc = (f"oracle port (CPU restatement of the reference's stock PyTorch path) fp32 on {threads} host threads: "
            f"the whole step un-scaled - attention fwd+bwd on all {ATT['O']} outer rows (chunks of {o_chunk}), "
            f"TriMul fwd+bwd outgoing and incoming at full size")
    return sec, threads, desc


REFERENCE_ARM_BUDGET_S = 180.0  # wall-clock bound of the whole CPU arm, whatever --steps / --warmup ask for


def run_reference(args, rank):
    """CPU arm: every step is the whole step on the oracle.  One step takes several seconds, so the
    number of warm-up and timed steps is capped by a wall-clock budget (at least one timed step);
    the line states how many were timed."""
    if rank != 0:
        return
    t_start = time.perf_counter()
    times = []
    cores, desc = None, None
    for _ in range(min(args.warmup, 1)):
        _, cores, desc = cpu_step_seconds()
    per_sample = time.perf_counter() - t_start
    while len(times) < max(1, args.steps):
        if times and time.perf_counter() - t_start + max(per_sample, times[-1]) > REFERENCE_ARM_BUDGET_S:
            break
        sec, cores, desc = cpu_step_seconds()
        times.append(sec)
    sec = statistics.mean(times)
    val = STEP_FLOPS / sec / 1e12
    desc = f"{desc}; {len(times)} timed step(s) within a {REFERENCE_ARM_BUDGET_S:.0f} s budget"
    line = dict(impl="reference", metric=METRIC, value=val, unit="TFLOP/s", n_gpus=args.gpus, steps=args.steps,
                warmup=args.warmup, ms_per_step=sec * 1e3, higher_is_better=True,
                scaling="weak" if args.gpus == 1 else "strong", vs_baseline=None,
                dtype="f32", data="synthetic", config=dict(workload=WORKLOAD), steps_timed=len(times),
                cpu_baseline=dict(value=val, unit="TFLOP/s", cores=cores, kind="port", sample=desc),
                e2e=dict(value=val, unit="TFLOP/s", h2d_bytes_per_step=0, d2h_bytes_per_step=0))
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------------
# GPU arm
# ------------------------------------------------------------------------------------------
class ClockSampler:
    """Polls SM clock and clock-event reasons through NVML every ~5 ms while the timed region runs."""
    REASONS = dict(hw_slowdown=0x8, sw_power_cap=0x4, hw_thermal_slowdown=0x40, sw_thermal_slowdown=0x20)

    def __init__(self, index):
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop = threading.Event()
        self.t = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            visible = os.environ.get("CUDA_VISIBLE_DEVICES")
            phys = int(visible.split(",")[index]) if visible and visible.split(",")[index].isdigit() else index
            self.h = pynvml.nvmlDeviceGetHandleByIndex(phys)
            self.max_mhz = float(pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM))
            self.t = threading.Thread(target=self._poll, daemon=True)
            self.t.start()
        except Exception:
            self.nv = None

    def _poll(self):
        nv = self.nv
        while not self._stop.is_set():
            try:
                self.samples.append(float(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM)))
                try:
                    bits = nv.nvmlDeviceGetCurrentClocksEventReasons(self.h)
                except Exception:
                    bits = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                for name, bit in self.REASONS.items():
                    if bits & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            time.sleep(0.005)

    def stop(self):
        self._stop.set()
        if self.t is not None:
            self.t.join(timeout=2)
        return dict(sm_mhz=statistics.median(self.samples) if self.samples else None, sm_max_mhz=self.max_mhz,
                    reasons=sorted(self.reasons), samples=len(self.samples))


_TRI_W_FWD = ("p_in_weight", "g_in_weight", "p_out_weight", "g_out_weight", "norm_in_weight", "norm_in_bias",
              "norm_out_weight", "norm_out_bias")
_TRI_W_BWD = ("p_in_weight", "g_in_weight", "p_out_weight", "g_out_weight", "norm_in_weight", "norm_out_weight")


class Workload:
    """The step on this rank's share of the inputs.

    world == 1: device-resident buffers and raw C-ABI calls (no allocation inside the timed region).
    world  > 1: the same inputs (same seeds on every rank) sharded axially: this rank keeps outer rows
    [rank*O/P, (rank+1)*O/P) of the attention tensors and pair rows [rank*N/P, ...) of z; attention
    runs the same raw C-ABI calls on its rows followed by the dBias all-reduce, TriMul runs the staged
    C-ABI entry points with the all-to-alls of dap.axial_trimul_forward / _backward between them."""

    def __init__(self, dev, rank=0, world=1, group=None):
        from openfold3_triangle_kernel_b200 import _cabi as C
        from openfold3_triangle_kernel_b200.synthetic import attention_inputs, trimul_inputs
        self.C, self.dev, self.rank, self.world, self.group = C, dev, rank, world, group
        B, O, H, N, D = (ATT[k] for k in "BOHND")
        if O % world or TRI["N"] % world or TRI["C"] % world:
            raise SystemExit(f"--gpus {world} must divide O={O}, N={TRI['N']} and C={TRI['C']}")
        self.Ol = O // world
        osl = slice(rank * self.Ol, (rank + 1) * self.Ol)
        a = attention_inputs(B, O, H, N, D, seed=2)
        self.full_att = a
        a = dict(q=a["q"][:, osl].contiguous(), k=a["k"][:, osl].contiguous(), v=a["v"][:, osl].contiguous(),
                 pair_bias=a["pair_bias"], res_mask=a["res_mask"][:, osl].contiguous())
        self.host_att = {k: v.pin_memory() for k, v in a.items()}
        self.q, self.k, self.v = (a[n].to(dev) for n in ("q", "k", "v"))
        self.bias = a["pair_bias"].to(dev).reshape(1, H, N, N).contiguous()
        self.mask = a["res_mask"].to(dev).reshape(B, self.Ol, N).contiguous()
        Ol = self.Ol
        self.out = torch.empty(B, Ol, N, H, D, device=dev, dtype=torch.bfloat16)
        self.lse = torch.empty(B, Ol, H, N, device=dev)
        self.d_out = torch.empty_like(self.out)
        self.dq, self.dk, self.dv = (torch.empty(B, Ol, H, N, D, device=dev, dtype=torch.bfloat16) for _ in range(3))
        self.dbias = torch.empty(1, H, N, N, device=dev)
        self.delta = torch.empty(B, Ol, H, N, device=dev)
        self.att_ws_bytes = C.load().tpf_attn_bwd_workspace_bytes(B, Ol, H, N, D, 1)
        self.att_ws = torch.empty(max(self.att_ws_bytes, 256), device=dev, dtype=torch.uint8)
        self.scale = 1.0 / math.sqrt(D)
        self.qs = C.i64_array(self.q.stride()[:4])
        self.att_numel = B * O * N * H * D   # the loss is the mean over the WHOLE output

        Bt, Nt, Ct = TRI["B"], TRI["N"], TRI["C"]
        t = trimul_inputs(Bt, Nt, Ct, seed=3)
        self.full_tri = t
        self.Nl = Nt // world
        rsl = slice(rank * self.Nl, (rank + 1) * self.Nl)
        zl, ml = t["z"][:, rsl].contiguous(), t["mask"][:, rsl].contiguous()
        self.host_tri = dict(z=zl.pin_memory(), mask=ml.pin_memory(),
                             weights={k: v.pin_memory() for k, v in t["weights"].items()})
        self.z = zl.to(dev)
        self.tmask = ml.to(dev)
        self.w = {k: v.to(dev).float().contiguous() for k, v in t["weights"].items()}
        self.tri_numel = Bt * Nt * Nt * Ct
        if world == 1:
            R = Bt * Nt * Nt
            bf = lambda *s: torch.empty(s, device=dev, dtype=torch.bfloat16)  # noqa: E731
            f32 = lambda *s: torch.empty(s, device=dev)  # noqa: E731
            self.t_out, self.t_dout, self.t_dz = bf(R, Ct), bf(R, Ct), bf(R, Ct)
            self.saved = [bf(R, Ct), f32(R), f32(R), bf(Bt * Ct, Nt * Nt), bf(Bt * Ct, Nt * Nt), bf(R, Ct),
                          bf(Bt * Ct, Nt * Nt), bf(R, Ct), f32(R), f32(R)]
            self.wgrads = [f32(2 * Ct, Ct), f32(2 * Ct, Ct), f32(Ct, Ct), f32(Ct, Ct), f32(Ct), f32(Ct), f32(Ct),
                           f32(Ct)]
            self.t_ws_f = C.load().tpf_trimul_fwd_workspace_bytes(Bt, Nt, Ct)
            self.t_ws_b = C.load().tpf_trimul_bwd_workspace_bytes(Bt, Nt, Ct)
            self.t_ws = torch.empty(max(self.t_ws_f, self.t_ws_b), device=dev, dtype=torch.uint8)
        else:
            from openfold3_triangle_kernel_b200 import dap
            self.dap = dap
            self.stages = dap.CudaTrimulStages(reuse_buffers=True)
            self.t_dout = torch.empty(Bt, self.Nl, Nt, Ct, device=dev, dtype=torch.bfloat16)

    # ---- raw kernels -------------------------------------------------------------------
    def attn_fwd(self):
        C, p = self.C, self.C.ptr
        B, _, H, N, D = (ATT[k] for k in "BOHND")
        C.call("tpf_attn_fwd", p(self.q), p(self.k), p(self.v), self.qs, self.qs, self.qs, p(self.mask), N,
               p(self.bias), N, 1, p(self.out), p(self.lse), B, self.Ol, H, N, D, self.scale, C.current_stream())

    def attn_bwd(self, stages=7):
        C, p = self.C, self.C.ptr
        B, _, H, N, D = (ATT[k] for k in "BOHND")
        C.call("tpf_attn_bwd_stages", p(self.q), p(self.k), p(self.v), p(self.d_out), self.qs, self.qs, self.qs,
               p(self.out), p(self.lse), p(self.mask), N, p(self.bias), N, 1, p(self.dq), p(self.dk), p(self.dv),
               p(self.dbias), p(self.delta), p(self.att_ws), self.att_ws_bytes, B, self.Ol, H, N, D, self.scale,
               stages, C.current_stream())
        if self.world > 1 and (stages & 4):
            import torch.distributed as dist
            dist.all_reduce(self.dbias, op=dist.ReduceOp.SUM, group=self.group)

    def _wptrs(self, names):
        return [self.C.ptr(self.w[n]) for n in names]

    def trimul_fwd(self, incoming, stages=7):
        C, p = self.C, self.C.ptr
        Bt, Nt, Ct = TRI["B"], TRI["N"], TRI["C"]
        C.call("tpf_trimul_fwd_stages", p(self.z), p(self.tmask), *self._wptrs(_TRI_W_FWD), int(incoming), Bt, Nt, Ct,
               p(self.t_out), *[p(t) for t in self.saved], p(self.t_ws), self.t_ws_f, 0, stages, C.current_stream())

    def trimul_bwd(self, incoming, stages=7):
        C, p = self.C, self.C.ptr
        Bt, Nt, Ct = TRI["B"], TRI["N"], TRI["C"]
        C.call("tpf_trimul_bwd_stages", p(self.t_dout), p(self.z), p(self.tmask), *self._wptrs(_TRI_W_BWD),
               int(incoming), Bt, Nt, Ct, p(self.t_out), *[p(t) for t in self.saved], p(self.t_dz),
               *[p(t) for t in self.wgrads], p(self.t_ws), self.t_ws_b, 0, stages, None, None, None,
               C.current_stream())

    def trimul_sharded(self, incoming):
        dap = self.dap
        out, state = dap.axial_trimul_forward(self.z, self.tmask, bool(incoming), self.group, self.stages, self.w)
        torch.mul(out, 2.0 / self.tri_numel, out=self.t_dout)
        return dap.axial_trimul_backward(state, self.t_dout)

    def step(self):
        """One pass of the hot path on resident inputs: attention fwd+bwd, TriMul out fwd+bwd, TriMul in fwd+bwd.
        d(mean(out^2))/d(out) = 2 out / numel is produced on the device by one elementwise op."""
        self.attn_fwd()
        torch.mul(self.out, 2.0 / self.att_numel, out=self.d_out)
        self.attn_bwd()
        for incoming in (0, 1):
            if self.world == 1:
                self.trimul_fwd(incoming)
                torch.mul(self.t_out, 2.0 / self.tri_numel, out=self.t_dout)
                self.trimul_bwd(incoming)
            else:
                self.trimul_sharded(incoming)

    # ---- public API, host buffers ----------------------------------------------------------
    def _e2e_setup(self):
        dev = self.dev
        self.copy_stream = torch.cuda.Stream(device=dev)
        t, h = self.host_tri, self.host_att
        self.e2e_wnames = list(t["weights"])
        hosts = [t["z"], t["mask"]] + [t["weights"][n] for n in self.e2e_wnames] + \
                [h[n] for n in ("q", "k", "v", "pair_bias", "res_mask")]
        self.e2e_hosts = hosts
        # two sets of device staging buffers: the copies of step i+1 run under the kernels of step i
        self.e2e_slots = [[torch.empty_like(x, device=dev) for x in hosts] for _ in range(2)]
        self.e2e_ready = [torch.cuda.Event() for _ in range(2)]
        self.e2e_free = [torch.cuda.Event() for _ in range(2)]
        for ev in self.e2e_free:
            ev.record(torch.cuda.current_stream())

    def e2e_issue_copies(self, slot):
        """Host -> device copies of one step's inputs (z once for both directions) on the copy stream."""
        cs = self.copy_stream
        cs.wait_event(self.e2e_free[slot])
        with torch.cuda.stream(cs):
            for d, h in zip(self.e2e_slots[slot], self.e2e_hosts):
                d.copy_(h, non_blocking=True)
            self.e2e_ready[slot].record(cs)

    def e2e_compute(self, slot):
        """The step through the public operators on the staged inputs; returns the loss on the host."""
        import openfold3_triangle_kernel_b200 as tk
        main = torch.cuda.current_stream()
        main.wait_event(self.e2e_ready[slot])
        bufs = self.e2e_slots[slot]
        nw = len(self.e2e_wnames)
        z_in, mask_in, wbufs, att = bufs[0], bufs[1], bufs[2:2 + nw], bufs[2 + nw:]
        total = None
        for direction in ("outgoing", "incoming"):
            z = z_in.detach().requires_grad_(True)
            w = {n: x.detach().requires_grad_(True) for n, x in zip(self.e2e_wnames, wbufs)}
            if self.world == 1:
                o = tk.turbo_trimul(z, direction, mask_in, **w)
            else:
                o = self.dap.axial_trimul(z, direction, mask_in, group=self.group, **w)
            l2 = o.float().square().sum() / self.tri_numel
            l2.backward()
            total = l2.detach() if total is None else total + l2.detach()
        q, k, v, b = (x.detach().requires_grad_(True) for x in att[:4])
        if self.world == 1:
            out = tk.turbo_attention(q, k, v, pair_bias=b, res_mask=att[4])
        else:
            out = self.dap.axial_attention(q, k, v, b, att[4], group=self.group)
        loss = out.float().square().sum() / self.att_numel
        loss.backward()
        total = total + loss.detach()
        self.e2e_free[slot].record(main)
        return float(total.item())  # device -> host read of the step's result

    def e2e_loop(self, n):
        """n steps; the inputs of every step are copied from pinned host memory inside the loop, one
        step ahead of the kernels that read them."""
        self.e2e_issue_copies(0)
        for i in range(n):
            if i + 1 < n:
                self.e2e_issue_copies((i + 1) % 2)
            self.e2e_compute(i % 2)

    def e2e_bytes(self):
        return sum(x.numel() * x.element_size() for x in self.e2e_hosts), 4


def _time_loop(fn, steps, barrier=None):
    """CUDA-event time of `steps` calls of fn on the current stream (seconds)."""
    if barrier:
        barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    if barrier:
        barrier()
    return e0.elapsed_time(e1) / 1e3


def _rel_l2(a, b):
    a, b = a.double(), b.double()
    return float((a - b).norm() / b.norm().clamp_min(1e-30))


def dap_parity(wl, rank, world, group):
    """Not timed.  The sharded public operators (dap.axial_attention / dap.axial_trimul) on every rank
    against the unsharded operators run on rank 0 over the whole inputs: rel-L2 of the gathered
    outputs and gradients."""
    import torch.distributed as dist
    import openfold3_triangle_kernel_b200 as tk
    dap, dev = wl.dap, wl.dev
    res = {}
    g = torch.Generator().manual_seed(11)
    a = wl.full_att
    d_o = torch.randn(a["q"].shape[0], a["q"].shape[1], a["q"].shape[3], a["q"].shape[2], a["q"].shape[4],
                      generator=g).bfloat16()
    q, k, v = (dap.shard_rows(a[n], 1, group).to(dev).requires_grad_(True) for n in ("q", "k", "v"))
    b = a["pair_bias"].to(dev).requires_grad_(True)
    o = dap.axial_attention(q, k, v, b, dap.shard_rows(a["res_mask"], 1, group).to(dev), group=group)
    o.backward(dap.shard_rows(d_o, 1, group).to(dev))
    got = dict(out=dap.gather_rows(o.detach(), 1, group), dq=dap.gather_rows(q.grad, 1, group),
               dk=dap.gather_rows(k.grad, 1, group), dv=dap.gather_rows(v.grad, 1, group), dbias=b.grad)
    if rank == 0:
        q2, k2, v2, b2 = (a[n].to(dev).requires_grad_(True) for n in ("q", "k", "v", "pair_bias"))
        o2 = tk.turbo_attention(q2, k2, v2, pair_bias=b2, res_mask=a["res_mask"].to(dev))
        o2.backward(d_o.to(dev))
        ref = dict(out=o2.detach(), dq=q2.grad, dk=k2.grad, dv=v2.grad, dbias=b2.grad)
        for n in got:
            res["attention_" + n] = _rel_l2(got[n], ref[n])
    del q, k, v, b, o, got
    t = wl.full_tri
    d_t = torch.randn(t["z"].shape, generator=g).bfloat16()
    for direction in ("outgoing", "incoming"):
        z = dap.shard_rows(t["z"], 1, group).to(dev).requires_grad_(True)
        w = {n: x.to(dev).requires_grad_(True) for n, x in t["weights"].items()}
        o = dap.axial_trimul(z, direction, dap.shard_rows(t["mask"], 1, group).to(dev), group=group, **w)
        o.backward(dap.shard_rows(d_t, 1, group).to(dev))
        full_o, full_dz = dap.gather_rows(o.detach(), 1, group), dap.gather_rows(z.grad, 1, group)
        if rank == 0:
            z2 = t["z"].to(dev).requires_grad_(True)
            w2 = {n: x.to(dev).requires_grad_(True) for n, x in t["weights"].items()}
            o2 = tk.turbo_trimul(z2, direction, t["mask"].to(dev), **w2)
            o2.backward(d_t.to(dev))
            res[f"trimul_{direction}_out"] = _rel_l2(full_o, o2.detach())
            res[f"trimul_{direction}_dz"] = _rel_l2(full_dz, z2.grad)
            res[f"trimul_{direction}_dw_max"] = max(_rel_l2(w[n].grad, w2[n].grad) for n in w
                                                     if float(w2[n].grad.norm()) > 0)
    torch.cuda.synchronize()
    dist.barrier(group=group)
    if rank == 0:
        res["ranks"] = world
        res["max"] = max(v for k, v in res.items() if k != "ranks")
        res["tolerance"] = 2e-2
        res["ok"] = bool(res["max"] <= 2e-2)
    return res


def block_ms(n, rank, world, group, dev, steps=5, warmup=3):
    """fwd+bwd of the whole pair-stack block at pair size n (C_z=128, H=4, D=32), row-sharded over the
    ranks of `group` (unsharded operators when world == 1).  Returns (ms per step, operator FLOPs)."""
    import torch.distributed as dist
    from openfold3_triangle_kernel_b200.pair_block import pair_stack_block
    from openfold3_triangle_kernel_b200.synthetic import block_params
    c, heads, d = 128, 4, 32
    g = torch.Generator().manual_seed(4)
    nl = n // world
    z = torch.randn(1, nl, n, c, generator=g).bfloat16().to(dev).requires_grad_(True)
    mask = torch.ones(1, nl, n, device=dev)
    d_out = torch.randn(1, nl, n, c, generator=g).bfloat16().to(dev)
    params = {k: {m: t.to(dev).requires_grad_(True) for m, t in v.items()} for k, v in block_params(c, heads, d, 5).items()}

    def step():
        out = pair_stack_block(z, mask, params, heads, group=group if world > 1 else None)
        out.backward(d_out)
        z.grad = None

    for _ in range(warmup):
        step()
    barrier = (lambda: dist.barrier(group=group)) if world > 1 else None
    sec = _time_loop(step, steps, barrier) / steps
    t = torch.tensor([sec], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
    flops = 2 * 3 * (12 * n * n * c * c + 2 * n ** 3 * c) + 2 * 14 * n * heads * n * n * d
    del z, params, d_out
    torch.cuda.empty_cache()
    return float(t) * 1e3, flops


def run_gpu(args, rank, world, local_rank):
    import faulthandler
    import torch.distributed as dist
    # a stuck phase ends the run with every thread's stack on stderr instead of waiting for the caller's limit
    faulthandler.dump_traceback_later(args.watchdog, exit=True)
    dev = torch.device("cuda", local_rank)
    torch.cuda.set_device(dev)
    group = None
    if world > 1:
        # plain peer-to-peer rings: the collectives here are small, and a rank that dies while bound to an
        # NVLink multicast object can fault its peers
        os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
        log(rank, f"init_process_group nccl world={world}")
        dist.init_process_group("nccl", device_id=dev, timeout=datetime.timedelta(seconds=PG_TIMEOUT_S))
        group = dist.group.WORLD
        # host-side rendezvous (barriers around timed regions, the max over ranks of the timings) goes
        # through gloo, so that no eager NCCL collective has to follow the replay of the captured step
        host_group = dist.new_group(backend="gloo", timeout=datetime.timedelta(seconds=PG_TIMEOUT_S))
    barrier = (lambda: dist.barrier(group=host_group)) if world > 1 else None
    from openfold3_triangle_kernel_b200 import _cabi as C
    C.load()
    log(rank, "building workload")
    wl = Workload(dev, rank, world, group)

    log(rank, "warm-up")
    for _ in range(max(args.warmup, 3)):
        wl.step()
    torch.cuda.synchronize()
    if C.device_status() != 0:
        raise RuntimeError("device status word is non-zero after warm-up (a bounded wait timed out)")

    # per-stage times (same buffers, CUDA events on the launching stream)
    log(rank, "stage timers")
    stage = {}
    n_st = max(3, min(args.steps, 10))
    stages = [("attn_fwd", wl.attn_fwd), ("attn_bwd_delta", lambda: wl.attn_bwd(1)),
              ("attn_bwd_dqkv", lambda: wl.attn_bwd(2)), ("attn_bwd_dbias", lambda: wl.attn_bwd(4))]
    if world == 1:
        stages += [("trimul_out_fwd", lambda: wl.trimul_fwd(0)), ("trimul_out_bwd", lambda: wl.trimul_bwd(0)),
                   ("trimul_in_fwd", lambda: wl.trimul_fwd(1)), ("trimul_in_bwd", lambda: wl.trimul_bwd(1)),
                   ("trimul_out_fwd_proj", lambda: wl.trimul_fwd(0, 1)), ("trimul_out_fwd_contract", lambda: wl.trimul_fwd(0, 2)),
                   ("trimul_out_fwd_outproj", lambda: wl.trimul_fwd(0, 4)),
                   ("trimul_out_bwd_outproj", lambda: wl.trimul_bwd(0, 1)), ("trimul_out_bwd_contract", lambda: wl.trimul_bwd(0, 2)),
                   ("trimul_out_bwd_proj", lambda: wl.trimul_bwd(0, 4))]
    else:
        # the collectives of the sharded step on their own (same shapes and dtypes as inside the step)
        ab = [torch.empty(1, TRI["C"], wl.Nl, TRI["N"], device=dev, dtype=torch.bfloat16) for _ in range(2)]
        xc = torch.empty(1, TRI["C"] // world, TRI["N"], TRI["N"], device=dev, dtype=torch.bfloat16)
        wflat = torch.empty(6 * TRI["C"] * TRI["C"] + 4 * TRI["C"], device=dev)
        stages += [("trimul_out_fwd_bwd_sharded", lambda: wl.trimul_sharded(0)),
                   ("trimul_in_fwd_bwd_sharded", lambda: wl.trimul_sharded(1)),
                   ("coll_all_to_all_a_b_rows_to_channels", lambda: wl.dap.rows_to_channels_many(ab, group)),
                   ("coll_all_to_all_x_channels_to_rows", lambda: wl.dap.channels_to_rows(xc, group)),
                   ("coll_all_reduce_dbias_fp32", lambda: dist.all_reduce(wl.dbias, group=group)),
                   ("coll_all_reduce_weight_grads", lambda: dist.all_reduce(wflat, group=group))]
    for name, fn in stages:
        fn()
        stage[name] = _time_loop(fn, n_st, barrier) / n_st * 1e6  # us

    # end to end through the public operators with host buffers
    log(rank, "end-to-end loop")
    wl._e2e_setup()
    wl.e2e_loop(2)
    if barrier:
        barrier()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    n_e2e = max(2, min(args.steps, 10))
    wl.e2e_loop(n_e2e)
    e1.record()
    torch.cuda.synchronize()
    e2e_sec = max(e0.elapsed_time(e1) / 1e3, time.perf_counter() - t0) / n_e2e
    status = C.device_status()

    parity = None
    if world > 1:
        log(rank, "dap parity (not timed)")
        parity = dap_parity(wl, rank, world, group)
    blocks = {}
    if not args.skip_block:
        for n in (768, 1536):
            if n % world == 0:
                log(rank, f"pair-stack block N={n}")
                ms, fl = block_ms(n, rank, world, group, dev)
                blocks[n] = (ms, fl)
    status |= C.device_status()

    # The sharded step is many small launches (per-rank kernels shrink with N, collectives sit between
    # them), so at N > 1 the host cannot keep the stream fed: the whole step - kernels and NCCL
    # collectives - is captured once in a CUDA graph and replayed.  N = 1 launches directly.
    step_fn, graphed = wl.step, False
    launches_per_step = None
    if world > 1 and not args.no_graph:
        log(rank, "capturing the sharded step in a CUDA graph")
        torch.cuda.synchronize()
        barrier()
        l0 = C.load().tpf_launch_count()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            wl.step()
        launches_per_step = C.load().tpf_launch_count() - l0
        step_fn, graphed = graph.replay, True
        for _ in range(3):
            step_fn()
        torch.cuda.synchronize()

    log(rank, f"timed region: {args.steps} steps")
    sampler = ClockSampler(local_rank) if rank == 0 else None
    launches0 = C.load().tpf_launch_count()
    sec = _time_loop(step_fn, args.steps, barrier)
    launches = C.load().tpf_launch_count() - launches0
    if graphed:
        launches = launches_per_step * args.steps   # replayed launches do not pass through the library's counter
    clocks = sampler.stop() if sampler else None

    status |= C.device_status()
    t_step = torch.tensor([sec / args.steps, e2e_sec] + [stage[k] for k in sorted(stage)], dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t_step, op=dist.ReduceOp.MAX, group=host_group)
    vals = [float(x) for x in t_step.tolist()]
    step_sec, e2e_sec = vals[0], vals[1]
    stage = dict(zip(sorted(stage), vals[2:]))

    if rank == 0:
        peaks = _peaks()
        # dominant kernel: the slowest of the three single-kernel attention stages (tensor roofline)
        share = 1.0 / world
        cands = {"attn_fwd_kernel (A384)": ("attn_fwd", ATT_FLOPS_FWD * share),
                 "attn_bwd_kernel (dq/dk/dv, A384)": ("attn_bwd_dqkv", 2.5 * ATT_FLOPS_FWD * share),
                 "attn_dbias_kernel (A384)": ("attn_bwd_dbias", ATT_FLOPS_FWD * share)}
        dom = max(cands, key=lambda k: stage[cands[k][0]])
        dom_us, dom_flops = stage[cands[dom][0]], cands[dom][1]
        achieved = dom_flops / (dom_us * 1e-6) / 1e12
        dram = _kernel_dram_bytes().get(dom.split(" ")[0]) if world == 1 else None
        traffic = (dram["dram_read_bytes"] + dram["dram_write_bytes"]) if dram else None
        rooflines = {k: dict(launch_us=round(stage[s], 1), tflops=fl / (stage[s] * 1e-6) / 1e12,
                             frac=fl / (stage[s] * 1e-6) / 1e12 / peaks["bf16_tflops"]) for k, (s, fl) in cands.items()}
        if world == 1:
            for d in ("fwd", "bwd"):
                us = stage[f"trimul_out_{d}_contract"]
                fl = TRI_BMM_FLOPS * (1 if d == "fwd" else 2)
                rooflines[f"trimul k-contraction {d} (gemm_umma_kernel, T384)"] = dict(
                    launch_us=round(us, 1), tflops=fl / (us * 1e-6) / 1e12, frac=fl / (us * 1e-6) / 1e12 / peaks["bf16_tflops"])
        # the CPU baseline is timed at N = 1 only (the other ranks of a multi-GPU run would sit in a barrier)
        cpu_sec, cores, desc = (None, None, None)
        if world == 1 and not args.skip_cpu:
            log(rank, "cpu baseline (oracle)")
            cpu_sec, cores, desc = cpu_step_seconds()
        h2d, d2h = wl.e2e_bytes()
        att_us = stage["attn_fwd"] + stage["attn_bwd_delta"] + stage["attn_bwd_dqkv"] + stage["attn_bwd_dbias"]
        stage_tflops = dict(attention_fwd_bwd=ATT_FLOPS / (att_us * 1e-6) / 1e12)
        if world == 1:
            stage_tflops["trimul_outgoing_fwd_bwd"] = TRI_FLOPS / ((stage["trimul_out_fwd"] + stage["trimul_out_bwd"]) * 1e-6) / 1e12
            stage_tflops["trimul_incoming_fwd_bwd"] = TRI_FLOPS / ((stage["trimul_in_fwd"] + stage["trimul_in_bwd"]) * 1e-6) / 1e12
        else:
            stage_tflops["trimul_outgoing_fwd_bwd"] = TRI_FLOPS / (stage["trimul_out_fwd_bwd_sharded"] * 1e-6) / 1e12
            stage_tflops["trimul_incoming_fwd_bwd"] = TRI_FLOPS / (stage["trimul_in_fwd_bwd_sharded"] * 1e-6) / 1e12
        line = dict(
            metric=METRIC, value=STEP_FLOPS / step_sec / 1e12, unit="TFLOP/s", n_gpus=world,
            steps=args.steps, warmup=max(args.warmup, 3), ms_per_step=step_sec * 1e3, higher_is_better=True,
            scaling="weak" if world == 1 else "strong", vs_baseline=None, dtype="bf16", data="synthetic",
            config=dict(workload=WORKLOAD,
                        parallelism=("single GPU" if world == 1 else
                                     f"axial x{world}: attention outer rows sharded + dBias all-reduce; TriMul pair rows "
                                     f"sharded, all-to-all to channel shards for the k-contraction and back"),
                        launch=("CUDA graph replay of the whole sharded step (kernels + NCCL collectives)" if graphed
                                else "direct launches"),
                        l2_policy="working set per step (>1 GB over all ranks) exceeds the 126 MB L2; inputs are "
                                  "re-read from HBM every step",
                        seeds=dict(attention=2, trimul=3)),
            stage_us={k: round(v, 1) for k, v in stage.items()},
            stage_tflops=stage_tflops,
            roofline=dict(bound="tensor", kernel=dom, achieved=achieved,
                          peak=peaks["bf16_tflops"], unit="TFLOP/s", frac=achieved / peaks["bf16_tflops"],
                          peak_source=peaks["source"] + " cuBLAS bf16 burst", traffic=traffic,
                          traffic_source=(dram or {}).get("source"),
                          algorithmic_flops_per_launch=dom_flops, launch_us=dom_us),
            rooflines=rooflines,
            cpu_baseline=(dict(value=STEP_FLOPS / cpu_sec / 1e12, unit="TFLOP/s", cores=cores, kind="port", sample=desc,
                               seconds=cpu_sec) if cpu_sec else None),
            e2e=dict(value=STEP_FLOPS / e2e_sec / 1e12, unit="TFLOP/s", h2d_bytes_per_step=h2d * world,
                     d2h_bytes_per_step=d2h * world, ms_per_step=e2e_sec * 1e3),
            gpu_launches=int(launches), device_status=status, clocks=clocks)
        if parity is not None:
            line["dap_parity"] = parity
        for n, (ms, fl) in blocks.items():
            line[f"block_n{n}_ms"] = ms
            line[f"block_n{n}_tflops"] = fl / (ms * 1e-3) / 1e12
        print(json.dumps(line), flush=True)
    if world > 1:
        barrier()
        faulthandler.cancel_dump_traceback_later()
        if graphed:
            # Tearing down an NCCL communicator whose collectives sit in an instantiated CUDA graph did not
            # return on this stack (NCCL 2.28 / torch 2.11): every rank has passed the barrier and rank 0 has
            # printed its line, so leave without the teardown.
            sys.stdout.flush()
            sys.stderr.flush()
            os._exit(0)
        dist.destroy_process_group()
    faulthandler.cancel_dump_traceback_later()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--skip-block", action="store_true", help="do not time the N=768 / N=1536 pair-stack block")
    ap.add_argument("--skip-cpu", action="store_true", help="do not time the CPU oracle beside the GPU run")
    ap.add_argument("--watchdog", type=int, default=900, help="seconds after which a hung run dumps its stacks and exits")
    ap.add_argument("--no-graph", action="store_true", help="N > 1: launch the sharded step directly instead of replaying a CUDA graph")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, rank)
        return
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (B200); there is no CPU fallback for the product path")
    run_gpu(args, rank, world, local_rank)


if __name__ == "__main__":
    main()
