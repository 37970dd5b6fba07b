#!/usr/bin/env python
"""Benchmark of the pair-stack hot path: triangle attention fwd+bwd (B=1, O=N=384, H=4, D=32)
plus the triangle multiplicative update fwd+bwd in both directions (z [1,384,384,128]), bf16.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

One step = one pass of the hot path over one batch of seeded synthetic input.  With N > 1
(launched under torch.distributed.run) every rank runs its own batch (weak scaling, no
data-path collective: the operators are independent per batch, which is also the only
parallelism the reference has - data-parallel replicas).  Rank 0 prints ONE JSON line.

`--impl reference` times the CPU restatement of the reference's PyTorch path (oracle/) on the
host cores of this box, on a bounded sample of the same workload.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import statistics
import subprocess
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
STEP_FLOPS = ATT_FLOPS + 2 * TRI_FLOPS
WORKLOAD = "A384 attention (B1,O384,H4,N384,D32) + T384 TriMul outgoing+incoming (z[1,384,384,128]), fwd+bwd of mean(out^2)"
METRIC = "pair_stack_hot_path_fwd_bwd_tflops"

# dram__bytes_read.sum + dram__bytes_write.sum per launch of the dominant kernel (attention
# dq/dk/dv kernel at A384): 157.71 MB read + 73.44 MB written in the ncu capture summarised in
# profiles/attention_kernels_a384.md (algorithmic minimum: q,k,v,dO in + dq,dk,dv out = 264 MB;
# part of the inputs is still L2-resident from the forward pass).
DOMINANT_KERNEL_DRAM_BYTES = 231.15e6


def _peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return dict(hbm_gbs=p["hbm_gbs"], bf16_tflops=p["bf16_tflops"], source="measured")
    return dict(hbm_gbs=6650.0, bf16_tflops=1590.0, source="fallback")


# ------------------------------------------------------------------------------------------
# CPU arm (oracle): bounded sample of the same workload
# ------------------------------------------------------------------------------------------
def cpu_sample_seconds(att_rows=24, threads=None):
    """Time the oracle on `att_rows` of the 384 outer rows of A384 and on full T384 (both
    directions).  Returns (seconds_scaled_to_full_step, cores, description)."""
    from oracle import attention_oracle as ao
    from oracle import trimul_oracle as to
    from oracle.inputs import attention_inputs, trimul_inputs
    threads = threads or os.cpu_count() or 1
    torch.set_num_threads(threads)
    a = attention_inputs(ATT["B"], att_rows, ATT["H"], ATT["N"], ATT["D"], seed=2, dtype=torch.float32)
    d_out = torch.randn(ATT["B"], att_rows, ATT["N"], ATT["H"], ATT["D"])
    t0 = time.perf_counter()
    ao.attention_forward_backward(a["q"], a["k"], a["v"], a["pair_bias"], a["res_mask"], d_out, dtype=torch.float32)
    t_att = (time.perf_counter() - t0) * (ATT["O"] / att_rows)
    t = trimul_inputs(TRI["B"], TRI["N"], TRI["C"], seed=3, dtype=torch.float32)
    d_o = torch.randn(TRI["B"], TRI["N"], TRI["N"], TRI["C"])
    t0 = time.perf_counter()
    to.trimul_forward_backward(t["z"], "outgoing", t["mask"], t["weights"], d_o, dtype=torch.float32)
    t_tri = (time.perf_counter() - t0) * 2
    desc = (f"oracle fp32 on {threads} host threads: attention fwd+bwd on {att_rows}/384 outer rows (scaled x"
            f"{ATT['O'] // att_rows}), TriMul fwd+bwd one direction at full size (scaled x2)")
    return t_att + t_tri, threads, desc


REFERENCE_ARM_BUDGET_S = 180.0  # wall-clock bound of the whole CPU arm, whatever --steps / --warmup ask for


def run_reference(args, rank):
    """CPU arm: every step is the bounded sample of cpu_sample_seconds().  One sample takes several
    seconds, so the number of warm-up and timed samples is capped by a wall-clock budget (at least
    one timed sample); the line states how many were timed."""
    if rank != 0:
        return
    t_start = time.perf_counter()
    times = []
    cores, desc = None, None
    for _ in range(min(args.warmup, 1)):
        _, cores, desc = cpu_sample_seconds()
    per_sample = time.perf_counter() - t_start
    while len(times) < max(1, args.steps):
        if times and time.perf_counter() - t_start + max(per_sample, times[-1]) > REFERENCE_ARM_BUDGET_S:
            break
        sec, cores, desc = cpu_sample_seconds()
        times.append(sec)
    sec = statistics.mean(times)
    val = STEP_FLOPS / sec / 1e12
    desc = f"{desc}; {len(times)} timed sample(s) within a {REFERENCE_ARM_BUDGET_S:.0f} s budget"
    line = dict(impl="reference", metric=METRIC, value=val, unit="TFLOP/s", n_gpus=args.gpus, steps=args.steps,
                warmup=args.warmup, ms_per_step=sec * 1e3, higher_is_better=True, scaling="weak", vs_baseline=None,
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


class Workload:
    """Device-resident buffers and raw C-ABI calls (no allocation inside the timed region)."""

    def __init__(self, dev):
        from openfold3_triangle_kernel_b200 import _cabi as C
        from openfold3_triangle_kernel_b200.synthetic import attention_inputs, trimul_inputs
        self.C = C
        self.dev = dev
        B, O, H, N, D = (ATT[k] for k in "BOHND")
        a = attention_inputs(B, O, H, N, D, seed=2)
        self.host_att = {k: v.pin_memory() for k, v in a.items()}
        self.q, self.k, self.v = (a[n].to(dev) for n in ("q", "k", "v"))
        self.bias = a["pair_bias"].to(dev).reshape(1, H, N, N).contiguous()
        self.mask = a["res_mask"].to(dev).reshape(B, O, N).contiguous()
        self.out = torch.empty(B, O, N, H, D, device=dev, dtype=torch.bfloat16)
        self.lse = torch.empty(B, O, H, N, device=dev)
        self.d_out = torch.empty_like(self.out)
        self.dq, self.dk, self.dv = (torch.empty(B, O, H, N, D, device=dev, dtype=torch.bfloat16) for _ in range(3))
        self.dbias = torch.empty(1, H, N, N, device=dev)
        self.delta = torch.empty(B, O, H, N, device=dev)
        self.att_ws_bytes = C.load().tpf_attn_bwd_workspace_bytes(B, O, H, N, D, 1)
        self.att_ws = torch.empty(max(self.att_ws_bytes, 256), device=dev, dtype=torch.uint8)
        self.scale = 1.0 / math.sqrt(D)
        self.qs = C.i64_array(self.q.stride()[:4])

        Bt, Nt, Ct = TRI["B"], TRI["N"], TRI["C"]
        t = trimul_inputs(Bt, Nt, Ct, seed=3)
        self.host_tri = dict(z=t["z"].pin_memory(), mask=t["mask"].pin_memory(),
                             weights={k: v.pin_memory() for k, v in t["weights"].items()})
        self.z = t["z"].to(dev)
        self.tmask = t["mask"].to(dev)
        self.w = {k: v.to(dev).float().contiguous() for k, v in t["weights"].items()}
        R = Bt * Nt * Nt
        bf = lambda *s: torch.empty(s, device=dev, dtype=torch.bfloat16)  # noqa: E731
        f32 = lambda *s: torch.empty(s, device=dev)  # noqa: E731
        self.t_out, self.t_dout, self.t_dz = bf(R, Ct), bf(R, Ct), bf(R, Ct)
        self.saved = [bf(R, Ct), f32(R), f32(R), bf(Bt * Ct, Nt * Nt), bf(Bt * Ct, Nt * Nt), bf(R, Ct),
                      bf(Bt * Ct, Nt * Nt), bf(R, Ct), f32(R), f32(R)]
        self.wgrads = [f32(2 * Ct, Ct), f32(2 * Ct, Ct), f32(Ct, Ct), f32(Ct, Ct), f32(Ct), f32(Ct), f32(Ct), f32(Ct)]
        self.t_ws_f = C.load().tpf_trimul_fwd_workspace_bytes(Bt, Nt, Ct)
        self.t_ws_b = C.load().tpf_trimul_bwd_workspace_bytes(Bt, Nt, Ct)
        self.t_ws = torch.empty(max(self.t_ws_f, self.t_ws_b), device=dev, dtype=torch.uint8)

    # ---- raw kernels -------------------------------------------------------------------
    def attn_fwd(self):
        C, p = self.C, self.C.ptr
        B, O, H, N, D = (ATT[k] for k in "BOHND")
        C.call("tpf_attn_fwd", p(self.q), p(self.k), p(self.v), self.qs, self.qs, self.qs, p(self.mask), N,
               p(self.bias), N, 1, p(self.out), p(self.lse), B, O, H, N, D, self.scale, C.current_stream())

    def attn_bwd(self, stages=7):
        C, p = self.C, self.C.ptr
        B, O, H, N, D = (ATT[k] for k in "BOHND")
        C.call("tpf_attn_bwd_stages", p(self.q), p(self.k), p(self.v), p(self.d_out), self.qs, self.qs, self.qs,
               p(self.out), p(self.lse), p(self.mask), N, p(self.bias), N, 1, p(self.dq), p(self.dk), p(self.dv),
               p(self.dbias), p(self.delta), p(self.att_ws), self.att_ws_bytes, B, O, H, N, D, self.scale, stages,
               C.current_stream())

    def _wptrs(self, names):
        return [self.C.ptr(self.w[n]) for n in names]

    def trimul_fwd(self, incoming):
        C, p = self.C, self.C.ptr
        Bt, Nt, Ct = TRI["B"], TRI["N"], TRI["C"]
        names = ("p_in_weight", "g_in_weight", "p_out_weight", "g_out_weight", "norm_in_weight", "norm_in_bias",
                 "norm_out_weight", "norm_out_bias")
        C.call("tpf_trimul_fwd", p(self.z), p(self.tmask), *self._wptrs(names), int(incoming), Bt, Nt, Ct,
               p(self.t_out), *[p(t) for t in self.saved], p(self.t_ws), self.t_ws_f, C.current_stream())

    def trimul_bwd(self, incoming):
        C, p = self.C, self.C.ptr
        Bt, Nt, Ct = TRI["B"], TRI["N"], TRI["C"]
        names = ("p_in_weight", "g_in_weight", "p_out_weight", "g_out_weight", "norm_in_weight", "norm_out_weight")
        C.call("tpf_trimul_bwd", p(self.t_dout), p(self.z), p(self.tmask), *self._wptrs(names), int(incoming), Bt, Nt,
               Ct, p(self.t_out), *[p(t) for t in self.saved], p(self.t_dz), *[p(t) for t in self.wgrads],
               p(self.t_ws), self.t_ws_b, C.current_stream())

    def step(self):
        """One pass of the hot path on resident inputs: attention fwd+bwd, TriMul out fwd+bwd, TriMul in fwd+bwd.
        d(mean(out^2))/d(out) = 2 out / numel is produced on the device by one elementwise op."""
        self.attn_fwd()
        torch.mul(self.out, 2.0 / self.out.numel(), out=self.d_out)
        self.attn_bwd()
        for incoming in (0, 1):
            self.trimul_fwd(incoming)
            torch.mul(self.t_out, 2.0 / self.t_out.numel(), out=self.t_dout)
            self.trimul_bwd(incoming)

    # ---- public API, host buffers ----------------------------------------------------------
    def e2e_step(self):
        """One step through the public operators with HOST inputs: every input tensor of the step is
        copied from pinned host memory (on a copy stream, so the copies of the later operators run
        under the earlier operators' kernels), and the step's loss is read back to the host."""
        import openfold3_triangle_kernel_b200 as tk
        dev = self.dev
        main = torch.cuda.current_stream()
        if not hasattr(self, "copy_stream"):
            self.copy_stream = torch.cuda.Stream(device=dev)
        cs = self.copy_stream
        start = torch.cuda.Event()
        start.record(main)
        cs.wait_event(start)  # the destination buffers may be blocks the previous step just released

        def stage(hosts):
            devs = [torch.empty_like(h, device=dev) for h in hosts]  # allocated in main-stream order
            with torch.cuda.stream(cs):
                for d, h in zip(devs, hosts):
                    d.copy_(h, non_blocking=True)
                ev = torch.cuda.Event()
                ev.record(cs)
            return devs, ev

        t = self.host_tri
        wnames = list(t["weights"])
        tri = [stage([t["z"], t["mask"]] + [t["weights"][n] for n in wnames]) for _ in range(2)]
        h = self.host_att
        att, att_ev = stage([h[n] for n in ("q", "k", "v", "pair_bias", "res_mask")])

        total = None
        for direction, (bufs, ev) in zip(("outgoing", "incoming"), tri):
            main.wait_event(ev)
            z = bufs[0].requires_grad_(True)
            w = {n: x.requires_grad_(True) for n, x in zip(wnames, bufs[2:])}
            o = tk.turbo_trimul(z, direction, bufs[1], **w)
            l2 = o.float().square().mean()
            l2.backward()
            total = l2.detach() if total is None else total + l2.detach()
        main.wait_event(att_ev)
        q, k, v, b = (x.requires_grad_(True) for x in att[:4])
        out = tk.turbo_attention(q, k, v, pair_bias=b, res_mask=att[4])
        loss = out.float().square().mean()
        loss.backward()
        total = total + loss.detach()
        return float(total.item())  # device -> host read of the step's result

    def e2e_bytes(self):
        h2d = sum(v.numel() * v.element_size() for v in self.host_att.values())
        t = self.host_tri
        per_dir = t["z"].numel() * 2 + t["mask"].numel() * 4 + sum(v.numel() * 4 for v in t["weights"].values())
        return h2d + 2 * per_dir, 4


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


def run_gpu(args, rank, world, local_rank):
    import torch.distributed as dist
    dev = torch.device("cuda", local_rank)
    torch.cuda.set_device(dev)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    barrier = (lambda: dist.barrier()) if world > 1 else None
    from openfold3_triangle_kernel_b200 import _cabi as C
    C.load()
    wl = Workload(dev)

    for _ in range(max(args.warmup, 3)):
        wl.step()
    torch.cuda.synchronize()
    if C.device_status() != 0:
        raise RuntimeError("device status word is non-zero after warm-up (a bounded wait timed out)")

    sampler = ClockSampler(local_rank) if rank == 0 else None
    launches0 = C.load().tpf_launch_count()
    sec = _time_loop(wl.step, args.steps, barrier)
    launches = C.load().tpf_launch_count() - launches0
    clocks = sampler.stop() if sampler else None

    # per-stage times (same buffers, CUDA events on the launching stream)
    stage = {}
    n_st = max(3, min(args.steps, 10))
    for name, fn in (("attn_fwd", wl.attn_fwd), ("attn_bwd_delta", lambda: wl.attn_bwd(1)),
                     ("attn_bwd_dqkv", lambda: wl.attn_bwd(2)), ("attn_bwd_dbias", lambda: wl.attn_bwd(4)),
                     ("trimul_out_fwd", lambda: wl.trimul_fwd(0)), ("trimul_out_bwd", lambda: wl.trimul_bwd(0)),
                     ("trimul_in_fwd", lambda: wl.trimul_fwd(1)), ("trimul_in_bwd", lambda: wl.trimul_bwd(1))):
        fn()
        stage[name] = _time_loop(fn, n_st) / n_st * 1e6  # us
    # end to end through the public operators with host buffers
    for _ in range(2):
        wl.e2e_step()
    if barrier:
        barrier()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    n_e2e = max(2, min(args.steps, 10))
    for _ in range(n_e2e):
        wl.e2e_step()
    e1.record()
    torch.cuda.synchronize()
    e2e_sec = max(e0.elapsed_time(e1) / 1e3, time.perf_counter() - t0) / n_e2e
    status = C.device_status()

    t_step = torch.tensor([sec / args.steps, e2e_sec], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t_step, op=dist.ReduceOp.MAX)
    step_sec, e2e_sec = (float(x) for x in t_step.tolist())

    if rank == 0:
        peaks = _peaks()
        dom_us = stage["attn_bwd_dqkv"]
        dom_flops = 2.5 * ATT_FLOPS_FWD
        achieved = dom_flops / (dom_us * 1e-6) / 1e12
        # the CPU baseline is timed at N = 1 only (the other ranks of a multi-GPU run would sit in a barrier)
        cpu_sec, cores, desc = cpu_sample_seconds() if world == 1 else (None, None, None)
        h2d, d2h = wl.e2e_bytes()
        line = dict(
            metric=METRIC, value=world * STEP_FLOPS / step_sec / 1e12, unit="TFLOP/s", n_gpus=world,
            steps=args.steps, warmup=max(args.warmup, 3), ms_per_step=step_sec * 1e3, higher_is_better=True,
            scaling="weak", vs_baseline=None, dtype="bf16", data="synthetic",
            config=dict(workload=WORKLOAD, per_gpu_batches=1, l2_policy="working set per step (>1 GB) exceeds the 126 MB L2",
                        seeds=dict(attention=2, trimul=3)),
            stage_us={k: round(v, 1) for k, v in stage.items()},
            stage_tflops=dict(
                attention_fwd_bwd=ATT_FLOPS / ((stage["attn_fwd"] + stage["attn_bwd_delta"] + stage["attn_bwd_dqkv"]
                                                + stage["attn_bwd_dbias"]) * 1e-6) / 1e12,
                trimul_outgoing_fwd_bwd=TRI_FLOPS / ((stage["trimul_out_fwd"] + stage["trimul_out_bwd"]) * 1e-6) / 1e12,
                trimul_incoming_fwd_bwd=TRI_FLOPS / ((stage["trimul_in_fwd"] + stage["trimul_in_bwd"]) * 1e-6) / 1e12),
            roofline=dict(bound="tensor", kernel="attn_bwd_kernel (dq/dk/dv, A384)", achieved=achieved,
                          peak=peaks["bf16_tflops"], unit="TFLOP/s", frac=achieved / peaks["bf16_tflops"],
                          peak_source=peaks["source"] + " cuBLAS bf16 burst", traffic=DOMINANT_KERNEL_DRAM_BYTES,
                          algorithmic_flops_per_launch=dom_flops, launch_us=dom_us),
            cpu_baseline=(dict(value=STEP_FLOPS / cpu_sec / 1e12, unit="TFLOP/s", cores=cores, kind="port", sample=desc)
                          if cpu_sec else None),
            e2e=dict(value=world * STEP_FLOPS / e2e_sec / 1e12, unit="TFLOP/s", h2d_bytes_per_step=h2d,
                     d2h_bytes_per_step=d2h, ms_per_step=e2e_sec * 1e3),
            gpu_launches=int(launches), device_status=status, clocks=clocks)
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def run_block(args, rank, world, local_rank):
    """Strong-scaling measurement of the whole pair-stack block (TriMul out -> in -> attention start ->
    end, residuals, fwd+bwd) at --block-n, row-sharded over the ranks (axial parallelism)."""
    import torch.distributed as dist
    from openfold3_triangle_kernel_b200 import dap
    from openfold3_triangle_kernel_b200.pair_block import pair_stack_block
    from openfold3_triangle_kernel_b200.synthetic import block_params
    dev = torch.device("cuda", local_rank)
    torch.cuda.set_device(dev)
    dist.init_process_group("nccl", device_id=dev) if world > 1 else dist.init_process_group(
        "nccl", init_method="tcp://127.0.0.1:29533", rank=0, world_size=1, device_id=dev)
    n, c, heads, d = args.block_n, 128, 4, 32
    g = torch.Generator().manual_seed(4)
    nl = n // world
    z = torch.randn(1, nl, n, c, generator=g).bfloat16().to(dev).requires_grad_(True)
    mask = torch.ones(1, nl, n, device=dev)
    d_out = torch.randn(1, nl, n, c, generator=g).bfloat16().to(dev)
    params = {k: {m: t.to(dev).requires_grad_(True) for m, t in v.items()} for k, v in block_params(c, heads, d, 5).items()}

    def step():
        out = pair_stack_block(z, mask, params, heads, group=dist.group.WORLD)
        out.backward(d_out)

    for _ in range(max(args.warmup, 3)):
        step()
    sec = _time_loop(step, args.steps, lambda: dist.barrier())
    t = torch.tensor([sec / args.steps], device=dev, dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    flops = 2 * 3 * (12 * n * n * c * c + 2 * n ** 3 * c) + 2 * 14 * n * heads * n * n * d
    if rank == 0:
        print(json.dumps(dict(metric="pair_stack_block_fwd_bwd_tflops", value=flops / float(t) / 1e12, unit="TFLOP/s",
                              n_gpus=world, steps=args.steps, warmup=max(args.warmup, 3), ms_per_step=float(t) * 1e3,
                              higher_is_better=True, scaling="strong", vs_baseline=None, dtype="bf16", data="synthetic",
                              config=dict(workload=f"pair-stack block N={n}, C_z=128, H=4, D=32, axially sharded over "
                                                   f"{world} ranks (operator FLOPs only; wrapper Linears uncounted)"))),
              flush=True)
    dist.barrier()
    dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="hotpath", choices=["hotpath", "block"],
                    help="hotpath: the N=384 operator benchmark (default); block: sharded pair-stack block")
    ap.add_argument("--block-n", type=int, default=768)
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, rank)
        return
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (B200); there is no CPU fallback for the product path")
    if args.workload == "block":
        run_block(args, rank, world, local_rank)
        return
    run_gpu(args, rank, world, local_rank)


if __name__ == "__main__":
    main()
