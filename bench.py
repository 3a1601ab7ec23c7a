#!/usr/bin/env python
"""Benchmark of the attention forward+backward path on B200.

  python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

One "step" is one forward plus one backward over the dense causal bf16 workload
(B=4, Hq=Hkv=32, Sq=Sk=4096, D=128, N(0,1) inputs from a seed) on every GPU; with N GPUs each
rank owns such a shard of a problem with batch 4*N (batch x head units are independent, so no
collective sits on the data path: weak scaling).  FLOPs follow the reference's convention
(modules/flash/tests/performance_forward.py:108-113): fwd = 4*B*H*S*S*D*0.5 (causal),
bwd = 2.5*fwd.  Rank 0 prints ONE JSON line.

`--impl reference` times the reference's own CPU implementation of the path -- its test oracle,
torch's fp32 math SDPA with autograd (modules/flash/tests/_common_test.py:61-79,436-454) -- on the
host cores, on a bounded sample of the same workload.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

WORK = dict(B=4, H=32, S=4096, D=128)
METRIC = "attn fwd+bwd TFLOPS/GPU (bf16, hd128) and % of B200 tensor peak, 1/2/4/8 GPUs"


def flops_fwd(B, H, S, D):
    return 4.0 * B * H * S * S * D * 0.5


def measured_peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return dict(bf16=d["bf16_tflops"], bf16_sustained=d.get("bf16_tflops_sustained"), hbm=d["hbm_gbs"],
                    src="measured")
    return dict(bf16=1590.0, bf16_sustained=1400.0, hbm=6650.0, src="fallback")


class ClockSampler:
    """Samples SM clock and throttle reasons with nvidia-smi while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.rows = []
        self.proc = None
        self.index = index

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "50",
                 "-i", str(self.index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            parts = [x.strip() for x in line.split(",")]
            if len(parts) >= 6:
                self.rows.append(parts)

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        mhz, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            try:
                mhz.append(float(r[0])); mx.append(float(r[1]))
            except ValueError:
                continue
            for n, v in zip(names, r[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": statistics.median(mhz) if mhz else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(mhz)}


def cpu_baseline(sample_heads: int, S: int, D: int, seed: int = 0):
    """fp32 math SDPA forward + autograd backward of `sample_heads` (batch, head) units on the host."""
    import torch
    from oracle import attention as A
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    g = torch.Generator().manual_seed(seed)
    mask = A.window_mask(S, S, 3, A.TOP_LEFT, A.TOP_LEFT)
    t = 0.0
    for _ in range(sample_heads):
        q, k, v, do = (torch.randn(1, 1, S, D, generator=g).bfloat16().float() for _ in range(4))
        t0 = time.perf_counter()
        A.sdpa_math_reference(q, k, v, sm_scale=D ** -0.5, mask=mask, dout=do)
        t += time.perf_counter() - t0
    fl = 3.5 * flops_fwd(1, sample_heads, S, D)
    return dict(value=fl / t / 1e12, unit="TFLOPS", cores=cores, kind="reference",
                sample=f"{sample_heads} of {WORK['B'] * WORK['H']} (batch, head) units of the workload, "
                       f"S={S} D={D} causal, fp32 math SDPA fwd + autograd bwd, {t:.2f} s"), t


def run_reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    S, D = WORK["S"], WORK["D"]
    heads = 2
    for _ in range(max(args.warmup, 0)):
        cpu_baseline(1, S, D)
    times, base = [], None
    for _ in range(args.steps):
        base, t = cpu_baseline(heads, S, D)
        times.append(t)
    fl = 3.5 * flops_fwd(1, heads, S, D)
    value = fl * len(times) / sum(times) / 1e12
    base["value"] = value
    line = dict(metric=METRIC, value=value, unit="TFLOPS", n_gpus=args.gpus, steps=args.steps, warmup=args.warmup,
                ms_per_step=1e3 * sum(times) / len(times), higher_is_better=True, scaling="weak", vs_baseline=None,
                dtype="f32", data="synthetic", impl="reference",
                config=dict(workload="dense causal bf16 B=4 H=32 S=4096 D=128 fwd+bwd (bounded sample per step)",
                            sample_units_per_step=heads, l2="inputs larger than L2 do not apply on the host"),
                cpu_baseline=base,
                e2e=dict(value=value, unit="TFLOPS", h2d_bytes_per_step=0, d2h_bytes_per_step=0), gpu_launches=0)
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--batch", type=int, default=WORK["B"],
                    help="per-GPU batch; smaller values give a short run for profiler captures")
    args = ap.parse_args()
    if args.impl == "reference":
        return run_reference_arm(args)

    import torch
    import torch.distributed as dist

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the library has no CPU path")
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))

    from aotriton_b200 import cabi, flash
    from aotriton_b200.flash import hipError_t

    B, H, S, D = args.batch, WORK["H"], WORK["S"], WORK["D"]
    warm = max(args.warmup, 3)
    dev = torch.device("cuda", local)
    g = torch.Generator().manual_seed(1234 + rank)
    host = [torch.randn(B, H, S, D, generator=g, dtype=torch.float32).to(torch.bfloat16).pin_memory()
            for _ in range(4)]
    q, k, v, do = (t.to(dev) for t in host)
    o = torch.empty_like(q); dq = torch.empty_like(q); dk = torch.empty_like(k); dv = torch.empty_like(v)
    lse = torch.empty(B * H, S, dtype=torch.float32, device=dev)
    delta = torch.empty_like(lse)
    host_out = [torch.empty(B, H, S, D, dtype=torch.bfloat16).pin_memory() for _ in range(4)]
    null64 = torch.empty(0, dtype=torch.uint64, device=dev)
    atomic = torch.zeros(1, dtype=torch.int32, device=dev)
    sm = D ** -0.5

    def fwd():
        e = flash.attn_fwd(q, k, v, None, sm, lse, o, 0.0, null64, null64, 0, null64, null64, None, True, atomic)
        assert e == hipError_t.hipSuccess, e

    def bwd():
        e = flash.attn_bwd(q, k, v, None, sm, o, do, dq, dk, dv, None, None, lse, flash.eager_delta(delta), 0.0,
                           null64, null64, 0, True)
        assert e == hipError_t.hipSuccess, e

    def step():
        fwd(); bwd()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, iters):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        a.record()
        for _ in range(iters):
            fn()
        b.record()
        barrier()
        ms = a.elapsed_time(b)
        if world > 1:
            t = torch.tensor([ms], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms

    for _ in range(warm):
        step()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    launches0 = cabi.lib().ab200_launch_count()
    ms_total = timed(step, args.steps)
    launches = cabi.lib().ab200_launch_count() - launches0
    clocks = sampler.stop() if rank == 0 else None
    status = cabi.lib().ab200_kernel_status(0)

    # per-kernel device times (same inputs, each kernel alone)
    def stage(name):
        return lambda: cabi.attn_bwd(q, k, v, o, do, dq, dk, dv, lse, delta, sm_scale=sm, causal_type=3,
                                     window_left=cabi.WINDOW_TOP_LEFT, window_right=cabi.WINDOW_TOP_LEFT, stage=name)

    iters = max(3, min(args.steps, 20))
    kern_ms = {"attn_fwd": timed(fwd, iters) / iters, "bwd_preprocess": timed(stage("preprocess"), iters) / iters,
               "bwd_dkdv": timed(stage("dkdv"), iters) / iters, "bwd_dq": timed(stage("dq"), iters) / iters}

    # End to end through the public API with host buffers: every step copies its four inputs from
    # pinned host memory and its four results back, inside the timed region.  Like an input pipeline
    # would, consecutive steps overlap: two sets of device buffers, copies in, compute and copies out
    # on three streams, ordered by events (PCIe is full duplex, so step i+1's inputs travel while step
    # i computes and step i-1's results go back).
    class BufSet:
        def __init__(self):
            self.q, self.k, self.v, self.do = (torch.empty_like(q) for _ in range(4))
            self.o, self.dq, self.dk, self.dv = (torch.empty_like(q) for _ in range(4))
            self.lse = torch.empty_like(lse)
            self.delta = torch.empty_like(lse)
            self.in_done, self.cmp_done, self.out_done = (torch.cuda.Event() for _ in range(3))

    sets = [BufSet(), BufSet()]
    s_in, s_cmp, s_out = (torch.cuda.Stream(device=dev) for _ in range(3))

    def e2e_steps(n):
        main = torch.cuda.current_stream()
        for st in (s_in, s_cmp, s_out):
            st.wait_stream(main)
        for i in range(n):
            b = sets[i & 1]
            with torch.cuda.stream(s_in):
                s_in.wait_event(b.cmp_done)          # the step two back has read these inputs
                for d_, h_ in zip((b.q, b.k, b.v, b.do), host):
                    d_.copy_(h_, non_blocking=True)
                b.in_done.record(s_in)
            with torch.cuda.stream(s_cmp):
                s_cmp.wait_event(b.in_done)
                s_cmp.wait_event(b.out_done)         # the step two back has copied its results out
                e = flash.attn_fwd(b.q, b.k, b.v, None, sm, b.lse, b.o, 0.0, null64, null64, 0, null64, null64, None,
                                   True, atomic)
                assert e == hipError_t.hipSuccess, e
                e = flash.attn_bwd(b.q, b.k, b.v, None, sm, b.o, b.do, b.dq, b.dk, b.dv, None, None, b.lse,
                                   flash.eager_delta(b.delta), 0.0, null64, null64, 0, True)
                assert e == hipError_t.hipSuccess, e
                b.cmp_done.record(s_cmp)
            with torch.cuda.stream(s_out):
                s_out.wait_event(b.cmp_done)
                for h_, d_ in zip(host_out, (b.o, b.dq, b.dk, b.dv)):
                    h_.copy_(d_, non_blocking=True)
                b.out_done.record(s_out)
        for st in (s_in, s_cmp, s_out):
            main.wait_stream(st)

    e2e_steps(2)
    e2e_iters = max(4, min(args.steps, 20))
    ms_e2e = timed(lambda: e2e_steps(e2e_iters), 1) / e2e_iters

    ffwd = flops_fwd(B, H, S, D)
    fbwd = 2.5 * ffwd
    ms_step = ms_total / args.steps
    peaks = measured_peaks()
    tfl = lambda f, ms: f / (ms * 1e-3) / 1e12
    value = world * tfl(ffwd + fbwd, ms_step)
    dom = max(("attn_fwd", "bwd_dkdv", "bwd_dq"), key=lambda n: kern_ms[n])
    # dram__bytes_read.sum + dram__bytes_write.sum per launch from the ncu capture at batch 2
    # (profiles/tcgen05_kernels_dense_causal_bf16_B2_H32_S4096_D128.md); traffic grows in
    # proportion to the batch (per-(batch, head) work is independent), so it is scaled by B / 2.
    traffic_b2 = {"attn_fwd": 201.6e6 + 54.0e6, "bwd_dkdv": 275.0e6 + 117.5e6, "bwd_dq": 270.6e6 + 55.7e6}
    dom_traffic = traffic_b2[dom] * B / 2.0 if (H, S, D) == (32, 4096, 128) else None
    dom_flops = {"attn_fwd": ffwd, "bwd_dkdv": 2.0 * ffwd, "bwd_dq": 1.5 * ffwd}[dom]
    nbytes = q.numel() * 2
    line = dict(
        metric=METRIC, value=value, unit="TFLOPS", n_gpus=world, steps=args.steps, warmup=warm,
        ms_per_step=ms_step, higher_is_better=True, scaling="weak", vs_baseline=None, dtype="bf16",
        data="synthetic",
        config=dict(workload=f"dense causal bf16 B={B}xN H={H} S={S} D={D} fwd+bwd", per_gpu_batch=B,
                    global_batch=B * world, parallelism=f"batch x head shards, {world} GPU(s), no collective",
                    l2="inputs (1 GiB of tensors per step) are larger than the 126 MB L2; no explicit flush"),
        per_gpu=dict(fwd_tflops=tfl(ffwd, kern_ms["attn_fwd"]),
                     bwd_tflops=tfl(fbwd, kern_ms["bwd_preprocess"] + kern_ms["bwd_dkdv"] + kern_ms["bwd_dq"]),
                     fwd_frac_of_peak=tfl(ffwd, kern_ms["attn_fwd"]) / peaks["bf16"],
                     bwd_frac_of_peak=tfl(fbwd, kern_ms["bwd_preprocess"] + kern_ms["bwd_dkdv"] + kern_ms["bwd_dq"])
                     / peaks["bf16"], kernel_ms=kern_ms,
                     # the timed loop runs for hundreds of milliseconds under the power cap: the
                     # cuBLAS figure measured the same way (seconds-long loop) is the fair yardstick
                     step_tflops=tfl(ffwd + fbwd, ms_step), bf16_peak_sustained=peaks["bf16_sustained"],
                     step_frac_of_sustained_peak=(tfl(ffwd + fbwd, ms_step) / peaks["bf16_sustained"]
                                                  if peaks["bf16_sustained"] else None),
                     fwd_family=cabi.lib().ab200_last_fwd_family(), bwd_family=cabi.lib().ab200_last_bwd_family(),
                     preprocess_gbs=(2 * nbytes + lse.numel() * 4) / (kern_ms["bwd_preprocess"] * 1e-3) / 1e9),
        roofline=dict(bound="tensor", kernel=dom, achieved=tfl(dom_flops, kern_ms[dom]), peak=peaks["bf16"],
                      unit="TFLOP/s", frac=tfl(dom_flops, kern_ms[dom]) / peaks["bf16"], traffic=dom_traffic,
                      traffic_unit="bytes per launch (ncu at batch 2, scaled by batch)",
                      peak_source=f"of {peaks['src']} (cuBLAS bf16 burst)",
                      flops_note="algorithmic: fwd 4BHS^2D/2; dK/dV 4 of the 5 counted backward GEMMs = 2x fwd; "
                                 "dQ 3 GEMMs = 1.5x fwd (two of them recomputed, counted here because this "
                                 "kernel executes them)"),
        e2e=dict(value=world * tfl(ffwd + fbwd, ms_e2e), unit="TFLOPS", ms_per_step=ms_e2e,
                 h2d_bytes_per_step=4 * nbytes, d2h_bytes_per_step=4 * nbytes,
                 how="pinned host buffers; copies in, compute and copies out of consecutive steps overlap "
                     "(two device buffer sets, three streams)"),
        gpu_launches=int(launches), kernel_status=int(status), clocks=clocks)
    if rank == 0:
        if not args.no_cpu_baseline:
            line["cpu_baseline"], _ = cpu_baseline(8, S, D)
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
