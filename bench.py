#!/usr/bin/env python
"""Benchmark of the attention forward+backward path on B200.

  python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--config c2|c3|c4|c5a|c5b]

Headline (always): one "step" is one forward plus one backward over the dense causal bf16 workload
C2 (B=4, Hq=Hkv=32, Sq=Sk=4096, D=128, N(0,1) inputs from a seed) on every GPU; with N GPUs each
rank owns such a shard of a problem with batch 4*N (batch x head units are independent, so no
collective sits on the data path: weak scaling).  FLOPs follow the reference's convention
(modules/flash/tests/performance_forward.py:108-113): fwd = 4*D*Hq*(unmasked pairs), causal counted
as half, bwd = 2.5*fwd.  Rank 0 prints ONE JSON line.

Beside the headline the line carries
  kernels   per-kernel device times of C2 measured the way the reference's tuner does
            (python/tune/gpu_utils.py:293-370): 1 GiB written before every timed call to flush L2,
            >= 20 repetitions, median and minimum;
  configs   (1 GPU) the same for the other benchmark configurations: C3 GQA + sliding window,
            C4 compact varlen with dropout, C5a/C5b bias + dropout at D=256 / D=72;
  sharded   (N > 1) ONE C3 problem split over the ranks by kv head (strong scaling), verified
            bit for bit against the unsharded run through an NCCL all-gather outside the timed region;
  e2e       C2 through the Python operator API with pinned host buffers copied in and out every step.

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

METRIC = "attn fwd+bwd TFLOPS/GPU (bf16, hd128) and % of B200 tensor peak, 1/2/4/8 GPUs"
TOP_LEFT = -2147483647

# The benchmark configurations (sizes, dtypes and distributions of the build target).
CONFIGS = {
    "c2": dict(desc="dense causal bf16 B=4 H=32 S=4096 D=128", dtype="bf16", B=4, Hq=32, Hk=32, S=4096, D=128,
               causal=(3, TOP_LEFT, TOP_LEFT)),
    "c3": dict(desc="GQA 64:8 sliding window (4096,0) bf16 B=1 S=16384 D=128", dtype="bf16", B=1, Hq=64, Hk=8,
               S=16384, D=128, causal=(3, 4096, 0)),
    "c4": dict(desc="compact varlen fp16, 16 seqs L~U[64,8192] (seed 42), Hq=32 Hk=8 D=128, causal, dropout 0.1",
               dtype="fp16", Hq=32, Hk=8, D=128, causal=(3, TOP_LEFT, TOP_LEFT), varlen_seed=42, nseq=16, p=0.1,
               philox_seed=42, philox_offset=0),
    "c5a": dict(desc="bias + dropout 0.2 fp16 B=8 H=16 S=2048 D=256, dBias", dtype="fp16", B=8, Hq=16, Hk=16, S=2048,
                D=256, causal=(0, 0, 0), p=0.2, bias=True),
    "c5b": dict(desc="bias + dropout 0.2 fp16 B=8 H=16 S=2048 D=72 (padded head dim), dBias", dtype="fp16", B=8,
                Hq=16, Hk=16, S=2048, D=72, causal=(0, 0, 0), p=0.2, bias=True),
}

# Profiling aids, reachable through --only-config only (they isolate one cost of the configurations
# above; no bench line is made from them).
PROFILE_CONFIGS = {
    "dropout_d128": dict(desc="dropout 0.1 bf16 B=4 H=16 S=2048 D=128", dtype="bf16", B=4, Hq=16, Hk=16, S=2048, D=128,
                         causal=(0, 0, 0), p=0.1),
    "plain_d256": dict(desc="dense fp16 B=8 H=16 S=2048 D=256", dtype="fp16", B=8, Hq=16, Hk=16, S=2048, D=256,
                       causal=(0, 0, 0)),
}

# dram__bytes_read.sum + dram__bytes_write.sum per launch (bytes) of the C2 kernels, from the ncu
# capture at batch 2 summarised in profiles/tcgen05_kernels_dense_causal_bf16_B2_H32_S4096_D128.md;
# per-(batch, head) work is independent, so a launch at batch B moves B/2 times as much.
C2_DRAM_TRAFFIC_B2 = {"attn_fwd": (296.3e6, 49.0e6), "bwd_dkdv": (275.0e6, 117.4e6), "bwd_dq": (270.7e6, 54.8e6)}


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


# ------------------------------------------------------------------------------------------------
# CPU arm: the reference's test oracle on the host cores.
def cpu_sample(units: int, S: int = 4096, D: int = 128, seed: int = 0):
    """fp32 math SDPA forward + autograd backward of `units` (batch, head) units of C2 on the host.
    One unit is run and discarded first (thread pool start-up, allocator warm-up), so that a single
    call and a loop of calls measure the same thing.  Returns (TFLOPS, seconds)."""
    import torch
    from oracle import attention as A
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    g = torch.Generator().manual_seed(seed)
    mask = A.window_mask(S, S, 3, A.TOP_LEFT, A.TOP_LEFT)
    t = 0.0
    for i in range(units + 1):
        q, k, v, do = (torch.randn(1, 1, S, D, generator=g).bfloat16().float() for _ in range(4))
        t0 = time.perf_counter()
        A.sdpa_math_reference(q, k, v, sm_scale=D ** -0.5, mask=mask, dout=do)
        if i > 0:
            t += time.perf_counter() - t0
    fl = 3.5 * 4.0 * units * S * S * D * 0.5
    return fl / t / 1e12, t


def cpu_baseline_record(units: int, value: float, seconds: float):
    c = CONFIGS["c2"]
    return dict(value=value, unit="TFLOPS", cores=os.cpu_count() or 1, kind="reference",
                sample=f"{units} of {c['B'] * c['Hq']} (batch, head) units of the workload (after one discarded "
                       f"warm-up unit), S={c['S']} D={c['D']} causal, fp32 math SDPA fwd + autograd bwd, "
                       f"{seconds:.2f} s")


def run_reference_arm(args):
    if int(os.environ.get("RANK", "0")) != 0:
        return
    units = 2
    for _ in range(max(args.warmup, 0)):
        cpu_sample(1)
    secs = []
    for _ in range(args.steps):
        _, t = cpu_sample(units)
        secs.append(t)
    c = CONFIGS["c2"]
    fl = 3.5 * 4.0 * units * c["S"] * c["S"] * c["D"] * 0.5
    value = fl * len(secs) / sum(secs) / 1e12
    line = dict(metric=METRIC, value=value, unit="TFLOPS", n_gpus=args.gpus, steps=args.steps, warmup=args.warmup,
                ms_per_step=1e3 * sum(secs) / len(secs), higher_is_better=True, scaling="weak", vs_baseline=None,
                dtype="f32", data="synthetic", impl="reference",
                config=dict(workload=c["desc"] + " fwd+bwd (bounded sample per step)", sample_units_per_step=units,
                            l2="inputs larger than L2 do not apply on the host"),
                cpu_baseline=cpu_baseline_record(units, value, sum(secs) / len(secs)),
                e2e=dict(value=value, unit="TFLOPS", h2d_bytes_per_step=0, d2h_bytes_per_step=0), gpu_launches=0)
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------------------
class Problem:
    """Device tensors of one configuration and closures that launch its kernels through the C-ABI."""

    def __init__(self, name: str, dev, seed: int = 1234, batch: int | None = None):
        import numpy as np
        import torch
        from aotriton_b200 import cabi
        c = dict(CONFIGS[name] if name in CONFIGS else PROFILE_CONFIGS[name])
        if batch is not None:
            c["B"] = batch
        self.name, self.c, self.cabi = name, c, cabi
        dt = torch.bfloat16 if c["dtype"] == "bf16" else torch.float16
        self.dt = dt
        D, Hq, Hk = c["D"], c["Hq"], c["Hk"]
        g = torch.Generator(device=dev).manual_seed(seed)
        rnd = lambda *shape: torch.randn(*shape, generator=g, device=dev, dtype=torch.float32).to(dt)
        ct, wl, wr = c["causal"]
        self.prob = dict(sm_scale=D ** -0.5, causal_type=ct, window_left=wl, window_right=wr)
        if "nseq" in c:                       # compact varlen, THD storage
            lens = np.random.default_rng(c["varlen_seed"]).integers(64, 8193, c["nseq"])
            cu = np.concatenate([[0], np.cumsum(lens)]).astype(np.int32)
            T, smax = int(cu[-1]), int(lens.max())
            mk = lambda H: rnd(1, T, H, D).transpose(1, 2)
            self.q, self.k, self.v, self.do = mk(Hq), mk(Hk), mk(Hk), mk(Hq)
            self.cu = torch.from_numpy(cu).to(dev)
            self.prob.update(cu_seqlens_q=self.cu, cu_seqlens_k=self.cu, max_seqlen_q=smax, max_seqlen_k=smax)
            self.lse_shape = (Hq, T)
            self.pairs = float(sum(0.5 * float(L) * float(L) for L in lens))
            self.tokens_q = T
            c["lens_sum"], c["lens_max"] = T, smax
        else:
            B, S = c["B"], c["S"]
            self.q, self.do = rnd(B, Hq, S, D), rnd(B, Hq, S, D)
            self.k, self.v = rnd(B, Hk, S, D), rnd(B, Hk, S, D)
            self.lse_shape = (B * Hq, S)
            if ct == 0:
                pairs = float(S) * S
            elif wl == TOP_LEFT:
                pairs = 0.5 * S * S
            else:                              # sliding window (W, 0): W(W+1)/2 + (S-W)(W+1) kept pairs per row set
                W = wl
                pairs = W * (W + 1) / 2.0 + (S - W) * (W + 1.0)
            self.pairs = B * pairs
            self.tokens_q = B * S
        self.bias = self.dbias = None
        if c.get("bias"):
            self.bias = rnd(c["B"], Hq, c["S"], c["S"])
            self.dbias = torch.empty_like(self.bias)
        self.p = float(c.get("p", 0.0))
        if self.p > 0:
            self.seed_t = torch.tensor([c.get("philox_seed", 0x1BF52)], dtype=torch.uint64, device=dev)
            self.off_t = torch.tensor([c.get("philox_offset", 0x1D4000)], dtype=torch.uint64, device=dev)
            self.prob.update(dropout_p=self.p, philox_seed=self.seed_t, philox_offset1=self.off_t)
        self.out = torch.empty_like(self.q)
        self.dq, self.dk, self.dv = torch.empty_like(self.q), torch.empty_like(self.k), torch.empty_like(self.v)
        self.lse = torch.empty(self.lse_shape, dtype=torch.float32, device=dev)
        self.delta = torch.empty_like(self.lse)
        self.flops_fwd = 4.0 * D * Hq * self.pairs
        el = 2
        self.bytes_fwd = (2 * self.q.numel() + self.k.numel() + self.v.numel()) * el + self.lse.numel() * 4 + \
                         (self.bias.numel() * el if self.bias is not None else 0)
        # backward: reads Q, K, V, dO, O (preprocess), LSE, delta; writes delta, dQ, dK, dV; bias read by both
        # kernels and dBias written once
        self.bytes_bwd = (4 * self.q.numel() + 2 * self.k.numel() + 2 * self.v.numel()) * el + \
                         4 * self.lse.numel() * 4 + (3 * self.bias.numel() * el if self.bias is not None else 0)

    def fwd(self):
        e = self.cabi.attn_fwd(self.q, self.k, self.v, self.out, self.lse, bias=self.bias, **self.prob)
        assert e == 0, f"ab200_attn_fwd returned {e}"

    def bwd(self, stage="all"):
        e = self.cabi.attn_bwd(self.q, self.k, self.v, self.out, self.do, self.dq, self.dk, self.dv, self.lse,
                               self.delta, bias=self.bias, dbias=self.dbias, stage=stage, **self.prob)
        assert e == 0, f"ab200_attn_bwd ({stage}) returned {e}"


class Timer:
    """CUDA-event timing on the current stream.  flushed(): the reference tuner's recipe, one timed call
    per repetition with 1 GiB written beforehand so that nothing of the previous call is left in L2."""

    def __init__(self, dev):
        import torch
        self.torch = torch
        self.flush = torch.empty(1 << 28, dtype=torch.int32, device=dev)      # 1 GiB

    def flushed(self, fn, reps=20, warm=3):
        torch = self.torch
        for _ in range(warm):
            fn()
        ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(reps)]
        for a, b in ev:
            self.flush.zero_()
            a.record()
            fn()
            b.record()
        torch.cuda.synchronize()
        ms = sorted(a.elapsed_time(b) for a, b in ev)
        return dict(median_ms=statistics.median(ms), min_ms=ms[0], reps=reps)


def bind_to_gpu_numa_node(local):
    """Best effort: run this process (and so first-touch its pinned host buffers) on the CPUs of the NUMA
    node the GPU hangs off, so that the host <-> device copies of different ranks do not all cross one
    socket's memory.  Returns what it did, for the e2e record; the caller restores the affinity once the
    buffers exist."""
    import torch
    try:
        pr = torch.cuda.get_device_properties(local)
        bdf = f"{pr.pci_domain_id:04x}:{pr.pci_bus_id:02x}:{pr.pci_device_id:02x}.0"
        base = Path("/sys/bus/pci/devices") / bdf
        node = int((base / "numa_node").read_text().strip())
        cpus = (base / "local_cpulist").read_text().strip()
        want = set()
        for part in cpus.split(","):
            lo, _, hi = part.partition("-")
            want.update(range(int(lo), int(hi or lo) + 1))
        allowed = os.sched_getaffinity(0)
        use = want & allowed
        if node < 0 or not use:
            return dict(numa_node=node, bound=False, why="no local CPUs among the allowed ones")
        os.sched_setaffinity(0, use)
        return dict(numa_node=node, bound=True, cpus=len(use), restore=allowed)
    except Exception as e:       # sysfs absent, attributes missing, not permitted ...
        return dict(bound=False, why=f"{type(e).__name__}: {e}"[:120])


def tfl(flops, ms):
    return flops / (ms * 1e-3) / 1e12


def config_block(name, dev, timer, peaks, lib):
    """Per-configuration record: flushed median/min of forward, backward and its stages, TFLOPS by the
    reference's FLOP convention, fraction of the measured tensor peak, GB/s of algorithmic bytes."""
    import torch
    pr = Problem(name, dev)
    pr.fwd(); pr.bwd()
    torch.cuda.synchronize()
    rec = dict(workload=pr.c["desc"], fwd_family=lib.ab200_last_fwd_family(), bwd_family=lib.ab200_last_bwd_family(),
               flops_fwd=pr.flops_fwd, flops_bwd=2.5 * pr.flops_fwd)
    f = timer.flushed(pr.fwd)
    b = timer.flushed(pr.bwd)
    stages = {s: timer.flushed(lambda s=s: pr.bwd(s)) for s in ("preprocess", "dkdv", "dq")}
    # backward time = sum of its three kernels' medians; the median of whole calls (which also shows
    # the host's launch work when every call starts on an idle GPU) is kept beside it
    bk = sum(v["median_ms"] for v in stages.values())
    rec.update(fwd_ms=f["median_ms"], fwd_min_ms=f["min_ms"], bwd_ms=bk, bwd_call_ms=b["median_ms"],
               bwd_call_min_ms=b["min_ms"], bwd_stage_ms={k: v["median_ms"] for k, v in stages.items()}, reps=f["reps"],
               fwd_tflops=tfl(pr.flops_fwd, f["median_ms"]), bwd_tflops=tfl(2.5 * pr.flops_fwd, bk),
               fwd_frac_of_peak=tfl(pr.flops_fwd, f["median_ms"]) / peaks["bf16"],
               bwd_frac_of_peak=tfl(2.5 * pr.flops_fwd, bk) / peaks["bf16"],
               fwd_gbs=pr.bytes_fwd / (f["median_ms"] * 1e-3) / 1e9, bwd_gbs=pr.bytes_bwd / (bk * 1e-3) / 1e9,
               fwd_frac_of_hbm=pr.bytes_fwd / (f["median_ms"] * 1e-3) / 1e9 / peaks["hbm"],
               bwd_frac_of_hbm=pr.bytes_bwd / (bk * 1e-3) / 1e9 / peaks["hbm"],
               kernel_status=int(lib.ab200_kernel_status(0)))
    if "lens_sum" in pr.c:
        rec.update(tokens=pr.c["lens_sum"], max_seqlen=pr.c["lens_max"])
    del pr
    torch.cuda.empty_cache()
    return rec


def sharded_c3(dev, rank, world, dist, lib, reps=10):
    """ONE C3 problem split over the ranks by kv head (aotriton_b200/sharding.py): every rank builds
    the same full inputs from the seed, runs the operator on views of its heads, and the shards are
    all-gathered (outside the timed region) and compared bit for bit with rank 0's unsharded run."""
    import torch
    from aotriton_b200 import cabi, sharding
    pr = Problem("c3", dev, seed=99)
    c = pr.c
    G = c["Hq"] // c["Hk"]
    segs = sharding.partition_dense(c["B"], c["Hk"], world, rank)
    assert len(segs) == 1, "C3 has one batch element: one segment per rank"
    seg = segs[0]
    hs, ks = slice(seg.hk_lo * G, seg.hk_hi * G), slice(seg.hk_lo, seg.hk_hi)
    nh = (seg.hk_hi - seg.hk_lo) * G
    sh = dict(q=pr.q[:, hs], k=pr.k[:, ks], v=pr.v[:, ks], do=pr.do[:, hs])
    out, dq = torch.empty_like(sh["q"]), torch.empty_like(sh["q"])
    dk, dv = torch.empty_like(sh["k"]), torch.empty_like(sh["v"])
    lse = torch.empty(nh, c["S"], dtype=torch.float32, device=dev)
    delta = torch.empty_like(lse)

    def step():
        e = cabi.attn_fwd(sh["q"], sh["k"], sh["v"], out, lse, **pr.prob)
        assert e == 0, e
        e = cabi.attn_bwd(sh["q"], sh["k"], sh["v"], out, sh["do"], dq, dk, dv, lse, delta, **pr.prob)
        assert e == 0, e

    for _ in range(3):
        step()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    dist.barrier(); torch.cuda.synchronize()
    a.record()
    for _ in range(reps):
        step()
    b.record()
    dist.barrier(); torch.cuda.synchronize()
    t = torch.tensor([a.elapsed_time(b) / reps], device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = float(t.item())
    # verification, outside the timed region
    verified = None
    gathered = {}
    for n, x in (("out", out), ("dq", dq), ("dk", dk), ("dv", dv), ("lse", lse)):
        buf = torch.empty((world,) + tuple(x.shape), dtype=x.dtype, device=dev)
        dist.all_gather_into_tensor(buf, x.contiguous())
        gathered[n] = buf
    if rank == 0:
        pr.fwd(); pr.bwd()
        torch.cuda.synchronize()
        S, D = c["S"], c["D"]
        verified = bool(
            torch.equal(gathered["out"].reshape(1, c["Hq"], S, D), pr.out)
            and torch.equal(gathered["dq"].reshape(1, c["Hq"], S, D), pr.dq)
            and torch.equal(gathered["dk"].reshape(1, c["Hk"], S, D), pr.dk)
            and torch.equal(gathered["dv"].reshape(1, c["Hk"], S, D), pr.dv)
            and torch.equal(gathered["lse"].reshape(c["Hq"], S), pr.lse))
    fl = 3.5 * pr.flops_fwd
    return dict(workload=c["desc"] + f", kv heads {c['Hk']} split over {world} ranks", scaling="strong",
                ms_per_step=ms, tflops_aggregate=tfl(fl, ms), kv_heads_per_rank=seg.hk_hi - seg.hk_lo,
                verified_bitwise_vs_unsharded=verified, collective="all_gather of O/LSE/dQ/dK/dV, verification only",
                kernel_status=int(lib.ab200_kernel_status(0)))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--config", default="all", choices=["all", "none"] + sorted(CONFIGS),
                    help="which configurations the `configs` block measures beside the C2 headline (1 GPU)")
    ap.add_argument("--only-config", default=None, choices=sorted(CONFIGS) + sorted(PROFILE_CONFIGS),
                    help="run just this configuration's forward and backward three times and print their times "
                         "(a short, exactly known launch sequence for profiler captures); no headline")
    ap.add_argument("--config-batch", type=int, default=None,
                    help="batch size override for --only-config (dense configurations)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-buffer leg (profiler captures)")
    ap.add_argument("--batch", type=int, default=CONFIGS["c2"]["B"],
                    help="per-GPU batch of the headline workload; smaller values give a short run for profiler captures")
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
    lib = cabi.lib()

    if args.only_config:
        pr = Problem(args.only_config, torch.device("cuda", local), batch=args.config_batch)
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
        for _ in range(3):
            ev[0].record(); pr.fwd(); ev[1].record(); pr.bwd(); ev[2].record()
        torch.cuda.synchronize()
        print(json.dumps(dict(only_config=args.only_config, workload=pr.c["desc"], batch=pr.c.get("B"),
                              fwd_ms=ev[0].elapsed_time(ev[1]), bwd_ms=ev[1].elapsed_time(ev[2]),
                              fwd_family=lib.ab200_last_fwd_family(), bwd_family=lib.ab200_last_bwd_family(),
                              kernel_status=int(lib.ab200_kernel_status(0)))), flush=True)
        return

    c2 = CONFIGS["c2"]
    B, H, S, D = args.batch, c2["Hq"], c2["S"], c2["D"]
    warm = max(args.warmup, 3)
    dev = torch.device("cuda", local)
    numa = bind_to_gpu_numa_node(local)
    g = torch.Generator().manual_seed(1234 + rank)
    host = [torch.randn(B, H, S, D, generator=g, dtype=torch.float32).to(torch.bfloat16).pin_memory()
            for _ in range(4)]
    q, k, v, do = (t.to(dev) for t in host)
    o = torch.empty_like(q); dq = torch.empty_like(q); dk = torch.empty_like(k); dv = torch.empty_like(v)
    lse = torch.empty(B * H, S, dtype=torch.float32, device=dev)
    delta = torch.empty_like(lse)
    host_out = [torch.empty(B, H, S, D, dtype=torch.bfloat16).pin_memory() for _ in range(4)]
    if numa.get("bound"):
        os.sched_setaffinity(0, numa.pop("restore"))
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

    # ---- headline: K looped steps, device-timed, max over ranks ---------------------------------
    for _ in range(warm):
        step()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    launches0 = lib.ab200_launch_count()
    ms_total = timed(step, args.steps)
    launches = lib.ab200_launch_count() - launches0
    clocks = sampler.stop() if rank == 0 else None
    status = lib.ab200_kernel_status(0)

    # ---- per-kernel device times of the same inputs: L2 flushed before every call, median / min --
    timer = Timer(dev)

    def stage(name):
        return lambda: cabi.attn_bwd(q, k, v, o, do, dq, dk, dv, lse, delta, sm_scale=sm, causal_type=3,
                                     window_left=cabi.WINDOW_TOP_LEFT, window_right=cabi.WINDOW_TOP_LEFT, stage=name)

    reps = 20
    kern = {"attn_fwd": timer.flushed(fwd, reps), "bwd_preprocess": timer.flushed(stage("preprocess"), reps),
            "bwd_dkdv": timer.flushed(stage("dkdv"), reps), "bwd_dq": timer.flushed(stage("dq"), reps),
            "bwd_all": timer.flushed(bwd, reps)}
    kern_ms = {n: r["median_ms"] for n, r in kern.items()}
    # the fused backward (dK, dV and atomically accumulated dQ in one kernel + conversion kernel),
    # which the library only uses on request: accumulator zeroing, kernel and conversion
    acc = torch.zeros(B, H, S, D, dtype=torch.float32, device=dev)
    fused = None
    if cabi.attn_bwd(q, k, v, o, do, dq, dk, dv, lse, delta, sm_scale=sm, causal_type=3, window_left=cabi.WINDOW_TOP_LEFT,
                     window_right=cabi.WINDOW_TOP_LEFT, stage="fused", dq_acc=acc) == 0:
        fz = lambda name: (lambda: cabi.attn_bwd(q, k, v, o, do, dq, dk, dv, lse, delta, sm_scale=sm, causal_type=3,
                                                 window_left=cabi.WINDOW_TOP_LEFT, window_right=cabi.WINDOW_TOP_LEFT,
                                                 stage=name, dq_acc=acc))
        fused = dict(zero_ms=timer.flushed(lambda: acc.zero_(), reps)["median_ms"],
                     kernel_ms=timer.flushed(fz("fused"), reps)["median_ms"],
                     convert_ms=timer.flushed(fz("postprocess"), reps)["median_ms"])
        fused["bwd_ms"] = kern_ms["bwd_preprocess"] + sum(fused.values())
    del acc

    # ---- end to end through the public API with host buffers -------------------------------------
    # Every step copies its four inputs from pinned host memory and its four results back, inside the
    # timed region.  Like an input pipeline would, consecutive steps overlap: two sets of device
    # buffers, copies in, compute and copies out on three streams, ordered by events (PCIe is full
    # duplex, so step i+1's inputs travel while step i computes and step i-1's results go back).
    class BufSet:
        def __init__(self):
            self.q, self.k, self.v, self.do = (torch.empty_like(q) for _ in range(4))
            self.o, self.dq, self.dk, self.dv = (torch.empty_like(q) for _ in range(4))
            self.lse = torch.empty_like(lse)
            self.delta = torch.empty_like(lse)
            self.in_done, self.cmp_done, self.out_done = (torch.cuda.Event() for _ in range(3))

    ms_e2e = None
    if not args.no_e2e:
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
                    e = flash.attn_fwd(b.q, b.k, b.v, None, sm, b.lse, b.o, 0.0, null64, null64, 0, null64, null64,
                                       None, True, atomic)
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
        del sets

    c2p = dict(c2); c2p["B"] = B
    ffwd = 4.0 * B * H * S * S * D * 0.5
    fbwd = 2.5 * ffwd
    ms_step = ms_total / args.steps
    peaks = measured_peaks()
    value = world * tfl(ffwd + fbwd, ms_step)
    dom = max(("attn_fwd", "bwd_dkdv", "bwd_dq"), key=lambda n: kern_ms[n])
    rd, wr = C2_DRAM_TRAFFIC_B2[dom]
    dom_traffic = (rd + wr) * B / 2.0 if (H, S, D) == (32, 4096, 128) else None
    dom_flops = {"attn_fwd": ffwd, "bwd_dkdv": 2.0 * ffwd, "bwd_dq": 1.5 * ffwd}[dom]
    nbytes = q.numel() * 2
    bwd_ms = kern_ms["bwd_preprocess"] + kern_ms["bwd_dkdv"] + kern_ms["bwd_dq"]      # sum of kernel medians
    line = dict(
        metric=METRIC, value=value, unit="TFLOPS", n_gpus=world, steps=args.steps, warmup=warm,
        ms_per_step=ms_step, higher_is_better=True, scaling="weak", vs_baseline=None, dtype="bf16",
        data="synthetic",
        config=dict(workload=f"dense causal bf16 B={B}xN H={H} S={S} D={D} fwd+bwd", per_gpu_batch=B,
                    global_batch=B * world, parallelism=f"batch x head shards, {world} GPU(s), no collective",
                    l2="headline loop: inputs (1 GiB of tensors per step) are larger than the 126 MB L2, no explicit "
                       "flush; per-kernel and per-config times: 1 GiB written before every timed call"),
        per_gpu=dict(fwd_tflops=tfl(ffwd, kern_ms["attn_fwd"]), bwd_tflops=tfl(fbwd, bwd_ms),
                     fwd_frac_of_peak=tfl(ffwd, kern_ms["attn_fwd"]) / peaks["bf16"],
                     bwd_frac_of_peak=tfl(fbwd, bwd_ms) / peaks["bf16"],
                     fwd_frac_of_sustained_peak=(tfl(ffwd, kern_ms["attn_fwd"]) / peaks["bf16_sustained"]
                                                 if peaks["bf16_sustained"] else None),
                     bwd_frac_of_sustained_peak=(tfl(fbwd, bwd_ms) / peaks["bf16_sustained"]
                                                 if peaks["bf16_sustained"] else None),
                     kernel_ms=kern_ms, kernel_min_ms={n: r["min_ms"] for n, r in kern.items()},
                     bwd_ms=bwd_ms, bwd_call_ms=kern_ms["bwd_all"],
                     fused_backward=(dict(fused, tflops=tfl(fbwd, fused["bwd_ms"]),
                                          frac_of_peak=tfl(fbwd, fused["bwd_ms"]) / peaks["bf16"],
                                          note="opt-in (kernel family 3 / force_backend_index 2): slower than the "
                                               "two-kernel backward here, its fp32 atomics saturate the L2")
                                     if fused else None),
                     kernel_timing=f"CUDA events, 1 GiB L2 flush before each call, median of {reps} (min beside it)",
                     # the timed loop runs for hundreds of milliseconds under the power cap: the
                     # cuBLAS figure measured the same way (seconds-long loop) is the fair yardstick
                     step_tflops=tfl(ffwd + fbwd, ms_step), bf16_peak_sustained=peaks["bf16_sustained"],
                     step_frac_of_sustained_peak=(tfl(ffwd + fbwd, ms_step) / peaks["bf16_sustained"]
                                                  if peaks["bf16_sustained"] else None),
                     fwd_family=lib.ab200_last_fwd_family(), bwd_family=lib.ab200_last_bwd_family(),
                     preprocess_gbs=(2 * nbytes + 2 * lse.numel() * 4 // 2) / (kern_ms["bwd_preprocess"] * 1e-3) / 1e9,
                     preprocess_frac_of_hbm=(2 * nbytes + lse.numel() * 4) / (kern_ms["bwd_preprocess"] * 1e-3) / 1e9
                     / peaks["hbm"]),
        roofline=dict(bound="tensor", kernel=dom, achieved=tfl(dom_flops, kern_ms[dom]), peak=peaks["bf16"],
                      unit="TFLOP/s", frac=tfl(dom_flops, kern_ms[dom]) / peaks["bf16"], traffic=dom_traffic,
                      traffic_unit="bytes per launch (ncu at batch 2, scaled by batch)",
                      peak_source=f"of {peaks['src']} (cuBLAS bf16 burst)",
                      flops_note="algorithmic: fwd 4BHS^2D/2; dK/dV 4 of the 5 counted backward GEMMs = 2x fwd; "
                                 "dQ 3 GEMMs = 1.5x fwd (two of them recomputed, counted here because this "
                                 "kernel executes them)"),
        gpu_launches=int(launches), kernel_status=int(status), clocks=clocks)
    if ms_e2e is not None:
        line["e2e"] = dict(value=world * tfl(ffwd + fbwd, ms_e2e), unit="TFLOPS", ms_per_step=ms_e2e,
                           h2d_bytes_per_step=4 * nbytes, d2h_bytes_per_step=4 * nbytes,
                           h2d_gbs_per_rank=4 * nbytes / (ms_e2e * 1e-3) / 1e9,
                           d2h_gbs_per_rank=4 * nbytes / (ms_e2e * 1e-3) / 1e9, host_numa=numa,
                           bound="host <-> device copies: 0.5 GiB each way per step per rank over the box's PCIe "
                                 "and host memory, shared by all ranks; the kernels take ms_per_step of the headline",
                           how="pinned host buffers; copies in, compute and copies out of consecutive steps overlap "
                               "(two device buffer sets, three streams)")
    del q, k, v, do, o, dq, dk, dv
    torch.cuda.empty_cache()
    if world > 1:
        line["sharded"] = sharded_c3(dev, rank, world, dist, lib)
    elif args.config != "none":
        names = sorted(CONFIGS) if args.config == "all" else [args.config]
        line["configs"] = {n: config_block(n, dev, timer, peaks, lib) for n in names if n != "c2"}
        line["configs"]["c2"] = dict(workload=c2["desc"], fwd_ms=kern_ms["attn_fwd"], bwd_ms=bwd_ms,
                                     fwd_tflops=tfl(ffwd, kern_ms["attn_fwd"]), bwd_tflops=tfl(fbwd, bwd_ms),
                                     fwd_frac_of_peak=tfl(ffwd, kern_ms["attn_fwd"]) / peaks["bf16"],
                                     bwd_frac_of_peak=tfl(fbwd, bwd_ms) / peaks["bf16"],
                                     fwd_family=line["per_gpu"]["fwd_family"], bwd_family=line["per_gpu"]["bwd_family"])
    if rank == 0:
        if not args.no_cpu_baseline and world == 1:
            units = 8
            val, secs = cpu_sample(units)
            line["cpu_baseline"] = cpu_baseline_record(units, val, secs)
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
