#!/usr/bin/env python
"""Benchmark of the permutohedral-encoding hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload train|sharded]

One step = forward + backward into the lattice values over one batch of synthetic points
(seeded; uniform points, N(0,1) upstream gradient -- the reference's performance script also
uses synthetic uniform points).  Workloads:

  train    pos_dim 3, 24 levels, capacity 2^18, 2^20 points            (default for --gpus 1)
  sharded  pos_dim 3, 24 levels, capacity 2^19, 2^24 points per step split evenly over the
           ranks, lattice replicated, all-reduce of the lattice gradient (default for N > 1)

Rank 0 prints ONE JSON line.  ``value`` is whole-job Mpoints/s with inputs resident in HBM,
timed on the device with CUDA events (max over ranks); ``e2e`` is the same step driven from
pinned host memory (host->device copy of the positions, forward, MSE loss, backward,
device->host read of the loss) through the public module API.

``--impl reference`` times the reference's own CUDA extension (oracle/_ref, rebuilt unmodified
for sm_100; the reference has no CPU path) through the call sequence of its Python module,
on the same workload; if that build is absent it falls back to the CPU restatement in oracle/.
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

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default=None, choices=[None, "train", "sharded", "train_f8"])
    ap.add_argument("--buckets", type=int, default=2, help="level buckets of the overlapped all-reduce")
    ap.add_argument("--collective", default="auto", choices=["auto", "nccl", "multimem"])
    ap.add_argument("--bucket-policy", default="halving", choices=["halving", "even"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    return ap.parse_args()


ARGS = parse_args()
RANK = int(os.environ.get("RANK", "0"))
LOCAL_RANK = int(os.environ.get("LOCAL_RANK", "0"))
WORLD = int(os.environ.get("WORLD_SIZE", "1"))
if ARGS.impl == "reference" and WORLD > 1:
    # the reference pins every allocation to cuda:0: give each rank its own GPU under that name
    _visible = [v for v in os.environ.get("CUDA_VISIBLE_DEVICES", "").split(",") if v]
    os.environ["CUDA_VISIBLE_DEVICES"] = _visible[LOCAL_RANK] if _visible else str(LOCAL_RANK)
    LOCAL_DEVICE = 0
else:
    LOCAL_DEVICE = LOCAL_RANK

if ARGS.impl == "ours" and WORLD == 1:
    from permutohedral_encoding_b200 import build as _ext_build  # noqa: E402
    if not os.path.isfile(_ext_build.LIB_PATH):  # a fresh checkout; multi-rank runs expect it built already
        _ext_build.build()

import numpy as np  # noqa: E402
import torch  # noqa: E402
import torch.distributed as dist  # noqa: E402

WORKLOADS = {
    "train": dict(pos_dim=3, nr_levels=24, capacity=2 ** 18, total_points=2 ** 20, sigma=(1.0, 1e-4)),
    "sharded": dict(pos_dim=3, nr_levels=24, capacity=2 ** 19, total_points=2 ** 24, sigma=(1.0, 1e-4)),
    # not a reference configuration (it has no 8-feature levels): the same 48 outputs from 6 levels of
    # 8 features, every table access a whole 32-byte sector
    "train_f8": dict(pos_dim=3, nr_levels=6, nr_feat=8, capacity=2 ** 18, total_points=2 ** 20, sigma=(1.0, 1e-4)),
}

# dram__bytes_read.sum + dram__bytes_write.sum per launch on the "train" workload, from the ncu
# capture summarised in profiles/train_step_forward_backward_kernels.txt; None = not captured.
NCU_TRAFFIC_BYTES = {"train": {"backward_kernel": 245.0e6, "forward_kernel": 202.5e6}, "sharded": None}


class ClockSampler:
    """nvidia-smi clocks and throttle reasons while the timed region runs."""
    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.rows, self.proc = [], None
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={index}", f"--query-gpu={self.Q}",
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([x.strip() for x in line.split(",")])

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            if len(r) < 7:
                continue
            try:
                sm.append(float(r[0]))
                mx.append(float(r[1]))
            except ValueError:
                continue
            for name, v in zip(names, r[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def make_data(w, n_local, seed, device):
    d, L, cap = w["pos_dim"], w["nr_levels"], w["capacity"]
    gen = torch.Generator(device="cpu").manual_seed(1234)  # lattice and shift identical on every rank
    table = ((torch.rand((L, cap, w.get("nr_feat", 2)), generator=gen) * 2 - 1) * 1e-4)
    shift = torch.randn((L, d), generator=gen) * 10
    gen = torch.Generator(device="cpu").manual_seed(seed)
    pos_host = torch.rand((n_local, d), generator=gen).pin_memory()
    return table.to(device), shift.to(device), pos_host


def device_randn(shape, seed, device):
    gen = torch.Generator(device=device).manual_seed(seed)
    return torch.randn(shape, generator=gen, device=device)


class OursStep:
    """forward + backward through the public module; the all-reduce hook is installed for N > 1."""

    def __init__(self, w, table, shift, device, world, buckets):
        from permutohedral_encoding_b200 import PermutoEncoding
        from permutohedral_encoding_b200.distributed import LatticeGradAllReduce
        sig = np.geomspace(w["sigma"][0], w["sigma"][1], w["nr_levels"])
        self.m = PermutoEncoding(w["pos_dim"], w["capacity"], w["nr_levels"], w.get("nr_feat", 2), sig)
        with torch.no_grad():
            self.m.lattice_values.copy_(table)
            self.m.random_shift_per_level.copy_(shift)
        mm = {"auto": "auto", "nccl": False, "multimem": True}[ARGS.collective]
        self.hook = LatticeGradAllReduce(self.m, nr_buckets=buckets, policy=ARGS.bucket_policy, multimem=mm) \
            if world > 1 else None
        self.collective = None if self.hook is None else ("multimem" if self.hook._symm is not None else "nccl")
        self.launches_per_step = 2 if world == 1 else 1 + len(self.hook.buckets)

    def step(self, pos, grad_out):
        self.m.lattice_values.grad = None
        out = self.m(pos)
        out.backward(grad_out)
        return out

    def e2e_step(self, feeder, pos_host, target):
        self.m.lattice_values.grad = None
        pos = feeder.next()          # this step's positions (their copy was started one step ahead)
        feeder.submit(pos_host)      # the next step's host->device copy runs beside this step
        out = self.m(pos)
        loss = torch.nn.functional.mse_loss(out, target.expand_as(out))
        loss.backward()
        return loss.item()

    def kernels(self, pos, grad_out):
        from permutohedral_encoding_b200 import _native as nat
        I = nat.EncodingInput(self.m.lattice_values.detach(), pos, self.m.anneal_window, True, False)
        lat = self.m.lattice
        buf = torch.empty_like(self.m.lattice_values)
        return (lambda: lat.forward(I)), (lambda: lat.backward(I, grad_out, lattice_grad_out=buf))


class ReferenceStep:
    """The reference's CUDA extension driven like its Python module; all-reduce appended for N > 1."""

    def __init__(self, w, table, shift, device, world):
        from oracle import ref_shim
        sig = np.geomspace(w["sigma"][0], w["sigma"][1], w["nr_levels"])
        self.enc = ref_shim.RefEncoding(w["pos_dim"], w["capacity"], w["nr_levels"], sig, shift)
        self.table = table.clone().requires_grad_(True)
        self.window = torch.ones(w["nr_levels"], device=device)
        self.world = world
        self.launches_per_step = 0

    def step(self, pos, grad_out):
        self.table.grad = None
        out = self.enc(self.table, pos, self.window)
        out.backward(grad_out)
        if self.world > 1:
            dist.all_reduce(self.table.grad)
        return out

    def e2e_step(self, feeder, pos_host, target):
        self.table.grad = None
        pos = feeder.next()
        feeder.submit(pos_host)
        out = self.enc(self.table, pos, self.window)
        loss = torch.nn.functional.mse_loss(out, target.expand_as(out))
        loss.backward()
        if self.world > 1:
            dist.all_reduce(self.table.grad)
        return loss.item()


def timed(fn, steps, warmup, sync):
    for _ in range(warmup):
        fn()
    sync()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(steps):
        fn()
    b.record()
    sync()
    return a.elapsed_time(b) / steps  # ms per step


def max_over_ranks(x, device):
    if WORLD == 1:
        return x
    t = torch.tensor([x], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return t.item()


def cpu_baseline(w):
    """The C restatement (oracle/) on the host cores: forward + backward into the table on a
    bounded sample of the same workload."""
    from oracle import permuto_oracle as po
    d, L, cap = w["pos_dim"], w["nr_levels"], w["capacity"]
    sig = np.geomspace(w["sigma"][0], w["sigma"][1], L)
    rng = np.random.default_rng(0)
    F = w.get("nr_feat", 2)
    table = (rng.random((L, cap, F), dtype=np.float32) * 2 - 1) * np.float32(1e-4)
    shift = (rng.standard_normal((L, d)) * 10).astype(np.float32)
    scale = po.scale_factor(sig, d)
    anneal = np.ones(L, np.float32)
    cores = len(os.sched_getaffinity(0))
    po.set_threads(cores)

    def run(n):
        pos = rng.random((n, d), dtype=np.float32)
        go = rng.standard_normal((n, F * L)).astype(np.float32)
        t0 = time.perf_counter()
        po.forward(pos, table, scale, shift, anneal)
        po.backward(pos, table, scale, shift, anneal, go, need_table=True, need_pos=False)
        return time.perf_counter() - t0

    n = int(min(w["total_points"], 2 ** 20))
    run(2 ** 12)  # page in the table, start the thread pool
    elapsed, points, reps = 0.0, 0, 0
    budget = float(os.environ.get("PERMUTO_CPU_BASELINE_SECONDS", "10"))
    while elapsed < budget and reps < 64:
        elapsed += run(n)
        points += n
        reps += 1
    return {"value": round(points / elapsed / 1e6, 4), "unit": "Mpoints/s", "cores": cores, "kind": "port",
            "sample": f"{reps} x forward+backward of {n} points of the same workload (C restatement in oracle/, "
                      f"OpenMP over {cores} host threads), {elapsed:.1f} s"}


def main():
    args = ARGS
    name = args.workload or ("train" if args.gpus == 1 else "sharded")
    w = WORKLOADS[name]
    d, L, cap = w["pos_dim"], w["nr_levels"], w["capacity"]
    use_ref_ext = False
    if args.impl == "reference" and w.get("nr_feat", 2) != 2:
        if RANK == 0:
            print(json.dumps({"impl": "reference", "unavailable": "the reference implements nr_feat_per_level == 2 only"}))
        return 0
    if args.impl == "reference":
        from oracle import ref_shim
        use_ref_ext = ref_shim.available() and torch.cuda.is_available()
        if not use_ref_ext:
            if RANK != 0:
                return 0
            cb = cpu_baseline(w)
            line = {"impl": "reference", "metric": "fwd+bwd throughput, pos_dim=3, 24 levels", "value": cb["value"],
                    "unit": "Mpoints/s", "n_gpus": args.gpus, "steps": 1, "warmup": 0, "higher_is_better": True,
                    "ms_per_step": None, "scaling": "strong" if name == "sharded" else "weak", "vs_baseline": None,
                    "dtype": "f32", "data": "synthetic", "config": {"workload": name, **w},
                    "cpu_baseline": cb, "e2e": {"value": cb["value"], "unit": "Mpoints/s", "h2d_bytes_per_step": 0,
                                                "d2h_bytes_per_step": 0},
                    "note": "reference CUDA extension build absent: CPU restatement timed instead"}
            print(json.dumps(line))
            return 0

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the encoding has no CPU path")
    torch.cuda.set_device(LOCAL_DEVICE)
    device = torch.device("cuda", LOCAL_DEVICE)
    if WORLD > 1:
        opts = dist.ProcessGroupNCCL.Options(is_high_priority_stream=True)  # collectives beside the backward kernels
        dist.init_process_group("nccl", device_id=device, pg_options=opts)
    assert WORLD == args.gpus, f"--gpus {args.gpus} but WORLD_SIZE={WORLD}: launch with torchrun for N > 1"

    total = w["total_points"]
    from permutohedral_encoding_b200.distributed import shard_bounds
    b, e = shard_bounds(total, RANK, WORLD)
    n_local = e - b
    table, shift, pos_host = make_data(w, n_local, 100 + RANK, device)
    pos = pos_host.to(device)
    F = w.get("nr_feat", 2)
    grad_out = device_randn((n_local, F * L), 200 + RANK, device)
    target = torch.full((1, 1), 0.3, device=device)

    if args.impl == "reference":
        runner = ReferenceStep(w, table, shift, device, WORLD)
    else:
        runner = OursStep(w, table, shift, device, WORLD, args.buckets)

    def sync():
        torch.cuda.synchronize()
        if WORLD > 1:
            dist.barrier()
            torch.cuda.synchronize()

    sampler = ClockSampler(LOCAL_RANK) if RANK == 0 else None
    ms = max_over_ranks(timed(lambda: runner.step(pos, grad_out), args.steps, args.warmup, sync), device)
    clocks = sampler.stop() if sampler else None
    e2e_steps = max(3, min(args.steps, 20))
    from permutohedral_encoding_b200.host_feed import HostPointFeeder
    feeder = HostPointFeeder(device)
    feeder.submit(pos_host)
    ms_e2e = max_over_ranks(timed(lambda: runner.e2e_step(feeder, pos_host, target), e2e_steps, 3, sync), device)

    line = {
        "metric": "fwd+bwd throughput, pos_dim=3, 24 levels",
        "value": round(total / ms / 1e3, 2), "unit": "Mpoints/s", "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": round(ms, 4), "higher_is_better": True,
        "scaling": "strong" if name == "sharded" else "weak", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic",
        "config": {"workload": name, **{k: v for k, v in w.items()}, "points_per_gpu": n_local,
                   "timing": "inputs larger than L2 (features and their gradient are 48*4 B per point)",
                   "parallelism": f"dp{args.gpus}: points sharded, lattice replicated"
                                  + (f", all-reduce of the lattice gradient in {args.buckets} level bucket(s) "
                                     f"({getattr(runner, 'collective', 'nccl')})" if WORLD > 1 else "")},
        "e2e": {"value": round(total / ms_e2e / 1e3, 2), "unit": "Mpoints/s", "h2d_bytes_per_step": n_local * d * 4,
                "d2h_bytes_per_step": 4, "ms_per_step": round(ms_e2e, 4),
                "what": "every step: pinned host positions -> device (double-buffered, copied beside the previous step), module forward, MSE loss, backward, loss.item()"},
        "clocks": clocks,
    }
    if args.impl == "reference":
        line["impl"] = "reference"
        line["gpu_launches"] = 0
        line["cpu_baseline"] = {"value": line["value"], "unit": "Mpoints/s", "cores": 0, "kind": "reference",
                                "sample": "the reference has no CPU path: its own CUDA extension (oracle/_ref, "
                                          "unmodified sources rebuilt for sm_100) on the full workload, on the GPU"}
        line["e2e"] = {"value": line["e2e"]["value"], "unit": "Mpoints/s", "h2d_bytes_per_step": n_local * d * 4,
                       "d2h_bytes_per_step": 4, "ms_per_step": round(ms_e2e, 4)}
    else:
        line["gpu_launches"] = runner.launches_per_step * args.steps
        with torch.no_grad():
            ms_fo = max_over_ranks(timed(lambda: runner.m(pos), max(5, min(args.steps, 30)), 3, sync), device)
        line["forward_only"] = {"value": round(total / ms_fo / 1e3, 2), "unit": "Mpoints/s", "ms_per_step": round(ms_fo, 4),
                                "what": "module forward alone, inputs resident"}
        # kernel-only durations on the launching stream, for the roofline of the dominant kernel
        fwd, bwd = runner.kernels(pos, grad_out)
        ms_f = timed(fwd, 20, 3, torch.cuda.synchronize)
        ms_b = timed(bwd, 20, 3, torch.cuda.synchronize)  # includes the memset of the gradient slices
        V = d + 1
        bytes_f = n_local * (4 * d + 4 * L * V * F + 4 * L * F)
        bytes_b = n_local * (4 * d + 4 * L * F + 4 * L * V * F) + 4 * L * cap * F
        peaks = {}
        try:
            peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
        except OSError:
            pass
        peak = float(peaks.get("hbm_gbs", 6650.0))
        dom = ("backward_kernel", ms_b, bytes_b) if ms_b >= ms_f else ("forward_kernel", ms_f, bytes_f)
        ach = dom[2] / (dom[1] * 1e-3) / 1e9
        line["roofline"] = {"bound": "hbm", "kernel": dom[0], "achieved": round(ach, 1), "peak": peak, "unit": "GB/s",
                            "frac": round(ach / peak, 4), "traffic": (NCU_TRAFFIC_BYTES.get(name) or {}).get(dom[0]),
                            "peak_source": "measured (MEASURED_PEAKS.json)" if peaks else "fallback",
                            "algorithmic_bytes_per_launch": dom[2], "ms_per_launch": round(dom[1], 4),
                            "forward_kernel": {"ms": round(ms_f, 4), "achieved": round(bytes_f / (ms_f * 1e-3) / 1e9, 1)},
                            "backward_kernel": {"ms": round(ms_b, 4), "achieved": round(bytes_b / (ms_b * 1e-3) / 1e9, 1)}}
        # the binding resource is the rate of random accesses that reach L2, not HBM bytes: measure
        # the device's ceilings for that pattern now (independent random accesses over an 8 MB region)
        from permutohedral_encoding_b200 import probe
        ceil_g = probe.measure("gather8" if F == 2 else "gather16", device=device) / 1e9
        ceil_r = probe.measure("red_v2" if F == 2 else "red_v4", device=device) / 1e9
        visits = n_local * L * V
        ops_per_visit = 2 if F == 8 else 1  # a 32-byte entry is two 16-byte operations
        line["roofline_l2_random_access"] = {
            "forward_kernel": {"achieved": round(visits * ops_per_visit / (ms_f * 1e-3) / 1e9, 1), "ceiling": round(ceil_g, 1),
                               "frac": round(visits * ops_per_visit / (ms_f * 1e-3) / 1e9 / ceil_g, 3),
                               "unit": "G random gathers/s"},
            "backward_kernel": {"achieved": round(visits * ops_per_visit / (ms_b * 1e-3) / 1e9, 1), "ceiling": round(ceil_r, 1),
                                "frac": round(visits * ops_per_visit / (ms_b * 1e-3) / 1e9 / ceil_r, 3),
                                "unit": "G vector reductions/s (counted before the in-warp merge)"},
            "ceiling_source": "permuto_probe_random_access, measured in this run over an L2-resident 8 MB region"}
        if RANK == 0 and WORLD == 1 and not args.no_cpu_baseline:
            line["cpu_baseline"] = cpu_baseline(w)
    if WORLD > 1:
        dist.barrier()
        dist.destroy_process_group()
    if RANK == 0:
        print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
