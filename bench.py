#!/usr/bin/env python
"""Benchmark of the permutohedral-encoding hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

One step = forward + backward into the lattice values over one batch of synthetic points
(seeded; uniform points, N(0,1) upstream gradient -- the reference's performance script also
uses synthetic uniform points).  The headline workload is the same at every N, so that the
per-N values form a scaling curve:

  sharded  pos_dim 3, 24 levels, capacity 2^19, 2^24 points per step split evenly over the
           ranks (strong scaling), lattice replicated, all-reduce of the lattice gradient for N > 1

At N = 1 the line also carries one block per other configuration of the baseline, each timed the
same way in both arms (``--impl ours`` and ``--impl reference``):

  train                 pos_dim 3, 24 levels, capacity 2^18, 2^20 points, forward + backward
  readme_forward        the same encoding, forward of 1000 points (latency per call)
  eikonal               capacity 2^19, 2^19 points in [-1,1)^3: forward, d/dx with create_graph,
                        loss on the gradient norm, double backward into the lattice values
  dim4, dim6            pos_dim 4 / 6, 16 levels, capacity 2^20, 2^20 points, forward + backward
  train_with_optimizer  the train step with MSE loss and an AdamW step on the table
                        (the reference's examples/performance.py loop)
  forward_linear        inference of the train workload followed by Linear(48, 32), the first layer
                        of the reference's toy MLP; this repo runs it as one fused kernel
  forward_mlp           the same with the toy example's whole MLP (48-32-32-32-1, GELU) fused

Rank 0 prints ONE JSON line.  ``value`` is whole-job Mpoints/s with inputs resident in HBM,
timed on the device with CUDA events (max over ranks, median over repeats of K steps);
``e2e`` is the same step driven from pinned host memory (host->device copy of the positions,
forward, MSE loss, backward, device->host read of the loss) through the public module API.

``--impl reference`` times the reference's own CUDA extension (oracle/_ref, rebuilt unmodified
for sm_100; the reference has no CPU path) through the call sequence of its Python module,
on the same workloads; if that build is absent it falls back to the CPU restatement in oracle/.
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

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="sharded", choices=["sharded", "train", "train_f8"])
    ap.add_argument("--buckets", type=int, default=2, help="level buckets of the overlapped all-reduce")
    ap.add_argument("--collective", default="auto", choices=["auto", "nccl", "multimem"])
    ap.add_argument("--bucket-policy", default="halving", choices=["halving", "even"])
    ap.add_argument("--copy-out", action="store_true", help="copy the reduced gradient out of the symmetric buffer")
    ap.add_argument("--clear", default="inline", choices=["inline", "early"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--blocks", default=None,
                    help="comma-separated per-configuration blocks to add at N = 1 (train, forward_linear, forward_mlp, "
                         "train_with_optimizer, readme_forward, eikonal, dim4, dim6); default: all of them for the "
                         "sharded workload, none otherwise")
    ap.add_argument("--no-blocks", action="store_true", help="same as --blocks ''")
    ap.add_argument("--total-points", type=int, default=None,
                    help="override the workload's points per step (small cases for profiler captures)")
    ap.add_argument("--min-timed-seconds", type=float, default=0.5)
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
    "sharded": dict(pos_dim=3, nr_levels=24, capacity=2 ** 19, total_points=2 ** 24, sigma=(1.0, 1e-4)),
    "train": dict(pos_dim=3, nr_levels=24, capacity=2 ** 18, total_points=2 ** 20, sigma=(1.0, 1e-4)),
    "readme_forward": dict(pos_dim=3, nr_levels=24, capacity=2 ** 18, total_points=1000, sigma=(1.0, 1e-4)),
    "eikonal": dict(pos_dim=3, nr_levels=24, capacity=2 ** 19, total_points=2 ** 19, sigma=(1.0, 1e-4), box=(-1.0, 1.0)),
    "dim4": dict(pos_dim=4, nr_levels=16, capacity=2 ** 20, total_points=2 ** 20, sigma=(1.0, 1e-3)),
    "dim6": dict(pos_dim=6, nr_levels=16, capacity=2 ** 20, total_points=2 ** 20, sigma=(1.0, 1e-3)),
    # not a reference configuration (it has no 8-feature levels): the same 48 outputs from 6 levels of
    # 8 features, every table access a whole 32-byte sector
    "train_f8": dict(pos_dim=3, nr_levels=6, nr_feat=8, capacity=2 ** 18, total_points=2 ** 20, sigma=(1.0, 1e-4)),
}
METRIC = "fwd+bwd throughput, pos_dim=3, 24 levels"


def load_json(path):
    try:
        with open(path) as f:
            return json.load(f)
    except (OSError, ValueError):
        return {}


PEAKS = load_json(os.path.join(ROOT, "MEASURED_PEAKS.json"))
HBM_PEAK = float(PEAKS.get("hbm_gbs", 6650.0))
PEAK_SOURCE = "measured (MEASURED_PEAKS.json)" if PEAKS else "fallback (6650 GB/s)"
# dram__bytes_read.sum + dram__bytes_write.sum per launch from the ncu captures summarised in profiles/
NCU_TRAFFIC = load_json(os.path.join(ROOT, "profiles", "ncu_dram_traffic.json"))


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
    lo, hi = w.get("box", (0.0, 1.0))
    pos_host = (torch.rand((n_local, d), generator=gen) * (hi - lo) + lo).pin_memory()
    return table.to(device), shift.to(device), pos_host


def device_randn(shape, seed, device):
    gen = torch.Generator(device=device).manual_seed(seed)
    return torch.randn(shape, generator=gen, device=device)


class OursStep:
    """forward + backward through the public module; the all-reduce hook is installed for N > 1."""
    impl = "ours"

    def __init__(self, w, table, shift, device, world, buckets=2):
        from permutohedral_encoding_b200 import PermutoEncoding
        from permutohedral_encoding_b200.distributed import LatticeGradAllReduce
        sig = np.geomspace(w["sigma"][0], w["sigma"][1], w["nr_levels"])
        self.m = PermutoEncoding(w["pos_dim"], w["capacity"], w["nr_levels"], w.get("nr_feat", 2), sig)
        with torch.no_grad():
            self.m.lattice_values.copy_(table)
            self.m.random_shift_per_level.copy_(shift)
        mm = {"auto": "auto", "nccl": False, "multimem": True}[ARGS.collective]
        self.hook = LatticeGradAllReduce(self.m, nr_buckets=buckets, policy=ARGS.bucket_policy, multimem=mm,
                                         copy_out=ARGS.copy_out, clear=ARGS.clear) if world > 1 else None
        self.collective = None if self.hook is None else ("multimem" if self.hook._symm is not None else "nccl")
        self.launches_per_step = 2 if world == 1 else 1 + len(self.hook.buckets)
        self.opt = None

    @property
    def values(self):
        return self.m.lattice_values

    def encode(self, pos):
        return self.m(pos)

    def step(self, pos, grad_out):
        self.m.lattice_values.grad = None
        out = self.m(pos)
        out.backward(grad_out)
        return out

    def make_optimizer(self):
        from permutohedral_encoding_b200.optim import LatticeAdamW
        self.opt = LatticeAdamW([self.m.lattice_values], lr=1e-3, betas=(0.9, 0.99), eps=1e-15, weight_decay=0.0,
                                skip_untouched=True)

    def kernels(self, pos, grad_out):
        from permutohedral_encoding_b200 import _native as nat
        I = nat.EncodingInput(self.m.lattice_values.detach(), pos, self.m.anneal_window, True, False)
        lat = self.m.lattice
        buf = torch.empty_like(self.m.lattice_values)
        return (lambda: lat.forward(I)), (lambda: lat.backward(I, grad_out, lattice_grad_out=buf))


class ReferenceStep:
    """The reference's CUDA extension driven like its Python module; all-reduce appended for N > 1."""
    impl = "reference"

    def __init__(self, w, table, shift, device, world, buckets=None):
        from oracle import ref_shim
        sig = np.geomspace(w["sigma"][0], w["sigma"][1], w["nr_levels"])
        self.enc = ref_shim.RefEncoding(w["pos_dim"], w["capacity"], w["nr_levels"], sig, shift)
        self.table = table.clone().requires_grad_(True)
        self.window = torch.ones(w["nr_levels"], device=device)
        self.world = world
        self.launches_per_step = 0
        self.collective = "nccl" if world > 1 else None
        self.opt = None

    @property
    def values(self):
        return self.table

    def encode(self, pos):
        return self.enc(self.table, pos, self.window)

    def step(self, pos, grad_out):
        self.table.grad = None
        out = self.enc(self.table, pos, self.window)
        out.backward(grad_out)
        if self.world > 1:
            dist.all_reduce(self.table.grad)
        return out

    def make_optimizer(self):  # examples/performance.py:161
        self.opt = torch.optim.AdamW([self.table], amsgrad=False, betas=(0.9, 0.99), eps=1e-15, weight_decay=0.0, lr=1e-3)


def e2e_step(runner, feeder, pos_host, target):
    runner.values.grad = None
    pos = feeder.next()          # this step's positions (their copy was started one step ahead)
    feeder.submit(pos_host)      # the next step's host->device copy runs beside this step
    out = runner.encode(pos)
    loss = torch.nn.functional.mse_loss(out, target.expand_as(out))
    loss.backward()
    if runner.impl == "reference" and WORLD > 1:
        dist.all_reduce(runner.values.grad)
    return loss.item()


def eikonal_step(runner, pos, w_vec):
    """PermutoSDF's eikonal term: y = F w, g = dy/dx (create_graph), loss = mean((|g| - 1)^2)."""
    runner.values.grad = None
    x = pos.detach().requires_grad_(True)
    y = runner.encode(x) @ w_vec
    (g,) = torch.autograd.grad(y.sum(), x, create_graph=True)
    loss = ((g.norm(dim=1) - 1.0) ** 2).mean()
    loss.backward()
    return loss


def optimizer_step(runner, pos):
    """The reference's training loop (examples/performance.py:96-101)."""
    pred = runner.encode(pos)
    loss = ((pred - 10) ** 2).mean()
    runner.opt.zero_grad()
    loss.backward()
    runner.opt.step()
    return loss


def sync_all():
    torch.cuda.synchronize()
    if WORLD > 1:
        dist.barrier()
        torch.cuda.synchronize()


def max_over_ranks(x, device):
    if WORLD == 1:
        return x
    t = torch.tensor([x], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return t.item()


def timed(fn, steps, warmup, device, min_seconds=None, sync=None):
    """ms per step: `warmup` untimed steps, then repeats of exactly `steps` steps, each bracketed
    by a synchronize (and a barrier for N > 1) on both sides and timed with CUDA events on the
    current stream; a repeat's time is the max over ranks; the median over the repeats is
    returned.  The number of repeats is chosen from the first one so that about `min_seconds` are
    timed in total (every rank derives it from the same max-over-ranks value)."""
    sync = sync or sync_all
    min_seconds = ARGS.min_timed_seconds if min_seconds is None else min_seconds
    for _ in range(warmup):
        fn()
    samples, repeats = [], 1
    while len(samples) < repeats:
        sync()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(steps):
            fn()
        b.record()
        sync()
        samples.append(max_over_ranks(a.elapsed_time(b) / steps, device))
        if len(samples) == 1:
            repeats = int(min(25, max(1, math.ceil(min_seconds * 1e3 / max(samples[0] * steps, 1e-3)))))
    return statistics.median(samples), len(samples)


def local_sync():
    torch.cuda.synchronize()


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


def algorithmic_bytes(w, n, kind):
    """Bytes an ideal implementation must move (independent of sector granularity): positions,
    8-byte table entries gathered or scattered, feature rows, and the zero-init of the gradient table."""
    d, L, cap, F = w["pos_dim"], w["nr_levels"], w["capacity"], w.get("nr_feat", 2)
    V = d + 1
    row, entries, table = 4 * L * F, 4 * L * V * F, 4 * L * cap * F
    per_point = {"fwd": 4 * d + entries + row, "bwd_table": 4 * d + row + entries,
                 "bwd_pos": 4 * d + row + entries + 4 * d, "dbl_table": 8 * d + row + entries}[kind]
    return n * per_point + (table if kind in ("bwd_table", "dbl_table") else 0)


def roofline_block(w, name, n_local, ms_f, ms_b, device, ceilings=None):
    """HBM roofline of the slower kernel plus the rate of random accesses against the device's
    ceilings for that pattern, which is what binds these kernels."""
    d, L, F = w["pos_dim"], w["nr_levels"], w.get("nr_feat", 2)
    bytes_f, bytes_b = algorithmic_bytes(w, n_local, "fwd"), algorithmic_bytes(w, n_local, "bwd_table")
    dom = ("backward_kernel", ms_b, bytes_b) if ms_b >= ms_f else ("forward_kernel", ms_f, bytes_f)
    ach = dom[2] / (dom[1] * 1e-3) / 1e9
    traffic = (NCU_TRAFFIC.get(name) or {}).get(dom[0])
    out = {"bound": "hbm", "kernel": dom[0], "achieved": round(ach, 1), "peak": HBM_PEAK, "unit": "GB/s",
           "frac": round(ach / HBM_PEAK, 4), "traffic": traffic, "traffic_source": (NCU_TRAFFIC.get(name) or {}).get("source"),
           "peak_source": PEAK_SOURCE, "algorithmic_bytes_per_launch": dom[2], "ms_per_launch": round(dom[1], 4),
           "forward_kernel": {"ms": round(ms_f, 4), "achieved": round(bytes_f / (ms_f * 1e-3) / 1e9, 1)},
           "backward_kernel": {"ms": round(ms_b, 4), "achieved": round(bytes_b / (ms_b * 1e-3) / 1e9, 1)}}
    if ceilings:
        visits = n_local * L * (d + 1) * (2 if F == 8 else 1)  # a 32-byte entry is two 16-byte operations
        g, r = visits / (ms_f * 1e-3) / 1e9, visits / (ms_b * 1e-3) / 1e9
        out["l2_random_access"] = {
            "forward_kernel": {"achieved": round(g, 1), "ceiling": ceilings["gather"], "frac": round(g / ceilings["gather"], 3),
                               "unit": "G random gathers/s"},
            "backward_kernel": {"achieved": round(r, 1), "ceiling": ceilings["red"], "frac": round(r / ceilings["red"], 3),
                                "unit": "G vector reductions/s (counted before the in-warp merge)"},
            "ceiling_source": "permuto_probe_random_access, measured in this run over an L2-resident 8 MB region"}
        out["frac_l2_ops"] = out["l2_random_access"][dom[0]]["frac"]
        out["ceiling"] = out["l2_random_access"][dom[0]]["ceiling"]
        out["binding"] = ("l2 random-access rate: the kernel moves 8-byte table entries whose 32-byte sectors stay in L2, "
                          "so DRAM bytes are not what limits it; frac is kept for the HBM roofline")
    return out


def make_runner(impl, w, table, shift, device, world=1):
    return (ReferenceStep if impl == "reference" else OursStep)(w, table, shift, device, world, ARGS.buckets)


def block_train(impl, name, device, steps, ceilings):
    """forward + backward into the table on one GPU; used for train, dim4, dim6."""
    w = WORKLOADS[name]
    n, L, F = w["total_points"], w["nr_levels"], w.get("nr_feat", 2)
    table, shift, pos_host = make_data(w, n, 100, device)
    pos = pos_host.to(device)
    grad_out = device_randn((n, F * L), 200, device)
    runner = make_runner(impl, w, table, shift, device)
    ms, reps = timed(lambda: runner.step(pos, grad_out), steps, 3, device, 0.2, local_sync)
    with torch.no_grad():
        ms_fo, _ = timed(lambda: runner.encode(pos), steps, 3, device, 0.1, local_sync)
    blk = {"value": round(n / ms / 1e3, 2), "unit": "Mpoints/s", "ms_per_step": round(ms, 4), "repeats": reps,
           "forward_only": {"value": round(n / ms_fo / 1e3, 2), "ms_per_step": round(ms_fo, 4)},
           "config": {k: v for k, v in w.items()}}
    if impl == "ours":
        fwd, bwd = runner.kernels(pos, grad_out)
        ms_f, _ = timed(fwd, 20, 3, device, 0.05, local_sync)
        ms_b, _ = timed(bwd, 20, 3, device, 0.05, local_sync)  # includes the memset of the gradient table
        blk["roofline"] = roofline_block(w, name, n, ms_f, ms_b, device, ceilings)
    return blk, runner, pos


def block_readme_forward(impl, device):
    w = WORKLOADS["readme_forward"]
    n = w["total_points"]
    table, shift, pos_host = make_data(w, n, 101, device)
    pos = pos_host.to(device)
    runner = make_runner(impl, w, table, shift, device)
    with torch.no_grad():
        ms, reps = timed(lambda: runner.encode(pos), 200, 20, device, 0.1, local_sync)
        for _ in range(20):
            runner.encode(pos)
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        for _ in range(500):
            runner.encode(pos)
        torch.cuda.synchronize()
        wall = (time.perf_counter() - t0) / 500
    return {"value": round(ms * 1e3, 2), "unit": "us per forward of 1000 points (CUDA events, back-to-back calls)",
            "wall_us_per_call": round(wall * 1e6, 2), "higher_is_better": False, "repeats": reps,
            "note": "host-dispatch bound: the kernel itself runs for a few microseconds"}


def block_eikonal(impl, device, steps):
    w = WORKLOADS["eikonal"]
    n, L = w["total_points"], w["nr_levels"]
    table, shift, pos_host = make_data(w, n, 102, device)
    pos = pos_host.to(device)
    gen = torch.Generator(device="cpu").manual_seed(5003)
    w_vec = (torch.randn(2 * L, generator=gen) * (1.0 / 48) ** 0.5).to(device)
    runner = make_runner(impl, w, table, shift, device)
    ms, reps = timed(lambda: eikonal_step(runner, pos, w_vec), steps, 3, device, 0.2, local_sync)
    total = algorithmic_bytes(w, n, "fwd") + algorithmic_bytes(w, n, "bwd_pos") + algorithmic_bytes(w, n, "dbl_table")
    ach = total / (ms * 1e-3) / 1e9
    return {"value": round(n / ms / 1e3, 2), "unit": "Mpoints/s", "ms_per_step": round(ms, 4), "repeats": reps,
            "config": {k: v for k, v in w.items()},
            "roofline": {"bound": "hbm", "what": "whole step: forward + position backward + double backward into the table "
                                                 "(the autograd elementwise kernels between them are not counted)",
                         "achieved": round(ach, 1), "peak": HBM_PEAK, "unit": "GB/s", "frac": round(ach / HBM_PEAK, 4),
                         "algorithmic_bytes_per_step": total}}


def block_optimizer(impl, runner, pos, device, steps):
    runner.make_optimizer()
    ms, reps = timed(lambda: optimizer_step(runner, pos), steps, 3, device, 0.2, local_sync)
    n = pos.shape[0]
    return {"value": round(n / ms / 1e3, 2), "unit": "Mpoints/s", "ms_per_step": round(ms, 4), "repeats": reps,
            "what": "train workload: forward, loss = mean((pred - 10)^2), zero_grad, backward, AdamW step on the table "
                    "(betas 0.9/0.99, eps 1e-15, no weight decay), as in the reference's examples/performance.py"}


def block_forward_linear(impl, runner, pos, device, steps):
    """Inference of the encoding followed by the consumer's first layer, Linear(48, 32) as in the
    reference's examples/train_toy_example.py:18-19, on the train workload.  Ours: one fused kernel
    (features never written; tensor cores) and, beside it, the unfused pair; reference: its module
    followed by the same torch layer."""
    gen = torch.Generator(device="cpu").manual_seed(77)
    width = runner.encode(pos[:8]).shape[1]
    lin = torch.nn.Linear(width, 32)
    with torch.no_grad():
        lin.weight.copy_(torch.randn((32, width), generator=gen) / width ** 0.5)
        lin.bias.copy_(torch.randn(32, generator=gen) * 0.1)
    lin = lin.to(device)
    n = pos.shape[0]
    with torch.no_grad():
        ms_pair, reps = timed(lambda: lin(runner.encode(pos)), steps, 3, device, 0.2, local_sync)
        blk = {"unit": "Mpoints/s", "out_features": 32,
               "what": "train workload, inference: encoding followed by torch.nn.Linear(48, 32)"}
        if impl == "ours":
            ms_fused, reps = timed(lambda: runner.m.forward_linear(pos, lin), steps, 3, device, 0.2, local_sync)
            d, L = 3, WORKLOADS["train"]["nr_levels"]
            alg = n * (4 * d + 4 * L * (d + 1) * 2 + 4 * 32)   # positions, gathered entries, [N, 32] output
            blk.update({"value": round(n / ms_fused / 1e3, 2), "ms_per_step": round(ms_fused, 4), "repeats": reps,
                        "unfused": {"value": round(n / ms_pair / 1e3, 2), "ms_per_step": round(ms_pair, 4),
                                    "what": "module forward, then the torch layer"},
                        "hbm_bytes_per_point": {"fused": 4 * d + 4 * 32, "unfused": 4 * d + 4 * width * 2 + 4 * 32},
                        "roofline": {"bound": "hbm", "achieved": round(alg / (ms_fused * 1e-3) / 1e9, 1), "peak": HBM_PEAK,
                                     "unit": "GB/s", "frac": round(alg / (ms_fused * 1e-3) / 1e9 / HBM_PEAK, 4),
                                     "algorithmic_bytes_per_launch": alg,
                                     "note": "bound by the rate of random table gathers, like the plain forward; the "
                                             "tensor-core product (2*48*32 flop per point) is negligible"}})
        else:
            blk.update({"value": round(n / ms_pair / 1e3, 2), "ms_per_step": round(ms_pair, 4), "repeats": reps})
    return blk


def block_forward_mlp(impl, runner, pos, device, steps):
    """Inference of the encoding followed by the WHOLE network of the reference's toy example
    (examples/train_toy_example.py:18-26): Linear(48,32) GELU Linear(32,32) GELU Linear(32,32) GELU
    Linear(32,1), on the train workload.  Ours: one fused kernel; beside it the unfused pair."""
    gen = torch.Generator(device="cpu").manual_seed(78)
    width = runner.encode(pos[:8]).shape[1]
    mlp = torch.nn.Sequential(torch.nn.Linear(width, 32), torch.nn.GELU(), torch.nn.Linear(32, 32), torch.nn.GELU(),
                              torch.nn.Linear(32, 32), torch.nn.GELU(), torch.nn.Linear(32, 1))
    with torch.no_grad():
        for m in mlp:
            if isinstance(m, torch.nn.Linear):
                m.weight.copy_(torch.randn(m.weight.shape, generator=gen) * (2.0 / m.in_features) ** 0.5)
                m.bias.copy_(torch.randn(m.bias.shape, generator=gen) * 0.1)
    mlp = mlp.to(device)
    n = pos.shape[0]
    with torch.no_grad():
        ms_pair, reps = timed(lambda: mlp(runner.encode(pos)), steps, 3, device, 0.2, local_sync)
        blk = {"unit": "Mpoints/s", "network": "48-32-32-32-1, GELU",
               "what": "train workload, inference: encoding followed by the toy example's MLP"}
        if impl == "ours":
            ms_fused, reps = timed(lambda: runner.m.forward_mlp(pos, mlp), steps, 3, device, 0.2, local_sync)
            blk.update({"value": round(n / ms_fused / 1e3, 2), "ms_per_step": round(ms_fused, 4), "repeats": reps,
                        "unfused": {"value": round(n / ms_pair / 1e3, 2), "ms_per_step": round(ms_pair, 4),
                                    "what": "module forward, then the torch.nn.Sequential"},
                        "hbm_bytes_per_point": {"fused": 4 * 3 + 4, "unfused": 4 * 3 + 4 * width * 2 + 4 * 32 * 6 + 4 * 32 * 6 + 4}})
        else:
            blk.update({"value": round(n / ms_pair / 1e3, 2), "ms_per_step": round(ms_pair, 4), "repeats": reps})
    return blk


def allreduce_check(runner, pos, grad_out, device):
    """Outside the timed region: the gradient the overlapped, bucketed all-reduce left in .grad
    against a plain all-reduce of an un-hooked local backward.  Largest error relative to the
    level's largest entry (atomics make each local gradient differ in the last bits from run to run)."""
    m = runner.m
    runner.step(pos, grad_out)
    torch.cuda.synchronize()
    hooked = m.lattice_values.grad.clone()
    hook_fn, hook2 = m.lattice.backward_hook, m.lattice.double_backward_hook
    m.lattice.backward_hook = m.lattice.double_backward_hook = None
    try:
        m.lattice_values.grad = None
        m(pos).backward(grad_out)
        plain = m.lattice_values.grad.clone()
    finally:
        m.lattice.backward_hook, m.lattice.double_backward_hook = hook_fn, hook2
    dist.all_reduce(plain)
    torch.cuda.synchronize()
    lvl = plain.abs().amax(dim=(1, 2)).clamp_min(1e-30)
    err = ((hooked - plain).abs().amax(dim=(1, 2)) / lvl).max()
    dist.all_reduce(err, op=dist.ReduceOp.MAX)
    m.lattice_values.grad = None
    return {"max_rel_err_per_level": float(err.item()), "tolerance": 1e-4, "ok": bool(err.item() <= 1e-4),
            "what": "hooked bucketed all-reduce vs dist.all_reduce of a plain local backward, max over levels and ranks"}


def reference_cpu_line(name, w):
    cb = cpu_baseline(w)
    return {"impl": "reference", "metric": METRIC, "value": cb["value"], "unit": "Mpoints/s", "n_gpus": ARGS.gpus,
            "steps": 1, "warmup": 0, "higher_is_better": True, "ms_per_step": None, "scaling": "strong",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic", "config": {"workload": name, **w},
            "cpu_baseline": cb, "e2e": {"value": cb["value"], "unit": "Mpoints/s", "h2d_bytes_per_step": 0,
                                        "d2h_bytes_per_step": 0},
            "note": "reference CUDA extension build absent: CPU restatement timed instead"}


def main():
    args = ARGS
    name = args.workload
    w = dict(WORKLOADS[name])
    if args.total_points:
        w["total_points"] = int(args.total_points)
    d, L = w["pos_dim"], w["nr_levels"]
    all_blocks = ["train", "forward_linear", "forward_mlp", "train_with_optimizer", "readme_forward", "eikonal", "dim4",
                  "dim6"]
    if args.no_blocks or WORLD > 1:
        blocks = []
    elif args.blocks is not None:
        blocks = [b for b in args.blocks.split(",") if b]
        unknown = [b for b in blocks if b not in all_blocks]
        if unknown:
            raise SystemExit(f"unknown block(s) {unknown}; choose from {all_blocks}")
    else:
        blocks = all_blocks if (name == "sharded" and not args.total_points) else []
    if args.impl == "reference" and w.get("nr_feat", 2) != 2:
        if RANK == 0:
            print(json.dumps({"impl": "reference", "unavailable": "the reference implements nr_feat_per_level == 2 only"}))
        return 0
    if args.impl == "reference":
        from oracle import ref_shim
        if not (ref_shim.available() and torch.cuda.is_available()):
            if RANK == 0:
                print(json.dumps(reference_cpu_line(name, w)))
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
    runner = make_runner(args.impl, w, table, shift, device, WORLD)

    sampler = ClockSampler(LOCAL_RANK) if RANK == 0 else None
    ms, repeats = timed(lambda: runner.step(pos, grad_out), args.steps, args.warmup, device)
    clocks = sampler.stop() if sampler else None
    e2e_steps = max(3, min(args.steps, 20))
    from permutohedral_encoding_b200.host_feed import HostPointFeeder
    feeder = HostPointFeeder(device)
    feeder.submit(pos_host)
    ms_e2e, _ = timed(lambda: e2e_step(runner, feeder, pos_host, target), e2e_steps, 3, device, 0.2)

    parallelism = f"dp{args.gpus}: points sharded, lattice replicated"
    if WORLD > 1:
        nr_buckets = len(runner.hook.buckets) if args.impl == "ours" else 1
        parallelism += f", all-reduce of the lattice gradient in {nr_buckets} level bucket(s) ({runner.collective})"
    line = {
        "metric": METRIC,
        "value": round(total / ms / 1e3, 2), "unit": "Mpoints/s", "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": round(ms, 4), "repeats": repeats, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": name, **{k: v for k, v in w.items()}, "points_per_gpu": n_local,
                   "timing": "inputs larger than L2 (features and their gradient are 48*4 B per point); "
                             f"median of {repeats} repeat(s) of {args.steps} steps, max over ranks",
                   "parallelism": parallelism},
        "e2e": {"value": round(total / ms_e2e / 1e3, 2), "unit": "Mpoints/s", "h2d_bytes_per_step": n_local * d * 4,
                "d2h_bytes_per_step": 4, "ms_per_step": round(ms_e2e, 4),
                "what": "every step: pinned host positions -> device (double-buffered, copied beside the previous step), "
                        "module forward, MSE loss, backward, loss.item()"},
        "clocks": clocks,
    }
    if args.impl == "reference":
        line["impl"] = "reference"
        line["gpu_launches"] = 0
        line["cpu_baseline"] = {"value": line["value"], "unit": "Mpoints/s", "cores": 0, "kind": "reference",
                                "sample": "the reference has no CPU path: its own CUDA extension (oracle/_ref, "
                                          "unmodified sources rebuilt for sm_100) on the full workload, on the GPU"}
    else:
        line["gpu_launches"] = runner.launches_per_step * args.steps * repeats
        with torch.no_grad():
            ms_fo, _ = timed(lambda: runner.encode(pos), max(5, min(args.steps, 30)), 3, device, 0.2)
        line["forward_only"] = {"value": round(total / ms_fo / 1e3, 2), "unit": "Mpoints/s", "ms_per_step": round(ms_fo, 4),
                                "what": "module forward alone, inputs resident"}
        # kernel-only durations on the launching stream, for the roofline of the dominant kernel
        fwd, bwd = runner.kernels(pos, grad_out)
        ms_f, _ = timed(fwd, 20, 3, device, 0.05, local_sync)
        ms_b, _ = timed(bwd, 20, 3, device, 0.05, local_sync)  # includes the memset of the gradient slices
        # the binding resource is the rate of random accesses that reach L2, not HBM bytes: measure
        # the device's ceilings for that pattern now (independent random accesses over an 8 MB region)
        from permutohedral_encoding_b200 import probe
        ceilings = {"gather": round(probe.measure("gather8" if F == 2 else "gather16", device=device) / 1e9, 1),
                    "red": round(probe.measure("red_v2" if F == 2 else "red_v4", device=device) / 1e9, 1)}
        line["roofline"] = roofline_block(w, name, n_local, ms_f, ms_b, device, ceilings)
        if WORLD > 1:
            line["allreduce_check"] = allreduce_check(runner, pos, grad_out, device)

    if blocks:
        del runner, pos, grad_out, feeder
        torch.cuda.empty_cache()
        ceil2 = ceilings if args.impl == "ours" else None
        if {"train", "forward_linear", "forward_mlp", "train_with_optimizer"} & set(blocks):
            blk, r2, p2 = block_train(args.impl, "train", device, args.steps, ceil2)
            if "train" in blocks:
                line["train"] = blk
            if "forward_linear" in blocks:
                line["forward_linear"] = block_forward_linear(args.impl, r2, p2, device, args.steps)
            if "forward_mlp" in blocks:
                line["forward_mlp"] = block_forward_mlp(args.impl, r2, p2, device, args.steps)
            if "train_with_optimizer" in blocks:
                line["train_with_optimizer"] = block_optimizer(args.impl, r2, p2, device, args.steps)
            del r2, p2
        if "readme_forward" in blocks:
            line["readme_forward"] = block_readme_forward(args.impl, device)
        if "eikonal" in blocks:
            line["eikonal"] = block_eikonal(args.impl, device, args.steps)
        for nm in ("dim4", "dim6"):
            if nm in blocks:
                torch.cuda.empty_cache()
                line[nm], r3, p3 = block_train(args.impl, nm, device, args.steps, None)
                del r3, p3
    if args.impl == "ours" and RANK == 0 and WORLD == 1 and not args.no_cpu_baseline:
        line["cpu_baseline"] = cpu_baseline(w)
    if WORLD > 1:
        dist.barrier()
        dist.destroy_process_group()
    if RANK == 0:
        print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
