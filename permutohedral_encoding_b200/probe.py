"""Random-access ceilings of the GPU for the lattice kernels' access pattern.

``python -m permutohedral_encoding_b200.probe`` prints, for a few region sizes, how many
independent random 8/16-byte gathers and vector reductions per second the device sustains
(`permuto_probe_random_access` in the C ABI).  The lattice kernels are bound by these operation
rates, not by bytes per second; ``bench.py`` reports its achieved rates against them.
"""
from __future__ import annotations

import ctypes as C

import torch

from . import _native as nat

KINDS = {"gather8": 0, "gather16": 1, "red_v2": 2, "red_v4": 3}


def measure(kind: str, region_bytes: int = 8 << 20, accesses_per_thread: int = 256, device=None, repeats: int = 3) -> float:
    """Sustained operations per second of one kind over a zero-filled region of ``region_bytes``."""
    device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    region = torch.zeros(region_bytes // 4, dtype=torch.float32, device=device)
    total = C.c_int64(0)
    best = 0.0
    with torch.cuda.device(device):
        stream = nat._stream(device)
        for i in range(repeats + 1):
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            nat.check(nat.lib.permuto_probe_random_access(KINDS[kind], region.data_ptr(), region.numel() * 4,
                                                          accesses_per_thread, C.byref(total), stream))
            b.record()
            torch.cuda.synchronize(device)
            if i > 0:  # first launch is a warm-up
                best = max(best, total.value / (a.elapsed_time(b) * 1e-3))
    return best


def ceilings(region_bytes: int = 8 << 20, device=None) -> dict:
    """G operations/s for the four access kinds over an L2-resident region."""
    return {k: round(measure(k, region_bytes, device=device) / 1e9, 1) for k in KINDS}


def main() -> int:
    print(f"{'region':>10}  " + "  ".join(f"{k:>10}" for k in KINDS) + "   (G operations/s)")
    for mb in (0.0625, 2, 8, 32, 64, 128, 512):
        row = ceilings(int(mb * (1 << 20)))
        print(f"{mb:>8} MB  " + "  ".join(f"{row[k]:>10.1f}" for k in KINDS))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
