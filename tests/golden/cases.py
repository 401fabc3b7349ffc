"""Seeded synthetic inputs for the parity cases, from a generator that does not depend on any
library's random stream (a counter-based SplitMix64), so the same bits are produced wherever
the fixtures are made or checked.

The reference project ships no tests and no golden vectors; the fixtures next to this file
(``*.npz``) hold the OUTPUTS of the reference's own CUDA extension (rebuilt unmodified for
sm_100, run on a B200 by ``make_golden.py``) for the inputs defined here.  Shapes and value
distributions follow the reference's usage example and performance script
(README.md:17-44, examples/performance.py:149-183): points uniform in a box, lattice values
small and uniform, shifts ~ N(0, 10^2), scales a geometric progression.
"""
from __future__ import annotations

import zlib

import numpy as np

_MASK = np.uint64(0xFFFFFFFFFFFFFFFF)


def _splitmix64(idx: np.ndarray, seed: int) -> np.ndarray:
    with np.errstate(over="ignore"):
        z = (idx.astype(np.uint64) + np.uint64(seed)) * np.uint64(0x9E3779B97F4A7C15)
        z = (z ^ (z >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)
        z = (z ^ (z >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)
        z = z ^ (z >> np.uint64(31))
    return z


def uniform01(shape, seed: int) -> np.ndarray:
    """float64 uniform in [0, 1) with 53 random bits."""
    n = int(np.prod(shape))
    bits = _splitmix64(np.arange(n, dtype=np.uint64), seed * 0x1000003 + 12345)
    return ((bits >> np.uint64(11)).astype(np.float64) * (1.0 / 9007199254740992.0)).reshape(shape)


def uniform(shape, seed: int, lo: float, hi: float) -> np.ndarray:
    return (lo + (hi - lo) * uniform01(shape, seed)).astype(np.float32)


def normal(shape, seed: int, std: float = 1.0) -> np.ndarray:
    """Box-Muller on two independent uniform streams; float32."""
    u1 = uniform01(shape, seed * 2 + 1)
    u2 = uniform01(shape, seed * 2 + 2)
    r = np.sqrt(-2.0 * np.log(1.0 - u1))
    return (std * r * np.cos(2.0 * np.pi * u2)).astype(np.float32)


def cosine_window(nr_levels: int, t: float) -> np.ndarray:
    x = np.clip(t * nr_levels - np.arange(nr_levels, dtype=np.float32), 0.0, 1.0).astype(np.float32)
    return (0.5 * (1 + np.cos(np.pi * x + np.pi))).astype(np.float32)


# name -> description of the case.  "n" is kept small: every output is stored in the fixture.
CASES = {
    # the README usage example (BASELINE config 1): forward only
    "readme_d3": dict(pos_dim=3, capacity=2 ** 18, nr_levels=24, sigma=(1.0, 1e-4), n=1000, box=(0.0, 1.0),
                      table=1e-4, parts=("forward",)),
    # training-step shape (config 2) at small N: forward, backward to table and positions, double backward
    "train_d3": dict(pos_dim=3, capacity=2 ** 18, nr_levels=24, sigma=(1.0, 1e-4), n=256, box=(0.0, 1.0),
                     table=1e-4, parts=("forward", "backward", "double")),
    # eikonal shape (config 3): points in [-1, 1)
    "sdf_d3": dict(pos_dim=3, capacity=2 ** 19, nr_levels=24, sigma=(1.0, 1e-4), n=256, box=(-1.0, 1.0),
                   table=1e-4, parts=("forward", "backward", "double")),
    # higher dimensions (config 4 shape) and the remaining supported dimensions
    "dim2": dict(pos_dim=2, capacity=2 ** 16, nr_levels=16, sigma=(1.0, 1e-3), n=256, box=(0.0, 1.0),
                 table=1.0, parts=("forward", "backward", "double")),
    "dim4": dict(pos_dim=4, capacity=2 ** 20, nr_levels=16, sigma=(1.0, 1e-3), n=256, box=(0.0, 1.0),
                 table=1.0, parts=("forward", "backward", "double")),
    "dim5": dict(pos_dim=5, capacity=2 ** 16, nr_levels=16, sigma=(1.0, 1e-3), n=256, box=(0.0, 1.0),
                 table=1.0, parts=("forward", "backward", "double")),
    "dim6": dict(pos_dim=6, capacity=2 ** 20, nr_levels=16, sigma=(1.0, 1e-3), n=256, box=(0.0, 1.0),
                 table=1.0, parts=("forward", "backward", "double")),
    "dim7": dict(pos_dim=7, capacity=2 ** 16, nr_levels=12, sigma=(1.0, 1e-2), n=256, box=(0.0, 1.0),
                 table=1.0, parts=("forward", "backward", "double")),
    # capacity that is not a power of two (the hash uses an unsigned modulo)
    "odd_capacity": dict(pos_dim=3, capacity=100003, nr_levels=10, sigma=(1.0, 1e-3), n=257, box=(0.0, 1.0),
                         table=1.0, parts=("forward", "backward", "double")),
    # raw points appended to the features
    "concat_d3": dict(pos_dim=3, capacity=2 ** 14, nr_levels=6, sigma=(1.0, 1e-2), n=65, box=(-1.0, 1.0),
                      table=1.0, concat=True, points_scaling=0.5, parts=("forward", "backward", "double")),
    # coarse-to-fine window partly open, level count not a multiple of 4
    "window_d3": dict(pos_dim=3, capacity=2 ** 14, nr_levels=10, sigma=(1.0, 1e-3), n=129, box=(0.0, 1.0),
                      table=1.0, window_t=0.45, parts=("forward", "backward", "double")),
    # a single point (ragged edge: one thread of one warp active)
    "single_point": dict(pos_dim=3, capacity=2 ** 12, nr_levels=4, sigma=(1.0, 1e-1), n=1, box=(0.0, 1.0),
                         table=1.0, parts=("forward", "backward", "double")),
}


def sigmas_of(case: dict) -> np.ndarray:
    hi, lo = case["sigma"]
    return np.geomspace(hi, lo, num=case["nr_levels"])  # float64, as the README passes it


def extra_levels(case: dict) -> int:
    feat = case.get("feat", 2)
    return (case["pos_dim"] + feat - 1) // feat if case.get("concat") else 0


def make_inputs(name: str) -> dict:
    """All input arrays of a case (float32 numpy)."""
    c = CASES[name]
    k = zlib.crc32(name.encode()) % 100000  # seed offset depends on the name only, not on the other cases
    d, cap, nl, n = c["pos_dim"], c["capacity"], c["nr_levels"], c["n"]
    feat = c.get("feat", 2)  # features per level; the reference (and every fixture) uses 2
    width = feat * (nl + extra_levels(c))
    lo, hi = c["box"]
    inputs = {
        "sigmas": sigmas_of(c),
        "table": uniform((nl, cap, feat), 1000000 + k, -c["table"], c["table"]),
        "shift": normal((nl, d), 2000000 + k, 10.0),
        "positions": uniform((n, d), 3000000 + k, lo, hi),
        "grad_out": normal((n, width), 4000000 + k, 1.0),
        "dpg": normal((n, d), 5000000 + k, 1.0),
        "anneal": cosine_window(nl, c["window_t"]) if "window_t" in c else np.ones(nl, np.float32),
    }
    return inputs
