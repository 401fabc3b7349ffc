"""numpy front end of the C restatement in ``permuto_oracle.c`` (ctypes).

TEST INFRASTRUCTURE ONLY: imported by the tests, the smoke check and the benchmark's CPU
baseline leg, never by the product package.

All arrays are float32 / int32 C-contiguous numpy arrays.  Layouts:
positions [N,d]; table [L,C,2]; scale, shift [L,d]; anneal [L];
features / upstream gradient [N,(L+extra)*2] with column = level*2 + feature
(the reference module's output ordering, src/pytorch_modules/modules.py:87).
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SRC = os.path.join(_HERE, "permuto_oracle.c")
_SO = os.path.join(_HERE, "libpermuto_oracle.so")

_f32p = C.POINTER(C.c_float)
_i32p = C.POINTER(C.c_int32)
_f64p = C.POINTER(C.c_double)


def build(force: bool = False) -> str:
    """gcc -O2 -ffp-contract=off -fopenmp; contraction is off so that only the explicit
    fmaf() calls fuse (they restate nvcc's contraction of the reference source)."""
    if force or not os.path.isfile(_SO) or os.path.getmtime(_SO) < os.path.getmtime(_SRC):
        cmd = ["gcc", "-O2", "-std=c11", "-ffp-contract=off", "-fno-fast-math", "-fopenmp",
               "-shared", "-fPIC", _SRC, "-o", _SO, "-lm"]
        subprocess.run(cmd, check=True)
    return _SO


_lib = None


def lib():
    global _lib
    if _lib is None:
        _lib = C.CDLL(build())
        _lib.permuto_oracle_extra_levels.restype = C.c_int
        _lib.permuto_oracle_max_threads.restype = C.c_int
    return _lib


def _f(a):
    a = np.ascontiguousarray(a, dtype=np.float32)
    return a, a.ctypes.data_as(_f32p)


def _opt(a, ptype):
    return a.ctypes.data_as(ptype) if a is not None else ptype()


def set_modes(fma_elevate: bool = True, scale_by_reciprocal: bool = True) -> None:
    lib().permuto_oracle_set_modes(int(fma_elevate), int(scale_by_reciprocal))


def set_threads(n: int) -> None:
    lib().permuto_oracle_set_threads(int(n))


def max_threads() -> int:
    return int(lib().permuto_oracle_max_threads())


def extra_levels(pos_dim: int, concat_points: bool, nr_feat: int = 2) -> int:
    lib().permuto_oracle_set_nfeat(int(nr_feat))
    return int(lib().permuto_oracle_extra_levels(int(pos_dim), int(bool(concat_points))))


def scale_factor(sigmas, pos_dim: int) -> np.ndarray:
    s = np.ascontiguousarray(sigmas, dtype=np.float64)
    out = np.empty((s.shape[0], pos_dim), dtype=np.float32)
    lib().permuto_oracle_scale_factor(s.ctypes.data_as(_f64p), C.c_int(s.shape[0]),
                                      C.c_int(pos_dim), out.ctypes.data_as(_f32p))
    return out


def _common(positions, table, scale, shift, anneal):
    positions, pp = _f(positions)
    table, tp = _f(table)
    scale, sp = _f(scale)
    shift, hp = _f(shift)
    anneal, ap = _f(anneal)
    n, d = positions.shape
    nl, cap, nf = table.shape
    assert nf in (2, 4, 8) and scale.shape == (nl, d) and shift.shape == (nl, d) and anneal.shape == (nl,)
    lib().permuto_oracle_set_nfeat(int(nf))
    keep = (positions, table, scale, shift, anneal)
    return keep, (n, d, nl, cap, nf), (pp, tp, sp, hp, ap)


def lattice(positions, scale, shift, capacity: int, want=("keys", "slots", "bary", "rank")):
    positions, pp = _f(positions)
    scale, sp = _f(scale)
    shift, hp = _f(shift)
    n, d = positions.shape
    nl = scale.shape[0]
    v = d + 1
    keys = np.empty((n, nl, v, d), np.int32) if "keys" in want else None
    slots = np.empty((n, nl, v), np.int32) if "slots" in want else None
    bary = np.empty((n, nl, v), np.float32) if "bary" in want else None
    rank = np.empty((n, nl, v), np.int32) if "rank" in want else None
    lib().permuto_oracle_lattice(C.c_int(d), C.c_int(nl), C.c_int(capacity), C.c_int64(n),
                                 pp, sp, hp, _opt(keys, _i32p), _opt(slots, _i32p),
                                 _opt(bary, _f32p), _opt(rank, _i32p))
    return {"keys": keys, "slots": slots, "bary": bary, "rank": rank}


def forward(positions, table, scale, shift, anneal, concat_points=False, points_scaling=1.0):
    keep, (n, d, nl, cap, nf), (pp, tp, sp, hp, ap) = _common(positions, table, scale, shift, anneal)
    extra = extra_levels(d, concat_points, nf)
    out = np.empty((n, (nl + extra) * nf), np.float32)
    lib().permuto_oracle_forward(C.c_int(d), C.c_int(nl), C.c_int(cap), C.c_int64(n), pp, tp, sp,
                                 hp, ap, C.c_int(int(concat_points)), C.c_float(points_scaling),
                                 out.ctypes.data_as(_f32p))
    return out


def backward(positions, table, scale, shift, anneal, grad_out, concat_points=False,
             need_table=True, need_pos=False, need_abs=False):
    keep, (n, d, nl, cap, nf), (pp, tp, sp, hp, ap) = _common(positions, table, scale, shift, anneal)
    extra = extra_levels(d, concat_points, nf)
    grad_out, gp = _f(grad_out)
    assert grad_out.shape == (n, (nl + extra) * nf)
    tg = np.empty((nl, cap, nf), np.float32) if need_table else None
    ta = np.empty((nl, cap, nf), np.float32) if (need_table and need_abs) else None
    pg = np.empty((n, d), np.float32) if need_pos else None
    lib().permuto_oracle_backward(C.c_int(d), C.c_int(nl), C.c_int(cap), C.c_int64(n), pp, tp, sp,
                                  hp, ap, C.c_int(int(concat_points)), gp, _opt(tg, _f32p),
                                  _opt(ta, _f32p), _opt(pg, _f32p))
    return {"table_grad": tg, "table_abs": ta, "pos_grad": pg}


def double_backward(positions, table, scale, shift, anneal, dpg, grad_out, concat_points=False,
                    need_table=True, need_ggo=True, need_abs=False):
    keep, (n, d, nl, cap, nf), (pp, tp, sp, hp, ap) = _common(positions, table, scale, shift, anneal)
    extra = extra_levels(d, concat_points, nf)
    grad_out, gp = _f(grad_out)
    dpg, dp = _f(dpg)
    assert grad_out.shape == (n, (nl + extra) * nf) and dpg.shape == (n, d)
    tg = np.empty((nl, cap, nf), np.float32) if need_table else None
    ta = np.empty((nl, cap, nf), np.float32) if (need_table and need_abs) else None
    gg = np.empty((n, (nl + extra) * nf), np.float32) if need_ggo else None
    lib().permuto_oracle_double_backward(C.c_int(d), C.c_int(nl), C.c_int(cap), C.c_int64(n), pp,
                                         tp, sp, hp, ap, C.c_int(int(concat_points)), dp, gp,
                                         _opt(tg, _f32p), _opt(ta, _f32p), _opt(gg, _f32p))
    return {"table_grad": tg, "table_abs": ta, "grad_grad_out": gg}
