"""Driver for the reference's own CUDA extension, rebuilt for sm_100 by ``build_ref.py``.

TEST INFRASTRUCTURE ONLY (golden-vector generation, differential GPU tests, the benchmark's
reference arm).  Never imported by the product package.

The extension (``oracle/_ref/permuto_ref_C.so``) is the reference's unmodified
``src/Encoding.cu`` + ``src/PyBridge.cxx``.  This shim calls it in the order the reference's
Python does (src/pytorch_modules/funcs.py:8-72, modules.py:65-93): forward -> permute/reshape
copy; backward -> ``.contiguous()`` of the upstream gradient -> native backward returning
permuted views; double backward from the position gradient.  The reference's Python package
itself cannot be imported on a Blackwell GPU (its extension finder stops at compute capability
90, src/pytorch_modules/find_cpp_package.py:7), which is the only reason this driver exists.
The reference pins every allocation to cuda:0.
"""
from __future__ import annotations

import importlib
import os
import sys

import torch

_REF_DIR = os.path.join(os.path.dirname(os.path.abspath(__file__)), "_ref")
_C = None


def available() -> bool:
    return os.path.isfile(os.path.join(_REF_DIR, "permuto_ref_C.so"))


def ext():
    global _C
    if _C is None:
        if not available():
            raise RuntimeError("oracle/_ref/permuto_ref_C.so not built (run oracle/build_ref.py where the "
                               "reference sources are present)")
        if _REF_DIR not in sys.path:
            sys.path.insert(0, _REF_DIR)
        _C = importlib.import_module("permuto_ref_C")
    return _C


class _Slice(torch.autograd.Function):
    @staticmethod
    def forward(ctx, enc, values, positions, window, need_values_grad, need_pos_grad):
        bundle = ext().EncodingInput(values, positions, window, need_values_grad, need_pos_grad)
        out = enc.native.forward(bundle)  # [L+extra, 2, N]
        ctx.enc, ctx.bundle = enc, bundle
        ctx.save_for_backward(out)
        return out

    @staticmethod
    def backward(ctx, g):
        b = ctx.bundle
        assert b.m_require_lattice_values_grad or b.m_require_positions_grad
        return _SliceBack.apply(ctx.enc, b, g, b.m_lattice_values, b.m_positions_raw, ctx.saved_tensors[0])


class _SliceBack(torch.autograd.Function):
    @staticmethod
    def forward(ctx, enc, bundle, g, values, positions, sliced):
        gv = gp = None
        if bundle.m_require_lattice_values_grad or bundle.m_require_positions_grad:
            g = g.contiguous()
            ctx.save_for_backward(g)
            ctx.enc, ctx.bundle = enc, bundle
            gv, gp = enc.native.backward(bundle, g)
        return None, gv, gp, None, None, None

    @staticmethod
    def backward(ctx, _a, _gg_values, gg_pos, _b, _c, _d):
        (g,) = ctx.saved_tensors
        gv, ggs = ctx.enc.native.double_backward_from_positions(ctx.bundle, gg_pos, g)
        return (None, None, ggs, gv) + (None,) * 10


class RefEncoding:
    """The reference encoding behind its native API, with explicit tensors (no nn.Module)."""

    def __init__(self, pos_dim, capacity, nr_levels, sigmas, shift, concat_points=False, points_scaling=1.0):
        c = ext()
        self.pos_dim, self.capacity, self.nr_levels = pos_dim, capacity, nr_levels
        self.shift = shift  # cuda fp32 [L, d]; captured by handle like the reference module does
        self.fixed = c.EncodingFixedParams(pos_dim, capacity, nr_levels, 2, [float(s) for s in sigmas], shift,
                                           bool(concat_points), float(points_scaling))
        self.native = c.EncodingWrapper.create(pos_dim, 2, self.fixed)

    # module-level path, as a user of the reference runs it (modules.py:65-93)
    def __call__(self, values, positions, window):
        need_v = values.requires_grad and torch.is_grad_enabled()
        need_p = positions.requires_grad and torch.is_grad_enabled()
        out = _Slice.apply(self, values, positions, window, need_v, need_p)
        return out.permute(2, 0, 1).reshape(positions.shape[0], -1)

    # raw native calls (kernel-only timing, golden vectors)
    def forward_raw(self, values, positions, window, need_v=False, need_p=False):
        return self.native.forward(ext().EncodingInput(values, positions, window, need_v, need_p))

    def backward_raw(self, values, positions, window, g_lfn, need_v=True, need_p=False):
        return self.native.backward(ext().EncodingInput(values, positions, window, need_v, need_p), g_lfn)

    def double_backward_raw(self, values, positions, window, gg_pos, g_lfn):
        return self.native.double_backward_from_positions(
            ext().EncodingInput(values, positions, window, True, True), gg_pos, g_lfn)


def aten_scale_factor(sigmas, pos_dim, device="cuda"):
    """The op sequence of EncodingFixedParams::compute_scale_factor_tensor
    (include/permutohedral_encoding/Encoding.cuh:55-69) replayed with the same ATen operators:
    a binary64 scalar stored into a binary32 CUDA tensor element, then the element divided by
    the binary32-rounded sigma as a host scalar."""
    import math

    import numpy as np

    t = torch.zeros((len(sigmas), pos_dim), dtype=torch.float32, device=device)
    for l, s in enumerate(sigmas):
        s32 = float(np.float32(s))
        for i in range(pos_dim):
            t[l][i] = 1.0 / math.sqrt(float((i + 1) * (i + 2))) * 1.0
            t[l][i] = t[l][i] / s32
    return t
