"""ctypes binding of ``libpermuto_b200.so`` (the C ABI in ``include/permuto_b200.h``) and the
three objects the reference's autograd code talks to.

The reference reaches its kernels through a pybind11 module exposing ``EncodingInput``,
``EncodingFixedParams`` and ``EncodingWrapper`` (reference: src/PyBridge.cxx:13-45).  The same
three names live here with the same constructor arguments and method names, implemented on
top of the C ABI, so the autograd functions read like the reference's
(src/pytorch_modules/funcs.py:8-72).  One deliberate difference: features and their gradients
are ``[N, 2*(L+extra)]`` tensors already in the module's output order instead of
``[L+extra, 2, N]``, which removes the three transposing copies the reference pays per step.

There is no CPU implementation and no fallback: if the shared library is missing this module
raises at import time with the command that builds it.
"""
from __future__ import annotations

import ctypes as C
import os
import threading

import numpy as np
import torch

_PKG_DIR = os.path.dirname(os.path.abspath(__file__))
# PERMUTO_B200_LIB names another build of the same library (`python -m permutohedral_encoding_b200.build --out ...`)
LIB_PATH = os.environ.get("PERMUTO_B200_LIB") or os.path.join(_PKG_DIR, "libpermuto_b200.so")

ABI_VERSION = 2
PERMUTO_OK = 0
PERMUTO_TABLE_F32 = 0
PERMUTO_TABLE_F16 = 1
PERMUTO_ERR_INVALID_ARGUMENT = -1
PERMUTO_ERR_UNSUPPORTED = -2
PERMUTO_ERR_CUDA = -3
PERMUTO_ZERO_OUTPUTS = 1
PERMUTO_NO_AGGREGATE = 2
PERMUTO_KEEP_POSITIONS_GRAD = 4
PERMUTO_CONCAT_POSITIONS_GRAD = 8
PERMUTO_ACT = {"none": 0, "relu": 1, "gelu": 2}
PERMUTO_ADAM_SKIP_UNTOUCHED = 1
PERMUTO_ADAM_ZERO_GRAD = 2

EXPORTED_SYMBOLS = (
    "permuto_abi_version", "permuto_last_error", "permuto_extra_levels", "permuto_scale_factor",
    "permuto_forward", "permuto_backward", "permuto_double_backward", "permuto_debug_lattice",
    "permuto_probe_random_access", "permuto_adam_step", "permuto_forward_linear", "permuto_forward_mlp",
)


class PermutoConfig(C.Structure):
    _fields_ = [("pos_dim", C.c_int32), ("nr_feat_per_level", C.c_int32), ("nr_levels", C.c_int32),
                ("capacity", C.c_int32), ("concat_points", C.c_int32), ("points_scaling", C.c_float),
                ("levels_per_pass", C.c_int32), ("table_dtype", C.c_int32)]


class PermutoMlpLayer(C.Structure):
    _fields_ = [("weight", C.c_void_p), ("bias", C.c_void_p), ("in_features", C.c_int32), ("out_features", C.c_int32)]


class PermutoInputs(C.Structure):
    _fields_ = [("nr_positions", C.c_int64), ("positions", C.c_void_p), ("pos_stride_n", C.c_int64),
                ("pos_stride_d", C.c_int64), ("lattice_values", C.c_void_p), ("scale_factor", C.c_void_p),
                ("random_shift", C.c_void_p), ("anneal_window", C.c_void_p)]


def _load() -> C.CDLL:
    if not os.path.isfile(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: the CUDA extension has not been built. Build it with "
            "`python -m permutohedral_encoding_b200.build` (needs nvcc; no GPU required). "
            "There is no CPU fallback.")
    lib = C.CDLL(LIB_PATH)
    lib.permuto_abi_version.restype = C.c_int
    lib.permuto_last_error.restype = C.c_char_p
    lib.permuto_extra_levels.restype = C.c_int
    lib.permuto_extra_levels.argtypes = [C.c_int32, C.c_int32, C.c_int32]
    lib.permuto_scale_factor.restype = C.c_int
    lib.permuto_scale_factor.argtypes = [C.c_void_p, C.c_int32, C.c_int32, C.c_void_p]
    cfgp, inp = C.POINTER(PermutoConfig), C.POINTER(PermutoInputs)
    lib.permuto_forward.restype = C.c_int
    lib.permuto_forward.argtypes = [cfgp, inp, C.c_void_p, C.c_void_p]
    lib.permuto_backward.restype = C.c_int
    lib.permuto_backward.argtypes = [cfgp, inp, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int32, C.c_int32,
                                     C.c_uint32, C.c_void_p]
    lib.permuto_double_backward.restype = C.c_int
    lib.permuto_double_backward.argtypes = [cfgp, inp, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p,
                                            C.c_uint32, C.c_void_p]
    lib.permuto_debug_lattice.restype = C.c_int
    lib.permuto_debug_lattice.argtypes = [cfgp, inp, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]
    lib.permuto_probe_random_access.restype = C.c_int
    lib.permuto_probe_random_access.argtypes = [C.c_int32, C.c_void_p, C.c_int64, C.c_int32, C.POINTER(C.c_int64),
                                                C.c_void_p]
    lib.permuto_forward_linear.restype = C.c_int
    lib.permuto_forward_linear.argtypes = [cfgp, inp, C.c_void_p, C.c_void_p, C.c_int32, C.c_void_p, C.c_void_p, C.c_void_p]
    lib.permuto_forward_mlp.restype = C.c_int
    lib.permuto_forward_mlp.argtypes = [cfgp, inp, C.POINTER(PermutoMlpLayer), C.c_int32, C.c_int32, C.c_void_p, C.c_void_p,
                                        C.c_void_p]
    lib.permuto_adam_step.restype = C.c_int
    lib.permuto_adam_step.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_double, C.c_double,
                                      C.c_double, C.c_double, C.c_double, C.c_int64, C.c_uint32, C.c_void_p]
    if lib.permuto_abi_version() != ABI_VERSION:
        raise ImportError(f"{LIB_PATH}: ABI version {lib.permuto_abi_version()} != {ABI_VERSION}; rebuild the extension")
    return lib


lib = _load()


def last_error() -> str:
    return (lib.permuto_last_error() or b"").decode("utf-8", "replace")


def check(status: int) -> None:
    """Turn a C-ABI status into the exception the reference would have raised (its CHECK
    macros and std::runtime_error both surface as RuntimeError in Python)."""
    if status != PERMUTO_OK:
        raise RuntimeError(last_error() or f"permuto_b200 error {status}")


def scale_factor(sigmas, pos_dim: int) -> np.ndarray:
    s = np.ascontiguousarray(np.asarray(sigmas, dtype=np.float64))
    out = np.empty((s.shape[0], int(pos_dim)), dtype=np.float32)
    check(lib.permuto_scale_factor(s.ctypes.data, s.shape[0], int(pos_dim), out.ctypes.data))
    return out


def extra_levels(pos_dim: int, concat_points: bool, nr_feat_per_level: int = 2) -> int:
    return int(lib.permuto_extra_levels(int(pos_dim), int(nr_feat_per_level), int(bool(concat_points))))


def _ptr(t):
    # plain integers are accepted for the void* parameters (argtypes are declared)
    return None if t is None else t.data_ptr()


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream(device):
    """Handle of the current CUDA stream of ``device`` as an integer."""
    if _raw_stream is not None:
        return _raw_stream(device.index if device.index is not None else torch.cuda.current_device())
    return torch.cuda.current_stream(device).cuda_stream


class _NoGuard:
    def __enter__(self):
        return self

    def __exit__(self, *exc):
        return False


_NO_GUARD = _NoGuard()


def _guard(device):
    """Device guard that costs nothing when ``device`` is already current (the usual case; the
    small README-sized calls are dominated by host overhead)."""
    if device.index is None or device.index == torch.cuda.current_device():
        return _NO_GUARD
    return torch.cuda.device(device)


class EncodingInput:
    """Per-call bundle (reference: include/permutohedral_encoding/Encoding.cuh:14-29)."""

    def __init__(self, lattice_values, positions, anneal_window, require_lattice_values_grad,
                 require_positions_grad, lattice_values_half=None):
        self.m_lattice_values = lattice_values
        # optional fp16 copy of the values that the kernels gather from instead (storage only:
        # arithmetic and gradients stay fp32); no counterpart in the reference
        self.m_lattice_values_half = lattice_values_half
        self.m_positions_raw = positions
        self.m_anneal_window = anneal_window
        self.m_require_lattice_values_grad = bool(require_lattice_values_grad)
        self.m_require_positions_grad = bool(require_positions_grad)


class EncodingFixedParams:
    """Fixed description of an encoding (reference: Encoding.cuh:31-70).  Holds the shift
    tensor by handle, so loading a state dict into the module's parameter is seen by the
    kernels; the scale factor is computed once on the host with the reference's rounding and
    cached per device."""

    def __init__(self, pos_dim, capacity, nr_levels, nr_feat_per_level, sigmas_list, random_shift_per_level,
                 concat_points, points_scaling):
        self.m_pos_dim = int(pos_dim)
        self.m_capacity = int(capacity)
        self.m_nr_levels = int(nr_levels)
        self.m_nr_feat_per_level = int(nr_feat_per_level)
        self.m_sigmas_list = [float(s) for s in np.asarray(sigmas_list, dtype=np.float64).reshape(-1)]
        self.m_random_shift_per_level = random_shift_per_level
        self.m_concat_points = bool(concat_points)
        self.m_points_scaling = float(points_scaling)
        if len(self.m_sigmas_list) != self.m_nr_levels:
            raise RuntimeError(f"scale list has {len(self.m_sigmas_list)} entries for {self.m_nr_levels} levels")
        if not (2 <= self.m_pos_dim <= 7):
            raise RuntimeError("Encoding: pos_dim must be 2,3,4,5,6 or 7")
        self.m_scale_factor_host = torch.from_numpy(scale_factor(self.m_sigmas_list, self.m_pos_dim))
        self._scale_by_device = {}
        self.levels_per_pass = 0  # scheduling hint of the kernels (0 = automatic; results never depend on it)

    def scale_factor_on(self, device) -> torch.Tensor:
        device = torch.device(device)
        t = self._scale_by_device.get(device)
        if t is None:
            t = self.m_scale_factor_host.to(device)
            self._scale_by_device[device] = t
        return t

    def config(self, table_half: bool = False) -> PermutoConfig:
        key = "_cfg_f16" if table_half else "_cfg_f32"
        cached = self.__dict__.get(key)
        if cached is None or cached.levels_per_pass != int(self.levels_per_pass):
            cached = PermutoConfig(self.m_pos_dim, self.m_nr_feat_per_level, self.m_nr_levels, self.m_capacity,
                                   int(self.m_concat_points), self.m_points_scaling, int(self.levels_per_pass),
                                   PERMUTO_TABLE_F16 if table_half else PERMUTO_TABLE_F32)
            self.__dict__[key] = cached
        return cached


class EncodingWrapper:
    """Type-erased encoding (reference: Encoding.cuh:159-188; launchers src/Encoding.cu:54-334)."""

    def __init__(self, pos_dim, nr_feat_per_level, fixed_params: EncodingFixedParams):
        if int(pos_dim) not in (2, 3, 4, 5, 6, 7):
            raise RuntimeError("Encoding: pos_dim must be 2,3,4,5,6 or 7")
        if int(nr_feat_per_level) not in (2, 4, 8):
            raise RuntimeError("Encoding: nr_feat_per_level must be 2, 4 or 8")
        self.fixed = fixed_params
        self.aggregate_collisions = True
        # The reference gives the positions no gradient through the concatenated raw points
        # (its backward skips those columns); True adds that term.
        self.concat_positions_grad = False
        self._tls = threading.local()      # per-thread memo of the validated static inputs
        self.backward_hook = None          # set by distributed.LatticeGradAllReduce
        self.double_backward_hook = None
        self._feat = int(nr_feat_per_level)
        self._width = self._feat * (fixed_params.m_nr_levels + extra_levels(
            fixed_params.m_pos_dim, fixed_params.m_concat_points, self._feat))

    @staticmethod
    def create(pos_dim, nr_feat_per_level, fixed_params) -> "EncodingWrapper":
        return EncodingWrapper(pos_dim, nr_feat_per_level, fixed_params)

    # -- validation mirroring src/Encoding.cu:37-45, :63-66, :119-125 ---------------------------
    # Split in two: the positions change with every call and are always checked; the lattice
    # values, shift and window usually are the same tensors call after call, so their checks and
    # the C struct built from them are remembered (per thread) until one of them is another tensor
    # or points at other memory.  README-sized batches are dominated by this host work.
    def _check_positions(self, pos):
        fp = self.fixed
        if not pos.is_cuda:
            raise RuntimeError("positions should be in GPU memory. Please call .cuda() on the tensor")
        if pos.dtype != torch.float32:
            raise RuntimeError("positions should be of type float")
        if pos.dim() != 2:
            raise RuntimeError(f"positions should have dim 2 correspondin to HW. However it has sizes {tuple(pos.shape)}")
        if pos.shape[0] == 0:
            raise RuntimeError("Why do we have 0 points")
        if pos.shape[1] != fp.m_pos_dim:
            raise RuntimeError("Pos dim for the lattice doesn't correspond with the position of the points. "
                               f"Lattice was initialized with {fp.m_pos_dim} and points have pos dim {pos.shape[1]}")

    def _check_static(self, inp: EncodingInput, device):
        fp = self.fixed
        lv, aw, shift = inp.m_lattice_values, inp.m_anneal_window, fp.m_random_shift_per_level
        if lv.dim() != 3 or tuple(lv.shape) != (fp.m_nr_levels, fp.m_capacity, self._feat):
            raise RuntimeError(f"lattice_values should be nr_levels x capacity x {self._feat}, got {tuple(lv.shape)}")
        if not lv.is_contiguous():
            raise RuntimeError("We assume that the lattice_values_monolithic are contiguous because in the cuda "
                               "code we make a load of 2 float values at a time")
        if lv.dtype not in (torch.float32, torch.float16) or lv.device != device:
            raise RuntimeError("lattice_values should be float32 (or float16 storage) on the device of the positions")
        half = inp.m_lattice_values_half
        if half is not None and (half.dtype != torch.float16 or half.shape != lv.shape or half.device != lv.device
                                 or not half.is_contiguous()):
            raise RuntimeError("lattice_values_half should be a contiguous float16 tensor of the shape and device "
                               "of lattice_values")
        if tuple(shift.shape) != (fp.m_nr_levels, fp.m_pos_dim):
            raise RuntimeError("Random shift should be nr of resolutions x pos dim")
        if aw.dim() != 1 or aw.shape[0] != fp.m_nr_levels:
            raise RuntimeError("anneal_window should have the first dimension the same as the nr of resolutions")

    def _check(self, inp: EncodingInput):
        """All of the reference's checks on one input bundle."""
        self._check_positions(inp.m_positions_raw)
        self._check_static(inp, inp.m_positions_raw.device)

    def _inputs(self, inp: EncodingInput):
        """Validated ``permuto_inputs`` struct for this call (and the tensors it points into, to be
        kept alive by the caller until the launch has been enqueued)."""
        pos = inp.m_positions_raw
        self._check_positions(pos)
        dev = pos.device
        table = self._table(inp)
        aw, shift = inp.m_anneal_window, self.fixed.m_random_shift_per_level
        memo = self._tls.__dict__.get("static")
        if (memo is not None and memo[0] is table and memo[1] is aw and memo[2] is shift and memo[3] is inp.m_lattice_values
                and memo[4] == dev and memo[5] == table.data_ptr() and memo[6] == aw.data_ptr()
                and memo[7] == shift.data_ptr()):
            ins, keep = memo[8], memo[9]
        else:
            self._check_static(inp, dev)
            ready = True   # no converted copies were needed: safe to remember
            shift_d, aw_d = shift, aw
            if shift.device != dev or shift.dtype != torch.float32 or not shift.is_contiguous():
                shift_d, ready = shift.detach().to(device=dev, dtype=torch.float32).contiguous(), False
            if aw.device != dev or aw.dtype != torch.float32 or not aw.is_contiguous():
                aw_d, ready = aw.detach().to(device=dev, dtype=torch.float32).contiguous(), False
            scale = self.fixed.scale_factor_on(dev)
            keep = (shift_d, aw_d, scale, table)
            ins = PermutoInputs(0, 0, 0, 0, table.data_ptr(), scale.data_ptr(), shift_d.data_ptr(), aw_d.data_ptr())
            self._tls.static = (table, aw, shift, inp.m_lattice_values, dev, table.data_ptr(), aw.data_ptr(),
                                shift.data_ptr(), ins, keep) if ready else None
        ins.nr_positions = pos.shape[0]
        ins.positions = pos.data_ptr()
        ins.pos_stride_n = pos.stride(0)
        ins.pos_stride_d = pos.stride(1)
        return ins, keep

    @staticmethod
    def _table(inp: EncodingInput) -> torch.Tensor:
        """The tensor the kernels gather from: the fp16 copy when one is attached."""
        return inp.m_lattice_values_half if inp.m_lattice_values_half is not None else inp.m_lattice_values

    def _config(self, inp: EncodingInput) -> PermutoConfig:
        return self.fixed.config(self._table(inp).dtype == torch.float16)

    def output_width(self) -> int:
        return self._width

    def _flags(self, zero=True) -> int:
        f = PERMUTO_ZERO_OUTPUTS if zero else 0
        if not self.aggregate_collisions:
            f |= PERMUTO_NO_AGGREGATE
        if self.concat_positions_grad:
            f |= PERMUTO_CONCAT_POSITIONS_GRAD
        return f

    # -- the three operations -------------------------------------------------------------------
    def forward(self, inp: EncodingInput) -> torch.Tensor:
        """features [N, 2*(L+extra)] (reference: Encoding<P,2>::forward + modules.py:87)."""
        pos = inp.m_positions_raw
        with _guard(pos.device):
            ins, keep = self._inputs(inp)   # validates
            cfg = self._config(inp)
            out = torch.empty((pos.shape[0], self._width), dtype=torch.float32, device=pos.device)
            check(lib.permuto_forward(C.byref(cfg), C.byref(ins), out.data_ptr(), _stream(pos.device)))
        return out

    def forward_linear(self, inp: EncodingInput, weight: torch.Tensor, bias=None, status=None) -> torch.Tensor:
        """``features @ weight.T + bias`` as ``[N, out_features]`` without materialising the features
        (tensor cores, operands rounded to tf32, fp32 accumulation).  ``weight`` is
        ``[out_features, output_width]`` like ``torch.nn.Linear.weight``; ``status`` is an optional
        int32 CUDA tensor of one element that the kernel sets non-zero if its bounded wait for the
        tensor core ran out.  No gradients.  The reference has no counterpart (its users run the
        module followed by ``torch.nn.Linear``: examples/train_toy_example.py:18-26)."""
        self._check(inp)
        pos = inp.m_positions_raw
        dev = pos.device
        if weight.dim() != 2 or weight.shape[1] != self.output_width():
            raise RuntimeError(f"weight should be out_features x {self.output_width()}, got {tuple(weight.shape)}")
        h = int(weight.shape[0])
        if h % 16 != 0 or not (16 <= h <= 256):
            raise RuntimeError(f"out_features must be a multiple of 16 in 16..256 (got {h})")
        weight = weight.detach()
        if weight.device != dev or weight.dtype != torch.float32 or not weight.is_contiguous():
            weight = weight.to(device=dev, dtype=torch.float32).contiguous()
        if bias is not None:
            bias = bias.detach()
            if tuple(bias.shape) != (h,):
                raise RuntimeError(f"bias should have {h} entries")
            if bias.device != dev or bias.dtype != torch.float32 or not bias.is_contiguous():
                bias = bias.to(device=dev, dtype=torch.float32).contiguous()
        if status is not None and (status.dtype != torch.int32 or status.device != dev or status.numel() != 1):
            raise RuntimeError("status should be a one-element int32 tensor on the device of the positions")
        cfg = self._config(inp)
        out = torch.empty((pos.shape[0], h), dtype=torch.float32, device=dev)
        with _guard(dev):
            ins, keep = self._inputs(inp)
            check(lib.permuto_forward_linear(C.byref(cfg), C.byref(ins), _ptr(weight), _ptr(bias), h, _ptr(out),
                                             _ptr(status), _stream(dev)))
        return out

    def forward_mlp(self, inp: EncodingInput, layers, activation: str = "gelu", status=None) -> torch.Tensor:
        """The encoding followed by a whole small MLP in one kernel: ``layers`` is a sequence of
        ``(weight [out, in], bias [out] | None)`` pairs, ``activation`` ("none", "relu", "gelu")
        is applied after every layer but the last.  Neither the features nor the hidden
        activations reach memory; layers whose width is a multiple of 16 run on the tensor cores
        (tf32 operands, fp32 accumulation), a narrower last layer as fp32 dot products.  Hidden
        widths: multiples of 16 up to 64.  No gradients.  The reference's toy example network
        (examples/train_toy_example.py:18-26) is the model case."""
        pos = inp.m_positions_raw
        dev = pos.device
        if activation not in PERMUTO_ACT:
            raise RuntimeError(f"activation must be one of {sorted(PERMUTO_ACT)}, got {activation!r}")
        layers = list(layers)
        if not 1 <= len(layers) <= 6:
            raise RuntimeError(f"the fused network takes 1..6 layers, got {len(layers)}")
        descr = (PermutoMlpLayer * len(layers))()
        keep_alive = []
        width = self.output_width()
        for i, (weight, bias) in enumerate(layers):
            if weight.dim() != 2 or weight.shape[1] != width:
                raise RuntimeError(f"layer {i}: weight should be out_features x {width}, got {tuple(weight.shape)}")
            weight = weight.detach()
            if weight.device != dev or weight.dtype != torch.float32 or not weight.is_contiguous():
                weight = weight.to(device=dev, dtype=torch.float32).contiguous()
            if bias is not None:
                bias = bias.detach()
                if tuple(bias.shape) != (weight.shape[0],):
                    raise RuntimeError(f"layer {i}: bias should have {weight.shape[0]} entries")
                if bias.device != dev or bias.dtype != torch.float32 or not bias.is_contiguous():
                    bias = bias.to(device=dev, dtype=torch.float32).contiguous()
            keep_alive += [weight, bias]
            descr[i] = PermutoMlpLayer(weight.data_ptr(), _ptr(bias), int(weight.shape[1]), int(weight.shape[0]))
            width = int(weight.shape[0])
        if status is not None and (status.dtype != torch.int32 or status.device != dev or status.numel() != 1):
            raise RuntimeError("status should be a one-element int32 tensor on the device of the positions")
        with _guard(dev):
            ins, keep = self._inputs(inp)   # validates
            cfg = self._config(inp)
            out = torch.empty((pos.shape[0], width), dtype=torch.float32, device=dev)
            check(lib.permuto_forward_mlp(C.byref(cfg), C.byref(ins), descr, len(layers), PERMUTO_ACT[activation],
                                          out.data_ptr(), _ptr(status), _stream(dev)))
        return out

    def backward(self, inp: EncodingInput, grad_features: torch.Tensor, lattice_grad_out=None,
                 level_begin=None, level_end=None, zero=True, positions_grad_out=None):
        """(lattice_values_grad [L,C,2] | None, positions_grad [N,d] | None)
        (reference: Encoding<P,2>::backward).  ``lattice_grad_out`` lets the caller provide the
        buffer; ``level_begin/level_end`` restrict the levels (bucketed all-reduce overlap);
        ``positions_grad_out`` is an existing position gradient to keep accumulating into;
        ``zero=False`` accumulates onto a lattice gradient the caller has cleared itself."""
        self._check(inp)
        fp = self.fixed
        pos = inp.m_positions_raw
        n = pos.shape[0]
        if grad_features.dim() != 2 or tuple(grad_features.shape) != (n, self.output_width()):
            raise RuntimeError("The nr of positions should match between the input positions and the sliced values: "
                               f"expected {(n, self.output_width())}, got {tuple(grad_features.shape)}")
        if not grad_features.is_contiguous():
            raise RuntimeError("Grad sliced values needs to be contiguous. Please call .contiguous() on it")
        cfg = self._config(inp)
        lv_grad = None
        if inp.m_require_lattice_values_grad:  # always fp32, whatever the storage type of the values
            lv_grad = lattice_grad_out if lattice_grad_out is not None else \
                torch.empty(inp.m_lattice_values.shape, dtype=torch.float32, device=pos.device)
        pos_grad = None
        flags = self._flags(zero)
        if inp.m_require_positions_grad:
            if positions_grad_out is not None:
                pos_grad = positions_grad_out
                flags |= PERMUTO_KEEP_POSITIONS_GRAD
            else:
                make = torch.empty if zero else torch.zeros  # without ZERO_OUTPUTS nothing clears it natively
                pos_grad = make((n, fp.m_pos_dim), dtype=torch.float32, device=pos.device)
        lb = 0 if level_begin is None else int(level_begin)
        le = fp.m_nr_levels if level_end is None else int(level_end)
        with _guard(pos.device):
            ins, keep = self._inputs(inp)
            check(lib.permuto_backward(C.byref(cfg), C.byref(ins), _ptr(grad_features), _ptr(lv_grad), _ptr(pos_grad),
                                       lb, le, flags, _stream(pos.device)))
        return lv_grad, pos_grad

    def double_backward_from_positions(self, inp: EncodingInput, double_positions_grad: torch.Tensor,
                                       grad_features: torch.Tensor, need_lattice_grad=True,
                                       need_grad_grad_features=True):
        """(lattice_values_grad [L,C,2], grad_grad_features [N,W])
        (reference: Encoding<P,2>::double_backward_from_positions)."""
        self._check(inp)
        fp = self.fixed
        pos = inp.m_positions_raw
        n = pos.shape[0]
        if tuple(double_positions_grad.shape) != (n, fp.m_pos_dim):
            raise RuntimeError("double_positions_grad should be nr_positions x pos_dim")
        if tuple(grad_features.shape) != (n, self.output_width()):
            raise RuntimeError("The nr of positions should match between the input positions and the sliced values")
        dpg = double_positions_grad.contiguous()
        gf = grad_features.contiguous()
        cfg = self._config(inp)
        lv_grad = torch.empty(inp.m_lattice_values.shape, dtype=torch.float32, device=pos.device) \
            if need_lattice_grad else None
        ggf = torch.empty_like(gf) if need_grad_grad_features else None
        with _guard(pos.device):
            ins, keep = self._inputs(inp)
            check(lib.permuto_double_backward(C.byref(cfg), C.byref(ins), _ptr(dpg), _ptr(gf), _ptr(lv_grad),
                                              _ptr(ggf), self._flags(True), _stream(pos.device)))
        return lv_grad, ggf

    def debug_lattice(self, inp: EncodingInput, want=("keys", "slots", "bary", "rank")):
        """Lattice keys / hash slots / barycentric weights / ranks per (point, level, vertex)."""
        self._check(inp)
        fp = self.fixed
        pos = inp.m_positions_raw
        n, d, nl = pos.shape[0], fp.m_pos_dim, fp.m_nr_levels
        dev = pos.device
        keys = torch.empty((n, nl, d + 1, d), dtype=torch.int32, device=dev) if "keys" in want else None
        slots = torch.empty((n, nl, d + 1), dtype=torch.int32, device=dev) if "slots" in want else None
        bary = torch.empty((n, nl, d + 1), dtype=torch.float32, device=dev) if "bary" in want else None
        rank = torch.empty((n, nl, d + 1), dtype=torch.int32, device=dev) if "rank" in want else None
        cfg = self._config(inp)
        with _guard(dev):
            ins, keep = self._inputs(inp)
            check(lib.permuto_debug_lattice(C.byref(cfg), C.byref(ins), _ptr(keys), _ptr(slots), _ptr(bary),
                                            _ptr(rank), _stream(dev)))
        return {"keys": keys, "slots": slots, "bary": bary, "rank": rank}
