"""``PermutoEncoding`` and ``Coarse2Fine`` with the reference's constructor arguments,
parameter names, defaults and output ordering (reference: src/pytorch_modules/modules.py)."""
import math

import torch

from . import _native as _C
from .funcs import PermutoEncodingFunc
from .utils import cosine_easing_window


class PermutoEncoding(torch.nn.Module):
    """Multi-resolution permutohedral-lattice hash encoding.

    ``forward(positions[N, pos_dim]) -> [N, nr_feat_per_level * (nr_levels + extra)]``, level-major
    then feature (reference: modules.py:65-93).  Parameters, as in the reference so that its
    checkpoints load unchanged: ``lattice_values`` fp32 ``[nr_levels, capacity, nr_feat_per_level]``
    and ``random_shift_per_level`` fp32 ``[nr_levels, pos_dim]`` (never receives a gradient).
    One exception: with ``appply_random_shift_per_level=False`` the reference stores a 1-element
    shift; such a checkpoint entry is accepted and read as the zero shift.
    The misspelt keyword ``appply_random_shift_per_level`` is part of the reference's public
    surface and is kept.  With ``appply_random_shift_per_level=False`` the reference creates an
    unusable 1-element shift (modules.py:34 fails the native shape checks); here the shift is
    a zero ``[nr_levels, pos_dim]`` tensor, which is what the flag means.
    ``nr_feat_per_level`` may be 2 (the only width the reference implements), 4 or 8: a table
    access moves a 32-byte sector whatever it uses of it (16-byte random gathers run at three
    quarters of the rate of 8-byte ones, 16-byte reductions at the same rate), so e.g. 12 levels
    of 4 features produce 48 outputs in 60 % of the time of 24 x 2.
    ``concat_points_grad=True`` completes the position gradient of ``concat_points``: the
    reference (and the default here) gives the positions no gradient through the concatenated raw
    coordinates, because its backward skips those columns (src/Encoding.cu:129-134).
    ``half_precision_table=True`` (not in the reference, which only hints at it,
    kernels/permutohedral_encoding/EncodingGPU.cuh:12) makes the kernels gather from an fp16 copy
    of ``lattice_values``: storage only -- products, sums, outputs, the parameter, its gradient
    and the optimizer state stay fp32 -- so the table takes half the room in L2 and a 4-feature
    entry is the 8 bytes a 2-feature fp32 entry is.
    """

    def __init__(self, pos_dim, capacity, nr_levels, nr_feat_per_level, scale_per_level,
                 appply_random_shift_per_level=True, concat_points=False, concat_points_scaling=1.0,
                 half_precision_table=False, concat_points_grad=False):
        super().__init__()
        self.concat_points_grad = bool(concat_points_grad)
        self.half_precision_table = bool(half_precision_table)
        self._half, self._half_version, self._half_ptr = None, -1, 0
        self.pos_dim = pos_dim
        self.capacity = capacity
        self.nr_levels = nr_levels
        self.nr_feat_per_level = nr_feat_per_level
        self.scale_per_level = scale_per_level
        self.appply_random_shift_per_level = appply_random_shift_per_level
        self.concat_points = concat_points
        self.concat_points_scaling = concat_points_scaling

        # same draws as the reference (modules.py:25-32): randn(C, L, F) permuted to [L, C, F]
        lattice_values = torch.randn(capacity, nr_levels, nr_feat_per_level) * 1e-5
        lattice_values = lattice_values.permute(1, 0, 2).contiguous()
        self.lattice_values = torch.nn.Parameter(lattice_values.cuda())
        if appply_random_shift_per_level:
            random_shift_per_level = torch.randn(nr_levels, pos_dim) * 10
        else:
            random_shift_per_level = torch.zeros(nr_levels, pos_dim)
        self.random_shift_per_level = torch.nn.Parameter(random_shift_per_level.cuda())

        self.anneal_window = torch.ones((nr_levels)).cuda()
        self.fixed_params, self.lattice = self._make_lattice_wrapper()

    def _make_lattice_wrapper(self):
        fixed_params = _C.EncodingFixedParams(self.pos_dim, self.capacity, self.nr_levels, self.nr_feat_per_level,
                                              self.scale_per_level, self.random_shift_per_level, self.concat_points,
                                              self.concat_points_scaling)
        lattice = _C.EncodingWrapper.create(self.pos_dim, self.nr_feat_per_level, fixed_params)
        lattice.concat_positions_grad = bool(getattr(self, "concat_points_grad", False))
        return fixed_params, lattice

    def __getstate__(self):
        state = self.__dict__.copy()
        del state["fixed_params"]  # native-side objects are rebuilt, not pickled
        del state["lattice"]
        state["_half"], state["_half_version"], state["_half_ptr"] = None, -1, 0  # the fp16 copy is rebuilt on first use
        return state

    def __setstate__(self, state):
        self.__dict__.update(state)
        self.fixed_params, self.lattice = self._make_lattice_wrapper()

    def _apply(self, fn, *args, **kwargs):
        # .to()/.cuda() may replace the parameter objects: re-bind the shift handle.  The kernels
        # compute in fp32 only, so a dtype conversion (.half(), .double()) is refused here, where
        # it is asked for, instead of surfacing later as a shape/dtype error inside a call.
        if fn(torch.empty(0, dtype=torch.float32, device=self.lattice_values.device)).dtype != torch.float32:
            raise RuntimeError("PermutoEncoding computes in float32 only: lattice_values and "
                               "random_shift_per_level cannot be converted to another dtype")
        out = super()._apply(fn, *args, **kwargs)
        # the window follows device moves only
        self.anneal_window = fn(self.anneal_window).to(torch.float32)
        self.fixed_params.m_random_shift_per_level = self.random_shift_per_level
        return out

    def _load_from_state_dict(self, state_dict, prefix, *args, **kwargs):
        # A reference checkpoint saved with appply_random_shift_per_level=False holds an
        # uninitialised 1-element shift (reference: modules.py:34); here that flag means a zero
        # shift of the regular shape, so such an entry is read as zeros.
        key = prefix + "random_shift_per_level"
        value = state_dict.get(key)
        if value is not None and tuple(value.shape) == (1,) and not self.appply_random_shift_per_level:
            state_dict = dict(state_dict)
            state_dict[key] = torch.zeros_like(self.random_shift_per_level)
        return super()._load_from_state_dict(state_dict, prefix, *args, **kwargs)

    def forward(self, positions, anneal_window=None):
        if anneal_window is None:
            anneal_window = self.anneal_window
        if anneal_window.device != positions.device:
            anneal_window = anneal_window.to(positions.device)
        # the shift parameter may have been replaced (load_state_dict(assign=True), .to())
        self.fixed_params.m_random_shift_per_level = self.random_shift_per_level

        half = self._half_copy() if getattr(self, "half_precision_table", False) else None
        grad_mode = torch.is_grad_enabled()
        require_lattice_values_grad = self.lattice_values.requires_grad and grad_mode
        require_positions_grad = positions.requires_grad and grad_mode
        if not (require_lattice_values_grad or require_positions_grad):
            # inference: nothing to record, skip the autograd machinery (host overhead dominates
            # README-sized batches)
            return self.lattice.forward(_C.EncodingInput(self.lattice_values, positions, anneal_window, False, False,
                                                         half))

        # [N, (L+extra)*F] already in the reference's output order: no permute/reshape copy
        return PermutoEncodingFunc.apply(self.lattice, self.lattice_values, positions, anneal_window,
                                         require_lattice_values_grad, require_positions_grad, half)

    def _half_copy(self):
        """fp16 copy of the lattice values the kernels gather from when ``half_precision_table`` is
        set; re-made whenever the parameter has been modified in place (an optimizer step) or
        replaced.  The parameter, its gradient and the optimizer state stay fp32."""
        v = self.lattice_values
        if self._half is None or self._half_version != v._version or self._half.device != v.device \
                or self._half_ptr != v.data_ptr():
            self._half = v.detach().to(torch.float16)
            self._half_version = v._version
            self._half_ptr = v.data_ptr()
        return self._half

    @torch.no_grad()
    def forward_linear(self, positions, linear, anneal_window=None, status=None):
        """Inference shortcut for ``linear(self(positions))`` where ``linear`` is the
        ``torch.nn.Linear`` (or a ``(weight, bias)`` pair) that consumes the features: one kernel,
        the ``[N, output_dims()]`` features stay on chip and the product runs on the tensor cores
        (operands rounded to tf32, fp32 accumulation -- about 1e-3 relative to the magnitude of
        the summed terms).  No gradients are recorded; train through ``forward``."""
        if anneal_window is None:
            anneal_window = self.anneal_window
        if anneal_window.device != positions.device:
            anneal_window = anneal_window.to(positions.device)
        self.fixed_params.m_random_shift_per_level = self.random_shift_per_level
        weight, bias = (linear.weight, linear.bias) if hasattr(linear, "weight") else linear
        half = self._half_copy() if getattr(self, "half_precision_table", False) else None
        inp = _C.EncodingInput(self.lattice_values, positions, anneal_window, False, False, half)
        return self.lattice.forward_linear(inp, weight, bias, status)

    @torch.no_grad()
    def forward_mlp(self, positions, mlp, anneal_window=None, status=None):
        """Inference shortcut for ``mlp(self(positions))`` where ``mlp`` is a ``torch.nn.Sequential``
        of ``Linear`` layers separated by one kind of activation (``GELU()`` or ``ReLU()``; none
        after the last layer) -- e.g. the network of the reference's toy example
        (examples/train_toy_example.py:18-26).  One kernel: neither the features nor the hidden
        activations are written to memory; see ``EncodingWrapper.forward_mlp`` for the limits
        (hidden widths multiples of 16 up to 64) and the precision (tf32 operands)."""
        if anneal_window is None:
            anneal_window = self.anneal_window
        if anneal_window.device != positions.device:
            anneal_window = anneal_window.to(positions.device)
        self.fixed_params.m_random_shift_per_level = self.random_shift_per_level
        layers, kinds = [], set()
        mods = list(mlp)
        prev = None
        for m in mods:
            if isinstance(m, torch.nn.Linear):
                if isinstance(prev, torch.nn.Linear):
                    kinds.add("none")     # two layers back to back
                layers.append((m.weight, m.bias))
            elif isinstance(m, (torch.nn.GELU, torch.nn.ReLU)):
                if not isinstance(prev, torch.nn.Linear):
                    raise RuntimeError("an activation must follow a Linear layer")
                if isinstance(m, torch.nn.GELU) and getattr(m, "approximate", "none") != "none":
                    raise RuntimeError("only the exact GELU (approximate='none') is fused")
                kinds.add("gelu" if isinstance(m, torch.nn.GELU) else "relu")
            else:
                raise RuntimeError(f"cannot fuse a {type(m).__name__} layer")
            prev = m
        if not layers or not isinstance(mods[-1], torch.nn.Linear):
            raise RuntimeError("the fused network must end with a Linear layer")
        if len(kinds) > 1:
            raise RuntimeError(f"one kind of activation between the layers, got {sorted(kinds)}")
        activation = kinds.pop() if kinds else "none"
        half = self._half_copy() if getattr(self, "half_precision_table", False) else None
        inp = _C.EncodingInput(self.lattice_values, positions, anneal_window, False, False, half)
        return self.lattice.forward_mlp(inp, layers, activation, status)

    def output_dims(self):
        nr_resolutions_extra = 0
        if self.concat_points:
            nr_resolutions_extra = math.ceil(float(self.pos_dim) / self.nr_feat_per_level)
        return self.nr_feat_per_level * (self.nr_levels + nr_resolutions_extra)


class Coarse2Fine(torch.nn.Module):
    """Coarse-to-fine annealing window over ``nr_values`` levels, ``t`` in [0, 1]
    (reference: modules.py:109-127)."""

    def __init__(self, nr_values):
        super().__init__()
        self.nr_values = nr_values
        self.last_t = 0

    def forward(self, t):
        alpha = t * self.nr_values
        window = cosine_easing_window(self.nr_values, alpha)
        self.last_t = t
        assert t <= 1.0, "t cannot be larger than 1.0"
        return window

    def get_last_t(self):
        return self.last_t
