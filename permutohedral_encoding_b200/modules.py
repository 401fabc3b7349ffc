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
    The misspelt keyword ``appply_random_shift_per_level`` is part of the reference's public
    surface and is kept.  With ``appply_random_shift_per_level=False`` the reference creates an
    unusable 1-element shift (modules.py:34 fails the native shape checks); here the shift is
    a zero ``[nr_levels, pos_dim]`` tensor, which is what the flag means.
    ``nr_feat_per_level`` may be 2 (the only width the reference implements), 4 or 8: a table
    access moves a 32-byte sector whatever it uses of it, and 16-byte accesses run at the rate of
    8-byte ones, so e.g. 12 levels of 4 features produce 48 outputs in 60 % of the time of 24 x 2.
    """

    def __init__(self, pos_dim, capacity, nr_levels, nr_feat_per_level, scale_per_level,
                 appply_random_shift_per_level=True, concat_points=False, concat_points_scaling=1.0):
        super().__init__()
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
        return fixed_params, lattice

    def __getstate__(self):
        state = self.__dict__.copy()
        del state["fixed_params"]  # native-side objects are rebuilt, not pickled
        del state["lattice"]
        return state

    def __setstate__(self, state):
        self.__dict__.update(state)
        self.fixed_params, self.lattice = self._make_lattice_wrapper()

    def _apply(self, fn, *args, **kwargs):
        # .to()/.cuda() may replace the parameter objects: re-bind the shift handle
        out = super()._apply(fn, *args, **kwargs)
        self.anneal_window = fn(self.anneal_window)
        self.fixed_params.m_random_shift_per_level = self.random_shift_per_level
        return out

    def forward(self, positions, anneal_window=None):
        if anneal_window is None:
            anneal_window = self.anneal_window
        if anneal_window.device != positions.device:
            anneal_window = anneal_window.to(positions.device)
        # the shift parameter may have been replaced (load_state_dict(assign=True), .to())
        self.fixed_params.m_random_shift_per_level = self.random_shift_per_level

        grad_mode = torch.is_grad_enabled()
        require_lattice_values_grad = self.lattice_values.requires_grad and grad_mode
        require_positions_grad = positions.requires_grad and grad_mode
        if not (require_lattice_values_grad or require_positions_grad):
            # inference: nothing to record, skip the autograd machinery (host overhead dominates
            # README-sized batches)
            return self.lattice.forward(_C.EncodingInput(self.lattice_values, positions, anneal_window, False, False))

        # [N, (L+extra)*F] already in the reference's output order: no permute/reshape copy
        return PermutoEncodingFunc.apply(self.lattice, self.lattice_values, positions, anneal_window,
                                         require_lattice_values_grad, require_positions_grad)

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
