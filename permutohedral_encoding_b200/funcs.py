"""Autograd wiring: forward -> backward -> double backward (reference:
src/pytorch_modules/funcs.py:8-72).

Two chained ``torch.autograd.Function``s, as in the reference: the backward of the first is
itself a Function, so that a position gradient taken with ``create_graph=True`` (PermutoSDF's
eikonal term) can be differentiated again into the lattice values and into the upstream
gradient.  Differences from the reference, all internal: tensors are kept with
``save_for_backward`` (version-counter checks apply), exactly as many gradients are returned as
there are inputs, and features are ``[N, 2*(L+extra)]`` so no transposing copy happens here.
"""
import torch

from . import _native as _C


class PermutoEncodingFunc(torch.autograd.Function):
    @staticmethod
    def forward(ctx, lattice, lattice_values, positions, anneal_window, require_lattice_values_grad,
                require_positions_grad, lattice_values_half=None):
        # lattice_values_half: optional fp16 copy of the values the kernels gather from (storage
        # only); gradients flow to the fp32 lattice_values
        input_struct = _C.EncodingInput(lattice_values, positions, anneal_window, require_lattice_values_grad,
                                        require_positions_grad, lattice_values_half)
        sliced_values = lattice.forward(input_struct)
        ctx.lattice = lattice
        ctx.require = (bool(require_lattice_values_grad), bool(require_positions_grad))
        ctx.half = lattice_values_half
        ctx.save_for_backward(lattice_values, positions, anneal_window)
        return sliced_values

    @staticmethod
    def backward(ctx, grad_sliced_values):
        lattice_values, positions, anneal_window = ctx.saved_tensors
        req_lv, req_pos = ctx.require
        # only what this backward pass was asked for: autograd.grad(y, positions) does not need the
        # lattice gradient (the reference computes and discards it)
        req_lv = req_lv and ctx.needs_input_grad[1]
        req_pos = req_pos and ctx.needs_input_grad[2]
        if not (req_lv or req_pos) and any(ctx.require):
            return None, None, None, None, None, None, None
        assert req_lv or req_pos, (
            "We cannot perform the backward function on the slicing because we did not precompute the required "
            "tensors in the forward pass. To enable this, set the model.train(), set torch.set_grad_enabled(True) "
            "and make lattice_values have required_grad=True")
        lattice_values_grad, positions_grad = PermutoEncodingFuncBack.apply(
            ctx.lattice, grad_sliced_values, lattice_values, positions, anneal_window, req_lv, req_pos, ctx.half)
        return None, lattice_values_grad, positions_grad, None, None, None, None


class PermutoEncodingFuncBack(torch.autograd.Function):
    """The first-order backward as a differentiable function of (upstream gradient, lattice
    values); its own backward is the double backward from the position gradient."""

    @staticmethod
    def forward(ctx, lattice, grad_sliced_values, lattice_values, positions, anneal_window,
                require_lattice_values_grad, require_positions_grad, lattice_values_half=None):
        grad_sliced_values = grad_sliced_values.contiguous()
        input_struct = _C.EncodingInput(lattice_values, positions, anneal_window, require_lattice_values_grad,
                                        require_positions_grad, lattice_values_half)
        hook = getattr(lattice, "backward_hook", None)
        if hook is not None and require_lattice_values_grad:
            lattice_values_grad, positions_grad = hook(lattice, input_struct, grad_sliced_values)
        else:
            lattice_values_grad, positions_grad = lattice.backward(input_struct, grad_sliced_values)
        ctx.lattice = lattice
        ctx.half = lattice_values_half
        ctx.save_for_backward(grad_sliced_values, lattice_values, positions, anneal_window)
        return lattice_values_grad, positions_grad

    @staticmethod
    def backward(ctx, double_lattice_values_grad, double_positions_grad):
        # As in the reference, only the path through the position gradient is differentiated
        # again; a second-order term through the lattice-value gradient is not propagated.
        if double_positions_grad is None:
            return None, None, None, None, None, None, None, None
        grad_sliced_values, lattice_values, positions, anneal_window = ctx.saved_tensors
        need_ggs = ctx.needs_input_grad[1]
        need_lv = ctx.needs_input_grad[2]
        if not (need_ggs or need_lv):
            return None, None, None, None, None, None, None, None
        input_struct = _C.EncodingInput(lattice_values, positions, anneal_window, need_lv, True, ctx.half)
        grad_lattice_values, grad_grad_sliced_values = ctx.lattice.double_backward_from_positions(
            input_struct, double_positions_grad, grad_sliced_values, need_lattice_grad=need_lv,
            need_grad_grad_features=need_ggs)
        # data-parallel use: this second-order lattice gradient is summed over the ranks like the
        # first-order one, otherwise the replicated tables drift apart (see distributed.py)
        hook = getattr(ctx.lattice, "double_backward_hook", None)
        if hook is not None and grad_lattice_values is not None:
            grad_lattice_values = hook(grad_lattice_values)
        return None, grad_grad_sliced_values, grad_lattice_values, None, None, None, None, None
