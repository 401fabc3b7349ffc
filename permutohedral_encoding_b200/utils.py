"""Small helpers of the reference's Python surface (reference: src/pytorch_modules/utils.py)."""
import math

import torch


def cosine_easing_window(num_freqs, alpha):
    """Window over ``num_freqs`` levels that opens them one after the other with a cosine ramp
    as ``alpha`` goes from 0 to ``num_freqs`` (reference: utils.py:5-16)."""
    x = torch.clip(alpha - torch.arange(num_freqs, dtype=torch.float32), 0.0, 1.0)
    return 0.5 * (1 + torch.cos(math.pi * x + math.pi))


def map_range_val(input_val, input_start, input_end, output_start, output_end):
    """Clamp ``input_val`` to [input_start, input_end] and map it linearly onto
    [output_start, output_end] (reference: utils.py:19-23)."""
    clamped = max(input_start, min(input_end, input_val))
    return output_start + ((output_end - output_start) / (input_end - input_start)) * (clamped - input_start)
