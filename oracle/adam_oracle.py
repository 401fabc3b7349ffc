"""CPU restatement (numpy, fp32) of the optimizer step the reference applies to the lattice values.

TEST INFRASTRUCTURE ONLY: imported by tests/ (and nothing in the product package).

The algorithm is not in the reference's tree: its training loops call ``torch.optim.AdamW``
(reference: examples/performance.py:161 and :101; examples/train_toy_example.py:30) from the
installed PyTorch (no version pinned by the reference, ``install_requires=[]``; 2.11.0 here).
This follows PyTorch's published single-tensor AdamW update, amsgrad off:

    p  *= 1 - lr * weight_decay
    m   = lerp(m, g, 1 - beta1)
    v   = v * beta2 + (1 - beta2) * g * g
    p  -= lr / (1 - beta1^t) * m / (sqrt(v) / sqrt(1 - beta2^t) + eps)

Pinned by tests/test_oracle_golden.py against ``torch.optim.AdamW`` itself run on CPU tensors.
"""
import math

import numpy as np


def adamw_step(p, g, m, v, step, lr, beta1, beta2, eps, weight_decay):
    """One step; all arrays float32, updated copies are returned as (p, m, v)."""
    f = np.float32
    p = (p * f(1.0 - lr * weight_decay)).astype(np.float32)
    m = (m + (g - m) * f(1.0 - beta1)).astype(np.float32)
    v = ((v * f(beta2)).astype(np.float32) + f(1.0 - beta2) * g * g).astype(np.float32)
    bc1 = 1.0 - beta1 ** step
    bc2 = 1.0 - beta2 ** step
    denom = (np.sqrt(v) / f(math.sqrt(bc2)) + f(eps)).astype(np.float32)
    p = (p - f(lr / bc1) * (m / denom)).astype(np.float32)
    return p, m, v
