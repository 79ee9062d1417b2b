"""Helpers shared by the tests: load the committed golden fixtures as torch tensors."""
import os

import numpy as np
import torch

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def load(name):
    return dict(np.load(os.path.join(GOLDEN, name + ".npz")))


def t(a, bf16=False):
    x = torch.from_numpy(np.ascontiguousarray(a))
    return x.view(torch.bfloat16) if bf16 else x


def same_bits(a: torch.Tensor, b: torch.Tensor) -> bool:
    """Bit equality (distinguishes -0 from +0, treats equal NaN payloads as equal)."""
    if a.shape != b.shape or a.dtype != b.dtype:
        return False
    a = a.contiguous()
    b = b.contiguous()
    if a.dtype == torch.bool:
        return bool(torch.equal(a, b))
    n = a.element_size()
    it = {1: torch.uint8, 2: torch.int16, 4: torch.int32, 8: torch.int64}[n]
    return bool(torch.equal(a.view(it), b.view(it)))
