"""Binding of the hand written causal attention kernel (``csrc/attention.cu``)."""
from __future__ import annotations

import torch


def available() -> bool:
    from . import cuda
    try:
        return hasattr(cuda.lib(), "slab_attn_fwd")
    except cuda.KernelError:
        return False


def supports(q, k, v, window: int) -> bool:
    return False
