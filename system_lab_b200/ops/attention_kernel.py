"""Binding of the hand-written causal attention kernels (``csrc/attention.cu``: tcgen05 GEMMs with TMEM accumulators,
softmax with one row per thread, GQA, sliding window, head dim 64 / 128): the forward (online softmax, output and
log-sum-exp) and the backward (five GEMMs per tile pair, dK / dV accumulated in TMEM, dQ through fp32 atomics).

State: the kernels are compiled with the rest of the library; they are **off by default** (``set_enabled(True)`` or
``SLAB_ATTENTION_KERNEL=1`` turns the forward on; ``SLAB_ATTENTION_KERNEL_BWD=1`` additionally routes the backward
to the kernel) because they have not yet been timed against the library's fused attention, which stays the default
path.  With only the forward enabled, the backward re-runs the library's attention under autograd.

Reference: attention in the measured runs is a library FMHA as well (aiter / CK-tile on MI355X,
``notes/2026-04/2026-04-21_gptoss_13_*:19-105``; cuDNN flash attention on B200,
``docs/b200-vs-mi355x-ep8-gbs16-trace.html:433``).
"""
from __future__ import annotations

import os

import torch

from . import cuda

cuda.register("slab_attn_fwd", "ppppp" + "iiiii" + "lll" + "i" + "f" + "p" + "s")
cuda.register("slab_attn_bwd", "p" * 9 + "iiiii" + "lll" + "i" + "f" + "p" + "s")
cuda._STATUS_NAMES.update({20: "ATTN_Q", 21: "ATTN_KV_FULL", 22: "ATTN_KV_EMPTY", 23: "ATTN_S", 24: "ATTN_P",
                           25: "ATTN_PV", 30: "ATTNB_KV", 31: "ATTNB_QDO_FULL", 32: "ATTNB_QDO_EMPTY", 33: "ATTNB_SDP",
                           34: "ATTNB_PDS", 35: "ATTNB_MMA2", 36: "ATTNB_DQ"})

_ENABLED = [os.environ.get("SLAB_ATTENTION_KERNEL", "0") == "1"]
_ENABLED_BWD = [os.environ.get("SLAB_ATTENTION_KERNEL_BWD", "0") == "1"]


def set_enabled(on: bool) -> None:
    _ENABLED[0] = bool(on)


def available() -> bool:
    try:
        return hasattr(cuda.lib(), "slab_attn_fwd")
    except cuda.KernelError:
        return False


def _row_stride(t: torch.Tensor):
    """Elements between consecutive tokens of a ``[B, S, H, D]`` view whose (H, D) block is contiguous and whose
    batch stride is ``S`` rows; None if the view is not of that form."""
    b, s, h, d = t.shape
    if t.stride(3) != 1 or t.stride(2) != d:
        return None
    row = t.stride(1)
    if row < h * d or (b > 1 and t.stride(0) != s * row):
        return None
    return row


def shape_ok(q, k, v, window: int) -> bool:
    """Shapes the kernel covers: bf16, equal q/k/v head dim of 64 or 128, sequence a multiple of 128, GQA."""
    if not (q.is_cuda and q.dtype == k.dtype == v.dtype == torch.bfloat16):
        return False
    b, s, hq, d = q.shape
    if k.shape != v.shape or k.shape[0] != b or k.shape[1] != s or k.shape[3] != d:
        return False
    if d not in (64, 128) or s % 128 or hq % k.shape[2]:
        return False
    for t in (q, k, v):
        row = _row_stride(t)
        if row is None or row % 8 or t.data_ptr() % 16:
            return False
    return True


def supports(q, k, v, window: int) -> bool:
    return _ENABLED[0] and shape_ok(q, k, v, window) and available()


def forward(q, k, v, scale: float, window: int = 0):
    """``(out [B, S, Hq, D] bf16, lse [B, Hq, S] fp32)``; q, k, v may be column slices of a packed projection."""
    b, s, hq, d = q.shape
    out = torch.empty((b, s, hq, d), dtype=torch.bfloat16, device=q.device)
    lse = torch.empty((b, hq, s), dtype=torch.float32, device=q.device)
    cuda.call("slab_attn_fwd", q, k, v, out, lse, b, s, hq, k.shape[2], d, _row_stride(q), _row_stride(k),
              _row_stride(v), int(window), float(scale), cuda.status_word(q.device), cuda.stream())
    return out, lse


def backward(q, k, v, out, lse, dout, scale: float, window: int = 0):
    """``(dq, dk, dv)`` from the forward's inputs, output and log-sum-exp.  ``delta = rowsum(dout * out)`` and the
    final cast of dq are library elementwise ops; the five GEMMs per tile pair run in the kernel."""
    b, s, hq, d = q.shape
    hkv = k.shape[2]
    dout = dout.contiguous()
    delta = (dout.float() * out.float()).sum(-1).transpose(1, 2).contiguous()          # [B, Hq, S]
    dq_acc = torch.zeros((b, s, hq, d), dtype=torch.float32, device=q.device)
    dk = torch.empty((b, s, hkv, d), dtype=torch.bfloat16, device=q.device)
    dv = torch.empty((b, s, hkv, d), dtype=torch.bfloat16, device=q.device)
    cuda.call("slab_attn_bwd", q, k, v, dout, lse, delta, dq_acc, dk, dv, b, s, hq, hkv, d, _row_stride(q),
              _row_stride(k), _row_stride(v), int(window), float(scale), cuda.status_word(q.device), cuda.stream())
    return dq_acc.to(torch.bfloat16), dk, dv


class _KernelAttention(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, scale, window):
        out, lse = forward(q, k, v, scale, window)
        ctx.kernel_bwd = _ENABLED_BWD[0]
        if ctx.kernel_bwd:
            ctx.save_for_backward(q, k, v, out, lse)
        else:
            ctx.save_for_backward(q, k, v)
        ctx.scale, ctx.window = scale, window
        return out

    @staticmethod
    def backward(ctx, g):
        if ctx.kernel_bwd:
            q, k, v, out, lse = ctx.saved_tensors
            dq, dk, dv = backward(q, k, v, out, lse, g, ctx.scale, ctx.window)
            return dq, dk, dv, None, None
        from .attention import _library
        q, k, v = (t.detach().requires_grad_(True) for t in ctx.saved_tensors)
        with torch.enable_grad():
            o = _library(q, k, v, ctx.scale, ctx.window)
        dq, dk, dv = torch.autograd.grad(o, (q, k, v), g)
        return dq, dk, dv, None, None


def attention(q, k, v, scale: float, window: int = 0):
    return _KernelAttention.apply(q, k, v, scale, window)
