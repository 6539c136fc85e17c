"""Causal attention on the GPU.

Default: the library's fused attention (cuDNN SDPA first, flash-attn for sliding windows, PyTorch SDPA otherwise),
the same class of kernel the reference's B200 trace ran (64.3 ms per step, ``docs/b200-vs-mi355x-ep8-gbs16-
trace.html:433``).  The hand-written forward (``csrc/attention.cu``, bound in ``attention_kernel.py``) takes over
for the shapes it covers once it is switched on (``attention_kernel.set_enabled`` / ``SLAB_ATTENTION_KERNEL=1``).
"""
from __future__ import annotations

import math

import torch
import torch.nn.functional as F

_IMPL = "auto"          # auto | library


def set_attention_impl(name: str) -> None:
    global _IMPL
    _IMPL = name


_CUDNN_OK = [None]        # None: untried, True/False afterwards


def _cudnn_sdpa(q, k, v, scale):
    from torch.nn.attention import SDPBackend, sdpa_kernel
    hq, hkv = q.shape[2], k.shape[2]
    with sdpa_kernel([SDPBackend.CUDNN_ATTENTION]):
        o = F.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), is_causal=True,
                                           scale=scale, enable_gqa=hq != hkv)
    return o.transpose(1, 2)


def _library(q, k, v, scale, window):
    d, dv = q.shape[-1], v.shape[-1]
    if q.is_cuda and dv < d:
        # latent attention has a narrower value head (128) than query/key head (192): the fused library kernels
        # want equal widths, so pad V with zero columns and drop them from the output
        vp = torch.nn.functional.pad(v, (0, d - dv))
        return _library(q, k, vp, scale, window)[..., :dv]
    if q.is_cuda and window == 0 and q.dtype in (torch.bfloat16, torch.float16) and _CUDNN_OK[0] is not False:
        try:
            o = _cudnn_sdpa(q, k, v, scale)
            _CUDNN_OK[0] = True
            return o
        except RuntimeError:
            if _CUDNN_OK[0]:
                raise
            _CUDNN_OK[0] = False
    if q.is_cuda and d == dv and d <= 256 and q.dtype in (torch.bfloat16, torch.float16):
        try:
            from flash_attn import flash_attn_func
            win = (window - 1, 0) if window > 0 else (-1, -1)
            return flash_attn_func(q, k, v, softmax_scale=scale, causal=True, window_size=win)
        except ImportError:
            pass
    b, s, hq, _ = q.shape
    hkv = k.shape[2]
    qt, kt, vt = q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2)
    if window > 0:
        i = torch.arange(s, device=q.device)
        mask = (i[None, :] <= i[:, None]) & (i[None, :] > i[:, None] - window)
        o = F.scaled_dot_product_attention(qt, kt, vt, attn_mask=mask, scale=scale, enable_gqa=hq != hkv)
    else:
        o = F.scaled_dot_product_attention(qt, kt, vt, is_causal=True, scale=scale, enable_gqa=hq != hkv)
    return o.transpose(1, 2)


def causal_attention(q, k, v, scale=None, window: int = 0):
    scale = scale if scale is not None else 1.0 / math.sqrt(q.shape[-1])
    if _IMPL == "auto":
        from . import attention_kernel
        if attention_kernel.supports(q, k, v, window):
            return attention_kernel.attention(q, k, v, scale, window)
    return _library(q, k, v, scale, window)
