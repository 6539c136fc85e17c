"""Public op surface.

Each op has exactly two implementations: the hand written sm_100a kernel (``ops/cuda.py`` over
``csrc/``) and the PyTorch oracle (``ops/reference.py``).  CUDA tensors take the kernel path; CPU
tensors take the oracle.  ``set_kernel_mode("reference")`` forces the oracle on the GPU too — that is
the measured library baseline (cuBLAS / ATen), never a silent fallback: if the extension is missing
on a GPU machine the kernel path raises.
"""
from __future__ import annotations

import torch

from . import reference as ref

_MODE = "auto"          # auto: kernels on CUDA tensors | reference: oracle everywhere


def set_kernel_mode(mode: str) -> None:
    global _MODE
    if mode not in ("auto", "reference"):
        raise ValueError(mode)
    _MODE = mode


def kernel_mode() -> str:
    return _MODE


_DENSE_KERNELS = [True]


def set_dense_kernels(on: bool) -> None:
    """Dense projections and the vocabulary GEMMs of the fused cross entropy on the hand-written GEMM (default) or
    on the library GEMM (the comparison path)."""
    _DENSE_KERNELS[0] = bool(on)


def dense_kernels() -> bool:
    return _DENSE_KERNELS[0]


def use_kernels(t: torch.Tensor) -> bool:
    return _MODE == "auto" and t.is_cuda


def _cuda():
    from . import cuda
    return cuda


def rmsnorm(x, weight, eps=1e-6):
    return _cuda().rmsnorm(x, weight, eps) if use_kernels(x) else ref.rmsnorm(x, weight, eps)


def rmsnorm_residual(x, residual, weight, eps=1e-6):
    if use_kernels(x):
        return _cuda().rmsnorm_residual(x, residual, weight, eps)
    return ref.rmsnorm_residual(x, residual, weight, eps)


def rope(x, cos, sin):
    return _cuda().rope(x, cos, sin) if use_kernels(x) else ref.rope(x, cos, sin)


def swiglu(gate_up):
    return _cuda().swiglu(gate_up) if use_kernels(gate_up) else ref.swiglu(gate_up)


def swiglu_probs(gate_up, probs, rows_dev=None):
    if use_kernels(gate_up):
        return _cuda().swiglu_probs(gate_up, probs, rows_dev)
    return ref.swiglu_probs(gate_up, probs)


def linear(x, weight):
    """``x @ weight^T`` for a dense projection (no bias).  bf16 CUDA operands whose shapes the tile sizes cover run on
    the hand-written tcgen05 GEMM (forward, input gradient and weight gradient); everything else is the library."""
    fg = getattr(weight, "_flat_group", None)
    pending = fg is not None and fg.pending_gather is not None      # the group's matrices are still on their owners
    if weight.dtype != x.dtype:
        weight = weight.to(x.dtype)
    if use_kernels(x) and _DENSE_KERNELS[0] and _cuda().linear_ok(x, weight):
        # FSDP: this GEMM pulls the layer's matrices from the peers while it multiplies the first of them
        return _cuda().linear(x, weight, fg.take_pending_gather(weight) if pending else None)
    if pending:
        fg.finish_pending_gather()
    return torch.nn.functional.linear(x, weight)


def router_logits(x, router_weight):
    """fp32 router logits ``x @ Wr^T``.  On the GPU the product runs on tensor cores from bf16 operands
    with fp32 accumulation and fp32 output; the oracle casts both operands to fp32 first."""
    if use_kernels(x) and x.dtype == torch.bfloat16 and router_weight.dtype == torch.bfloat16:
        return _cuda().router_logits(x, router_weight)
    return torch.nn.functional.linear(x.float(), router_weight.float())


def router_fused(logits, topk, score_function="softmax", bias=None, norm_topk_prob=True, scaling_factor=1.0,
                 aux_coeff=0.0):
    """Router selection plus the Switch-style load-balancing loss ``aux_coeff * E * sum_e f_e * P_e`` (zero when
    ``aux_coeff`` is): ``(weights [T, K] fp32, idx [T, K], aux scalar)``.  One kernel forward, one backward on the GPU."""
    if use_kernels(logits):
        w, idx, aux, _ = _cuda().router_fused(logits, topk, score_function, bias, norm_topk_prob, scaling_factor,
                                              aux_coeff)
        return w, idx, aux
    w, idx, scores = ref.router_topk(logits, topk, score_function, bias, norm_topk_prob, scaling_factor)
    aux = ref.aux_loss(scores, idx.long(), logits.shape[-1], aux_coeff) if aux_coeff else \
        torch.zeros((), dtype=torch.float32, device=logits.device)
    return w, idx, aux


def router_topk(logits, topk, score_function="softmax", bias=None, norm_topk_prob=True, scaling_factor=1.0):
    if use_kernels(logits):
        return _cuda().router_topk(logits, topk, score_function, bias, norm_topk_prob, scaling_factor)
    return ref.router_topk(logits, topk, score_function, bias, norm_topk_prob, scaling_factor)


def rope_packed(qkv, cos, sin, n_heads: int, head_dim: int):
    """Rotate the first ``n_heads`` heads of each row of a packed ``[B, S, W]`` projection (q and k of a
    fused qkv).  The kernel path rotates in place; the oracle path builds a new tensor."""
    if use_kernels(qkv):
        out = _cuda().rope_packed(qkv, cos, sin, n_heads, head_dim)
        if out is not None:
            return out
    b, s, w = qkv.shape
    rot = ref.rope(qkv[..., :n_heads * head_dim].reshape(b, s, n_heads, head_dim), cos, sin)
    return torch.cat([rot.reshape(b, s, n_heads * head_dim), qkv[..., n_heads * head_dim:]], dim=-1)


def grouped_linear(a, w, offsets, counts, fp8: bool = False, out=None, dgrad_out=None, dead: bool = False,
                   ready=None, bwd_ready=None):
    """``out[rows of e] = a[rows of e] @ w[e].T`` (``w: [E, N, K]``), differentiable in ``a`` and ``w``.
    ``out`` (kernel path only) names the buffer the result is written to, e.g. the peer-visible
    expert-output buffer of the fused dispatcher.  ``dead``: only the autograd node is wanted (a recomputed
    forward whose result nobody reads); the product is not computed and the returned values are unspecified.
    ``ready`` / ``bwd_ready``: arrival flags of rows that peers are still delivering (fused dispatcher): the kernel
    waits for them expert by expert; every other route waits for the whole exchange before it reads a row."""
    if use_kernels(a):
        return _cuda().grouped_linear(a, w, offsets, counts, fp8, out, dgrad_out, dead, ready, bwd_ready)
    if ready is not None:
        ready.wait()
    return _GroupedLinearRef.apply(a, w, offsets, counts, dead, fp8)


def grouped_kernel_ok(a, w) -> bool:
    """True if ``grouped_linear(a, w, ...)`` runs on the hand-written grouped GEMM (and can therefore wait for rows
    that are still arriving inside the kernel)."""
    return use_kernels(a) and _cuda().grouped_kernel_ok(a, w)


def causal_attention(q, k, v, scale=None, window=0):
    if use_kernels(q):
        return _cuda().causal_attention(q, k, v, scale, window)
    return ref.causal_attention(q, k, v, scale, window)


def linear_cross_entropy(h, weight, targets):
    if use_kernels(h):
        return _cuda().linear_cross_entropy(h, weight, targets)
    return ref.linear_cross_entropy(h, weight, targets)


class _GroupedLinearRef(torch.autograd.Function):
    """Oracle grouped linear with explicit fwd/dgrad/wgrad (mirrors the three CUDA kernels)."""

    @staticmethod
    def forward(ctx, a, w, offsets, counts, dead=False, fp8=False):
        ctx.save_for_backward(a, w, offsets, counts)
        if dead:
            return a.new_zeros(a.shape[0], w.shape[1])
        if fp8:
            # emulation of the fp8 forward: operands rounded to e4m3 with the recipe's scales, product in fp32;
            # the backward stays on the unquantised operands, like the kernel path
            if fp8 == "blockwise" and a.shape[1] % 128 == 0 and w.shape[1] % 128 == 0:
                aq = ref.dequant_1x128(*ref.quant_1x128(a)).to(a.dtype)
                wq = ref.dequant_128x128(*ref.quant_128x128(w)).to(w.dtype)
            elif fp8 == "tensorwise":
                qa, sa = ref.quant_tensorwise(a)
                qw, sw = ref.quant_tensorwise(w)
                aq, wq = (qa.float() * sa).to(a.dtype), (qw.float() * sw).to(w.dtype)
            else:
                qa, sa = ref.quant_rowwise(a)
                qw, sw = ref.quant_rowwise(w)
                aq = (qa.float() * sa.unsqueeze(-1)).to(a.dtype)
                wq = (qw.float() * sw.unsqueeze(-1)).to(w.dtype)
            return ref.grouped_gemm(aq, wq, offsets, counts)
        return ref.grouped_gemm(a, w, offsets, counts)

    @staticmethod
    def backward(ctx, g):
        a, w, offsets, counts = ctx.saved_tensors
        g = g.contiguous()
        da = ref.grouped_gemm_dgrad(g, w, offsets, counts) if ctx.needs_input_grad[0] else None
        dw = ref.grouped_gemm_wgrad(g, a, offsets, counts, out_dtype=w.dtype) if ctx.needs_input_grad[1] else None
        return da, dw, None, None, None, None
