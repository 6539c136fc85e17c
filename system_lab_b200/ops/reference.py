"""Plain PyTorch implementations of every hot op.

These are (a) the CPU / gloo execution path, (b) the numerical oracle that each
CUDA kernel is tested against, and (c) the measured "library baseline" on the
GPU.  They compute in fp32 internally and return the input dtype, which is the
contract the CUDA kernels follow as well.

Reference analogues: Triton RMSNorm (``notes/2026-04/2026-04-20_gptoss_02_triton_rmsnorm_optimization.md:47-62``),
fused residual+RMSNorm (``notes/2026-04/2026-04-24_gptoss_17_fused_residual_rmsnorm_impl.md:43-83``),
SwiGLU-with-probs (``notes/2026-04/2026-04-25_gptoss_23_swiglu_nocat_triton_verify.md:92-113``).
"""
from __future__ import annotations

import math

import torch
import torch.nn.functional as F

FP8_MAX = 448.0  # e4m3fn


# ----------------------------------------------------------------------------
# normalisation
# ----------------------------------------------------------------------------
def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    xf = x.float()
    rstd = torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
    return (xf * rstd * weight.float()).to(x.dtype)


def rmsnorm_residual(x: torch.Tensor, residual: torch.Tensor, weight: torch.Tensor, eps: float):
    """``xpr = x + residual`` (sum formed in fp32); ``y = rmsnorm(xpr)``.  Returns ``(y, xpr)``."""
    xpr_f = x.float() + residual.float()
    rstd = torch.rsqrt(xpr_f.pow(2).mean(-1, keepdim=True) + eps)
    y = (xpr_f * rstd * weight.float()).to(x.dtype)
    return y, xpr_f.to(x.dtype)


# ----------------------------------------------------------------------------
# rotary embedding (half-split "neox" convention)
# ----------------------------------------------------------------------------
def rope_tables(seq_len: int, dim: int, base: float, device, offset: int = 0):
    inv = 1.0 / (base ** (torch.arange(0, dim, 2, device=device, dtype=torch.float32) / dim))
    pos = torch.arange(offset, offset + seq_len, device=device, dtype=torch.float32)
    ang = torch.outer(pos, inv)
    return ang.cos(), ang.sin()          # [S, dim/2]


def rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """x: [B, S, H, D] (rotates all of D); cos/sin: [S, D/2]."""
    d2 = x.shape[-1] // 2
    xf = x.float()
    x1, x2 = xf[..., :d2], xf[..., d2:]
    c = cos[None, :, None, :]
    s = sin[None, :, None, :]
    return torch.cat([x1 * c - x2 * s, x2 * c + x1 * s], dim=-1).to(x.dtype)


# ----------------------------------------------------------------------------
# activations
# ----------------------------------------------------------------------------
def swiglu(gate_up: torch.Tensor) -> torch.Tensor:
    """``silu(gate) * up`` for ``gate_up = [gate | up]`` along the last dim."""
    f = gate_up.shape[-1] // 2
    g, u = gate_up[..., :f].float(), gate_up[..., f:].float()
    return (F.silu(g) * u).to(gate_up.dtype)


def swiglu_probs(gate_up: torch.Tensor, probs: torch.Tensor) -> torch.Tensor:
    """``silu(gate) * up * p`` with one fp32 probability per row."""
    f = gate_up.shape[-1] // 2
    g, u = gate_up[..., :f].float(), gate_up[..., f:].float()
    return (F.silu(g) * u * probs.float().unsqueeze(-1)).to(gate_up.dtype)


# ----------------------------------------------------------------------------
# router
# ----------------------------------------------------------------------------
def router_topk(logits: torch.Tensor, topk: int, score_function: str = "softmax",
                bias: torch.Tensor | None = None, norm_topk_prob: bool = True,
                scaling_factor: float = 1.0):
    """Returns ``(weights [T,K] fp32, indices [T,K] int64, scores [T,E] fp32)``.

    ``bias`` (aux-loss-free balancing) only influences *which* experts are chosen,
    never the gate weights.
    """
    lf = logits.float()
    scores = torch.softmax(lf, dim=-1) if score_function == "softmax" else torch.sigmoid(lf)
    sel = scores if bias is None else scores + bias.float()
    _, idx = torch.topk(sel, topk, dim=-1)
    w = torch.gather(scores, 1, idx)
    if norm_topk_prob:
        w = w / (w.sum(-1, keepdim=True) + 1e-20)
    return w * scaling_factor, idx, scores


def aux_loss(scores: torch.Tensor, idx: torch.Tensor, num_experts: int, coeff: float) -> torch.Tensor:
    """Switch-style load balancing loss ``E * sum_e f_e * P_e``."""
    t, k = idx.shape
    f = torch.zeros(num_experts, device=scores.device, dtype=torch.float32)
    f.scatter_add_(0, idx.reshape(-1), torch.ones(t * k, device=scores.device))
    f = f / (t * k)
    p = scores.mean(0)
    return coeff * num_experts * (f * p).sum()


# ----------------------------------------------------------------------------
# block scaled fp8
# ----------------------------------------------------------------------------
def quant_1x128(x: torch.Tensor):
    """Per-row, per-128-column scaling to e4m3.  Returns ``(q [.., H] fp8, scale [.., H/128] fp32)``
    with ``x ~= q * scale``."""
    *lead, h = x.shape
    assert h % 128 == 0
    xb = x.float().reshape(*lead, h // 128, 128)
    amax = xb.abs().amax(-1).clamp_min(1e-12)
    scale = amax / FP8_MAX
    q = (xb / scale.unsqueeze(-1)).clamp(-FP8_MAX, FP8_MAX).to(torch.float8_e4m3fn)
    return q.reshape(*lead, h), scale


def quant_128x128(w: torch.Tensor):
    """Per 128x128 block scaling of a ``[..., N, K]`` weight.  Returns ``(q, scale [..., N/128, K/128])``."""
    *lead, n, k = w.shape
    assert n % 128 == 0 and k % 128 == 0
    wb = w.float().reshape(*lead, n // 128, 128, k // 128, 128)
    amax = wb.abs().amax(dim=(-3, -1)).clamp_min(1e-12)
    scale = amax / FP8_MAX
    q = (wb / scale[..., :, None, :, None]).clamp(-FP8_MAX, FP8_MAX).to(torch.float8_e4m3fn)
    return q.reshape(*lead, n, k), scale


def quant_rowwise(x: torch.Tensor):
    """One scale per row of the last dimension.  Returns ``(q fp8, scale [...] fp32)`` with ``x ~= q * scale``."""
    amax = x.float().abs().amax(-1).clamp_min(1e-12)
    scale = amax / FP8_MAX
    q = (x.float() / scale.unsqueeze(-1)).clamp(-FP8_MAX, FP8_MAX).to(torch.float8_e4m3fn)
    return q, scale


def quant_tensorwise(x: torch.Tensor):
    """One scale for the whole tensor.  Returns ``(q fp8, scale 0-d fp32)`` with ``x ~= q * scale``."""
    amax = x.detach().abs().amax().float().clamp_min(1e-12)
    scale = amax / FP8_MAX
    q = (x.float() / scale).clamp(-FP8_MAX, FP8_MAX).to(torch.float8_e4m3fn)
    return q, scale


def dequant_1x128(q: torch.Tensor, scale: torch.Tensor) -> torch.Tensor:
    *lead, h = q.shape
    return (q.float().reshape(*lead, h // 128, 128) * scale.unsqueeze(-1)).reshape(*lead, h)


def dequant_128x128(q: torch.Tensor, scale: torch.Tensor) -> torch.Tensor:
    *lead, n, k = q.shape
    qb = q.float().reshape(*lead, n // 128, 128, k // 128, 128)
    return (qb * scale[..., :, None, :, None]).reshape(*lead, n, k)


# ----------------------------------------------------------------------------
# grouped GEMM: rows of `a` are grouped by expert, `offsets[e]..offsets[e]+counts[e]`
# ----------------------------------------------------------------------------
def grouped_gemm(a: torch.Tensor, b: torch.Tensor, offsets: torch.Tensor, counts: torch.Tensor) -> torch.Tensor:
    """``out[rows of e] = a[rows of e] @ b[e].T`` with ``b: [E, N, K]``.  Rows outside every
    segment (alignment padding) come back as zeros."""
    out = a.new_zeros(a.shape[0], b.shape[1])
    offs, cnts = offsets.tolist(), counts.tolist()
    for e, (o, c) in enumerate(zip(offs, cnts)):
        if c:
            out[o:o + c] = (a[o:o + c].float() @ b[e].float().t()).to(a.dtype)
    return out


def grouped_gemm_dgrad(dy: torch.Tensor, b: torch.Tensor, offsets, counts) -> torch.Tensor:
    """``dx[rows of e] = dy[rows of e] @ b[e]``."""
    out = dy.new_zeros(dy.shape[0], b.shape[2])
    for e, (o, c) in enumerate(zip(offsets.tolist(), counts.tolist())):
        if c:
            out[o:o + c] = (dy[o:o + c].float() @ b[e].float()).to(dy.dtype)
    return out


def grouped_gemm_wgrad(dy: torch.Tensor, a: torch.Tensor, offsets, counts, out_dtype=None) -> torch.Tensor:
    """``db[e] = dy[rows of e].T @ a[rows of e]`` -> ``[E, N, K]`` (variable reduction length)."""
    e_n = offsets.numel()
    out = torch.zeros(e_n, dy.shape[1], a.shape[1], device=a.device, dtype=out_dtype or a.dtype)
    for e, (o, c) in enumerate(zip(offsets.tolist(), counts.tolist())):
        if c:
            out[e] = (dy[o:o + c].float().t() @ a[o:o + c].float()).to(out.dtype)
    return out


# ----------------------------------------------------------------------------
# attention
# ----------------------------------------------------------------------------
def causal_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float | None = None,
                     window: int = 0) -> torch.Tensor:
    """q: [B,S,Hq,D], k: [B,S,Hkv,D], v: [B,S,Hkv,Dv] -> [B,S,Hq,Dv].  ``window>0`` restricts each
    query to the last ``window`` keys (sliding-window layers of GPT-OSS)."""
    b, s, hq, d = q.shape
    hkv = k.shape[2]
    g = hq // hkv
    scale = scale if scale is not None else 1.0 / math.sqrt(d)
    qf = q.float().permute(0, 2, 1, 3).reshape(b, hkv, g, s, d)
    kf = k.float().permute(0, 2, 1, 3)
    vf = v.float().permute(0, 2, 1, 3)
    att = torch.einsum("bhgsd,bhtd->bhgst", qf, kf) * scale
    i = torch.arange(s, device=q.device)
    mask = i[None, :] > i[:, None]
    if window > 0:
        mask = mask | (i[None, :] <= i[:, None] - window)
    att = att.masked_fill(mask, float("-inf")).softmax(-1)
    out = torch.einsum("bhgst,bhtd->bhgsd", att, vf)
    return out.reshape(b, hq, s, -1).permute(0, 2, 1, 3).to(q.dtype)


# ----------------------------------------------------------------------------
# loss
# ----------------------------------------------------------------------------
def cross_entropy(logits: torch.Tensor, targets: torch.Tensor) -> torch.Tensor:
    """Mean next-token cross entropy over all rows; fp32 accumulate."""
    return F.cross_entropy(logits.float(), targets, reduction="mean")


def linear_cross_entropy(h: torch.Tensor, weight: torch.Tensor, targets: torch.Tensor,
                         chunk: int = 0) -> torch.Tensor:
    """``mean CE(h @ weight.T, targets)``; the CUDA path never materialises all logits."""
    return cross_entropy(h @ weight.t(), targets)


# ----------------------------------------------------------------------------
# optimizer
# ----------------------------------------------------------------------------
def adamw_step(p: torch.Tensor, g: torch.Tensor, m: torch.Tensor, v: torch.Tensor, *, lr: float,
               beta1: float, beta2: float, eps: float, weight_decay: float, step: int,
               grad_scale: float = 1.0) -> None:
    """In-place decoupled AdamW on fp32 tensors (the oracle for the fused kernel)."""
    gf = g.float() * grad_scale
    m.mul_(beta1).add_(gf, alpha=1 - beta1)
    v.mul_(beta2).addcmul_(gf, gf, value=1 - beta2)
    bc1 = 1 - beta1 ** step
    bc2 = 1 - beta2 ** step
    denom = (v / bc2).sqrt_().add_(eps)
    p.mul_(1 - lr * weight_decay).addcdiv_(m / bc1, denom, value=-lr)
