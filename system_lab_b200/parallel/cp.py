"""Context parallelism, head-sharded ("Ulysses") form.

Each context rank holds ``S/cp`` tokens of every sequence.  Around attention, one all-to-all swaps
the sharded axis from sequence to heads (``[B, S/cp, H, D] -> [B, S, H/cp, D]``), attention runs
on whole sequences for a slice of heads, and a second all-to-all swaps back.  This is the CP-A2A
variant of ``moe/MegatronCore_MoE_reading_notes.md:631-680``; it reuses all-to-all machinery and is
the intra-node choice on an NVSwitch box (ring/P2P CP is the inter-node choice and is not built).
KV heads are replicated up to ``cp`` when there are fewer KV heads than context ranks.
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from .. import ops


def _seq_to_heads(x: torch.Tensor, group) -> torch.Tensor:
    """[B, s, H, D] -> [B, s*cp, H/cp, D]"""
    cp = dist.get_world_size(group)
    b, s, h, d = x.shape
    xs = x.reshape(b, s, cp, h // cp, d).permute(2, 0, 1, 3, 4).contiguous()      # [cp, B, s, H/cp, D]
    out = torch.empty_like(xs)
    dist.all_to_all_single(out, xs, group=group)
    return out.permute(1, 0, 2, 3, 4).reshape(b, cp * s, h // cp, d)             # chunks in rank order


def _heads_to_seq(x: torch.Tensor, group) -> torch.Tensor:
    """[B, s*cp, H/cp, D] -> [B, s, H, D]"""
    cp = dist.get_world_size(group)
    b, S, hl, d = x.shape
    s = S // cp
    xs = x.reshape(b, cp, s, hl, d).permute(1, 0, 2, 3, 4).contiguous()           # [cp, B, s, H/cp, D]
    out = torch.empty_like(xs)
    dist.all_to_all_single(out, xs, group=group)
    return out.permute(1, 2, 0, 3, 4).reshape(b, s, cp * hl, d)


class _SeqToHeads(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return _seq_to_heads(x, group)

    @staticmethod
    def backward(ctx, g):
        return _heads_to_seq(g.contiguous(), ctx.group), None


class _HeadsToSeq(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return _heads_to_seq(x, group)

    @staticmethod
    def backward(ctx, g):
        return _seq_to_heads(g.contiguous(), ctx.group), None


def ulysses_attention(q, k, v, group, scale=None, window: int = 0):
    cp = dist.get_world_size(group)
    hkv = k.shape[2]
    if hkv % cp:
        rep = cp // hkv if cp % hkv == 0 else cp
        k = k.repeat_interleave(rep, dim=2)
        v = v.repeat_interleave(rep, dim=2)
    qh = _SeqToHeads.apply(q.contiguous(), group)
    kh = _SeqToHeads.apply(k.contiguous(), group)
    vh = _SeqToHeads.apply(v.contiguous(), group)
    o = ops.causal_attention(qh, kh, vh, scale, window)
    return _HeadsToSeq.apply(o.contiguous(), group)
