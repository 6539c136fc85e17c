"""Tensor parallelism: attention heads and dense feed-forward columns split over ``tp`` ranks that share the same
tokens; MoE blocks treat those ranks as extra data ranks (each takes ``1 / tp`` of the tokens).

The four autograd links are the usual conjugate pairs: ``copy_to`` (identity forward, all-reduce backward) in front
of a column-split matrix, ``reduce_from`` (all-reduce forward, identity backward) behind a row-split one;
``scatter_rows`` (slice forward, all-gather backward) in front of a MoE block and ``gather_rows`` (all-gather
forward, slice backward) behind it.  Parameters that stay replicated but see only a slice of the tokens (router,
shared expert) are marked ``tp_partial_grad``; the engine sums their gradients over the group.

Reference: tensor parallelism is a configuration axis of the tuner (legality rules
``skills/pilot/constraints/config.md:41-48``); every measured configuration of the reference ran ``tp = 1``.  The
attention ``tp x cp x dp`` / MoE ``ep x edp`` folding follows ``moe/MegatronCore_MoE_reading_notes.md:159-195``.
"""
from __future__ import annotations

import torch
import torch.distributed as dist


class _CopyTo(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return x.view_as(x)

    @staticmethod
    def backward(ctx, g):
        g = g.contiguous()
        dist.all_reduce(g, group=ctx.group)
        return g, None


class _ReduceFrom(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group):
        x = x.contiguous()
        dist.all_reduce(x, group=group)
        return x

    @staticmethod
    def backward(ctx, g):
        return g, None


class _ScatterRows(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group, rank, size):
        ctx.group, ctx.rank, ctx.size = group, rank, size
        per = x.shape[0] // size
        return x[rank * per:(rank + 1) * per].contiguous()

    @staticmethod
    def backward(ctx, g):
        g = g.contiguous()
        out = torch.empty((g.shape[0] * ctx.size,) + tuple(g.shape[1:]), dtype=g.dtype, device=g.device)
        dist.all_gather_into_tensor(out, g, group=ctx.group)
        return out, None, None, None


class _GatherRows(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group, rank, size):
        ctx.group, ctx.rank, ctx.size = group, rank, size
        x = x.contiguous()
        out = torch.empty((x.shape[0] * size,) + tuple(x.shape[1:]), dtype=x.dtype, device=x.device)
        dist.all_gather_into_tensor(out, x, group=group)
        return out

    @staticmethod
    def backward(ctx, g):
        per = g.shape[0] // ctx.size
        return g[ctx.rank * per:(ctx.rank + 1) * per].contiguous(), None, None, None


class TensorParallel:
    """The group as the model sees it.  ``None`` stands for ``tp == 1`` everywhere in the model code."""

    def __init__(self, group, rank: int, size: int):
        self.group, self.rank, self.size = group, rank, size

    def copy_to(self, x):
        return _CopyTo.apply(x, self.group)

    def reduce_from(self, x):
        return _ReduceFrom.apply(x, self.group)

    def scatter_rows(self, x):
        return _ScatterRows.apply(x, self.group, self.rank, self.size)

    def gather_rows(self, x):
        return _GatherRows.apply(x, self.group, self.rank, self.size)

    def segments(self, parts: list[int]) -> list[tuple[int, int]]:
        """This rank's ``(start, length)`` pieces of a dimension that is the concatenation of ``parts``, each part
        split evenly over the group (e.g. the q, k and v row blocks of a packed projection)."""
        out, base = [], 0
        for n in parts:
            per = n // self.size
            out.append((base + self.rank * per, per))
            base += n
        return out


def mark_sharded(p, dim: int, global_shape, segments) -> None:
    """Record how ``p`` is cut out of its global tensor: weight init draws the global tensor and keeps
    ``segments`` of dimension ``dim``; the checkpoint stores the piece under its tensor-parallel rank."""
    p.tp_dim, p.tp_global_shape, p.tp_segments = dim, tuple(global_shape), list(segments)


def take_segments(full: torch.Tensor, dim: int, segments) -> torch.Tensor:
    return torch.cat([full.narrow(dim, s, n) for s, n in segments], dim=dim)
