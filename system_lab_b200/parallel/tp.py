"""Tensor parallelism: attention heads and dense feed-forward columns split over ``tp`` ranks that share the same
tokens; MoE blocks treat those ranks as extra data ranks (each takes ``1 / tp`` of the tokens).

The four autograd links are the usual conjugate pairs: ``copy_to`` (identity forward, all-reduce backward) in front
of a column-split matrix, ``reduce_from`` (all-reduce forward, identity backward) behind a row-split one;
``scatter_rows`` (slice forward, all-gather backward) in front of a MoE block and ``gather_rows`` (all-gather
forward, slice backward) behind it.  Parameters that stay replicated but see only a slice of the tokens (router,
shared expert) are marked ``tp_partial_grad``; the engine sums their gradients over the group.

Sequence parallelism (``sequence_parallel``, needs ``tp > 1``): between the tensor-parallel regions the residual
stream, the norms and the MoE blocks hold ``1 / tp`` of every sequence (``[B, S / tp, H]``).  ``enter`` then is an
all-gather along the sequence in front of a column-split matrix (reduce-scatter in backward) and ``leave`` a
reduce-scatter behind a row-split one (all-gather in backward): the same bytes as the two all-reduces of plain tensor
parallelism, with ``tp`` times less activation memory outside the attention and feed-forward matrices.  Parameters that
are replicated but see only the local part of the sequence (norm gains, embedding, head) get partial gradients like
the router's (``tp_partial_grad``), and the loss is the mean over the group of the per-rank means.

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


def _gather_seq(x, group, size):
    """[B, S/size, ...] on every rank -> [B, S, ...] (rank r holds positions [r S/size, (r+1) S/size))."""
    x = x.contiguous()
    out = torch.empty((size * x.shape[0],) + tuple(x.shape[1:]), dtype=x.dtype, device=x.device)
    dist.all_gather_into_tensor(out, x, group=group)
    out = out.view((size,) + tuple(x.shape))
    return out.transpose(0, 1).reshape((x.shape[0], size * x.shape[1]) + tuple(x.shape[2:]))


def _reduce_scatter_seq(x, group, size):
    """Sum over the group of [B, S, ...], this rank keeps its [B, S/size, ...]."""
    b, s = x.shape[0], x.shape[1]
    parts = x.reshape((b, size, s // size) + tuple(x.shape[2:])).transpose(0, 1).contiguous()
    out = torch.empty(parts.shape[1:], dtype=x.dtype, device=x.device)
    dist.reduce_scatter_tensor(out, parts.view((size * b,) + tuple(parts.shape[2:])), group=group)
    return out


class _GatherSeq(torch.autograd.Function):
    """All-gather along the sequence; backward reduce-scatters (the consumers are this rank's slices of a
    column-split matrix, so the gradients of the ranks add up) or, with ``reduce=False``, keeps this rank's slice
    (the consumers compute the same thing on every rank)."""

    @staticmethod
    def forward(ctx, x, group, rank, size, reduce):
        ctx.group, ctx.rank, ctx.size, ctx.reduce = group, rank, size, reduce
        return _gather_seq(x, group, size)

    @staticmethod
    def backward(ctx, g):
        if ctx.reduce:
            return _reduce_scatter_seq(g, ctx.group, ctx.size), None, None, None, None
        per = g.shape[1] // ctx.size
        return g[:, ctx.rank * per:(ctx.rank + 1) * per].contiguous(), None, None, None, None


class _ReduceScatterSeq(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group, size):
        ctx.group, ctx.size = group, size
        return _reduce_scatter_seq(x, group, size)

    @staticmethod
    def backward(ctx, g):
        return _gather_seq(g, ctx.group, ctx.size), None, None


class _MeanOverGroup(torch.autograd.Function):
    """The scalar loss of a sequence-parallel group: mean of the per-rank means (every rank holds the same number of
    positions); each rank's own loss gets ``1 / size`` of the gradient."""

    @staticmethod
    def forward(ctx, loss, group, size):
        ctx.size = size
        out = loss.detach().clone()
        dist.all_reduce(out, group=group)
        return out / size

    @staticmethod
    def backward(ctx, g):
        return g / ctx.size, None, None


class TensorParallel:
    """The group as the model sees it.  ``None`` stands for ``tp == 1`` everywhere in the model code."""

    def __init__(self, group, rank: int, size: int, sequence_parallel: bool = False):
        self.group, self.rank, self.size = group, rank, size
        self.sequence_parallel = sequence_parallel
        self.fused_gemm_rs = False        # set by the engine (``tp_fused_gemm_reduce_scatter``)
        self._gemm_rs = {}                # (batch, sequence, output width) -> GemmReduceScatter

    def enter(self, x):
        """In front of a column-split matrix whose input nothing else on this rank consumes."""
        if self.sequence_parallel:
            return _GatherSeq.apply(x, self.group, self.rank, self.size, True)
        return _CopyTo.apply(x, self.group)

    def leave(self, x):
        """Behind a row-split matrix: sum the partial products over the group."""
        if self.sequence_parallel:
            return _ReduceScatterSeq.apply(x, self.group, self.size)
        return _ReduceFrom.apply(x, self.group)

    def linear_leave(self, x, w):
        """``leave(x @ w^T)`` for a row-split ``w``.  With sequence parallelism on the GPU kernel path
        (``fused_gemm_rs``) the GEMM's epilogue pushes its tiles to the owners of the rows over peer memory and the
        owners sum the partial rows: one exchange inside the GEMM instead of a GEMM followed by a reduce-scatter."""
        from .. import ops
        if self.sequence_parallel and self.fused_gemm_rs and x.dim() == 3 and x.is_cuda and ops.dense_kernels() \
                and ops.kernel_mode() == "auto":
            from ..ops import cuda as cops
            if cops.linear_ok(x, w) and x.shape[1] % self.size == 0:
                from ..comm.gemm_rs import GemmReduceScatter
                key = (x.shape[0], x.shape[1], w.shape[0])
                op = self._gemm_rs.get(key)
                if op is None:
                    op = self._gemm_rs[key] = GemmReduceScatter(self.group, self.size, self.rank, x.device, *key)
                return op(x, w)
        return self.leave(ops.linear(x, w))

    def gather_seq(self, x):
        """Whole sequences for a computation every rank repeats (identity without sequence parallelism)."""
        if self.sequence_parallel:
            return _GatherSeq.apply(x, self.group, self.rank, self.size, False)
        return x

    def local_seq(self, x):
        """This rank's positions of ``[B, S, ...]`` data that every rank of the group holds (token ids, targets)."""
        if not self.sequence_parallel:
            return x
        per = x.shape[1] // self.size
        return x[:, self.rank * per:(self.rank + 1) * per].contiguous()

    def mean_loss(self, loss):
        return _MeanOverGroup.apply(loss, self.group, self.size) if self.sequence_parallel else loss

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
