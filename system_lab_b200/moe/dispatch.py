"""Token dispatch / combine across the expert-parallel group.

Four primitives act on a fixed :class:`RoutingPlan`:

=================  =======================================================  ====================
primitive          computes                                                 backward
=================  =======================================================  ====================
dispatch_rows      row of token ``t`` -> the slot of every pair ``(t,k)``   combine_rows (sum)
dispatch_scalars   ``p[t,k]`` -> one fp32 per slot                          combine_scalars
combine_rows       ``y[t] = sum_k w[t,k] * ye[slot(t,k)]``                  dispatch_rows
combine_scalars    per-slot fp32 -> ``s[t,k]``                              dispatch_scalars
=================  =======================================================  ====================

Two back-ends implement them:

* :class:`AllToAllDispatcher` — the library baseline: sort by expert, ``all_to_all_single``
  (NCCL on GPUs, gloo on CPU), re-sort chunks on the receiver.  This is the
  Gate→Permute→A2A→GEMM→A2A→Permute→Combine pipeline the reference measures
  (``notes/2026-04/2026-04-14_moe_e2e_performance_benchmark.md:25-37``).  It needs the
  per-rank counts on the host to size the collective.
* ``FusedDispatcher`` (``moe/fused_dispatch.py``) — hand written kernels that write rows
  straight into the peers' expert-major buffers over NVLink.

Receiver layout (both back-ends): rows grouped by local expert, each expert's segment starts at a
multiple of ``pad_to`` rows (a GEMM M-tile), sources in rank order inside a segment — the
"Layout C" grouping of ``notes/2026-04/2026-04-14_data_layout_analysis.md:322-330`` folded into one
contiguous expert-major array so the grouped GEMM needs no second permute.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.distributed as dist


@dataclass
class RoutingPlan:
    num_tokens: int
    topk: int
    num_experts: int
    ep: int
    pad_to: int
    sort_idx: torch.Tensor          # [T*K] pair index in (dst rank, local expert, token) order
    send_counts: torch.Tensor       # [ep, E_local] rows this rank sends
    recv_counts: torch.Tensor       # [ep, E_local] rows this rank receives, by source
    expert_offsets: torch.Tensor    # [E_local] first row of each local expert (aligned)
    expert_counts: torch.Tensor     # [E_local] valid rows per local expert
    num_rows: int                   # rows of the receive array (incl. alignment padding)
    recv_row_index: torch.Tensor    # [n_recv] row in the receive array for each arriving row
    in_splits: list | None = None   # host copies for all_to_all_single
    out_splits: list | None = None
    tokens_per_expert_global: torch.Tensor | None = None  # [E] routed pairs from this rank

    @property
    def e_local(self) -> int:
        return self.num_experts // self.ep


def _round_up(x: torch.Tensor, m: int) -> torch.Tensor:
    return (x + m - 1) // m * m


class AllToAllDispatcher:
    """Baseline dispatcher on ``torch.distributed.all_to_all_single``."""

    def __init__(self, group: dist.ProcessGroup | None, num_experts: int, pad_to: int = 1):
        self.group = group
        self.ep = dist.get_world_size(group) if (group is not None and dist.is_initialized()) else 1
        self.num_experts = num_experts
        self.pad_to = max(int(pad_to), 1)

    # -- plan ------------------------------------------------------------
    @torch.no_grad()
    def plan(self, topk_idx: torch.Tensor) -> RoutingPlan:
        t, k = topk_idx.shape
        e, ep = self.num_experts, self.ep
        e_local = e // ep
        flat = topk_idx.reshape(-1)
        sort_idx = torch.argsort(flat, stable=True)
        counts = torch.bincount(flat, minlength=e)
        send_counts = counts.reshape(ep, e_local)
        if ep > 1:
            recv_counts = torch.empty_like(send_counts)
            dist.all_to_all_single(recv_counts, send_counts.contiguous(), group=self.group)
        else:
            recv_counts = send_counts.clone()
        expert_counts = recv_counts.sum(0)
        padded = _round_up(expert_counts, self.pad_to)
        expert_offsets = torch.cumsum(padded, 0) - padded
        # arriving order is [src][local expert][slot]; target is [local expert][src][slot]
        src_base = torch.cumsum(recv_counts, 0) - recv_counts            # rows of e from sources < src
        seg_start = (expert_offsets[None, :] + src_base).reshape(-1)       # [ep*E_local]
        seg_len = recv_counts.reshape(-1)
        n_recv = int(seg_len.sum())
        seg_first = torch.cumsum(seg_len, 0) - seg_len
        seg_id = torch.repeat_interleave(torch.arange(seg_len.numel(), device=flat.device), seg_len,
                                         output_size=n_recv)
        pos = torch.arange(n_recv, device=flat.device)
        recv_row_index = seg_start[seg_id] + (pos - seg_first[seg_id])
        num_rows = int(padded.sum())
        return RoutingPlan(
            num_tokens=t, topk=k, num_experts=e, ep=ep, pad_to=self.pad_to, sort_idx=sort_idx,
            send_counts=send_counts, recv_counts=recv_counts, expert_offsets=expert_offsets,
            expert_counts=expert_counts, num_rows=max(num_rows, self.pad_to), recv_row_index=recv_row_index,
            in_splits=send_counts.sum(1).tolist(), out_splits=recv_counts.sum(1).tolist(),
            tokens_per_expert_global=counts)

    # -- raw data movement (no autograd) ----------------------------------
    def _a2a(self, x: torch.Tensor, in_splits, out_splits) -> torch.Tensor:
        if self.ep == 1:
            return x
        out = x.new_empty((sum(out_splits),) + tuple(x.shape[1:]))
        dist.all_to_all_single(out, x.contiguous(), out_splits, in_splits, group=self.group)
        return out

    def _send_pairs(self, plan: RoutingPlan, pairs: torch.Tensor) -> torch.Tensor:
        """pairs: [T*K, ...] in pair order -> receive array [num_rows, ...] (padding rows zero)."""
        got = self._a2a(pairs[plan.sort_idx], plan.in_splits, plan.out_splits)
        out = got.new_zeros((plan.num_rows,) + tuple(got.shape[1:]))
        out[plan.recv_row_index] = got
        return out

    def _return_pairs(self, plan: RoutingPlan, rows: torch.Tensor) -> torch.Tensor:
        """receive-array rows [num_rows, ...] -> [T*K, ...] in pair order."""
        back = self._a2a(rows[plan.recv_row_index], plan.out_splits, plan.in_splits)
        out = torch.empty_like(back)
        out[plan.sort_idx] = back
        return out

    # -- differentiable primitives -----------------------------------------
    def dispatch_rows(self, plan: RoutingPlan, x: torch.Tensor) -> torch.Tensor:
        return _DispatchRows.apply(x, self, plan)

    def dispatch_scalars(self, plan: RoutingPlan, p: torch.Tensor) -> torch.Tensor:
        return _DispatchScalars.apply(p, self, plan)

    def combine_rows(self, plan: RoutingPlan, ye: torch.Tensor, weights: torch.Tensor | None = None,
                     dead: bool = False) -> torch.Tensor:
        """``dead``: the caller only needs the autograd node (a recomputed forward whose result nobody reads), so
        the exchange is skipped and the returned values are unspecified.  Every rank must pass the same flag."""
        if weights is None:
            return _CombineRows.apply(ye, self, plan, dead)
        return _CombineRowsWeighted.apply(ye, weights, self, plan)

    def keep_dispatched(self, plan: RoutingPlan, xe: torch.Tensor, pe: torch.Tensor | None):
        """What a recomputed block keeps of its first dispatch (the all-to-all results are fresh tensors)."""
        return xe.detach(), (pe.detach() if pe is not None else None)

    def redispatch_kept(self, plan: RoutingPlan, x: torch.Tensor, probs: torch.Tensor | None, xs: torch.Tensor,
                        ps: torch.Tensor | None):
        """Differentiable stand-in for the two dispatch calls that moves nothing forward: returns the kept
        rows / scalars; the backward passes are those of ``dispatch_rows`` / ``dispatch_scalars``."""
        xe = _KeptRows.apply(x, xs, self, plan)
        pe = _KeptScalars.apply(probs, ps, self, plan) if probs is not None else None
        return xe, pe

    def combine_scalars(self, plan: RoutingPlan, se: torch.Tensor) -> torch.Tensor:
        return _CombineScalars.apply(se, self, plan)


class _DispatchRows(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, d, plan):
        ctx.d, ctx.plan = d, plan
        t, k = plan.num_tokens, plan.topk
        pairs = x[:, None, :].expand(t, k, x.shape[-1]).reshape(t * k, -1)
        return d._send_pairs(plan, pairs)

    @staticmethod
    def backward(ctx, g):
        d, plan = ctx.d, ctx.plan
        back = d._return_pairs(plan, g.contiguous())
        return back.reshape(plan.num_tokens, plan.topk, -1).sum(1), None, None


class _KeptRows(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, xs, d, plan):
        ctx.d, ctx.plan = d, plan
        return xs.view_as(xs)

    @staticmethod
    def backward(ctx, g):
        return _DispatchRows.backward(ctx, g) + (None,)


class _KeptScalars(torch.autograd.Function):
    @staticmethod
    def forward(ctx, p, ps, d, plan):
        ctx.d, ctx.plan = d, plan
        return ps.view_as(ps)

    @staticmethod
    def backward(ctx, g):
        return _DispatchScalars.backward(ctx, g) + (None,)


class _DispatchScalars(torch.autograd.Function):
    @staticmethod
    def forward(ctx, p, d, plan):
        ctx.d, ctx.plan = d, plan
        return d._send_pairs(plan, p.reshape(-1).float())

    @staticmethod
    def backward(ctx, g):
        d, plan = ctx.d, ctx.plan
        return d._return_pairs(plan, g.contiguous()).reshape(plan.num_tokens, plan.topk), None, None


class _CombineRows(torch.autograd.Function):
    @staticmethod
    def forward(ctx, ye, d, plan, dead=False):
        ctx.d, ctx.plan = d, plan
        if dead:
            return ye.new_zeros(plan.num_tokens, ye.shape[-1])
        back = d._return_pairs(plan, ye)
        return back.reshape(plan.num_tokens, plan.topk, -1).float().sum(1).to(ye.dtype)

    @staticmethod
    def backward(ctx, g):
        d, plan = ctx.d, ctx.plan
        t, k = plan.num_tokens, plan.topk
        pairs = g[:, None, :].expand(t, k, g.shape[-1]).reshape(t * k, -1)
        return d._send_pairs(plan, pairs), None, None, None


class _CombineRowsWeighted(torch.autograd.Function):
    @staticmethod
    def forward(ctx, ye, w, d, plan):
        ctx.d, ctx.plan = d, plan
        back = d._return_pairs(plan, ye).reshape(plan.num_tokens, plan.topk, -1)
        ctx.save_for_backward(back, w)
        return (back.float() * w.float().unsqueeze(-1)).sum(1).to(ye.dtype)

    @staticmethod
    def backward(ctx, g):
        d, plan = ctx.d, ctx.plan
        back, w = ctx.saved_tensors
        t, k = plan.num_tokens, plan.topk
        gw = (back.float() * g.float().unsqueeze(1)).sum(-1).to(w.dtype)
        pairs = (g.float().unsqueeze(1) * w.float().unsqueeze(-1)).to(g.dtype).reshape(t * k, -1)
        return d._send_pairs(plan, pairs), gw, None, None


class _CombineScalars(torch.autograd.Function):
    @staticmethod
    def forward(ctx, se, d, plan):
        ctx.d, ctx.plan = d, plan
        return d._return_pairs(plan, se).reshape(plan.num_tokens, plan.topk)

    @staticmethod
    def backward(ctx, g):
        d, plan = ctx.d, ctx.plan
        return d._send_pairs(plan, g.reshape(-1).contiguous()), None, None
