"""Row-parallel GEMM fused with its reduce-scatter over peer memory (tensor parallelism with sequence parallelism).

``y_r = sum over ranks q of (a_q @ w_q^T)[rows of rank r]``: every rank multiplies its slice of the contraction
dimension (attention output projection, second feed-forward matrix) and the partial products have to be summed and
scattered along the sequence.  Here the tcgen05 GEMM never writes its result locally: the epilogue of every 128-row
tile stores each row straight into the symmetric buffer of the rank that owns that row
(``csrc/gemm_tcgen05.cu: grouped_gemm_kernel<.., PUSH>``, plain 16-byte peer stores issued while the MMA warp runs the
next tile), slot ``local_row * world + sender``; the last block releases one flag per destination.  The owner then
sums its ``world`` partial rows in fp32 from local memory (``csrc/dispatch.cu: moe_combine_kernel<.., PUSHED>``), in
rank order, so the result does not depend on arrival order.  Two alternating receive regions and an acknowledgement
flag per peer keep a sender from overwriting partials the owner has not summed yet; every wait is bounded and ends in
the status word.

The same three kernels serve the expert GEMM + combine of the MoE block; this module only builds the row -> (owner,
slot) table of a ``[B, S, K]`` activation whose sequence dimension is split over the group.

Reference: GEMM + reduce-scatter in one kernel (``moe_reduce_rs.py``, "GEMM+Reduce-Scatter") in the tile-overlap study,
``notes/2026-04/2026-04-09_tileflow_mi355x_tile_overlap_analysis.md:18-28``; in-kernel P2P reduction,
``moe/research_direction_C.md:236-257``.
"""
from __future__ import annotations

import ctypes

import torch
import torch.distributed as dist

from ..ops import cuda as cops
from . import symm

cops.register("slab_moe_wait", "ppiiiips")
cops.register("slab_moe_signal_out", "ppiiis")
cops.register("slab_moe_reduce_pairs", "ppiiippiiipis")
cops.register("slab_grouped_gemm_bf16_push", "ipppp" + "iiii" + "ii" + "pp" + "ll" + "iiii" + "pp" + "s")

_MAXW = 16
_FLAGS = 4096            # bytes in front of the regions: push flags at 0, acknowledgement flags at 1024
_N_OFFSETS = 13          # fields of the dispatcher's workspace layout (csrc/dispatch.cu: WsLayout)
_OUT_FLAG, _COMB, _PUSH_FLAG = 3, 10, 11


class GemmReduceScatter:
    """One instance per (group, activation shape); ``__call__(a, w)`` returns this rank's ``[B, S / world, N]``."""

    def __init__(self, group, world: int, rank: int, device, batch: int, seq: int, n: int, workspace=None):
        if seq % world:
            raise ValueError(f"sequence length {seq} is not a multiple of the group size {world}")
        self.group, self.world, self.rank, self.device = group, world, rank, torch.device(device)
        self.batch, self.seq, self.n = batch, seq, n
        self.rows = batch * seq
        self.rows_local = self.rows // world
        self.region = (self.rows_local * world * n * 2 + 255) // 256 * 256
        nbytes = _FLAGS + 2 * self.region
        self.ws = workspace if workspace is not None else symm.SymmetricWorkspace(nbytes, group, world, rank,
                                                                                  self.device)
        self._ptrs = (ctypes.c_long * _MAXW)(*(list(self.ws.ptrs) + [0] * (_MAXW - len(self.ws.ptrs))))
        self._lay = []
        for half in range(2):
            off = [0] * _N_OFFSETS
            off[_PUSH_FLAG], off[_OUT_FLAG], off[_COMB] = 0, 1024, _FLAGS + half * self.region
            self._lay.append((ctypes.c_long * _N_OFFSETS)(*off))
        i32 = dict(dtype=torch.int32, device=self.device)
        # flattened row b * S + s belongs to rank s // (S / world), local row b * (S / world) + s % (S / world)
        s_local = seq // world
        r = torch.arange(self.rows, device=self.device)
        b, s = r // seq, r % seq
        slot = (b * s_local + s % s_local) * world + rank
        self.origin = (((s // s_local) << 24) | slot).to(torch.int32)
        self.pair_ok = torch.zeros(self.rows_local * world, **i32)          # every slot of the region holds a row
        self.counter = torch.zeros(1, **i32)
        self.status = cops.status_word(self.device)
        self.epoch = 0

    @staticmethod
    def nbytes(batch: int, seq: int, n: int, world: int) -> int:
        return _FLAGS + 2 * ((batch * seq * n * 2 + 255) // 256 * 256)

    # The two halves of an exchange are separate so that ranks emulated on one GPU can be run phase by phase.
    def push(self, a: torch.Tensor, w: torch.Tensor) -> int:
        """Multiply and send: ``a`` [rows, K] bf16, ``w`` [N, K] bf16.  Returns the epoch to pass to :meth:`reduce`."""
        self.epoch += 1
        ep = self.epoch
        lay = self._lay[ep & 1]
        if ep > 2:          # the owners must have summed what this rank sent into the same region two calls ago
            cops.call("slab_moe_wait", ctypes.addressof(self._ptrs), ctypes.addressof(lay), self.world, self.rank,
                      ep - 2, 1, self.status, cops.stream())
        offsets, counts = cops._dense_segments(self.device, self.rows)
        k = a.shape[1]
        cops.call("slab_grouped_gemm_bf16_push", 0, a, w, offsets, counts, 1, self.rows, self.n, k,
                  256 if self.n % 256 == 0 else 128, 0, self.origin, ctypes.addressof(self._ptrs),
                  _FLAGS + (ep & 1) * self.region, 0, self.world, self.rank, ep, self.rows_local * self.world,
                  self.counter, self.status, cops.stream())
        return ep

    def reduce(self, ep: int) -> torch.Tensor:
        lay = self._lay[ep & 1]
        y = torch.empty(self.rows_local, self.n, dtype=torch.bfloat16, device=self.device)
        cops.call("slab_moe_reduce_pairs", y, self.pair_ok, self.rows_local, self.world, self.n,
                  ctypes.addressof(self._ptrs), ctypes.addressof(lay), self.world, self.rank, ep, self.status, 0,
                  cops.stream())
        cops.call("slab_moe_signal_out", ctypes.addressof(self._ptrs), ctypes.addressof(lay), self.world, self.rank, ep,
                  cops.stream())
        return y

    def __call__(self, a: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
        return _GemmRS.apply(a, w, self)


class _GemmRS(torch.autograd.Function):
    """Forward: fused GEMM + reduce-scatter.  Backward: all-gather of the output gradient along the sequence (NCCL),
    then the two dense GEMMs of a linear layer on the gathered gradient."""

    @staticmethod
    def forward(ctx, a, w, op: GemmReduceScatter):
        a2 = a.reshape(-1, a.shape[-1])
        if not a2.is_contiguous():
            a2 = a2.contiguous()
        ctx.op, ctx.w_ref = op, w
        ctx.save_for_backward(a2, w)
        ctx.a_shape = a.shape
        y = op.reduce(op.push(a2, w))
        return y.view(op.batch, op.seq // op.world, op.n)

    @staticmethod
    def backward(ctx, g):
        from ..parallel.tp import _gather_seq
        op = ctx.op
        a2, w = ctx.saved_tensors
        g_full = _gather_seq(g.contiguous(), op.group, op.world).reshape(op.rows, op.n)
        n, k = w.shape
        off, cnt = cops._dense_segments(g.device, op.rows)
        da = dw = None
        if ctx.needs_input_grad[0]:
            da = torch.empty(ctx.a_shape, dtype=torch.bfloat16, device=g.device)
            cops.grouped_gemm_raw(1, g_full, w, off, cnt, n, k, out=da.view(-1, k), block_n=cops._pick_bn(k))
        if ctx.needs_input_grad[1]:
            mg = getattr(ctx.w_ref, "main_grad", None)
            if mg is not None:             # straight into the flat gradient buffer of the parameter's group
                cops.grouped_gemm_raw(2, g_full, a2, off, cnt, n, k, out=mg, accumulate=ctx.w_ref.main_grad_written,
                                      block_n=cops._pick_bn(k))
                ctx.w_ref.main_grad_written = True
            else:
                dw = cops.grouped_gemm_raw(2, g_full, a2, off, cnt, n, k, block_n=cops._pick_bn(k)).view(n, k)
        return da, dw, None
