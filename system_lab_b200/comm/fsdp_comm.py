"""Peer-memory FSDP collectives (kernels in ``csrc/fsdp_comm.cu``): parameter all-gather and gradient
reduce-scatter (+ cast, optionally + sharded AdamW) that pull slices straight from the peers' staging
slots over NVLink instead of calling NCCL.

One :class:`FsdpPeerComm` per shard group.  Its symmetric workspace holds ``NSLOT`` staging slots used in
rotation; a slot is reused only after every peer acknowledged reading its previous content, so a fast
rank can run at most ``NSLOT`` collectives ahead of the slowest.  The workspace grows (collectively) the
first time a larger operand shows up.
"""
from __future__ import annotations

import ctypes

import torch

from ..ops import cuda as cops
from .symm import SymmetricWorkspace

NSLOT = 4
_MAXW = 16

for _name, _sig in {
    "slab_fsdp_stage": "plppiiiiipps",
    "slab_fsdp_all_gather": "plppiiiipps",
    "slab_fsdp_reduce_scatter": "plppiiiifpps",
    "slab_fsdp_reduce_scatter_adamw": "lppiiiif" + "ppppp" + "p" + "fffffff" + "l" + "pps",
    "slab_fsdp_set_wait_limit_ms": "l",
    "slab_fsdp_gather_range": "plllppiiiips",
    "slab_dense_gemm_gather": "pppp" + "iiii" + "p" + "llll" + "pp" + "iiii" + "pip" + "ps",
}.items():
    cops.register(_name, _sig)


class FsdpPeerComm:
    def __init__(self, group, world: int, rank: int, device: torch.device, workspace_factory=None):
        self.group, self.world, self.rank, self.device = group, world, rank, device
        self.ws = None
        self.slot_bytes = 0
        self.epoch = 0
        self.slot_last = [0] * NSLOT
        self.done = torch.zeros(1, dtype=torch.int32, device=device)
        self.status = cops.status_word(device)
        self._factory = workspace_factory or (lambda nbytes: SymmetricWorkspace(nbytes, group, world, rank, device))
        # reduce-scatter through the switch (``multimem.ld_reduce`` on the workspaces' multicast address) instead of
        # one peer load per rank; needs a multicast mapping (NVSwitch) and a free entry in the pointer table
        self.nvls = False

    def _ensure(self, nbytes: int) -> None:
        if self.ws is not None and nbytes <= self.slot_bytes:
            return
        self.slot_bytes = (max(nbytes, 1 << 20) + 255) // 256 * 256
        self.ws = self._factory(4096 + NSLOT * self.slot_bytes)
        self._ptrs = (ctypes.c_long * _MAXW)(*(list(self.ws.ptrs) + [0] * (_MAXW - len(self.ws.ptrs))))
        mc = int(getattr(self.ws, "multicast_ptr", 0) or 0)
        self.nvls_active = bool(self.nvls and mc and self.world < _MAXW)
        if self.nvls_active:
            self._ptrs[self.world] = mc         # the entry behind the last rank: multicast address (csrc/fsdp_comm.cu)
        self._lay = (ctypes.c_long * 4)(0, 1024, 4096, self.slot_bytes)
        self.slot_last = [0] * NSLOT

    def _next(self):
        self.epoch += 1
        slot = self.epoch % NSLOT
        ack = self.slot_last[slot]
        self.slot_last[slot] = self.epoch
        return slot, self.epoch, ack

    def _stage(self, src: torch.Tensor, slot: int, ep: int, ack: int) -> None:
        cops.call("slab_fsdp_stage", src, src.numel() * src.element_size(), ctypes.addressof(self._ptrs),
                  ctypes.addressof(self._lay), self.world, self.rank, slot, ep, ack, self.status, self.done,
                  cops.stream())

    # ---- the FlatGroup interface --------------------------------------------------------------------
    def all_gather(self, dst: torch.Tensor, src: torch.Tensor, fg=None) -> None:
        src = src.contiguous()
        nbytes = src.numel() * src.element_size()
        self._ensure(nbytes)
        slot, ep, ack = self._next()
        self._stage(src, slot, ep, ack)
        cops.call("slab_fsdp_all_gather", dst, nbytes, ctypes.addressof(self._ptrs), ctypes.addressof(self._lay),
                  self.world, self.rank, slot, ep, self.status, self.done, cops.stream())

    # ---- all-gather fused into the first GEMM that consumes the gathered weights -----------------------------------
    PIECE_BYTES = 1024 * 1024

    def begin_gather(self, dst: torch.Tensor, src: torch.Tensor, head_bytes: int):
        """First half of a fused all-gather: stage this rank's shard and pull only the bytes behind ``head_bytes`` of
        the gathered buffer (the group's 1-D parameters, which the layer's norm reads before its first GEMM).  The
        head -- the matrices -- is gathered by :meth:`gemm_gather`, inside the GEMM that multiplies the first of them
        (or by :meth:`finish_gather` if no such GEMM comes).  Returns the ticket both take."""
        ticket = self.stage_for_gather(src, head_bytes)
        self.gather_tail(ticket, dst)
        return ticket

    def stage_for_gather(self, src: torch.Tensor, head_bytes: int):
        """Stage this rank's shard (sets flags only: the emulated-rank tests run this phase for every rank first)."""
        src = src.contiguous()
        nbytes = src.numel() * src.element_size()
        self._ensure(nbytes)
        slot, ep, ack = self._next()
        self._stage(src, slot, ep, ack)
        total = nbytes * self.world
        head = min(max(head_bytes, 0), total) // 512 * 512          # the GEMM gathers [0, head_up), the tail kernel the rest
        head_up = min((head_bytes + 511) // 512 * 512, total // 512 * 512)
        return {"slot": slot, "epoch": ep, "shard_bytes": nbytes, "head_bytes": head_up, "tail_from": head, "total": total}

    def gather_tail(self, ticket, dst: torch.Tensor) -> None:
        """Pull the bytes behind the matrices (waits for every rank's staged flag)."""
        if ticket["tail_from"] < ticket["total"]:
            cops.call("slab_fsdp_gather_range", dst, ticket["tail_from"], ticket["total"], ticket["shard_bytes"],
                      ctypes.addressof(self._ptrs), ctypes.addressof(self._lay), self.world, self.rank, ticket["slot"],
                      ticket["epoch"], self.status, cops.stream())

    def gemm_gather(self, ticket, x2: torch.Tensor, w: torch.Tensor, out2: torch.Tensor, flat: torch.Tensor, w_off: int,
                    seg, pieces: torch.Tensor, call_index: int, block_n: int) -> None:
        """``out2 = x2 @ w^T`` while the kernel gathers bytes ``[0, head_bytes)`` of ``flat`` from the staged shards
        (``csrc/gemm_tcgen05.cu``, gather warp) and acknowledges the slot."""
        n, k = w.shape
        cops.call("slab_dense_gemm_gather", x2, out2, seg[0], seg[1], x2.shape[0], n, k, block_n, flat,
                  w_off * 2, ticket["head_bytes"], ticket["shard_bytes"], self.PIECE_BYTES,
                  ctypes.addressof(self._ptrs), ctypes.addressof(self._lay), self.world, self.rank, ticket["slot"],
                  ticket["epoch"], pieces, call_index, self.done, self.status, cops.stream())

    def finish_gather(self, ticket, dst: torch.Tensor) -> None:
        """Plain gather of everything (and the acknowledgement) for a ticket no GEMM consumed."""
        cops.call("slab_fsdp_all_gather", dst, ticket["shard_bytes"], ctypes.addressof(self._ptrs),
                  ctypes.addressof(self._lay), self.world, self.rank, ticket["slot"], ticket["epoch"], self.status,
                  self.done, cops.stream())

    def reduce_scatter(self, grad_full: torch.Tensor, fg=None, scale: float = 1.0) -> torch.Tensor:
        """bf16 ``grad_full`` (``world * shard`` elements) -> fp32 sum of every rank's slice ``rank``."""
        if grad_full.dtype != torch.bfloat16:
            raise ValueError("peer reduce-scatter takes bf16 gradients")
        shard = grad_full.numel() // self.world
        self._ensure(grad_full.numel() * 2)
        slot, ep, ack = self._next()
        self._stage(grad_full, slot, ep, ack)
        piece = torch.empty(shard, dtype=torch.float32, device=self.device)
        cops.call("slab_fsdp_reduce_scatter", piece, shard, ctypes.addressof(self._ptrs), ctypes.addressof(self._lay),
                  self.world, self.rank, slot, ep, float(scale), self.status, self.done, cops.stream())
        return piece

    def reduce_scatter_adamw(self, grad_full, master, m, v, out_bf16, coef, sq_out, *, lr, beta1, beta2, eps,
                             weight_decay, step, scale: float = 1.0, decay_end: int | None = None) -> None:
        """Reduce-scatter fused with the AdamW update of this rank's fp32 master shard and moments."""
        shard = grad_full.numel() // self.world
        self._ensure(grad_full.numel() * 2)
        slot, ep, ack = self._next()
        self._stage(grad_full, slot, ep, ack)
        cops.call("slab_fsdp_reduce_scatter_adamw", shard, ctypes.addressof(self._ptrs), ctypes.addressof(self._lay),
                  self.world, self.rank, slot, ep, float(scale), master, m, v, out_bf16, coef, sq_out, float(lr),
                  float(beta1), float(beta2), float(eps), float(weight_decay), float(1 - beta1 ** step),
                  float(1 - beta2 ** step), int(shard if decay_end is None else decay_end), self.status, self.done,
                  cops.stream())


def make_fsdp_comms(mesh, device, nvls: bool = False):
    """(dense_comm, expert_comm) for the engine; ``None`` where the group has a single rank."""
    dense, expert = _make_fsdp_comms(mesh, device)
    for c in (dense, expert):
        if c is not None:
            c.nvls = nvls
    return dense, expert


def _make_fsdp_comms(mesh, device):
    if mesh.replicas > 1:          # hybrid sharding: the peer collectives span one block of the data axis
        dense = (FsdpPeerComm(mesh.data_shard_group, mesh.data_shard_size, mesh.data_shard_rank, device)
                 if mesh.data_shard_size > 1 else None)
    else:
        dense = FsdpPeerComm(mesh.data_group, mesh.data_size, mesh.data_rank, device) if mesh.data_size > 1 else None
    expert = None
    if mesh.edp_replicas > 1:
        if mesh.edp_shard_size > 1:
            expert = FsdpPeerComm(mesh.edp_shard_group, mesh.edp_shard_size, mesh.edp_shard_rank, device)
    elif mesh.edp > 1:
        expert = FsdpPeerComm(mesh.edp_group, mesh.edp, mesh.edp_rank * mesh.cp + mesh.cp_rank, device)
    return dense, expert
