"""Fully sharded data parallel engine: flat, block-aligned parameter shards per layer.

Design (B200-first; digests: ``moe/veScale_FSDP_reading_notes.md:74-100`` block-aligned ragged
shards, ``moe/MegatronCore_MoE_reading_notes.md:266-284`` dual dense/expert mesh with persistent
buffers):

* A **unit** is one decoder layer (or the embedding, or the head).  Its parameters are packed into at
  most two **flat groups**: dense parameters sharded over every data rank of the pipeline stage, and
  expert parameters sharded over the ranks that own the same experts.
* Every parameter starts on a multiple of 128 elements inside the flat buffer and the per-rank shard
  length is a multiple of 128, so a 1x128 / 128x128 fp8 scale block never straddles two ranks and
  every shard is 256-byte aligned for bulk copies.
* The owned shard (fp32 master, or the bf16 weights themselves when ``master_weights`` is off) is the
  source of truth.  ``gather()`` materialises the full flat buffer in the compute dtype and the
  module's parameters are views into it; ``release()`` drops its storage.
* Gradients are written by autograd straight into a flat gradient buffer (``p.grad`` are views),
  reduce-scattered into the shard, accumulated over micro-batches in fp32 and consumed by the
  fused AdamW kernel.

With one rank in a group nothing is gathered or freed: the flat buffer is persistent.
"""
from __future__ import annotations

import torch
import torch.distributed as dist
import torch.nn as nn

ALIGN = 128

_DT = {"fp32": torch.float32, "bf16": torch.bfloat16}


def _round_up(x: int, m: int) -> int:
    return (x + m - 1) // m * m


class FlatGroup:
    def __init__(self, name: str, named_params: list[tuple[str, nn.Parameter]], group, group_size: int,
                 group_rank: int, compute_dtype: torch.dtype, master_weights: bool, device: torch.device,
                 comm=None):
        self.name = name
        self.group, self.world, self.rank = group, group_size, group_rank
        self.compute_dtype = compute_dtype
        self.device = device
        self.comm = comm                          # optional fused peer-memory collectives
        # matrices first, 1-D parameters (norm gains) at the tail: weight decay applies to [0, decay_numel) only,
        # one boundary the fused AdamW kernels take as an argument
        named_params = [np for np in named_params if np[1].dim() > 1] + [np for np in named_params if np[1].dim() <= 1]
        self.names = [n for n, _ in named_params]
        self.params = [p for _, p in named_params]
        self.shapes = [tuple(p.shape) for p in self.params]
        self.offsets = []
        off = 0
        for p in self.params:
            self.offsets.append(off)
            off += _round_up(p.numel(), ALIGN)
        self.decay_numel = next((o for p, o in zip(self.params, self.offsets) if p.dim() <= 1), off)
        self.total = _round_up(max(off, ALIGN), ALIGN * self.world)
        self.shard_numel = self.total // self.world
        # elements of the flat buffer that belong to no parameter (alignment between parameters, tail padding)
        self.gaps = [(o + p.numel(), nxt) for p, o, nxt in zip(self.params, self.offsets, self.offsets[1:] + [self.total])
                     if o + p.numel() < nxt]
        self.sharded = self.world > 1
        # a group of frozen parameters (LoRA fine-tuning: everything but the adapters) keeps only its compute-dtype
        # shard: no master copy, no gradient buffers, no optimizer state
        self.frozen = bool(named_params) and not any(p.requires_grad for _, p in named_params)
        self.keep_master = master_weights and compute_dtype != torch.float32 and not self.frozen

        # full buffer (compute dtype); parameters become views into it.  Parameters created on the
        # meta device carry no values yet: the caller initialises the views, then calls finalize().
        self.full = torch.zeros(self.total, dtype=compute_dtype, device=device)
        hi_src = None
        for p, o in zip(self.params, self.offsets):
            if not p.is_meta:
                self.full[o:o + p.numel()].copy_(p.detach().reshape(-1))
                if self.keep_master and p.dtype == torch.float32:
                    if hi_src is None:
                        hi_src = torch.zeros(self.total, dtype=torch.float32, device=device)
                    hi_src[o:o + p.numel()].copy_(p.detach().reshape(-1))
        self._hi_src = hi_src
        for i, (p, o, shp) in enumerate(zip(self.params, self.offsets, self.shapes)):
            if p.is_meta:
                newp = nn.Parameter(self.full[o:o + p.numel()].view(shp), requires_grad=p.requires_grad)
                for attr in ("is_expert", "tp_dim", "tp_global_shape", "tp_segments", "tp_partial_grad"):
                    if hasattr(p, attr):
                        setattr(newp, attr, getattr(p, attr))
                self.params[i] = newp
            else:
                p.data = self.full[o:o + p.numel()].view(shp)
        self.shard: torch.Tensor | None = None
        self.grad_full: torch.Tensor | None = None
        self.grad_shard: torch.Tensor | None = None     # fp32 accumulation over micro-batches
        self.replica_group = None                       # ranks holding the same shard (plain DDP when unsharded,
                                                        # the cross-replica axis of hybrid sharding when sharded)
        self.gathered = True
        self.tp_replicas = 1                            # tensor-parallel ranks holding identical copies of this group
        self.prefetch_comm = None                       # second peer-comm instance used only by prefetch()
        self._pf_event = None                           # set while a prefetched gather is in flight
        # all-gather fused into the first GEMM that multiplies one of the group's matrices (forward passes of decoder
        # layers; set by the engine): gather() stages the shard and pulls only the 1-D tail, the GEMM pulls the rest
        self.fuse_gather = False
        self.pending_gather = None                      # ticket of a gather whose matrices have not been pulled yet
        self._gather_pieces = None
        self._gather_calls = 0
        for p in self.params:
            p._flat_group = self

    def finalize(self) -> None:
        """Take the owned shard (the optimizer's source of truth) from the initialised full buffer."""
        lo = self.rank * self.shard_numel
        if self.keep_master:
            src = self._hi_src if self._hi_src is not None else self.full
            self.shard = src[lo:lo + self.shard_numel].float().clone()
        elif self.sharded:
            self.shard = self.full[lo:lo + self.shard_numel].clone()
        else:
            self.shard = self.full                # single rank, no master: optimizer updates in place
        self._hi_src = None
        # sharded groups with fp32 masters keep a compute-dtype copy of the shard (written by the optimizer
        # kernel in the same pass as the master) so a gather never has to cast
        self.shard_lp = self.shard.to(self.compute_dtype) if (self.sharded and self.keep_master) else None
        if self.sharded:
            self.release()

    # ---- parameters -------------------------------------------------------
    def shard_decay_end(self) -> int:
        """Elements at the head of this rank's shard that get weight decay (the group's 1-D parameters sit at the tail
        of the flat buffer; every parameter starts on a 128-element boundary, so this is a multiple of 128)."""
        lo = self.rank * self.shard_numel if self.sharded else 0
        return min(max(self.decay_numel - lo, 0), self.shard_numel if self.sharded else self.total)

    def shard_in_compute_dtype(self) -> torch.Tensor:
        if getattr(self, "shard_lp", None) is not None:
            return self.shard_lp
        return self.shard if self.shard.dtype == self.compute_dtype else self.shard.to(self.compute_dtype)

    def sync_low_precision(self) -> None:
        """Refresh the compute-dtype copies after the master shard changed outside the fused kernel."""
        if getattr(self, "shard_lp", None) is not None:
            self.shard_lp.copy_(self.shard)
        self.refresh_full_from_shard()

    def can_fuse_rs_adamw(self) -> bool:
        """Reduce-scatter + cast + AdamW in one peer-memory kernel: needs the peer comm, bf16 gradients and an
        fp32 master shard."""
        return (self.sharded and self.comm is not None and self.keep_master and self.grad_full is not None
                and self.grad_full.dtype == torch.bfloat16 and self.grad_shard is None
                and self.replica_group is None)      # hybrid sharding sums across replicas between the two halves

    def take_grad_full(self) -> torch.Tensor:
        """Hand the flat gradient buffer to a fused reduce-scatter+update (nothing is left to reduce)."""
        self._collect_fused_grads()
        g, self.grad_full = self.grad_full, None
        for p in self.params:
            p.grad = None
        return g

    def prefetch(self, stream) -> None:
        """Start this group's all-gather on ``stream`` so that it runs beside the current unit's compute; the next
        ``gather()`` only waits for it.  Uses its own peer workspace: the flag protocol of a comm instance assumes
        one stream issues its calls in order."""
        if not self.sharded or self.gathered or self._pf_event is not None or self.prefetch_comm is None:
            return
        st = self.full.untyped_storage()
        if st.size() == 0:
            st.resize_(self.total * self.full.element_size())      # allocated on the compute stream's pool
        main = torch.cuda.current_stream(self.device)
        stream.wait_stream(main)                                    # the shard (optimizer output) is final
        src = self.shard_in_compute_dtype()
        with torch.cuda.stream(stream):
            self.prefetch_comm.all_gather(self.full.data, src, self)
            ev = torch.cuda.Event()
            ev.record(stream)
        self._pf_event = ev

    def param_offset(self, p) -> int:
        for q, o in zip(self.params, self.offsets):
            if q is p:
                return o
        raise KeyError("parameter is not part of this flat group")

    def take_pending_gather(self, w):
        """Called by the dense linear op before it multiplies ``w``: the ticket of a gather that still has to pull the
        group's matrices, plus what the fused kernel needs, if ``w`` can be the GEMM that does it; otherwise the
        gather is completed the plain way first and None is returned."""
        ticket = self.pending_gather
        if ticket is None:
            return None
        self.pending_gather = None
        try:
            w_off = self.param_offset(w)
        except KeyError:
            w_off = -1
        if w_off < 0 or w.dim() != 2 or (w_off + w.numel()) * 2 > ticket["head_bytes"]:
            self.comm.finish_gather(ticket, self.full.data)
            return None
        if self._gather_pieces is None:
            n = (self.total * 2 + self.comm.PIECE_BYTES - 1) // self.comm.PIECE_BYTES
            self._gather_pieces = torch.zeros(n, dtype=torch.int32, device=self.device)
        self._gather_calls += 1
        return {"ticket": ticket, "w_off": w_off, "pieces": self._gather_pieces, "call": self._gather_calls,
                "flat": self.full.data, "comm": self.comm, "group": self}

    def finish_pending_gather(self) -> None:
        if self.pending_gather is not None:
            ticket, self.pending_gather = self.pending_gather, None
            self.comm.finish_gather(ticket, self.full.data)

    def gather(self, fused: bool = False) -> None:
        if self.gathered:
            return
        if self._pf_event is not None:
            torch.cuda.current_stream(self.device).wait_event(self._pf_event)
            self._pf_event = None
            self.gathered = True
            return
        if self.sharded:
            st = self.full.untyped_storage()
            if st.size() == 0:
                st.resize_(self.total * self.full.element_size())
            src = self.shard_in_compute_dtype()
            # write through an alias with its own version counter: autograd may hold parameter views
            # saved by a forward that ran before this (re-)gather, and the values are the same
            dst = self.full.data
            if fused and self.fuse_gather and self.comm is not None and hasattr(self.comm, "begin_gather") \
                    and self.compute_dtype == torch.bfloat16:
                self.pending_gather = self.comm.begin_gather(dst, src, self.decay_numel * 2)
            elif self.comm is not None:
                self.comm.all_gather(dst, src, self)
            else:
                dist.all_gather_into_tensor(dst, src.contiguous(), group=self.group)
        self.gathered = True

    def release(self) -> None:
        self.finish_pending_gather()          # a staged slot must be read and acknowledged even if nobody multiplied
        if self.sharded and self.gathered:
            self.full.untyped_storage().resize_(0)
            self.gathered = False

    def refresh_full_from_shard(self) -> None:
        """After an optimizer step on an unsharded group with fp32 masters: recast into the compute copy."""
        if not self.sharded and self.shard is not self.full:
            self.full.data.copy_(self.shard)

    # ---- gradients ----------------------------------------------------------
    def _fused_wgrad(self) -> bool:
        """On the kernel path the weight-gradient GEMMs (expert and dense) write straight into the flat gradient
        buffer through ``p.main_grad``; gradients that arrive the ordinary way (norm gains, the router, anything that
        took a library route) are copied in by ``_collect_fused_grads``."""
        from .. import ops
        return self.compute_dtype == torch.bfloat16 and self.device.type == "cuda" and ops.kernel_mode() == "auto"

    def prepare_grads(self) -> None:
        if self.frozen:
            return
        fused = self._fused_wgrad()
        if self.grad_full is None:
            alloc = torch.empty if fused else torch.zeros
            self.grad_full = alloc(self.total, dtype=self.compute_dtype, device=self.device)
            if fused:
                for lo, hi in self.gaps:             # nobody writes the padding; the reduction and the norm read it
                    self.grad_full[lo:hi].zero_()
            for p in self.params:
                p.main_grad_written = False
        for p, o, shp in zip(self.params, self.offsets, self.shapes):
            view = self.grad_full[o:o + p.numel()].view(shp)
            if fused:
                p.main_grad = view
                p.grad = None
            else:
                p.grad = view

    def _collect_fused_grads(self) -> None:
        for p in self.params:
            mg = getattr(p, "main_grad", None)
            if mg is None:
                continue
            if p.grad is not None:                    # an op took the oracle path and returned a gradient
                if p.main_grad_written:
                    mg.add_(p.grad)
                else:
                    mg.copy_(p.grad)
            elif not p.main_grad_written:
                mg.zero_()
            p.main_grad = None

    def reduce_grads(self, keep_full: bool = False) -> None:
        """Sum ``grad_full`` over the group into this rank's ``grad_shard`` (fp32 once it accumulates)."""
        if self.grad_full is None:
            return
        self._collect_fused_grads()
        if self.sharded:
            if self.comm is not None:
                piece = self.comm.reduce_scatter(self.grad_full, self)
            else:
                piece = torch.empty(self.shard_numel, dtype=self.grad_full.dtype, device=self.device)
                dist.reduce_scatter_tensor(piece, self.grad_full, op=dist.ReduceOp.SUM, group=self.group)
        else:
            piece = self.grad_full
        if self.replica_group is not None:
            dist.all_reduce(piece, op=dist.ReduceOp.SUM, group=self.replica_group)
        if self.grad_shard is None:
            self.grad_shard = piece                    # consumed as is when there is one micro-batch
        else:
            if self.grad_shard.dtype != torch.float32:
                self.grad_shard = self.grad_shard.float()
            self.grad_shard.add_(piece)
        for p in self.params:
            p.grad = None
        self.grad_full = None

    def zero_grad(self) -> None:
        self.grad_shard = None
        self.grad_full = None
        for p in self.params:
            p.grad = None

    # ---- checkpoint views -----------------------------------------------------
    def param_slices(self):
        """Yield ``(name, shape, flat_offset, numel)`` for checkpoint resharding."""
        for n, o, shp, p in zip(self.names, self.offsets, self.shapes, self.params):
            yield n, shp, o, p.numel()


class Unit:
    """One FSDP unit: a module plus its flat groups."""

    def __init__(self, name: str, module: nn.Module, groups: list[FlatGroup]):
        self.name, self.module, self.groups = name, module, groups

    def gather(self, fused: bool = False):
        for g in self.groups:
            g.gather(fused)

    def prefetch(self, stream):
        for g in self.groups:
            g.prefetch(stream)

    def release(self):
        for g in self.groups:
            g.release()

    def prepare_grads(self):
        for g in self.groups:
            g.prepare_grads()

    def reduce_grads(self):
        for g in self.groups:
            g.reduce_grads()


def build_unit(name: str, module: nn.Module, mesh, compute_dtype: torch.dtype, master_weights: bool,
               device: torch.device, fsdp: bool = True, dense_comm=None, expert_comm=None) -> Unit:
    dense, expert, tp_sharded, frozen = [], [], [], []
    for n, p in module.named_parameters():
        if getattr(p, "is_expert", False):
            expert.append((f"{name}.{n}", p))
        elif hasattr(p, "tp_segments"):
            tp_sharded.append((f"{name}.{n}", p))
        elif not p.requires_grad:
            frozen.append((f"{name}.{n}", p))
        else:
            dense.append((f"{name}.{n}", p))
    groups = []
    if frozen:
        # frozen dense parameters (the base model under LoRA) are sharded like the trainable ones but own no
        # gradient or optimizer state; keeping them apart lets the trainable group stay a few megabytes
        if fsdp and mesh.data_size > 1 and mesh.replicas == 1:
            groups.append(FlatGroup(f"{name}/frozen", frozen, mesh.data_group, mesh.data_size, mesh.data_rank,
                                    compute_dtype, False, device, dense_comm))
        else:
            g = FlatGroup(f"{name}/frozen", frozen, None, 1, 0, compute_dtype, False, device)
            g.replica_group = mesh.data_group if mesh.data_size > 1 else None
            groups.append(g)
    if tp_sharded:
        # this rank's slice of the head- / column-split matrices: sharded over the data ranks like the dense group,
        # but distinct on every tensor-parallel rank (the dense group is replicated over them)
        if fsdp and mesh.data_size > 1:
            groups.append(FlatGroup(f"{name}/tp", tp_sharded, mesh.data_group, mesh.data_size, mesh.data_rank,
                                    compute_dtype, master_weights, device, dense_comm))
        else:
            g = FlatGroup(f"{name}/tp", tp_sharded, None, 1, 0, compute_dtype, master_weights, device)
            g.replica_group = mesh.data_group if mesh.data_size > 1 else None
            groups.append(g)
    if dense:
        if fsdp and mesh.replicas > 1 and mesh.data_shard_size > 1:
            # hybrid sharding (``num_distributed_optimizer_instances`` of ``notes/2026-04/2026-04-20_gptoss_14_*``):
            # shard inside the block, replicate across blocks
            g = FlatGroup(f"{name}/dense", dense, mesh.data_shard_group, mesh.data_shard_size, mesh.data_shard_rank,
                          compute_dtype, master_weights, device, dense_comm)
            g.replica_group = mesh.data_repl_group
            groups.append(g)
        elif fsdp and mesh.data_size > 1 and mesh.replicas == 1:
            groups.append(FlatGroup(f"{name}/dense", dense, mesh.data_group, mesh.data_size, mesh.data_rank,
                                    compute_dtype, master_weights, device, dense_comm))
        else:
            g = FlatGroup(f"{name}/dense", dense, None, 1, 0, compute_dtype, master_weights, device)
            g.replica_group = mesh.data_group if mesh.data_size > 1 else None
            groups.append(g)
    if expert:
        if fsdp and mesh.edp_replicas > 1 and mesh.edp_shard_size > 1:
            g = FlatGroup(f"{name}/expert", expert, mesh.edp_shard_group, mesh.edp_shard_size, mesh.edp_shard_rank,
                          compute_dtype, master_weights, device, expert_comm)
            g.replica_group = mesh.edp_repl_group
            groups.append(g)
        elif fsdp and mesh.edp > 1 and mesh.edp_replicas == 1:
            edp_rank = mesh.edp_rank * mesh.cp + mesh.cp_rank
            groups.append(FlatGroup(f"{name}/expert", expert, mesh.edp_group, mesh.edp, edp_rank,
                                    compute_dtype, master_weights, device, expert_comm))
        else:
            g = FlatGroup(f"{name}/expert", expert, None, 1, 0, compute_dtype, master_weights, device)
            g.replica_group = mesh.edp_group if mesh.edp > 1 else None
            groups.append(g)
    if mesh.tp > 1:
        for g in groups:
            if g.name.endswith("/dense") or g.name.endswith("/frozen"):
                g.tp_replicas = mesh.tp
    # parameters that were on the meta device have been re-created as views: re-register them
    for g in groups:
        for full_name, p in zip(g.names, g.params):
            rel = full_name[len(name) + 1:]
            owner = module
            *path, leaf = rel.split(".")
            for part in path:
                owner = getattr(owner, part)
            if owner._parameters.get(leaf) is not p:
                owner._parameters[leaf] = p
    return Unit(name, module, groups)
