"""Layer-granular execution engine: explicit gather → compute → reduce per FSDP unit.

Instead of module hooks or a tracing compiler, every unit (embedding, decoder layer, head) runs
inside one autograd node that the engine controls:

* forward: gather the unit's parameters, run it (without building a graph when the unit is
  recomputed in backward), release the parameters;
* backward: gather again, rebuild the unit's graph from the saved input if needed, run the unit's
  backward into flat gradient buffers, reduce-scatter them, optionally apply AdamW to the shard
  right there (``optimizer_in_backward``), release.

This gives one place to overlap the next unit's parameter traffic with the current unit's math and
keeps at most one unit's full parameters (plus one in flight) resident — the memory plan that lets
the 30B-parameter shape fit 180 GB of HBM3e on few GPUs.
"""
from __future__ import annotations

import torch
import torch.nn as nn

from ..config import Config
from ..models.simple_moe import SimpleMoE, seeded_normal_
from ..moe.dispatch import AllToAllDispatcher
from .fsdp import Unit, build_unit
from .mesh import Mesh

_DT = {"fp32": torch.float32, "bf16": torch.bfloat16}


def init_unit_weights(module: nn.Module, global_prefix: str, std: float, seed: int, ep_rank: int) -> None:
    """N(0, std) for matrices, ones for norm gains; expert tensors one *global* expert at a time so
    every parallel layout produces the same logical weights."""
    with torch.no_grad():
        for name, p in module.named_parameters():
            gname = f"{global_prefix}.{name}"
            if p.dim() == 1:
                p.fill_(1.0)
            elif name.endswith("lora_b"):
                p.zero_()                      # adapters start as a zero update
            elif hasattr(p, "tp_segments") and getattr(p, "is_expert", False):
                # expert tensor parallelism: draw every local expert's global matrices, keep this rank's columns
                from .tp import take_segments
                e_local = p.shape[0]
                for j in range(e_local):
                    full = torch.empty(p.tp_global_shape[1:], dtype=p.dtype if p.is_cuda else torch.float32,
                                       device=p.device)
                    seeded_normal_(full, std, seed, f"{gname}.{ep_rank * e_local + j}")
                    p[j].copy_(take_segments(full, p.tp_dim - 1, p.tp_segments))
            elif hasattr(p, "tp_segments"):
                # draw the global matrix, keep this tensor-parallel rank's rows / columns
                from .tp import take_segments
                full = torch.empty(p.tp_global_shape, dtype=p.dtype if p.is_cuda else torch.float32, device=p.device)
                seeded_normal_(full, std, seed, gname)
                p.copy_(take_segments(full, p.tp_dim, p.tp_segments))
            elif getattr(p, "is_expert", False):
                e_local = p.shape[0]
                for j in range(e_local):
                    seeded_normal_(p[j], std, seed, f"{gname}.{ep_rank * e_local + j}")
            else:
                seeded_normal_(p, std, seed, gname)


class _UnitFn(torch.autograd.Function):
    """Runs ``unit.module(x, *extra)`` under engine control.  ``anchor`` is a dummy tensor that
    requires grad so the node always takes part in backward (the embedding's input does not)."""

    @staticmethod
    def forward(ctx, anchor, engine, unit, x, *extra):
        ctx.engine, ctx.unit, ctx.extra = engine, unit, extra
        recompute = engine.recompute or engine.inference      # forward-only passes keep no graph
        ctx.recompute = recompute
        unit.gather(fused=True)          # dense matrices may arrive inside the first GEMM that multiplies one of them
        engine.after_gather(unit, forward=True)
        engine.prefetch_neighbour(unit, +1)
        x_needs_grad = x.is_floating_point()
        if recompute:
            with torch.no_grad():
                out = unit.module(x, *extra)
            aux = engine.pop_aux(unit)
            ctx.x = x
            outs = (out,) if aux is None else (out, aux)
        else:
            with torch.enable_grad():
                xin = x.detach().requires_grad_(True) if x_needs_grad else x
                out_inner = unit.module(xin, *extra)
                aux = engine.pop_aux(unit)
            ctx.xin = xin
            ctx.inner = (out_inner,) if aux is None else (out_inner, aux)
            outs = tuple(t.detach() for t in ctx.inner)
        ctx.n_out = len(outs)
        ctx.x_needs_grad = x_needs_grad
        unit.release()
        return outs if len(outs) > 1 else outs[0]

    @staticmethod
    def backward(ctx, *grads):
        engine, unit = ctx.engine, ctx.unit
        unit.gather()
        engine.after_gather(unit, forward=False)
        engine.prefetch_neighbour(unit, -1)
        if ctx.recompute:
            from ..models import simple_moe
            simple_moe.RECOMPUTE_PHASE[0] = True
            try:
                with torch.enable_grad():
                    xin = ctx.x.detach().requires_grad_(True) if ctx.x_needs_grad else ctx.x
                    out_inner = unit.module(xin, *ctx.extra)
                    aux = engine.pop_aux(unit)
            finally:
                simple_moe.RECOMPUTE_PHASE[0] = False
            inner = (out_inner,) if aux is None else (out_inner, aux)
        else:
            xin, inner = ctx.xin, ctx.inner
        unit.prepare_grads()
        pairs = [(t, g) for t, g in zip(inner, grads) if g is not None and t.requires_grad]
        if pairs:                              # a unit without trainable parameters or inputs (a frozen embedding)
            torch.autograd.backward([t for t, _ in pairs], [g for _, g in pairs])
        gx = xin.grad if ctx.x_needs_grad else None
        engine.after_unit_backward(unit)
        unit.release()
        ctx.x = ctx.xin = ctx.inner = None
        return (None, None, None, gx) + (None,) * len(ctx.extra)


class Engine:
    def __init__(self, cfg: Config, mesh: Mesh, device: torch.device):
        self.cfg, self.mesh, self.device = cfg, mesh, device
        self.inference = False               # set around forward-only passes (evaluation)
        m = cfg.model
        self.compute_dtype = _DT[cfg.precision.params_dtype]
        gran = cfg.precision.recompute_granularity
        # selective = keep attention activations, re-run the feed-forward block in backward (the block's
        # load-balancing loss travels through the recompute node as a second output); full = re-run the whole layer
        self.selective = gran == "selective"
        self.recompute = gran == "full"
        pp = mesh.pp
        # Virtual pipeline stages: the decoder is cut into pp * vpp equal blocks, block v lives on rank v % pp as
        # that rank's chunk v // pp, so a micro-batch visits every rank vpp times (interleaved schedule).
        self.vpp = max(cfg.parallel.virtual_pipeline_model_parallel_size, 1) if pp > 1 else 1
        per_block = m.num_layers // (pp * self.vpp)
        self.chunk_layer_ids = [list(range((c * pp + mesh.pp_rank) * per_block, (c * pp + mesh.pp_rank + 1) * per_block))
                                for c in range(self.vpp)]
        self.layer_start = self.chunk_layer_ids[0][0]
        self.layer_end = self.chunk_layer_ids[-1][-1] + 1
        self.tp = None
        if mesh.tp > 1:
            from .tp import TensorParallel
            self.tp = TensorParallel(mesh.tp_group, mesh.tp_rank, mesh.tp, cfg.parallel.sequence_parallel)
            self.tp.fused_gemm_rs = cfg.parallel.tp_fused_gemm_reduce_scatter and device.type == "cuda"
        with torch.device("meta"):
            self.model = SimpleMoE(
                m, ep_rank=mesh.ep_rank, ep_size=mesh.ep, fp8=(cfg.precision.fp8_recipe if cfg.precision.fp8 else False),
                layer_ids=[i for ids in self.chunk_layer_ids for i in ids],
                first_stage=mesh.is_first_stage(), last_stage=mesh.is_last_stage(),
                cp_group=mesh.cp_group if mesh.cp > 1 else None, cp_rank=mesh.cp_rank, cp_size=mesh.cp,
                bf16_first_layers=cfg.precision.num_layers_at_start_in_bf16,
                bf16_last_layers=cfg.precision.num_layers_at_end_in_bf16, tp=self.tp, expert_tp=mesh.etp > 1)
        self.units: list[Unit] = []
        self.anchor = torch.zeros(1, device=device, requires_grad=True)
        self._aux_out: list[torch.Tensor] = []
        self.optimizer = None            # set by the trainer when optimizer_in_backward is on
        fsdp = cfg.parallel.fsdp
        mw = cfg.precision.master_weights
        seed, std = cfg.train.seed, m.init_method_std
        dense_comm, expert_comm = self._make_comms()

        def add(name, module):
            u = build_unit(name, module, mesh, self.compute_dtype, mw, device, fsdp, dense_comm, expert_comm)
            for bn, b in list(module.named_buffers()):
                if b.is_meta:
                    owner = module
                    *path, leaf = bn.split(".")
                    for part in path:
                        owner = getattr(owner, part)
                    if leaf == "expert_map":        # identity placement: logical expert l lives in slot l
                        owner._buffers[leaf] = torch.arange(b.shape[0], dtype=b.dtype, device=device)
                    else:
                        owner._buffers[leaf] = torch.zeros(b.shape, dtype=b.dtype, device=device)
            init_unit_weights(module, name, std, seed, mesh.ep_rank)
            for g in u.groups:
                g.finalize()
            self.units.append(u)
            return u

        self.embed_unit = add("embed", self.model.embed) if self.model.embed is not None else None
        self.layer_units = [add(f"layers.{l.layer_idx}", l) for l in self.model.layers]
        for l in self.model.layers:
            l.recompute_ffn = self.selective
            if l.is_moe:
                l.ffn.keep_dispatched = self.selective and cfg.model.moe_keep_dispatched_factor != 0
        self.head_unit = add("head", self.model.head) if self.model.head is not None else None
        if cfg.parallel.fsdp_gather_in_gemm and dense_comm is not None and not cfg.parallel.fsdp_prefetch:
            for u in self.layer_units:
                for g in u.groups:
                    if g.comm is dense_comm and g.name.endswith("/dense") and g.sharded:
                        g.fuse_gather = True
        self._make_dispatchers()
        self._unit_index = {u.name: i for i, u in enumerate(self.units)}
        self._prefetch_stream = None
        if cfg.parallel.fsdp_prefetch and dense_comm is not None and self.vpp == 1:
            from ..comm.fsdp_comm import FsdpPeerComm
            pf = FsdpPeerComm(mesh.data_group, mesh.data_size, mesh.data_rank, device)
            for u in self.units:
                for g in u.groups:
                    if g.comm is dense_comm:
                        g.prefetch_comm = pf
            self._prefetch_stream = torch.cuda.Stream(device=device)

    # ---- construction helpers ---------------------------------------------------
    def _make_comms(self):
        """Peer-memory collectives for FSDP when running on GPUs with the fused path enabled."""
        if (self.device.type == "cuda" and self.cfg.parallel.fsdp_fused_collectives
                and self.cfg.parallel.fsdp and self.mesh.world > 1 and self.compute_dtype == torch.bfloat16):
            from ..comm.fsdp_comm import make_fsdp_comms
            return make_fsdp_comms(self.mesh, self.device, self.cfg.parallel.fsdp_nvls_reduce)
        return None, None

    def _make_dispatchers(self):
        m = self.cfg.model
        fused = (m.moe_token_dispatcher_type == "fused" and self.device.type == "cuda")
        shared = None
        for layer in self.model.layers:
            if not layer.is_moe:
                continue
            if fused:
                if shared is None:
                    from ..moe.fused_dispatch import FusedDispatcher
                    # tokens one MoE block sees: 1 / tp of the group's tokens, or all of them under expert tensor parallelism
                    tokens = self.cfg.train.micro_batch_size * m.seq_length // (
                        self.mesh.cp * (self.mesh.tp // self.mesh.etp))
                    shared = FusedDispatcher(self.mesh, m.num_experts, m.moe_router_topk, m.hidden_size,
                                             max_tokens=tokens, pad_to=m.moe_pad_expert_rows_to,
                                             device=self.device, dtype=self.compute_dtype,
                                             clone_outputs=not (self.recompute or self.selective),
                                             capacity_factor=m.moe_capacity_factor,
                                             push=m.moe_combine_push and self.mesh.ep > 1,   # nothing to overlap on one rank
                                             keep_factor=m.moe_keep_dispatched_factor if self.selective else 0.0)
                    # (one rank: nothing arrives from anywhere, the token-ordered scatter reads every row once)
                    shared.expert_ordered = m.moe_expert_ordered_dispatch and self.mesh.ep > 1
                    shared.overlap = m.moe_scatter_overlap and self.mesh.ep > 1
                    if shared.expert_ordered:
                        from ..moe.fused_dispatch import set_scatter_bulk
                        set_scatter_bulk(m.moe_scatter_bulk_store)
                layer.ffn.dispatcher = shared
            else:
                if shared is None:
                    shared = AllToAllDispatcher(self.mesh.ep_group if self.mesh.ep > 1 else None,
                                                m.num_experts, m.moe_pad_expert_rows_to)
                layer.ffn.dispatcher = shared
        self.dispatcher = shared

    # ---- hooks called from the autograd node -----------------------------------------
    def after_gather(self, unit: Unit, forward: bool) -> None:
        pass

    def prefetch_neighbour(self, unit: Unit, direction: int) -> None:
        """``fsdp_prefetch``: start gathering the unit that runs next (forward: the following one, backward: the
        preceding one) on a side stream while this unit computes."""
        if self._prefetch_stream is None:
            return
        i = self._unit_index.get(unit.name, -1) + direction
        if 0 <= i < len(self.units):
            self.units[i].prefetch(self._prefetch_stream)

    def pop_aux(self, unit: Unit):
        ffn = getattr(unit.module, "ffn", None)
        aux = getattr(ffn, "aux", None)
        if aux is not None:
            ffn.aux = None
        return aux

    def after_unit_backward(self, unit: Unit) -> None:
        in_bwd = self.optimizer is not None and self.cfg.train.optimizer_in_backward
        if self.tp is not None:
            import torch.distributed as dist
            for p in unit.module.parameters():
                # replicated parameters inside a MoE block saw only this rank's slice of the tokens
                if not getattr(p, "tp_partial_grad", False):
                    continue
                if getattr(p, "main_grad", None) is not None and getattr(p, "main_grad_written", False):
                    dist.all_reduce(p.main_grad, group=self.tp.group)      # written in place by a wgrad kernel
                if p.grad is not None:
                    dist.all_reduce(p.grad, group=self.tp.group)
        for g in unit.groups:
            if not (in_bwd and self.optimizer.fusable(g)):
                g.reduce_grads()              # fusable groups are reduced inside the optimizer kernel
        if in_bwd:
            self.optimizer.step_unit(unit)

    # ---- running one micro-batch through this pipeline stage --------------------------------
    def run_unit(self, unit: Unit, x: torch.Tensor, *extra):
        return _UnitFn.apply(self.anchor, self, unit, x, *extra)

    def stage_forward(self, inp: torch.Tensor, targets: torch.Tensor | None, chunk: int | None = None):
        """First stage: ``inp`` are token ids ``[B, S]``; later stages: hidden ``[B, S, H]``.
        Returns ``(output, aux_losses)`` where output is the scalar loss on the last stage.  ``chunk`` selects one
        of this rank's virtual pipeline stages (None: all local layers, the non-interleaved case)."""
        aux_all = []
        x = inp
        first_chunk = chunk is None or chunk == 0
        last_chunk = chunk is None or chunk == self.vpp - 1
        sp = self.tp.size if self.tp is not None and self.tp.sequence_parallel else 1
        if self.embed_unit is not None and first_chunk:
            if sp > 1:
                x = self.tp.local_seq(x)          # every rank of the group got the same token ids
            x = self.run_unit(self.embed_unit, x, self.compute_dtype)
        cos, sin = self.model.rope_tables(x.shape[1] * sp, x.device)     # attention sees whole sequences
        if chunk is None:
            units = self.layer_units
        else:
            per = len(self.layer_units) // self.vpp
            units = self.layer_units[chunk * per:(chunk + 1) * per]
        for u in units:
            out = self.run_unit(u, x, cos, sin)
            if isinstance(out, tuple):
                x, aux = out
                aux_all.append(aux)
            else:
                x = out
        if self.head_unit is not None and last_chunk:
            if sp > 1:
                x = self.tp.mean_loss(self.run_unit(self.head_unit, x, self.tp.local_seq(targets)))
            else:
                x = self.run_unit(self.head_unit, x, targets)
        return x, aux_all

    def seq_shards(self) -> int:
        """Into how many parts sequence parallelism cuts the sequences this rank's stage receives and sends."""
        return self.tp.size if self.tp is not None and self.tp.sequence_parallel else 1

    def all_groups(self):
        for u in self.units:
            yield from u.groups

    def moe_ffns(self):
        return self.model.moe_layers()

    def num_local_params(self) -> int:
        return sum(g.shard_numel for g in self.all_groups())
