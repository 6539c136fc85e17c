"""SimpleMoE decoder family: GQA or MLA attention, dense or MoE SwiGLU feed-forward, RMSNorm, RoPE.

One class covers the tiny plumbing model, the Qwen3-30B-A3B shape, the DeepSeek-V3 shaped proxy
(MLA, shared expert, sigmoid router with bias balancing, first layer dense) and the GPT-OSS-20B
shape (sliding window on alternate layers) the reference profiles
(``notes/2026-04/2026-04-21_gptoss_13_attn_bwd_recompile_postmortem.md:19-26``).

Per layer data flow (the fused residual+norm form of
``notes/2026-04/2026-04-24_gptoss_17_fused_residual_rmsnorm_impl.md:43-83``)::

    a      = attention(rmsnorm(x))
    y, h   = rmsnorm_residual(a, x)          # h = x + a ; y = norm(h)
    out    = h + ffn(y)

MoE feed-forward (gate probability applied inside SwiGLU so no expert output has to be kept for
the router gradient, ``moe/MegatronCore_MoE_reading_notes.md:201-218``)::

    w, idx = router_topk(y @ Wr.T)           # fp32
    xe, pe = dispatch(y, w)                  # expert-major rows on the owning rank
    ye     = grouped_linear(swiglu_probs(grouped_linear(xe, W1), pe), W2)
    ffn    = combine(ye) (+ shared expert)
"""
from __future__ import annotations

import hashlib
import math

import torch
import torch.nn as nn
import torch.nn.functional as F

from .. import ops
from ..config import ModelConfig
from ..ops import reference as ref


def _seed_for(base_seed: int, name: str) -> int:
    h = hashlib.sha256(f"{base_seed}:{name}".encode()).digest()
    return int.from_bytes(h[:7], "little")


def seeded_normal_(t: torch.Tensor, std: float, base_seed: int, name: str) -> None:
    """Fill ``t`` with N(0, std) from a generator keyed by the parameter's *global* name, so the
    same logical weight gets the same values under every parallel layout."""
    g = torch.Generator(device=t.device)
    g.manual_seed(_seed_for(base_seed, name))
    if t.dtype in (torch.float32, torch.float64) or t.is_cuda:
        t.normal_(0.0, std, generator=g)
    else:
        t.copy_(torch.empty(t.shape, dtype=torch.float32, device=t.device).normal_(0.0, std, generator=g))


# True while a layer's forward is being re-run inside backward (activation recompute): statistics that are
# collected once per micro-batch (expert load) skip the replay.
RECOMPUTE_PHASE = [False]
# State a recomputed block keeps between its two runs: a dict owned by the autograd node, visible to the modules
# inside the block while either run is in progress (None outside).
KEPT = [None]

_BALANCE_TABLES: dict = {}


def _balance_table(like: torch.Tensor) -> torch.Tensor:
    key = (tuple(like.shape), str(like.device))
    if key not in _BALANCE_TABLES:
        g = torch.Generator(device=like.device)
        g.manual_seed(20240607)
        _BALANCE_TABLES[key] = torch.rand(like.shape, generator=g, device=like.device, dtype=torch.float32)
    return _BALANCE_TABLES[key]


class LoRA(nn.Module):
    """Rank-r update of a frozen projection: ``y += (alpha / r) * (x A^T) B^T`` with ``A ~ N(0, std)`` and ``B = 0``, so
    the adapted model starts out equal to the base model (the Llama-2-70B LoRA workload of
    ``notes/mlperf-llama/2026-04-29_llama2_70b_lora_baseline_trace_breakdown.md``)."""

    def __init__(self, out_features: int, in_features: int, rank: int, alpha: float):
        super().__init__()
        self.lora_a = nn.Parameter(torch.empty(rank, in_features))
        self.lora_b = nn.Parameter(torch.empty(out_features, rank))
        self.scale = alpha / rank

    def forward(self, x):
        return F.linear(F.linear(x, self.lora_a.to(x.dtype)), self.lora_b.to(x.dtype)) * self.scale


class RMSNorm(nn.Module):
    def __init__(self, dim: int, eps: float):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(dim))
        self.eps = eps

    def forward(self, x):
        return ops.rmsnorm(x, self.weight, self.eps)


class GQAttention(nn.Module):
    def __init__(self, cfg: ModelConfig, layer_idx: int, cp_group=None, tp=None):
        super().__init__()
        nq, nkv, d = cfg.num_attention_heads, cfg.num_query_groups, cfg.kv_channels
        h = cfg.hidden_size
        self.tp = tp
        t = tp.size if tp is not None else 1
        self.nq, self.nkv, self.d = nq // t, nkv // t, d            # this rank's heads
        self.wqkv = nn.Parameter(torch.empty((self.nq + 2 * self.nkv) * d, h))
        self.wo = nn.Parameter(torch.empty(h, self.nq * d))
        if tp is not None:
            from ..parallel.tp import mark_sharded
            mark_sharded(self.wqkv, 0, ((nq + 2 * nkv) * d, h), tp.segments([nq * d, nkv * d, nkv * d]))
            mark_sharded(self.wo, 1, (h, nq * d), tp.segments([nq * d]))
        self.window = cfg.sliding_window if (cfg.sliding_window and layer_idx % 2 == 0) else 0
        self.cp_group = cp_group
        self.qkv_lora = self.o_lora = None
        if cfg.lora_rank > 0:
            if tp is not None:
                raise ValueError("LoRA adapters are not combined with tensor parallelism")
            self.qkv_lora = LoRA(self.wqkv.shape[0], h, cfg.lora_rank, cfg.lora_alpha)
            self.o_lora = LoRA(h, self.wo.shape[1], cfg.lora_rank, cfg.lora_alpha)

    def forward(self, x, cos, sin):
        if self.tp is not None:
            x = self.tp.enter(x)              # sequence parallel: whole sequences from here to the output projection
        b, s, _ = x.shape
        qkv = ops.linear(x, self.wqkv)
        if self.qkv_lora is not None:
            qkv = qkv + self.qkv_lora(x)
        qkv = ops.rope_packed(qkv, cos, sin, self.nq + self.nkv, self.d)      # q and k heads, one pass
        q, k, v = qkv.split([self.nq * self.d, self.nkv * self.d, self.nkv * self.d], dim=-1)
        q = q.unflatten(-1, (self.nq, self.d))
        k = k.unflatten(-1, (self.nkv, self.d))
        v = v.unflatten(-1, (self.nkv, self.d))
        if self.cp_group is not None:
            from ..parallel.cp import ulysses_attention
            o = ulysses_attention(q, k, v, self.cp_group, window=self.window)
        else:
            o = ops.causal_attention(q, k, v, None, self.window)
        o2 = o.reshape(b, s, self.nq * self.d)
        if self.tp is not None:
            return self.tp.linear_leave(o2, self.wo)
        out = ops.linear(o2, self.wo)
        if self.o_lora is not None:
            out = out + self.o_lora(o2)
        return out


class MLAttention(nn.Module):
    """Multi-head latent attention (DeepSeek-V3): low-rank q and kv projections, a shared rotary
    key of ``qk_rope_head_dim`` and per-head no-position keys of ``qk_nope_head_dim``."""

    def __init__(self, cfg: ModelConfig, layer_idx: int, cp_group=None, tp=None):
        super().__init__()
        h, nh_all = cfg.hidden_size, cfg.num_attention_heads
        self.tp = tp
        nh = nh_all // (tp.size if tp is not None else 1)           # this rank's heads
        self.nh, self.nope, self.rope_d, self.vd = nh, cfg.qk_nope_head_dim, cfg.qk_rope_head_dim, cfg.v_head_dim
        self.q_lora, self.kv_lora = cfg.q_lora_rank, cfg.kv_lora_rank
        qk = self.nope + self.rope_d
        if self.q_lora:
            self.wq_a = nn.Parameter(torch.empty(self.q_lora, h))
            self.q_norm = RMSNorm(self.q_lora, cfg.norm_epsilon)
            self.wq_b = nn.Parameter(torch.empty(nh * qk, self.q_lora))
        else:
            self.wq = nn.Parameter(torch.empty(nh * qk, h))
        self.wkv_a = nn.Parameter(torch.empty(self.kv_lora + self.rope_d, h))
        self.kv_norm = RMSNorm(self.kv_lora, cfg.norm_epsilon)
        self.wkv_b = nn.Parameter(torch.empty(nh * (self.nope + self.vd), self.kv_lora))
        self.wo = nn.Parameter(torch.empty(h, nh * self.vd))
        if tp is not None:
            # heads are split; the low-rank down projections and their norms stay replicated
            from ..parallel.tp import mark_sharded
            qp = self.wq_b if self.q_lora else self.wq
            mark_sharded(qp, 0, (nh_all * qk, qp.shape[1]), tp.segments([nh_all * qk]))
            mark_sharded(self.wkv_b, 0, (nh_all * (self.nope + self.vd), self.kv_lora),
                         tp.segments([nh_all * (self.nope + self.vd)]))
            mark_sharded(self.wo, 1, (h, nh_all * self.vd), tp.segments([nh_all * self.vd]))
        self.scale = 1.0 / math.sqrt(qk)
        self.cp_group = cp_group

    def forward(self, x, cos, sin):
        tp = self.tp
        if tp is not None:
            # the low-rank down projections are repeated on every rank and need whole sequences as well
            x = tp.gather_seq(x)
        b, s, _ = x.shape
        dt = x.dtype
        link = tp.copy_to if tp is not None else (lambda t: t)     # replicated value feeding this rank's heads
        if self.q_lora:
            q = ops.linear(link(self.q_norm(ops.linear(x, self.wq_a))), self.wq_b)
        else:
            q = ops.linear(link(x), self.wq)
        q = q.reshape(b, s, self.nh, self.nope + self.rope_d)
        q_nope, q_rope = q.split([self.nope, self.rope_d], dim=-1)
        kv_a = ops.linear(x, self.wkv_a)
        c_kv, k_rope = kv_a.split([self.kv_lora, self.rope_d], dim=-1)
        k_rope = link(k_rope.contiguous())
        kv = ops.linear(link(self.kv_norm(c_kv)), self.wkv_b).reshape(b, s, self.nh, self.nope + self.vd)
        k_nope, v = kv.split([self.nope, self.vd], dim=-1)
        q_rope = ops.rope(q_rope.contiguous(), cos, sin)
        k_rope = ops.rope(k_rope.reshape(b, s, 1, self.rope_d).contiguous(), cos, sin)
        qf = torch.cat([q_nope, q_rope], dim=-1)
        kf = torch.cat([k_nope, k_rope.expand(b, s, self.nh, self.rope_d)], dim=-1)
        if self.cp_group is not None:
            from ..parallel.cp import ulysses_attention
            o = ulysses_attention(qf, kf, v.contiguous(), self.cp_group, scale=self.scale)
        else:
            o = ops.causal_attention(qf, kf, v.contiguous(), self.scale, 0)
        o2 = o.reshape(b, s, self.nh * self.vd)
        return tp.linear_leave(o2, self.wo) if tp is not None else ops.linear(o2, self.wo)


class DenseFFN(nn.Module):
    def __init__(self, hidden: int, ffn: int, tp=None, lora_rank: int = 0, lora_alpha: float = 32.0):
        super().__init__()
        self.tp = tp
        self.w1_lora = self.w2_lora = None
        if lora_rank > 0 and tp is None:
            self.w1_lora = LoRA(2 * ffn, hidden, lora_rank, lora_alpha)
            self.w2_lora = LoRA(hidden, ffn, lora_rank, lora_alpha)
        f = ffn // (tp.size if tp is not None else 1)          # this rank's columns
        self.w1 = nn.Parameter(torch.empty(2 * f, hidden))     # [gate | up]
        self.w2 = nn.Parameter(torch.empty(hidden, f))
        if tp is not None:
            from ..parallel.tp import mark_sharded
            mark_sharded(self.w1, 0, (2 * ffn, hidden), tp.segments([ffn, ffn]))
            mark_sharded(self.w2, 1, (hidden, ffn), tp.segments([ffn]))

    def forward(self, x):
        if self.tp is not None:
            x = self.tp.enter(x)
        gu = ops.linear(x, self.w1)
        if self.w1_lora is not None:
            gu = gu + self.w1_lora(x)
        act = ops.swiglu(gu)
        if self.tp is not None:
            return self.tp.linear_leave(act, self.w2)
        out = ops.linear(act, self.w2)
        if self.w2_lora is not None:
            out = out + self.w2_lora(act)
        return out


class MoEFFN(nn.Module):
    """Routed experts (this rank owns ``num_experts / ep`` of them) plus an optional shared expert."""

    def __init__(self, cfg: ModelConfig, ep_rank: int, ep_size: int, fp8: bool = False, etp=None):
        super().__init__()
        h, f_all = cfg.hidden_size, cfg.moe_ffn_hidden_size
        self.cfg = cfg
        self.ep_rank, self.ep_size = ep_rank, ep_size
        self.e_local = cfg.num_experts // ep_size
        self.fp8 = fp8
        # expert tensor parallelism: this rank holds 1 / etp.size of every local expert's feed-forward columns and
        # routes all of the group's tokens; the partial outputs are summed over the group
        self.etp = etp
        f = f_all // (etp.size if etp is not None else 1)
        self.router = nn.Parameter(torch.empty(cfg.num_experts, h))
        self.experts_w1 = nn.Parameter(torch.empty(self.e_local, 2 * f, h))
        self.experts_w2 = nn.Parameter(torch.empty(self.e_local, h, f))
        self.experts_w1.is_expert = True
        self.experts_w2.is_expert = True
        if etp is not None:
            from ..parallel.tp import mark_sharded
            mark_sharded(self.experts_w1, 1, (self.e_local, 2 * f_all, h), etp.segments([f_all, f_all]))
            mark_sharded(self.experts_w2, 2, (self.e_local, h, f_all), etp.segments([f_all]))
        if cfg.moe_router_load_balancing_type == "bias":
            self.register_buffer("router_bias", torch.zeros(cfg.num_experts), persistent=True)
        else:
            self.router_bias = None
        self.shared = DenseFFN(h, cfg.moe_shared_expert_intermediate_size, etp) \
            if cfg.moe_shared_expert_intermediate_size else None
        # logical (router) expert id -> physical slot (rank * E_local + local index); changed by expert relocation
        self.register_buffer("expert_map", torch.arange(cfg.num_experts), persistent=True)
        self.relocated = False
        self.dispatcher = None            # set by the engine (needs the process group)
        self.keep_dispatched = False      # set by the engine: a recomputed block reuses the rows of its first run
        self.aux = None                   # last aux loss (added to the objective by the trainer)
        self.aux_scale = 1.0
        self.last_tokens_per_expert = None
        self.step_tokens_per_expert = None   # summed over the micro-batches of the current step

    def aux_enabled(self) -> bool:
        cfg = self.cfg
        return cfg.moe_router_load_balancing_type == "aux_loss" and cfg.moe_aux_loss_coeff > 0 and self.training

    def forward(self, x):
        cfg = self.cfg
        x_in = x
        if self.etp is not None:
            # whole sequences for the router, which every rank of the group repeats (identity without sequence
            # parallelism; its backward keeps this rank's slice: the repeated computation's gradients are equal)
            x = self.etp.gather_seq(x)
        shp = x.shape
        x2 = x.reshape(-1, shp[-1])
        logits = ops.router_logits(x2, self.router)
        if cfg.moe_router_force_load_balancing:
            # Random-init routers send most tokens to a few experts; for throughput measurements route by a fixed
            # table of random logits instead (same table in forward and in the recomputed forward), keeping the
            # router GEMM and its gradient path in the graph.
            logits = _balance_table(logits) + (logits - logits.detach())
        # one kernel: scores, selection, gate weights, per-expert counts and the load-balancing loss
        # (aux_scale: 1 / tp when the block sees a tensor-parallel slice of the tokens; the slices' terms add up)
        aux_coeff = cfg.moe_aux_loss_coeff * self.aux_scale if self.aux_enabled() else 0.0
        w, idx, aux = ops.router_fused(logits, cfg.moe_router_topk, cfg.moe_router_score_function, self.router_bias,
                                       cfg.moe_norm_topk_prob, cfg.moe_router_topk_scaling_factor, aux_coeff)
        if aux_coeff:
            self.aux = aux
        if self.etp is not None:
            # the experts below are this rank's column slices: gradients of the rows and of the gate weights are
            # partial sums, added up over the group on the way back
            x2 = self.etp.copy_to(x2)
            w = self.etp.copy_to(w)
        d = self.dispatcher
        kept = KEPT[0] if (self.keep_dispatched and getattr(d, "keep_rows", 1) > 0) else None
        reuse = kept is not None and RECOMPUTE_PHASE[0] and "plan" in kept
        if reuse and hasattr(d, "kept_rows_fit") and not d.kept_rows_fit(kept["plan"]):
            kept.clear()                 # some rank received more rows than the fixed-size copy holds: dispatch again
            reuse = False
        if self.relocated and not reuse:
            idx = self.expert_map[idx.long()].to(idx.dtype)      # experts live where the placement put them
        plan = kept["plan"] if reuse else d.plan(idx)
        self.last_tokens_per_expert = plan.tokens_per_expert_global
        if not RECOMPUTE_PHASE[0]:
            c = plan.tokens_per_expert_global                    # by physical slot
            if self.relocated:
                c = c[self.expert_map]                           # ... reported by logical expert
            self.step_tokens_per_expert = c.clone() if self.step_tokens_per_expert is None \
                else self.step_tokens_per_expert + c
        if reuse:
            # the dispatched rows of the first run were kept: no plan exchange and no second dispatch, only the
            # autograd link from the rows back to the tokens (its backward is the usual exchange of gradients)
            xe, pe = d.redispatch_kept(plan, x2, w, kept["xe"], kept["pe"])
            out_buf = d.push_target(plan) if (getattr(d, "push", False) and ops.use_kernels(x2)) else \
                (d.expert_output_buffer() if hasattr(d, "expert_output_buffer") else None)
        elif hasattr(d, "dispatch"):            # fused path: rows and gate probabilities travel together
            # rows arrive expert by expert; when both expert GEMMs run on the hand-written kernel, the first one waits
            # for each expert's rows inside the kernel instead of this stream waiting for the whole exchange
            plan.defer_ready = defer = (getattr(d, "expert_ordered", False) and not self.fp8
                                        and ops.grouped_kernel_ok(x2, self.experts_w1)
                                        and ops.grouped_kernel_ok(x2, self.experts_w2))
            xe, pe = d.dispatch(plan, x2, w)
            # push mode: the GEMM epilogues write result rows into the token owners' memory themselves;
            # otherwise the GEMMs write the peer-visible buffer the owners pull from
            out_buf = d.push_target(plan) if (d.push and ops.use_kernels(x2)) else d.expert_output_buffer()
        else:
            xe = d.dispatch_rows(plan, x2)
            pe = d.dispatch_scalars(plan, w)
            out_buf = None
        ready = getattr(plan, "ready", None)
        if kept is not None and not RECOMPUTE_PHASE[0] and not torch.is_grad_enabled():
            if ready is not None:                   # the copy reads every row
                ready.wait()
                d.join_side()
                ready = plan.ready = None
            kept["plan"] = plan
            kept["xe"], kept["pe"] = d.keep_dispatched(plan, xe, pe)
        h1 = ops.grouped_linear(xe, self.experts_w1.to(x.dtype), plan.expert_offsets, plan.expert_counts, self.fp8,
                                dgrad_out=out_buf, ready=ready)
        if ready is not None:
            plan.ready = None
            d.join_side()
        act = ops.swiglu_probs(h1, pe, rows_dev=getattr(plan, "meta", None))
        # In a recomputed forward nothing reads the block's result (it only feeds a residual add), so the second
        # expert GEMM and the combine exchange are skipped: their autograd nodes are all that backward needs.
        dead = RECOMPUTE_PHASE[0]
        defer_bwd = bool(getattr(plan, "defer_ready", False)) and hasattr(d, "take_bwd_ready")
        ye = ops.grouped_linear(act, self.experts_w2.to(x.dtype), plan.expert_offsets, plan.expert_counts, self.fp8,
                                out=out_buf, dead=dead, bwd_ready=d if defer_bwd else None)
        out = d.combine_rows(plan, ye, dead=dead, defer_bwd=True) if defer_bwd else d.combine_rows(plan, ye, dead=dead)
        if self.etp is not None:
            out = self.etp.leave(out.reshape(shp))          # sum of the column slices' partial outputs
            if self.shared is not None:
                out = out + self.shared(x_in)               # column-split like a dense block, with its own links
            return out
        if self.shared is not None:
            out = out + self.shared(x2)
        return out.reshape(shp)

    @torch.no_grad()
    def update_router_bias(self, global_tokens_per_expert: torch.Tensor) -> None:
        """Aux-loss-free balancing: nudge under-loaded experts up, over-loaded down
        (``moe/MegatronCore_MoE_reading_notes.md:686-698``)."""
        if self.router_bias is None:
            return
        load = global_tokens_per_expert.float()
        self.router_bias += self.cfg.moe_router_bias_update_rate * torch.sign(load.mean() - load)


class _Recompute(torch.autograd.Function):
    """Run ``fn(*inputs)`` without keeping its graph; rebuild and back-propagate it in backward.  Parameter
    gradients accumulate where the engine pointed them (``p.grad`` / ``main_grad`` views of the flat buffer).
    ``fn`` may return one tensor or a tuple (the block's output and its load-balancing loss).
    A plain Function instead of ``torch.utils.checkpoint``: no per-tensor hooks on the hot path."""

    @staticmethod
    def forward(ctx, fn, *inputs):
        ctx.fn = fn
        ctx.kept = {}
        ctx.save_for_backward(*inputs)
        KEPT[0] = ctx.kept
        try:
            with torch.no_grad():
                return fn(*inputs)
        finally:
            KEPT[0] = None

    @staticmethod
    def backward(ctx, *grads):
        ins = [t.detach().requires_grad_(t.is_floating_point()) for t in ctx.saved_tensors]
        prev, RECOMPUTE_PHASE[0] = RECOMPUTE_PHASE[0], True
        KEPT[0] = ctx.kept
        try:
            with torch.enable_grad():
                out = ctx.fn(*ins)
        finally:
            RECOMPUTE_PHASE[0] = prev
            KEPT[0] = None
            ctx.kept = None
        outs = out if isinstance(out, tuple) else (out,)
        pairs = [(o, g) for o, g in zip(outs, grads) if g is not None and o.requires_grad]
        torch.autograd.backward([o for o, _ in pairs], [g for _, g in pairs])
        return (None,) + tuple(t.grad for t in ins)


class DecoderLayer(nn.Module):
    def __init__(self, cfg: ModelConfig, layer_idx: int, ep_rank: int, ep_size: int, fp8: bool = False,
                 cp_group=None, tp=None, expert_tp: bool = False):
        super().__init__()
        self.expert_tp = expert_tp and tp is not None
        self.layer_idx = layer_idx
        self.eps = cfg.norm_epsilon
        self.tp = tp
        self.attn_norm = RMSNorm(cfg.hidden_size, cfg.norm_epsilon)
        attn_cls = MLAttention if cfg.attention_type == "mla" else GQAttention
        self.attn = attn_cls(cfg, layer_idx, cp_group, tp) if tp is not None else attn_cls(cfg, layer_idx, cp_group)
        self.ffn_norm = RMSNorm(cfg.hidden_size, cfg.norm_epsilon)
        self.is_moe = cfg.num_experts > 0 and layer_idx >= cfg.first_k_dense
        if self.is_moe:
            self.ffn = MoEFFN(cfg, ep_rank, ep_size, fp8, tp if self.expert_tp else None)
            if tp is not None and not self.expert_tp:
                # the block sees this rank's slice of the tokens: replicated parameters inside it (router, shared
                # expert) get partial gradients, summed over the tensor-parallel group by the engine
                self.ffn.aux_scale = 1.0 / tp.size
                for name, p in self.ffn.named_parameters():
                    if not getattr(p, "is_expert", False):
                        p.tp_partial_grad = True
        else:
            mlp_rank = cfg.lora_rank if "mlp" in cfg.lora_targets else 0
            self.ffn = DenseFFN(cfg.hidden_size, cfg.ffn_hidden_size, tp) if tp is not None \
                else DenseFFN(cfg.hidden_size, cfg.ffn_hidden_size, None, mlp_rank, cfg.lora_alpha)
        if tp is not None and tp.sequence_parallel:
            # the norms see this rank's part of every sequence only
            self.attn_norm.weight.tp_partial_grad = True
            self.ffn_norm.weight.tp_partial_grad = True
        self.recompute_ffn = False        # set by the engine for recompute_granularity=selective

    def _ffn_block(self, y, h):
        if self.tp is not None and self.is_moe and not self.tp.sequence_parallel and not self.expert_tp:
            # MoE under tensor parallelism: every rank of the group routes 1 / tp of the shared tokens through the
            # expert-parallel exchange, then the group reassembles the block's output
            shp = y.shape
            out = self.tp.gather_rows(self.ffn(self.tp.scatter_rows(y.reshape(-1, shp[-1]))))
            return h + out.reshape(shp)
        return h + self.ffn(y)

    def _ffn_block_aux(self, y, h):
        """The block plus the load-balancing loss its router produced, as a second output: inside a recomputed block
        the loss cannot leave through the module attribute (the first run builds no graph), so it travels through
        the recompute node like the block's output does."""
        out = self._ffn_block(y, h)
        aux, self.ffn.aux = self.ffn.aux, None
        if aux is None:
            aux = torch.zeros((), dtype=torch.float32, device=out.device)
        return out, aux

    def forward(self, x, cos, sin):
        a = self.attn(self.attn_norm(x), cos, sin)
        y, h = ops.rmsnorm_residual(a, x, self.ffn_norm.weight, self.eps)
        if self.recompute_ffn and torch.is_grad_enabled():
            # selective recompute: attention activations are kept, the feed-forward block (for MoE layers the
            # dispatch, both grouped GEMMs and the combine) is re-run in backward
            if self.is_moe and self.ffn.aux_enabled():
                out, aux = _Recompute.apply(self._ffn_block_aux, y, h)
                self.ffn.aux = aux            # picked up by the engine and added to the objective
                return out
            return _Recompute.apply(self._ffn_block, y, h)
        return self._ffn_block(y, h)


class Embedding(nn.Module):
    def __init__(self, cfg: ModelConfig):
        super().__init__()
        self.weight = nn.Parameter(torch.empty(cfg.vocab_size, cfg.hidden_size))

    def forward(self, tokens, dtype):
        return F.embedding(tokens, self.weight).to(dtype)


class Head(nn.Module):
    """Final norm + vocabulary projection + next-token cross entropy (never stores full logits on
    the kernel path)."""

    def __init__(self, cfg: ModelConfig):
        super().__init__()
        self.norm = RMSNorm(cfg.hidden_size, cfg.norm_epsilon)
        self.weight = nn.Parameter(torch.empty(cfg.vocab_size, cfg.hidden_size))

    def forward(self, x, targets):
        h = self.norm(x).reshape(-1, x.shape[-1])
        return ops.linear_cross_entropy(h, self.weight.to(h.dtype), targets.reshape(-1))

    def logits(self, x):
        return F.linear(self.norm(x), self.weight.to(x.dtype))


class SimpleMoE(nn.Module):
    """The layers ``[layer_start, layer_end)`` of the decoder plus, on the first/last pipeline
    stage, the embedding / head."""

    def __init__(self, cfg: ModelConfig, *, ep_rank: int = 0, ep_size: int = 1, fp8: bool = False,
                 layer_start: int = 0, layer_end: int | None = None, first_stage: bool = True,
                 last_stage: bool = True, cp_group=None, cp_rank: int = 0, cp_size: int = 1,
                 bf16_first_layers: int = 0, bf16_last_layers: int = 0, layer_ids=None, tp=None,
                 expert_tp: bool = False):
        super().__init__()
        self.cfg = cfg
        layer_end = cfg.num_layers if layer_end is None else layer_end
        # layer_ids: explicit (possibly non-contiguous) global layer indices, for interleaved pipeline stages
        ids = list(layer_ids) if layer_ids is not None else list(range(layer_start, layer_end))
        self.embed = Embedding(cfg) if first_stage else None

        def layer_fp8(i):          # the first / last layers of the whole decoder may be kept out of fp8
            return fp8 if bf16_first_layers <= i < cfg.num_layers - bf16_last_layers else False
        self.layers = nn.ModuleList(
            [DecoderLayer(cfg, i, ep_rank, ep_size, layer_fp8(i), cp_group, tp, expert_tp) for i in ids])
        self.head = Head(cfg) if last_stage else None
        if tp is not None and tp.sequence_parallel:
            # embedding, final norm and vocabulary projection run on this rank's part of every sequence
            for mod in (self.embed, self.head):
                if mod is not None:
                    for p in mod.parameters():
                        p.tp_partial_grad = True
        if cfg.lora_rank > 0:
            if cfg.attention_type != "gqa":
                raise ValueError("LoRA adapters are implemented for GQA attention")
            for name, p in self.named_parameters():          # only the adapters train
                p.requires_grad_(".lora_" in name or name.startswith("lora_"))
        self.ep_rank, self.ep_size = ep_rank, ep_size
        self.cp_rank, self.cp_size = cp_rank, cp_size
        self.rope_dim = cfg.qk_rope_head_dim if cfg.attention_type == "mla" else cfg.kv_channels
        self._rope_cache = {}

    def rope_tables(self, seq_local: int, device):
        key = (seq_local, str(device))
        if key not in self._rope_cache:
            # rotary positions of this rank's sequence chunk (context parallel shards the sequence)
            self._rope_cache[key] = ref.rope_tables(seq_local, self.rope_dim, self.cfg.rotary_base, device,
                                                    offset=self.cp_rank * seq_local)
        return self._rope_cache[key]

    @torch.no_grad()
    def init_weights(self, seed: int) -> None:
        """N(0, init_method_std) for matrices, ones for norm gains.  Expert tensors are filled one
        global expert at a time so every expert-parallel layout sees the same values."""
        std = self.cfg.init_method_std
        for name, p in self.named_parameters():
            gname = self._global_name(name)
            if name.endswith("norm.weight") or ".q_norm." in name or ".kv_norm." in name:
                p.fill_(1.0)
            elif name.endswith("lora_b"):
                p.zero_()
            elif getattr(p, "is_expert", False):
                e_local = p.shape[0]
                for j in range(e_local):
                    seeded_normal_(p[j], std, seed, f"{gname}.{self.ep_rank * e_local + j}")
            else:
                seeded_normal_(p, std, seed, gname)

    def _global_name(self, name: str) -> str:
        parts = name.split(".")
        if parts[0] == "layers":
            parts[1] = str(self.layers[int(parts[1])].layer_idx)
        return ".".join(parts)

    def forward(self, tokens_or_hidden, targets=None, dtype=torch.float32):
        """Plain (engine-less) forward for tests and small runs: tokens -> loss or hidden."""
        x = self.embed(tokens_or_hidden, dtype) if self.embed is not None else tokens_or_hidden
        cos, sin = self.rope_tables(x.shape[1], x.device)
        for layer in self.layers:
            x = layer(x, cos, sin)
        if self.head is None:
            return x
        return self.head(x, targets) if targets is not None else self.head.logits(x)

    def moe_layers(self):
        return [l.ffn for l in self.layers if l.is_moe]
