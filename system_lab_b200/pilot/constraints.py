"""Config legality rules and the memory model (the tuner's ``constraint.*`` tools).

Behavioural spec: ``skills/pilot/constraints/config.md:29-150`` (legality rules and
their stable output order), ``skills/pilot/constraints/oom.md:36-103`` (memory
model and the 92 % HBM rule).  The reference ships these as prose plus stub tool
handlers (``pilot/agent/worker_tools.py:268-307``); here they are executable and
the trainer's own ``Config.validate`` calls the same function, so a plan the
tuner accepts is a plan the trainer accepts.
"""
from __future__ import annotations

from typing import Any

HBM_BYTES_B200 = 180 * 1024**3
HBM_SAFE_FRACTION = 0.92

_DTYPE_BYTES = {"fp32": 4, "bf16": 2, "fp16": 2, "fp8": 1}


def _p(rule: str, message: str, hint: str = "", severity: str = "error") -> dict:
    return {"rule": rule, "message": message, "hint": hint, "severity": severity}


def check_config(cfg: Any, world_size: int | None = None) -> list[dict]:
    """Return violations/warnings in the stable order: world size, model dims,
    micro-batching, MoE, dtype/numerics, sequence length."""
    m, p, pr, t = cfg.model, cfg.parallel, cfg.precision, cfg.train
    tp, pp, ep, cp = (p.tensor_model_parallel_size, p.pipeline_model_parallel_size,
                      p.expert_model_parallel_size, p.context_parallel_size)
    out: list[dict] = []
    # 1. world size
    dp = None
    if world_size is not None:
        if world_size % (tp * pp * cp) != 0:
            out.append(_p("world_size_match", f"tp*pp*cp={tp*pp*cp} does not divide world_size={world_size}",
                          "rebalance one of {tp, pp, cp}"))
        else:
            dp = world_size // (tp * pp * cp)
            if ep > world_size:
                out.append(_p("ep_le_world_size", f"ep={ep} > world_size={world_size}"))
            elif dp % ep != 0 and world_size % ep != 0:
                out.append(_p("ep_divides_dp_or_world", f"ep={ep} divides neither dp={dp} nor world={world_size}",
                              "pick ep from divisors(dp)"))
    if m.lora_rank > 0:
        if m.attention_type != "gqa":
            out.append(_p("lora_needs_gqa", "lora_rank > 0 is implemented for attention_type=gqa"))
        if tp > 1:
            out.append(_p("lora_excludes_tp", "LoRA adapters are not combined with tensor parallelism"))
        if m.lora_targets not in ("attn", "attn+mlp"):
            out.append(_p("lora_targets", f"lora_targets={m.lora_targets!r}: use 'attn' or 'attn+mlp'"))
    if getattr(p, "sequence_parallel", False):
        if tp <= 1:
            out.append(_p("sp_needs_tp", "sequence_parallel needs tensor_model_parallel_size > 1",
                          "set tp >= 2 or turn sequence_parallel off"))
        elif (m.seq_length // max(cp, 1)) % tp:
            out.append(_p("tp_divides_sequence", f"seq_length / cp = {m.seq_length // max(cp, 1)} % tp={tp} != 0 "
                                                 "(sequence_parallel shards every sequence over tp)"))
    etp = getattr(p, "expert_tensor_parallel_size", 1)
    if etp not in (1, tp):
        out.append(_p("etp_is_one_or_tp", f"expert_tensor_parallel_size={etp}: use 1 or tensor_model_parallel_size={tp}"))
    elif etp > 1:
        if m.num_experts > 0 and m.moe_ffn_hidden_size % etp:
            out.append(_p("etp_divides_moe_ffn", f"moe_ffn_hidden_size={m.moe_ffn_hidden_size} % etp={etp} != 0"))
        if dp is not None and dp % ep:
            out.append(_p("etp_ep_divides_dp", f"with expert tensor parallelism ep={ep} must divide dp={dp}"))
    if tp > 1:
        # heads and dense feed-forward columns split over tp; MoE blocks take 1/tp of the tokens per rank
        if (t.micro_batch_size * m.seq_length // max(cp, 1)) % tp:
            out.append(_p("tp_divides_tokens", f"tokens per micro-batch % tp={tp} != 0 (MoE blocks slice the tokens)"))
        if m.ffn_hidden_size % tp:
            out.append(_p("tp_divides_ffn", f"ffn_hidden_size={m.ffn_hidden_size} % tp={tp} != 0"))
        if p.num_distributed_optimizer_instances > 1:
            out.append(_p("tp_excludes_hsdp", "tensor parallelism is not combined with num_distributed_optimizer_instances > 1"))
        if m.moe_expert_relocation_interval > 0:
            out.append(_p("tp_excludes_relocation", "expert relocation needs tp == 1"))
    inst = p.num_distributed_optimizer_instances
    if inst > 1:
        # hybrid sharding: shard inside a block of data ranks, replicate across ``inst`` blocks
        if not p.fsdp:
            out.append(_p("hsdp_needs_fsdp", "num_distributed_optimizer_instances > 1 needs fsdp=true"))
        if dp is not None and (dp * cp) % inst:
            out.append(_p("hsdp_divides_data_ranks", f"data ranks per stage ({dp * cp}) % instances ({inst}) != 0",
                          "pick instances from divisors(dp*cp)"))
    # 2. model dims
    if m.num_attention_heads % tp:
        out.append(_p("tp_divides_num_heads", f"num_attention_heads={m.num_attention_heads} % tp={tp} != 0"))
    if m.num_query_groups % tp:
        out.append(_p("tp_divides_kv_heads_for_gqa", f"num_query_groups={m.num_query_groups} % tp={tp} != 0"))
    if m.num_attention_heads % max(m.num_query_groups, 1):
        out.append(_p("heads_divisible_by_groups",
                      f"num_attention_heads={m.num_attention_heads} % num_query_groups={m.num_query_groups} != 0"))
    if m.num_layers % (pp * p.virtual_pipeline_model_parallel_size):
        out.append(_p("pp_divides_num_layers", f"num_layers={m.num_layers} % (pp*vpp)="
                      f"{pp * p.virtual_pipeline_model_parallel_size} != 0"))
    if m.num_experts and m.num_experts % ep:
        out.append(_p("ep_divides_num_experts", f"num_experts={m.num_experts} % ep={ep} != 0",
                      "pick ep from divisors(num_experts)"))
    if m.attention_type not in ("gqa", "mla"):
        out.append(_p("attention_type", f"attention_type={m.attention_type!r} not in (gqa, mla)"))
    if m.attention_type == "mla" and min(m.kv_lora_rank, m.qk_nope_head_dim, m.qk_rope_head_dim, m.v_head_dim) <= 0:
        out.append(_p("mla_dims", "mla needs kv_lora_rank, qk_nope_head_dim, qk_rope_head_dim, v_head_dim > 0"))
    # 3. micro-batching
    if dp is not None:
        denom = t.micro_batch_size * dp
        if t.global_batch_size % denom:
            out.append(_p("gbs_decomposes", f"global_batch_size={t.global_batch_size} is not a multiple of mbs*dp={denom}",
                          "set gbs to a multiple of mbs x dp"))
        else:
            nmb = t.global_batch_size // denom
            if nmb < pp:
                out.append(_p("num_microbatch_geq_pp", f"num_microbatch={nmb} < pp={pp}"))
            elif pp > 1 and nmb < 2 * pp:
                out.append(_p("very_small_num_microbatch", f"num_microbatch={nmb} < 2*pp: bubble will dominate",
                              "mbs down or gbs up", severity="warning"))
            if t.optimizer_in_backward and nmb > 1:
                out.append(_p("optimizer_in_backward_single_microbatch",
                              "optimizer_in_backward needs exactly one micro-batch per step"))
    if p.virtual_pipeline_model_parallel_size > 1 and pp == 1:
        out.append(_p("vpp_requires_pp_gt_1", "vpp > 1 needs pp > 1"))
    if p.virtual_pipeline_model_parallel_size > 1 and pp > 1 and dp is not None:
        nmb_here = t.global_batch_size // max(t.micro_batch_size * dp, 1)
        if nmb_here % pp:
            out.append(_p("vpp_microbatches_multiple_of_pp", f"interleaved stages need micro-batches per step "
                          f"({nmb_here}) to be a multiple of pp ({pp})"))
    # 4. MoE
    if m.num_experts and m.moe_router_topk > m.num_experts:
        out.append(_p("top_k_le_num_experts", f"topk={m.moe_router_topk} > num_experts={m.num_experts}"))
    if m.moe_router_score_function not in ("softmax", "sigmoid"):
        out.append(_p("router_score_function", f"unknown score function {m.moe_router_score_function!r}"))
    if m.moe_token_dispatcher_type not in ("fused", "alltoall"):
        out.append(_p("dispatcher_type", f"unknown dispatcher {m.moe_token_dispatcher_type!r}"))
    if m.moe_router_load_balancing_type not in ("aux_loss", "bias", "none"):
        out.append(_p("load_balancing_type", f"unknown load balancing {m.moe_router_load_balancing_type!r}"))
    if m.num_experts and m.moe_expert_relocation_interval > 0 and dp is not None and (ep != dp or cp > 1):
        out.append(_p("expert_relocation_layout", "expert relocation moves whole experts between the ranks of one "
                      f"expert-parallel group: it needs ep == dp on the stage and cp == 1 (ep={ep}, dp={dp}, cp={cp})",
                      "set expert_model_parallel_size to dp"))
    if m.num_experts and pr.params_dtype == "bf16" and m.moe_pad_expert_rows_to % 128:
        out.append(_p("expert_rows_alignment", "bf16 models run the tcgen05 grouped GEMM, whose 128-row tiles need "
                      f"moe_pad_expert_rows_to % 128 == 0 (got {m.moe_pad_expert_rows_to})"))
    # 5. dtype / numerics
    if pr.params_dtype not in ("fp32", "bf16"):
        out.append(_p("params_dtype", f"params_dtype={pr.params_dtype!r} not in (fp32, bf16)"))
    if pr.optimizer_state_dtype not in ("fp32", "bf16", "fp8"):
        out.append(_p("optimizer_state_dtype", f"optimizer_state_dtype={pr.optimizer_state_dtype!r}"))
    if pr.fp8 and pr.fp8_recipe not in ("rowwise", "tensorwise", "blockwise"):
        out.append(_p("fp8_recipe", f"fp8_recipe={pr.fp8_recipe!r}"))
    if pr.fp8 and pr.optimizer_state_dtype != "fp32":
        out.append(_p("optim_state_dtype_for_dtype",
                      "fp8 compute with non-fp32 optimizer state: updates may stall", severity="warning"))
    if t.lr_decay_style not in ("constant", "cosine", "linear", "wsd"):
        out.append(_p("lr_decay_style", f"lr_decay_style={t.lr_decay_style!r} not in (constant, cosine, linear, wsd)"))
    if pr.recompute_granularity not in ("none", "selective", "full"):
        out.append(_p("recompute_granularity", f"recompute_granularity={pr.recompute_granularity!r}"))
    # knobs kept for vocabulary compatibility with Megatron-style launch files: a value that asks for behaviour this
    # trainer does not have is reported instead of being ignored silently
    if m.tie_embeddings:
        out.append(_p("tie_embeddings", "tie_embeddings=true is not implemented: embedding and head are separate matrices"))
    inert = [(m.moe_router_dtype != "fp32", "moe_router_dtype", "the router always runs in fp32"),
             (not m.moe_grouped_gemm, "moe_grouped_gemm", "experts always run as one grouped GEMM"),
             (not m.moe_permute_fusion, "moe_permute_fusion", "dispatch writes rows in their final order: no permute kernels"),
             (not p.use_distributed_optimizer, "use_distributed_optimizer",
              "optimizer state lives with the parameter shards (fsdp=true) or is replicated (fsdp=false)"),
             (not p.overlap_grad_reduce, "overlap_grad_reduce", "gradients are reduced per layer inside backward"),
             (not p.overlap_param_gather, "overlap_param_gather", "parameters are gathered per layer; see fsdp_prefetch"),
             (not p.grad_reduce_in_bf16 and pr.params_dtype == "bf16", "grad_reduce_in_bf16",
              "gradients are reduced in the parameter dtype and accumulated in fp32"),
             (not p.ddp_average_in_collective, "ddp_average_in_collective", "the loss is pre-scaled, sums need no average")]
    for hit, knob, why in inert:
        if hit:
            out.append(_p("knob_has_no_effect", f"{knob} is set to a non-default value but has no effect: {why}",
                          severity="warning"))
    # 6. sequence length
    if cp > 1 and m.seq_length % cp:
        out.append(_p("cp_divides_seq_len", f"seq_length={m.seq_length} % cp={cp} != 0"))
    if cp > 1 and m.num_attention_heads % cp:
        out.append(_p("cp_divides_heads", f"head-sharded context parallel needs num_attention_heads % cp == 0"))
    return out


# --------------------------------------------------------------------------
# parameter counts and the memory model
# --------------------------------------------------------------------------
def param_counts(m: Any) -> dict:
    """Parameter counts of the decoder described by ``ModelConfig`` (elements)."""
    h = m.hidden_size
    if m.attention_type == "mla":
        qk = m.qk_nope_head_dim + m.qk_rope_head_dim
        nh = m.num_attention_heads
        q = (h * m.q_lora_rank + m.q_lora_rank + m.q_lora_rank * nh * qk) if m.q_lora_rank else h * nh * qk
        kv = h * (m.kv_lora_rank + m.qk_rope_head_dim) + m.kv_lora_rank \
            + m.kv_lora_rank * nh * (m.qk_nope_head_dim + m.v_head_dim)
        attn = q + kv + nh * m.v_head_dim * h
    else:
        d = m.kv_channels
        attn = h * m.num_attention_heads * d + 2 * h * m.num_query_groups * d + m.num_attention_heads * d * h
    norms = 2 * h
    dense_ffn = 3 * h * m.ffn_hidden_size
    expert = 3 * h * m.moe_ffn_hidden_size
    shared = 3 * h * m.moe_shared_expert_intermediate_size
    router = h * m.num_experts + (m.num_experts if m.moe_router_load_balancing_type == "bias" else 0)
    n_moe = max(m.num_layers - m.first_k_dense, 0) if m.num_experts else 0
    n_dense = m.num_layers - n_moe
    embed = m.vocab_size * h * (1 if m.tie_embeddings else 2) + h
    non_expert = (attn + norms) * m.num_layers + dense_ffn * n_dense + (router + shared) * n_moe + embed
    experts = expert * m.num_experts * n_moe
    active = non_expert + expert * m.moe_router_topk * n_moe
    lora = 0
    r = getattr(m, "lora_rank", 0)
    if r > 0:
        d = m.kv_channels
        qkv_out = (m.num_attention_heads + 2 * m.num_query_groups) * d
        lora = m.num_layers * r * (h + qkv_out + m.num_attention_heads * d + h)
        if "mlp" in getattr(m, "lora_targets", ""):
            lora += n_dense * r * (h + 2 * m.ffn_hidden_size + m.ffn_hidden_size + h)
    return {"total": non_expert + experts + lora, "non_expert": non_expert, "experts": experts,
            "active_per_token": active, "per_layer_expert": expert * m.num_experts,
            "per_layer_non_expert": attn + norms + router + shared + (dense_ffn if n_moe == 0 else 0),
            "lora": lora, "trainable": lora if r > 0 else non_expert + experts}


def bytes_per_param(pr: Any, optimizer_in_backward: bool = False, microbatches: int = 1) -> float:
    """Resident bytes per (sharded) parameter: weight + master + grad + two moments.  Gradients of a single
    micro-batch are consumed in the compute dtype; accumulation over several micro-batches is fp32."""
    w = _DTYPE_BYTES[pr.params_dtype]
    master = 4 if (pr.params_dtype != "fp32" and pr.master_weights) else 0
    grad = 0 if optimizer_in_backward else (2 if (pr.params_dtype == "bf16" and microbatches <= 1) else 4)
    mom = {"fp32": 8.0, "bf16": 4.0, "fp8": 2.0 + 8.0 / 128}[pr.optimizer_state_dtype]
    return w + master + grad + mom


def estimate_memory(cfg: Any, world_size: int) -> dict:
    """Per-GPU peak memory estimate (bytes) of one training step.

    ``Mem_peak = params + grads + optimizer state + activations + transient buffers``
    (``skills/pilot/execution-model/SKILL.md:28-35``).  Expert parameters are
    sharded over ``ep`` and then over the remaining data ranks (``edp``); everything
    else over all data ranks when FSDP is on.
    """
    m, p, pr, t = cfg.model, cfg.parallel, cfg.precision, cfg.train
    pc = param_counts(m)
    pp = p.pipeline_model_parallel_size
    dp = max(world_size // (pp * p.tensor_model_parallel_size * p.context_parallel_size), 1)
    tp = max(p.tensor_model_parallel_size, 1)
    ep = min(p.expert_model_parallel_size, dp * tp)         # the MoE blocks' data axis runs over dp x tp
    edp = max(dp * tp // ep, 1)
    inst = max(p.num_distributed_optimizer_instances, 1)
    data = dp * p.context_parallel_size
    shard_dense = max(data // inst, 1) if p.fsdp else 1
    edp_all = edp * p.context_parallel_size
    edp_shard = (edp_all // inst if edp_all % inst == 0 else edp_all) if p.fsdp else 1
    shard_exp = ep * max(edp_shard, 1)
    nmb = max(t.global_batch_size // max(t.micro_batch_size * dp, 1), 1)
    bpp = bytes_per_param(pr, t.optimizer_in_backward, nmb)
    # tensor parallelism splits the attention / dense feed-forward matrices (most of the non-expert parameters);
    # embedding, head, norms and routers stay replicated: count them as unsplit to stay on the safe side
    emb_head = 2 * m.vocab_size * m.hidden_size
    non_expert = emb_head + max(pc["non_expert"] - emb_head, 0) / tp
    if pc["lora"]:
        # LoRA: the base model is frozen (compute-dtype shard only); adapters carry master, gradient and moments
        state = (non_expert / pp / shard_dense + pc["experts"] / pp / shard_exp) * _DTYPE_BYTES[pr.params_dtype] \
            + pc["lora"] / pp / shard_dense * bpp
    else:
        state = (non_expert / pp / shard_dense + pc["experts"] / pp / shard_exp) * bpp
    wbytes = _DTYPE_BYTES[pr.params_dtype]
    # transient: one layer's gathered params (+ its grads when optimizer runs in backward)
    layer_params = pc["per_layer_non_expert"] + pc["per_layer_expert"] / ep
    transient = layer_params * wbytes * (2 if p.fsdp else 0) + (layer_params * 2 if t.optimizer_in_backward else 0)
    tokens = t.micro_batch_size * m.seq_length // p.context_parallel_size
    h = m.hidden_size
    act_b = 2 if pr.params_dtype == "bf16" else 4
    layers_here = m.num_layers // pp
    slots = tokens * m.moe_router_topk // tp               # each tensor-parallel rank routes its slice of the tokens
    f = m.moe_ffn_hidden_size
    per_layer_full = tokens * h * act_b * 10 + slots * (2 * h + 3 * f) * act_b
    if pr.recompute_granularity == "full":
        acts = layers_here * tokens * h * act_b + per_layer_full
    elif pr.recompute_granularity == "selective":
        # attention side kept per layer (x, normed x, packed qkv twice, attention output, residual, normed
        # residual, layer output); one feed-forward block live at a time
        if m.attention_type == "mla":
            qkv_w = m.num_attention_heads * (2 * (m.qk_nope_head_dim + m.qk_rope_head_dim) + m.v_head_dim)
        else:
            qkv_w = (m.num_attention_heads + 2 * m.num_query_groups) * m.kv_channels
        attn_keep = tokens * act_b * (7 * h + 2 * qkv_w)
        acts = layers_here * attn_keep + per_layer_full
        if m.num_experts > 0 and m.moe_keep_dispatched_factor != 0:
            # dispatched rows (+ gate scalar, origin) of every MoE layer kept for the recomputed block
            moe_layers = max(layers_here - (m.first_k_dense if pp == 1 else 0), 0)
            kf = m.moe_keep_dispatched_factor if m.moe_keep_dispatched_factor > 0 else 2.0   # < 0: exact rows, bounded here by 2x
            kept_rows = kf * slots + (m.num_experts // ep) * m.moe_pad_expert_rows_to
            acts += moe_layers * kept_rows * (h * act_b + 8) * min(nmb, pp)
    else:
        acts = layers_here * per_layer_full
    logits = tokens * m.vocab_size * 4 / 4 + tokens * h * act_b * 2     # chunked cross entropy: quarter at a time
    total = state + transient + acts + logits
    cap = HBM_BYTES_B200
    return {"state_bytes": state, "transient_bytes": transient, "activation_bytes": acts,
            "logits_bytes": logits, "total_bytes": total, "hbm_bytes": cap,
            "fraction": total / cap, "fits": total <= HBM_SAFE_FRACTION * cap,
            "bytes_per_param": bpp}
