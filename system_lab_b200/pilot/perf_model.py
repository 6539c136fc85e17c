"""Analytic execution model for one B200 NVSwitch box: ``T_step = T_comp + T_comm_exposed + T_bubble``.

The tuner needs an *expected* step time before anything has run (PROJECTION's prior, the ``tps < 0.8 x expected``
soft signal of DIAGNOSE, the gain estimates of REPLAN).  The reference specifies the decomposition and a cache of
fitted coefficients (``skills/pilot/execution-model/SKILL.md:28-63``) but ships no numbers; the coefficients here
are the achieved rates of this framework's kernels on B200, each a measured figure (see ``RATES``), so the model is
a roofline with measured efficiencies rather than nominal peaks.  ``projection.py`` refines it from micro-runs.

All times in milliseconds, per optimizer step, for the slowest rank.
"""
from __future__ import annotations

from dataclasses import dataclass, asdict
from typing import Any

from .constraints import param_counts

# Achieved rates (measured with CUDA events on B200, see the benchmark scripts next to each figure)
RATES = {
    "expert_gemm_tflops": 1085.0,      # grouped GEMM fwd+bwd average, benchmarks/grouped_gemm.py
    "dense_gemm_tflops": 1400.0,       # library GEMMs (qkv / out / head projections, 8k-token batches) inside a step
    "attention_tflops": 1100.0,        # library flash attention fwd+bwd, seq 4096, head dim <= 128 (fwd ~1330, bwd ~1010)
    "attention_tflops_wide_head": 300.0,   # head dim > 128 (MLA 192): falls off the library's fast path
    "elementwise_tbs": 4.0,            # norms / SwiGLU / RoPE / residual adds: bytes moved per second
    "adamw_tbs": 4.3,                  # fused AdamW kernel, bytes read + written
    "link_gbs": 770.0,                 # peer copy, per direction
    "dispatch_eff": 0.62,              # scatter kernels' share of link_gbs (incl. flag waits with balanced load)
    "combine_eff": 0.80,
    "fsdp_eff": 0.20,                  # peer all-gather / reduce-scatter of ~40 MB layers (latency and flag waits dominate)
    "launch_gap_ms_per_layer": 0.25,   # residual host / launch gaps per layer per pass
    # Waiting at the cross-rank meeting points of a MoE layer (five per layer: three exchanges of rows one way, two the
    # other) beyond what load imbalance explains, per layer, by expert-parallel size.  Fitted to the measured
    # Qwen3-30B-A3B steps (354 / 384 / 430 / 539 ms at 1 / 2 / 4 / 8 GPUs): the other terms reproduce 1 to 4 GPUs within
    # 5 % and leave 2.3 ms per layer at 8 unexplained (arrival skew among eight ranks; no 8-GPU trace exists).
    "meeting_wait_ms_per_layer": {8: 2.3},
    "tp_allreduce_eff": 0.55,          # NCCL all-reduce / all-gather of a micro-batch's activations (tens of MB): share of
                                       # the 725 GB/s bus bandwidth of a 1 GiB all-reduce; not measured under tp yet
}


@dataclass
class StepEstimate:
    t_expert_gemm: float
    t_dense_gemm: float
    t_attention: float
    t_elementwise: float
    t_optimizer: float
    t_dispatch: float
    t_fsdp: float
    t_imbalance: float
    t_bubble: float
    t_step: float
    tokens_per_step: int
    tps: float
    t_tp_comm: float = 0.0

    def to_dict(self) -> dict:
        return asdict(self)


def estimate_step(cfg: Any, world: int, *, rank_load_ratio: float = 1.0, rates: dict | None = None) -> StepEstimate:
    """Step time of ``cfg`` on ``world`` GPUs.  ``rank_load_ratio`` = max / mean rows per expert-parallel rank
    (1.0 = balanced): the most loaded rank's expert GEMMs and ingress set the pace of every layer."""
    r = dict(RATES)
    r.update(rates or {})
    m, p, pr, t = cfg.model, cfg.parallel, cfg.precision, cfg.train
    pp = max(p.pipeline_model_parallel_size, 1)
    cp = max(p.context_parallel_size, 1)
    tp = max(p.tensor_model_parallel_size, 1)
    dp = max(world // (pp * cp * tp), 1)
    ep = max(min(p.expert_model_parallel_size, dp * tp), 1)     # the MoE blocks' data axis runs over dp x tp
    nmb = max(t.global_batch_size // max(t.micro_batch_size * dp, 1), 1)
    tokens = t.micro_batch_size * m.seq_length // cp           # per micro-batch per rank
    layers = m.num_layers // pp
    moe_layers = max(layers - (m.first_k_dense if pp == 1 else m.first_k_dense // pp), 0) if m.num_experts else 0
    dense_layers = layers - moe_layers
    h, f, k = m.hidden_size, m.moe_ffn_hidden_size, m.moe_router_topk
    gran = pr.recompute_granularity
    # forward passes of the FFN block: 1 + recompute (the recomputed one skips fc2: 2/3 of the expert FLOPs)
    ffn_fwd = 1.0 + (2.0 / 3.0 if gran in ("selective", "full") else 0.0)
    attn_fwd = 1.0 + (1.0 if gran == "full" else 0.0)

    # ---- compute -------------------------------------------------------------------------------------------------
    slots = tokens * k // tp                                   # rows per rank at balanced load (EP keeps it constant)
    expert_fwd = 2.0 * slots * 3 * h * f                       # fc1 (2f x h) + fc2 (h x f)
    expert_flops = expert_fwd * (ffn_fwd + 2.0) * moe_layers
    shared_f = m.moe_shared_expert_intermediate_size
    dense_ffn_fwd = 2.0 * tokens * 3 * h * m.ffn_hidden_size / tp
    shared_fwd = 2.0 * tokens * 3 * h * shared_f / tp
    if m.attention_type == "mla":
        qk, vd = m.qk_nope_head_dim + m.qk_rope_head_dim, m.v_head_dim
        proj = h * m.q_lora_rank + m.q_lora_rank * m.num_attention_heads * qk + h * (m.kv_lora_rank + m.qk_rope_head_dim) \
            + m.kv_lora_rank * m.num_attention_heads * (m.qk_nope_head_dim + vd) + m.num_attention_heads * vd * h
    else:
        qk = vd = m.kv_channels
        proj = h * (m.num_attention_heads + 2 * m.num_query_groups) * m.kv_channels + m.num_attention_heads * m.kv_channels * h
    proj_fwd = 2.0 * tokens * proj / tp                        # heads split (the replicated low-rank parts are small)
    # LoRA fine-tuning: the frozen projections need their input gradient but no weight gradient (the rank-r adapter
    # GEMMs are negligible)
    bwd = 1.0 if getattr(m, "lora_rank", 0) > 0 else 2.0
    head_flops = (1.0 + bwd) * 2.0 * tokens * h * m.vocab_size
    dense_flops = (proj_fwd * (attn_fwd + bwd)) * layers + (shared_fwd * (ffn_fwd + bwd)) * moe_layers \
        + (dense_ffn_fwd * (ffn_fwd + bwd)) * dense_layers + head_flops / pp
    attn_fwd_flops = 2.0 * tokens * m.seq_length * m.num_attention_heads * (qk + vd) / 2.0      # causal
    attn_flops = attn_fwd_flops * (attn_fwd + 2.5) * layers / tp
    act_b = 2
    ew_bytes = layers * tokens * h * act_b * 30 + moe_layers * slots * f * act_b * 10 * (ffn_fwd + 1.0) / 2.0
    t_expert = expert_flops / (r["expert_gemm_tflops"] * 1e9)
    t_dense = dense_flops / (r["dense_gemm_tflops"] * 1e9)
    t_attn = attn_flops / ((r["attention_tflops"] if max(qk, vd) <= 128 else r["attention_tflops_wide_head"]) * 1e9)
    t_ew = ew_bytes / (r["elementwise_tbs"] * 1e9) + r["launch_gap_ms_per_layer"] * layers * (1 + ffn_fwd / 2)

    # ---- optimizer (once per step) -----------------------------------------------------------------------------------
    pc = param_counts(m)
    shard = (pc["non_expert"] / pp / (dp if p.fsdp else 1)) + \
        (pc["experts"] / pp / ep / (max(dp * tp // ep, 1) if p.fsdp else 1))
    wb = 2 if pr.params_dtype == "bf16" else 4
    state_b = {"fp32": 8, "bf16": 4, "fp8": 2}[pr.optimizer_state_dtype]
    master_b = 4 if (wb == 2 and pr.master_weights) else 0
    if pc.get("lora"):
        shard = pc["lora"] / pp / (dp if p.fsdp else 1)         # only the adapters are updated
    adam_bytes = shard * (2 * (master_b or wb) + 2 * state_b + 2 + (2 if master_b else 0))
    t_opt = adam_bytes / (r["adamw_tbs"] * 1e9)
    # An update that runs beside backward on a side stream is not free on this part: it shares HBM bandwidth and
    # the 1 kW power budget with the expert GEMMs (measured: the GEMMs slow down by what the update takes).

    # ---- communication -------------------------------------------------------------------------------------------------
    t_disp = 0.0
    if moe_layers:
        scatters = 1.0 + (1.0 if gran in ("selective", "full") and m.moe_keep_dispatched_factor == 0 else 0.0) + 1.0
        combines = 1.0 + 1.0                                    # forward combine + backward of dispatch
        local = slots * h * act_b / ep * 2.0                    # rows that stay on the rank: read + write in HBM
        t_disp = moe_layers * local * (scatters + combines) / (r["elementwise_tbs"] * 1e9)
        if ep > 1:
            remote = slots * h * act_b * (ep - 1) / ep          # bytes leaving a rank per scatter / combine
            t_disp += moe_layers * remote * (scatters / (r["dispatch_eff"] * r["link_gbs"]) +
                                             combines / (r["combine_eff"] * r["link_gbs"])) / 1e6
    t_fsdp = 0.0
    if p.fsdp and dp > 1:
        layer_dense = pc["per_layer_non_expert"] * wb
        gathers = 2.0                                           # forward and backward re-gather
        t_fsdp = layers * layer_dense * (dp - 1) / dp * (gathers + 1.0) / (r["fsdp_eff"] * r["link_gbs"]) / 1e6
        edp = max(dp * tp // ep, 1)
        if edp > 1:
            layer_exp = pc["per_layer_expert"] / ep * wb
            t_fsdp += moe_layers * layer_exp * (edp - 1) / edp * 3.0 / (r["fsdp_eff"] * r["link_gbs"]) / 1e6
    # the most loaded rank of every layer: its share of expert compute and of the ingress traffic
    t_imb = (rank_load_ratio - 1.0) * (t_expert + t_disp) if ep > 1 else 0.0
    waits = r.get("meeting_wait_ms_per_layer") or {}
    if ep > 1 and waits:
        known = sorted(waits)
        at = max([k for k in known if k <= ep], default=None)       # the largest measured size not above ep
        if at is not None:
            t_imb += moe_layers * float(waits[at]) * (ep / at)      # grows with the number of ranks met

    # tensor parallelism: per layer and pass one all-reduce behind attention and one all-reduce (dense FFN) or
    # all-gather (MoE block) behind the feed-forward block, each over the micro-batch's activations; nothing hides them
    t_tp = 0.0
    if tp > 1:
        one = tokens * h * act_b * 2.0 * (tp - 1) / tp / (r["tp_allreduce_eff"] * 725.0) / 1e6
        t_tp = layers * one * ((attn_fwd + 1.0) + (ffn_fwd + 1.0))
    per_mb = t_expert + t_dense + t_attn + t_ew + t_disp + t_fsdp + t_imb + t_tp
    bubble = (pp - 1) / max(pp - 1 + nmb * max(p.virtual_pipeline_model_parallel_size, 1), 1)
    t_busy = per_mb * nmb
    t_bubble = t_busy * bubble / max(1.0 - bubble, 1e-9) if pp > 1 else 0.0
    t_step = t_busy + t_bubble + t_opt
    tokens_per_step = t.global_batch_size * m.seq_length
    return StepEstimate(t_expert * nmb, t_dense * nmb, t_attn * nmb, t_ew * nmb, t_opt, t_disp * nmb, t_fsdp * nmb,
                        t_imb * nmb, t_bubble, t_step, tokens_per_step, tokens_per_step / (t_step / 1e3), t_tp * nmb)


def expected_tps(cfg: Any, world: int, **kw) -> float:
    return estimate_step(cfg, world, **kw).tps
