"""Named model/run presets (nested dicts applied on top of the dataclass defaults)."""

PRESETS: dict[str, dict] = {
    # 2-layer plumbing model: runs on CPU/gloo, doubles as the oracle for every kernel.
    "simplemoe-tiny": {
        "model": dict(name="simplemoe-tiny", num_layers=2, hidden_size=256, num_attention_heads=4,
                      num_query_groups=4, kv_channels=64, vocab_size=1024, seq_length=128,
                      num_experts=8, moe_router_topk=2, moe_ffn_hidden_size=512,
                      moe_router_score_function="softmax", init_method_std=0.02,
                      moe_token_dispatcher_type="alltoall", moe_pad_expert_rows_to=1),
        "parallel": dict(expert_model_parallel_size=2, fsdp=True),
        "precision": dict(params_dtype="fp32"),
        "train": dict(micro_batch_size=4, global_batch_size=8, train_iters=20, lr=3e-4, seed=0),
    },
    # Qwen3-30B-A3B shape: 48 layers, GQA 32q/4kv x 128, 128 experts top-8, ffn 768.
    "qwen3-30b-a3b": {
        "model": dict(name="qwen3-30b-a3b", num_layers=48, hidden_size=2048, num_attention_heads=32,
                      num_query_groups=4, kv_channels=128, vocab_size=151936, seq_length=4096,
                      rotary_base=1e6, num_experts=128, moe_router_topk=8, moe_ffn_hidden_size=768,
                      moe_shared_expert_intermediate_size=0, moe_router_score_function="softmax",
                      moe_norm_topk_prob=True, first_k_dense=0,
                      # the model's own balancing: load-balancing loss with coefficient 1e-3; on top of it experts are
                      # re-placed on the expert-parallel ranks by measured load (-1: wherever the layout allows it,
                      # once at step 3 and then every 50 steps)
                      moe_router_load_balancing_type="aux_loss", moe_aux_loss_coeff=1e-3,
                      moe_expert_relocation_interval=-1),
        "parallel": dict(expert_model_parallel_size=8, fsdp=True),
        # expert GEMMs in bf16: at this model's K = 2048 / 768 the fp8 recipes do not pay for their quantisation
        # passes (fp8=true fp8_recipe=rowwise|blockwise|tensorwise switches them on)
        "precision": dict(params_dtype="bf16", fp8=False, fp8_recipe="rowwise",
                          recompute_granularity="full"),
        "train": dict(micro_batch_size=2, global_batch_size=16, lr=3e-4),
    },
    # DeepSeek-V3 shaped proxy: 8 layers (1 dense + 7 MoE), MLA, 256 routed + 1 shared expert.
    "deepseek-v3-proxy": {
        "model": dict(name="deepseek-v3-proxy", num_layers=8, hidden_size=7168, num_attention_heads=128,
                      num_query_groups=128, kv_channels=128, vocab_size=129280, seq_length=4096,
                      attention_type="mla", q_lora_rank=1536, kv_lora_rank=512, qk_nope_head_dim=128,
                      qk_rope_head_dim=64, v_head_dim=128, ffn_hidden_size=18432, first_k_dense=1,
                      num_experts=256, moe_router_topk=8, moe_ffn_hidden_size=2048,
                      moe_shared_expert_intermediate_size=2048, moe_router_score_function="sigmoid",
                      moe_router_load_balancing_type="bias", moe_router_topk_scaling_factor=2.5),
        "parallel": dict(pipeline_model_parallel_size=2, expert_model_parallel_size=4, fsdp=True),
        "precision": dict(params_dtype="bf16", fp8=True, fp8_recipe="blockwise",
                          recompute_granularity="full"),
        "train": dict(micro_batch_size=1, global_batch_size=32, lr=3e-4),
    },
    # Llama-2-70B with LoRA adapters on the attention projections (the MLPerf fine-tuning workload the reference
    # traced: notes/mlperf-llama/2026-04-29_llama2_70b_lora_baseline_trace_breakdown.md): dense, GQA 64q/8kv x 128,
    # 80 layers, sequence 8192; the base model is frozen, rank-16 adapters train.
    "llama2-70b-lora": {
        "model": dict(name="llama2-70b-lora", num_layers=80, hidden_size=8192, num_attention_heads=64,
                      num_query_groups=8, kv_channels=128, vocab_size=32000, seq_length=8192, rotary_base=10000.0,
                      ffn_hidden_size=28672, num_experts=0, first_k_dense=0, lora_rank=16, lora_alpha=32.0,
                      lora_targets="attn"),
        "parallel": dict(expert_model_parallel_size=1, fsdp=True),
        "precision": dict(params_dtype="bf16", recompute_granularity="selective"),
        "train": dict(micro_batch_size=1, global_batch_size=8, lr=4e-4),
    },
    # GPT-OSS-20B shape (the reference's measured workload): hd64 GQA 64q/8kv, 32 experts top-4,
    # sliding window 128 on alternate layers, rotary base 150000.
    "gpt-oss-20b": {
        "model": dict(name="gpt-oss-20b", num_layers=24, hidden_size=2880, num_attention_heads=64,
                      num_query_groups=8, kv_channels=64, vocab_size=201088, seq_length=8192,
                      rotary_base=150000.0, sliding_window=128, num_experts=32, moe_router_topk=4,
                      moe_ffn_hidden_size=2880, moe_router_score_function="softmax",
                      # with 32 experts a random-init router loads the expert-parallel ranks 1.8 : 1; the balancing loss
                      # plus re-placement of the experts by measured load brings that to 1.1 and the 4-GPU step from 938 to 838 ms
                      moe_router_load_balancing_type="aux_loss", moe_aux_loss_coeff=1e-3,
                      moe_expert_relocation_interval=-1),
        "parallel": dict(expert_model_parallel_size=8, fsdp=True),
        "precision": dict(params_dtype="bf16", fp8=True, recompute_granularity="full"),
        "train": dict(micro_batch_size=2, global_batch_size=16),
    },
}
