import json

import pytest

from system_lab_b200.config import Config, ConfigError, parse_bool
from system_lab_b200.pilot.constraints import check_config, estimate_memory, param_counts


def test_strict_bool_parsing():
    assert parse_bool("false") is False and parse_bool("True") is True and parse_bool("0") is False
    for bad in ("flase", "", "2", None, 3):
        with pytest.raises(ConfigError):
            parse_bool(bad)


def test_string_false_is_false_not_truthy():
    cfg = Config.load(preset="simplemoe-tiny", overrides=["fsdp=false", "fp8=False"])
    assert cfg.parallel.fsdp is False and cfg.precision.fp8 is False


def test_resolution_order_and_dump(tmp_path):
    y = tmp_path / "c.yaml"
    y.write_text("preset: simplemoe-tiny\nmodel:\n  num_layers: 3\ntrain:\n  lr: 1.0e-3\n")
    cfg = Config.load(str(y), overrides=["lr=2e-3", "model.hidden_size=128", "num_attention_heads=2",
                                         "num_query_groups=2"])
    assert cfg.model.num_layers == 3 and cfg.train.lr == 2e-3 and cfg.model.hidden_size == 128
    cfg.dump(tmp_path / "resolved.json")
    assert json.loads((tmp_path / "resolved.json").read_text())["train"]["lr"] == 2e-3


def test_unknown_and_ambiguous_keys():
    with pytest.raises(ConfigError):
        Config.load(preset="simplemoe-tiny", overrides=["no_such_key=1"])
    with pytest.raises(ConfigError):
        Config.load(preset="simplemoe-tiny", overrides=["lr"])
    with pytest.raises(ConfigError):
        Config.load(preset="simplemoe-tiny", overrides=["num_layers=2.5"])


def test_legality_rules_in_stable_order():
    cfg = Config.load(preset="simplemoe-tiny")
    cfg.parallel.expert_model_parallel_size = 3
    cfg.model.moe_router_topk = 99
    rules = [p["rule"] for p in check_config(cfg, world_size=4)]
    assert rules.index("ep_divides_dp_or_world") < rules.index("ep_divides_num_experts") < rules.index("top_k_le_num_experts")
    with pytest.raises(ConfigError):
        cfg.validate(4)


def test_gbs_and_pp_rules():
    cfg = Config.load(preset="simplemoe-tiny", overrides=["global_batch_size=6"])
    assert any(p["rule"] == "gbs_decomposes" for p in check_config(cfg, 2))
    cfg = Config.load(preset="simplemoe-tiny", overrides=["pipeline_model_parallel_size=2", "global_batch_size=8",
                                                         "micro_batch_size=4", "expert_model_parallel_size=1"])
    assert any(p["rule"] == "num_microbatch_geq_pp" for p in check_config(cfg, 2)) is False
    assert any(p["rule"] == "very_small_num_microbatch" and p["severity"] == "warning" for p in check_config(cfg, 2))


def test_param_counts_and_memory_model():
    cfg = Config.load(preset="qwen3-30b-a3b")
    pc = param_counts(cfg.model)
    assert 30.0e9 < pc["total"] < 31.0e9 and 3.2e9 < pc["active_per_token"] < 3.5e9
    assert not estimate_memory(cfg, 1)["fits"]            # fp32 master + fp32 moments cannot fit one GPU
    assert estimate_memory(cfg, 8)["fits"]
    cfg.precision.master_weights, cfg.precision.optimizer_state_dtype = False, "fp8"
    cfg.train.optimizer_in_backward = True
    cfg.train.global_batch_size = 2
    est = estimate_memory(cfg, 1)
    assert est["fits"] and 110 < est["total_bytes"] / 2**30 < 135
    ds = Config.load(preset="deepseek-v3-proxy")
    assert param_counts(ds.model)["total"] > 80e9


def test_tensor_parallel_and_hybrid_sharding_rules():
    def rules(ov, world):
        cfg = Config.load(preset="simplemoe-tiny")
        cfg.train.micro_batch_size = 1
        for item in ov:                      # set fields directly: Config.load would refuse an illegal combination
            k, v = item.split("=")
            sec = cfg.parallel if hasattr(cfg.parallel, k) else cfg.model
            setattr(sec, k, {"false": False, "true": True}.get(v, int(v) if v.isdigit() else v))
        return [p["rule"] for p in check_config(cfg, world) if p["severity"] == "error"]
    assert rules(["tensor_model_parallel_size=2", "expert_model_parallel_size=2"], 2) == []
    assert "tp_divides_num_heads" in rules(["tensor_model_parallel_size=8", "expert_model_parallel_size=1"], 8)
    assert "etp_is_one_or_tp" in rules(["tensor_model_parallel_size=2", "expert_tensor_parallel_size=4",
                                        "expert_model_parallel_size=1"], 2)
    assert rules(["tensor_model_parallel_size=2", "expert_tensor_parallel_size=2", "expert_model_parallel_size=1"], 2) == []
    assert "sp_needs_tp" in rules(["sequence_parallel=true", "expert_model_parallel_size=1"], 1)
    assert rules(["tensor_model_parallel_size=2", "expert_model_parallel_size=2", "sequence_parallel=true"], 2) == []
    assert "tp_excludes_hsdp" in rules(["tensor_model_parallel_size=2", "num_distributed_optimizer_instances=2"], 8)
    assert rules(["num_distributed_optimizer_instances=2", "expert_model_parallel_size=2"], 4) == []
    assert "hsdp_divides_data_ranks" in rules(["num_distributed_optimizer_instances=3", "expert_model_parallel_size=2"], 4)
    assert "hsdp_needs_fsdp" in rules(["num_distributed_optimizer_instances=2", "fsdp=false",
                                       "expert_model_parallel_size=2"], 4)
    # tensor parallelism shrinks the sharded attention state and the MoE activations of a rank
    big = Config.load(preset="qwen3-30b-a3b", overrides=["expert_model_parallel_size=8"])
    tp2 = Config.load(preset="qwen3-30b-a3b", overrides=["expert_model_parallel_size=8", "tensor_model_parallel_size=2"])
    assert estimate_memory(tp2, 8)["activation_bytes"] < estimate_memory(big, 8)["activation_bytes"]


def test_inert_knobs_are_reported_not_ignored():
    cfg = Config.load(preset="simplemoe-tiny", overrides=["overlap_grad_reduce=false", "moe_permute_fusion=false"])
    warns = [p for p in check_config(cfg, 2) if p["rule"] == "knob_has_no_effect"]
    assert len(warns) == 2 and all(p["severity"] == "warning" for p in warns)
    assert not [p for p in check_config(Config.load(preset="simplemoe-tiny"), 2) if p["rule"] == "knob_has_no_effect"]
    with pytest.raises(ConfigError, match="tie_embeddings"):
        Config.load(preset="simplemoe-tiny", overrides=["tie_embeddings=true"])


@pytest.mark.parametrize("name,world", [("qwen3_30b_a3b_8gpu", 8), ("deepseek_v3_proxy_pp2_ep4", 8),
                                        ("llama2_70b_lora_8gpu", 8), ("simplemoe_tiny_cpu", 2),
                                        ("gpt_oss_20b_tp2_sp_8gpu", 8)])
def test_example_configs_load_and_fit(name, world):
    from pathlib import Path
    cfg = Config.load(Path(__file__).resolve().parent.parent / "configs" / f"{name}.yaml")
    cfg.validate(world)
    assert estimate_memory(cfg, world)["fits"]


def test_lr_schedules():
    from system_lab_b200.trainer.optim import lr_at
    kw = dict(lr=1.0, min_lr=0.1, warmup=2, decay_iters=10)
    assert [round(lr_at(s, style="wsd", wsd_decay_iters=4, **kw), 3) for s in (1, 2, 6, 7, 10, 12)] == \
        [0.5, 1.0, 1.0, 0.775, 0.1, 0.1]
    assert lr_at(10, style="cosine", **kw) == pytest.approx(0.1) and lr_at(6, style="linear", **kw) == pytest.approx(0.55)
    assert lr_at(50, style="constant", **kw) == 1.0
    with pytest.raises(ValueError):
        lr_at(5, style="nope", **kw)


def test_fused_reduce_scatter_update_is_refused_for_replicated_groups():
    """The fused reduce-scatter + AdamW kernel accumulates the undivided sum of squared gradients; a group that other
    ranks hold copies of (dense parameters under tensor parallelism) must take the path that divides by its
    replication, or the global norm (and the next step's clip coefficient) would count it twice."""
    import types
    import torch
    from system_lab_b200.trainer.optim import ShardedAdamW
    opt = ShardedAdamW.__new__(ShardedAdamW)
    opt.state_dtype = "fp32"
    g = types.SimpleNamespace(device=torch.device("cuda"), can_fuse_rs_adamw=lambda: True, replica_group=None,
                              tp_replicas=1)
    assert opt.fusable(g)
    g.tp_replicas = 2
    assert not opt.fusable(g)
