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
