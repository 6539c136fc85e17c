"""LoRA fine-tuning: adapters on the attention (and dense feed-forward) projections train, everything else is frozen
and owns neither gradients nor optimizer state; layouts agree; a base-model checkpoint loads into a LoRA job."""
import pytest
import torch

from tests.distutil import run_ranks

DENSE = ["num_experts=0", "ffn_hidden_size=256", "global_batch_size=8", "micro_batch_size=2", "train_iters=6", "lr=3e-3"]
LORA = DENSE + ["lora_rank=4", "lora_alpha=8", "lora_targets=attn+mlp"]


def _train(rank, world, overrides, steps, save=None, load=None):
    from system_lab_b200.config import Config
    from system_lab_b200.trainer.loop import Trainer
    cfg = Config.load(preset="simplemoe-tiny", overrides=list(overrides) + ["device=cpu"])
    tr = Trainer(cfg)
    if load:
        tr.load_checkpoint(load)
    frozen0 = {g.name: g.shard.clone() for g in tr.engine.all_groups() if g.frozen}
    losses = [float(tr.train_step()["loss"]) for _ in range(steps)]
    if save:
        tr.save_checkpoint(save)
    for u in tr.engine.units:                     # parameters of sharded groups are only readable while gathered
        u.gather()
    lora_b = float(sum(p.detach().float().norm() for u in tr.engine.units for n, p in u.module.named_parameters()
                       if n.endswith("lora_b")))
    for u in tr.engine.units:
        u.release()
    info = {
        "frozen_groups": sorted(g.name.rsplit("/", 1)[1] for g in tr.engine.all_groups() if g.frozen),
        "trainable_elems": sum(g.shard_numel for g in tr.engine.all_groups() if not g.frozen),
        "frozen_unchanged": all(torch.equal(g.shard, frozen0[g.name]) for g in tr.engine.all_groups() if g.frozen),
        "moments": sorted(tr.optimizer.m),
        "lora_b_norm": lora_b,
    }
    return losses, info


def test_adapters_train_and_the_base_model_stays_frozen():
    (base, _), = run_ranks(_train, 1, DENSE + ["expert_model_parallel_size=1"], 1)
    (lora, info), = run_ranks(_train, 1, LORA + ["expert_model_parallel_size=1"], 6)
    assert lora[0] == pytest.approx(base[0], rel=1e-6)            # B = 0: the adapted model starts as the base model
    assert lora[-1] < lora[0]                                      # ... and the adapters learn (same batch stream)
    assert info["frozen_unchanged"] and info["lora_b_norm"] > 0
    assert set(info["frozen_groups"]) == {"frozen"}
    assert all(not k.endswith("/frozen") for k in info["moments"])                 # no optimizer state for frozen groups
    # adapters: 2 layers x (qkv + o + w1 + w2) x rank 4; far below the 1.4 M base parameters
    assert info["trainable_elems"] < 60_000


def test_lora_layouts_agree_and_a_base_checkpoint_loads(tmp_path):
    (single, _), = run_ranks(_train, 1, LORA + ["expert_model_parallel_size=1"], 4)
    res = run_ranks(_train, 2, LORA + ["expert_model_parallel_size=1"], 4)
    for losses, info in res:
        assert losses == pytest.approx(single, rel=2e-5, abs=2e-5)
        assert info["frozen_unchanged"]
    # pre-train the dense model for two steps, then fine-tune adapters from that checkpoint on another layout
    ck = str(tmp_path / "base")
    run_ranks(_train, 2, DENSE + ["expert_model_parallel_size=1"], 2, ck)
    (ft, info), = run_ranks(_train, 1, LORA + ["expert_model_parallel_size=1"], 3, None, ck)
    assert info["frozen_unchanged"] and info["lora_b_norm"] > 0
    assert abs(ft[0] - 6.93) < 0.3
