"""Model family coverage on CPU: MLA + shared expert + sigmoid/bias router (DeepSeek-V3 shaped), sliding window
(GPT-OSS shaped), dense-first layers; single process vs pipeline x expert parallel."""
import pytest

from tests.distutil import run_ranks

DSV3_TINY = ["attention_type=mla", "q_lora_rank=48", "kv_lora_rank=32", "qk_nope_head_dim=16", "qk_rope_head_dim=8",
             "v_head_dim=16", "num_layers=4", "first_k_dense=1", "ffn_hidden_size=256",
             "moe_shared_expert_intermediate_size=128", "moe_router_score_function=sigmoid",
             "moe_router_load_balancing_type=bias", "moe_router_topk_scaling_factor=2.5", "global_batch_size=8",
             "micro_batch_size=2"]


def _train(rank, world, overrides, steps):
    from system_lab_b200.config import Config
    from system_lab_b200.trainer.loop import Trainer
    cfg = Config.load(preset="simplemoe-tiny", overrides=list(overrides) + ["device=cpu"])
    tr = Trainer(cfg)
    out = [float(tr.train_step()["loss"]) for _ in range(steps)]
    bias = [f.router_bias.abs().sum().item() for f in tr.engine.moe_ffns() if f.router_bias is not None]
    return out, bias


def test_dsv3_shape_single_vs_pp2_ep2():
    (single, bias), = run_ranks(_train, 1, DSV3_TINY + ["expert_model_parallel_size=1"], 4)
    assert all(abs(l - 6.93) < 0.4 for l in single)
    assert bias and all(b > 0 for b in bias)                 # aux-loss-free balancing moved the bias
    res = run_ranks(_train, 4, DSV3_TINY + ["expert_model_parallel_size=2", "pipeline_model_parallel_size=2"], 4)
    assert res[0][0] == pytest.approx(single, rel=5e-5, abs=5e-5)


def test_sliding_window_and_aux_loss_run():
    ov = ["sliding_window=16", "moe_aux_loss_coeff=0.01", "expert_model_parallel_size=2", "global_batch_size=8",
          "micro_batch_size=2", "recompute_granularity=selective"]
    res = run_ranks(_train, 2, ov, 3)
    assert all(abs(l - 6.93) < 0.4 for l in res[0][0])


def test_fp8_expert_forward_tracks_the_unquantised_model():
    """fp8 (e4m3) forward of the expert GEMMs, emulated on the oracle path: the loss stays within quantisation noise of
    the unquantised run for both recipes, gradients flow through the unquantised operands, and the first / last
    layers can be kept out of fp8."""
    import torch
    from system_lab_b200.config import Config
    from system_lab_b200.trainer.loop import Trainer
    base = ["train_iters=4", "global_batch_size=4", "micro_batch_size=2", "expert_model_parallel_size=1",
            "hidden_size=256", "moe_ffn_hidden_size=128", "num_layers=3"]

    def run(extra):
        torch.manual_seed(0)
        tr = Trainer(Config.load(preset="simplemoe-tiny", overrides=base + extra))
        losses = [float(tr.train_step()["loss"]) for _ in range(4)]
        flags = [bool(l.ffn.fp8) for l in tr.engine.model.layers if l.is_moe]
        return losses, flags

    ref_l, ref_f = run([])
    assert not any(ref_f)
    for recipe in ("rowwise", "tensorwise", "blockwise"):
        l, f = run(["fp8=true", f"fp8_recipe={recipe}"])
        assert all(f)
        assert l != ref_l                                       # the forward really is quantised
        assert max(abs(a - b) for a, b in zip(l, ref_l)) < 2e-2
    _, f = run(["fp8=true", "num_layers_at_start_in_bf16=1", "num_layers_at_end_in_bf16=1"])
    assert f == [False, True, False]


def test_dsv3_shape_tensor_parallel_with_context_parallel():
    """MLA under tensor parallelism: heads split, low-rank down projections replicated; dense first layer
    column-split; shared expert and router see a token slice (gradients summed over the group)."""
    (single, _), = run_ranks(_train, 1, DSV3_TINY + ["expert_model_parallel_size=1"], 4)
    res = run_ranks(_train, 4, DSV3_TINY + ["expert_model_parallel_size=2", "tensor_model_parallel_size=2",
                                            "context_parallel_size=2"], 4)
    for losses, _ in res:
        assert losses == pytest.approx(single, rel=5e-5, abs=5e-5)


def test_dsv3_shape_sequence_parallel():
    """MLA under sequence parallelism: the repeated low-rank projections get whole sequences through a gather whose
    backward keeps the local slice; the dense first layer gathers and reduce-scatters."""
    (single, _), = run_ranks(_train, 1, DSV3_TINY + ["expert_model_parallel_size=1"], 4)
    res = run_ranks(_train, 2, DSV3_TINY + ["expert_model_parallel_size=2", "tensor_model_parallel_size=2",
                                            "sequence_parallel=true"], 4)
    for losses, _ in res:
        assert losses == pytest.approx(single, rel=5e-5, abs=5e-5)


def test_dsv3_shape_expert_tensor_parallel():
    """Shared expert column-split with the routed experts; MLA heads split; first layer dense."""
    (single, _), = run_ranks(_train, 1, DSV3_TINY + ["expert_model_parallel_size=1"], 4)
    res = run_ranks(_train, 2, DSV3_TINY + ["expert_model_parallel_size=1", "tensor_model_parallel_size=2",
                                            "expert_tensor_parallel_size=2"], 4)
    for losses, _ in res:
        assert losses == pytest.approx(single, rel=5e-5, abs=5e-5)


def test_aux_loss_is_carried_through_every_recompute_mode():
    """The load-balancing loss reaches the objective (and the router's gradient) whether the MoE block is kept,
    recomputed alone (selective: the loss leaves the recompute node as a second output) or with its whole layer
    (full): same loss curve, and a different one from the run without the loss term."""
    import torch
    from system_lab_b200.config import Config
    from system_lab_b200.trainer.loop import Trainer
    base = ["global_batch_size=4", "micro_batch_size=2", "expert_model_parallel_size=1", "device=cpu", "lr=1e-2"]

    def run(extra):
        torch.manual_seed(0)
        tr = Trainer(Config.load(preset="simplemoe-tiny", overrides=base + extra))
        return [float(tr.train_step()["loss"]) for _ in range(5)]

    plain = run(["moe_aux_loss_coeff=0.5", "recompute_granularity=none"])
    assert run(["moe_aux_loss_coeff=0.5", "recompute_granularity=selective"]) == pytest.approx(plain, rel=2e-6, abs=2e-6)
    assert run(["moe_aux_loss_coeff=0.5", "recompute_granularity=full"]) == pytest.approx(plain, rel=2e-6, abs=2e-6)
    without = run(["moe_aux_loss_coeff=0.0", "recompute_granularity=selective"])
    assert max(abs(a - b) for a, b in zip(plain[1:], without[1:])) > 1e-5      # the term moved the router
