"""End-to-end plumbing on CPU ranks (gloo): the same tiny model under different layouts must
produce the same loss curve; checkpoints resume bit-exactly and reload under another layout."""
import os

import pytest
import torch

from tests.distutil import run_ranks


def _train(rank, world, overrides, steps, save=None, load=None, steps_after_load=0):
    from system_lab_b200.config import Config
    from system_lab_b200.trainer.loop import Trainer
    cfg = Config.load(preset="simplemoe-tiny", overrides=list(overrides) + ["device=cpu"])
    tr = Trainer(cfg)
    if load:
        tr.load_checkpoint(load)
    losses = []
    for _ in range(steps):
        out = tr.train_step()
        losses.append(float(out["loss"]))
    if save:
        tr.save_checkpoint(save)
        for _ in range(steps_after_load):
            losses.append(float(tr.train_step()["loss"]))
    w = torch.cat([g.shard.float().reshape(-1)[:64] for g in tr.engine.all_groups()])
    return losses, float(w.double().sum())


BASE = ["global_batch_size=8", "micro_batch_size=2", "train_iters=6"]


@pytest.fixture(scope="module")
def single_curve():
    (losses, _), = run_ranks(_train, 1, BASE + ["expert_model_parallel_size=1"], 6)
    return losses


def test_single_process_loss_is_finite_and_near_log_vocab(single_curve):
    assert all(abs(l - 6.93) < 0.3 for l in single_curve)


def test_ep2_fsdp_matches_single(single_curve):
    res = run_ranks(_train, 2, BASE + ["expert_model_parallel_size=2"], 6)
    for losses, _ in res:
        assert losses == pytest.approx(single_curve, rel=2e-5, abs=2e-5)


def test_full_recompute_matches(single_curve):
    res = run_ranks(_train, 2, BASE + ["expert_model_parallel_size=2", "recompute_granularity=full"], 6)
    assert res[0][0] == pytest.approx(single_curve, rel=2e-5, abs=2e-5)


def test_selective_recompute_matches(single_curve):
    res = run_ranks(_train, 2, BASE + ["expert_model_parallel_size=2", "recompute_granularity=selective"], 6)
    assert res[0][0] == pytest.approx(single_curve, rel=2e-5, abs=2e-5)


def test_selective_recompute_with_kept_dispatch_matches(single_curve):
    """The recomputed block reuses the rows of its first dispatch (no second plan exchange / dispatch); with two
    micro-batches per step the kept state must stay attached to the right autograd node."""
    res = run_ranks(_train, 2, BASE + ["expert_model_parallel_size=2", "recompute_granularity=selective",
                                       "moe_keep_dispatched_factor=2.0"], 6)
    assert res[0][0] == pytest.approx(single_curve, rel=2e-5, abs=2e-5)


def test_dp2_ep1_fsdp_matches(single_curve):
    res = run_ranks(_train, 2, BASE + ["expert_model_parallel_size=1"], 6)
    assert res[0][0] == pytest.approx(single_curve, rel=2e-5, abs=2e-5)


def test_ddp_without_fsdp_matches(single_curve):
    res = run_ranks(_train, 2, BASE + ["expert_model_parallel_size=1", "fsdp=false"], 6)
    assert res[0][0] == pytest.approx(single_curve, rel=2e-5, abs=2e-5)


def test_pp2_ep2_matches(single_curve):
    res = run_ranks(_train, 4, BASE + ["expert_model_parallel_size=2", "pipeline_model_parallel_size=2"], 6)
    assert res[0][0] == pytest.approx(single_curve, rel=2e-5, abs=2e-5)


def test_cp2_matches(single_curve):
    res = run_ranks(_train, 2, BASE + ["expert_model_parallel_size=1", "context_parallel_size=2"], 6)
    assert res[0][0] == pytest.approx(single_curve, rel=5e-5, abs=5e-5)


def test_optimizer_in_backward_runs():
    ov = ["global_batch_size=4", "micro_batch_size=2", "expert_model_parallel_size=2",
          "optimizer_in_backward=true", "recompute_granularity=full"]
    res = run_ranks(_train, 2, ov, 4)
    assert all(abs(l - 6.93) < 0.3 for l in res[0][0])


def test_checkpoint_resume_bit_exact(tmp_path):
    ov = BASE + ["expert_model_parallel_size=2"]
    ck = str(tmp_path / "ck")
    full = run_ranks(_train, 2, ov, 3, ck, None, 3)          # 3 steps, save, 3 more
    resumed = run_ranks(_train, 2, ov, 3, None, ck)           # load, 3 steps
    assert resumed[0][0] == full[0][0][3:]                    # bit-exact continuation
    assert resumed[0][1] == full[0][1] and resumed[1][1] == full[1][1]


def test_checkpoint_reshard_ws2_to_ws1(tmp_path):
    ck = str(tmp_path / "ck")
    full = run_ranks(_train, 2, BASE + ["expert_model_parallel_size=2"], 3, ck, None, 3)
    resumed = run_ranks(_train, 1, BASE + ["expert_model_parallel_size=1"], 3, None, ck)
    assert resumed[0][0] == pytest.approx(full[0][0][3:], rel=2e-5, abs=2e-5)


def test_interleaved_virtual_pipeline_matches():
    """pp=2 with two virtual stages per rank (blocks 0,2 on rank 0 and 1,3 on rank 1) reproduces the single-process
    curve of the same 4-layer model; so does pp=2 x ep=2 on four ranks, and evaluation goes through the same path."""
    four = BASE + ["num_layers=4"]
    (ref, _), = run_ranks(_train, 1, four + ["expert_model_parallel_size=1"], 5)
    res = run_ranks(_train, 2, four + ["expert_model_parallel_size=1", "pipeline_model_parallel_size=2",
                                       "virtual_pipeline_model_parallel_size=2"], 5)
    assert res[0][0] == pytest.approx(ref, rel=2e-5, abs=2e-5) and res[1][0] == res[0][0]
    res4 = run_ranks(_train, 4, four + ["expert_model_parallel_size=2", "pipeline_model_parallel_size=2",
                                        "virtual_pipeline_model_parallel_size=2", "recompute_granularity=selective"], 5)
    assert res4[0][0] == pytest.approx(ref, rel=2e-5, abs=2e-5)


def test_interleaved_needs_microbatches_multiple_of_pp():
    from system_lab_b200.config import Config, ConfigError
    cfg = Config.load(preset="simplemoe-tiny", overrides=["num_layers=4", "global_batch_size=2", "micro_batch_size=2",
                                                          "pipeline_model_parallel_size=2", "expert_model_parallel_size=1",
                                                          "virtual_pipeline_model_parallel_size=2"])
    with pytest.raises(ConfigError, match="multiple of pp"):
        cfg.validate(2)


def _ckpt_corruption(rank, world, root, phase):
    from system_lab_b200.ckpt.sharded import CheckpointCorrupt
    from system_lab_b200.config import Config
    from system_lab_b200.trainer.loop import Trainer
    cfg = Config.load(preset="simplemoe-tiny", overrides=BASE + [f"expert_model_parallel_size={world}", "device=cpu",
                                                                f"save={root}", "keep_last=3"])
    tr = Trainer(cfg)
    if phase == "write":
        for _ in range(2):
            tr.train_step()
        tr.save_checkpoint(root)
        w2 = float(torch.cat([g.shard.float().reshape(-1)[:64] for g in tr.engine.all_groups()]).double().sum())
        for _ in range(2):
            tr.train_step()
        tr.save_checkpoint(root)
        return w2
    try:
        tr.load_checkpoint(root)
    except CheckpointCorrupt as e:
        return ("corrupt", str(e)[:80])
    w = float(torch.cat([g.shard.float().reshape(-1)[:64] for g in tr.engine.all_groups()]).double().sum())
    return (tr.step, w)


def test_corrupt_checkpoint_shard_is_detected_and_every_rank_falls_back_together(tmp_path):
    """Host-side fault: one rank's file of the newest checkpoint is damaged.  Only that rank can see it, yet both
    ranks must reject the step and load the previous one; with no older checkpoint the load fails with a typed error."""
    import pathlib
    root = str(tmp_path / "ck")
    w2 = run_ranks(_ckpt_corruption, 2, root, "write")
    newest = pathlib.Path(root) / "step_000004"
    assert (newest / "rank_00001.sha256").exists()
    clean = run_ranks(_ckpt_corruption, 2, root, "load")
    assert [c[0] for c in clean] == [4, 4]
    victim = newest / "rank_00001.pt"
    data = bytearray(victim.read_bytes())
    data[len(data) // 2] ^= 0xFF
    victim.write_bytes(bytes(data))
    res = run_ranks(_ckpt_corruption, 2, root, "load")
    assert [r[0] for r in res] == [2, 2]                              # both ranks fell back to step 2
    assert res[0][1] == pytest.approx(w2[0], rel=1e-12) and res[1][1] == pytest.approx(w2[1], rel=1e-12)
    (pathlib.Path(root) / "step_000002" / "rank_00000.pt").write_bytes(b"not a checkpoint")
    res = run_ranks(_ckpt_corruption, 2, root, "load")
    assert [r[0] for r in res] == ["corrupt", "corrupt"]


def test_hybrid_sharding_matches_and_checkpoints(single_curve, tmp_path):
    """Two optimizer instances on four data ranks: parameters sharded over blocks of two ranks, gradients
    reduce-scattered inside a block and all-reduced across the blocks.  Same curve as one process (clipping on, so
    the gradient norm must not double-count replicas), and a checkpoint written under it reloads on one rank."""
    ov = BASE + ["expert_model_parallel_size=2", "num_distributed_optimizer_instances=2", "global_batch_size=8",
                 "micro_batch_size=1"]
    ck = str(tmp_path / "ck")
    res = run_ranks(_train, 4, ov, 3, ck, None, 3)
    for losses, _ in res:
        assert losses == pytest.approx(single_curve, rel=2e-5, abs=2e-5)
    resumed = run_ranks(_train, 1, BASE + ["expert_model_parallel_size=1"], 3, None, ck)
    assert resumed[0][0] == pytest.approx(single_curve[3:], rel=2e-5, abs=2e-5)


def _layout(rank, world, overrides):
    import torch.distributed as dist
    from system_lab_b200.config import Config
    from system_lab_b200.trainer.loop import Trainer
    tr = Trainer(Config.load(preset="simplemoe-tiny", overrides=list(overrides) + ["device=cpu"]))
    out = {}
    for g in tr.engine.all_groups():
        kind = g.name.rsplit("/", 1)[1]
        out[kind] = (g.world, dist.get_world_size(g.replica_group) if g.replica_group is not None else 1)
    return out


def test_hybrid_sharding_layout():
    res = run_ranks(_layout, 4, BASE + ["expert_model_parallel_size=1", "num_distributed_optimizer_instances=2"])
    assert all(r == {"dense": (2, 2), "expert": (2, 2)} for r in res), res
    res = run_ranks(_layout, 4, BASE + ["expert_model_parallel_size=2", "num_distributed_optimizer_instances=2"])
    assert all(r == {"dense": (2, 2), "expert": (1, 2)} for r in res), res


def test_tensor_parallel_matches(single_curve):
    """Heads split over two ranks; the MoE block takes half of the tokens on each and exchanges them over an
    expert-parallel group that spans the tensor-parallel ranks."""
    res = run_ranks(_train, 2, BASE + ["expert_model_parallel_size=2", "tensor_model_parallel_size=2"], 6)
    for losses, _ in res:
        assert losses == pytest.approx(single_curve, rel=2e-5, abs=2e-5)


def test_sequence_parallel_matches(single_curve):
    """Residual stream, norms and MoE blocks on half of every sequence per rank; all-gather in front of the
    column-split matrices, reduce-scatter behind the row-split ones; norm gains, embedding and head sum their partial
    gradients over the group; the loss is the mean of the two ranks' means."""
    res = run_ranks(_train, 2, BASE + ["expert_model_parallel_size=2", "tensor_model_parallel_size=2",
                                       "sequence_parallel=true"], 6)
    for losses, _ in res:
        assert losses == pytest.approx(single_curve, rel=2e-5, abs=2e-5)


def test_sequence_parallel_with_pipeline_and_selective_recompute(single_curve):
    """Stages exchange [B, S / tp, H] activations."""
    ov = BASE + ["expert_model_parallel_size=2", "tensor_model_parallel_size=2", "sequence_parallel=true",
                 "pipeline_model_parallel_size=2", "recompute_granularity=selective"]
    res = run_ranks(_train, 4, ov, 4)
    assert res[-1][0] == pytest.approx(single_curve[:4], rel=2e-5, abs=2e-5)


def test_expert_tensor_parallel_matches(single_curve, tmp_path):
    """Every tensor-parallel rank routes all tokens and holds half of each expert's feed-forward columns; the expert
    axis runs over the data ranks inside each tensor-parallel plane; partial outputs are summed over the group.
    Plain, with sequence parallelism, and resumed from a checkpoint."""
    etp = ["tensor_model_parallel_size=2", "expert_tensor_parallel_size=2"]
    res = run_ranks(_train, 2, BASE + ["expert_model_parallel_size=1"] + etp, 6)
    for losses, _ in res:
        assert losses == pytest.approx(single_curve, rel=2e-5, abs=2e-5)
    ov = BASE + ["expert_model_parallel_size=2", "sequence_parallel=true"] + etp
    ck = str(tmp_path / "ck")
    full = run_ranks(_train, 4, ov, 3, ck, None, 3)
    assert full[0][0] == pytest.approx(single_curve, rel=2e-5, abs=2e-5)
    resumed = run_ranks(_train, 4, ov, 3, None, ck)
    assert resumed[0][0] == full[0][0][3:]


def test_tensor_parallel_with_data_parallel_selective_and_resume(single_curve, tmp_path):
    ov = BASE + ["expert_model_parallel_size=4", "tensor_model_parallel_size=2", "recompute_granularity=selective"]
    ck = str(tmp_path / "ck")
    full = run_ranks(_train, 4, ov, 3, ck, None, 3)
    assert full[0][0] == pytest.approx(single_curve, rel=2e-5, abs=2e-5)
    resumed = run_ranks(_train, 4, ov, 3, None, ck)
    assert resumed[0][0] == full[0][0][3:]
    assert [r[1] for r in resumed] == [r[1] for r in full]
    with pytest.raises(Exception, match="tensor_model_parallel_size"):
        run_ranks(_train, 1, BASE + ["expert_model_parallel_size=1"], 1, None, ck)


def _fit(rank, world, overrides):
    import gc
    from system_lab_b200.config import Config
    from system_lab_b200.trainer.loop import Trainer
    tr = Trainer(Config.load(preset="simplemoe-tiny", overrides=list(overrides) + ["device=cpu"]))
    tr.fit()
    return tr.step, tr.stopped_on_time, gc.isenabled()


def _fit_curve(rank, world, overrides):
    from system_lab_b200.config import Config
    from system_lab_b200.trainer.loop import Trainer
    tr = Trainer(Config.load(preset="simplemoe-tiny", overrides=list(overrides) + ["device=cpu"]))
    tr.fit()
    return tr.loss_curve, tr.eval_curve, tr.step, len(tr.step_times_ms)


def test_deferred_loss_read_gives_the_same_run(tmp_path):
    """``fit`` with the numbers of a step read after the next step's launch: same loss curve, one entry per step,
    evaluation and checkpoints at the same steps as the run that reads at once."""
    ov = BASE + ["expert_model_parallel_size=2", "train_iters=7", "eval_interval=3", "eval_iters=1", "log_interval=2"]
    sync = run_ranks(_fit_curve, 2, ov + [f"save={tmp_path / 'a'}", "save_interval=4"])
    late = run_ranks(_fit_curve, 2, ov + [f"save={tmp_path / 'b'}", "save_interval=4", "deferred_loss_read=true"])
    assert late[0][0] == sync[0][0] and len(late[0][0]) == 7
    assert late[0][1] == sync[0][1] and late[0][2] == 7 and late[0][3] == 7
    assert sorted(p.name for p in (tmp_path / "a").iterdir()) == sorted(p.name for p in (tmp_path / "b").iterdir())


def test_wall_clock_exit_is_collective_and_manual_gc_restores_the_collector():
    """Rank 0 decides that the time is up and every rank leaves after the same step; manual garbage collection runs
    with the collector off and turns it back on."""
    ov = BASE + ["expert_model_parallel_size=2", "train_iters=50", "exit_duration_in_mins=0.0005", "manual_gc=true",
                 "manual_gc_interval=1", "log_interval=100"]
    res = run_ranks(_fit, 2, ov)
    steps = {r[0] for r in res}
    assert len(steps) == 1 and 1 <= steps.pop() < 50
    assert all(r[1] and r[2] for r in res)


def _fit_with_sigterm(rank, world, overrides, save):
    import os
    import signal
    from system_lab_b200.config import Config
    from system_lab_b200.trainer.loop import Trainer
    tr = Trainer(Config.load(preset="simplemoe-tiny", overrides=list(overrides) + ["device=cpu", f"save={save}"]))
    if rank == 1:                      # the scheduler's preemption notice reaches one rank only
        orig = tr.train_step

        def step_then_signal(*a, **k):
            out = orig(*a, **k)
            if tr.step == 2:
                os.kill(os.getpid(), signal.SIGTERM)
            return out
        tr.train_step = step_then_signal
    tr.fit()
    return tr.step, tr.stopped_on_signal


def test_sigterm_on_one_rank_makes_every_rank_save_and_leave(tmp_path):
    from system_lab_b200.launch import newest_checkpoint
    ov = BASE + ["expert_model_parallel_size=2", "train_iters=30", "exit_signal_handler=true", "log_interval=100"]
    res = run_ranks(_fit_with_sigterm, 2, ov, str(tmp_path / "ck"))
    assert [r[0] for r in res] == [2, 2] and all(r[1] for r in res)
    assert newest_checkpoint(str(tmp_path / "ck")).endswith("step_000002")


def _fit_async(rank, world, overrides, save, load=None):
    from system_lab_b200.config import Config
    from system_lab_b200.trainer.loop import Trainer
    tr = Trainer(Config.load(preset="simplemoe-tiny", overrides=list(overrides) + ["device=cpu", f"save={save}"]))
    if load:
        tr.load_checkpoint(load)
    tr.fit(max(tr.cfg.train.train_iters - tr.step, 0))
    return tr.loss_curve, getattr(tr, "_pending_ckpt", None) is None


def test_async_checkpoint_is_published_later_and_resumes_bit_exactly(tmp_path):
    from pathlib import Path
    ov = BASE + ["expert_model_parallel_size=2", "train_iters=5", "save_interval=2", "log_interval=100", "keep_last=5"]
    sync = run_ranks(_fit_async, 2, ov, str(tmp_path / "sync"))
    asyn = run_ranks(_fit_async, 2, ov + ["async_save=true"], str(tmp_path / "async"))
    assert asyn[0][0] == sync[0][0] and all(r[1] for r in asyn)          # same training, nothing left pending
    names = sorted(p.name for p in Path(tmp_path / "async").glob("step_*"))
    assert names == ["step_000002", "step_000004", "step_000005"]
    assert not list(Path(tmp_path / "async").glob(".tmp_step_*"))
    # resume from the asynchronously written step 4 and reproduce step 5
    res = run_ranks(_fit_async, 2, ov, str(tmp_path / "resumed"), str(tmp_path / "async" / "step_000004"))
    assert res[0][0][-1] == sync[0][0][-1]


def test_checkpoint_cli_inspect_verify_consolidate(tmp_path, capsys):
    """Offline tools: the consolidated tensors of a checkpoint written by two ranks (experts split) equal those of a
    checkpoint written by one rank after the same training; a damaged rank file fails `verify`."""
    import json
    from system_lab_b200.ckpt.__main__ import main as ckpt_cli
    two, one = str(tmp_path / "two"), str(tmp_path / "one")
    run_ranks(_train, 2, BASE + ["expert_model_parallel_size=2"], 2, two)
    run_ranks(_train, 1, BASE + ["expert_model_parallel_size=1"], 2, one)
    assert ckpt_cli(["verify", two]) == 0
    capsys.readouterr()
    assert ckpt_cli(["inspect", two, "--json"]) == 0
    info = json.loads(capsys.readouterr().out)
    assert info["step"] == 2 and info["world"] == 2 and info["parameters"] == 17
    assert all(t["covered"] >= t["elements"] for t in info["tensors"])
    assert ckpt_cli(["consolidate", two, "--out", str(tmp_path / "a.pt")]) == 0
    assert ckpt_cli(["consolidate", one, "--out", str(tmp_path / "b.pt")]) == 0
    a, b = torch.load(tmp_path / "a.pt"), torch.load(tmp_path / "b.pt")
    assert a.keys() == b.keys() and a["layers.0.ffn.experts_w1"].shape == (8, 1024, 256)
    for k in a:
        torch.testing.assert_close(a[k], b[k], rtol=1e-3, atol=2e-5)      # two layouts, two summation orders
    victim = next((tmp_path / "two").glob("step_*/rank_00001.pt"))
    victim.write_bytes(victim.read_bytes()[:-100])
    assert ckpt_cli(["verify", two]) == 1


def test_norm_gains_are_excluded_from_weight_decay():
    """1-D parameters sit at the tail of their flat group and get no weight decay: with a zero learning-rate effect
    removed (huge eps kills the Adam term) a matrix shrinks by (1 - lr * wd) per step and a norm gain does not move."""
    import torch
    from system_lab_b200.config import Config
    from system_lab_b200.trainer.loop import Trainer
    cfg = Config.load(preset="simplemoe-tiny", overrides=[
        "global_batch_size=4", "micro_batch_size=4", "expert_model_parallel_size=1", "device=cpu", "lr=0.1",
        "weight_decay=0.5", "adam_eps=1e30", "clip_grad=0.0"])
    tr = Trainer(cfg)
    layer = tr.engine.model.layers[0]
    g0, w0 = layer.attn_norm.weight.detach().clone(), layer.attn.wqkv.detach().clone()
    for grp in tr.engine.all_groups():
        assert all(p.dim() > 1 for p, o in zip(grp.params, grp.offsets) if o < grp.decay_numel)
        assert all(p.dim() <= 1 for p, o in zip(grp.params, grp.offsets) if o >= grp.decay_numel)
    tr.train_step()
    assert torch.allclose(layer.attn_norm.weight, g0, atol=1e-6)
    assert torch.allclose(layer.attn.wqkv, w0 * (1 - 0.1 * 0.5), rtol=1e-5, atol=1e-7)
