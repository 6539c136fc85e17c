"""Token-file data, the evaluation loop and the stop-at-target rule (CPU)."""
import numpy as np
import pytest
import torch

from distutil import run_ranks


def _write(tmp_path, name="tokens.u16", n=20000, vocab=64, period=7):
    from system_lab_b200.trainer.data import write_token_file
    toks = (np.arange(n) % period) + 3            # a periodic stream: next token is predictable
    p = tmp_path / name
    write_token_file(p, toks)
    return str(p)


def test_token_file_batches_are_a_function_of_seed_and_step(tmp_path):
    from system_lab_b200.trainer.data import SyntheticData, TokenFileData, make_data
    path = _write(tmp_path)
    kw = dict(vocab_size=64, seq_length=16, global_batch_size=8, micro_batch_size=2, seed=5)
    one = TokenFileData(path, dp_rank=0, dp_size=1, **kw)
    a, b = one.global_batch(3), one.global_batch(3)
    assert torch.equal(a, b) and not torch.equal(a, one.global_batch(4)) and a.shape == (8, 17)
    assert torch.equal(a[:, 1:] - 3, (a[:, :-1] - 3 + 1) % 7)          # rows are contiguous windows of the stream
    # two data ranks see the two halves of the same global batch; targets are tokens shifted by one
    halves = [TokenFileData(path, dp_rank=r, dp_size=2, **kw).microbatches(3) for r in range(2)]
    got = torch.cat([torch.cat([t for t, _ in h]) for h in halves])
    assert torch.equal(got, a[:, :16])
    tok, tgt = halves[0][0]
    assert torch.equal(tgt[:, :-1], tok[:, 1:])
    assert isinstance(make_data("synthetic", dp_rank=0, dp_size=1, **kw), SyntheticData)
    assert isinstance(make_data(path, dp_rank=0, dp_size=1, **kw), TokenFileData)
    npy = _write(tmp_path, "t.npy")
    assert torch.equal(TokenFileData(npy, dp_rank=0, dp_size=1, **kw).global_batch(3), a)
    with pytest.raises(ValueError):
        TokenFileData(path, dp_rank=0, dp_size=1, **dict(kw, vocab_size=5)).global_batch(0)
    with pytest.raises(FileNotFoundError):
        make_data(str(tmp_path / "missing.bin"), dp_rank=0, dp_size=1, **kw)


def _fit(rank, world, path, extra):
    from system_lab_b200.config import Config
    from system_lab_b200.trainer.loop import Trainer
    cfg = Config.load(preset="simplemoe-tiny", overrides=[
        "vocab_size=64", "seq_length=32", "global_batch_size=8", "micro_batch_size=2", "train_iters=60", "lr=3e-3",
        f"data={path}", "eval_interval=5", "eval_iters=2", "log_interval=100"] + extra)
    tr = Trainer(cfg)
    first = tr.evaluate()
    again = tr.evaluate()
    tr.fit()
    return first, again, tr.step, tr.eval_curve, tr.reached_target


def test_eval_loss_falls_on_a_learnable_stream_and_training_stops_at_the_target(tmp_path):
    path = _write(tmp_path)
    (first, again, steps, curve, reached), = run_ranks(_fit, 1, path, ["expert_model_parallel_size=1",
                                                                       "eval_target_loss=0.2"], timeout=400)
    assert first == again                        # evaluation is repeatable and does not consume training data
    assert abs(first - np.log(64)) < 0.5         # untrained model: about log(vocab)
    assert reached and steps < 60 and steps % 5 == 0
    assert curve[-1][1] <= 0.2 < first and all(v > 0.2 for _, v in curve[:-1])


def test_eval_is_layout_invariant(tmp_path):
    path = _write(tmp_path)
    (one, _, _, c1, _), = run_ranks(_fit, 1, path, ["expert_model_parallel_size=1", "train_iters=5"], timeout=400)
    res = run_ranks(_fit, 2, path, ["expert_model_parallel_size=2", "train_iters=5"], timeout=400)
    assert res[0][0] == pytest.approx(one, rel=2e-5) and res[1][0] == res[0][0]
    assert res[0][3][0][1] == pytest.approx(c1[0][1], rel=1e-4)
    pp = run_ranks(_fit, 2, path, ["expert_model_parallel_size=1", "pipeline_model_parallel_size=2", "train_iters=5"],
                   timeout=400)
    assert pp[0][0] == pytest.approx(one, rel=2e-5) and pp[1][0] == pp[0][0]


def test_eval_through_interleaved_pipeline_stages(tmp_path):
    path = _write(tmp_path)
    four = ["num_layers=4", "train_iters=2"]
    (one, _, _, _, _), = run_ranks(_fit, 1, path, four + ["expert_model_parallel_size=1"], timeout=400)
    vp = run_ranks(_fit, 2, path, four + ["expert_model_parallel_size=1", "pipeline_model_parallel_size=2",
                                          "virtual_pipeline_model_parallel_size=2"], timeout=400)
    assert vp[0][0] == pytest.approx(one, rel=2e-5) and vp[1][0] == vp[0][0]
