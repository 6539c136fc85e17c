"""The single-node supervisor: a rank that exits mid-run (injected on the host) makes the job restart from the newest
checkpoint, on the same or a smaller number of CPU ranks, and the run ends where an undisturbed one does."""
import json
import sys
from pathlib import Path

from system_lab_b200.launch import Supervisor, newest_checkpoint

COMMON = ["--preset", "simplemoe-tiny", "device=cpu", "train_iters=8", "global_batch_size=8", "micro_batch_size=2",
          "expert_model_parallel_size=1", "save_interval=2", "log_interval=1"]


def _final(log: Path) -> dict:
    lines = [l for l in log.read_text().splitlines() if l.startswith("{") and "final_loss" in l]
    return json.loads(lines[-1])


def _run(tmp_path, name, extra, **kw):
    save = tmp_path / name / "ck"
    sup = Supervisor(2, COMMON + [f"save={save}"] + extra, log_dir=str(tmp_path / name / "logs"), grace_s=5.0,
                     python=sys.executable, **kw)
    return sup, sup.run(), save


def test_restart_from_newest_checkpoint_after_a_rank_exits(tmp_path):
    clean, rc, save0 = _run(tmp_path, "clean", [])
    assert rc == 0 and len(clean.history) == 1 and clean.history[0]["ok"]
    want = _final(tmp_path / "clean" / "logs" / "attempt0_rank0.log")
    assert want["steps"] == 8

    sup, rc, save = _run(tmp_path, "faulty", ["fault_injection=exit:rank=1,step=5"], max_restarts=2)
    assert rc == 0
    first, second = sup.history
    assert not first["ok"] and first["first_failed_rank"] == 1 and first["exit_code"] == 17
    assert second["ok"] and second["resumed_from"].endswith("step_000004") and second["world"] == 2
    got = _final(tmp_path / "faulty" / "logs" / "attempt1_rank0.log")
    assert got["steps"] == 8 and got["final_loss"] == want["final_loss"]          # bit-exact continuation
    assert newest_checkpoint(str(save)).endswith("step_000008")


def test_restart_on_fewer_ranks_reshards_the_checkpoint(tmp_path):
    sup, rc, save = _run(tmp_path, "shrink", ["fault_injection=raise:rank=0,step=4"], max_restarts=1, shrink=True)
    assert rc == 0
    first, second = sup.history
    assert not first["ok"] and second["ok"] and second["world"] == 1
    assert second["resumed_from"].endswith("step_000002")
    got = _final(tmp_path / "shrink" / "logs" / "attempt1_rank0.log")
    assert got["steps"] == 8 and abs(got["final_loss"] - 6.93) < 0.3


def test_gives_up_after_max_restarts(tmp_path):
    # no checkpoint directory: every attempt starts from scratch with the fault plan off after the first, so use a
    # configuration that fails on its own (an unknown key) to see the supervisor stop
    sup = Supervisor(1, ["--preset", "simplemoe-tiny", "device=cpu", "no_such_key=1"], max_restarts=1, grace_s=1.0)
    assert sup.run() == 1
    assert [h["ok"] for h in sup.history] == [False, False]
