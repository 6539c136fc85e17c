"""Failure detection without touching a GPU: host-side fault injection, the rank heartbeat watchdog on gloo ranks,
and the job runner's hang / numerical / crash classification of real child processes."""
import time

import pytest

from distutil import run_ranks


def test_fault_plan_parsing_and_actions():
    from system_lab_b200.trainer.watchdog import FaultPlan, InjectedFault
    p = FaultPlan.parse("delay:rank=1,step=3,seconds=0.05; nan:rank=0,step=4;mute:rank=1,step=2;raise:rank=0,step=9")
    assert [a["kind"] for a in p.actions] == ["delay", "nan", "mute", "raise"]
    assert p.before_step(0, 1) == {}
    t0 = time.time()
    assert p.before_step(1, 3) == {} and time.time() - t0 >= 0.05
    assert p.before_step(0, 4) == {"nan": True} and p.before_step(1, 2) == {"mute": True}
    with pytest.raises(InjectedFault):
        p.before_step(0, 9)
    with pytest.raises(ValueError):
        FaultPlan.parse("explode:rank=0")
    assert FaultPlan.parse("").actions == []


def _train_with_faults(rank, world, faults, iters, timeout_s):
    from system_lab_b200.config import Config
    from system_lab_b200.trainer.loop import Trainer
    from system_lab_b200.trainer.watchdog import PeerFailure
    cfg = Config.load(preset="simplemoe-tiny", overrides=[
        "global_batch_size=4", "micro_batch_size=2", f"expert_model_parallel_size={world}",
        f"hang_timeout_s={timeout_s}", f"fault_injection={faults}"])
    tr = Trainer(cfg)
    tr.heartbeat.poll_s = 0.05
    try:
        for _ in range(iters):
            float(tr.train_step()["loss"])
    except PeerFailure as e:
        return ("peer_failure", e.kind, e.rank, tr.step)
    except Exception as e:                       # the delayed rank loses its peer: whatever gloo raises is fine
        return ("error", type(e).__name__, -1, tr.step)
    finally:
        tr.heartbeat.stop()
    return ("done", "", -1, tr.step)


def test_delayed_rank_is_reported_by_the_watchdog_before_the_next_launch():
    """Rank 1 sleeps 4 s before step 3 with a 1 s hang limit: rank 0 waits for it inside step 3's collectives, its
    watchdog sees rank 1 stuck behind, and rank 0 raises HANG for rank 1 at the start of step 4 (between steps,
    nothing in flight)."""
    res = run_ranks(_train_with_faults, 2, "delay:rank=1,step=3,seconds=4", 6, 1.0, timeout=120)
    assert res[0][:3] == ("peer_failure", "HANG", 1)
    assert res[0][3] == 3                         # rank 0 finished step 3 and stopped before launching step 4
    assert res[1][0] in ("error", "done", "peer_failure")


def test_muted_heartbeat_is_a_hang_even_if_the_rank_keeps_stepping():
    res = run_ranks(_train_with_faults, 2, "mute:rank=1,step=2", 40, 0.6, timeout=120)
    assert res[0][:3] == ("peer_failure", "HANG", 1)


def test_healthy_run_raises_nothing():
    res = run_ranks(_train_with_faults, 2, "", 5, 5.0, timeout=120)
    assert [r[0] for r in res] == ["done", "done"] and res[0][3] == 5


def _runner(tmp_path, faults):
    from system_lab_b200.pilot.runner import JobRunner
    return JobRunner(tmp_path / "jobs", "simplemoe-tiny", base_overrides=[f"fault_injection={faults}"], nproc=1,
                     device="cpu")


def _plan():
    from system_lab_b200.pilot import policy
    p = policy.default_plan(1, mbs=2, gbs=4)
    p["comm"]["dispatcher"] = "alltoall"
    return p


def test_runner_kills_a_silent_job_and_reports_hang(tmp_path):
    r = _runner(tmp_path, "delay:rank=0,step=3,seconds=120")
    job = r.submit(_plan(), 6)
    t0 = time.time()
    snap = r.wait(job, hang_timeout_s=4.0, poll_s=0.2)
    assert time.time() - t0 < 60
    assert snap["status"] == "hung" and snap["failure_kind"] == "HANG" and snap["early_stop_reason"] == "hang_5min"
    assert r.procs[job].poll() is not None        # the child (its own process group) is gone


def test_runner_classifies_numerical_and_crash(tmp_path):
    r = _runner(tmp_path, "nan:rank=0,step=2")
    snap = r.wait(r.submit(_plan(), 4), hang_timeout_s=60)
    assert snap["status"] == "failed" and snap["failure_kind"] == "NUMERICAL"
    r2 = _runner(tmp_path / "b", "exit:rank=0,step=2,code=17")
    snap2 = r2.wait(r2.submit(_plan(), 4), hang_timeout_s=60)
    assert snap2["status"] == "failed" and snap2["exit_code"] == 17
    r3 = _runner(tmp_path / "c", "")
    snap3 = r3.wait(r3.submit(_plan(), 3), hang_timeout_s=60)
    assert snap3["status"] == "ok" and snap3["metrics"]["tps"] > 0


def test_fit_stops_on_a_device_status_code_before_it_checkpoints(tmp_path):
    """A kernel that gave up (bounded wait, bounds check, capacity) leaves a code in the status word; ``fit`` reads it
    right after the step's loss and raises before the step is logged or saved."""
    import torch
    from system_lab_b200.config import Config
    from system_lab_b200.ops import cuda as cops
    from system_lab_b200.trainer.loop import Trainer
    cfg = Config.load(preset="simplemoe-tiny", overrides=[
        "global_batch_size=4", "micro_batch_size=2", "expert_model_parallel_size=1", "train_iters=4",
        f"save={tmp_path / 'ck'}", "save_interval=1"])
    tr = Trainer(cfg)
    tr.fit(1)                                                    # a healthy step saves its checkpoint
    saved = sorted(p.name for p in (tmp_path / "ck").iterdir())
    word = cops.status_word(tr.device)
    word.fill_(5)                                                # what a timed-out peer-flag wait writes
    try:
        with pytest.raises(cops.DeviceHang, match="TIMEOUT_PEER_FLAG"):
            tr.fit(1)
        assert sorted(p.name for p in (tmp_path / "ck").iterdir()) == saved     # nothing written after the failure
        assert int(word.item()) == 0                             # consumed: a restarted loop starts clean
    finally:
        word.zero_()
        tr.close()


def _fit_with_status_on_one_rank(rank, world):
    import torch
    from system_lab_b200.config import Config
    from system_lab_b200.ops import cuda as cops
    from system_lab_b200.trainer.loop import Trainer
    cfg = Config.load(preset="simplemoe-tiny", overrides=[
        "global_batch_size=4", "micro_batch_size=2", f"expert_model_parallel_size={world}", "train_iters=3"])
    tr = Trainer(cfg)
    if rank == 1:
        cops.status_word(tr.device).fill_(7)                     # only rank 1's kernels overflowed a buffer
    try:
        tr.fit(2)
    except cops.DeviceHang as e:
        return ("hang", str(e), tr.step)
    finally:
        cops.status_word(tr.device).zero_()
        tr.close()
    return ("done", "", tr.step)


def test_every_rank_leaves_the_step_when_one_rank_reports_a_status_code():
    res = run_ranks(_fit_with_status_on_one_rank, 2, timeout=120)
    assert [r[0] for r in res] == ["hang", "hang"]
    assert all("CAPACITY" in r[1] and r[2] == 1 for r in res)


def test_deferred_loss_read_still_stops_on_a_non_finite_loss():
    """With the numbers of a step read one step late, a NaN injected at step 3 (on the host) stops ``fit`` when step 3
    is accounted for, i.e. after step 4 has been launched: the error names step 3 and the curve ends there."""
    import pytest
    from system_lab_b200.config import Config
    from system_lab_b200.trainer.loop import NumericalError, Trainer
    cfg = Config.load(preset="simplemoe-tiny", overrides=[
        "global_batch_size=4", "micro_batch_size=2", "expert_model_parallel_size=1", "train_iters=8", "device=cpu",
        "deferred_loss_read=true", "fault_injection=nan:rank=0,step=3"])
    tr = Trainer(cfg)
    with pytest.raises(NumericalError, match="step 3"):
        tr.fit()
    assert len(tr.loss_curve) == 3 and tr.loss_curve[2] != tr.loss_curve[2] and tr.step == 4
    tr.close()
