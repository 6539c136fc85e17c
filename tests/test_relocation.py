"""Load-adaptive expert placement: the planner, the exchange of expert rows between ranks, and invariance of training
under relocation (CPU, gloo)."""
import random

import pytest
import torch

from distutil import run_ranks


def test_planner_balances_and_is_stable():
    from system_lab_b200.moe.relocation import imbalance, plan_placement
    random.seed(0)
    e, ep = 32, 4
    load = [1000.0 / (i + 1) ** 1.1 for i in range(e)]           # Zipf: the hot experts start on rank 0
    ident = list(range(e))
    before = imbalance(load, ident, ep)
    new = plan_placement(load, ep, ident)
    after = imbalance(load, new, ep)
    assert sorted(new) == ident                                   # a permutation of the slots
    assert all(sum(1 for s in new if s // 8 == r) == 8 for r in range(ep))
    assert before > 2.0 and after < 1.35 and after < before
    assert plan_placement(load, ep, new) == new                   # deciding again moves nothing
    flat = plan_placement([1.0] * e, ep, ident)
    assert imbalance([1.0] * e, flat, ep) == 1.0


def _exchange(rank, world):
    import torch.distributed as dist
    from system_lab_b200.moe.relocation import _exchange_rows
    from system_lab_b200.parallel.mesh import init_distributed
    init_distributed("cpu")
    e_local, e = 4, 4 * world
    g = torch.Generator().manual_seed(1)
    perm = torch.randperm(e, generator=g).tolist()               # slot a -> slot perm[a]
    moves = [(a, b) for a, b in enumerate(perm) if a != b]
    out = {}
    for dt in (torch.float32, torch.bfloat16, torch.uint8):
        glob = (torch.arange(e * 6).reshape(e, 6) % 251).to(dt)  # row a holds a recognisable pattern
        mine = glob[rank * e_local:(rank + 1) * e_local].clone()
        _exchange_rows(mine, moves, world, rank, e_local, dist.group.WORLD if world > 1 else None)
        want = glob.clone()
        for a, b in enumerate(perm):
            want[b] = glob[a]
        out[str(dt)] = bool(torch.equal(mine, want[rank * e_local:(rank + 1) * e_local]))
    return out


@pytest.mark.parametrize("world", [1, 2, 4])
def test_rows_arrive_where_the_moves_say(world):
    for res in run_ranks(_exchange, world):
        assert all(res.values()), res


def _train(rank, world, extra, iters, force_perm):
    from system_lab_b200.config import Config
    from system_lab_b200.moe.relocation import relocate_ffn
    from system_lab_b200.trainer.loop import Trainer
    cfg = Config.load(preset="simplemoe-tiny", overrides=[
        "global_batch_size=8", "micro_batch_size=2", f"expert_model_parallel_size={world}"] + extra)
    tr = Trainer(cfg)
    losses = []
    for i in range(iters):
        if force_perm and i == 2:
            # a fixed non-trivial permutation of every layer's experts, applied between two steps
            for li, (ffn, grp) in enumerate(zip(tr.engine.moe_ffns(), [g for u in tr.engine.layer_units for g in u.groups
                                                                      if g.name.endswith("/expert")])):
                e = ffn.expert_map.numel()
                perm = torch.randperm(e, generator=torch.Generator().manual_seed(7 + li)).tolist()
                relocate_ffn(ffn, grp, tr.optimizer, perm, tr.mesh.ep, tr.mesh.ep_rank,
                             tr.mesh.ep_group if tr.mesh.ep > 1 else None)
        losses.append(float(tr.train_step()["loss"]))
    hist = tr.relocator.history if tr.relocator else []
    return losses, hist, tr.rank_load_ratio()


@pytest.mark.parametrize("state", ["fp32", "fp8"])
def test_training_is_invariant_under_a_forced_relocation(state):
    """Moving experts (weights, master, moments, 8-bit block scales) between ranks changes where they are computed,
    not what is computed."""
    ov = [f"optimizer_state_dtype={state}"]
    base = run_ranks(_train, 2, ov, 6, False, timeout=400)[0][0]
    moved = run_ranks(_train, 2, ov, 6, True, timeout=400)
    assert moved[0][0] == pytest.approx(base, rel=3e-5, abs=3e-5)
    assert moved[1][0] == moved[0][0]


def test_relocation_interval_runs_and_reports():
    res = run_ranks(_train, 2, ["moe_expert_relocation_interval=2", "moe_expert_relocation_min_gain=0.0"], 6, False,
                    timeout=400)
    losses, hist, ratio = res[0]
    assert [h["step"] for h in hist] == [2, 4, 6]
    assert all(h["imbalance_after_predicted"] <= h["imbalance_before"] + 1e-9 for h in hist)
    assert ratio is not None and ratio >= 1.0
    base = run_ranks(_train, 2, [], 6, False, timeout=400)[0][0]
    assert losses == pytest.approx(base, rel=3e-5, abs=3e-5)
    early = run_ranks(_train, 2, ["moe_expert_relocation_interval=100", "moe_expert_relocation_first_step=3"], 5, False,
                      timeout=400)[0][1]
    assert [h["step"] for h in early] == [3]
    # automatic mode: on (once at step 3, then every 50) where experts can move, off on a single rank
    auto = run_ranks(_train, 2, ["moe_expert_relocation_interval=-1"], 4, False, timeout=400)[0][1]
    assert [h["step"] for h in auto] == [3]
    assert run_ranks(_train, 1, ["moe_expert_relocation_interval=-1"], 3, False, timeout=400)[0][1] == []
