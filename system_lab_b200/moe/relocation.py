"""Load-adaptive expert placement: move hot experts apart so that expert-parallel ranks carry equal loads.

With expert parallelism the most loaded rank of every layer sets the pace of that layer (its expert GEMMs finish
last, its NVLink ingress is the busiest, everyone else waits in combine).  Which experts are hot is stable over
hundreds of steps, so the placement can follow the load: every ``interval`` steps the trainer takes the tokens
each expert received since the last decision, assigns experts to ranks with a longest-processing-time-first
greedy (each rank keeps exactly ``E / ep`` slots) and, if the predicted max/mean rank load improves enough, moves
the experts: parameters, master weights and both Adam moments travel together through one all-to-all per tensor.
The router and the model's math do not change: a per-layer table maps the router's (logical) expert id to the
physical slot ``rank * E_local + local index`` that currently holds it.

Reference: the load-adaptive re-layout of LAER-MoE (planner every K steps, ``moe/LAER_MoE_FSEP_reading_notes.md:
405-627``) listed as the optional load-balance feature, and the EP retune rule of the tuner's MoE skill
(``skills/pilot/optimization/moe/SKILL.md:63-72``), which this makes unnecessary for pure placement skew.

Scope: expert groups that are not sharded or replicated any further (``ep == dp`` on the stage and ``cp == 1``).
"""
from __future__ import annotations

import torch
import torch.distributed as dist


def rank_loads(load, phys_of_logical, ep: int):
    """Per-rank load under a placement.  ``load[l]`` = tokens of logical expert ``l``."""
    e_local = len(load) // ep
    out = [0.0] * ep
    for l, w in enumerate(load):
        out[int(phys_of_logical[l]) // e_local] += float(w)
    return out


def imbalance(load, phys_of_logical, ep: int) -> float:
    r = rank_loads(load, phys_of_logical, ep)
    mean = sum(r) / max(len(r), 1)
    return max(r) / mean if mean > 0 else 1.0


def plan_placement(load, ep: int, current=None):
    """Longest-processing-time-first assignment of ``E`` experts to ``ep`` ranks with ``E / ep`` slots each.
    Returns ``phys_of_logical`` (list of ``E`` slot ids).  Experts that stay on their current rank keep their
    slot, so an unchanged decision moves nothing.  Deterministic: ties break on the expert id."""
    e = len(load)
    e_local = e // ep
    order = sorted(range(e), key=lambda l: (-float(load[l]), l))
    rank_load = [0.0] * ep
    members: list[list[int]] = [[] for _ in range(ep)]
    for l in order:
        r = min((rr for rr in range(ep) if len(members[rr]) < e_local), key=lambda rr: (rank_load[rr], rr))
        members[r].append(l)
        rank_load[r] += float(load[l])
    phys = [-1] * e
    for r in range(ep):
        free = set(range(r * e_local, (r + 1) * e_local))
        movers = []
        for l in members[r]:
            cur = int(current[l]) if current is not None else -1
            if cur in free:
                phys[l] = cur
                free.discard(cur)
            else:
                movers.append(l)
        for l, slot in zip(sorted(movers), sorted(free)):
            phys[l] = slot
    return phys


def _exchange_rows(t2d: torch.Tensor, moves, ep: int, me: int, e_local: int, group) -> None:
    """In place: row ``a % e_local`` of rank ``a // e_local`` goes to row ``b % e_local`` of rank ``b // e_local`` for
    every ``(a, b)`` in ``moves`` (global slot ids, the same list on every rank, ``a != b``)."""
    # rows travel as bytes: every backend moves uint8, and row indexing then works for every element type
    t2d = t2d.view(torch.uint8)
    mine_out = sorted((b // e_local, a % e_local, b) for a, b in moves if a // e_local == me)
    incoming = sorted((a // e_local, b // e_local, a % e_local, b) for a, b in moves if b // e_local == me)
    # arrival order from source s = s's send order to me = sorted by (dest rank, source local row)
    dst_rows = [b % e_local for _, _, _, b in incoming]
    if ep == 1 or group is None:
        src_rows = [al for _, al, _ in mine_out]
        data = t2d[src_rows].clone()
        # single rank: sends and arrivals are the same list in the same order
        t2d[[b % e_local for _, _, b in mine_out]] = data
        return
    send = t2d[[al for _, al, _ in mine_out]].contiguous() if mine_out else t2d[:0].contiguous()
    in_splits = [sum(1 for d, _, _ in mine_out if d == r) for r in range(ep)]
    out_splits = [sum(1 for s, _, _, _ in incoming if s == r) for r in range(ep)]
    recv = torch.empty((sum(out_splits),) + tuple(t2d.shape[1:]), dtype=t2d.dtype, device=t2d.device)
    dist.all_to_all_single(recv, send, out_splits, in_splits, group=group)
    if dst_rows:
        t2d[dst_rows] = recv


def relocate_ffn(ffn, group_obj, optimizer, new_phys_of_logical, ep: int, me: int, ep_group) -> int:
    """Move the experts of one MoE layer to ``new_phys_of_logical`` and update the layer's table.  ``group_obj`` is
    the layer's expert ``FlatGroup`` (unsharded), ``optimizer`` the ``ShardedAdamW`` that owns its state.
    Returns the number of experts moved (global)."""
    old = [int(x) for x in ffn.expert_map.tolist()]
    new = [int(x) for x in new_phys_of_logical]
    moves = [(a, b) for a, b in zip(old, new) if a != b]
    if not moves:
        return 0
    if group_obj.sharded or group_obj.replica_group is not None:
        raise RuntimeError("expert relocation needs expert groups that are neither sharded nor replicated (ep == dp, cp == 1)")
    e_local = ffn.e_local
    m, v = optimizer.m[group_obj.name], optimizer.v[group_obj.name]
    with torch.no_grad():
        for p, off, shape in zip(group_obj.params, group_obj.offsets, group_obj.shapes):
            if shape[0] != e_local:
                raise RuntimeError(f"expert tensor of shape {shape} does not lead with {e_local} experts")
            n = p.numel()
            per = n // e_local
            flats = [group_obj.full.data]
            if group_obj.shard is not group_obj.full:
                flats.append(group_obj.shard)
            flats += [m.data, v.data]
            for flat in flats:
                _exchange_rows(flat[off:off + n].view(e_local, per), moves, ep, me, e_local, ep_group)
            for mom in (m, v):
                if mom.kind == "fp8":                      # block scales (one per 128 elements) travel with their blocks
                    so, sn = off // 128, n // 128
                    _exchange_rows(mom.scale.reshape(-1)[so:so + sn].view(e_local, per // 128), moves, ep, me,
                                   e_local, ep_group)
        ffn.expert_map.copy_(torch.tensor(new, dtype=ffn.expert_map.dtype, device=ffn.expert_map.device))
        ffn.relocated = True
    return len(moves)


class ExpertRelocator:
    """Trainer-side driver: accumulates per-layer loads, decides and applies placements every ``interval`` steps."""

    def __init__(self, engine, optimizer, mesh, interval: int, min_gain: float = 0.05, first_step: int = 0):
        self.engine, self.optimizer, self.mesh = engine, optimizer, mesh
        self.interval, self.min_gain, self.first_step = interval, min_gain, first_step
        self.acc: torch.Tensor | None = None          # [layers, E] logical loads since the last decision
        self.history: list[dict] = []

    def observe(self, tpe_logical: torch.Tensor) -> None:
        self.acc = tpe_logical.clone() if self.acc is None else self.acc + tpe_logical

    def maybe_relocate(self, step: int) -> dict | None:
        due = (self.interval and step % self.interval == 0) or (self.first_step and step == self.first_step)
        if not due or self.acc is None:
            return None
        ffns = self.engine.moe_ffns()
        loads = self.acc.cpu().tolist()               # one host read per interval
        self.acc = None
        ep, me = self.mesh.ep, self.mesh.ep_rank
        moved, before, after = 0, [], []
        for ffn, unit_groups, load in zip(ffns, self._expert_groups(), loads):
            cur = ffn.expert_map.tolist()
            b = imbalance(load, cur, ep)
            new = plan_placement(load, ep, cur)
            a = imbalance(load, new, ep)
            before.append(b)
            if b - a >= self.min_gain * b:
                moved += relocate_ffn(ffn, unit_groups, self.optimizer, new, ep, me,
                                      self.mesh.ep_group if ep > 1 else None)
                after.append(a)
            else:
                after.append(b)
        rec = {"step": step, "experts_moved": moved, "imbalance_before": sum(before) / max(len(before), 1),
               "imbalance_after_predicted": sum(after) / max(len(after), 1)}
        self.history.append(rec)
        return rec

    def _expert_groups(self):
        out = []
        for u in self.engine.layer_units:
            if getattr(u.module, "is_moe", False):
                eg = [g for g in u.groups if g.name.endswith("/expert")]
                out.append(eg[0])
        return out
