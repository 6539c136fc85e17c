"""Device mesh: ``world = pp x dp x cp x tp`` with the expert-parallel group folded into ``dp x tp``.

Rank order (fastest varying last): ``rank = ((pp_rank * dp + dp_rank) * cp + cp_rank) * tp + tp_rank``.  The MoE
blocks see the tensor-parallel ranks as extra data ranks (each takes a slice of the tokens its tensor-parallel group
shares), so the expert axis runs over ``x = dp_rank * tp + tp_rank``: ``ep_rank = x % ep``, ``edp_rank = x // ep``
(the attention ``tp x cp x dp`` / MoE ``ep x edp`` folding of ``moe/MegatronCore_MoE_reading_notes.md:159-195``).
With ``tp == 1`` this is ``dp_rank = edp_rank * ep + ep_rank``.  Attention-side parameters are sharded over all ``dp * cp``
data ranks of a stage; expert parameters are owned by their ``ep`` rank and sharded over the
``edp`` ranks that hold the same experts — the dual dense/expert mesh of
``moe/MegatronCore_MoE_reading_notes.md:266-284`` and ``summary/torchtitan/*:98-113``.

On an NVSwitch box every pair of GPUs has the same bandwidth, so the mapping is chosen for simple
group arithmetic, not for locality.
"""
from __future__ import annotations

import datetime
import os
from dataclasses import dataclass

import torch
import torch.distributed as dist


@dataclass
class Mesh:
    world: int
    rank: int
    pp: int
    dp: int
    cp: int
    ep: int
    pp_rank: int
    dp_rank: int
    cp_rank: int
    ep_rank: int
    edp_rank: int
    data_group: object = None      # all dp*cp ranks of this stage (dense parameter shards, grad sync)
    dp_group: object = None        # dp ranks with the same cp rank
    ep_group: object = None        # expert all-to-all
    edp_group: object = None       # ranks holding the same experts (expert parameter shards)
    cp_group: object = None
    pp_group: object = None
    world_group: object = None
    tp: int = 1
    tp_rank: int = 0
    etp: int = 1                   # expert tensor parallelism: 1 (MoE blocks fold tp into their data axis) or tp
    tp_group: object = None        # ranks that split the heads / feed-forward columns of the same tokens
    stage_group: object = None     # every rank of this pipeline stage (equals data_group when tp == 1)
    data_ranks: tuple = ()
    ep_ranks: tuple = ()
    edp_ranks: tuple = ()
    pp_ranks: tuple = ()
    # one-directional channels for the interleaved pipeline schedule: "up" carries messages from a lower to a
    # higher stage index, "down" the rest, so two neighbours that both have a send at the head of their queues
    # (possible with the wrap-around link) never wait on each other within one communicator
    pp_group_up: object = None
    pp_group_down: object = None
    # hybrid sharding (``replicas`` > 1): parameters are sharded inside a block of ``data_size / replicas``
    # consecutive data ranks and replicated across the blocks; gradients are reduce-scattered inside the block and
    # all-reduced across the blocks.  The same split applies to the expert-data axis when it divides.
    replicas: int = 1
    data_shard_group: object = None
    data_shard_size: int = 0
    data_shard_rank: int = 0
    data_repl_group: object = None
    edp_shard_group: object = None
    edp_shard_size: int = 0
    edp_shard_rank: int = 0
    edp_repl_group: object = None
    edp_replicas: int = 1

    @property
    def edp(self) -> int:
        return (self.dp * self.tp // (self.ep * self.etp)) * self.cp

    @property
    def data_size(self) -> int:
        return self.dp * self.cp

    @property
    def data_rank(self) -> int:
        return self.dp_rank * self.cp + self.cp_rank

    def is_first_stage(self) -> bool:
        return self.pp_rank == 0

    def is_last_stage(self) -> bool:
        return self.pp_rank == self.pp - 1

    def prev_stage_rank(self) -> int:
        return self.pp_ranks[self.pp_rank - 1]

    def next_stage_rank(self) -> int:
        return self.pp_ranks[self.pp_rank + 1]


def single_process_mesh() -> Mesh:
    return Mesh(world=1, rank=0, pp=1, dp=1, cp=1, ep=1, pp_rank=0, dp_rank=0, cp_rank=0, ep_rank=0,
                edp_rank=0, data_ranks=(0,), ep_ranks=(0,), edp_ranks=(0,), pp_ranks=(0,))


def init_distributed(device: str = "auto", timeout_s: float = 600.0) -> tuple[int, int, torch.device]:
    """Join the job described by RANK / WORLD_SIZE / MASTER_* (torchrun).  NCCL on GPUs, gloo on CPU."""
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    use_cuda = (device == "cuda") or (device == "auto" and torch.cuda.is_available())
    if use_cuda:
        torch.cuda.set_device(local)
        dev = torch.device("cuda", local)
    else:
        dev = torch.device("cpu")
    if world > 1 and not dist.is_initialized():
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29500")
        kw = dict(device_id=dev) if use_cuda else {}
        dist.init_process_group("nccl" if use_cuda else "gloo", rank=rank, world_size=world,
                                timeout=datetime.timedelta(seconds=timeout_s), **kw)
    return rank, world, dev


def _hybrid_split(lists, replicas: int, rank: int):
    """Split every rank list into ``replicas`` consecutive blocks.  Returns, for this rank, ``(shard_group,
    shard_size, shard_rank, replica_group)``: its block, and the ranks at its position of every block.  Every rank
    creates every group, in the same order."""
    got = (None, 1, 0, None)
    for ranks in lists:
        size = len(ranks) // replicas
        blocks = [ranks[b * size:(b + 1) * size] for b in range(replicas)]
        shard_groups = [dist.new_group(b) if len(b) > 1 else None for b in blocks]
        repl_groups = [dist.new_group([b[i] for b in blocks]) for i in range(size)]
        if rank in ranks:
            at = ranks.index(rank)
            got = (shard_groups[at // size], size, at % size, repl_groups[at % size])
    return got


def build_mesh(pp: int = 1, ep: int = 1, cp: int = 1, replicas: int = 1, tp: int = 1, etp: int = 1) -> Mesh:
    if etp not in (1, tp):
        raise ValueError(f"expert tensor parallel size {etp}: use 1 or the tensor parallel size {tp}")
    if not dist.is_initialized():
        if pp * cp * tp != 1:
            raise ValueError("pp/cp/tp > 1 needs an initialised process group")
        return single_process_mesh()
    world, rank = dist.get_world_size(), dist.get_rank()
    if tp > 1:
        return _build_mesh_tp(pp, ep, cp, replicas, tp, etp)
    if world % (pp * cp):
        raise ValueError(f"world={world} not divisible by pp*cp={pp * cp}")
    dp = world // (pp * cp)
    ep = min(ep, dp)
    if dp % ep:
        raise ValueError(f"dp={dp} not divisible by ep={ep}")
    edp_n = dp // ep

    def rid(p, d, c):
        return (p * dp + d) * cp + c

    cp_rank = rank % cp
    dp_rank = (rank // cp) % dp
    pp_rank = rank // (cp * dp)
    ep_rank, edp_rank = dp_rank % ep, dp_rank // ep
    m = Mesh(world=world, rank=rank, pp=pp, dp=dp, cp=cp, ep=ep, pp_rank=pp_rank, dp_rank=dp_rank,
             cp_rank=cp_rank, ep_rank=ep_rank, edp_rank=edp_rank, world_group=dist.group.WORLD)

    # every rank must create every group, in the same order
    def mk(all_lists, mine_pred):
        got, got_ranks = None, ()
        for ranks in all_lists:
            g = dist.new_group(ranks) if len(ranks) > 1 else None
            if rank in ranks:
                got, got_ranks = g, tuple(ranks)
        return got, got_ranks

    data_lists = [[rid(p, d, c) for d in range(dp) for c in range(cp)] for p in range(pp)]
    m.data_group, m.data_ranks = mk(data_lists, None)
    dp_lists = [[rid(p, d, c) for d in range(dp)] for p in range(pp) for c in range(cp)]
    m.dp_group, _ = mk(dp_lists, None)
    ep_lists = [[rid(p, g * ep + e, c) for e in range(ep)] for p in range(pp) for g in range(edp_n) for c in range(cp)]
    m.ep_group, m.ep_ranks = mk(ep_lists, None)
    edp_lists = [[rid(p, g * ep + e, c) for g in range(edp_n) for c in range(cp)] for p in range(pp) for e in range(ep)]
    m.edp_group, m.edp_ranks = mk(edp_lists, None)
    cp_lists = [[rid(p, d, c) for c in range(cp)] for p in range(pp) for d in range(dp)]
    m.cp_group, _ = mk(cp_lists, None)
    pp_lists = [[rid(p, d, c) for p in range(pp)] for d in range(dp) for c in range(cp)]
    m.pp_group, m.pp_ranks = mk(pp_lists, None)
    m.pp_group_up, _ = mk(pp_lists, None)
    m.pp_group_down, _ = mk(pp_lists, None)
    m.stage_group = m.data_group
    if replicas > 1:
        if (dp * cp) % replicas:
            raise ValueError(f"data ranks per stage ({dp * cp}) not divisible by {replicas} optimizer instances")
        m.replicas = replicas
        m.data_shard_group, m.data_shard_size, m.data_shard_rank, m.data_repl_group = _hybrid_split(
            data_lists, replicas, rank)
        edp_total = edp_n * cp
        if edp_total > 1 and edp_total % replicas == 0:
            m.edp_replicas = replicas
            m.edp_shard_group, m.edp_shard_size, m.edp_shard_rank, m.edp_repl_group = _hybrid_split(
                edp_lists, replicas, rank)
    return m


def _build_mesh_tp(pp: int, ep: int, cp: int, replicas: int, tp: int, etp: int = 1) -> Mesh:
    """The mesh with a tensor-parallel axis (kept apart so that the ``tp == 1`` construction, and the order in which
    it creates its communicators, stays exactly as it was).

    ``etp == 1``: the MoE blocks treat the tensor-parallel ranks as data ranks (each takes ``1 / tp`` of the tokens)
    and the expert axis runs over ``dp * tp``.  ``etp == tp`` (expert tensor parallelism, the ``ETP x EP x EDP``
    folding of ``moe/MegatronCore_MoE_reading_notes.md:159-195``): every tensor-parallel rank routes all the group's
    tokens and holds ``1 / tp`` of every local expert's feed-forward columns; the expert axis runs over ``dp`` inside
    each tensor-parallel plane."""
    world, rank = dist.get_world_size(), dist.get_rank()
    if world % (pp * cp * tp):
        raise ValueError(f"world={world} not divisible by pp*cp*tp={pp * cp * tp}")
    if replicas > 1:
        raise ValueError("num_distributed_optimizer_instances > 1 is not combined with tensor parallelism")
    dp = world // (pp * cp * tp)
    xs = dp * tp if etp == 1 else dp              # the MoE blocks' data axis
    ep = min(ep, xs)
    if xs % ep:
        raise ValueError(f"dp*tp={xs} not divisible by ep={ep}")
    edp_n = xs // ep

    def rid(p, d, c, t):
        return ((p * dp + d) * cp + c) * tp + t

    tp_rank = rank % tp

    def rid_x(p, x, c, t=0):
        return rid(p, x // tp, c, x % tp) if etp == 1 else rid(p, x, c, t)

    cp_rank = (rank // tp) % cp
    dp_rank = (rank // (tp * cp)) % dp
    pp_rank = rank // (tp * cp * dp)
    x = dp_rank * tp + tp_rank if etp == 1 else dp_rank
    m = Mesh(world=world, rank=rank, pp=pp, dp=dp, cp=cp, ep=ep, pp_rank=pp_rank, dp_rank=dp_rank,
             cp_rank=cp_rank, ep_rank=x % ep, edp_rank=x // ep, world_group=dist.group.WORLD, tp=tp, tp_rank=tp_rank,
             etp=etp)

    def mk(all_lists):
        got, got_ranks = None, ()
        for ranks in all_lists:
            g = dist.new_group(ranks) if len(ranks) > 1 else None
            if rank in ranks:
                got, got_ranks = g, tuple(ranks)
        return got, got_ranks

    P, D, C, T, X = range(pp), range(dp), range(cp), range(tp), range(xs)
    m.data_group, m.data_ranks = mk([[rid(p, d, c, t) for d in D for c in C] for p in P for t in T])
    m.dp_group, _ = mk([[rid(p, d, c, t) for d in D] for p in P for c in C for t in T])
    planes = range(1) if etp == 1 else T          # with expert tensor parallelism every plane has expert groups of its own
    m.ep_group, m.ep_ranks = mk([[rid_x(p, g * ep + e, c, t) for e in range(ep)]
                                 for p in P for g in range(edp_n) for c in C for t in planes])
    m.edp_group, m.edp_ranks = mk([[rid_x(p, g * ep + e, c, t) for g in range(edp_n) for c in C]
                                   for p in P for e in range(ep) for t in planes])
    m.cp_group, _ = mk([[rid(p, d, c, t) for c in C] for p in P for d in D for t in T])
    pp_lists = [[rid(p, d, c, t) for p in P] for d in D for c in C for t in T]
    m.pp_group, m.pp_ranks = mk(pp_lists)
    m.pp_group_up, _ = mk(pp_lists)
    m.pp_group_down, _ = mk(pp_lists)
    m.tp_group, _ = mk([[rid(p, d, c, t) for t in T] for p in P for d in D for c in C])
    m.stage_group, _ = mk([[rid(p, d, c, t) for d in D for c in C for t in T] for p in P])
    return m
