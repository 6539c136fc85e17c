"""Sharded, reshardable checkpoints.

Layout (the reference defines no model-checkpoint format; it only describes Megatron's distributed
checkpoint — sharded-tensor descriptors, parallel save, load under a different layout,
``moe/MegatronCore_MoE_reading_notes.md:724-728``)::

    <root>/step_000020/
        meta.json                  resolved config, mesh, step, data cursor, loss curve, tensor index
        rank_00000.pt              this rank's tensors (weights, optimizer moments, RNG state)
    <root>/latest                  text file naming the newest complete step directory

Every logical tensor is stored as pieces ``{fqn, global_shape, flat_start, flat_len}``: a piece is a
contiguous range of the flattened *global* tensor (for expert tensors the global tensor spans all
experts).  Loading walks the pieces that intersect what the new layout owns, so a checkpoint written
under one ``dp/ep/pp`` loads under another.  Directories are written under a temporary name and
renamed, so a killed save never leaves a half checkpoint that looks complete.  Every rank file has a SHA-256
sidecar; a file that fails its check (or cannot be unpickled) makes *all* ranks reject that step together and
fall back to the previous complete one.
"""
from __future__ import annotations

import hashlib
import json
import logging
import os
import shutil
from pathlib import Path

import torch
import torch.distributed as dist


log = logging.getLogger(__name__)


class CheckpointCorrupt(RuntimeError):
    """A rank file is missing, fails its checksum or cannot be read."""


def _sha256(path: Path) -> str:
    h = hashlib.sha256()
    with open(path, "rb") as f:
        for chunk in iter(lambda: f.read(1 << 24), b""):
            h.update(chunk)
    return h.hexdigest()


def _barrier():
    if dist.is_initialized() and dist.get_world_size() > 1:
        dist.barrier()


def _global_view(group, name: str, shape: tuple, e_rank: int, e_size: int, is_expert: bool):
    """Global shape and the flat offset of this rank's copy of the parameter inside it."""
    if is_expert:
        gshape = (shape[0] * e_size,) + tuple(shape[1:])
        per = 1
        for s in shape:
            per *= s
        return gshape, e_rank * per
    return tuple(shape), 0


def _owned_pieces(trainer):
    """Yield ``(kind, fqn, global_shape, global_flat_start, length, source_tensor_slice_fn)`` for
    every piece of every parameter that this rank's shards own."""
    mesh = trainer.mesh
    for g in trainer.engine.all_groups():
        lo = g.rank * g.shard_numel if g.sharded else 0
        hi = lo + (g.shard_numel if g.sharded else g.total)
        for (fqn, shape, off, numel), p in zip(g.param_slices(), g.params):
            a, b = max(off, lo), min(off + numel, hi)
            if a >= b:
                continue
            is_exp = getattr(p, "is_expert", False)
            if hasattr(p, "tp_segments"):
                # a tensor-parallel slice is stored as a tensor of its own, named after its rank in the group
                fqn = f"{fqn}#tp{mesh.tp_rank}of{mesh.tp}"
            gshape, base = _global_view(g, fqn, shape, mesh.ep_rank, mesh.ep, is_exp)
            yield g, fqn, gshape, base + (a - off), b - a, a - lo


def _is_writer(trainer, g) -> bool:
    """Groups replicated across data ranks (unsharded ones, or the blocks of hybrid sharding): only the first
    replica writes."""
    if getattr(g, "tp_replicas", 1) > 1 and trainer.mesh.tp_rank != 0:
        return False                      # dense groups are identical on every tensor-parallel rank
    if g.replica_group is None:
        return True
    return dist.get_rank(g.replica_group) == 0


def _snapshot(trainer) -> tuple[dict, dict]:
    """Host copies of everything this rank writes, plus the metadata rank 0 adds: the state of the job at this step."""
    mesh, opt = trainer.mesh, trainer.optimizer
    tensors, index = {}, []
    for g, fqn, gshape, gstart, length, soff in _owned_pieces(trainer):
        if not _is_writer(trainer, g):
            continue
        key = f"{fqn}@{gstart}"
        rec = {"fqn": fqn, "global_shape": list(gshape), "start": gstart, "len": length, "key": key}
        tensors[f"w/{key}"] = g.shard[soff:soff + length].detach().cpu().clone()
        moments = () if getattr(g, "frozen", False) else (("m", opt.m[g.name]), ("v", opt.v[g.name]))
        for mom_name, mom in moments:
            tensors[f"{mom_name}/{key}"] = mom.data[soff:soff + length].detach().cpu().clone()
            if mom.kind == "fp8":
                # scales are per 128 elements of the shard; pieces start on 128-element boundaries
                tensors[f"{mom_name}s/{key}"] = mom.scale[soff // 128:(soff + length + 127) // 128].cpu().clone()
        index.append(rec)
    buffers = {}
    for u in trainer.engine.units:
        for bn, b in u.module.named_buffers():
            buffers[f"{u.name}.{bn}"] = b.detach().cpu().clone()
    prev = opt._prev_norm
    payload = {"tensors": tensors, "index": index, "buffers": buffers,
               "opt_step": opt.step_count, "prev_norm": prev.detach().cpu().clone() if torch.is_tensor(prev) else prev,
               "torch_rng": torch.get_rng_state()}
    meta = {"format": "system_lab_b200.ckpt.v1", "step": trainer.step, "world": mesh.world,
            "mesh": {"pp": mesh.pp, "dp": mesh.dp, "cp": mesh.cp, "ep": mesh.ep, "tp": mesh.tp},
            "data_cursor": trainer.data.cursor, "loss_curve": list(trainer.loss_curve),
            "optimizer_state_dtype": trainer.cfg.precision.optimizer_state_dtype,
            "config": trainer.cfg.to_dict()}
    return payload, meta


def _write_rank_file(tmp: Path, rank: int, payload: dict) -> None:
    mine = tmp / f"rank_{rank:05d}.pt"
    torch.save(payload, mine)
    mine.with_suffix(".sha256").write_text(_sha256(mine))


def _publish(root_p: Path, tmp: Path, final: Path, meta: dict, keep_last: int) -> None:
    """Rank 0, after every rank's file is on disk: metadata, atomic rename, ``latest`` pointer, retention."""
    (tmp / "meta.json").write_text(json.dumps(meta, indent=2))
    if final.exists():
        shutil.rmtree(final)
    os.replace(tmp, final)
    (root_p / "latest.tmp").write_text(final.name)
    os.replace(root_p / "latest.tmp", root_p / "latest")
    _prune(root_p, keep_last)


def save_checkpoint(trainer, root: str) -> str:
    """Synchronous by default.  With ``checkpoint.async_save`` the state is copied to host memory here and written
    by a background thread while training goes on; the checkpoint becomes visible (metadata, rename) at a later step
    boundary, once every rank's file is complete (``finish_pending``).  The reference's runs paid 6 minutes per
    268 GB save with training stopped (``notes/2026-04/2026-04-22_gptoss_22_*:170,180-181``)."""
    finish_pending(trainer, wait=True)                # at most one save in flight
    mesh = trainer.mesh
    root_p = Path(root)
    final = root_p / f"step_{trainer.step:06d}"
    tmp = root_p / f".tmp_step_{trainer.step:06d}"
    if mesh.rank == 0:
        if tmp.exists():
            shutil.rmtree(tmp)
        tmp.mkdir(parents=True, exist_ok=True)
    _barrier()
    payload, meta = _snapshot(trainer)
    keep = trainer.cfg.checkpoint.keep_last
    if getattr(trainer.cfg.checkpoint, "async_save", False):
        import threading
        box = {"error": None}

        def work():
            try:
                _write_rank_file(tmp, mesh.rank, payload)
            except BaseException as e:                # surfaced by finish_pending on the main thread
                box["error"] = e
        th = threading.Thread(target=work, name="slab-ckpt-writer", daemon=False)
        th.start()
        trainer._pending_ckpt = {"thread": th, "box": box, "root": root_p, "tmp": tmp, "final": final, "meta": meta,
                                 "keep": keep}
        return str(final)
    _write_rank_file(tmp, mesh.rank, payload)
    _barrier()
    if mesh.rank == 0:
        _publish(root_p, tmp, final, meta, keep)
    _barrier()
    return str(final)


def finish_pending(trainer, wait: bool = False) -> bool:
    """Complete an asynchronous save if every rank's writer has finished (``wait``: block until they have).
    Collective: every rank calls it at the same points (step boundaries, the next save, the end of ``fit``).
    Returns True if nothing is pending any more."""
    pend = getattr(trainer, "_pending_ckpt", None)
    if pend is None:
        return True
    th = pend["thread"]
    if wait:
        th.join()
    done = torch.tensor([0.0 if th.is_alive() else 1.0])
    if dist.is_initialized() and dist.get_world_size() > 1:
        done = done.to(trainer.device)
        dist.all_reduce(done, op=dist.ReduceOp.MIN)
    if float(done) < 1.0:
        return False
    th.join()
    trainer._pending_ckpt = None
    err = torch.tensor([1.0 if pend["box"]["error"] is not None else 0.0])
    if dist.is_initialized() and dist.get_world_size() > 1:
        err = err.to(trainer.device)
        dist.all_reduce(err, op=dist.ReduceOp.MAX)
    if float(err) > 0:
        raise RuntimeError(f"asynchronous checkpoint {pend['final']} failed on some rank: {pend['box']['error']!r}")
    if trainer.mesh.rank == 0:
        _publish(pend["root"], pend["tmp"], pend["final"], pend["meta"], pend["keep"])
    _barrier()
    return True


def _prune(root: Path, keep: int) -> None:
    if keep <= 0:
        return
    steps = sorted(p for p in root.glob("step_*") if p.is_dir())
    for p in steps[:-keep]:
        shutil.rmtree(p, ignore_errors=True)


def resolve(path: str) -> Path:
    p = Path(path)
    if (p / "meta.json").exists():
        return p
    latest = p / "latest"
    if latest.exists():
        return p / latest.read_text().strip()
    raise FileNotFoundError(f"no checkpoint under {path}")


def _candidates(path: str) -> list[Path]:
    """The checkpoint ``path`` names (or its parent's ``latest``) followed by older complete steps beside it."""
    first = resolve(path)
    older = sorted((p for p in first.parent.glob("step_*") if p.is_dir() and (p / "meta.json").exists()
                    and p.name < first.name), reverse=True)
    return [first] + older


def _agree(ok: bool, device) -> bool:
    """True only if every rank says ok (one small all-reduce), so all ranks accept or reject a step together."""
    if not (dist.is_initialized() and dist.get_world_size() > 1):
        return ok
    t = torch.tensor([1 if ok else 0], dtype=torch.int32, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MIN)
    return bool(int(t.item()))


def load_checkpoint(trainer, path: str, fallback: bool = True) -> str:
    """Load the newest usable checkpoint under ``path``; returns the directory that was loaded."""
    cands = _candidates(path)
    if not fallback:
        cands = cands[:1]
    last_err: Exception | None = None
    for ck in cands:
        err = None
        try:
            _load_one(trainer, ck)
        except Exception as e:           # every rank must reach the agreement below, whatever went wrong here
            err = e
        if _agree(err is None, trainer.device):
            if ck != cands[0] and trainer.mesh.rank == 0:
                log.warning("loaded %s instead of %s", ck, cands[0])
            _barrier()
            return str(ck)
        last_err = err or CheckpointCorrupt(f"{ck}: rejected by another rank")
        if trainer.mesh.rank == 0:
            log.warning("checkpoint %s is not usable (%s); trying an older one", ck, last_err)
    raise CheckpointCorrupt(f"no usable checkpoint under {path}: {last_err}")


def _load_one(trainer, ck: Path) -> None:
    meta = json.loads((ck / "meta.json").read_text())
    if meta.get("format") != "system_lab_b200.ckpt.v1":
        raise ValueError(f"unknown checkpoint format in {ck}")
    saved = dict(meta["mesh"])
    saved.setdefault("tp", 1)
    if saved["tp"] != trainer.mesh.tp:
        raise ValueError(f"checkpoint was written with tensor_model_parallel_size={saved['tp']}; tensor-parallel slices "
                         f"are not re-cut on load (this job runs {trainer.mesh.tp})")
    same_layout = (meta["world"] == trainer.mesh.world and
                   saved == {"pp": trainer.mesh.pp, "dp": trainer.mesh.dp, "cp": trainer.mesh.cp,
                             "ep": trainer.mesh.ep, "tp": trainer.mesh.tp})
    own = ck / f"rank_{trainer.mesh.rank:05d}.pt"
    files = sorted(ck.glob("rank_*.pt"))
    if same_layout:                       # own file first; others only if a replica did not write
        files = [own] + [f for f in files if f != own]
    opt = trainer.optimizer
    if not same_layout and meta.get("optimizer_state_dtype") == "fp8":
        raise ValueError("resharding 8-bit optimizer state is not supported; load under the saved layout")
    want = list(_owned_pieces(trainer))
    filled = {id(g): 0 for g, *_ in want}
    buffers_needed = {f"{u.name}.{bn}" for u in trainer.engine.units for bn, _ in u.module.named_buffers()}
    buffers_done = not buffers_needed
    need_total = {id(g): 0 for g, *_ in want}
    for g, _, _, _, length, _ in want:
        need_total[id(g)] += length
    for f in files:
        if all(filled[k] >= need_total[k] for k in filled) and buffers_done:
            break
        if not f.exists():
            raise CheckpointCorrupt(f"{f} is missing")
        side = f.with_suffix(".sha256")
        if side.exists() and side.read_text().strip() != _sha256(f):
            raise CheckpointCorrupt(f"{f} fails its SHA-256 check")
        try:
            payload = torch.load(f, map_location="cpu", weights_only=False)
        except Exception as e:                                   # truncated or damaged pickle
            raise CheckpointCorrupt(f"{f} cannot be read: {type(e).__name__}: {e}") from e
        by_fqn: dict[str, list] = {}
        for rec in payload["index"]:
            by_fqn.setdefault(rec["fqn"], []).append(rec)
        for g, fqn, gshape, gstart, length, soff in want:
            for rec in by_fqn.get(fqn, ()):
                a, b = max(gstart, rec["start"]), min(gstart + length, rec["start"] + rec["len"])
                if a >= b:
                    continue
                src = slice(a - rec["start"], b - rec["start"])
                dst = slice(soff + (a - gstart), soff + (b - gstart))
                g.shard[dst].copy_(payload["tensors"][f"w/{rec['key']}"][src])
                moments = () if getattr(g, "frozen", False) else (("m", opt.m[g.name]), ("v", opt.v[g.name]))
                for mom_name, mom in moments:
                    if f"{mom_name}/{rec['key']}" not in payload["tensors"]:
                        continue              # written by a job in which this parameter was frozen: state starts at zero
                    mom.data[dst].copy_(payload["tensors"][f"{mom_name}/{rec['key']}"][src])
                    if mom.kind == "fp8":
                        sc = payload["tensors"][f"{mom_name}s/{rec['key']}"]
                        mom.scale[dst.start // 128:dst.start // 128 + sc.numel()].copy_(sc)
                filled[id(g)] += b - a
        if not buffers_done:
            for u in trainer.engine.units:
                for bn, b in u.module.named_buffers():
                    k = f"{u.name}.{bn}"
                    if k in buffers_needed and k in payload["buffers"]:
                        b.copy_(payload["buffers"][k])
                        buffers_needed.discard(k)
            buffers_done = not buffers_needed
        if same_layout and f == own:
            torch.set_rng_state(payload["torch_rng"])
        opt.step_count = payload["opt_step"]
        pn = payload.get("prev_norm")
        opt._prev_norm = pn.to(trainer.device) if torch.is_tensor(pn) else pn
    # replicas of unsharded groups did not write: they read the writer's pieces above (same fqn ranges)
    for g in trainer.engine.all_groups():
        need = sum(l for gg, _, _, _, l, _ in want if gg is g)
        if filled[id(g)] < need and all(".lora_" in n for n in g.names) and filled[id(g)] == 0:
            log.info("checkpoint %s has no adapters for %s: they keep their initial values", ck, g.name)
            continue                      # a base-model checkpoint loaded into a LoRA job
        if filled[id(g)] < need:
            raise ValueError(f"checkpoint {ck} does not cover group {g.name}: {filled[id(g)]}/{need} elements")
        if not g.sharded:
            if g.shard is not g.full:
                g.full.copy_(g.shard)
        elif getattr(g, "shard_lp", None) is not None:
            g.shard_lp.copy_(g.shard)
    trainer.step = meta["step"]
    trainer.data.cursor = meta["data_cursor"]
    trainer.loss_curve = list(meta.get("loss_curve", []))
