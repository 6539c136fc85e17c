"""``python -m system_lab_b200.ckpt <command> <checkpoint dir or its parent>``: offline checkpoint tools.

    inspect      step, mesh, optimizer dtype, parameter table (name, global shape, pieces, bytes) of a checkpoint
    verify       re-hash every rank file against its SHA-256 sidecar; exit code 1 on a mismatch or a missing file
    consolidate  assemble full tensors from the pieces of all ranks and write one ``{name: tensor}`` file
                 (weights only; tensor-parallel slices keep their ``#tpRofN`` suffix)
    prune        keep the newest N step directories of a checkpoint root

No process group, no GPU: the tools read the rank files directly.  The piece index every rank file carries
(``fqn``, ``global_shape``, flat ``start`` / ``len``) is what makes a checkpoint independent of the layout that wrote
it; ``consolidate`` is the same walk the loader does, for all parameters at once.

Reference: the "checkpoint manager" role of the tuner design (resume configuration, resharding on a parallelism
change, cleanup policy; PTA.pdf p.5) and Megatron's distributed checkpoints as described in
``moe/MegatronCore_MoE_reading_notes.md:724-728``; the reference ships no checkpoint code.
"""
from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path

import torch

from .sharded import _prune, _sha256, resolve


def _rank_files(ck: Path) -> list[Path]:
    return sorted(ck.glob("rank_*.pt"))


def _index(ck: Path) -> dict:
    """fqn -> {"shape": global shape, "pieces": [(start, len, file, key)]} over all rank files."""
    table: dict[str, dict] = {}
    for f in _rank_files(ck):
        payload = torch.load(f, map_location="cpu", weights_only=False)
        for rec in payload["index"]:
            ent = table.setdefault(rec["fqn"], {"shape": tuple(rec["global_shape"]), "pieces": []})
            ent["pieces"].append((rec["start"], rec["len"], f.name, rec["key"]))
    return table


def cmd_inspect(ck: Path, as_json: bool) -> int:
    meta = json.loads((ck / "meta.json").read_text())
    table = _index(ck)
    rows = []
    for fqn in sorted(table):
        shape = table[fqn]["shape"]
        numel = 1
        for d in shape:
            numel *= d
        covered = sum(n for _, n, _, _ in table[fqn]["pieces"])
        rows.append({"name": fqn, "shape": list(shape), "elements": numel, "pieces": len(table[fqn]["pieces"]),
                     "covered": covered})
    out = {"path": str(ck), "step": meta["step"], "world": meta["world"], "mesh": meta["mesh"],
           "optimizer_state_dtype": meta.get("optimizer_state_dtype"), "rank_files": len(_rank_files(ck)),
           "parameters": len(rows), "elements": sum(r["elements"] for r in rows), "tensors": rows}
    if as_json:
        print(json.dumps(out, indent=2))
        return 0
    print(f"{ck}: step {out['step']}, written by {out['world']} rank(s), mesh {out['mesh']}, "
          f"optimizer state {out['optimizer_state_dtype']}, {out['parameters']} tensors, {out['elements']:,} elements")
    for r in rows:
        flag = "" if r["covered"] >= r["elements"] else f"  INCOMPLETE ({r['covered']:,} of {r['elements']:,})"
        print(f"  {r['name']:60s} {str(tuple(r['shape'])):24s} {r['pieces']:3d} piece(s){flag}")
    return 0


def cmd_verify(ck: Path) -> int:
    meta = json.loads((ck / "meta.json").read_text())
    bad = 0
    files = _rank_files(ck)
    for f in files:
        side = f.with_suffix(".sha256")
        if not side.exists():
            print(f"{f.name}: no checksum file")
            bad += 1
        elif side.read_text().strip() != _sha256(f):
            print(f"{f.name}: checksum mismatch")
            bad += 1
    table = _index(ck) if not bad else {}
    for fqn, ent in table.items():
        numel = 1
        for d in ent["shape"]:
            numel *= d
        spans = sorted((s, s + n) for s, n, _, _ in ent["pieces"])
        pos = 0
        for a, b in spans:
            if a > pos:
                break
            pos = max(pos, b)
        if pos < numel:
            print(f"{fqn}: pieces cover {pos:,} of {numel:,} elements")
            bad += 1
    print(f"{ck}: {len(files)} rank file(s) of {meta['world']} rank(s), {'OK' if not bad else f'{bad} problem(s)'}")
    return 1 if bad else 0


def cmd_consolidate(ck: Path, out: Path, dtype: str) -> int:
    table = _index(ck)
    payloads = {f.name: torch.load(f, map_location="cpu", weights_only=False)["tensors"] for f in _rank_files(ck)}
    state = {}
    for fqn, ent in table.items():
        numel = 1
        for d in ent["shape"]:
            numel *= d
        flat = None
        for start, n, fname, key in ent["pieces"]:
            piece = payloads[fname][f"w/{key}"]
            if flat is None:
                flat = torch.zeros(numel, dtype=piece.dtype)
            flat[start:start + n] = piece[:n]
        t = flat.view(ent["shape"])
        state[fqn] = t.to(getattr(torch, dtype)) if dtype else t
    out.parent.mkdir(parents=True, exist_ok=True)
    torch.save(state, out)
    print(f"wrote {len(state)} tensors, {sum(t.numel() for t in state.values()):,} elements to {out}")
    return 0


def main(argv=None) -> int:
    ap = argparse.ArgumentParser("system_lab_b200.ckpt")
    sub = ap.add_subparsers(dest="cmd", required=True)
    p = sub.add_parser("inspect")
    p.add_argument("path")
    p.add_argument("--json", action="store_true")
    p = sub.add_parser("verify")
    p.add_argument("path")
    p = sub.add_parser("consolidate")
    p.add_argument("path")
    p.add_argument("--out", required=True)
    p.add_argument("--dtype", default="", help="cast to this torch dtype (e.g. bfloat16); default: as stored")
    p = sub.add_parser("prune")
    p.add_argument("path", help="checkpoint root (the directory holding step_* directories)")
    p.add_argument("--keep", type=int, required=True)
    a = ap.parse_args(argv)
    if a.cmd == "prune":
        _prune(Path(a.path), a.keep)
        print("kept:", ", ".join(sorted(p.name for p in Path(a.path).glob("step_*"))))
        return 0
    ck = resolve(a.path)
    if a.cmd == "inspect":
        return cmd_inspect(ck, a.json)
    if a.cmd == "verify":
        return cmd_verify(ck)
    return cmd_consolidate(ck, Path(a.out), a.dtype)


if __name__ == "__main__":
    sys.exit(main())
