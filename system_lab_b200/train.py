"""``python -m system_lab_b200.train --config cfg.yaml [--preset NAME] [key=value ...]``

Resolution order: defaults < preset < YAML < ``key=value`` overrides; the resolved config is
written to ``resolved_config.json`` in the job's own directory (the checkpoint save directory, else the directory of
the snapshot or metrics file) before the first step; a job that names none of them writes no file.  Under ``torchrun`` each
process drives one GPU (NCCL); without GPUs the same command runs on CPU ranks over gloo.
"""
from __future__ import annotations

import argparse
import json
import logging
import sys
from pathlib import Path

from .config import Config


def _job_dir(cfg) -> Path | None:
    """Directory that belongs to this job: where it saves checkpoints, else where it writes its snapshot or metrics."""
    if cfg.checkpoint.save:
        return Path(cfg.checkpoint.save)
    for f in (cfg.profile.snapshot_path, cfg.train.metrics_file):
        if f:
            return Path(f).parent
    return None


def main(argv=None) -> int:
    ap = argparse.ArgumentParser("system_lab_b200.train")
    ap.add_argument("--config", default=None, help="YAML file")
    ap.add_argument("--preset", default=None, help="named preset (see models/presets.py)")
    ap.add_argument("--resume", default=None, help="checkpoint directory (or its parent) to resume from")
    ap.add_argument("--print-config", action="store_true", help="print the resolved config and exit")
    ap.add_argument("overrides", nargs="*", help="key=value overrides")
    args = ap.parse_args(argv)
    logging.basicConfig(level=logging.INFO, format="%(asctime)s %(levelname)-7s %(name)s :: %(message)s")
    cfg = Config.load(args.config, args.overrides, args.preset)
    if args.print_config:
        print(json.dumps(cfg.to_dict(), indent=2, sort_keys=True))
        return 0
    from .trainer.loop import Trainer
    tr = Trainer(cfg)
    if tr.mesh.rank == 0:
        from .pilot.constraints import check_config
        for prob in check_config(cfg, tr.mesh.world):
            if prob["severity"] == "warning":
                logging.getLogger("system_lab_b200.config").warning("%s: %s", prob["rule"], prob["message"])
        out_dir = _job_dir(cfg)
        if out_dir is not None:
            cfg.dump(out_dir / "resolved_config.json")
    resume = args.resume or cfg.checkpoint.load
    if resume:
        tr.load_checkpoint(resume)
    try:
        snap = tr.fit(max(cfg.train.train_iters - tr.step, 0))
    except BaseException as e:
        # tell the peers at once (they would otherwise learn of it from a heartbeat or collective timeout)
        if tr.heartbeat is not None:
            tr.heartbeat.fail(f"{type(e).__name__}: {e}")
        raise
    finally:
        tr.close()
    if tr.mesh.rank == 0:
        m = snap["metrics"]
        print(json.dumps({"final_loss": tr.loss_curve[-1] if tr.loss_curve else None, "tps": m["tps"],
                          "step_time_ms": m["step_time_ms"], "steps": tr.step}))
    import torch.distributed as dist
    if dist.is_initialized():
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
