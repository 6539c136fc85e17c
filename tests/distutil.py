"""Helpers to run a function on N CPU ranks (gloo) as child processes."""
import os
import socket
import sys
import traceback

import torch.multiprocessing as mp


def _free_port() -> int:
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _entry(rank, world, port, fn, args, q):
    os.environ.update(RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank),
                      MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    try:
        import torch
        torch.set_num_threads(1)
        out = fn(rank, world, *args)
        q.put((rank, "ok", out))
    except Exception:
        q.put((rank, "err", traceback.format_exc()))
    finally:
        import torch.distributed as dist
        if dist.is_initialized():
            try:
                dist.destroy_process_group()
            except Exception:
                pass


_CTX = []


def _context():
    """Children fork from a helper process that has already imported torch (seconds saved per rank); nothing in the
    helper has touched a process group, a thread pool or a device."""
    if not _CTX:
        ctx = mp.get_context("forkserver")
        ctx.set_forkserver_preload(["torch", "torch.distributed", "system_lab_b200.trainer.loop"])
        _CTX.append(ctx)
    return _CTX[0]


def run_ranks(fn, world: int, *args, timeout: float = 240.0):
    """Run ``fn(rank, world, *args)`` on ``world`` spawned processes; returns results by rank."""
    ctx = _context()
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_entry, args=(r, world, port, fn, args, q)) for r in range(world)]
    for p in procs:
        p.start()
    import queue
    import time
    results = {}
    deadline = time.monotonic() + timeout
    try:
        while len(results) < world:
            try:
                rank, status, payload = q.get(timeout=1.0)
            except queue.Empty:
                # a child that died without reporting (a crash in native code) would otherwise cost the whole timeout
                dead = [(r, p.exitcode) for r, p in enumerate(procs)
                        if r not in results and p.exitcode not in (None, 0)]
                if dead:
                    raise RuntimeError(f"rank(s) died without a result: {dead}")
                if time.monotonic() > deadline:
                    raise
                continue
            if status == "err":
                raise RuntimeError(f"rank {rank} failed:\n{payload}")
            results[rank] = payload
    finally:
        for p in procs:
            p.join(timeout=10)
            if p.is_alive():
                p.kill()
    return [results[r] for r in range(world)]
