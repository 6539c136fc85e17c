"""Small stand-alone cases of single kernels, sized for profiler captures (inputs larger than the 126 MB L2, at most
a few hundred MB on the device, a handful of launches) and timed with CUDA events when run without a profiler.

    python benchmarks/kernel_cases.py --case rmsnorm_bwd [--rows 16384] [--hidden 2048] [--iters 3]
    python benchmarks/kernel_cases.py --case scatter_ordered      # 4 emulated ranks on one GPU, phase by phase
    python benchmarks/kernel_cases.py --case combine
    python benchmarks/kernel_cases.py --case reduce_scatter
    python benchmarks/kernel_cases.py --case gemm_ready           # grouped GEMM that takes per-expert arrival flags

The multi-rank kernels (dispatch scatter, combine, FSDP reduce-scatter) run through the single-GPU emulation of
``comm/symm.py``: every emulated rank's phase is enqueued before the next phase starts, so no kernel ever waits for
a later launch.  Peer stores then land in the same GPU's memory: the capture shows the kernel's instruction mix, its
memory traffic and its stalls, not NVLink time.
"""
from __future__ import annotations

import argparse
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


class _Mesh:
    def __init__(self, ep, rank):
        self.ep, self.ep_rank, self.ep_group = ep, rank, None


def _timed(fn, iters):
    fn()
    torch.cuda.synchronize()
    ts = []
    for _ in range(iters):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        ts.append(e0.elapsed_time(e1))
    return sorted(ts)[len(ts) // 2]


def _dispatchers(world, tokens, topk, experts, hidden):
    from system_lab_b200.comm.symm import EmulatedWorld
    from system_lab_b200.moe.fused_dispatch import FusedDispatcher, compute_layout
    dev = torch.device("cuda")
    nbytes = compute_layout(world, experts, topk, hidden, tokens, 128, 0.0, False)[2]
    emu = EmulatedWorld(nbytes, world, dev)
    return [FusedDispatcher(_Mesh(world, r), experts, topk, hidden, tokens, 128, dev, workspace=emu.workspace(r))
            for r in range(world)]


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--case", required=True,
                    choices=["rmsnorm_bwd", "rmsnorm_fwd", "scatter_ordered", "combine", "reduce_scatter", "gemm_ready"])
    ap.add_argument("--rows", type=int, default=16384)
    ap.add_argument("--hidden", type=int, default=2048)
    ap.add_argument("--world", type=int, default=4)
    ap.add_argument("--tokens", type=int, default=4096)
    ap.add_argument("--experts", type=int, default=64)
    ap.add_argument("--topk", type=int, default=8)
    ap.add_argument("--iters", type=int, default=3)
    a = ap.parse_args(argv)
    from system_lab_b200.ops import cuda as cops
    dev = torch.device("cuda")
    torch.manual_seed(0)
    if a.case in ("rmsnorm_bwd", "rmsnorm_fwd"):
        x = torch.randn(a.rows, a.hidden, device=dev, dtype=torch.bfloat16, requires_grad=True)
        w = torch.ones(a.hidden, device=dev, dtype=torch.bfloat16, requires_grad=True)
        g = torch.randn(a.rows, a.hidden, device=dev, dtype=torch.bfloat16)
        if a.case == "rmsnorm_fwd":
            ms = _timed(lambda: cops.rmsnorm(x.detach(), w.detach(), 1e-6), a.iters)
            nbytes = 2 * x.numel() * 2
        else:
            y = cops.rmsnorm(x, w, 1e-6)
            ms = _timed(lambda: torch.autograd.grad(y, (x, w), g, retain_graph=True), a.iters)
            nbytes = 3 * x.numel() * 2
        print(f"{a.case} [{a.rows}, {a.hidden}]: {ms * 1e3:.1f} us, {nbytes / ms / 1e6:.0f} GB/s")
    elif a.case in ("scatter_ordered", "combine", "gemm_ready"):
        ds = _dispatchers(a.world, a.tokens, a.topk, a.experts, a.hidden)
        idx = [torch.stack([torch.randperm(a.experts, device=dev)[:a.topk] for _ in range(a.tokens)]).int()
               for _ in range(a.world)]
        x = [torch.randn(a.tokens, a.hidden, device=dev, dtype=torch.bfloat16) for _ in range(a.world)]
        pr = [torch.rand(a.tokens, a.topk, device=dev) for _ in range(a.world)]
        plans = [d.plan_finish(*p) for d, p in zip(ds, [d.plan_publish(i) for d, i in zip(ds, idx)])]
        nbytes = a.world * a.tokens * a.topk * a.hidden * 2
        if a.case == "scatter_ordered":
            def run():
                for d, pl, xx, pp in zip(ds, plans, x, pr):
                    d.scatter_ordered(pl, xx, pp, 0)
            ms = _timed(run, a.iters)
            print(f"scatter_ordered x{a.world} ranks, {a.tokens} tokens x top-{a.topk} x {a.hidden}: {ms * 1e3:.1f} us, "
                  f"{2 * nbytes / ms / 1e6:.0f} GB/s read+write (local memory)")
        elif a.case == "combine":
            rd = [d.scatter_ordered(pl, xx, pp, 0) for d, pl, xx, pp in zip(ds, plans, x, pr)]
            for r in rd:
                r.wait()
            for d in ds:
                d.out_rows.copy_(d.rows[0])

            def run():
                eps = [d.signal_out() for d in ds]
                for d, pl, e in zip(ds, plans, eps):
                    d.pull_rows(pl, e)
            ms = _timed(run, a.iters)
            print(f"combine (pull) x{a.world} ranks: {ms * 1e3:.1f} us, {nbytes / ms / 1e6:.0f} GB/s gathered (local memory)")
        else:
            n = 1536
            e_local = a.experts // a.world
            w = (0.02 * torch.randn(e_local, n, a.hidden, device=dev)).to(torch.bfloat16)

            def run():
                rd = [d.scatter_ordered(pl, xx, pp, 0) for d, pl, xx, pp in zip(ds, plans, x, pr)]
                for d, pl, r in zip(ds, plans, rd):
                    cops.grouped_gemm_raw(0, d.rows[0], w, pl.expert_offsets, pl.expert_counts, n, a.hidden, ready=r)
            ms = _timed(run, a.iters)
            print(f"scatter_ordered + grouped GEMM with arrival flags x{a.world} ranks: {ms * 1e3:.1f} us")
    else:
        from system_lab_b200.comm.fsdp_comm import FsdpPeerComm
        from system_lab_b200.comm.symm import EmulatedWorld
        shard = 8 * 1024 * 1024
        emu = {}

        def factory(rank):
            def make(nbytes):
                key = nbytes
                if key not in emu:
                    emu[key] = EmulatedWorld(nbytes, a.world, dev)
                return emu[key].workspace(rank)
            return make
        cs = [FsdpPeerComm(None, a.world, r, dev, workspace_factory=factory(r)) for r in range(a.world)]
        grads = [torch.randn(shard * a.world, device=dev).to(torch.bfloat16) for _ in range(a.world)]

        def run():
            import ctypes
            meta = []
            for c, g in zip(cs, grads):
                c._ensure(g.numel() * 2)
                slot, ep, ack = c._next()
                c._stage(g, slot, ep, ack)
                meta.append((slot, ep))
            for c, (slot, ep) in zip(cs, meta):
                piece = torch.empty(shard, dtype=torch.float32, device=dev)
                cops.call("slab_fsdp_reduce_scatter", piece, shard, ctypes.addressof(c._ptrs), ctypes.addressof(c._lay),
                          a.world, c.rank, slot, ep, 1.0, c.status, c.done, cops.stream())
        ms = _timed(run, a.iters)
        print(f"fsdp stage + reduce-scatter x{a.world} ranks, {shard * a.world * 2 / 1e6:.0f} MB gradients each: {ms * 1e3:.1f} us")
    cops.check_status()
    return 0


if __name__ == "__main__":
    sys.exit(main())
