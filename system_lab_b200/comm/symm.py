"""Symmetric peer memory: one workspace per rank, every rank holds the base pointers of all of them.

On a multi-GPU job the workspace is allocated with ``torch.distributed._symmetric_memory`` (CUDA VMM
allocations exchanged by file descriptor) so kernels can load/store peers' buffers over NVLink.  With a
single rank the workspace is an ordinary allocation.  ``EmulatedWorld`` gives several *emulated* ranks
on one device (each with its own workspace and a pointer table of all of them) so the multi-rank flag
protocol can be exercised phase by phase on one GPU.

Reference analogue: HIP IPC mapped buffers plus system-scope atomics, chosen after rocSHMEM and
compiler-generated system atomics failed (``notes/2026-04/2026-04-09_tileflow_mi355x_tile_overlap_analysis.md:55-107``).
"""
from __future__ import annotations

import torch
import torch.distributed as dist


class SymmetricWorkspace:
    def __init__(self, nbytes: int, group, world: int, rank: int, device: torch.device):
        self.nbytes, self.world, self.rank, self.device = nbytes, world, rank, device
        self.multicast_ptr = 0
        if world > 1:
            import torch.distributed._symmetric_memory as symm
            group = group if group is not None else dist.group.WORLD
            self.buf = symm.empty(nbytes, dtype=torch.uint8, device=device)
            self.buf.zero_()
            self.handle = symm.rendezvous(self.buf, group)
            self.ptrs = [int(p) for p in self.handle.buffer_ptrs]
            try:
                self.multicast_ptr = int(self.handle.multicast_ptr or 0)
            except Exception:
                self.multicast_ptr = 0
            torch.cuda.synchronize()
            dist.barrier(group=group)
        else:
            self.buf = torch.zeros(nbytes, dtype=torch.uint8, device=device)
            self.handle = None
            self.ptrs = [self.buf.data_ptr()]

    def view(self, offset: int, shape, dtype) -> torch.Tensor:
        n = 1
        for s in shape:
            n *= s
        nb = n * torch.empty((), dtype=dtype).element_size()
        # `.data` gives an alias with its own autograd version counter: a kernel or copy that writes one
        # region must not invalidate tensors autograd saved from another region of the same workspace
        return self.buf[offset:offset + nb].view(dtype).view(*shape).data


class EmulatedWorld:
    """``world`` workspaces on one device sharing a pointer table (tests only)."""

    def __init__(self, nbytes: int, world: int, device: torch.device):
        self.bufs = [torch.zeros(nbytes, dtype=torch.uint8, device=device) for _ in range(world)]
        self.ptrs = [b.data_ptr() for b in self.bufs]
        self.world = world

    def workspace(self, rank: int) -> "SymmetricWorkspace":
        ws = SymmetricWorkspace.__new__(SymmetricWorkspace)
        ws.nbytes, ws.world, ws.rank = self.bufs[0].numel(), self.world, rank
        ws.device, ws.buf, ws.handle, ws.ptrs, ws.multicast_ptr = self.bufs[0].device, self.bufs[rank], None, self.ptrs, 0
        return ws
