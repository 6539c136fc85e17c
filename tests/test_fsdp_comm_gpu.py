"""Peer-memory FSDP collectives, several ranks emulated on one GPU phase by phase."""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _comms(world, nbytes):
    from system_lab_b200.comm.fsdp_comm import NSLOT, FsdpPeerComm
    from system_lab_b200.comm.symm import EmulatedWorld
    dev = torch.device("cuda")
    slot = (max(nbytes, 1 << 20) + 255) // 256 * 256
    emu = EmulatedWorld(4096 + NSLOT * slot, world, dev)
    return [FsdpPeerComm(None, world, r, dev, workspace_factory=lambda n, r=r: emu.workspace(r)) for r in range(world)]


@pytest.mark.parametrize("world", [2, 4])
def test_all_gather_and_reduce_scatter(world):
    from system_lab_b200.ops import cuda as cops
    shard = 128 * 37
    cs = _comms(world, shard * world * 2)
    for it in range(6):                                   # more calls than slots: exercises the ack path
        torch.manual_seed(it)
        shards = [torch.randn(shard, device="cuda").to(torch.bfloat16) for _ in range(world)]
        outs = [torch.empty(shard * world, device="cuda", dtype=torch.bfloat16) for _ in range(world)]
        meta = []
        for c, s in zip(cs, shards):
            c._ensure(shard * 2)
            slot, ep, ack = c._next()
            c._stage(s, slot, ep, ack)
            meta.append((slot, ep))
        for c, o, (slot, ep) in zip(cs, outs, meta):
            cops.call("slab_fsdp_all_gather", o, shard * 2, ctypes.addressof(c._ptrs), ctypes.addressof(c._lay),
                      world, c.rank, slot, ep, c.status, c.done, cops.stream())
        torch.cuda.synchronize()
        cops.check_status()
        exp = torch.cat(shards)
        assert all(torch.equal(o, exp) for o in outs)
        grads = [torch.randn(shard * world, device="cuda").to(torch.bfloat16) for _ in range(world)]
        meta = []
        for c, g in zip(cs, grads):
            c._ensure(g.numel() * 2)
            slot, ep, ack = c._next()
            c._stage(g, slot, ep, ack)
            meta.append((slot, ep))
        pieces = []
        for c, (slot, ep) in zip(cs, meta):
            p = torch.empty(shard, dtype=torch.float32, device="cuda")
            cops.call("slab_fsdp_reduce_scatter", p, shard, ctypes.addressof(c._ptrs), ctypes.addressof(c._lay), world,
                      c.rank, slot, ep, 0.5, c.status, c.done, cops.stream())
            pieces.append(p)
        torch.cuda.synchronize()
        cops.check_status()
        total = sum(g.float() for g in grads) * 0.5
        for r, p in enumerate(pieces):
            assert torch.allclose(p, total[r * shard:(r + 1) * shard], atol=1e-5)


def test_reduce_scatter_fused_adamw_matches_two_step():
    from system_lab_b200.ops import cuda as cops, reference as ref
    world, shard = 2, 128 * 20
    decay_end = 128 * 15
    cs = _comms(world, shard * world * 2)
    torch.manual_seed(3)
    grads = [torch.randn(shard * world, device="cuda").to(torch.bfloat16) * 0.01 for _ in range(world)]
    masters = [torch.randn(shard, device="cuda") * 0.02 for _ in range(world)]
    refs = [m.clone() for m in masters]
    ms = [torch.zeros(shard, device="cuda") for _ in range(world)]
    vs = [torch.zeros(shard, device="cuda") for _ in range(world)]
    outs = [torch.empty(shard, device="cuda", dtype=torch.bfloat16) for _ in range(world)]
    sq = torch.zeros(1, device="cuda")
    coef = torch.tensor(0.7, device="cuda")
    meta = []
    for c, g in zip(cs, grads):
        c._ensure(g.numel() * 2)
        slot, ep, ack = c._next()
        c._stage(g, slot, ep, ack)
        meta.append((slot, ep))
    for r, (c, (slot, ep)) in enumerate(zip(cs, meta)):
        cops.call("slab_fsdp_reduce_scatter_adamw", shard, ctypes.addressof(c._ptrs), ctypes.addressof(c._lay), world,
                  c.rank, slot, ep, 1.0, masters[r], ms[r], vs[r], outs[r], coef, sq, 1e-2, 0.9, 0.95, 1e-8, 0.1,
                  1 - 0.9, 1 - 0.95, decay_end, c.status, c.done, cops.stream())
    torch.cuda.synchronize()
    cops.check_status()
    total = sum(g.float() for g in grads)
    for r in range(world):
        gr = total[r * shard:(r + 1) * shard]
        m0, v0 = torch.zeros(shard, device="cuda"), torch.zeros(shard, device="cuda")
        for lo, hi, wd in ((0, decay_end, 0.1), (decay_end, shard, 0.0)):       # no decay behind the boundary
            ref.adamw_step(refs[r][lo:hi], gr[lo:hi] * 0.7, m0[lo:hi], v0[lo:hi], lr=1e-2, beta1=0.9, beta2=0.95,
                           eps=1e-8, weight_decay=wd, step=1)
        assert torch.allclose(masters[r], refs[r], atol=1e-6)
        assert torch.allclose(outs[r].float(), refs[r], atol=2e-3)
    assert abs(sq.item() - total.pow(2).sum().item()) / total.pow(2).sum().item() < 1e-4
