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


@pytest.mark.parametrize("world", [2, 4, 8])
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


@pytest.mark.parametrize("world", [2, 4, 8])
def test_all_gather_fused_into_the_consuming_gemm(world):
    """A flat parameter buffer (three matrices, then a tail of 1-D parameters) sharded over `world` ranks: every rank
    stages its shard and pulls the tail, then multiplies by the second matrix with the kernel whose gather warps pull
    all matrices from the staged shards.  Afterwards every rank holds the whole buffer, the product equals the fp32
    reference, and the slots have been acknowledged (six rounds reuse the four slots).  Ranks are emulated phase by
    phase: every rank stages before any rank's GEMM starts."""
    from system_lab_b200.ops import cuda as cops
    torch.manual_seed(11)
    dev = torch.device("cuda")
    k, n0, n1, n2 = 512, 256, 1152, 384                       # matrices [n, k]; the GEMM multiplies the second one
    mats = (n0 + n1 + n2) * k
    tail = 128 * 5
    total = (mats + tail + 128 * world - 1) // (128 * world) * (128 * world)
    shard = total // world
    cs = _comms(world, shard * 2)
    pieces = [torch.zeros((total * 2 + cs[0].PIECE_BYTES - 1) // cs[0].PIECE_BYTES, dtype=torch.int32, device=dev)
              for _ in range(world)]
    rows = 777
    for call in range(1, 7):
        flat_ref = (0.05 * torch.randn(total, device=dev)).to(torch.bfloat16)
        x = torch.randn(rows, k, device=dev, dtype=torch.bfloat16)
        fulls = [torch.full((total,), float("nan"), device=dev, dtype=torch.bfloat16) for _ in range(world)]
        tickets = [c.stage_for_gather(flat_ref[r * shard:(r + 1) * shard].clone(), mats * 2) for r, c in enumerate(cs)]
        for r, c in enumerate(cs):                             # every rank has staged: now the tails can be pulled
            c.gather_tail(tickets[r], fulls[r])
        torch.cuda.synchronize()
        for r in range(world):                                 # the tail is there before any GEMM runs
            assert torch.equal(fulls[r][mats:], flat_ref[mats:])
        outs = []
        for r, c in enumerate(cs):
            w_off = n0 * k
            w = fulls[r][w_off:w_off + n1 * k].view(n1, k)
            out = torch.empty(rows, n1, device=dev, dtype=torch.bfloat16)
            c.gemm_gather(tickets[r], x, w, out, fulls[r], w_off, cops._dense_segments(dev, rows), pieces[r], call,
                          cops._pick_bn(n1))
            outs.append(out)
        torch.cuda.synchronize()
        cops.check_status()
        want = x.float() @ flat_ref[n0 * k:(n0 + n1) * k].view(n1, k).float().t()
        for r in range(world):
            assert torch.equal(fulls[r], flat_ref), f"rank {r}: gathered buffer differs (call {call})"
            err = (outs[r].float() - want).abs().max().item()
            assert err < 2e-2 * (want.abs().max().item() + 1e-6), (r, call, err)


@pytest.mark.parametrize("world,batch,seq,n,k", [(2, 2, 256, 256, 128), (4, 1, 1024, 2048, 192), (8, 2, 512, 576, 64)])
def test_gemm_fused_with_reduce_scatter(world, batch, seq, n, k):
    """Row-parallel GEMM whose epilogue pushes every output row to the rank that owns it (sequence split over the
    group) and owners that sum the partial rows: equal to the fp32 sum of the ranks' products, three calls in a row
    so that both receive regions and the acknowledgement wait are used.  Ranks are emulated phase by phase."""
    from system_lab_b200.comm.gemm_rs import GemmReduceScatter
    from system_lab_b200.comm.symm import EmulatedWorld
    from system_lab_b200.ops import cuda as cops
    dev = torch.device("cuda")
    torch.manual_seed(world)
    emu = EmulatedWorld(GemmReduceScatter.nbytes(batch, seq, n, world), world, dev)
    ops = [GemmReduceScatter(None, world, r, dev, batch, seq, n, workspace=emu.workspace(r)) for r in range(world)]
    s_local = seq // world
    for _ in range(3):
        a = [torch.randn(batch * seq, k, device=dev).to(torch.bfloat16) for _ in range(world)]
        w = [(0.1 * torch.randn(n, k, device=dev)).to(torch.bfloat16) for _ in range(world)]
        eps = [op.push(a[r], w[r]) for r, op in enumerate(ops)]
        ys = [op.reduce(e) for op, e in zip(ops, eps)]
        torch.cuda.synchronize()
        cops.check_status()
        full = sum(a[r].float() @ w[r].float().t() for r in range(world)).view(batch, seq, n)
        for r in range(world):
            want = full[:, r * s_local:(r + 1) * s_local].reshape(-1, n)
            err = (ys[r].float() - want).abs().max().item()
            assert err < 2e-2 * want.abs().max().item(), (r, err)
