"""Host-side half of the fused dispatcher that needs no GPU: workspace layout, construction in every mode, kept-row
sizing, push-target bookkeeping.  (The kernels themselves are covered by the GPU suite.)"""
import pytest
import torch


class _Mesh:
    def __init__(self, ep=1, ep_rank=0):
        self.ep, self.ep_rank, self.ep_group = ep, ep_rank, None


def _lib_or_skip():
    from system_lab_b200.ops import cuda as cops
    try:
        cops.lib()
    except Exception as e:                                   # the library is built by __graft_entry__.build()
        pytest.skip(f"kernel library not built: {e}")
    return cops


def test_layout_regions_are_aligned_and_disjoint():
    from system_lab_b200.moe.fused_dispatch import compute_layout
    for ep, e, k, h, t, factor, fp8 in ((1, 8, 2, 256, 64, 0.0, False), (8, 128, 8, 2048, 8192, 0.0, False),
                                        (4, 256, 8, 7168, 4096, 1.25, True)):
        cap, off, total = compute_layout(ep, e, k, h, t, 128, factor, fp8)
        assert cap % 128 == 0 and cap < 1 << 24
        spans = sorted(off.values())
        assert all(o % 256 == 0 for o in spans) and spans == sorted(set(spans)) and total > spans[-1]
        for name in ("origin", "comb", "push_flag", "rows0", "rows1", "out_rows"):
            assert name in off
        worst = ep * t * min(k, e // ep)
        assert cap >= min(worst, int(factor * t * k) if (ep > 1 and factor > 0) else worst)
        # the pair-major region holds one row per (token, k) pair
        nxt = min(o for o in spans if o > off["comb"])
        assert nxt - off["comb"] >= t * k * h * 2


@pytest.mark.parametrize("keep,push", [(0.0, False), (2.0, True), (-1.0, True), (0.5, False)])
def test_construction_in_every_mode(keep, push):
    _lib_or_skip()
    from system_lab_b200.moe.fused_dispatch import FusedDispatcher, PushTarget
    d = FusedDispatcher(_Mesh(), 8, 2, 256, 64, 128, torch.device("cpu"), keep_factor=keep, push=push)
    assert d.capacity % 128 == 0 and d.rows[0].shape == (d.capacity, 256) and d.comb.shape == (64 * 2, 256)
    assert d.origin.dtype == torch.int32 and d.push == push and d._pending_push == {}
    if keep < 0:
        assert d.keep_exact and d.keep_rows == d.capacity
    elif keep > 0:
        assert not d.keep_exact and 0 < d.keep_rows <= d.capacity and d.keep_rows % 128 == 0
        assert d.keep_rows >= min(d.capacity, int(keep * 128))
    else:
        assert d.keep_rows == 0
    assert len(d._lay[0]) == 13 and d._lay[1][9] == -1 and d._lay[0][9] == d.off["origin"]
    assert isinstance(d.push_target(object()), PushTarget)
    # views alias the workspace, not copies of it
    d.rows[0][0, 0] = 3.0
    assert d.ws.buf[d.off["rows0"]:d.off["rows0"] + 2].view(torch.bfloat16)[0] == 3.0


def test_push_target_checks_width_before_launching():
    _lib_or_skip()
    from system_lab_b200.moe.fused_dispatch import FusedDispatcher
    d = FusedDispatcher(_Mesh(), 8, 2, 256, 64, 128, torch.device("cpu"), push=True)
    tgt = d.push_target(object())
    a = torch.zeros(128, 64, dtype=torch.bfloat16)
    w = torch.zeros(8, 128, 64, dtype=torch.bfloat16)           # forward output width 128 != dispatcher's 256
    with pytest.raises(ValueError, match="wide"):
        tgt.launch(0, a, w, torch.zeros(8, dtype=torch.int32), torch.zeros(8, dtype=torch.int32), 128, 64, 128)
    assert d.push_epoch == 0 and d._pending_push == {}


def test_gemm_reduce_scatter_row_table():
    """Row b * S + s of the full product belongs to the rank that holds positions [r S/w, (r+1) S/w) and lands in slot
    (local row) * world + sender of that rank's receive region: every slot of every rank is written exactly once when
    all senders are taken together."""
    from system_lab_b200.comm.gemm_rs import GemmReduceScatter
    from system_lab_b200.comm.symm import EmulatedWorld
    world, batch, seq, n = 4, 2, 16, 64
    dev = torch.device("cpu")
    emu = EmulatedWorld(GemmReduceScatter.nbytes(batch, seq, n, world), world, dev)
    ops_ = [GemmReduceScatter(None, world, r, dev, batch, seq, n, workspace=emu.workspace(r)) for r in range(world)]
    s_local = seq // world
    seen = {r: set() for r in range(world)}
    for sender, op in enumerate(ops_):
        assert op.rows == batch * seq and op.rows_local == batch * s_local
        org = op.origin.tolist()
        for row, o in enumerate(org):
            b, s = divmod(row, seq)
            dst, slot = o >> 24, o & 0xFFFFFF
            assert dst == s // s_local
            assert slot == (b * s_local + s % s_local) * world + sender
            assert slot not in seen[dst]
            seen[dst].add(slot)
    assert all(seen[r] == set(range(batch * s_local * world)) for r in range(world))
    with pytest.raises(ValueError, match="multiple"):
        GemmReduceScatter(None, 3, 0, dev, 1, 16, 64, workspace=emu.workspace(0))
