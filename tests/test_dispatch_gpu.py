"""Fused dispatch/combine kernels.  Several expert-parallel ranks are emulated on one GPU by running
each phase of the protocol for all ranks in turn (no kernel waits on a flag of a later launch)."""
import pytest
import torch

pytestmark = pytest.mark.gpu


class _Mesh:
    def __init__(self, ep, ep_rank):
        self.ep, self.ep_rank, self.ep_group = ep, ep_rank, None


def _make(world, T, K, E, H, fp8=False, factor=4.0):
    from system_lab_b200.comm.symm import EmulatedWorld
    from system_lab_b200.moe.fused_dispatch import FusedDispatcher
    dev = torch.device("cuda")
    nbytes = _workspace_bytes(world, T, K, E, H, fp8, factor)
    emu = EmulatedWorld(nbytes, world, dev)
    return [FusedDispatcher(_Mesh(world, r), E, K, H, T, 128, dev, capacity_factor=factor,
                            workspace=emu.workspace(r), fp8_payload=fp8) for r in range(world)]


def _workspace_bytes(world, T, K, E, H, fp8, factor):
    from system_lab_b200.moe.fused_dispatch import compute_layout
    return compute_layout(world, E, K, H, T, 128, factor, fp8)[2]


def _expected_layout(idx_all, world, E, pad=128):
    """For every owner: (expert_offsets, expert_counts, list of (src, pair) per row)."""
    e_local = E // world
    out = []
    for owner in range(world):
        offs, cnts, rows = [], [], {}
        acc = 0
        for j in range(e_local):
            e = owner * e_local + j
            members = []
            for src in range(world):
                flat = idx_all[src].reshape(-1).tolist()
                members += [(src, p) for p, ee in enumerate(flat) if ee == e]
            offs.append(acc)
            cnts.append(len(members))
            for i, m in enumerate(members):
                rows[acc + i] = m
            acc += (len(members) + pad - 1) // pad * pad
        out.append((offs, cnts, rows))
    return out


@pytest.mark.parametrize("world,T,K,E,H", [(1, 200, 2, 8, 256), (2, 300, 4, 16, 512), (4, 257, 8, 32, 1024),
                                           (8, 190, 8, 128, 2048)])
def test_dispatch_combine_roundtrip(world, T, K, E, H):
    from system_lab_b200.ops import cuda as cops
    torch.manual_seed(world)
    ds = _make(world, T, K, E, H)
    dev = torch.device("cuda")
    idx = [torch.stack([torch.randperm(E, device=dev)[:K] for _ in range(T)]).int() for _ in range(world)]
    x = [torch.randn(T, H, device=dev, dtype=torch.bfloat16) for _ in range(world)]
    pr = [torch.rand(T, K, device=dev) for _ in range(world)]
    pubs = [d.plan_publish(i) for d, i in zip(ds, idx)]
    plans = [d.plan_finish(*p) for d, p in zip(ds, pubs)]
    eps = [d.scatter(pl, xx, pp.contiguous(), 0) for d, pl, xx, pp in zip(ds, plans, x, pr)]
    for d, e in zip(ds, eps):
        d.wait_rows(0, e)
    torch.cuda.synchronize()
    cops.check_status()
    exp = _expected_layout([i.cpu() for i in idx], world, E)
    for owner, (offs, cnts, rows) in enumerate(exp):
        assert plans[owner].expert_offsets.tolist() == offs
        assert plans[owner].expert_counts.tolist() == cnts
        got_rows, got_sc = ds[owner].rows[0], ds[owner].scalars[0]
        for row, (src, p) in list(rows.items())[::7]:
            assert torch.equal(got_rows[row], x[src][p // K]), f"owner {owner} row {row}"
            assert got_sc[row].item() == pr[src].reshape(-1)[p].item()
        # alignment padding rows are zero
        for o, c in zip(offs, cnts):
            padded = (c + 127) // 128 * 128
            if padded > c:
                assert not got_rows[o + c:o + padded].any()
    # combine: owners publish f(row) = 2 * row content; every source pulls and sums over k
    for d in ds:
        d.out_rows.copy_((d.rows[0].float() * 2).to(torch.bfloat16))
        d.out_scalars.copy_(d.scalars[0] * 3)
    eps = [d.signal_out() for d in ds]
    for r, d in enumerate(ds):
        y = d.pull_rows(plans[r], eps[r])
        yw = d.pull_rows(plans[r], eps[r], pr[r].contiguous())
        s = d.pull_scalars(plans[r], eps[r])
        torch.cuda.synchronize()
        ref = (x[r].float() * 2 * K)
        assert torch.allclose(y.float(), ref, rtol=2e-2, atol=2e-2)
        refw = x[r].float() * 2 * pr[r].sum(1, keepdim=True)
        assert torch.allclose(yw.float(), refw, rtol=2e-2, atol=2e-2)
        assert torch.allclose(s, pr[r] * 3)
    cops.check_status()


def test_fp8_payload_matches_reference_quant():
    from system_lab_b200.ops import cuda as cops, reference as ref
    world, T, K, E, H = 2, 128, 2, 8, 512
    ds = _make(world, T, K, E, H, fp8=True)
    dev = torch.device("cuda")
    torch.manual_seed(0)
    idx = [torch.stack([torch.randperm(E, device=dev)[:K] for _ in range(T)]).int() for _ in range(world)]
    x = [torch.randn(T, H, device=dev, dtype=torch.bfloat16) * 2 for _ in range(world)]
    plans = [d.plan_finish(*p) for d, p in zip(ds, [d.plan_publish(i) for d, i in zip(ds, idx)])]
    eps = [d.scatter(pl, xx, None, 0, fp8=True) for d, pl, xx in zip(ds, plans, x)]
    for d, e in zip(ds, eps):
        d.wait_rows(0, e)
    torch.cuda.synchronize()
    cops.check_status()
    exp = _expected_layout([i.cpu() for i in idx], world, E)
    for owner, (offs, cnts, rows) in enumerate(exp):
        for row, (src, p) in list(rows.items())[::5]:
            deq = ref.dequant_1x128(ds[owner].rows_fp8[row], ds[owner].row_scales[row])
            xr = x[src][p // K].float()
            assert torch.allclose(deq, xr, rtol=0.07, atol=1e-3)


def test_missing_flag_times_out_with_status_not_hang():
    """A wait on a flag nobody sets returns within the bound and reports TIMEOUT_PEER_FLAG."""
    from system_lab_b200.ops import cuda as cops
    ds = _make(2, 64, 2, 8, 256)
    d = ds[0]
    import ctypes
    cops.register("slab_moe_wait_limit", "ppiiiipls")
    cops.call("slab_moe_wait_limit", ctypes.addressof(d._peer_ptrs), ctypes.addressof(d._lay[0]), d.ep, d.me,
              12345, 0, d.status, 50_000_000, cops.stream())        # 50 ms bound
    torch.cuda.synchronize()
    with pytest.raises(cops.DeviceHang):
        cops.check_status()
    cops.check_status()   # status word is cleared; the context is still usable
    assert torch.ones(4, device="cuda").sum().item() == 4


@pytest.mark.parametrize("world,T,K,E,H,F", [(1, 200, 2, 8, 256, 128), (2, 300, 4, 16, 512, 256), (4, 257, 8, 32, 1024, 192),
                                             (8, 150, 8, 64, 512, 128)])
def test_gemm_push_epilogue_matches_pull_combine(world, T, K, E, H, F):
    """Expert GEMMs whose epilogue pushes result rows to the token owners (forward: act @ w2^T, width H; dgrad:
    dY @ w1, width H), reduced by the owners, against an fp32 oracle on the same bf16 inputs.  Ranks are
    emulated phase by phase: every push GEMM finishes (and releases its flags) before any reduction starts."""
    from system_lab_b200.ops import cuda as cops
    torch.manual_seed(10 + world)
    ds = _make(world, T, K, E, H)
    dev = torch.device("cuda")
    e_local = E // world
    idx = [torch.stack([torch.randperm(E, device=dev)[:K] for _ in range(T)]).int() for _ in range(world)]
    x = [torch.randn(T, H, device=dev, dtype=torch.bfloat16) for _ in range(world)]
    pubs = [d.plan_publish(i) for d, i in zip(ds, idx)]
    plans = [d.plan_finish(*p) for d, p in zip(ds, pubs)]
    eps = [d.scatter(pl, xx, None, 0) for d, pl, xx in zip(ds, plans, x)]
    for d, e in zip(ds, eps):
        d.wait_rows(0, e)
    for d, pl in zip(ds, plans):
        pl.origin = d.origin
    # the origin table names the sender and the pair of every received row
    torch.cuda.synchronize()
    exp = _expected_layout([i.cpu() for i in idx], world, E)
    for owner, (offs, cnts, rows) in enumerate(exp):
        org = ds[owner].origin.cpu()
        for row, (src, p) in list(rows.items())[::5]:
            assert org[row].item() == (src << 24) | p
    # ---- forward: per-owner activations [cap, F] (zero on padding rows), weights [e_local, H, F]
    act = [torch.zeros(d.capacity, F, device=dev, dtype=torch.bfloat16) for d in ds]
    w2 = [(0.05 * torch.randn(e_local, H, F, device=dev)).to(torch.bfloat16) for _ in range(world)]
    for owner, (offs, cnts, rows) in enumerate(exp):
        for o, c in zip(offs, cnts):
            act[owner][o:o + c] = torch.randn(c, F, device=dev)
    for owner, d in enumerate(ds):
        tgt = d.push_target(plans[owner])
        tgt.launch(0, act[owner], w2[owner], plans[owner].expert_offsets, plans[owner].expert_counts, H, F, 256)
        assert d._pending_push.pop(0) == tgt.epoch == 1
    got = [d.reduce_pairs(pl, 1) for d, pl in zip(ds, plans)]
    torch.cuda.synchronize()
    cops.check_status()

    def oracle(vals, weights, transpose):
        # vals[owner][row] -> result row = vals @ W ; summed over the K pairs of every source token
        want = [torch.zeros(T, H, device=dev) for _ in range(world)]
        for owner, (offs, cnts, rows) in enumerate(exp):
            for j, (o, c) in enumerate(zip(offs, cnts)):
                if not c:
                    continue
                wj = weights[owner][j].float()
                res = vals[owner][o:o + c].float() @ (wj.t() if transpose else wj)
                res = res.to(torch.bfloat16).float()           # each pushed row is rounded to bf16 once
                for i in range(c):
                    src, p = rows[o + i]
                    want[src][p // K] += res[i]
        return want

    want = oracle(act, w2, True)
    for r in range(world):
        err = (got[r].float() - want[r]).abs().max().item()
        assert err <= 2e-2 * want[r].abs().max().item() + 1e-3, f"fwd rank {r}: {err}"
    # ---- dgrad: dY [cap, 2F'] with N = 256 columns, weights [e_local, N, H]; result width H
    N = 256
    dy = [torch.zeros(d.capacity, N, device=dev, dtype=torch.bfloat16) for d in ds]
    w1 = [(0.05 * torch.randn(e_local, N, H, device=dev)).to(torch.bfloat16) for _ in range(world)]
    for owner, (offs, cnts, rows) in enumerate(exp):
        for o, c in zip(offs, cnts):
            dy[owner][o:o + c] = torch.randn(c, N, device=dev)
    for owner, d in enumerate(ds):
        d.push_target(plans[owner]).launch(1, dy[owner], w1[owner], plans[owner].expert_offsets,
                                           plans[owner].expert_counts, N, H, 128)
        assert d._pending_push.pop(1) == 2
    got = [d.reduce_pairs(pl, 2) for d, pl in zip(ds, plans)]
    torch.cuda.synchronize()
    cops.check_status()
    want = oracle(dy, w1, False)
    for r in range(world):
        err = (got[r].float() - want[r]).abs().max().item()
        assert err <= 2e-2 * want[r].abs().max().item() + 1e-3, f"dgrad rank {r}: {err}"


def test_fit_raises_after_a_wait_that_ran_out():
    """The training loop reads the status word after every step: a bounded wait that ran out between two steps (a flag
    nothing sets, 20 ms limit; the kernel returns, nothing faults) stops ``fit`` with a typed error."""
    import ctypes
    from system_lab_b200.config import Config
    from system_lab_b200.ops import cuda as cops
    from system_lab_b200.trainer.loop import Trainer
    cfg = Config.load(preset="simplemoe-tiny", overrides=[
        "params_dtype=bf16", "device=cuda", "global_batch_size=2", "micro_batch_size=2",
        "expert_model_parallel_size=1", "moe_token_dispatcher_type=fused", "moe_pad_expert_rows_to=128",
        "train_iters=4"])
    from system_lab_b200.parallel.mesh import single_process_mesh
    tr = Trainer(cfg, mesh=single_process_mesh(), device=torch.device("cuda", 0))
    try:
        tr.fit(1)
        d = tr.engine.dispatcher
        cops.register("slab_moe_wait_limit", "ppiiiipls")
        cops.call("slab_moe_wait_limit", ctypes.addressof(d._peer_ptrs), ctypes.addressof(d._lay[0]), d.ep, d.me,
                  1 << 30, 0, d.status, 20_000_000, cops.stream())
        with pytest.raises(cops.DeviceHang, match="TIMEOUT_PEER_FLAG"):
            tr.fit(1)
        cops.check_status()                    # consumed
        tr.fit(1)                              # the context and the trainer are still usable
    finally:
        cops.clear_status()
        tr.close()


def test_out_of_range_expert_id_is_reported_not_written():
    """An expert id outside [0, E) (a corrupt expert map, logical ids passed with the wrong E) is skipped by the
    histogram and the slot assignment, its pair gets no destination and the status word says BAD_INDEX."""
    from system_lab_b200.ops import cuda as cops
    ds = _make(1, 64, 2, 8, 256)
    d = ds[0]
    idx = torch.stack([torch.randperm(8, device="cuda")[:2] for _ in range(64)]).int()
    idx[5, 1] = 8
    idx[9, 0] = -3
    plan = d.plan(idx)
    torch.cuda.synchronize()
    assert cops.peek_status() == 6
    cops.clear_status()
    loc = plan.pair_loc.cpu().view(64, 2)
    assert loc[5, 1] == -1 and loc[9, 0] == -1
    assert (loc.flatten() >= 0).sum() == 64 * 2 - 2
    assert int(plan.expert_counts.sum()) == 64 * 2 - 2


@pytest.mark.parametrize("bulk", [False, True])
@pytest.mark.parametrize("world,T,K,E,H,skew", [(1, 200, 2, 8, 256, False), (2, 300, 4, 16, 512, False),
                                                (4, 257, 8, 32, 1024, False), (4, 513, 4, 16, 2048, True),
                                                (2, 130, 4, 16, 7168, False), (8, 200, 8, 128, 2048, False)])
def test_expert_ordered_scatter_and_gemm_that_waits_per_expert(world, T, K, E, H, skew, bulk):
    """``bulk``: rows leave through bulk stores out of shared memory, 4 KB at a time (hidden 7168 makes a row three
    and a half pieces), instead of per-lane 16-byte stores; same result.

    The expert-ordered scatter writes the same rows, scalars and origins into the same places as the token-ordered
    one, releases one flag per (source, expert) -- also for pairs without rows -- and leaves its chunk counters at
    zero; a grouped GEMM handed those flags gives the fp32 oracle's result.  Ranks are emulated phase by phase (all
    scatters are enqueued before any GEMM, so no kernel waits for a later launch)."""
    from system_lab_b200.ops import cuda as cops
    from system_lab_b200.ops import reference as ref
    torch.manual_seed(20 + world)
    ds = _make(world, T, K, E, H)
    dev = torch.device("cuda")
    if skew:       # most pairs go to two experts: many chunks for some (source, expert) pairs, none for others
        idx = [torch.stack([torch.cat([torch.tensor([0, E - 1], device=dev),
                                       1 + torch.randperm(E - 2, device=dev)[:K - 2]]) for _ in range(T)]).int()
               for _ in range(world)]
    else:
        idx = [torch.stack([torch.randperm(E, device=dev)[:K] for _ in range(T)]).int() for _ in range(world)]
    x = [torch.randn(T, H, device=dev, dtype=torch.bfloat16) for _ in range(world)]
    pr = [torch.rand(T, K, device=dev) for _ in range(world)]
    plans = [d.plan_finish(*p) for d, p in zip(ds, [d.plan_publish(i) for d, i in zip(ds, idx)])]
    # the permutation groups the pairs by expert, in pair order
    for r in range(world):
        flat = idx[r].reshape(-1).cpu()
        perm, pre = plans[r].perm.cpu(), plans[r].send_prefix.cpu()
        for e in range(E):
            want = (flat == e).nonzero().flatten()
            assert torch.equal(perm[pre[e]:pre[e + 1]].long(), want)
    from system_lab_b200.moe.fused_dispatch import set_scatter_bulk
    set_scatter_bulk(bulk)
    try:
        readies = [d.scatter_ordered(pl, xx, pp.contiguous(), 0) for d, pl, xx, pp in zip(ds, plans, x, pr)]
    finally:
        set_scatter_bulk(False)
    n, e_local = 256, E // world
    w = (0.05 * torch.randn(world, e_local, n, H, device=dev)).to(torch.bfloat16)
    outs = [cops.grouped_gemm_raw(0, d.rows[0], w[r], pl.expert_offsets, pl.expert_counts, n, H, ready=rd)
            for r, (d, pl, rd) in enumerate(zip(ds, plans, readies))]
    torch.cuda.synchronize()
    cops.check_status()
    exp = _expected_layout([i.cpu() for i in idx], world, E)
    for owner, (offs, cnts, rows) in enumerate(exp):
        d = ds[owner]
        assert readies[owner].consumed
        assert bool((d.eflags[0] >= readies[owner].epoch).all()), "a (source, expert) flag was never released"
        assert int(d.chunk_done.abs().sum()) == 0
        got_rows, got_sc, org = d.rows[0], d.scalars[0], d.origin.cpu()
        for row, (src, p) in list(rows.items())[::1 if bulk else 5]:
            assert torch.equal(got_rows[row], x[src][p // K]), f"owner {owner} row {row}"
            assert got_sc[row].item() == pr[src].reshape(-1)[p].item()
            assert org[row].item() == (src << 24) | p
        for o, c in zip(offs, cnts):
            padded = (c + 127) // 128 * 128
            if padded > c:
                assert not got_rows[o + c:o + padded].any()
        want = ref.grouped_gemm(got_rows, w[owner], plans[owner].expert_offsets, plans[owner].expert_counts)
        for o, c in zip(offs, cnts):
            err = (outs[owner][o:o + c].float() - want[o:o + c].float()).abs().max().item() if c else 0.0
            assert err < 2e-2 * (want.float().abs().max().item() + 1e-6)


def test_gemm_that_waits_for_rows_gives_up_with_a_status_code():
    """Per-expert arrival flags nobody sets (epoch far in the future), 30 ms limit: the producer warp's wait runs out,
    the kernel unwinds (no copy was issued, the accumulators are released) and the status word says so."""
    from system_lab_b200.ops import cuda as cops
    ds = _make(2, 64, 2, 8, 256)
    d = ds[0]
    idx = torch.stack([torch.randperm(8, device="cuda")[:2] for _ in range(64)]).int()
    plans = [dd.plan_finish(*p) for dd, p in zip(ds, [dd.plan_publish(idx) for dd in ds])]   # publish all, then finish all
    torch.cuda.synchronize()
    cops.check_status()
    rdy = d.scatter_ordered(plans[0], torch.randn(64, 256, device="cuda", dtype=torch.bfloat16), None, 0)
    ds[1].scatter_ordered(plans[1], torch.randn(64, 256, device="cuda", dtype=torch.bfloat16), None, 0)
    rdy.epoch = 1 << 30
    w = torch.zeros(4, 128, 256, device="cuda", dtype=torch.bfloat16)
    cops.register("slab_moe_set_wait_limit_ms", "l")
    cops.lib().slab_moe_set_wait_limit_ms(30)
    try:
        cops.grouped_gemm_raw(0, d.rows[0], w, plans[0].expert_offsets, plans[0].expert_counts, 128, 256, ready=rdy)
        torch.cuda.synchronize()
        assert cops.peek_status() == 5
    finally:
        cops.lib().slab_moe_set_wait_limit_ms(60000)
        cops.clear_status()
    w.fill_(1.0)
    out = cops.grouped_gemm_raw(0, d.rows[0], w, plans[0].expert_offsets, plans[0].expert_counts, 128, 256)
    torch.cuda.synchronize()
    cops.check_status()                     # the next launch on the same context is healthy
    o0, c0 = int(plans[0].expert_offsets[0]), int(plans[0].expert_counts[0])
    want = d.rows[0][o0:o0 + c0].float().sum(-1, keepdim=True).expand(c0, 128)
    assert torch.allclose(out[o0:o0 + c0].float(), want, rtol=2e-2, atol=0.25)


def test_kept_dispatch_falls_back_when_the_copy_is_too_small():
    """Selective recompute with a fixed-size copy of the dispatched rows: a copy that holds the rows is reused in the
    recomputed block, a copy that is too small makes every layer dispatch again (decided from the plan's row count,
    which reaches the host through a pinned buffer); either way the losses equal those of the run that keeps nothing."""
    from system_lab_b200.config import Config
    from system_lab_b200.ops import cuda as cops
    from system_lab_b200.parallel.mesh import single_process_mesh
    from system_lab_b200.trainer.loop import Trainer
    curves, fallbacks = {}, {}
    for factor in (0.0, 1.5, 0.5):          # 0.5 stands for "too small": its copy is cut to one tile of rows below
        cfg = Config.load(preset="simplemoe-tiny", overrides=[
            "params_dtype=bf16", "device=cuda", "global_batch_size=2", "micro_batch_size=2",
            "expert_model_parallel_size=1", "moe_token_dispatcher_type=fused", "moe_pad_expert_rows_to=128",
            "recompute_granularity=selective", f"moe_keep_dispatched_factor={factor}"])
        tr = Trainer(cfg, mesh=single_process_mesh(), device=torch.device("cuda", 0))
        try:
            if factor == 0.5:
                tr.engine.dispatcher.keep_rows = 128
            curves[factor] = [float(tr.train_step()["loss"]) for _ in range(3)]
            torch.cuda.synchronize()
            cops.check_status()
            fallbacks[factor] = tr.engine.dispatcher.keep_fallbacks
        finally:
            tr.close()
    assert curves[1.5] == pytest.approx(curves[0.0], rel=1e-3, abs=1e-3)
    assert curves[0.5] == pytest.approx(curves[0.0], rel=1e-3, abs=1e-3)
    assert fallbacks[1.5] == 0 and fallbacks[0.5] > 0
