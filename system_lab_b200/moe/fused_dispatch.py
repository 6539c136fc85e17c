"""Fused dispatch / combine over peer memory (kernels in ``csrc/dispatch.cu``).

Same primitives and receiver layout as :class:`~system_lab_b200.moe.dispatch.AllToAllDispatcher`,
but rows move once, written by the sender straight into the owner's expert-major buffer (forward
dispatch, backward of combine) or pulled and reduced by the token's owner (forward combine, backward of
dispatch).  Nothing is read back to the host: segment offsets and counts stay on the device and buffers
are sized by capacity (host syncs on ``tokens_per_expert`` cost the reference 20-100 ms per iteration,
``notes/2026-04/2026-04-21_gptoss_10_moe_fp8_grouped_gemm_diagnosis.md:93-99``).

Buffers are views of the symmetric workspace and are reused by the next call of the same kind:
``dispatch`` outputs stay valid until the next forward ``dispatch``, ``combine`` gradients until the
next backward of ``combine``.  That is exactly the lifetime a layer needs when it is recomputed in
backward; callers that keep activations across layers must ask for copies (``clone_outputs=True``).

All ranks must issue the same sequence of calls: flags carry a call counter (epoch).
"""
from __future__ import annotations

import ctypes
import os
from dataclasses import dataclass

import torch

from ..comm.symm import SymmetricWorkspace
from ..ops import cuda as cops

for _name, _sig in {
    "slab_moe_count_blocks": "i",
    "slab_moe_count_publish": "piippppiiips",
    "slab_moe_plan_slots": "piip" + "pp" + "iii" + "ii" + "pppppp" + "pppp" + "s",
    "slab_moe_scatter": "pppp" + "iii" + "pp" + "iii" + "pp" + "iii" + "p" + "i" + "s",
    "slab_moe_wait": "ppiiiips",
    "slab_moe_scatter_sorted": "pppp" + "pppp" + "iiii" + "pp" + "iii" + "pp" + "iii" + "p" + "ii" + "s",
    "slab_moe_wait_experts": "ppiiiips",
    "slab_moe_set_scatter_bulk": "i",
    "slab_moe_signal_out": "ppiiis",
    "slab_moe_combine": "pppiiippiiipis",
    "slab_moe_combine_scalars": "ppippiiips",
    "slab_moe_reduce_pairs": "ppiiippiiipis",
    "slab_moe_check_rows": "pipps",
    "slab_grouped_gemm_bf16_push": "ipppp" + "iiii" + "ii" + "pp" + "ll" + "iiii" + "pp" + "s",
}.items():
    cops.register(_name, _sig)


def set_scatter_bulk(on: bool) -> None:
    """Expert-ordered bf16 scatter: send rows with bulk stores out of shared memory (``cp.async.bulk``) instead of
    per-lane 16-byte stores.  A setting of the kernel library, shared by every dispatcher of the process."""
    cops.lib().slab_moe_set_scatter_bulk(1 if on else 0)


def _align(x: int, a: int = 256) -> int:
    return (x + a - 1) // a * a


def compute_layout(ep: int, num_experts: int, topk: int, hidden: int, max_tokens: int, pad: int,
                   capacity_factor: float, fp8_payload: bool):
    """Capacity (rows) and the byte offsets of every workspace region; ``(capacity, offsets, nbytes)``.

    ``capacity_factor <= 0`` sizes for the dropless worst case (every token of every rank picks this rank's
    experts: nothing can overflow, whatever the router does).  A positive factor sizes for that multiple of
    the balanced load instead; overflow is then detected by the plan kernel and reported as ``CAPACITY``."""
    e_local = num_experts // ep
    pairs = max_tokens * topk
    worst = ep * max_tokens * min(topk, e_local)
    want = int(capacity_factor * pairs) if (ep > 1 and capacity_factor > 0) else worst
    cap = _align(min(worst, want) + e_local * pad, pad)
    if cap >= 1 << 24:
        raise ValueError("capacity exceeds the 24-bit row field of pair_loc")
    off, cur = {}, 0
    # channel 0 = forward rows, channel 1 = rows of the backward of combine
    for name, nbytes in (("counts_all", ep * num_experts * 4), ("counts_flag", ep * 4), ("data_flag0", ep * 4),
                         ("data_flag1", ep * 4), ("out_flag", ep * 4), ("rows0", cap * hidden * 2),
                         ("rows1", cap * hidden * 2),
                         ("row_scales", cap * (hidden // 128) * 4 if fp8_payload else 256),
                         ("scalars0", cap * 4), ("scalars1", cap * 4), ("out_rows", cap * hidden * 2),
                         ("out_scalars", cap * 4), ("origin", cap * 4), ("comb", pairs * hidden * 2),
                         ("push_flag", ep * 4), ("eflag0", num_experts * 4), ("eflag1", num_experts * 4)):
        off[name] = cur
        cur = _align(cur + nbytes)
    return cap, off, cur


@dataclass
class FusedPlan:
    num_tokens: int
    topk: int
    num_experts: int
    ep: int
    pad_to: int
    capacity: int
    expert_offsets: torch.Tensor      # [E_local] int32 (device)
    expert_counts: torch.Tensor       # [E_local] int32 (device)
    pair_loc: torch.Tensor            # [T*K] int32: (owner << 24) | row
    meta: torch.Tensor                # [4] int32: rows used on this rank
    tokens_per_expert_global: torch.Tensor   # [E] pairs routed from this rank
    num_rows: int                     # == capacity (host-side bound)
    origin: torch.Tensor | None = None       # [capacity] int32: (source rank << 24) | pair index of received rows
    send_prefix: torch.Tensor | None = None  # [E + 1] int32: start of every expert's run in `perm`
    item_prefix: torch.Tensor | None = None  # [E + 1] int32: scatter work items before each position of the send order
    perm: torch.Tensor | None = None         # [T*K] int32: pair indices grouped by expert (pair order inside an expert)
    ready: "ReadyFlags | None" = None        # arrival flags of the forward rows while their consumer has not waited yet
    defer_ready: bool = False                # the consumer of the forward rows (expert GEMM) does the waiting

    @property
    def e_local(self) -> int:
        return self.num_experts // self.ep


class ReadyFlags:
    """Arrival flags of the rows one expert-ordered scatter is delivering to this rank: ``flags[s, j] >= epoch`` once
    source ``s`` has written all its rows of local expert ``j``.  Handed to the grouped GEMM that consumes the rows
    (it waits expert by expert inside the kernel); any other consumer calls :meth:`wait` first."""

    def __init__(self, d: "FusedDispatcher", channel: int, epoch: int):
        self.d, self.channel, self.epoch = d, channel, epoch
        self.flags = d.eflags[channel]
        self.world = d.ep
        self.consumed = False
        self.gemm_max_ctas = 0               # > 0: SMs the consuming GEMM may take (the rest run the held-back scatter)

    def mark_consumed(self) -> None:
        self.consumed = True

    def wait(self) -> None:
        """One small kernel that waits for every (source, expert) flag: afterwards every row has arrived."""
        if not self.consumed:
            d = self.d
            d.join_side()                    # a held-back remote half must be under way before anything waits for rows
            cops.call("slab_moe_wait_experts", ctypes.addressof(d._peer_ptrs), ctypes.addressof(d._lay[self.channel]),
                      d.ep, d.me, d.E // d.ep, self.epoch, d.status, cops.stream())
            self.consumed = True


class FusedDispatcher:
    def __init__(self, mesh, num_experts: int, topk: int, hidden: int, max_tokens: int, pad_to: int = 128,
                 device=None, dtype=torch.bfloat16, capacity_factor: float = 0.0, workspace=None,
                 ep: int | None = None, ep_rank: int | None = None, fp8_payload: bool = False,
                 clone_outputs: bool = False, push: bool = False, keep_factor: float = 0.0):
        self.E, self.K, self.H, self.T = num_experts, topk, hidden, max_tokens
        self.ep = mesh.ep if ep is None else ep
        self.me = mesh.ep_rank if ep_rank is None else ep_rank
        self.pad = max(pad_to, 1)
        self.device = device
        self.dtype = dtype
        self.fp8 = fp8_payload
        self.clone_outputs = clone_outputs
        # push: expert GEMM epilogues write result rows straight into the token owners' memory (see PushTarget)
        self.push = push
        self.push_epoch = 0
        self._pending_push = {}           # GEMM mode (0 fwd / 1 dgrad) -> push epoch not yet reduced by its consumer
        # debug aid (SLAB_POISON=1): fill the receive regions with NaN patterns at the points where the protocol says
        # nobody reads or writes them, so a row consumed without having been written this round, or a flag that let a
        # reader through early, shows up as a NaN loss instead of a plausible number
        self.poison = os.environ.get("SLAB_POISON", "0") == "1"
        if dtype != torch.bfloat16:
            raise ValueError("the fused dispatcher moves bf16 rows")
        self.capacity, off, cur = compute_layout(self.ep, num_experts, topk, hidden, max_tokens, self.pad,
                                                  capacity_factor, fp8_payload)
        cap, H = self.capacity, hidden
        pairs = max_tokens * topk
        self.off = off
        self.nbytes = cur
        if workspace is None:
            workspace = SymmetricWorkspace(cur, mesh.ep_group if self.ep > 1 else None, self.ep, self.me, device)
        self.ws = workspace
        self._peer_ptrs = (ctypes.c_long * 16)(*(list(workspace.ptrs) + [0] * (16 - len(workspace.ptrs))))
        self._lay = [self._layout(0), self._layout(1)]
        self.epoch = 0
        # Rows a recomputed block keeps of its first dispatch.  keep_factor > 0: a fixed copy of that multiple of
        # the balanced per-rank load (no host sync; more rows in use than the copy holds is reported as CAPACITY);
        # keep_factor < 0: exactly the rows in use, read back from the plan (one host sync per layer and forward
        # pass, nothing can overflow); 0: never.
        self.keep_exact = keep_factor < 0
        self.keep_rows = cap if self.keep_exact else 0
        if keep_factor > 0:
            self.set_keep_rows(int(keep_factor * pairs))
        # fixed-size copies: whether every rank's rows fitted is known on every rank from the plan (meta[1], the most
        # rows any rank receives); it reaches the host through a pinned ring filled on a copy stream, read when the
        # recomputed block needs it.  A layer whose rows did not fit is dispatched again, on every rank alike.
        self.keep_fallbacks = 0
        self._fits_host = self._fits_stream = None
        self._fits_next = 0
        self.rows_seen = torch.zeros(1, dtype=torch.int32, device=device)
        n_blocks = max(cops.lib().slab_moe_count_blocks(pairs), 1)
        i32 = dict(dtype=torch.int32, device=device)
        self.block_hist = torch.zeros(n_blocks * num_experts, **i32)
        self.send_counts = torch.zeros(num_experts, **i32)
        self.send_base = torch.zeros(num_experts, **i32)
        self.done_counter = torch.zeros(1, **i32)
        self.chunk_done = torch.zeros(num_experts, **i32)       # expert-ordered scatter: finished chunks per expert
        self.status = cops.status_word(device)
        # expert_ordered: rows are sent expert by expert with one completion flag per (source, expert), and the expert
        # GEMM that consumes them waits per expert inside the kernel (no wait for the whole exchange in between)
        self.expert_ordered = True
        # overlap: with real peers the remote half of a scatter runs on a side stream beside the consuming GEMM (the
        # local half goes first on the compute stream; the GEMM waits only on flags other GPUs set)
        self.overlap = False
        self.overlap_sms = 16             # SMs the consuming GEMM leaves to the remote half of the scatter
        self.sm_count = (torch.cuda.get_device_properties(device).multi_processor_count
                         if (device is not None and torch.device(device).type == "cuda" and torch.cuda.is_available())
                         else 148)
        self._side = None
        self._deferred = None
        self._bwd_ready = None
        # typed views of this rank's regions
        self.rows = [workspace.view(off["rows0"], (cap, H), torch.bfloat16),
                     workspace.view(off["rows1"], (cap, H), torch.bfloat16)]
        self.scalars = [workspace.view(off["scalars0"], (cap,), torch.float32),
                        workspace.view(off["scalars1"], (cap,), torch.float32)]
        self.out_rows = workspace.view(off["out_rows"], (cap, H), torch.bfloat16)
        self.out_scalars = workspace.view(off["out_scalars"], (cap,), torch.float32)
        self.origin = workspace.view(off["origin"], (cap,), torch.int32)
        self.comb = workspace.view(off["comb"], (pairs, H), torch.bfloat16)
        self.push_counter = torch.zeros(1, **i32)
        self.eflags = [workspace.view(off["eflag0"], (self.ep, num_experts // self.ep), torch.int32),
                       workspace.view(off["eflag1"], (self.ep, num_experts // self.ep), torch.int32)]
        if fp8_payload:
            self.rows_fp8 = workspace.view(off["rows0"], (cap, H), torch.float8_e4m3fn)
            self.row_scales = workspace.view(off["row_scales"], (cap, H // 128), torch.float32)

    def _layout(self, channel: int):
        o = self.off
        vals = [o["counts_all"], o["counts_flag"], o[f"data_flag{channel}"], o["out_flag"], o[f"rows{channel}"],
                o["row_scales"], o[f"scalars{channel}"], o["out_rows"], o["out_scalars"],
                o["origin"] if channel == 0 else -1,       # only forward rows are ever pushed back
                o["comb"], o["push_flag"], o[f"eflag{channel}"]]
        return (ctypes.c_long * 13)(*vals)

    def _next_epoch(self) -> int:
        self.epoch += 1
        return self.epoch

    # ---- plan ----------------------------------------------------------------------------------
    @torch.no_grad()
    def plan_publish(self, topk_idx: torch.Tensor):
        """Phase 1 (sets flags): histogram and publish this rank's counts."""
        idx = topk_idx.to(torch.int32).contiguous()
        t, k = idx.shape
        if t > self.T or k != self.K:
            raise ValueError(f"plan for {t}x{k} pairs exceeds the dispatcher's {self.T}x{self.K}")
        ep = self._next_epoch()
        if self.poison:
            # forward rows: their last readers (this rank's GEMMs of the previous layer) are earlier in this stream, and
            # no peer writes them before it has seen the counts published below
            self.rows[0].view(torch.int16).fill_(-1)
            self.scalars[0].fill_(float("nan"))
        cops.call("slab_moe_count_publish", idx, t * k, self.E, self.block_hist, self.send_counts,
                  ctypes.addressof(self._peer_ptrs), ctypes.addressof(self._lay[0]), self.ep, self.me, ep,
                  self.status, cops.stream())
        return idx, ep

    @torch.no_grad()
    def plan_finish(self, idx: torch.Tensor, ep: int) -> FusedPlan:
        """Phase 2 (waits on flags): segments, send bases and the destination row of every pair."""
        t, k = idx.shape
        e_local = self.E // self.ep
        i32 = dict(dtype=torch.int32, device=self.device)
        expert_offsets = torch.empty(e_local, **i32)
        expert_counts = torch.empty(e_local, **i32)
        meta = torch.zeros(4, **i32)
        pair_loc = torch.empty(t * k, **i32)
        prefixes = torch.empty(2, self.E + 1, **i32)
        perm = torch.empty(t * k, **i32)
        cops.call("slab_moe_plan_slots", idx, t * k, self.E, self.block_hist, ctypes.addressof(self._peer_ptrs),
                  ctypes.addressof(self._lay[0]), self.ep, self.me, ep, self.pad, self.capacity, expert_offsets,
                  expert_counts, self.send_base, meta, pair_loc, self.status, self.send_counts, prefixes[0],
                  prefixes[1], perm, cops.stream())
        if self.poison:
            # result regions: every peer has published this layer's counts, so it has finished pulling / pushing the
            # previous layer's results; the next writers (this rank's GEMM, the peers' push epilogues) come later
            self.out_rows.view(torch.int16).fill_(-1)
            self.comb.view(torch.int16).fill_(-1)
        return FusedPlan(t, k, self.E, self.ep, self.pad, self.capacity, expert_offsets, expert_counts, pair_loc,
                         meta, self.send_counts.clone(), self.capacity, send_prefix=prefixes[0],
                         item_prefix=prefixes[1], perm=perm)

    def plan(self, topk_idx: torch.Tensor) -> FusedPlan:
        idx, ep = self.plan_publish(topk_idx)
        return self.plan_finish(idx, ep)

    # ---- raw phases (also used one by one by the single-GPU multi-rank emulation) ------------------
    def scatter(self, plan: FusedPlan, x, scalars, channel: int, scale_in=None, fp8: bool = False) -> int:
        ep = self._next_epoch()
        cops.call("slab_moe_scatter", x, scalars, scale_in, plan.pair_loc, plan.num_tokens, plan.topk, self.H,
                  ctypes.addressof(self._peer_ptrs), ctypes.addressof(self._lay[channel]), self.ep, self.me, ep,
                  plan.expert_offsets, plan.expert_counts, plan.e_local, self.pad, 1 if fp8 else 0,
                  self.done_counter, 0, cops.stream())
        return ep

    def scatter_ordered(self, plan: FusedPlan, x, scalars, channel: int, scale_in=None, fp8: bool = False) -> ReadyFlags:
        """Expert-ordered scatter (``csrc/dispatch.cu: moe_scatter_sorted_kernel``); returns the arrival flags the
        consumer of this rank's receive buffer has to honour.

        With ``overlap`` (real peers only) the exchange runs beside the expert GEMM that consumes it.  A persistent
        GEMM block takes a whole SM's shared memory, so nothing else can share an SM with it: the two kernels get
        disjoint SMs instead.  The rows for this rank are written now, on the compute stream; the rows for the peers
        are held back until the consumer has been launched on ``sm_count - overlap_sms`` SMs (``ReadyFlags.
        gemm_max_ctas``), then :meth:`join_side` launches them on a side stream, sized to fit the SMs left over, and
        makes the compute stream wait for that stream.  Every rank's GEMM waits only for flags that other GPUs'
        scatters set, and every rank's scatter always has SMs of its own, so the exchange cannot wait for itself."""
        ep = self._next_epoch()

        def launch(part: int, n_blocks: int = 0) -> None:
            cops.call("slab_moe_scatter_sorted", x, scalars, scale_in, plan.pair_loc, plan.perm,
                      plan.tokens_per_expert_global, plan.send_prefix, plan.item_prefix, plan.num_tokens, plan.topk,
                      self.H, self.E, ctypes.addressof(self._peer_ptrs), ctypes.addressof(self._lay[channel]), self.ep,
                      self.me, ep, plan.expert_offsets, plan.expert_counts, plan.e_local, self.pad, 1 if fp8 else 0,
                      self.chunk_done, part, n_blocks, cops.stream())

        rdy = ReadyFlags(self, channel, ep)
        if self.overlap and self.ep > 1 and self.device is not None and torch.device(self.device).type == "cuda":
            self.join_side()                              # a previous exchange nobody joined yet
            launch(2)                                     # this rank's own rows: the consumer finds them in stream order
            ev = torch.cuda.Event()
            ev.record(torch.cuda.current_stream(self.device))
            keep = [t for t in (x, scalars, scale_in) if isinstance(t, torch.Tensor)]
            self._deferred = (lambda: launch(1, self.overlap_sms * self.SCATTER_CTAS_PER_SM), ev, keep)
            rdy.gemm_max_ctas = max(self.sm_count - self.overlap_sms, 1)
        else:
            launch(0)
        return rdy

    SCATTER_CTAS_PER_SM = 3          # 256-thread blocks of the scatter kernel one SM holds (80 registers per thread)

    def join_side(self) -> None:
        """Launch the held-back remote half of the last scatter on the side stream (it starts after this rank's own
        rows were written, not after what the compute stream has enqueued since) and make the compute stream wait
        for it.  Call right after the consumer of the received rows has been launched."""
        pending = getattr(self, "_deferred", None)
        if pending is None:
            return
        self._deferred = None
        fn, ev, keep = pending
        if self._side is None:
            self._side = torch.cuda.Stream(device=self.device)
        main = torch.cuda.current_stream(self.device)
        self._side.wait_event(ev)
        for t in keep:                                    # inputs stay allocated until the side stream has read them
            t.record_stream(self._side)
        with torch.cuda.stream(self._side):
            fn()
        main.wait_stream(self._side)

    def take_bwd_ready(self):
        """Arrival flags of the gradient rows the last backward of combine is delivering (None if it already waited)."""
        r, self._bwd_ready = self._bwd_ready, None
        return r

    def wait_rows(self, channel: int, ep: int) -> None:
        cops.call("slab_moe_wait", ctypes.addressof(self._peer_ptrs), ctypes.addressof(self._lay[channel]), self.ep,
                  self.me, ep, 0, self.status, cops.stream())

    def signal_out(self) -> int:
        ep = self._next_epoch()
        cops.call("slab_moe_signal_out", ctypes.addressof(self._peer_ptrs), ctypes.addressof(self._lay[0]), self.ep,
                  self.me, ep, cops.stream())
        return ep

    def pull_rows(self, plan: FusedPlan, ep: int, weights=None) -> torch.Tensor:
        y = torch.empty(plan.num_tokens, self.H, dtype=torch.bfloat16, device=self.device)
        cops.call("slab_moe_combine", y, weights, plan.pair_loc, plan.num_tokens, plan.topk, self.H,
                  ctypes.addressof(self._peer_ptrs), ctypes.addressof(self._lay[0]), self.ep, self.me, ep,
                  self.status, 0, cops.stream())
        return y

    def pull_scalars(self, plan: FusedPlan, ep: int) -> torch.Tensor:
        s = torch.empty(plan.num_tokens * plan.topk, dtype=torch.float32, device=self.device)
        cops.call("slab_moe_combine_scalars", s, plan.pair_loc, plan.num_tokens * plan.topk,
                  ctypes.addressof(self._peer_ptrs), ctypes.addressof(self._lay[0]), self.ep, self.me, ep,
                  self.status, cops.stream())
        return s.view(plan.num_tokens, plan.topk)

    def reduce_pairs(self, plan: FusedPlan, push_epoch: int) -> torch.Tensor:
        """Sum of the K rows the owners pushed for every token (waits for all owners' push flags)."""
        y = torch.empty(plan.num_tokens, self.H, dtype=torch.bfloat16, device=self.device)
        cops.call("slab_moe_reduce_pairs", y, plan.pair_loc, plan.num_tokens, plan.topk, self.H,
                  ctypes.addressof(self._peer_ptrs), ctypes.addressof(self._lay[0]), self.ep, self.me, push_epoch,
                  self.status, 0, cops.stream())
        return y

    def set_keep_rows(self, rows_in_use: int) -> int:
        """Size the kept copy for ``rows_in_use`` received rows (plus per-expert alignment padding)."""
        e_local = self.E // self.ep
        want = rows_in_use + e_local * self.pad
        self.keep_rows = min(self.capacity, (want + self.pad - 1) // self.pad * self.pad)
        return self.keep_rows

    def keep_dispatched(self, plan: FusedPlan, xe: torch.Tensor, pe: torch.Tensor | None):
        """Copies of the received rows and gate probabilities for a later ``redispatch_kept``: exactly the rows in
        use (``keep_exact``) or the first ``keep_rows`` (more rows in use is reported as CAPACITY through the status
        word).  The plan is made self-contained (its origin table no longer aliases the workspace)."""
        if self.keep_exact:
            used = int(plan.meta[0].item())               # host sync: rows in use on this rank (padded segments)
            n = min(max(used, self.pad), self.capacity)
        else:
            n = self.keep_rows
            cops.call("slab_moe_check_rows", plan.meta, 0, self.status, self.rows_seen, cops.stream())   # high-water mark only
            plan.kept_fits = self._fits_ticket(plan)
        plan.origin = self.origin[:n].clone() if self.keep_exact else self.origin.clone()
        return xe[:n].clone(), (pe[:n].clone() if pe is not None else None)

    def _fits_ticket(self, plan: FusedPlan):
        """Start the copy of ``plan.meta[1]`` (most rows on any rank) to the host; ``(slot, event)``."""
        if torch.device(self.device).type != "cuda":
            return None
        if self._fits_host is None:
            self._fits_host = torch.zeros(1024, dtype=torch.int32).pin_memory()
            self._fits_stream = torch.cuda.Stream(device=self.device)
        slot = self._fits_next % self._fits_host.numel()
        self._fits_next += 1
        self._fits_stream.wait_stream(torch.cuda.current_stream(self.device))
        ev = torch.cuda.Event()
        with torch.cuda.stream(self._fits_stream):
            self._fits_host[slot:slot + 1].copy_(plan.meta[1:2], non_blocking=True)
            ev.record(self._fits_stream)
        return slot, ev

    def kept_rows_fit(self, plan: FusedPlan) -> bool:
        """Whether the fixed-size copy taken in the first run holds every rank's rows of this layer (the same answer
        on every rank).  Waits, on the host, until the device has got as far as that run's plan: in backward that is
        the past, except for the first layer it is asked about."""
        if self.keep_exact:
            return True
        t = getattr(plan, "kept_fits", None)
        if t is None:
            return True
        slot, ev = t
        ev.synchronize()
        ok = int(self._fits_host[slot]) <= self.keep_rows
        if not ok:
            self.keep_fallbacks += 1
        return ok

    def redispatch_kept(self, plan: FusedPlan, x: torch.Tensor, probs: torch.Tensor | None, xs: torch.Tensor,
                        ps: torch.Tensor | None):
        """Differentiable stand-in for ``dispatch`` that moves nothing forward: returns the kept rows; its
        backward is the backward of ``dispatch`` (gradients of the rows travel back to the tokens)."""
        return _FusedKept.apply(x, probs, xs, ps, self, plan)

    def push_target(self, plan: FusedPlan) -> "PushTarget":
        return PushTarget(self, plan)

    def stage_out_rows(self, ye: torch.Tensor) -> None:
        if ye.data_ptr() != self.out_rows.data_ptr():
            self.out_rows[:ye.shape[0]].copy_(ye)

    def expert_output_buffer(self) -> torch.Tensor:
        """Where the last expert GEMM should write so that combine needs no staging copy."""
        return self.out_rows

    # ---- differentiable API ------------------------------------------------------------------------
    def dispatch(self, plan: FusedPlan, x: torch.Tensor, probs: torch.Tensor | None):
        """Returns ``(xe [capacity, H], pe [capacity] or None)``."""
        return _FusedDispatch.apply(x, probs, self, plan)

    def dispatch_rows(self, plan, x):
        return self.dispatch(plan, x, None)[0]

    def dispatch_scalars(self, plan, p):
        raise NotImplementedError("use dispatch(plan, x, probs): rows and gate probabilities travel together")

    def combine_rows(self, plan: FusedPlan, ye: torch.Tensor, weights: torch.Tensor | None = None,
                     dead: bool = False, defer_bwd: bool = False):
        """``dead``: only the autograd node is wanted (recomputed forward whose result nobody reads): no signal, no
        wait, no pull; the returned values are unspecified.  Every rank of the group must pass the same flag.
        ``defer_bwd``: in backward, hand the arrival flags of the gradient rows to the consumer (the expert GEMM that
        produced ``ye`` calls :meth:`take_bwd_ready`) instead of waiting for the whole exchange here."""
        return _FusedCombine.apply(ye, weights, self, plan, dead and weights is None, defer_bwd)


class PushTarget:
    """Destination of an expert GEMM whose epilogue pushes every result row to the rank that owns the row's
    token (``csrc/gemm_tcgen05.cu``, PUSH epilogue).  Passed as ``out=`` (second expert GEMM, forward combine)
    or ``dgrad_out=`` (first expert GEMM, backward of dispatch) of ``ops.grouped_linear``.  ``launch`` runs the
    GEMM and records the push epoch the matching ``reduce_pairs`` has to wait for."""

    def __init__(self, d: "FusedDispatcher", plan: FusedPlan):
        self.d, self.plan = d, plan
        self.epoch = 0

    def launch(self, mode: int, a: torch.Tensor, b: torch.Tensor, offsets, counts, n: int, k: int, block_n: int):
        d = self.d
        out_cols = n if mode == 0 else k
        if out_cols != d.H:
            raise ValueError(f"pushed rows are {out_cols} wide, the dispatcher moves {d.H}")
        d.push_epoch += 1
        self.epoch = d.push_epoch
        d._pending_push[mode] = self.epoch
        cops.call("slab_grouped_gemm_bf16_push", mode, a, b, offsets, counts, offsets.numel(), a.shape[0], n, k,
                  block_n, 0, self.plan.origin, ctypes.addressof(d._peer_ptrs), d.off["comb"], d.off["push_flag"],
                  d.ep, d.me, self.epoch, d.T * d.K, d.push_counter, d.status, cops.stream())


class _FusedDispatch(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, probs, d: FusedDispatcher, plan: FusedPlan):
        ctx.d, ctx.plan, ctx.has_probs = d, plan, probs is not None
        xc = x.contiguous()
        pc = probs.float().contiguous() if probs is not None else None
        plan.ready = None
        if d.expert_ordered and plan.perm is not None:
            rdy = d.scatter_ordered(plan, xc, pc, channel=0)
            if d.clone_outputs or not getattr(plan, "defer_ready", False):
                rdy.wait()                       # the caller reads the rows itself
                d.join_side()
            else:
                plan.ready = rdy                 # the expert GEMM waits expert by expert
        else:
            ep = d.scatter(plan, xc, pc, channel=0)
            d.wait_rows(0, ep)
        xe, pe = d.rows[0], d.scalars[0]
        plan.origin = d.origin
        if d.clone_outputs:
            xe, pe = xe.clone(), pe.clone()
            plan.origin = d.origin.clone()
        return xe, (pe if probs is not None else None)

    @staticmethod
    def backward(ctx, g_xe, g_pe):
        return _dispatch_backward(ctx, g_xe, g_pe) + (None, None)


def _dispatch_backward(ctx, g_xe, g_pe):
    """Gradients of the dispatched rows (and of the per-row gate probabilities) travel back to the tokens."""
    d, plan = ctx.d, ctx.plan
    pushed = d._pending_push.pop(1, None)             # epoch if the fc1 dgrad already pushed its rows to the owners
    if pushed is None:
        d.stage_out_rows(g_xe.contiguous())
    if ctx.has_probs and g_pe is not None:
        d.out_scalars[:g_pe.shape[0]].copy_(g_pe)
    ep = d.signal_out()
    gx = d.reduce_pairs(plan, pushed) if pushed is not None else d.pull_rows(plan, ep)
    gp = d.pull_scalars(plan, ep) if (ctx.has_probs and g_pe is not None) else None
    return gx, gp


class _FusedKept(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, probs, xs, ps, d: FusedDispatcher, plan: FusedPlan):
        ctx.d, ctx.plan, ctx.has_probs = d, plan, probs is not None
        return xs.view_as(xs), (ps.view_as(ps) if (probs is not None and ps is not None) else None)

    @staticmethod
    def backward(ctx, g_xe, g_pe):
        return _dispatch_backward(ctx, g_xe, g_pe) + (None, None, None, None)


class _FusedCombine(torch.autograd.Function):
    @staticmethod
    def forward(ctx, ye, weights, d: FusedDispatcher, plan: FusedPlan, dead: bool = False, defer_bwd: bool = False):
        ctx.d, ctx.plan = d, plan
        ctx.defer_bwd = defer_bwd
        if weights is not None:
            weights = weights.float().contiguous()
            ctx.save_for_backward(weights)
        ctx.weighted = weights is not None
        ctx.ye_rows = ye.shape[0]
        if dead:
            return torch.empty(plan.num_tokens, d.H, dtype=torch.bfloat16, device=d.device)
        pushed = d._pending_push.pop(0, None)             # epoch if the fc2 GEMM already pushed its rows to the owners
        if pushed is not None:
            if weights is not None:
                raise NotImplementedError("pushed rows are reduced unweighted: apply the gate inside SwiGLU")
            return d.reduce_pairs(plan, pushed)
        d.stage_out_rows(ye.contiguous())
        ep = d.signal_out()
        return d.pull_rows(plan, ep, weights)

    @staticmethod
    def backward(ctx, g):
        d, plan = ctx.d, ctx.plan
        w = ctx.saved_tensors[0] if ctx.weighted else None
        if d.expert_ordered and plan.perm is not None:
            rdy = d.scatter_ordered(plan, g.contiguous(), None, channel=1, scale_in=w)
            if ctx.defer_bwd and not d.clone_outputs:
                d._bwd_ready = rdy               # taken by the expert GEMM's backward (dgrad waits expert by expert)
            else:
                rdy.wait()
                d.join_side()
        else:
            ep = d.scatter(plan, g.contiguous(), None, channel=1, scale_in=w)
            d.wait_rows(1, ep)
        g_ye = d.rows[1][:ctx.ye_rows]
        if d.clone_outputs:
            g_ye = g_ye.clone()
        if ctx.weighted and ctx.needs_input_grad[1]:
            raise NotImplementedError("gate-weighted fused combine has no weight gradient: apply the gate "
                                      "inside SwiGLU (swiglu_probs) for training")
        return g_ye, None, None, None, None, None
