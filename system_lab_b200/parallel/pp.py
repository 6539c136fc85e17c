"""Pipeline parallel 1F1B schedule over point-to-point send/recv (NCCL on GPUs, gloo on CPU).

Each stage runs ``min(pp - stage - 1, M)`` warm-up forwards, then alternates one forward and one
backward, then drains.  Paired transfers (send forward + receive backward, send backward + receive
forward) are posted together with ``batch_isend_irecv`` so neighbouring stages never wait on each
other's send.  Bubble fraction is ``(pp-1)/(pp-1+M)`` (``pilot/README.v2.md:771``).

Pipeline transfers stay on the library p2p path by design: they are small
(``mbs x seq x hidden``) next to the expert all-to-all and overlap with compute.
"""
from __future__ import annotations

import torch
import torch.distributed as dist


def _p2p(ops_list):
    if not ops_list:
        return
    for r in dist.batch_isend_irecv(ops_list):
        r.wait()


def pipeline_1f1b(engine, mesh, batches, scale: float, cfg) -> torch.Tensor:
    """Run all micro-batches of one step through this stage.  Returns the summed (unscaled) loss on the
    last stage and zero elsewhere."""
    dev = engine.device
    nmb = len(batches)
    first, last = mesh.is_first_stage(), mesh.is_last_stage()
    prev_r = mesh.prev_stage_rank() if not first else None
    next_r = mesh.next_stage_rank() if not last else None
    mbs, seq = batches[0][0].shape
    act_shape = (mbs, seq // engine.seq_shards(), cfg.model.hidden_size)
    dt = engine.compute_dtype
    loss_sum = torch.zeros((), dtype=torch.float32, device=dev)
    pending = []            # (input hidden or None, output, aux list) awaiting backward

    def new_act():
        return torch.empty(act_shape, dtype=dt, device=dev)

    def fwd(i, recv_buf):
        tok, tgt = batches[i]
        if first:
            inp, x = None, tok
        else:
            inp = recv_buf.requires_grad_(True)
            x = inp
        out, aux = engine.stage_forward(x, tgt if last else None)
        pending.append((inp, out, aux))
        return out

    def bwd(grad_out):
        nonlocal loss_sum
        inp, out, aux = pending.pop(0)
        if last:
            loss_sum = loss_sum + out.detach().float()
            tensors, grads = [out], [torch.full_like(out, scale)]
        else:
            tensors, grads = [out], [grad_out]
        for a in aux:
            tensors.append(a)
            grads.append(torch.full_like(a, scale))
        torch.autograd.backward(tensors, grads)
        return inp.grad if inp is not None else None

    warm = min(mesh.pp - mesh.pp_rank - 1, nmb)
    steady = nmb - warm
    recv_f = None
    if not first:
        recv_f = new_act()
        _p2p([dist.P2POp(dist.irecv, recv_f, prev_r)])
    # warm-up forwards
    for i in range(warm):
        out = fwd(i, recv_f)
        ops_l = []
        if not last:
            ops_l.append(dist.P2POp(dist.isend, out.detach().contiguous(), next_r))
        more_fwd = (i + 1 < warm) or steady > 0
        if not first and more_fwd:
            recv_f = new_act()
            ops_l.append(dist.P2POp(dist.irecv, recv_f, prev_r))
        _p2p(ops_l)
    # steady state: one forward, one backward
    for j in range(steady):
        i = warm + j
        out = fwd(i, recv_f)
        grad_out = None
        ops_l = []
        if not last:
            grad_out = new_act()
            ops_l.append(dist.P2POp(dist.isend, out.detach().contiguous(), next_r))
            ops_l.append(dist.P2POp(dist.irecv, grad_out, next_r))
        _p2p(ops_l)
        gin = bwd(grad_out)
        ops_l = []
        if not first:
            ops_l.append(dist.P2POp(dist.isend, gin.contiguous(), prev_r))
            if j + 1 < steady:
                recv_f = new_act()
                ops_l.append(dist.P2POp(dist.irecv, recv_f, prev_r))
        _p2p(ops_l)
    # cool-down backwards
    for _ in range(warm):
        grad_out = None
        if not last:
            grad_out = new_act()
            _p2p([dist.P2POp(dist.irecv, grad_out, next_r)])
        gin = bwd(grad_out)
        if not first:
            _p2p([dist.P2POp(dist.isend, gin.contiguous(), prev_r)])
    return loss_sum


@torch.no_grad()
def pipeline_forward_only(engine, mesh, batches, cfg) -> torch.Tensor:
    """Evaluation pass: every micro-batch goes through the stages once, nothing is kept for backward.
    Returns the summed loss on the last stage and zero elsewhere."""
    dev = engine.device
    first, last = mesh.is_first_stage(), mesh.is_last_stage()
    prev_r = mesh.prev_stage_rank() if not first else None
    next_r = mesh.next_stage_rank() if not last else None
    mbs, seq = batches[0][0].shape
    act_shape = (mbs, seq // engine.seq_shards(), cfg.model.hidden_size)
    loss_sum = torch.zeros((), dtype=torch.float32, device=dev)
    for tok, tgt in batches:
        if first:
            x = tok
        else:
            x = torch.empty(act_shape, dtype=engine.compute_dtype, device=dev)
            _p2p([dist.P2POp(dist.irecv, x, prev_r)])
        out, _ = engine.stage_forward(x, tgt if last else None)
        if last:
            loss_sum = loss_sum + out.float()
        else:
            _p2p([dist.P2POp(dist.isend, out.contiguous(), next_r)])
    return loss_sum


# ---------------------------------------------------------------------------------------------------------------
# Interleaved (virtual) pipeline stages.  The decoder is cut into pp * vpp blocks; block v runs on rank v % pp as
# that rank's chunk v // pp.  Micro-batches go through in groups of pp: a rank runs chunk 0 for the whole group,
# then chunk 1, ...; every rank therefore sends to its right neighbour and receives from its left neighbour in
# one fixed order (group, chunk, micro-batch), which is also the order the neighbour consumes / produces, so
# FIFO point-to-point channels need no tags.  All forwards of the step run before the backwards (the layers are
# recomputed in backward, so what stays alive per micro-batch is one boundary activation per chunk); the bubble
# shrinks to (pp-1) / (pp-1 + M*vpp) as for any interleaved schedule.
def _vstage_order(nmb: int, pp: int, vpp: int, reverse_chunks: bool = False):
    chunks = range(vpp - 1, -1, -1) if reverse_chunks else range(vpp)
    for g0 in range(0, nmb, pp):
        for c in chunks:
            for i in range(g0, min(g0 + pp, nmb)):
                yield c, i


def pipeline_interleaved(engine, mesh, batches, scale: float, cfg, forward_only: bool = False) -> torch.Tensor:
    """All micro-batches of one step through this rank's ``vpp`` chunks.  Returns the summed (unscaled) loss on
    the rank that holds the last block and zero elsewhere."""
    dev, pp, vpp, r = engine.device, mesh.pp, engine.vpp, mesh.pp_rank
    nmb = len(batches)
    if nmb % pp:
        raise ValueError(f"interleaved stages need micro-batches per step ({nmb}) to be a multiple of pp ({pp})")
    right, left = mesh.pp_ranks[(r + 1) % pp], mesh.pp_ranks[(r - 1) % pp]
    mbs, seq = batches[0][0].shape
    act_shape = (mbs, seq // engine.seq_shards(), cfg.model.hidden_size)
    dt = engine.compute_dtype
    last_v = pp * vpp - 1
    loss_sum = torch.zeros((), dtype=torch.float32, device=dev)
    kept = {}                         # (chunk, micro-batch) -> (input hidden or None, output, aux list)
    sends = []                        # outstanding isend handles (buffers are referenced until waited)

    r_right, r_left = (r + 1) % pp, (r - 1) % pp

    def chan(src_stage: int, dst_stage: int):
        return mesh.pp_group_up if dst_stage > src_stage else mesh.pp_group_down

    def send(t, dst, dst_stage):
        t = t.contiguous()
        sends.append((dist.isend(t, dst, group=chan(r, dst_stage)), t))

    def recv(src, src_stage):
        buf = torch.empty(act_shape, dtype=dt, device=dev)
        dist.recv(buf, src, group=chan(src_stage, r))
        return buf

    # ---- forwards ---------------------------------------------------------------------------------------------------
    for c, i in _vstage_order(nmb, pp, vpp):
        v = c * pp + r
        tok, tgt = batches[i]
        if v == 0:
            inp, x = None, tok
        else:
            inp = recv(left, r_left)
            if not forward_only:
                inp.requires_grad_(True)
            x = inp
        out, aux = engine.stage_forward(x, tgt if v == last_v else None, chunk=c)
        if v == last_v:
            if forward_only:
                loss_sum = loss_sum + out.detach().float()
        else:
            send(out.detach(), right, r_right)
        if not forward_only:
            kept[(c, i)] = (inp, out, aux)
    if forward_only:
        for h, _ in sends:
            h.wait()
        return loss_sum
    # ---- backwards: same groups, chunks from last to first ----------------------------------------------------------------
    for c, i in _vstage_order(nmb, pp, vpp, reverse_chunks=True):
        v = c * pp + r
        inp, out, aux = kept.pop((c, i))
        if v == last_v:
            loss_sum = loss_sum + out.detach().float()
            tensors, grads = [out], [torch.full_like(out, scale)]
        else:
            tensors, grads = [out], [recv(right, r_right)]
        for a in aux:
            tensors.append(a)
            grads.append(torch.full_like(a, scale))
        torch.autograd.backward(tensors, grads)
        if v != 0:
            send(inp.grad, left, r_left)
    for h, _ in sends:
        h.wait()
    return loss_sum
