"""Training loop: micro-batches → (pipeline) forward/backward → sharded AdamW → metrics.

Public API (also what ``bench.py`` times end to end)::

    trainer = Trainer(cfg)                # joins the torchrun job, builds mesh/engine/optimizer
    out = trainer.train_step()            # one optimizer step on the next synthetic global batch
    trainer.fit()                         # cfg.train.train_iters steps with logging/checkpoints

Per-iteration log line carries what the reference's trainer printed
(``notes/2026-04/2026-04-19_gptoss_01_mlperf_best_e2e_run.md:116-131``): elapsed ms, TFLOP/s/GPU,
tokens/s/GPU, lm loss, grad norm, NaN/skipped iterations, device memory.
"""
from __future__ import annotations

import os

import json
import logging
import time
from pathlib import Path

import torch
import torch.distributed as dist

from .. import ops
from ..config import Config
from ..parallel.engine import Engine
from ..parallel.mesh import Mesh, build_mesh, init_distributed
from ..pilot.constraints import param_counts
from .data import make_data
from .optim import ShardedAdamW, lr_at

log = logging.getLogger("system_lab_b200.train")


def model_flops_per_token(m) -> float:
    """Training FLOPs per token (forward + backward = 3x forward): dense matmuls on the *active*
    parameters plus causal attention."""
    pc = param_counts(m)
    embed = m.vocab_size * m.hidden_size            # the lookup is not a matmul
    matmul = 2.0 * (pc["active_per_token"] - embed - m.hidden_size)
    if m.attention_type == "mla":
        d_qk, d_v = m.qk_nope_head_dim + m.qk_rope_head_dim, m.v_head_dim
    else:
        d_qk = d_v = m.kv_channels
    attn = 2.0 * m.seq_length * m.num_attention_heads * (d_qk + d_v) / 2.0 * m.num_layers
    return 3.0 * (matmul + attn)


class NumericalError(RuntimeError):
    """Loss or gradient norm is NaN/Inf (failure kind NUMERICAL)."""


class Trainer:
    def __init__(self, cfg: Config, mesh: Mesh | None = None, device: torch.device | None = None):
        self.cfg = cfg
        if mesh is None:
            rank, world, device = init_distributed(cfg.train.device, timeout_s=max(cfg.train.hang_timeout_s, 60))
            cfg.validate(world)
            mesh = build_mesh(cfg.parallel.pipeline_model_parallel_size, cfg.parallel.expert_model_parallel_size,
                              cfg.parallel.context_parallel_size, cfg.parallel.num_distributed_optimizer_instances,
                              cfg.parallel.tensor_model_parallel_size, cfg.parallel.expert_tensor_parallel_size)
        self.mesh, self.device = mesh, device or torch.device("cpu")
        mode = cfg.train.use_cuda_kernels
        if mode == "false" or self.device.type != "cuda":
            ops.set_kernel_mode("reference")
        else:
            ops.set_kernel_mode("auto")
        ops.set_dense_kernels(cfg.train.dense_gemm_kernels)
        if self.device.type == "cuda":
            from ..ops import cuda as _cops
            _cops.set_fp8_dgrad(cfg.precision.fp8 and cfg.precision.fp8_dgrad)
        torch.manual_seed(cfg.train.seed)
        self.engine = Engine(cfg, mesh, self.device)
        t = cfg.train
        self.optimizer = ShardedAdamW(self.engine, lr=t.lr, beta1=t.adam_beta1, beta2=t.adam_beta2, eps=t.adam_eps,
                                      weight_decay=t.weight_decay, clip_grad=t.clip_grad,
                                      state_dtype=cfg.precision.optimizer_state_dtype)
        if t.optimizer_in_backward:
            self.engine.optimizer = self.optimizer
            if self.device.type == "cuda" and ops.kernel_mode() == "auto":
                from ..ops import cuda as _cops
                _cops.set_adamw_background_piece(t.optimizer_background_piece)
        data_kw = dict(vocab_size=cfg.model.vocab_size, seq_length=cfg.model.seq_length,
                       global_batch_size=t.global_batch_size, micro_batch_size=t.micro_batch_size,
                       dp_rank=mesh.dp_rank, dp_size=mesh.dp, cp_rank=mesh.cp_rank, cp_size=mesh.cp, seed=t.seed,
                       pin=self.device.type == "cuda")
        self.data = make_data(t.data, **data_kw)
        # evaluation batches: their own file, or steps of the training source that training never reaches
        self.eval_data = make_data(t.eval_data, **data_kw) if t.eval_data else self.data
        self.eval_curve: list[tuple[int, float]] = []
        if dist.is_initialized() and mesh.world > 1:
            dist.barrier()                     # ranks leave construction together (peer kernels wait on each other)
        self.step = 0
        self.loss_curve: list[float] = []
        self._read_ring, self._read_next = None, 0       # pinned slots of begin_loss_read
        self.last_status_any = False
        self.step_times_ms: list[float] = []
        self.nan_iters = 0
        self.flops_per_token = model_flops_per_token(cfg.model)
        self.tokens_per_step = t.global_batch_size * cfg.model.seq_length
        self._tpe_accum = None
        self.reached_target = False
        self.stopped_on_time = False
        self.stopped_on_signal = False
        self.relocator = None
        self._rank_load_accum = None      # [layers, ep]: tokens each expert-parallel rank received
        reloc, reloc_first = cfg.model.moe_expert_relocation_interval, cfg.model.moe_expert_relocation_first_step
        reloc_ok = mesh.edp == 1 and mesh.cp == 1 and mesh.tp == 1
        if reloc < 0:                           # automatic: on where whole experts can move inside one group
            reloc, reloc_first = (50, reloc_first or 3) if (reloc_ok and mesh.ep > 1) else (0, 0)
        if reloc > 0 and cfg.model.num_experts > 0 and mesh.ep > 1:
            from ..moe.relocation import ExpertRelocator
            if not reloc_ok:
                raise ValueError("moe_expert_relocation_interval needs ep == dp on the stage and cp == 1")
            self.relocator = ExpertRelocator(self.engine, self.optimizer, mesh, reloc,
                                             cfg.model.moe_expert_relocation_min_gain, reloc_first)
        from .watchdog import FaultPlan, Heartbeat
        # a job restarted by the supervisor (launch.py) does not repeat the injected failure
        restarted = int(os.environ.get("SLAB_RESTART_COUNT", "0") or 0) > 0
        self.faults = FaultPlan.parse("" if restarted else t.fault_injection)
        self.heartbeat = None
        if t.heartbeat and dist.is_initialized() and mesh.world > 1:
            store = dist.PrefixStore("slab_heartbeat", dist.distributed_c10d._get_default_store())
            self.heartbeat = Heartbeat(store, mesh.rank, mesh.world, t.hang_timeout_s).start()
        self.events = None
        if t.mllog:
            from .mllog import MLLogger
            self.events = MLLogger(enabled=mesh.rank == 0)

    def close(self) -> None:
        """Stop background helpers (the heartbeat watchdog thread).  Safe to call more than once."""
        hb, self.heartbeat = getattr(self, "heartbeat", None), None
        if hb is not None:
            hb.stop()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    # ---- one optimizer step ---------------------------------------------------------------
    def train_step(self, batches=None) -> dict:
        """Runs one full step.  ``batches``: optional list of host ``(tokens, targets)`` micro-batches;
        by default the next synthetic global batch.  Returns ``{"loss": device scalar, "grad_norm": ...}``."""
        cfg, mesh = self.cfg, self.mesh
        step = self.step + 1
        flags = self.faults.before_step(mesh.rank, step) if self.faults.actions else {}
        if self.heartbeat is not None:
            if flags.get("mute"):
                self.heartbeat.muted = True
            self.heartbeat.check()             # a peer that hung or failed is reported before anything is launched
            self.heartbeat.begin(step)
        if batches is None:
            batches = self.data.microbatches(self.step)
        nmb = len(batches)
        dev = self.device
        dev_batches = [(tok.to(dev, non_blocking=True), tgt.to(dev, non_blocking=True)) for tok, tgt in batches]
        lr = lr_at(step, lr=cfg.train.lr, min_lr=cfg.train.min_lr, warmup=cfg.train.lr_warmup_iters,
                   decay_iters=cfg.train.lr_decay_iters, style=cfg.train.lr_decay_style,
                   wsd_decay_iters=cfg.train.lr_wsd_decay_iters)
        in_bwd = cfg.train.optimizer_in_backward
        if in_bwd:
            self.optimizer.begin_step(lr)
        scale = 1.0 / (nmb * mesh.data_size)
        loss_sum = torch.zeros((), dtype=torch.float32, device=dev)
        if mesh.pp > 1 and self.engine.vpp > 1:
            from ..parallel.pp import pipeline_interleaved
            loss_sum = pipeline_interleaved(self.engine, mesh, dev_batches, scale, cfg)
        elif mesh.pp > 1:
            from ..parallel.pp import pipeline_1f1b
            loss_sum = pipeline_1f1b(self.engine, mesh, dev_batches, scale, cfg)
        else:
            for tok, tgt in dev_batches:
                loss, aux = self.engine.stage_forward(tok, tgt)
                total = loss * scale
                for a in aux:
                    total = total + a * scale
                total.backward()
                loss_sum = loss_sum + loss.detach().float()
        grad_norm = self.optimizer.end_step_in_backward() if in_bwd else self.optimizer.step(lr)
        self._update_router_bias()
        # mean loss over micro-batches and data ranks (reported from the last pipeline stage)
        loss_mean = loss_sum / nmb
        # the kernels' status word travels with the loss: after the sum every rank knows, without a host read of its
        # own, whether a bounded wait ran out or a bounds check failed anywhere in this step
        status_any = None
        if dev.type == "cuda" and ops.kernel_mode() == "auto":
            from ..ops import cuda as _cops
            status_any = (_cops.status_word(dev) != 0).float().reshape(())
        if dist.is_initialized() and mesh.world > 1:
            pack = torch.stack([loss_mean.reshape(()), status_any if status_any is not None else torch.zeros_like(loss_mean).reshape(())])
            dist.all_reduce(pack)
            # pipeline: only last-stage ranks hold a loss, the others contribute zero
            loss_mean = pack[0] / ((mesh.data_size * mesh.tp) if mesh.pp > 1 else mesh.world)
            status_any = pack[1]
        if flags.get("nan"):
            loss_mean = loss_mean * float("nan")
        self.step = step
        if self.heartbeat is not None:
            self.heartbeat.beat(step)
        return {"loss": loss_mean, "grad_norm": grad_norm, "lr": lr, "status_any": status_any}

    # ---- reading a step's numbers without stalling the launch of the next step -------------------------
    def begin_loss_read(self, out: dict):
        """Start copying the step's loss and gradient norm into pinned host memory (on the current stream, after the
        step's kernels) and return a ticket for :meth:`finish_loss_read`.  Taking the ticket of step ``s`` only after
        step ``s + 1`` has been launched keeps the device busy while the host waits: the host then blocks until step
        ``s`` is done with all of step ``s + 1`` already queued."""
        dev = out["loss"].device
        st = out.get("status_any")
        vals = torch.stack([out["loss"].detach().float().reshape(()),
                            torch.as_tensor(out["grad_norm"], dtype=torch.float32, device=dev).detach().reshape(()),
                            st.float().reshape(()) if st is not None else torch.zeros((), device=dev)])
        if self.device.type != "cuda":
            return vals, None
        if self._read_ring is None:
            self._read_ring = torch.zeros(16, 3, dtype=torch.float32).pin_memory()
        slot = self._read_next % self._read_ring.shape[0]
        self._read_next += 1
        self._read_ring[slot].copy_(vals, non_blocking=True)
        ev = torch.cuda.Event()
        ev.record(torch.cuda.current_stream(self.device))
        return slot, ev

    def finish_loss_read(self, ticket) -> tuple[float, float]:
        """``(loss, grad_norm)`` of the step the ticket was taken for; waits on the host until that step is done."""
        slot, ev = ticket
        if ev is None:
            row = slot
        else:
            ev.synchronize()
            row = self._read_ring[slot]
        self.last_status_any = float(row[2]) > 0          # some rank's kernels reported an error in that step
        return float(row[0]), float(row[1])

    def check_device_status(self) -> None:
        """Read the status word the kernels write when a bounded wait runs out or a bounds check fails (a lost peer
        flag leaves zeroed combine outputs and a skipped update behind; a capacity overflow drops token-expert
        pairs), agree on it across ranks and stop the run before the damaged state is trained on or checkpointed.
        Call at a point where the device is idle anyway (``fit`` does, right after it has read the loss)."""
        from ..ops import cuda as cops
        code = cops.peek_status(self.device)
        if dist.is_initialized() and self.mesh.world > 1:
            t = torch.tensor([float(code)], device=self.device)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)       # every rank leaves the step together
            code = int(t.item())
        if code:
            cops.clear_status(self.device)
            msg = f"step {self.step}: a device kernel reported {cops.status_name(code)}"
            if self.heartbeat is not None:
                self.heartbeat.fail(msg)                    # the supervisor restarts from the last good checkpoint
            raise cops.DeviceHang(msg)

    def _should_leave(self, started: float, minutes: float) -> bool:
        """One small collective after a step: has rank 0's clock passed the limit, has any rank received SIGTERM?
        Every rank gets the same answer, so no rank enters the next step alone."""
        late = minutes > 0 and self.mesh.rank == 0 and (time.time() - started) > 60.0 * minutes
        flags = torch.tensor([1.0 if late else 0.0, 1.0 if self._term_seen else 0.0], device=self.device)
        if dist.is_initialized() and self.mesh.world > 1:
            dist.all_reduce(flags, op=dist.ReduceOp.MAX)
        self.stopped_on_time = bool(flags[0] > 0)
        self.stopped_on_signal = bool(flags[1] > 0)
        return self.stopped_on_time or self.stopped_on_signal

    EVAL_STEP_OFFSET = 1 << 40            # held-out region of the (seed, step) -> batch map

    @torch.no_grad()
    def evaluate(self, iters: int | None = None) -> float:
        """Mean loss over ``iters`` held-out global batches (forward only, no dropout in this model family so no
        mode switch is needed); identical on every rank."""
        cfg, mesh, dev = self.cfg, self.mesh, self.device
        iters = iters if iters is not None else max(cfg.train.eval_iters, 1)
        offset = 0 if self.eval_data is not self.data else self.EVAL_STEP_OFFSET
        total = torch.zeros((), dtype=torch.float32, device=dev)
        count = 0
        self.engine.inference = True
        try:
            total, count = self._eval_batches(iters, offset, total)
        finally:
            self.engine.inference = False
        for f in self.engine.moe_ffns():                # evaluation tokens do not count towards router balancing
            f.step_tokens_per_expert = None
        mean = total / max(count, 1)
        if dist.is_initialized() and mesh.world > 1:
            dist.all_reduce(mean)
            mean = mean / (mesh.data_size * mesh.tp if mesh.pp > 1 else mesh.world)
        return float(mean)

    def _eval_batches(self, iters: int, offset: int, total: torch.Tensor):
        cfg, mesh, dev = self.cfg, self.mesh, self.device
        count = 0
        for i in range(iters):
            batches = [(a.to(dev), b.to(dev)) for a, b in self.eval_data.microbatches(offset + i)]
            if self.eval_data is self.data:
                self.data.cursor = self.step            # serving evaluation batches does not move the training cursor
            if mesh.pp > 1 and self.engine.vpp > 1:
                from ..parallel.pp import pipeline_interleaved
                total = total + pipeline_interleaved(self.engine, mesh, batches, 1.0, cfg, forward_only=True)
            elif mesh.pp > 1:
                from ..parallel.pp import pipeline_forward_only
                total = total + pipeline_forward_only(self.engine, mesh, batches, cfg)
            else:
                for tok, tgt in batches:
                    loss, _ = self.engine.stage_forward(tok, tgt)
                    total = total + loss.float()
            count += len(batches)
        return total, count

    def _update_router_bias(self) -> None:
        m = self.cfg.model
        ffns = self.engine.moe_ffns()
        if not ffns:
            return
        counts = [f.step_tokens_per_expert for f in ffns if f.step_tokens_per_expert is not None]
        for f in ffns:
            f.step_tokens_per_expert = None
        if len(counts) != len(ffns):
            return
        tpe = torch.stack(counts).float()
        if dist.is_initialized() and self.mesh.data_size * self.mesh.tp > 1:
            dist.all_reduce(tpe, group=self.mesh.stage_group)
        self._tpe_accum = tpe if self._tpe_accum is None else self._tpe_accum + tpe
        # load per expert-parallel rank under the placement that was in force during this step
        e_local = tpe.shape[1] // max(self.mesh.ep, 1)
        rank_of = torch.stack([f.expert_map for f in ffns]).to(tpe.device) // e_local
        per_rank = torch.zeros(tpe.shape[0], self.mesh.ep, dtype=tpe.dtype, device=tpe.device).scatter_add_(1, rank_of, tpe)
        self._rank_load_accum = per_rank if self._rank_load_accum is None else self._rank_load_accum + per_rank
        if m.moe_router_load_balancing_type == "bias":
            for f, c in zip(ffns, tpe):
                f.update_router_bias(c)
        if self.relocator is not None:
            self.relocator.observe(tpe)
            rec = self.relocator.maybe_relocate(self.step + 1)
            if rec and self.mesh.rank == 0:
                print(f" expert placement at iteration {rec['step']}: moved {rec['experts_moved']} experts, rank load "
                      f"max/mean {rec['imbalance_before']:.3f} -> {rec['imbalance_after_predicted']:.3f} (predicted)",
                      flush=True)

    def rank_load_ratio(self) -> float | None:
        """Mean over MoE layers of max/mean tokens per expert-parallel rank, over the steps so far."""
        if self._rank_load_accum is None:
            return None
        pr = self._rank_load_accum.float()
        return float((pr.max(1).values / pr.mean(1).clamp_min(1)).mean())

    # ---- full run ----------------------------------------------------------------------------
    def fit(self, iters: int | None = None) -> dict:
        cfg, t = self.cfg, self.cfg.train
        iters = t.train_iters if iters is None else iters
        is_cuda = self.device.type == "cuda"
        if self.events:
            self.events.start(cfg)
        prof = None
        if cfg.profile.profile and self.mesh.rank in cfg.profile.profile_ranks:
            from ..observe.profiler import StepProfiler
            prof = StepProfiler(cfg.profile, self.mesh.rank)
        target = self.step + iters
        import gc
        if t.manual_gc:
            gc.disable()
            gc.collect()
        started = time.time()
        self._term_seen = False
        old_handler = None
        if t.exit_signal_handler:
            import signal
            import threading
            if threading.current_thread() is threading.main_thread():
                old_handler = signal.signal(signal.SIGTERM, lambda *_: setattr(self, "_term_seen", True))
        # deferred_loss_read: the numbers of step s are read after step s + 1 has been launched, so the device never
        # waits for the host between steps; steps that evaluate, save, may leave, or end the run are read at once
        deferred = bool(t.deferred_loss_read) and prof is None
        pending = None                                  # (step, ticket, lr, host time at launch) of the unread step
        t_prev = time.perf_counter()

        def account(step: int, loss: float, gn: float, lr: float, dt_ms: float) -> None:
            self.step_times_ms.append(dt_ms)
            self.loss_curve.append(loss)
            bad = not (loss == loss and abs(loss) != float("inf") and gn == gn and gn != float("inf"))
            if bad:
                self.nan_iters += 1
                if t.check_for_nan_in_loss_and_grad:
                    raise NumericalError(f"step {step}: loss={loss} grad_norm={gn}")
            if self.mesh.rank == 0 and (step % max(t.log_interval, 1) == 0):
                self._log_line(dt_ms, loss, gn, lr, step)

        def drain() -> None:
            nonlocal pending, t_prev
            if pending is not None:
                st, ticket, lr_, _ = pending
                loss_, gn_ = self.finish_loss_read(ticket)
                now = time.perf_counter()
                if self.last_status_any:                  # the same answer on every rank: all of them stop here together
                    self.check_device_status()
                account(st, loss_, gn_, lr_, (now - t_prev) * 1e3)      # time between two steps' completions
                t_prev, pending = now, None

        while self.step < target:
            if deferred:
                out = self.train_step()
                ticket = self.begin_loss_read(out)
                drain()                                  # the previous step, with this one already queued
                pending = (self.step, ticket, out["lr"], time.perf_counter())
                ck_ = cfg.checkpoint
                boundary = (self.step >= target or (t.eval_interval and self.step % t.eval_interval == 0)
                            or (ck_.save and ck_.save_interval and self.step % ck_.save_interval == 0)
                            or getattr(self, "_pending_ckpt", None) is not None
                            or t.exit_duration_in_mins > 0 or t.exit_signal_handler
                            or (t.manual_gc and self.step % max(t.manual_gc_interval, 1) == 0))
                if not boundary:
                    continue
                drain()
            else:
                if is_cuda:
                    torch.cuda.synchronize()
                t0 = time.perf_counter()
                if prof:
                    prof.step_begin(self.step + 1)
                out = self.train_step()
                loss = float(out["loss"])              # host read: also the step's device sync
                gn = float(out["grad_norm"])
                self.check_device_status()             # before anything is logged, evaluated or saved from this step
                if prof:
                    prof.step_end(self.step)
                account(self.step, loss, gn, out["lr"], (time.perf_counter() - t0) * 1e3)
            if t.eval_interval and self.step % t.eval_interval == 0:
                ev = self.evaluate()
                self.eval_curve.append((self.step, ev))
                if self.mesh.rank == 0:
                    print(f" validation loss at iteration {self.step:6d} | lm loss value: {ev:.6E}", flush=True)
                if self.events:
                    self.events.eval(ev, self.step * t.global_batch_size)
                if t.eval_target_loss > 0 and ev <= t.eval_target_loss:
                    self.reached_target = True
                    break
            ck = cfg.checkpoint
            if getattr(self, "_pending_ckpt", None) is not None:
                from ..ckpt.sharded import finish_pending
                finish_pending(self)                  # publishes an asynchronous save once every rank has written
            if ck.save and ck.save_interval and self.step % ck.save_interval == 0:
                self.save_checkpoint(ck.save)
            if t.manual_gc and self.step % max(t.manual_gc_interval, 1) == 0:
                gc.collect()                          # same step on every rank: one aligned pause instead of scattered ones
            if (t.exit_duration_in_mins > 0 or t.exit_signal_handler) and \
                    self._should_leave(started, t.exit_duration_in_mins):
                break
        if t.manual_gc:
            gc.enable()
        if old_handler is not None:
            import signal
            signal.signal(signal.SIGTERM, old_handler)
        if cfg.checkpoint.save and not cfg.checkpoint.disable_last_saving:
            self.save_checkpoint(cfg.checkpoint.save)
        if getattr(self, "_pending_ckpt", None) is not None:
            from ..ckpt.sharded import finish_pending
            finish_pending(self, wait=True)
        if self.events:
            ok = self.reached_target or not t.eval_target_loss
            self.events.stop(self.tokens_per_step * self.step, status="success" if ok else "aborted")
        snap = self.snapshot()
        if cfg.profile.snapshot_path and self.mesh.rank == 0:
            Path(cfg.profile.snapshot_path).parent.mkdir(parents=True, exist_ok=True)
            Path(cfg.profile.snapshot_path).write_text(json.dumps(snap, indent=2))
        return snap

    def _log_line(self, dt_ms: float, loss: float, gn: float, lr: float, step: int | None = None) -> None:
        step = self.step if step is None else step
        tps_gpu = self.tokens_per_step / (dt_ms / 1e3) / self.mesh.world
        tflops = tps_gpu * self.flops_per_token / 1e12
        mem = torch.cuda.max_memory_allocated() / 2**30 if self.device.type == "cuda" else 0.0
        log.info("iteration %6d | elapsed ms/iter %9.1f | TFLOP/s/GPU %7.1f | tokens/s/GPU %9.0f | lm loss %.6f | "
                 "grad norm %.4f | lr %.3e | nan iters %d | mem GiB %.1f",
                 step, dt_ms, tflops, tps_gpu, loss, gn, lr, self.nan_iters, mem)
        path = self.cfg.train.metrics_file
        if path:
            rec = {"step": step, "time": time.time(), "step_ms": dt_ms, "loss": loss, "grad_norm": gn, "lr": lr,
                   "tokens_per_s": self.tokens_per_step / (dt_ms / 1e3), "tflops_per_gpu": tflops, "mem_gib": mem,
                   "nan_iters": self.nan_iters, "ep_rank_load_max_over_mean": self.rank_load_ratio()}
            Path(path).parent.mkdir(parents=True, exist_ok=True)
            with open(path, "a") as f:
                f.write(json.dumps(rec) + "\n")

    # ---- the tuner's Snapshot (metric contract: skills/pilot/workflow/observe.md:36-112) ------------
    def snapshot(self) -> dict:
        from ..observe.snapshot import build_snapshot
        return build_snapshot(self)

    # ---- checkpoints -----------------------------------------------------------------------------
    def save_checkpoint(self, root: str) -> str:
        from ..ckpt.sharded import save_checkpoint
        return save_checkpoint(self, root)

    def load_checkpoint(self, path: str) -> None:
        from ..ckpt.sharded import load_checkpoint
        load_checkpoint(self, path)
        for f in self.engine.moe_ffns():              # a checkpoint written after expert relocation carries its placement
            ident = torch.arange(f.expert_map.numel(), device=f.expert_map.device)
            f.relocated = bool((f.expert_map != ident).any())
