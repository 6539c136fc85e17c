"""Sharded AdamW over the engine's flat groups, with global-norm clipping.

Every flat group owns one contiguous shard, so the optimizer is a handful of large launches of the
fused kernel (``csrc/elementwise.cu``) instead of the per-parameter ``multi_tensor_apply`` tail the
reference traces show (``notes/2026-04/2026-04-22_gptoss_15_*:119-131``, 369 L2-norm launches per
iteration in ``notes/2026-04/2026-04-21_gptoss_09_*:102-108``).  The clip coefficient stays on the
device: no ``.item()`` in the step.

Moments may be stored in fp32, bf16 or block-scaled 8 bit (e4m3 per 128 elements; the second
moment is stored as its square root to halve the exponent range it needs).
"""
from __future__ import annotations

import math

import torch
import torch.distributed as dist

from ..ops import reference as ref
from ..parallel.engine import Engine


class _Moment:
    """One optimizer moment for a flat shard in the configured storage format."""

    def __init__(self, n: int, kind: str, device, sqrt_domain: bool = False):
        self.kind, self.n, self.sqrt_domain = kind, n, sqrt_domain
        if kind == "fp32":
            self.data = torch.zeros(n, dtype=torch.float32, device=device)
        elif kind == "bf16":
            self.data = torch.zeros(n, dtype=torch.bfloat16, device=device)
        else:
            self.data = torch.zeros(n, dtype=torch.float8_e4m3fn, device=device)
            self.scale = torch.zeros(n // 128, dtype=torch.float32, device=device)

    def load(self) -> torch.Tensor:
        if self.kind == "fp32":
            return self.data
        if self.kind == "bf16":
            x = self.data.float()
        else:
            x = ref.dequant_1x128(self.data, self.scale)
        return x * x if self.sqrt_domain else x

    def store(self, x: torch.Tensor) -> None:
        if self.kind == "fp32":
            if x is not self.data:
                self.data.copy_(x)
            return
        if self.sqrt_domain:
            x = x.sqrt()
        if self.kind == "bf16":
            self.data.copy_(x)
        else:
            q, s = ref.quant_1x128(x)
            self.data.copy_(q)
            self.scale.copy_(s)

    def state(self) -> dict:
        d = {"data": self.data}
        if self.kind == "fp8":
            d["scale"] = self.scale
        return d


class ShardedAdamW:
    def __init__(self, engine: Engine, *, lr: float, beta1: float, beta2: float, eps: float,
                 weight_decay: float, clip_grad: float, state_dtype: str = "fp32"):
        self.engine = engine
        self.lr, self.beta1, self.beta2, self.eps = lr, beta1, beta2, eps
        self.weight_decay, self.clip_grad = weight_decay, clip_grad
        self.state_dtype = state_dtype
        self.step_count = 0
        self.m, self.v = {}, {}
        dev = engine.device
        for g in engine.all_groups():
            if getattr(g, "frozen", False):
                continue                  # frozen groups (the base model under LoRA) own no optimizer state
            n = g.shard.numel()
            self.m[g.name] = _Moment(n, state_dtype, dev)
            self.v[g.name] = _Moment(n, state_dtype, dev, sqrt_domain=(state_dtype != "fp32"))
        self.last_grad_norm: torch.Tensor | None = None
        self._prev_norm: torch.Tensor | None = None     # for delayed clipping in optimizer-in-backward mode
        self._sq_accum: torch.Tensor | None = None
        self._side = None                 # side stream for in-backward updates
        self.background_ctas = 2          # resident CTAs per SM of a side-stream update (of 8 thread-slot-filling ones)
        self._coef_for_step = None

    # ---- gradient norm ------------------------------------------------------------
    def _replication(self, g) -> int:
        tp = getattr(g, "tp_replicas", 1)                # dense groups are replicated over the tensor-parallel ranks
        if g.replica_group is None:
            return tp
        return tp * dist.get_world_size(g.replica_group)  # unsharded replicas, or the blocks of hybrid sharding

    def _add_sumsq(self, acc: torch.Tensor, g) -> torch.Tensor:
        """acc (1-element fp32 tensor) += sum(grad_shard^2) / replication."""
        from .. import ops
        if g.grad_shard is None:
            return acc
        if ops.use_kernels(g.grad_shard):
            from ..ops import cuda as cops
            cops.sumsq(g.grad_shard, 1.0 / self._replication(g), acc)
            return acc
        return acc + g.grad_shard.float().pow(2).sum() / self._replication(g)

    def global_grad_norm(self) -> torch.Tensor:
        sq = torch.zeros(1, dtype=torch.float32, device=self.engine.device)
        for g in self.engine.all_groups():
            sq = self._add_sumsq(sq, g)
        if dist.is_initialized() and dist.get_world_size() > 1:
            dist.all_reduce(sq)
        return sq.sqrt().squeeze(0)

    def _clip_coef(self, norm: torch.Tensor) -> torch.Tensor:
        if self.clip_grad <= 0:
            return torch.ones((), dtype=torch.float32, device=self.engine.device)
        return torch.clamp(self.clip_grad / (norm + 1e-6), max=1.0)

    # ---- update -----------------------------------------------------------------------
    def fusable(self, g) -> bool:
        # the fused kernel adds the undivided sum of squares to the norm accumulator: only for groups that no other
        # rank holds a copy of (a dense group under tensor parallelism is replicated and goes the two-kernel way)
        return (self.state_dtype == "fp32" and g.device.type == "cuda" and g.can_fuse_rs_adamw()
                and self._replication(g) == 1)

    def _fused_rs_update(self, g, coef: torch.Tensor, lr: float, sq_out: torch.Tensor) -> None:
        """One kernel: pull every rank's gradient slice over NVLink, sum in fp32, AdamW on the master shard and
        moments, write the bf16 shard the next all-gather will publish."""
        grad_full = g.take_grad_full()
        g.comm.reduce_scatter_adamw(grad_full, g.shard, self.m[g.name].data, self.v[g.name].data, g.shard_lp, coef,
                                    sq_out, lr=lr, beta1=self.beta1, beta2=self.beta2, eps=self.eps,
                                    weight_decay=self.weight_decay, step=self.step_count,
                                    decay_end=g.shard_decay_end())

    def _update_group(self, g, coef: torch.Tensor, lr: float, sq_out: torch.Tensor | None = None,
                      background: bool = False) -> None:
        """``sq_out``: also accumulate ``sum(grad^2) / replication`` of this group there (fused into the
        kernel on the GPU path).  ``background``: the update shares the GPU with another stream's compute, so
        its kernel keeps only a few CTAs resident per SM instead of filling every thread slot."""
        if g.grad_shard is None:
            return
        from .. import ops
        if ops.use_kernels(g.shard):
            from ..ops import cuda as cops
            fuse = sq_out is not None and self._replication(g) == 1
            if sq_out is not None and not fuse:
                self._add_sumsq(sq_out, g)
            cops.adamw_flat(g, self.m[g.name], self.v[g.name], coef, lr=lr, beta1=self.beta1, beta2=self.beta2,
                            eps=self.eps, weight_decay=self.weight_decay, step=self.step_count,
                            sq_out=sq_out if fuse else None, ctas_per_sm=self.background_ctas if background else 0)
        else:
            if sq_out is not None:
                sq_out += g.grad_shard.float().pow(2).sum() / self._replication(g)
            p32 = g.shard.float() if g.shard.dtype != torch.float32 else g.shard
            m, v = self.m[g.name].load(), self.v[g.name].load()
            m = m.clone() if m is not self.m[g.name].data else m
            v = v.clone() if v is not self.v[g.name].data else v
            gs = g.grad_shard.float() * coef
            de = g.shard_decay_end()                     # matrices [0, de) decay, the 1-D parameters behind them do not
            for lo, hi, wd in ((0, de, self.weight_decay), (de, p32.numel(), 0.0)):
                if hi > lo:
                    ref.adamw_step(p32[lo:hi], gs[lo:hi], m[lo:hi], v[lo:hi], lr=lr, beta1=self.beta1,
                                   beta2=self.beta2, eps=self.eps, weight_decay=wd, step=self.step_count)
            self.m[g.name].store(m)
            self.v[g.name].store(v)
            if p32 is not g.shard:
                g.shard.copy_(p32)
            g.sync_low_precision()
        g.grad_shard = None

    @staticmethod
    def _new_weight_generation() -> None:
        """Cached derivatives of the weights (quantised copies) are stale after this step's update."""
        try:
            from ..ops import cuda as cops
            cops.WEIGHT_GENERATION[0] += 1
        except Exception:
            pass

    def begin_step(self, lr: float | None = None) -> None:
        """Call before backward when the update runs inside backward."""
        self._new_weight_generation()
        self.step_count += 1
        self._cur_lr = self.lr if lr is None else lr
        self._sq_accum = torch.zeros(1, dtype=torch.float32, device=self.engine.device)

    def step_unit(self, unit) -> None:
        """optimizer-in-backward: update one unit as soon as its gradients are reduced.  Clipping uses
        the previous step's global norm (the current one is not known until backward ends).

        On the GPU the update runs on a side stream: AdamW is bound by HBM bandwidth while the next layer's
        backward is bound by the tensor cores, so the two overlap; the step ends by joining the streams."""
        dev = self.engine.device
        if self._coef_for_step is None:
            self._coef_for_step = self._clip_coef(self._prev_norm) if self._prev_norm is not None else \
                torch.ones((), dtype=torch.float32, device=dev)
        coef = self._coef_for_step
        if dev.type != "cuda":
            for g in unit.groups:
                self._update_group(g, coef, self._cur_lr, sq_out=self._sq_accum)
            return
        if self._side is None:
            self._side = torch.cuda.Stream(device=dev)
        main = torch.cuda.current_stream(dev)
        self._side.wait_stream(main)
        for g in unit.groups:
            if self.fusable(g):                          # peers wait on this kernel: keep it on the main stream
                self._fused_rs_update(g, coef, self._cur_lr, self._sq_accum)
        with torch.cuda.stream(self._side):
            for g in unit.groups:
                if g.grad_shard is not None:
                    g.grad_shard.record_stream(self._side)
                self._update_group(g, coef, self._cur_lr, sq_out=self._sq_accum, background=True)

    def end_step_in_backward(self) -> torch.Tensor:
        if self._side is not None:
            torch.cuda.current_stream(self.engine.device).wait_stream(self._side)
        self._coef_for_step = None
        sq = self._sq_accum
        if dist.is_initialized() and dist.get_world_size() > 1:
            dist.all_reduce(sq)
        self._prev_norm = self.last_grad_norm = sq.sqrt().squeeze(0)
        return self.last_grad_norm

    def step(self, lr: float | None = None) -> torch.Tensor:
        self._new_weight_generation()
        self.step_count += 1
        lr = self.lr if lr is None else lr
        norm = self.global_grad_norm()
        self.last_grad_norm = norm
        coef = self._clip_coef(norm)
        for g in self.engine.all_groups():
            self._update_group(g, coef, lr)
        return norm

    # ---- checkpoint -----------------------------------------------------------------------
    def state_dict(self) -> dict:
        return {"step": self.step_count,
                "m": {k: m.state() for k, m in self.m.items()},
                "v": {k: v.state() for k, v in self.v.items()},
                "prev_norm": self._prev_norm}

    def load_state_dict(self, sd: dict) -> None:
        self.step_count = sd["step"]
        for k, st in sd["m"].items():
            for f, t in st.items():
                getattr(self.m[k], f).copy_(t)
        for k, st in sd["v"].items():
            for f, t in st.items():
                getattr(self.v[k], f).copy_(t)
        self._prev_norm = sd.get("prev_norm")


def lr_at(step: int, *, lr: float, min_lr: float, warmup: int, decay_iters: int, style: str,
          wsd_decay_iters: int = 0) -> float:
    """Learning rate for 1-based ``step``.  ``constant`` ignores decay; a launcher default must never
    silently change the schedule (``notes/2026-04/2026-04-28_gptoss_27_mlperf_legal_baseline.md:193-214``)."""
    if warmup > 0 and step <= warmup:
        return lr * step / warmup
    if style == "constant" or decay_iters <= 0:
        return lr
    t = min(max(step - warmup, 0) / max(decay_iters - warmup, 1), 1.0)
    if style == "cosine":
        return min_lr + 0.5 * (lr - min_lr) * (1 + math.cos(math.pi * t))
    if style == "linear":
        return lr + (min_lr - lr) * t
    if style == "wsd":
        # warm-up, stable, decay: flat at `lr` until the last `wsd_decay_iters` of `decay_iters`, then linear to min_lr
        tail = max(min(wsd_decay_iters, decay_iters - warmup), 1)
        into = step - (decay_iters - tail)
        return lr if into <= 0 else lr + (min_lr - lr) * min(into / tail, 1.0)
    raise ValueError(f"unknown lr_decay_style {style!r}")
