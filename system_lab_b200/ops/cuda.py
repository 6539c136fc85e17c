"""Kernel path of the op surface: ctypes bindings to ``lib/libslab_kernels.so`` wrapped in autograd
Functions.  bf16 activations only; a call with another dtype goes to the oracle explicitly (fp32
models are a CPU/plumbing configuration).  Missing library on a GPU machine is an error, never a
silent fallback.
"""
from __future__ import annotations

import ctypes
import os
from pathlib import Path

import torch

from . import reference as ref

_LIB_PATH = Path(__file__).resolve().parent.parent / "lib" / "libslab_kernels.so"
_lib = None

# p: pointer, i: int32, l: int64, f: float, s: stream
_SIGS = {
    "slab_rmsnorm_fwd": "ppppppiifs",
    "slab_rmsnorm_bwd_blocks": "i",
    "slab_rmsnorm_bwd": "pppppppppiis",
    "slab_rmsnorm_bwd_counters": "",
    "slab_swiglu_fwd": "ppplips",
    "slab_swiglu_bwd": "ppppplips",
    "slab_rope": "ppppliiillfs",
    "slab_quant_1x128": "ppplis",
    "slab_quant_128x128": "pppiiis",
    "slab_quant_rowwise": "ppplis",
    "slab_sumsq": "pilfps",
    "slab_adamw": "pipi" + "p" * 7 + "li" + "f" * 7 + "lis",
    "slab_router_topk": "ppppiiiiifs",
    "slab_router_fused_fwd": "ppppiiiiifpfps",
    "slab_router_fused_bwd": "pppppfpiiiiifs",
    "slab_ce_fwd_bwd": "pppiifs",
    "slab_grouped_gemm_bf16": "i" + "p" * 5 + "i" * 7 + "pii" + "ps",
    "slab_grouped_gemm_fp8": "p" * 7 + "iiiii" + "ps",
    "slab_grouped_gemm_fp8_rowwise": "p" * 7 + "iiiii" + "ps",
}
_CT = {"p": ctypes.c_void_p, "i": ctypes.c_int, "l": ctypes.c_long, "f": ctypes.c_float, "s": ctypes.c_void_p}


class KernelError(RuntimeError):
    pass


def lib():
    global _lib
    if _lib is None:
        if not _LIB_PATH.exists():
            raise KernelError(f"{_LIB_PATH} is missing: run `python -m system_lab_b200.csrc.build` "
                              "(or __graft_entry__.build()) before using the CUDA ops")
        _lib = ctypes.CDLL(str(_LIB_PATH))
        for name, sig in _SIGS.items():
            fn = getattr(_lib, name, None)
            if fn is None:
                continue
            fn.argtypes = [_CT[c] for c in sig]
            fn.restype = ctypes.c_int
    return _lib


def register(name: str, sig: str) -> None:
    """Used by other modules (dispatch, attention) to declare their entry points."""
    _SIGS[name] = sig
    if _lib is not None:
        fn = getattr(_lib, name, None)       # a library built before the entry point existed simply lacks it
        if fn is not None:
            fn.argtypes = [_CT[c] for c in sig]
            fn.restype = ctypes.c_int


def _ptr(t):
    if t is None:
        return None
    if isinstance(t, torch.Tensor):
        return t.data_ptr()
    return t


# kernels launched per entry point (entry points not listed launch one); LAUNCHES[0] counts launches
_KERNELS_PER_CALL = {}
LAUNCHES = [0]


_Tensor = torch.Tensor


def call(name: str, *args) -> int:
    # on the launch path of every kernel (about two thousand calls per training step): no helper calls per argument
    fn = getattr(_lib if _lib is not None else lib(), name)
    LAUNCHES[0] += _KERNELS_PER_CALL.get(name, 1)
    rc = fn(*[a.data_ptr() if isinstance(a, _Tensor) else a for a in args])
    if rc != 0:
        raise KernelError(f"{name} failed with code {rc}")
    return rc


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)
_raw_device = getattr(torch._C, "_cuda_getDevice", None)


def stream() -> int:
    """Handle of the current stream of the current device.  Asked once per kernel launch, so it goes to the two C
    entry points directly; ``torch.cuda.current_stream()`` builds a Python stream object and re-derives the device
    from the environment every time (about 8 us a call)."""
    if _raw_stream is not None and _raw_device is not None:
        return _raw_stream(_raw_device())
    return torch.cuda.current_stream().cuda_stream


_STATUS = {}
_STATUS_NAMES = {1: "TIMEOUT_FULL", 2: "TIMEOUT_EMPTY", 3: "TIMEOUT_TMEM_FULL", 4: "TIMEOUT_TMEM_EMPTY",
                 5: "TIMEOUT_PEER_FLAG", 6: "BAD_INDEX", 7: "CAPACITY"}


def status_word(device) -> torch.Tensor:
    """Per-device int32 the kernels write on a bounded-wait timeout or a failed bounds check."""
    key = str(device)
    if key not in _STATUS:
        _STATUS[key] = torch.zeros(1, dtype=torch.int32, device=device)
    return _STATUS[key]


class DeviceHang(RuntimeError):
    """A kernel's bounded wait ran out (failure kind HANG): the kernel returned, the context is usable."""


def peek_status(device=None) -> int:
    """Host read of the status word(s): the first non-zero code, 0 if every kernel so far was happy."""
    for key, t in _STATUS.items():
        if device is not None and key != str(device):
            continue
        v = int(t.item())
        if v:
            return v
    return 0


def status_name(code: int) -> str:
    return str(_STATUS_NAMES.get(code, code))


def clear_status(device=None) -> None:
    for key, t in _STATUS.items():
        if device is None or key == str(device):
            t.zero_()


def check_status(device=None) -> None:
    """Host read of the status word; raises a typed error.  Call between steps, not per kernel."""
    v = peek_status(device)
    if v:
        clear_status(device)
        raise DeviceHang(f"device kernel reported {status_name(v)} on {device if device is not None else 'a device'}")


def _bf16(*ts) -> bool:
    return all(t is None or t.dtype == torch.bfloat16 for t in ts)


# ------------------------------------------------------------------------------ RMSNorm
_NORM_SCRATCH = {}


def _norm_scratch(device, h: int):
    """Per (device, stream) scratch of the RMSNorm backward: fp32 partial rows (contents irrelevant) and the zeroed
    ticket counters of its in-kernel reduction (every launch leaves them zero).  Calls on one stream run in order,
    so they can share both; another stream gets its own."""
    key = (str(device), stream())
    ent = _NORM_SCRATCH.get(key)
    if ent is None or ent[0].shape[1] < h:
        nb = lib().slab_rmsnorm_bwd_blocks(0)
        part = torch.empty(nb, max(h, 2048), dtype=torch.float32, device=device)
        counters = ent[1] if ent is not None else torch.zeros(lib().slab_rmsnorm_bwd_counters(), dtype=torch.int32,
                                                              device=device)
        ent = (part, counters)
        _NORM_SCRATCH[key] = ent
    return ent


class _RMSNorm(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, eps):
        shp = x.shape
        x2 = x.reshape(-1, shp[-1]).contiguous()
        rows, h = x2.shape
        y = torch.empty_like(x2)
        rstd = torch.empty(rows, dtype=torch.float32, device=x.device)
        call("slab_rmsnorm_fwd", x2, None, w, y, None, rstd, rows, h, float(eps), stream())
        ctx.save_for_backward(x2, w, rstd)
        ctx.shp = shp
        return y.reshape(shp)

    @staticmethod
    def backward(ctx, g):
        x2, w, rstd = ctx.saved_tensors
        rows, h = x2.shape
        g2 = g.reshape(rows, h).contiguous()
        part, counters = _norm_scratch(g.device, h)
        dx = torch.empty_like(x2)
        dw = torch.empty_like(w)
        call("slab_rmsnorm_bwd", g2, x2, w, rstd, None, dx, part, counters, dw, rows, h, stream())
        return dx.reshape(ctx.shp), dw, None


class _RMSNormResidual(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, res, w, eps):
        shp = x.shape
        x2 = x.reshape(-1, shp[-1]).contiguous()
        r2 = res.reshape(-1, shp[-1]).contiguous()
        rows, h = x2.shape
        y = torch.empty_like(x2)
        xpr = torch.empty_like(x2)
        rstd = torch.empty(rows, dtype=torch.float32, device=x.device)
        call("slab_rmsnorm_fwd", x2, r2, w, y, xpr, rstd, rows, h, float(eps), stream())
        ctx.save_for_backward(xpr, w, rstd)
        ctx.shp = shp
        return y.reshape(shp), xpr.reshape(shp)

    @staticmethod
    def backward(ctx, gy, gxpr):
        xpr, w, rstd = ctx.saved_tensors
        rows, h = xpr.shape
        gy2 = gy.reshape(rows, h).contiguous()
        gx2 = gxpr.reshape(rows, h).contiguous() if gxpr is not None else None
        part, counters = _norm_scratch(gy.device, h)
        dx = torch.empty_like(xpr)
        dw = torch.empty_like(w)
        call("slab_rmsnorm_bwd", gy2, xpr, w, rstd, gx2, dx, part, counters, dw, rows, h, stream())
        dx = dx.reshape(ctx.shp)
        return dx, dx, dw, None          # the same tensor is the gradient of x and of the residual


def rmsnorm(x, w, eps):
    if not _bf16(x, w):
        return ref.rmsnorm(x, w, eps)
    return _RMSNorm.apply(x, w, eps)


def rmsnorm_residual(x, res, w, eps):
    if not _bf16(x, res, w):
        return ref.rmsnorm_residual(x, res, w, eps)
    return _RMSNormResidual.apply(x, res, w, eps)


# ------------------------------------------------------------------------------ RoPE
class _Rope(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, cos, sin):
        b, s, hh, d = x.shape
        xc = x.contiguous()
        y = torch.empty_like(xc)
        ctx.save_for_backward(cos, sin)
        call("slab_rope", xc, cos, sin, y, b * s, s, hh, d, hh * d, hh * d, 1.0, stream())
        return y

    @staticmethod
    def backward(ctx, g):
        cos, sin = ctx.saved_tensors
        b, s, hh, d = g.shape
        gc = g.contiguous()
        out = torch.empty_like(gc)
        call("slab_rope", gc, cos, sin, out, b * s, s, hh, d, hh * d, hh * d, -1.0, stream())
        return out, None, None


def rope(x, cos, sin):
    if not _bf16(x) or x.shape[-1] % 16:
        return ref.rope(x, cos, sin)
    return _Rope.apply(x, cos.contiguous(), sin.contiguous())


class _RopePackedInplace(torch.autograd.Function):
    """Rotates the first ``n_heads`` heads of every row of a packed ``[B, S, W]`` buffer in place (the q and
    k heads of a fused qkv projection); the remaining columns (v) are untouched."""

    @staticmethod
    def forward(ctx, qkv, cos, sin, n_heads, d):
        b, s, w = qkv.shape
        ctx.save_for_backward(cos, sin)
        ctx.meta = (n_heads, d)
        call("slab_rope", qkv, cos, sin, qkv, b * s, s, n_heads, d, w, w, 1.0, stream())
        ctx.mark_dirty(qkv)
        return qkv

    @staticmethod
    def backward(ctx, g):
        cos, sin = ctx.saved_tensors
        n_heads, d = ctx.meta
        g = g.contiguous()
        b, s, w = g.shape
        call("slab_rope", g, cos, sin, g, b * s, s, n_heads, d, w, w, -1.0, stream())
        return g, None, None, None, None


def rope_packed(qkv, cos, sin, n_heads, d):
    if not _bf16(qkv) or d % 16 or not qkv.is_contiguous():
        return None
    return _RopePackedInplace.apply(qkv, cos.contiguous(), sin.contiguous(), n_heads, d)


# ------------------------------------------------------------------------------ SwiGLU
class _SwiGLU(torch.autograd.Function):
    @staticmethod
    def forward(ctx, gu, probs, rows_dev):
        shp = gu.shape
        g2 = gu.reshape(-1, shp[-1]).contiguous()
        rows, f2 = g2.shape
        out = torch.empty(rows, f2 // 2, dtype=gu.dtype, device=gu.device)
        call("slab_swiglu_fwd", g2, probs, out, rows, f2 // 2, rows_dev, stream())
        ctx.save_for_backward(g2, probs, rows_dev)
        ctx.shp = shp
        return out.reshape(*shp[:-1], f2 // 2)

    @staticmethod
    def backward(ctx, g):
        g2, probs, rows_dev = ctx.saved_tensors
        rows, f2 = g2.shape
        gc = g.reshape(rows, f2 // 2).contiguous()
        dgu = torch.empty_like(g2)
        dp = torch.empty(rows, dtype=torch.float32, device=g.device) if probs is not None else None
        call("slab_swiglu_bwd", gc, g2, probs, dgu, dp, rows, f2 // 2, rows_dev, stream())
        return dgu.reshape(ctx.shp), dp, None


def swiglu(gate_up):
    if not _bf16(gate_up) or gate_up.shape[-1] % 16:
        return ref.swiglu(gate_up)
    return _SwiGLU.apply(gate_up, None, None)


def swiglu_probs(gate_up, probs, rows_dev=None):
    """``rows_dev``: optional device int32 holding the number of rows in use (rows past it are left
    uninitialised: they are capacity slack no consumer reads)."""
    if not _bf16(gate_up) or gate_up.shape[-1] % 16:
        return ref.swiglu_probs(gate_up, probs)
    return _SwiGLU.apply(gate_up, probs.float().contiguous(), rows_dev)


# ------------------------------------------------------------------------------ router
class _RouterTopK(torch.autograd.Function):
    @staticmethod
    def forward(ctx, logits, topk, score_function, bias, norm, scaling):
        t, e = logits.shape
        lc = logits.contiguous()
        w = torch.empty(t, topk, dtype=torch.float32, device=logits.device)
        idx = torch.empty(t, topk, dtype=torch.int32, device=logits.device)
        call("slab_router_topk", lc, bias, w, idx, t, e, topk, 0 if score_function == "softmax" else 1,
             1 if norm else 0, float(scaling), stream())
        ctx.save_for_backward(lc, idx)
        ctx.cfg = (score_function, norm, scaling)
        ctx.mark_non_differentiable(idx)
        return w, idx

    @staticmethod
    def backward(ctx, gw, _gidx):
        logits, idx = ctx.saved_tensors
        score_function, norm, scaling = ctx.cfg
        with torch.enable_grad():
            lg = logits.detach().requires_grad_(True)
            scores = torch.softmax(lg, -1) if score_function == "softmax" else torch.sigmoid(lg)
            w = torch.gather(scores, 1, idx.long())
            if norm:
                w = w / (w.sum(-1, keepdim=True) + 1e-20)
            w = w * scaling
            (gl,) = torch.autograd.grad(w, lg, gw)
        return gl, None, None, None, None, None


class _RouterFused(torch.autograd.Function):
    """Score function, selection bias, top-k, gate normalisation, per-expert load counts and the load-balancing loss
    in one launch; its backward (gate-weight path plus the dense loss term through the score function) in one more.
    The fused router with aux score of ``notes/2026-04/2026-04-25_gptoss_22_sync_free_moe_stage_audit.md:118-127``."""

    @staticmethod
    def forward(ctx, logits, topk, score_function, bias, norm, scaling, aux_coeff):
        t, e = logits.shape
        lc = logits.contiguous()
        dev = logits.device
        w = torch.empty(t, topk, dtype=torch.float32, device=dev)
        idx = torch.empty(t, topk, dtype=torch.int32, device=dev)
        e2 = e + (e & 1)
        stats = torch.zeros(e2 + 2 * e + 2, dtype=torch.int32, device=dev)   # counts | 64-bit score sums | ticket
        aux = torch.empty(1, dtype=torch.float32, device=dev)
        sc = 0 if score_function == "softmax" else 1
        call("slab_router_fused_fwd", lc, bias, w, idx, t, e, topk, sc, 1 if norm else 0, float(scaling), stats,
             float(aux_coeff), aux, stream())
        counts = stats[:e]
        ctx.save_for_backward(lc, idx, counts)
        ctx.cfg = (topk, sc, norm, float(scaling), float(aux_coeff))
        ctx.mark_non_differentiable(idx, counts)
        return w, idx, aux.squeeze(0), counts

    @staticmethod
    def backward(ctx, gw, _gidx, g_aux, _gcounts):
        logits, idx, counts = ctx.saved_tensors
        topk, sc, norm, scaling, aux_coeff = ctx.cfg
        t, e = logits.shape
        dl = torch.empty_like(logits)
        gw = gw.contiguous() if gw is not None else torch.zeros(t, topk, dtype=torch.float32, device=logits.device)
        use_aux = g_aux is not None and aux_coeff != 0.0
        ga = g_aux.float().reshape(1).contiguous() if use_aux else None
        call("slab_router_fused_bwd", logits, idx, gw, counts if use_aux else None, ga, aux_coeff, dl, t, e, topk, sc,
             1 if norm else 0, scaling, stream())
        return dl, None, None, None, None, None, None


def router_fused(logits, topk, score_function, bias, norm_topk_prob, scaling_factor, aux_coeff):
    """``(weights [T, K] fp32, idx [T, K] int32, aux scalar, counts [E] int32)``; see :class:`_RouterFused`."""
    return _RouterFused.apply(logits.float(), topk, score_function,
                              bias.float().contiguous() if bias is not None else None, norm_topk_prob,
                              scaling_factor, aux_coeff)


class _RouterLogits(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w):
        ctx.save_for_backward(x, w)
        if not x.is_cuda:                      # the fp32-output GEMM variant exists on the GPU only
            return x.float() @ w.float().t()
        return torch.mm(x, w.t(), out_dtype=torch.float32)

    @staticmethod
    def backward(ctx, g):
        x, w = ctx.saved_tensors
        gb = g.to(torch.bfloat16)
        return gb @ w, gb.t() @ x


def router_logits(x, w):
    return _RouterLogits.apply(x, w)


def router_topk(logits, topk, score_function, bias, norm_topk_prob, scaling_factor):
    lf = logits.float()
    w, idx = _RouterTopK.apply(lf, topk, score_function, bias.float().contiguous() if bias is not None else None,
                               norm_topk_prob, scaling_factor)
    return w, idx, None


# ------------------------------------------------------------------------------ grouped GEMM
def _check_segments(offsets, counts):
    if offsets.dtype != torch.int32:
        offsets = offsets.to(torch.int32)
    if counts.dtype != torch.int32:
        counts = counts.to(torch.int32)
    return offsets.contiguous(), counts.contiguous()


def grouped_gemm_raw(mode: int, a, b, offsets, counts, n: int, k: int, out=None, accumulate=False,
                     block_n: int = 256, max_ctas: int = 0, ready=None):
    """mode 0: out[R,N] = a[R,K] @ b[e]^T ; 1: out[R,K] = a[R,N] @ b[e] ; 2: out[E,N,K] = a[R,N]^T @ b[R,K].

    ``ready`` (modes 0 and 1): arrival flags of the row operand (an object with ``flags`` int32 [world, E], ``world``,
    ``epoch`` and ``mark_consumed()``): the kernel waits per expert for every source instead of the caller waiting
    for the whole exchange."""
    e = offsets.numel()
    r = a.shape[0]
    if out is None:
        if mode == 0:
            out = torch.empty(r, n, dtype=torch.bfloat16, device=a.device)
        elif mode == 1:
            out = torch.empty(r, k, dtype=torch.bfloat16, device=a.device)
        else:
            out = torch.empty(e, n, k, dtype=torch.bfloat16, device=a.device)
    if ready is not None and mode != 2:
        call("slab_grouped_gemm_bf16", mode, a, b, out, offsets, counts, e, r, n, k, 1 if accumulate else 0,
             block_n, int(getattr(ready, "gemm_max_ctas", 0) or max_ctas), ready.flags, int(ready.world),
             int(ready.epoch), status_word(a.device), stream())
        ready.mark_consumed()
        ready.d.join_side()              # the remote half of the exchange, held back until this launch, starts now
        return out
    if ready is not None:
        ready.wait()
    call("slab_grouped_gemm_bf16", mode, a, b, out, offsets, counts, e, r, n, k, 1 if accumulate else 0,
         block_n, max_ctas, None, 0, 0, status_word(a.device), stream())
    return out


def grouped_gemm_fp8_raw(a_q, sa, b_q, sb, offsets, counts, out=None, max_ctas: int = 0):
    """Block-scaled fp8 forward: ``out[R, N] = (a_q * sa) @ (b_q[e] * sb[e])^T`` with ``a_q [R, K]`` e4m3 +
    ``sa [R, K/128]`` and ``b_q [E, N, K]`` e4m3 + ``sb [E, N/128, K/128]``; bf16 result."""
    e, n, k = b_q.shape
    r = a_q.shape[0]
    if out is None:
        out = torch.empty(r, n, dtype=torch.bfloat16, device=a_q.device)
    call("slab_grouped_gemm_fp8", a_q, sa, b_q, sb, out, offsets, counts, e, r, n, k, max_ctas,
         status_word(a_q.device), stream())
    return out


def grouped_gemm_fp8_rowwise_raw(a_q, sa, b_q, sb, offsets, counts, out=None, max_ctas: int = 0):
    """Row-scaled fp8 forward: ``out[r, n] = sa[r] * sb[e, n] * sum_k a_q[r, k] * b_q[e, n, k]`` with one scale
    per activation row (``sa [R]``) and one per expert output channel (``sb [E, N]``); bf16 result.  The scales
    are constant along K, so the kernel accumulates all of K in TMEM at the fp8 tensor rate."""
    e, n, k = b_q.shape
    r = a_q.shape[0]
    if out is None:
        out = torch.empty(r, n, dtype=torch.bfloat16, device=a_q.device)
    call("slab_grouped_gemm_fp8_rowwise", a_q, sa, b_q, sb, out, offsets, counts, e, r, n, k, max_ctas,
         status_word(a_q.device), stream())
    return out


def _pick_bn(cols: int) -> int:
    return 256 if cols % 256 == 0 or cols > 1024 else 128


class _GroupedLinear(torch.autograd.Function):
    """``out = a @ w[e]^T`` per expert segment.  Two fusions on the backward side:

    * if the weight carries ``main_grad`` (a view of the flat gradient buffer set by the FSDP engine), wgrad
      writes or accumulates straight into it and autograd sees no weight gradient (no zero fill, no add);
    * ``dgrad_out`` names the buffer the input gradient is written to (the dispatcher's peer-visible
      buffer, so the backward of dispatch needs no staging copy).
    """

    @staticmethod
    def forward(ctx, a, w, offsets, counts, out=None, dgrad_out=None, dead=False, ready=None, bwd_ready=None):
        e, n, k = w.shape
        a = a.contiguous()
        w = w.contiguous() if not w.is_contiguous() else w
        push = out if hasattr(out, "launch") else None      # a dispatcher PushTarget: rows go to the token owners
        if push is not None:
            out = None
        ctx.bwd_ready = bwd_ready            # source of the arrival flags of this node's incoming gradient rows
        if ready is not None and (dead or push is not None):
            ready.wait()                     # no kernel here takes the flags: wait for the whole exchange
            ready = None
        if dead or push is not None:
            # node only: the caller never reads the product (recomputed forward), or the rows leave through the
            # push epilogue; either way the returned tensor is a shape carrier without storage behind every row
            if push is not None and not dead:
                push.launch(0, a, w, offsets, counts, n, k, _pick_bn(n))
            out = out if out is not None else torch.empty(1, dtype=torch.bfloat16, device=a.device).expand(a.shape[0], n)
        else:
            out = grouped_gemm_raw(0, a, w, offsets, counts, n, k, out=out, block_n=_pick_bn(n), ready=ready)
        ctx.save_for_backward(a, w, offsets, counts)
        ctx.w_ref = w
        ctx.dgrad_out = dgrad_out
        # a caller-provided buffer may hold more rows than the operand (capacity-sized peer buffer, kept rows):
        # the result, and therefore the gradient autograd hands back, has exactly the operand's rows
        return out[:a.shape[0]] if out.shape[0] != a.shape[0] else out

    @staticmethod
    def backward(ctx, g):
        a, w, offsets, counts = ctx.saved_tensors
        e, n, k = w.shape
        # the gradient rows may still be arriving from the peers (backward of combine): the dgrad kernel waits for
        # them expert by expert; anything else waits for all of them first
        src = getattr(ctx, "bwd_ready", None)
        rdy = src.take_bwd_ready() if src is not None else None
        if rdy is not None and not g.is_contiguous():
            rdy.wait()
            rdy = None
        g = g.contiguous()
        da = dw = None
        if ctx.needs_input_grad[0]:
            do = ctx.dgrad_out
            if hasattr(do, "launch"):                  # PushTarget: the input gradient goes to the token owners
                if rdy is not None:
                    rdy.wait()
                    rdy = None
                do.launch(1, g, w, offsets, counts, n, k, _pick_bn(k))
                da = torch.empty(1, dtype=torch.bfloat16, device=g.device).expand(g.shape[0], k)
            else:
                if do is not None and (do.shape[0] < g.shape[0] or do.shape[1] != k):
                    do = None
                da = grouped_gemm_raw(1, g, w, offsets, counts, n, k, out=do, block_n=_pick_bn(k), ready=rdy)
                rdy = None
                if src is not None:
                    src.join_side()          # the side-stream half of the gradient scatter, if there was one
                if do is not None:
                    da = do[:g.shape[0]]
        if rdy is not None:
            rdy.wait()
        if ctx.needs_input_grad[1]:
            mg = getattr(ctx.w_ref, "main_grad", None)
            if mg is not None:
                grouped_gemm_raw(2, g, a, offsets, counts, n, k, out=mg, accumulate=ctx.w_ref.main_grad_written,
                                 block_n=_pick_bn(k))
                ctx.w_ref.main_grad_written = True
            else:
                dw = grouped_gemm_raw(2, g, a, offsets, counts, n, k, block_n=_pick_bn(k))
        return da, dw, None, None, None, None, None, None, None


_WT_CACHE = {}
FP8_DGRAD = [False]
WEIGHT_GENERATION = [0]      # bumped by the optimizer every step: kernels update weights without autograd noticing


def set_fp8_dgrad(on: bool) -> None:
    """Input gradients of the fp8 expert GEMMs in e4m3 too (row-scaled recipe; weight gradients stay bf16)."""
    FP8_DGRAD[0] = bool(on)


def _transposed_rowwise_weight(w):
    """e4m3 copy of ``w`` in the layout its input gradient needs: ``[E, K, N]`` with one scale per (expert, k) row, so
    the reduction over N keeps constant scales.  Cached per weight storage and version: it is rebuilt once after each
    optimizer step, not per GEMM (the NK-layout cache of ``summary/fp8_expert_gemm_optimization.md:107-116``)."""
    key = (w.data_ptr(), tuple(w.shape))
    ver = (w._version, WEIGHT_GENERATION[0])
    ent = _WT_CACHE.get(key)
    if ent is None or ent[0] != ver:
        if len(_WT_CACHE) > 512:
            _WT_CACHE.clear()
        q, s = quant_rowwise(w.transpose(1, 2).contiguous())
        ent = (ver, q, s.contiguous())
        _WT_CACHE[key] = ent
    return ent[1], ent[2]


def grouped_gemm_fp8_dgrad_rowwise(g, w, offsets, counts, out=None):
    """``da[r, k] = sum_n g[r, n] * w[e, n, k]`` on the fp8 tensor path: ``g`` quantised per row, ``w`` per (expert, k)
    from its cached transposed copy, the row-scaled forward kernel run with N as the reduction."""
    gq, gs = quant_rowwise(g)
    wq, ws = _transposed_rowwise_weight(w)
    return grouped_gemm_fp8_rowwise_raw(gq, gs, wq, ws, offsets, counts, out=out)


class _GroupedLinearFp8(torch.autograd.Function):
    """Forward in e4m3 on the tensor cores' fp8 path, backward in bf16 on the saved bf16 operands (the reference's
    fused fp8 grouped GEMM keeps dW in bf16 too, ``summary/fp8_expert_gemm_optimization.md:137-143``).  Operands
    are quantised on the fly: activations per row, weights per output channel (``recipe == "rowwise"``, scales
    constant along K so the kernel accumulates all of K in TMEM), or 1x128 / 128x128 blocks (``"blockwise"``)."""

    @staticmethod
    def forward(ctx, a, w, offsets, counts, recipe, out=None, dgrad_out=None, ready=None, bwd_ready=None):
        e, n, k = w.shape
        a = a.contiguous()
        w = w.contiguous() if not w.is_contiguous() else w
        ctx.bwd_ready = bwd_ready
        if ready is not None:
            ready.wait()                     # the quantiser reads every row
        if recipe == "blockwise":
            aq, sa = quant_1x128(a)
            wq, sw = quant_128x128(w)
            out = grouped_gemm_fp8_raw(aq, sa.contiguous(), wq, sw.contiguous(), offsets, counts, out=out)
        elif recipe == "tensorwise":
            # one scale per tensor: a special case of the row-scaled kernel (all row / channel scales equal)
            aq, s_a = quant_tensorwise(a)
            wq, s_w = quant_tensorwise(w)
            out = grouped_gemm_fp8_rowwise_raw(aq, s_a.expand(a.shape[0]).contiguous(), wq,
                                               s_w.expand(e, n).contiguous(), offsets, counts, out=out)
        else:
            aq, sa = quant_rowwise(a)
            wq, sw = quant_rowwise(w)
            out = grouped_gemm_fp8_rowwise_raw(aq, sa, wq, sw.contiguous(), offsets, counts, out=out)
        ctx.save_for_backward(a, w, offsets, counts)
        ctx.w_ref = w
        ctx.dgrad_out = dgrad_out
        return out[:a.shape[0]] if out.shape[0] != a.shape[0] else out

    @staticmethod
    def backward(ctx, g):
        a, w, offsets, counts = ctx.saved_tensors
        e, n, k = w.shape
        if (FP8_DGRAD[0] and ctx.needs_input_grad[0] and not hasattr(ctx.dgrad_out, "launch") and n % 128 == 0
                and k % 64 == 0 and getattr(ctx, "bwd_ready", None) is None):
            # input gradient in e4m3 (row-scaled), weight gradient in bf16 on the saved bf16 operands
            g = g.contiguous()
            do = ctx.dgrad_out
            if do is not None and (do.shape[0] < g.shape[0] or do.shape[1] != k):
                do = None
            da = grouped_gemm_fp8_dgrad_rowwise(g, w, offsets, counts, out=do)
            da = da[:g.shape[0]]
            dw = None
            if ctx.needs_input_grad[1]:
                mg = getattr(ctx.w_ref, "main_grad", None)
                if mg is not None:
                    grouped_gemm_raw(2, g, a, offsets, counts, n, k, out=mg, accumulate=ctx.w_ref.main_grad_written,
                                     block_n=_pick_bn(k))
                    ctx.w_ref.main_grad_written = True
                else:
                    dw = grouped_gemm_raw(2, g, a, offsets, counts, n, k, block_n=_pick_bn(k))
            return (da, dw) + (None,) * 7
        return _GroupedLinear.backward(ctx, g)          # same arity: (da, dw) + one None per remaining input


def _fp8_recipe(fp8) -> str:
    """``fp8`` as passed down from the model: False / "" = bf16; True = the default recipe; a string names one."""
    if not fp8:
        return ""
    return fp8 if isinstance(fp8, str) else "rowwise"


# the weights' N must be a multiple of 64; with N % 128 == 64 (hidden 2880, MLA's 576-wide projection) wgrad writes
# its last row tile with guarded stores
_N_MULTIPLE = 64


def grouped_kernel_ok(a, w) -> bool:
    """Shapes and dtypes the tcgen05 grouped GEMM takes (everything else goes to the library loop)."""
    return _bf16(a, w) and w.shape[2] % 64 == 0 and w.shape[1] % _N_MULTIPLE == 0


def grouped_linear(a, w, offsets, counts, fp8=False, out=None, dgrad_out=None, dead: bool = False, ready=None,
                   bwd_ready=None):
    """``ready``: arrival flags of ``a``'s rows (see ``grouped_gemm_raw``); ``bwd_ready``: the dispatcher that will hold
    the arrival flags of this node's incoming gradient rows when backward runs (``take_bwd_ready()``)."""
    e, n, k = w.shape
    if not grouped_kernel_ok(a, w):
        if ready is not None:
            ready.wait()
        from . import _GroupedLinearRef
        return _GroupedLinearRef.apply(a, w, offsets, counts, dead)
    offsets, counts = _check_segments(offsets, counts)
    if out is not None and not hasattr(out, "launch") and \
            (out.dtype != torch.bfloat16 or out.shape[0] < a.shape[0] or out.shape[1] != n):
        out = None
    recipe = _fp8_recipe(fp8)
    fp8_ok = recipe and not dead and not hasattr(out, "launch") and \
        (k % 128 == 0 and n % (128 if recipe == "blockwise" else 64) == 0)          # rowwise / tensorwise share a kernel
    if fp8_ok:           # a pushed output stays on the bf16 kernel: the fp8 kernels store through TMA only
        res = _GroupedLinearFp8.apply(a, w, offsets, counts, recipe, out, dgrad_out, ready, bwd_ready)
    else:
        res = _GroupedLinear.apply(a, w, offsets, counts, out, dgrad_out, dead, ready, bwd_ready)
    return res[:a.shape[0]] if res.shape[0] != a.shape[0] else res


# ------------------------------------------------------------------------------ dense linear on the same kernel
_DENSE_SEG = {}


def _dense_segments(device, rows: int):
    """A dense GEMM is the grouped GEMM with one segment that starts at row 0: ``(offsets [1], counts [1])``."""
    key = (str(device), rows)
    seg = _DENSE_SEG.get(key)
    if seg is None:
        if len(_DENSE_SEG) > 256:
            _DENSE_SEG.clear()
        seg = (torch.zeros(1, dtype=torch.int32, device=device),
               torch.full((1,), rows, dtype=torch.int32, device=device))
        _DENSE_SEG[key] = seg
    return seg


class _Linear(torch.autograd.Function):
    """``y = x @ w^T`` for the dense projections (attention qkv / output, dense and shared-expert feed-forward, MLA
    low-rank projections) on the tcgen05 kernel of the expert GEMMs run with a single segment: forward, input
    gradient (the weight read as an MN-major operand, no transposed copy) and weight gradient (both operands
    MN-major), the last one written or accumulated straight into the flat gradient buffer when the parameter
    carries ``main_grad``."""

    @staticmethod
    def forward(ctx, x, w, gather=None):
        shp = x.shape
        n, k = w.shape
        x2 = x.reshape(-1, k)
        if not x2.is_contiguous():
            x2 = x2.contiguous()
        off, cnt = _dense_segments(x.device, x2.shape[0])
        # the result is allocated in its final shape (callers rotate q and k in place: it must not be a view made here)
        out = torch.empty(*shp[:-1], n, dtype=torch.bfloat16, device=x.device)
        if gather is not None:
            # FSDP all-gather fused into this GEMM: the kernel's gather warps pull the flat buffer's matrices from the
            # ranks' staged shards while its tiles are multiplied (csrc/gemm_tcgen05.cu, GATHER)
            gather["comm"].gemm_gather(gather["ticket"], x2, w, out.view(-1, n), gather["flat"], gather["w_off"],
                                       (off, cnt), gather["pieces"], gather["call"], _pick_bn(n))
        else:
            grouped_gemm_raw(0, x2, w, off, cnt, n, k, out=out.view(-1, n), block_n=_pick_bn(n))
        ctx.save_for_backward(x2, w, off, cnt)
        ctx.w_ref = w
        ctx.shp = shp
        return out

    @staticmethod
    def backward(ctx, g):
        x2, w, off, cnt = ctx.saved_tensors
        n, k = w.shape
        g2 = g.reshape(-1, n)
        if not g2.is_contiguous():
            g2 = g2.contiguous()
        dx = dw = None
        if ctx.needs_input_grad[0]:
            dx = torch.empty(ctx.shp, dtype=torch.bfloat16, device=g.device)
            grouped_gemm_raw(1, g2, w, off, cnt, n, k, out=dx.view(-1, k), block_n=_pick_bn(k))
        if ctx.needs_input_grad[1]:
            mg = getattr(ctx.w_ref, "main_grad", None)
            if mg is not None:
                grouped_gemm_raw(2, g2, x2, off, cnt, n, k, out=mg, accumulate=ctx.w_ref.main_grad_written,
                                 block_n=_pick_bn(k))
                ctx.w_ref.main_grad_written = True
            else:
                dw = grouped_gemm_raw(2, g2, x2, off, cnt, n, k, block_n=_pick_bn(k)).view(n, k)
        return dx, dw, None


def linear_ok(x, w) -> bool:
    return (_bf16(x, w) and w.dim() == 2 and x.shape[-1] == w.shape[1] and w.shape[1] % 64 == 0
            and w.shape[0] % _N_MULTIPLE == 0 and x.numel() > 0 and w.is_contiguous())


def linear(x, w, gather=None):
    return _Linear.apply(x, w, gather)


# ------------------------------------------------------------------------------ attention
def causal_attention(q, k, v, scale, window):
    from .attention import causal_attention as impl
    return impl(q, k, v, scale, window)


# ------------------------------------------------------------------------------ linear + cross entropy
class _LinearCE(torch.autograd.Function):
    """loss = mean CE(h @ W^T, targets), chunked over rows: logits of one chunk are produced by the tcgen05 GEMM
    (one segment), turned into their own gradient in place by one kernel, and consumed by the two gradient GEMMs
    (input gradient; weight gradient overwriting on the first chunk, accumulating on later ones) before the next
    chunk, so at most ``chunk_rows x vocab`` logits exist at a time."""

    @staticmethod
    def forward(ctx, h, weight, targets, chunk_rows):
        n, hd = h.shape
        v = weight.shape[0]
        loss_sum = torch.zeros(1, dtype=torch.float32, device=h.device)
        dh = torch.empty_like(h)
        need_dw = ctx.needs_input_grad[1]            # a frozen projection (LoRA fine-tuning) needs no weight gradient
        dw = torch.zeros_like(weight) if need_dw else None
        gscale = 1.0 / n
        from . import dense_kernels
        own = dense_kernels() and hd % 64 == 0 and v % _N_MULTIPLE == 0
        if own and need_dw:
            dw = torch.empty_like(weight)            # the first chunk's wgrad overwrites, later chunks accumulate
        for lo in range(0, n, chunk_rows):
            hi = min(lo + chunk_rows, n)
            if own:
                off, cnt = _dense_segments(h.device, hi - lo)
                hc = h[lo:hi]
                logits = grouped_gemm_raw(0, hc, weight, off, cnt, v, hd, block_n=256)
                call("slab_ce_fwd_bwd", logits, targets[lo:hi].contiguous(), loss_sum, hi - lo, v, gscale, stream())
                grouped_gemm_raw(1, logits, weight, off, cnt, v, hd, out=dh[lo:hi], block_n=_pick_bn(hd))
                if need_dw:
                    grouped_gemm_raw(2, logits, hc, off, cnt, v, hd, out=dw, accumulate=lo > 0, block_n=_pick_bn(hd))
                continue
            logits = h[lo:hi] @ weight.t()
            call("slab_ce_fwd_bwd", logits, targets[lo:hi].contiguous(), loss_sum, hi - lo, v, gscale, stream())
            torch.mm(logits, weight, out=dh[lo:hi])
            if need_dw:
                dw.addmm_(logits.t(), h[lo:hi])
        ctx.save_for_backward(dh, dw)
        return (loss_sum / n).squeeze(0)

    @staticmethod
    def backward(ctx, g):
        dh, dw = ctx.saved_tensors
        return dh * g.to(dh.dtype), (dw * g.to(dw.dtype) if dw is not None else None), None, None


def linear_cross_entropy(h, weight, targets, chunk_rows: int = 8192):
    if not _bf16(h, weight) or weight.shape[0] % 8:
        return ref.linear_cross_entropy(h, weight, targets)
    return _LinearCE.apply(h.contiguous(), weight.contiguous(), targets.contiguous(), chunk_rows)


# ------------------------------------------------------------------------------ quantisation
def quant_1x128(x):
    if not _bf16(x):
        return ref.quant_1x128(x)
    shp = x.shape
    x2 = x.reshape(-1, shp[-1]).contiguous()
    q = torch.empty(x2.shape, dtype=torch.float8_e4m3fn, device=x.device)
    s = torch.empty(x2.shape[0], shp[-1] // 128, dtype=torch.float32, device=x.device)
    call("slab_quant_1x128", x2, q, s, x2.shape[0], shp[-1], stream())
    return q.reshape(shp), s.reshape(*shp[:-1], shp[-1] // 128)


def quant_rowwise(x):
    """e4m3 with one fp32 scale per row of the last dimension: returns ``(q, scale[...])``."""
    if not _bf16(x):
        return ref.quant_rowwise(x)
    shp = x.shape
    x2 = x.reshape(-1, shp[-1]).contiguous()
    q = torch.empty(x2.shape, dtype=torch.float8_e4m3fn, device=x.device)
    s = torch.empty(x2.shape[0], dtype=torch.float32, device=x.device)
    call("slab_quant_rowwise", x2, q, s, x2.shape[0], shp[-1], stream())
    return q.reshape(shp), s.reshape(shp[:-1])


def quant_tensorwise(x):
    """e4m3 with a single fp32 scale for the whole tensor (current scaling: the scale comes from this tensor's own
    absolute maximum, no history).  Library elementwise kernels; the row-scaled recipe is the fused one."""
    return ref.quant_tensorwise(x)


def quant_128x128(w):
    if not _bf16(w):
        return ref.quant_128x128(w)
    *lead, n, k = w.shape
    mats = 1
    for d in lead:
        mats *= d
    wc = w.contiguous()
    q = torch.empty(wc.shape, dtype=torch.float8_e4m3fn, device=w.device)
    s = torch.empty(*lead, n // 128, k // 128, dtype=torch.float32, device=w.device)
    call("slab_quant_128x128", wc, q, s, mats, n, k, stream())
    return q, s


# ------------------------------------------------------------------------------ optimizer
def sumsq(g: torch.Tensor, scale: float, out: torch.Tensor) -> None:
    """``out += scale * sum(g^2)`` for an fp32 or bf16 flat tensor (no host sync)."""
    call("slab_sumsq", g, 1 if g.dtype == torch.bfloat16 else 0, g.numel(), float(scale), out, stream())


_KIND = {"fp32": 0, "bf16": 1, "fp8": 2}


_ADAMW_PIECE = [1 << 25]    # elements per launch of a background update (csrc/elementwise.cu); 0 = one launch


def set_adamw_background_piece(elements: int) -> None:
    """A side-stream AdamW update is cut into launches of this many elements (a multiple of 512; 0: one launch), so
    that a compute-stream kernel with large blocks waits for one piece at most before it finds room on the SMs."""
    register("slab_set_adamw_background_piece", "l")
    rc = lib().slab_set_adamw_background_piece(int(elements))
    if rc != 0:
        raise KernelError(f"slab_set_adamw_background_piece({elements}) failed with code {rc}")
    _ADAMW_PIECE[0] = int(elements)


def adamw_flat(group, m, v, coef, *, lr, beta1, beta2, eps, weight_decay, step, sq_out=None,
               ctas_per_sm: int = 0) -> None:
    """Fused AdamW on one flat shard: reads the (fp32 or bf16) gradient shard, updates moments (any storage
    format) and the master/weight shard, and writes the bf16 compute copy in the same pass.  ``ctas_per_sm``
    (1..7) limits the kernel's resident CTAs so that it can run beside compute kernels of another stream."""
    p = group.shard
    n = p.numel()
    g = group.grad_shard
    out_bf16 = None
    if not group.sharded and group.shard is not group.full:
        out_bf16 = group.full.data           # unsharded with fp32 masters: refresh the compute copy in-kernel
    elif getattr(group, "shard_lp", None) is not None:
        out_bf16 = group.shard_lp            # sharded: the copy the next all-gather publishes
    bc1 = 1.0 - beta1 ** step
    bc2 = 1.0 - beta2 ** step
    call("slab_adamw", p, 1 if p.dtype == torch.bfloat16 else 0, g, 1 if g.dtype == torch.bfloat16 else 0,
         m.data, v.data, getattr(m, "scale", None), getattr(v, "scale", None), out_bf16, coef, sq_out, n,
         _KIND[m.kind],
         float(lr), float(beta1), float(beta2), float(eps), float(weight_decay), float(bc1), float(bc2),
         int(group.shard_decay_end() if hasattr(group, "shard_decay_end") else n), int(ctas_per_sm), stream())
    if 0 < ctas_per_sm < 8 and _ADAMW_PIECE[0] > 0:        # a background update is cut into several launches
        LAUNCHES[0] += max((n + _ADAMW_PIECE[0] - 1) // _ADAMW_PIECE[0] - 1, 0)
