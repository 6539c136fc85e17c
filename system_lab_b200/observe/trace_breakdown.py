"""Kineto trace breakdown: where one training step's GPU time goes.

    python -m system_lab_b200.observe.trace_breakdown <trace.json[.gz]> [ProfilerStep#N] [--json out.json]

Reports, for the chosen ``ProfilerStep#N`` window (default: the middle one): per-stream busy time,
a category table, the top kernels, per-stream category mix, compute/communication overlap measured on
50 us slots ("hidden behind compute" %), and an 80-bin time-binned mix.  Functional counterpart of the
reference's analyzer (``.cursor/skills/gpu-trace-analysis/scripts/full_breakdown.py:36-326``), rebuilt
around a rule table and a single event pass; it also knows this framework's kernel names, so hand
written kernels and library kernels are reported separately.

Opaque collective kernels (``nccl_generic``) are relabelled from the ``c10d::``/``nccl:`` CPU ops that
overlap them (5 ms slack), unless ``SPLIT_NCCL_BY_CPU=0``.
"""
from __future__ import annotations

import bisect
import gzip
import json
import os
import sys
from collections import defaultdict

# (category, substrings) — first match wins; names are lower-cased first.
RULES: list[tuple[str, tuple[str, ...]]] = [
    ("slab_grouped_gemm", ("grouped_gemm_kernel", "grouped_gemm_fp8")),
    ("slab_dispatch", ("moe_scatter_kernel", "moe_combine", "moe_count", "moe_publish", "moe_plan", "moe_slots",
                       "moe_wait", "moe_signal", "moe_reduce", "moe_check", "moe_gather")),
    ("slab_norm", ("rmsnorm_fwd_kernel", "rmsnorm_bwd_kernel", "colsum_to_bf16")),
    ("slab_act", ("swiglu_fwd_kernel", "swiglu_bwd_kernel", "rope_kernel")),
    ("slab_router", ("router_topk_kernel",)),
    ("slab_ce", ("ce_fwd_bwd_kernel",)),
    ("slab_quant", ("quant_1x128_kernel", "quant_128x128_kernel", "quant_rowwise_kernel")),
    ("slab_optimizer", ("adamw_kernel", "sumsq_kernel")),
    ("slab_attn", ("slab_attn", "attn_fwd_kernel", "attn_bwd_kernel")),
    ("slab_fsdp", ("fsdp_gather_kernel", "fsdp_reduce_scatter_kernel", "fsdp_stage_kernel", "fsdp_rs_adamw")),
    ("nccl_rs", ()), ("nccl_ar", ()), ("nccl_ag", ()), ("nccl_a2a", ()), ("nccl_bcast", ()), ("nccl_generic", ()),
    ("grouped_gemm", ("_grouped", "groupedgemm", "grouped_gemm", "groupedlinear", "te_grouped")),
    ("attn_kernel", ("fmha", "fmhca", "flash", "scaled_dot_product", "_sdpa_", "_attn_", "attention", "ck_v3")),
    ("norm", ("rmsnorm", "layernorm", "ln_fwd", "ln_bwd", "norm_kernel", "normalization::")),
    ("gemm", ("cutlass", "sm100_xmma", "sm100_gemm", "sm100_warpspecialized", "blackwell_", "ampere_fp", "cublaslt",
              "cublas", "fp8_gemm", "_qmm", "wgrad_kernel", "dgrad_kernel", "_8bit_gemm", "matmul_kernel", "nvjet",
              "hgemm", "hipblaslt", "ck_gemm", "ck_kernel", "rocblas", "sm90_xmma", "gemv")),
    ("moe_dispatch", ("permute", "unpermute", "_moe_", "moechunk", "topk", "_sort", "histogram", "indices",
                      "dispatch", "_compute_routing", "index_", "gather", "scatter", "radixsort", "bincount")),
    ("fp8_cast", ("amax", "to_fp8", "fp8cast", "_quantize", "dequant", "cast_to_fp8", "scale_kernel", "cast_fp8")),
    ("elementwise", ("silu", "swiglu", "gelu", "relu", "sigmoid", "elementwise", "vectorized", "unrolled")),
    ("softmax", ("softmax", "logsumexp")),
    ("memcpy", ("memcpy", "memset")),
    ("optimizer", ("adam", "optimizer", "multi_tensor")),
    ("reduction", ("reduce",)),
]
_NCCL_MARKS = ("nccldevkernel", "ncclkernel", "ncclbackend")
_NCCL_KIND = [("nccl_rs", ("reducescatter", "reduce_scatter")), ("nccl_ar", ("allreduce", "all_reduce")),
              ("nccl_ag", ("allgather", "all_gather")), ("nccl_a2a", ("alltoall", "all_to_all", "a2a", "sendrecv",
                                                                      "send_recv", "send", "recv", "p2p")),
              ("nccl_bcast", ("broadcast",))]
COMM_CATS = {"nccl_rs", "nccl_ar", "nccl_ag", "nccl_a2a", "nccl_bcast", "nccl_generic", "slab_dispatch", "slab_fsdp"}


def categorize(name: str) -> str:
    n = name.lower()
    if any(m in n for m in _NCCL_MARKS) or n.startswith(("nccl_", "rccl_")):
        for cat, keys in _NCCL_KIND:
            if any(k in n for k in keys):
                return cat
        return "nccl_generic"
    if n.startswith("cijk_") or "_userargs_mt" in n:
        return "gemm"
    for cat, keys in RULES:
        if keys and any(k in n for k in keys):
            return cat
    return "other"


def _events(path: str):
    """Yield trace events.  Streams with ijson when available (traces reach hundreds of MB)."""
    opener = gzip.open if path.endswith(".gz") else open
    try:
        import ijson
        with opener(path, "rb") as f:
            for ev in ijson.items(f, "traceEvents.item"):
                yield ev
        return
    except ImportError:
        pass
    with opener(path, "rt") as f:
        yield from _stream_events(f)


def _stream_events(f, chunk: int = 1 << 22):
    """Incremental reader for ``{"traceEvents": [ {...}, ... ], ...}`` (or a bare list of events): decodes one
    event object at a time from a sliding text buffer, so memory stays at a few MB whatever the trace size."""
    dec = json.JSONDecoder()
    buf, pos, eof = "", 0, False

    def refill():
        nonlocal buf, pos, eof
        data = f.read(chunk)
        if not data:
            eof = True
            return False
        buf = buf[pos:] + data
        pos = 0
        return True

    # find the start of the event array
    while True:
        if not buf and not refill():
            return
        stripped = buf.lstrip()
        if stripped.startswith("["):
            pos = buf.index("[") + 1
            break
        k = buf.find('"traceEvents"')
        if k >= 0:
            b = buf.find("[", k)
            if b >= 0:
                pos = b + 1
                break
        if not refill():
            return
    while True:
        # skip separators
        while True:
            while pos < len(buf) and buf[pos] in " \t\r\n,":
                pos += 1
            if pos < len(buf) or not refill():
                break
        if pos >= len(buf) or buf[pos] == "]":
            return
        try:
            obj, end = dec.raw_decode(buf, pos)
        except json.JSONDecodeError:
            if not refill():
                raise
            continue
        yield obj
        pos = end
        if pos > chunk:
            buf, pos = buf[pos:], 0


def _union_len(intervals: list[tuple[float, float]]) -> float:
    if not intervals:
        return 0.0
    intervals.sort()
    total, (cs, ce) = 0.0, intervals[0]
    for s, e in intervals[1:]:
        if s > ce:
            total += ce - cs
            cs, ce = s, e
        else:
            ce = max(ce, e)
    return total + ce - cs


def analyze(path: str, window: str | None = None, slot_us: float = 50.0, bins: int = 80) -> dict:
    split_nccl = os.environ.get("SPLIT_NCCL_BY_CPU", "1") != "0"
    steps, kernels, c10d = {}, [], []
    launches = {}                     # correlation id -> host time of the runtime call that launched it
    runtime_calls = []                # (ts, dur, name) of every CUDA runtime / driver call on the host
    for ev in _events(path):
        if ev.get("ph") != "X":
            continue
        name = ev.get("name", "")
        cat = ev.get("cat", "")
        ts, dur = float(ev.get("ts", 0)), float(ev.get("dur", 0))
        if name.startswith("ProfilerStep#") and cat in ("user_annotation", "cpu_op", ""):
            steps.setdefault(name, (ts, ts + dur))
        elif cat in ("kernel", "gpu_memcpy", "gpu_memset"):
            a = ev.get("args") or {}
            stream = a.get("stream", ev.get("tid"))
            kernels.append((ts, dur, name, stream, a.get("correlation")))
        elif cat in ("cuda_runtime", "cuda_driver"):
            corr = (ev.get("args") or {}).get("correlation")
            if corr is not None:
                launches[corr] = ts
            runtime_calls.append((ts, dur, name))
        elif cat == "cpu_op" and (name.startswith("c10d::") or name.startswith("nccl:")):
            c10d.append((ts, ts + dur, name))
    if not kernels:
        raise ValueError("no GPU kernel events in trace")
    if steps:
        if window is None:
            names = sorted(steps, key=lambda s: int(s.split("#")[1]))
            window = names[len(names) // 2]
        if window not in steps:
            raise KeyError(f"{window} not in trace; have {sorted(steps)}")
        w0, w1 = steps[window]
    else:
        window = "whole-trace"
        w0 = min(k[0] for k in kernels)
        w1 = max(k[0] + k[1] for k in kernels)
    c10d.sort()
    c10d_starts = [c[0] for c in c10d]

    def relabel(ts, dur):
        lo = bisect.bisect_left(c10d_starts, ts - 5000.0)
        hi = bisect.bisect_right(c10d_starts, ts + dur)
        for s, e, nm in c10d[lo:hi]:
            if s - 5000.0 <= ts <= e + 5000.0:
                n = nm.lower()
                for cat, keys in _NCCL_KIND:
                    if any(k in n for k in keys):
                        return cat
        return "nccl_generic"

    by_cat, by_name, cnt_name = defaultdict(float), defaultdict(float), defaultdict(int)
    by_stream = defaultdict(list)
    stream_cat = defaultdict(lambda: defaultdict(float))
    comm_iv, comp_iv = [], []
    timeline = []
    for ts, dur, name, stream, _corr in kernels:
        s, e = max(ts, w0), min(ts + dur, w1)
        if e <= s:
            continue
        cat = categorize(name)
        if cat == "nccl_generic" and split_nccl and c10d:
            cat = relabel(ts, dur)
        d = e - s
        by_cat[cat] += d
        by_name[name] += d
        cnt_name[name] += 1
        by_stream[stream].append((s, e))
        stream_cat[stream][cat] += d
        (comm_iv if cat in COMM_CATS else comp_iv).append((s, e))
        timeline.append((s, e, cat))
    span = w1 - w0
    stream_busy = {str(k): _union_len(v) for k, v in by_stream.items()}
    # overlap on fixed slots
    n_slots = max(int(span / slot_us) + 1, 1)
    comp = bytearray(n_slots)
    comm = bytearray(n_slots)
    for arr, ivs in ((comp, comp_iv), (comm, comm_iv)):
        for s, e in ivs:
            for i in range(int((s - w0) / slot_us), min(int((e - w0) / slot_us) + 1, n_slots)):
                arr[i] = 1
    comm_slots = sum(comm)
    both = sum(1 for a, b in zip(comp, comm) if a and b)
    any_busy = sum(1 for a, b in zip(comp, comm) if a or b)
    # time-binned category mix
    bin_w = span / bins
    mix = [defaultdict(float) for _ in range(bins)]
    for s, e, cat in timeline:
        b0, b1 = int((s - w0) / bin_w), min(int((e - w0) / bin_w), bins - 1)
        for b in range(b0, b1 + 1):
            lo, hi = w0 + b * bin_w, w0 + (b + 1) * bin_w
            mix[b][cat] += max(0.0, min(e, hi) - max(s, lo))
    total_kernel = sum(by_cat.values())
    gaps = _gap_report(kernels, w0, w1, by_stream, launches, runtime_calls)
    return {
        "main_stream_gaps": gaps,
        "trace": path, "window": window, "window_ms": span / 1e3,
        "stream_busy_ms": {k: v / 1e3 for k, v in sorted(stream_busy.items(), key=lambda kv: -kv[1])},
        "oversubscription_pct": 100.0 * (sum(stream_busy.values()) / max(_union_len(comp_iv + comm_iv), 1e-9) - 1.0),
        "compute_busy_pct": 100.0 * _union_len(list(comp_iv)) / span,
        "idle_pct": 100.0 * (1 - any_busy / n_slots),
        "category_ms": {k: v / 1e3 for k, v in sorted(by_cat.items(), key=lambda kv: -kv[1])},
        "category_pct_of_kernel_time": {k: 100.0 * v / total_kernel for k, v in by_cat.items()},
        "top_kernels": [{"name": n[:120], "ms": d / 1e3, "count": cnt_name[n]}
                        for n, d in sorted(by_name.items(), key=lambda kv: -kv[1])[:25]],
        "per_stream_category_ms": {str(s): {c: v / 1e3 for c, v in sorted(cs.items(), key=lambda kv: -kv[1])}
                                   for s, cs in stream_cat.items()},
        "comm_ms": _union_len(list(comm_iv)) / 1e3,
        "comm_hidden_pct": 100.0 * both / comm_slots if comm_slots else 0.0,
        "comm_ratio_exposed": (comm_slots - both) * slot_us / span,
        "alltoall_share_pct": 100.0 * (by_cat.get("nccl_a2a", 0) + by_cat.get("slab_dispatch", 0)) /
        max(sum(v for k, v in by_cat.items() if k in COMM_CATS), 1e-9),
        "time_bins": [{k: v / 1e3 for k, v in m.items()} for m in mix],
    }


def _short(name: str) -> str:
    name = name.split("(")[0]
    for pre in ("void ", "slab::", "at::native::"):
        name = name.replace(pre, "")
    return name[:60]


def _gap_report(kernels, w0: float, w1: float, by_stream: dict, launches: dict | None = None,
                runtime_calls: list | None = None, min_gap_us: float = 5.0, top: int = 12) -> dict:
    """Idle gaps of the busiest stream inside the window: how much of the step the critical stream spends
    not running anything, how much of that another stream covers, and which kernel pairs the gaps sit between
    (a large total under one pair points at a host sync, an event wait or launch latency at that spot).

    Each gap is also split by where the kernel that ends it was when the stream went idle: the part of the gap
    before the host issued that kernel's launch call is ``host_late`` (the host had not got there yet: a host
    sync, an allocation, Python time), the rest is ``held_on_device`` (launched already, but kept back by an event
    wait on another stream, by the work distributor, or by launch latency).  ``host_calls`` of a pair lists the
    runtime calls the host spent the most time in while those gaps were open."""
    if not by_stream:
        return {}
    launches = launches or {}
    main = max(by_stream, key=lambda k: _union_len(by_stream[k]))
    evs = sorted((max(ts, w0), min(ts + dur, w1), name, launches.get(corr)) for ts, dur, name, st, corr in kernels
                 if st == main and min(ts + dur, w1) > max(ts, w0))
    others = sorted(iv for st, ivs in by_stream.items() if st != main for iv in ivs)
    o_starts = [iv[0] for iv in others]

    def covered(a: float, b: float) -> float:
        tot, i = 0.0, max(bisect.bisect_left(o_starts, a) - 64, 0)
        ivs = []
        while i < len(others) and others[i][0] < b:
            if others[i][1] > a:
                ivs.append((max(others[i][0], a), min(others[i][1], b)))
            i += 1
        return _union_len(ivs) if ivs else tot

    pairs, pair_n, pair_host = defaultdict(float), defaultdict(int), defaultdict(float)
    pair_calls = defaultdict(lambda: defaultdict(float))
    rt = sorted(runtime_calls or [])
    rt_starts = [c[0] for c in rt]

    def host_calls_in(a: float, b: float, into) -> None:
        i = max(bisect.bisect_left(rt_starts, a) - 32, 0)
        while i < len(rt) and rt[i][0] < b:
            ts, dur, name = rt[i]
            ov = min(ts + dur, b) - max(ts, a)
            if ov > 0:
                into[name] += ov
            i += 1

    total = cov = host_late = 0.0
    hist = {"5-20us": 0.0, "20-100us": 0.0, "100us-1ms": 0.0, ">1ms": 0.0}
    end, prev = (evs[0][0], "window start") if evs else (w0, "window start")
    end = w0
    for s, e, name, launched in evs:
        g = s - end
        if g >= min_gap_us:
            total += g
            cov += covered(end, s)
            key = f"{_short(prev)} -> {_short(name)}"
            pairs[key] += g
            pair_n[key] += 1
            if launched is not None:
                late = min(max(launched - end, 0.0), g)
                host_late += late
                pair_host[key] += late
            if g >= 100.0:
                host_calls_in(end, s, pair_calls[key])
            hist["5-20us" if g < 20 else "20-100us" if g < 100 else "100us-1ms" if g < 1000 else ">1ms"] += g
        if e > end:
            end, prev = e, name
    tail = w1 - end
    if tail >= min_gap_us:
        total += tail
        cov += covered(end, w1)
        pairs[f"{_short(prev)} -> window end"] += tail
        pair_n[f"{_short(prev)} -> window end"] += 1
    return {"stream": str(main), "gap_ms": total / 1e3, "gap_covered_by_other_streams_ms": cov / 1e3,
            "host_late_ms": host_late / 1e3, "held_on_device_ms": (total - host_late) / 1e3,
            "by_size_ms": {k: v / 1e3 for k, v in hist.items()},
            "top_pairs": [{"between": k, "ms": v / 1e3, "count": pair_n[k], "host_late_ms": pair_host[k] / 1e3,
                           "host_calls": [{"name": n, "ms": t / 1e3} for n, t in
                                          sorted(pair_calls[k].items(), key=lambda kv: -kv[1])[:4]]}
                          for k, v in sorted(pairs.items(), key=lambda kv: -kv[1])[:top]]}


def format_report(r: dict) -> str:
    out = [f"trace   : {r['trace']}", f"window  : {r['window']}  ({r['window_ms']:.2f} ms)",
           f"compute busy {r['compute_busy_pct']:.1f} %   idle {r['idle_pct']:.1f} %   "
           f"oversubscription {r['oversubscription_pct']:.1f} %",
           f"communication {r['comm_ms']:.2f} ms, hidden behind compute {r['comm_hidden_pct']:.1f} %", "",
           "per-stream busy (ms):"]
    out += [f"  stream {k:>6}: {v:9.2f}" for k, v in r["stream_busy_ms"].items()]
    out += ["", "category (ms, % of kernel time):"]
    out += [f"  {k:20s} {v:9.2f}  {r['category_pct_of_kernel_time'][k]:5.1f} %" for k, v in r["category_ms"].items()]
    out += ["", "top kernels:"]
    out += [f"  {k['ms']:9.2f} ms  x{k['count']:<5d} {k['name']}" for k in r["top_kernels"]]
    g = r.get("main_stream_gaps") or {}
    if g:
        out += ["", f"idle gaps of stream {g['stream']}: {g['gap_ms']:.2f} ms "
                    f"({g['gap_covered_by_other_streams_ms']:.2f} ms of it covered by other streams; "
                    f"{g.get('host_late_ms', 0.0):.2f} ms before the host had launched the next kernel, "
                    f"{g.get('held_on_device_ms', 0.0):.2f} ms with it launched but held back); by gap size: "
                    + ", ".join(f"{k} {v:.2f}" for k, v in g["by_size_ms"].items())]
        for p in g["top_pairs"]:
            out.append(f"  {p['ms']:9.2f} ms  x{p['count']:<5d} host-late {p.get('host_late_ms', 0.0):7.2f} ms  {p['between']}")
            if p.get("host_calls"):
                out.append("             host during these gaps: " +
                           ", ".join(f"{c['name']} {c['ms']:.2f} ms" for c in p["host_calls"]))
    return "\n".join(out)


def main(argv=None) -> int:
    argv = list(sys.argv[1:] if argv is None else argv)
    out_json = None
    if "--json" in argv:
        i = argv.index("--json")
        out_json = argv[i + 1]
        del argv[i:i + 2]
    if not argv:
        print(__doc__)
        return 2
    rep = analyze(argv[0], argv[1] if len(argv) > 1 else None)
    print(format_report(rep))
    if out_json:
        with open(out_json, "w") as f:
            json.dump(rep, f, indent=1)
    return 0


if __name__ == "__main__":
    sys.exit(main())
