"""Static HTML reports from trace breakdowns: one run, or two runs side by side.

Input is the JSON that ``observe/trace_breakdown.py --json`` writes (window, per-category kernel time, stream
busy time, communication overlap, top kernels, time bins), optionally the JSON line of ``bench.py`` (identity
strip: model, parallelism, tokens/s, TFLOP/s per GPU) and a VRAM block from ``observe/vram.py --json``.  Output
is one self-contained ``.html`` file (inline CSS, no scripts, no network), so it can be attached to a run
record or opened from a cluster's file browser.

Reference behaviour: the rendered two-platform comparison ``docs/b200-vs-mi355x-ep8-gbs16-trace.html`` (identity
strip, headline stats, per-category table with deltas, stacked timeline) and the single-run / VRAM templates
under ``.cursor/skills/gpu-trace-analysis/templates`` and ``.cursor/skills/trace-vram-canvas/templates``, which
are filled by replacing top-of-file constants; here the same sections are generated from the JSON.
"""
from __future__ import annotations

import argparse
import html
import json
from pathlib import Path

PALETTE = ["#4e79a7", "#f28e2b", "#e15759", "#76b7b2", "#59a14f", "#edc948", "#b07aa1", "#ff9da7", "#9c755f",
           "#bab0ac", "#1f77b4", "#aec7e8", "#ffbb78", "#98df8a", "#c5b0d5", "#c49c94"]

CSS = """
body{font:14px/1.45 -apple-system,Segoe UI,Helvetica,Arial,sans-serif;margin:24px;color:#1b1f23;background:#fff}
h1{font-size:22px;margin:0 0 4px} h2{font-size:16px;margin:28px 0 8px;border-bottom:1px solid #e1e4e8;padding-bottom:4px}
.sub{color:#586069;margin-bottom:16px}
.strip{display:flex;flex-wrap:wrap;gap:8px;margin:8px 0 16px}
.chip{background:#f6f8fa;border:1px solid #e1e4e8;border-radius:6px;padding:4px 10px}
.chip b{color:#24292e}
.stats{display:flex;flex-wrap:wrap;gap:12px}
.stat{border:1px solid #e1e4e8;border-radius:8px;padding:10px 14px;min-width:130px}
.stat .v{font-size:20px;font-weight:600} .stat .l{color:#586069;font-size:12px}
.good{color:#22863a} .warn{color:#b08800} .bad{color:#cb2431}
table{border-collapse:collapse;width:100%;margin:6px 0} th,td{padding:4px 8px;border-bottom:1px solid #eaecef;text-align:right}
th:first-child,td:first-child{text-align:left} th{background:#f6f8fa;font-weight:600}
.bar{height:12px;border-radius:2px;display:inline-block;vertical-align:middle}
.stack{display:flex;height:22px;border-radius:4px;overflow:hidden;border:1px solid #e1e4e8}
.timeline{display:flex;align-items:flex-end;height:90px;gap:1px;border-bottom:1px solid #d1d5da}
.timeline .col{flex:1;display:flex;flex-direction:column-reverse}
.legend{display:flex;flex-wrap:wrap;gap:10px;margin:6px 0;font-size:12px}
.sw{display:inline-block;width:10px;height:10px;border-radius:2px;margin-right:4px}
.cols{display:grid;grid-template-columns:1fr 1fr;gap:24px}
code{background:#f6f8fa;padding:1px 4px;border-radius:3px}
"""


def _esc(x) -> str:
    return html.escape(str(x))


def _colors(categories: list[str]) -> dict:
    return {c: PALETTE[i % len(PALETTE)] for i, c in enumerate(categories)}


def _stat(label: str, value: str, tone: str = "") -> str:
    return f'<div class="stat"><div class="v {tone}">{_esc(value)}</div><div class="l">{_esc(label)}</div></div>'


def _identity(bench: dict | None, breakdown: dict) -> str:
    chips = []
    if bench:
        cfg = bench.get("config", {})
        for k, v in (("model", cfg.get("model")), ("GPUs", bench.get("n_gpus")), ("parallelism", cfg.get("parallelism")),
                     ("global batch", cfg.get("global_batch")), ("seq", cfg.get("seq_len")),
                     ("dtype", bench.get("dtype")), ("recompute", cfg.get("recompute")),
                     ("dispatcher", cfg.get("dispatcher"))):
            if v is not None:
                chips.append(f'<span class="chip">{_esc(k)} <b>{_esc(v)}</b></span>')
    chips.append(f'<span class="chip">window <b>{_esc(breakdown.get("window", "?"))}</b></span>')
    chips.append(f'<span class="chip">trace <b>{_esc(Path(str(breakdown.get("trace", ""))).name)}</b></span>')
    return '<div class="strip">' + "".join(chips) + "</div>"


def _headline(bench: dict | None, b: dict) -> str:
    s = [_stat("step window", f'{b.get("window_ms", 0):.1f} ms')]
    if bench:
        s.append(_stat("tokens/s (whole job)", f'{bench.get("value", 0):,.0f}'))
        tf = bench.get("config", {}).get("tflops_per_gpu")
        if tf:
            s.append(_stat("model TFLOP/s per GPU", f"{tf:.0f}"))
        if bench.get("mem_peak_gb"):
            s.append(_stat("peak allocated", f'{bench["mem_peak_gb"]:.1f} GB'))
    busy = b.get("compute_busy_pct", 0.0)
    s.append(_stat("GPU busy", f"{busy:.1f} %", "good" if busy >= 90 else "warn" if busy >= 75 else "bad"))
    s.append(_stat("idle", f'{b.get("idle_pct", 0):.1f} %'))
    exposed = 100.0 * b.get("comm_ratio_exposed", 0.0)
    s.append(_stat("exposed communication", f"{exposed:.1f} % of step",
                   "good" if exposed < 10 else "warn" if exposed < 20 else "bad"))
    s.append(_stat("communication hidden", f'{b.get("comm_hidden_pct", 0):.0f} %'))
    return '<div class="stats">' + "".join(s) + "</div>"


def _category_table(b: dict, colors: dict) -> str:
    cats = sorted(b.get("category_ms", {}).items(), key=lambda kv: -kv[1])
    total = sum(v for _, v in cats) or 1.0
    top = cats[0][1] if cats else 1.0
    rows = []
    for c, ms in cats:
        w = 220.0 * ms / top
        rows.append(f'<tr><td><span class="sw" style="background:{colors.get(c, "#999")}"></span>{_esc(c)}</td>'
                    f'<td>{ms:.2f}</td><td>{100 * ms / total:.1f} %</td>'
                    f'<td style="text-align:left"><span class="bar" style="width:{w:.0f}px;background:{colors.get(c, "#999")}"></span></td></tr>')
    stack = "".join(f'<div title="{_esc(c)} {ms:.1f} ms" style="width:{100 * ms / total:.2f}%;background:{colors.get(c, "#999")}"></div>'
                    for c, ms in cats)
    return (f'<div class="stack">{stack}</div><table><tr><th>category</th><th>ms</th><th>share of kernel time</th>'
            f'<th style="text-align:left"></th></tr>{"".join(rows)}</table>')


def _timeline(b: dict, colors: dict) -> str:
    bins = b.get("time_bins") or []
    if not bins:
        return ""
    peak = max((sum(x.values()) for x in bins), default=1.0) or 1.0
    cols = []
    for x in bins:
        segs = "".join(f'<div title="{_esc(c)}" style="height:{90.0 * v / peak:.1f}px;background:{colors.get(c, "#999")}"></div>'
                       for c, v in sorted(x.items(), key=lambda kv: -kv[1]))
        cols.append(f'<div class="col">{segs}</div>')
    legend = "".join(f'<span><span class="sw" style="background:{col}"></span>{_esc(c)}</span>' for c, col in colors.items())
    return f'<div class="timeline">{"".join(cols)}</div><div class="legend">{legend}</div>'


def _streams(b: dict) -> str:
    rows = "".join(f"<tr><td>stream {_esc(s)}</td><td>{ms:.2f}</td><td>{100 * ms / max(b.get('window_ms', 1), 1e-9):.1f} %</td></tr>"
                   for s, ms in sorted(b.get("stream_busy_ms", {}).items(), key=lambda kv: -kv[1]))
    return f"<table><tr><th>stream</th><th>busy ms</th><th>of window</th></tr>{rows}</table>"


def _top_kernels(b: dict, n: int = 15) -> str:
    rows = "".join(f'<tr><td><code>{_esc(k["name"][:110])}</code></td><td>{k["ms"]:.2f}</td><td>{k["count"]}</td>'
                   f'<td>{1e3 * k["ms"] / max(k["count"], 1):.1f}</td></tr>' for k in b.get("top_kernels", [])[:n])
    return f"<table><tr><th>kernel</th><th>ms</th><th>launches</th><th>us / launch</th></tr>{rows}</table>"


def _vram(v: dict | None) -> str:
    if not v:
        return ""
    h, bk = v["health"], v["buckets"]
    tone = {"OK": "good", "PRESSURE": "warn", "TIGHT": "warn", "CRITICAL": "bad"}.get(h["verdict"], "")
    stats = "".join([_stat("VRAM verdict", h["verdict"], tone), _stat("reserved", f'{h["reserved_pct"]:.1f} %'),
                     _stat("allocated", f'{h["alloc_pct"]:.1f} %'), _stat("fragmentation", f'{h["frag_pct"]:.1f} %'),
                     _stat("headroom", f'{h["headroom_gb"]:.1f} GB'), _stat("allocator retries", str(h["retires"]),
                                                                           "bad" if h["retires"] else "")])
    rows = "".join(f'<tr><td>{_esc(r["bucket"])}</td><td>{r["gb"]:.2f}</td><td style="text-align:left">{_esc(r["how"])}</td></tr>'
                   for r in bk["rows"])
    warn = "" if bk.get("consistent", True) else \
        f'<p class="bad">{bk["unaccounted_pct"]:.0f} % of the peak is unaccounted: the bucket estimate is wrong.</p>'
    return (f'<h2>VRAM</h2><div class="stats">{stats}</div><table><tr><th>bucket (mode {_esc(bk["mode"])})</th><th>GB</th>'
            f'<th style="text-align:left">how</th></tr>{rows}</table>{warn}')


def render_single(breakdown: dict, bench: dict | None = None, vram: dict | None = None, title: str = "") -> str:
    colors = _colors([c for c, _ in sorted(breakdown.get("category_ms", {}).items(), key=lambda kv: -kv[1])])
    title = title or "Training step trace report"
    body = [f"<h1>{_esc(title)}</h1>", _identity(bench, breakdown), _headline(bench, breakdown),
            "<h2>Where the step goes</h2>", _category_table(breakdown, colors),
            "<h2>Timeline (kernel time per category across the step)</h2>", _timeline(breakdown, colors),
            "<h2>Streams</h2>", _streams(breakdown), "<h2>Top kernels</h2>", _top_kernels(breakdown), _vram(vram)]
    return f"<!doctype html><html><head><meta charset='utf-8'><title>{_esc(title)}</title><style>{CSS}</style></head><body>" \
           + "".join(body) + "</body></html>"


def render_comparison(a: dict, b: dict, name_a: str, name_b: str, bench_a: dict | None = None,
                      bench_b: dict | None = None, title: str = "") -> str:
    """Side-by-side report; the delta column is ``b - a`` (negative = b is faster)."""
    cats = sorted(set(a.get("category_ms", {})) | set(b.get("category_ms", {})),
                  key=lambda c: -(a.get("category_ms", {}).get(c, 0) + b.get("category_ms", {}).get(c, 0)))
    colors = _colors(cats)
    title = title or f"{name_a} vs {name_b}"
    rows = []
    for c in cats:
        x, y = a.get("category_ms", {}).get(c, 0.0), b.get("category_ms", {}).get(c, 0.0)
        d = y - x
        tone = "good" if d < -0.05 * max(x, 1e-9) else "bad" if d > 0.05 * max(x, 1e-9) else ""
        ratio = f"{y / x:.2f}x" if x > 0 else "-"
        rows.append(f'<tr><td><span class="sw" style="background:{colors[c]}"></span>{_esc(c)}</td><td>{x:.2f}</td>'
                    f'<td>{y:.2f}</td><td class="{tone}">{d:+.2f}</td><td>{ratio}</td></tr>')
    wa, wb = a.get("window_ms", 0.0), b.get("window_ms", 0.0)
    head = [_stat(f"step, {name_a}", f"{wa:.1f} ms"), _stat(f"step, {name_b}", f"{wb:.1f} ms"),
            _stat("speed-up of the second", f"{wa / wb:.2f}x" if wb else "-", "good" if wb and wa / wb >= 1 else "bad")]
    if bench_a and bench_b:
        head.append(_stat(f"tokens/s, {name_a}", f'{bench_a.get("value", 0):,.0f}'))
        head.append(_stat(f"tokens/s, {name_b}", f'{bench_b.get("value", 0):,.0f}'))
    body = [f"<h1>{_esc(title)}</h1>", '<div class="cols"><div>', f"<b>{_esc(name_a)}</b>", _identity(bench_a, a),
            "</div><div>", f"<b>{_esc(name_b)}</b>", _identity(bench_b, b), "</div></div>",
            '<div class="stats">' + "".join(head) + "</div>",
            "<h2>Per-category kernel time (ms)</h2>",
            f'<table><tr><th>category</th><th>{_esc(name_a)}</th><th>{_esc(name_b)}</th><th>delta</th><th>ratio</th></tr>'
            + "".join(rows) + "</table>",
            '<h2>Timelines</h2><div class="cols"><div>', _timeline(a, colors), "</div><div>", _timeline(b, colors), "</div></div>",
            '<h2>Overlap</h2><div class="cols"><div>', _headline(bench_a, a), "</div><div>", _headline(bench_b, b), "</div></div>",
            '<h2>Top kernels</h2><div class="cols"><div>', _top_kernels(a, 10), "</div><div>", _top_kernels(b, 10), "</div></div>"]
    return f"<!doctype html><html><head><meta charset='utf-8'><title>{_esc(title)}</title><style>{CSS}</style></head><body>" \
           + "".join(body) + "</body></html>"


def _load(path: str | None) -> dict | None:
    if not path:
        return None
    text = Path(path).read_text().strip()
    if not text.startswith("{"):                       # a log whose last JSON line is the bench result
        text = [ln for ln in text.splitlines() if ln.startswith("{")][-1]
    return json.loads(text)


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description="HTML report from trace breakdown JSON (one run, or two side by side)")
    ap.add_argument("breakdown", help="JSON written by `python -m system_lab_b200.observe.trace_breakdown --json`")
    ap.add_argument("--bench", default=None, help="bench.py JSON line (or a log ending with it)")
    ap.add_argument("--vram", default=None, help="JSON written by `python -m system_lab_b200.observe.vram --json`")
    ap.add_argument("--against", default=None, help="second breakdown JSON: write a comparison instead")
    ap.add_argument("--against-bench", default=None)
    ap.add_argument("--names", default="baseline,candidate")
    ap.add_argument("--title", default="")
    ap.add_argument("-o", "--out", required=True)
    a = ap.parse_args(argv)
    first = _load(a.breakdown)
    if a.against:
        na, nb = (a.names.split(",") + ["candidate"])[:2]
        page = render_comparison(first, _load(a.against), na, nb, _load(a.bench), _load(a.against_bench), a.title)
    else:
        page = render_single(first, _load(a.bench), _load(a.vram), a.title)
    Path(a.out).parent.mkdir(parents=True, exist_ok=True)
    Path(a.out).write_text(page)
    print(f"wrote {a.out} ({len(page)} bytes)")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
