"""VRAM verdict / bucket table and the HTML report generator (CPU)."""
import json

from system_lab_b200.config import Config
from system_lab_b200.observe import report_html, vram


def test_vram_verdict_thresholds():
    mk = lambda r, retires=0: vram.health(vram.VramSample(50, 100, r, retires, 192.0))
    assert mk(150)["verdict"] == "OK"
    assert mk(150, retires=2)["verdict"] == "PRESSURE"
    assert mk(0.96 * 192)["verdict"] == "TIGHT"
    assert mk(0.985 * 192)["verdict"] == "CRITICAL"
    h = mk(150)
    assert abs(h["frag_pct"] - 100 * 50 / 150) < 1e-6 and abs(h["headroom_gb"] - 42.0) < 1e-6


def test_vram_buckets_moe_sum_and_unaccounted_rule():
    cfg = Config.load(preset="qwen3-30b-a3b", overrides=["params_dtype=bf16", "global_batch_size=16", "micro_batch_size=2",
                                                          "expert_model_parallel_size=8", "recompute_granularity=selective"])
    b = vram.decompose(cfg, 8)
    assert b.mode == "C"
    names = [r["bucket"] for r in b.rows]
    assert "MoE expert weights" in names and "Dense weights" in names
    total = sum(r["gb"] for r in b.rows)
    ok = vram.decompose(cfg, 8, vram.VramSample(0, total * 1.05, total * 1.2, 0, 192.0))
    assert ok.consistent and abs(ok.unaccounted_gb - 0.05 * total) < 1e-6
    bad = vram.decompose(cfg, 8, vram.VramSample(0, total * 1.5, total * 1.6, 0, 192.0))
    assert not bad.consistent
    assert "unaccounted" in vram.format_table(vram.health(vram.VramSample(0, total * 1.5, total * 1.6, 0, 192.0)), bad)


def test_vram_modes():
    dense = Config.load(preset="simplemoe-tiny", overrides=["num_experts=0"])
    assert vram.pick_mode(dense) == "B"
    assert vram.pick_mode(dense, trainable_fraction=0.001) == "A"
    rows = [r["bucket"] for r in vram.decompose(dense, 1).rows]
    assert rows[:4] == ["Weights", "Master copy", "Adam state (m + v)", "Gradients"]


def _breakdown(scale=1.0):
    return {"trace": "x/t.json", "window": "ProfilerStep#0", "window_ms": 100.0 * scale,
            "stream_busy_ms": {"7": 80.0 * scale, "9": 20.0},
            "compute_busy_pct": 90.0, "idle_pct": 2.0, "comm_ms": 10.0, "comm_hidden_pct": 70.0,
            "comm_ratio_exposed": 0.03, "category_ms": {"slab_grouped_gemm": 40.0 * scale, "attn_kernel": 20.0, "<odd&name>": 1.0},
            "top_kernels": [{"name": "void slab::k<1>(int*)", "ms": 40.0, "count": 96}],
            "time_bins": [{"slab_grouped_gemm": 0.5, "attn_kernel": 0.2}, {"attn_kernel": 0.4}]}


def test_html_single_and_comparison(tmp_path):
    bench = {"value": 12345.0, "n_gpus": 8, "dtype": "bf16", "mem_peak_gb": 77.0,
             "config": {"model": "m", "parallelism": "fsdp+ep8", "global_batch": 16, "seq_len": 4096, "tflops_per_gpu": 500.0}}
    page = report_html.render_single(_breakdown(), bench)
    assert page.startswith("<!doctype html>") and "slab_grouped_gemm" in page and "12,345" in page
    assert "&lt;odd&amp;name&gt;" in page and "<odd&name>" not in page          # names are escaped
    assert "<script" not in page
    cmp_page = report_html.render_comparison(_breakdown(), _breakdown(0.5), "a", "b")
    assert "2.00x" in cmp_page and "-20.00" in cmp_page
    p1, p2, out = tmp_path / "a.json", tmp_path / "b.json", tmp_path / "o" / "r.html"
    p1.write_text(json.dumps(_breakdown()))
    p2.write_text("log line\n" + json.dumps(_breakdown(0.5)))
    assert report_html.main([str(p1), "--against", str(p2), "--names", "x,y", "-o", str(out)]) == 0
    assert out.exists() and "x vs y" in out.read_text()


def test_trace_gap_analysis(tmp_path):
    """Idle gaps of the busiest stream: total, the part another stream covers, and the kernel pair they sit between."""
    from system_lab_b200.observe import trace_breakdown as tb
    ev = [{"ph": "X", "name": "ProfilerStep#0", "cat": "user_annotation", "ts": 0, "dur": 1000},
          {"ph": "X", "name": "void slab::grouped_gemm_kernel<0, 256>(x)", "cat": "kernel", "ts": 10, "dur": 200, "args": {"stream": 7}},
          {"ph": "X", "name": "void slab::adamw_kernel<f>(x)", "cat": "kernel", "ts": 250, "dur": 100, "args": {"stream": 9}},
          {"ph": "X", "name": "void slab::swiglu_fwd_kernel(x)", "cat": "kernel", "ts": 400, "dur": 300, "args": {"stream": 7}}]
    p = tmp_path / "t.json"
    p.write_text(json.dumps({"traceEvents": ev}))
    r = tb.analyze(str(p))
    g = r["main_stream_gaps"]
    assert g["stream"] == "7"
    assert abs(g["gap_ms"] - 0.5) < 1e-6                       # 10 us head + 190 us between + 300 us tail
    assert abs(g["gap_covered_by_other_streams_ms"] - 0.1) < 1e-6
    top = g["top_pairs"][0]
    assert top["between"].endswith("window end") and abs(top["ms"] - 0.3) < 1e-6
    assert any("grouped_gemm_kernel" in x["between"] and "swiglu_fwd_kernel" in x["between"] for x in g["top_pairs"])
    assert "idle gaps of stream 7" in tb.format_report(r)


def test_trace_gaps_are_split_into_host_late_and_held_on_device(tmp_path):
    """The kernel that ends a gap carries the correlation id of its launch call: the part of the gap before that
    call is the host's, the rest is the device holding a kernel that was already launched."""
    from system_lab_b200.observe import trace_breakdown as tb
    k = lambda name, ts, dur, corr, stream=7: {"ph": "X", "name": name, "cat": "kernel", "ts": ts, "dur": dur,
                                                "args": {"stream": stream, "correlation": corr}}
    rt = lambda ts, corr: {"ph": "X", "name": "cudaLaunchKernel", "cat": "cuda_runtime", "ts": ts, "dur": 4,
                           "args": {"correlation": corr}}
    ev = [{"ph": "X", "name": "ProfilerStep#0", "cat": "user_annotation", "ts": 0, "dur": 1000},
          rt(0, 1), k("a_kernel", 0, 100, 1),
          rt(160, 2), k("b_kernel", 200, 100, 2),          # gap 100..200: host launched at 160 -> 60 late, 40 held
          rt(20, 3), k("c_kernel", 500, 500, 3)]           # gap 300..500: launched long before -> all held on the device
    p = tmp_path / "t.json"
    p.write_text(json.dumps({"traceEvents": ev}))
    g = tb.analyze(str(p))["main_stream_gaps"]
    assert abs(g["gap_ms"] - 0.3) < 1e-9
    assert abs(g["host_late_ms"] - 0.06) < 1e-9 and abs(g["held_on_device_ms"] - 0.24) < 1e-9
    ab = next(x for x in g["top_pairs"] if "a_kernel" in x["between"])
    assert abs(ab["host_late_ms"] - 0.06) < 1e-9


def test_trace_reader_streams_large_files_in_small_chunks(tmp_path):
    import io
    from system_lab_b200.observe import trace_breakdown as tb
    events = [{"ph": "X", "name": f"kernel_{i} \"quoted\" [x] {{y}}", "cat": "kernel", "ts": i * 10, "dur": 5,
               "args": {"stream": 7, "nested": {"a": [1, 2, {"b": "]"}]}}} for i in range(3000)]
    doc = json.dumps({"schemaVersion": 1, "traceEvents": events, "displayTimeUnit": "ms"})
    for chunk in (64, 1000, 1 << 20):
        got = list(tb._stream_events(io.StringIO(doc), chunk=chunk))
        assert got == events
    assert list(tb._stream_events(io.StringIO(json.dumps(events[:10])), chunk=50)) == events[:10]     # bare list
    assert list(tb._stream_events(io.StringIO('{"traceEvents": []}'))) == []
    p = tmp_path / "t.json"
    p.write_text(doc)
    assert sum(1 for _ in tb._events(str(p))) == 3000


def test_metrics_file_gets_one_json_line_per_logged_step(tmp_path):
    import json
    from system_lab_b200.config import Config
    from system_lab_b200.trainer.loop import Trainer
    path = tmp_path / "m" / "metrics.jsonl"
    cfg = Config.load(preset="simplemoe-tiny", overrides=["device=cpu", "train_iters=4", "log_interval=2",
                                                         "expert_model_parallel_size=1", f"metrics_file={path}"])
    tr = Trainer(cfg)
    tr.fit()
    tr.close()
    recs = [json.loads(l) for l in path.read_text().splitlines()]
    assert [r["step"] for r in recs] == [2, 4]
    assert all(r["loss"] > 0 and r["tokens_per_s"] > 0 and r["ep_rank_load_max_over_mean"] >= 1.0 for r in recs)


def test_vram_buckets_pick_the_adapter_mode_for_lora():
    from system_lab_b200.config import Config
    from system_lab_b200.observe.vram import decompose
    b = decompose(Config.load(preset="llama2-70b-lora"), 8)
    assert b.mode == "A"
    rows = {r["bucket"]: r["gb"] for r in b.rows}
    assert 15 < rows["Weights (frozen base)"] < 20 and rows["Adapter grads + Adam state"] < 1.0
