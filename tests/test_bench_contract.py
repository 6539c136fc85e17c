"""The benchmark's command-line contract, on CPU with the tiny preset: one JSON line with the agreed keys, the
reference arm's `unavailable` line, and the build entry point."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _run(*args, timeout=600):
    env = dict(os.environ, CUDA_VISIBLE_DEVICES="")
    p = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), *args], cwd=ROOT, env=env, capture_output=True,
                       text=True, timeout=timeout)
    assert p.returncode == 0, p.stderr[-2000:]
    lines = [ln for ln in p.stdout.splitlines() if ln.startswith("{")]
    assert len(lines) == 1, p.stdout
    return json.loads(lines[0])


def test_reference_arm_reports_unavailable():
    d = _run("--impl", "reference", "--gpus", "1", "--steps", "2", "--warmup", "3")
    assert d["impl"] == "reference" and isinstance(d["unavailable"], str) and d["unavailable"]


def test_json_line_has_the_contract_keys():
    d = _run("--preset", "simplemoe-tiny", "--steps", "2", "--warmup", "3", "--kernels", "false")
    for k in ("metric", "value", "unit", "n_gpus", "steps", "warmup", "ms_per_step", "higher_is_better", "scaling",
              "vs_baseline", "dtype", "data", "config", "clocks", "e2e", "gpu_launches", "impl"):
        assert k in d, k
    assert d["steps"] == 2 and d["warmup"] == 3 and d["n_gpus"] == 1 and d["higher_is_better"] is True
    assert d["scaling"] == "weak" and d["impl"] == "ours"
    for k in ("model", "global_batch", "seq_len", "parallelism", "memory_plan"):
        assert k in d["config"], k
    tokens = d["config"]["global_batch"] * d["config"]["seq_len"]
    assert abs(d["value"] - tokens / (d["ms_per_step"] / 1e3)) < 1e-6 * d["value"]
    e = d["e2e"]
    assert e["h2d_bytes_per_step"] == tokens * 8 * 2 and e["d2h_bytes_per_step"] == 12    # int64 tokens + targets; fp32 loss, gradient norm, status
    assert e["value"] > 0 and e["value"] != d["value"]
    assert set(d["clocks"]) >= {"sm_mhz", "sm_max_mhz", "reasons"}


def test_memory_plan_prefers_fidelity_and_fits():
    sys.path.insert(0, ROOT)
    from bench import choose_memory_plan
    from system_lab_b200.config import Config
    names = {}
    for n in (1, 2, 4, 8):
        cfg = Config.load(preset="qwen3-30b-a3b", overrides=[f"global_batch_size={2 * n}", "micro_batch_size=2",
                                                            f"expert_model_parallel_size={n}"])
        plan = choose_memory_plan(cfg, n)
        assert plan["fits"] and plan["est_gb"] < 0.92 * 180 * 1e9 / 2**30
        names[n] = plan["name"]
        assert cfg.model.moe_keep_dispatched_factor == 0          # not without being allowed to
        cfg2 = Config.load(preset="qwen3-30b-a3b", overrides=[f"global_batch_size={2 * n}", "micro_batch_size=2",
                                                             f"expert_model_parallel_size={n}"])
        plan2 = choose_memory_plan(cfg2, n, allow_keep=True)
        assert plan2["name"] == plan["name"] and plan2["est_gb"] < 0.88 * 180 * 1e9 / 2**30
        if "keep_dispatched" in plan2:                            # a fixed-size copy, never the host-synchronising mode
            assert cfg2.model.moe_keep_dispatched_factor == (1.0 if n == 1 else 1.5) == plan2["keep_dispatched"]
            print(n, plan2)
        assert plan["optimizer_in_backward"]                       # one micro-batch per step: update inside backward
    assert names[8] == names[4] == "fp32-master+fp32-moments"
    assert names[1] == "bf16-weights+8bit-moments"


def test_moe_layer_benchmark_runs_on_cpu(tmp_path, capsys):
    """The end-to-end MoE layer benchmark on the library path (tiny shapes): a logic check of the script."""
    import importlib.util
    import json
    from pathlib import Path
    spec = importlib.util.spec_from_file_location("moe_layer_bench", Path(__file__).resolve().parent.parent / "benchmarks" / "moe_layer.py")
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    out = tmp_path / "r.json"
    assert mod.main(["--device", "cpu", "--tokens", "128", "--hidden", "64", "--ffn", "32", "--experts", "4", "--topk", "2",
                     "--iters", "2", "--json", str(out)]) == 0
    r = json.loads(out.read_text())
    assert r["world"] == 1 and r["rows_most_loaded_rank"] == 256 and r["fwd_ms"] > 0 and r["fwd_bwd_ms"] > r["fwd_ms"] * 0.5
