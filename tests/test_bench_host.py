"""CPU-side checks of bench.py: the reference arm and the CPU-baseline leg run the CPU port for as
many decode steps as the driver asks for (page tables sized for every appended token) and print the
keys the bench contract names. Run on a model cut down to two layers and a small vocabulary so the
whole file takes seconds."""
import argparse
import json
import os
import subprocess
import sys

import bench

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def small_args(**over):
    base = dict(gpus=1, steps=20, warmup=5, impl="reference", lanes=128, seed=0, pool_pages=36000, ctx_max=8192, layers=2, no_cpu_baseline=False, no_graph_replay=False, no_moe=True, moe_lanes=256, moe_steps=8, moe_layers=0, repeats=0)
    base.update(over)
    return argparse.Namespace(**base)


def test_reference_arm_crosses_page_boundaries(monkeypatch):
    # 1 + warmup + steps = 26 appended tokens: more than one 16-token page beyond the context
    monkeypatch.setitem(bench.QWEN3_06B, "vocab", 4096)
    line = bench.run_reference(small_args())
    assert line["impl"] == "reference" and line["steps"] == 20 and line["warmup"] == 5
    assert line["value"] > 0 and line["unit"] == "tok/s" and line["higher_is_better"] is True
    assert line["cpu_baseline"]["kind"] == "port" and line["cpu_baseline"]["cores"] >= 1
    assert line["e2e"] == {"value": line["value"], "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}
    json.dumps(line)


def test_cpu_sample_tables_hold_every_appended_token(monkeypatch):
    monkeypatch.setitem(bench.QWEN3_06B, "vocab", 4096)
    cfg = dict(bench.QWEN3_06B, layers=1)
    for appended in (2, 27, 260):
        _, pick, tables, _ = bench.cpu_sample(small_args(), cfg, 3, 1, appended)
        for (ctx, _), table in zip(pick, tables):
            assert table.shape[0] * bench.PAGE >= ctx + appended


def test_cpu_baseline_reports_one_core_and_all_cores(monkeypatch):
    monkeypatch.setitem(bench.QWEN3_06B, "vocab", 4096)
    cfg = dict(bench.QWEN3_06B, layers=2)
    base = bench.cpu_baseline(small_args(), cfg)
    assert base["kind"] == "port" and base["cores"] >= 1 and base["value"] > 0
    assert base["one_core"]["cores"] == 1 and base["one_core"]["value"] > 0
    assert "median of 5" in base["sample"]


def test_reference_arm_command_line_prints_one_json_line():
    env = dict(os.environ, PYTHONPATH=ROOT)
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--steps", "3", "--warmup", "1", "--layers", "1"],
                         capture_output=True, text=True, env=env, timeout=600)
    assert out.returncode == 0, out.stderr[-2000:]
    lines = [l for l in out.stdout.splitlines() if l.strip()]
    assert len(lines) == 1
    line = json.loads(lines[0])
    assert line["impl"] == "reference" and line["value"] > 0
