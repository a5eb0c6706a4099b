"""The CPU arm of bench.py (--impl reference) on a tiny sample: it must run without a GPU and print the contract's keys."""
import argparse
import importlib.util
import os

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _load_bench():
    spec = importlib.util.spec_from_file_location("xg_bench_under_test", os.path.join(ROOT, "bench.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def test_reference_arm_line(monkeypatch):
    b = _load_bench()
    monkeypatch.setattr(b, "_pick_cpu_seq", lambda budget, passes: 64)  # a 64-token sample instead of seconds of CPU work
    args = argparse.Namespace(gpus=1, steps=1, warmup=1, impl="reference", no_cpu_baseline=True, no_xpu_graph=False,
                              global_batch=0)
    line = b.run_reference(args)
    for key in ("metric", "value", "unit", "n_gpus", "steps", "warmup", "ms_per_step", "higher_is_better", "scaling",
                "vs_baseline", "dtype", "data", "config", "impl", "cpu_baseline", "e2e"):
        assert key in line, key
    assert line["impl"] == "reference" and line["scaling"] == "weak" and line["value"] > 0
    assert line["cpu_baseline"]["kind"] in ("port", "reference") and line["cpu_baseline"]["cores"] >= 1
    assert line["e2e"]["h2d_bytes_per_step"] == 0 and line["e2e"]["d2h_bytes_per_step"] == 0
    assert line["config"]["workload"] == b.WORKLOAD
