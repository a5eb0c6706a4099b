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
    monkeypatch.setattr(b, "_pick_cpu_sample", lambda budget, passes: (1, 64))  # a 64-token sample instead of seconds of CPU work
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
    # the same config keys as the GPU arm's line, so that the two lines describe one workload
    assert line["config"] == {**b._config(1, b.BATCH, line["config"]["graph"]), "tokens_per_s": line["config"]["tokens_per_s"]}
    from xpu_graph_b200.target.compat import reference_available

    if reference_available():  # the reference's own pipeline ran, not the eager stand-in
        assert line["cpu_baseline"]["kind"] == "reference" and "Target.none" in line["cpu_baseline"]["sample"]


def test_kernel_timers_read_the_abi_arguments():
    """bench.py derives FLOPs from the marshalled C-ABI arguments: the positions must follow include/xg_sm100.h."""
    from xpu_graph_b200 import lib

    b = _load_bench()
    gemm = [0] * len(lib.SIGNATURES["xg_gemm_bias_act_ws"][1])
    gemm[5:8] = [16384, 4096, 11008]
    assert b.KernelTimers._work("xg_gemm_bias_act_ws", gemm)[:2] == ("gemm", 2 * 16384 * 4096 * 11008)
    sw = [0] * len(lib.SIGNATURES["xg_gemm_swiglu"][1])
    sw[4:7] = [16384, 11008, 4096]
    assert b.KernelTimers._work("xg_gemm_swiglu", sw)[1] == 4 * 16384 * 11008 * 4096
    rp = [0] * len(lib.SIGNATURES["xg_gemm_rope"][1])
    rp[5:8] = [16384, 4096, 4096]
    assert b.KernelTimers._work("xg_gemm_rope", rp)[1] == 2 * 16384 * 4096 * 4096
    at = [0] * len(lib.SIGNATURES["xg_sdpa_fwd"][1])
    at[5:10] = [8, 32, 2048, 2048, 128]
    at[16] = 1
    assert b.KernelTimers._work("xg_sdpa_fwd", at)[:2] == ("attn", 4 * 8 * 32 * 2048 * 2048 * 128 // 2)
    assert b.KernelTimers._work("xg_rmsnorm", [0] * 13)[0] is None
    assert len(lib.SIGNATURES["xg_gemm_bias_act_ws"][1]) == 18 and len(lib.SIGNATURES["xg_sdpa_fwd"][1]) == 19
