#!/usr/bin/env python
"""Benchmark of the cuda_sm100 hot path: compiled-graph samples/s on the Llama-style decoder layer
(hidden 4096, 32 heads x 128, SwiGLU FFN 11008, RoPE, causal SDPA; batch 8 x seq 2048 prefill, bf16).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

One JSON line is printed by rank 0. For N > 1 launch with torch.distributed.run (one rank per GPU);
the ranks are independent replicas (weak scaling: every GPU runs its own batch of 8), the only
collectives are the barrier and the max-over-ranks of the timed region.

``--impl reference`` times the reference's CPU path for the same graph: the eager (pattern-disabled)
decoder layer on the host cores, on a bounded sample of the workload.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import torch  # noqa: E402

METRIC = "compiled_graph_samples_per_s"
UNIT = "samples/s"
HIDDEN, HEADS, FFN, BATCH, SEQ = 4096, 32, 11008, 8, 2048
WORKLOAD = "llama_decoder_layer_prefill(hidden=4096,heads=32x128,ffn=11008,rope,causal_sdpa,batch=8,seq=2048)"

# FLOPs of the dense layers of one step (2*M*N*K each): q, k, v, o projections + gate/up (dual GEMM) + down.
TOKENS = BATCH * SEQ
GEMM_FLOPS = {
    "proj": 2 * TOKENS * HIDDEN * HIDDEN,
    "gate_up": 2 * 2 * TOKENS * FFN * HIDDEN,
    "down": 2 * TOKENS * HIDDEN * FFN,
}


def _peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return {"hbm_gbs": d["hbm_gbs"], "tflops": d["bf16_tflops_sustained"], "source": "measured (MEASURED_PEAKS.json, sustained)"}
    return {"hbm_gbs": 6650.0, "tflops": 1400.0, "source": "fallback (earlier measurement on this pool, sustained)"}


class ClockSampler(threading.Thread):
    """Samples SM clock and throttle reasons through NVML while the timed region runs."""

    def __init__(self, index: int, period_s: float = 0.1):
        super().__init__(daemon=True)
        self.index, self.period = index, period_s
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop = threading.Event()
        self.ok = False
        try:
            import pynvml

            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
            self.ok = True
        except Exception:
            self.ok = False

    def run(self):
        if not self.ok:
            return
        nv = self.nv
        names = {
            nv.nvmlClocksThrottleReasonHwSlowdown: "hw_slowdown",
            nv.nvmlClocksThrottleReasonHwThermalSlowdown: "hw_thermal_slowdown",
            nv.nvmlClocksThrottleReasonSwThermalSlowdown: "sw_thermal_slowdown",
            nv.nvmlClocksThrottleReasonSwPowerCap: "sw_power_cap",
        }
        while not self._stop.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                mask = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                for bit, name in names.items():
                    if mask & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            self._stop.wait(self.period)

    def stop(self):
        self._stop.set()

    def summary(self):
        if not self.ok or not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": ["unavailable"]}
        s = sorted(self.samples)
        return {"sm_mhz": s[len(s) // 2], "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons)}


def _physical_gpu_index(local_rank: int) -> int:
    vis = os.environ.get("CUDA_VISIBLE_DEVICES")
    if vis:
        try:
            return int(vis.split(",")[local_rank])
        except Exception:
            return local_rank
    return local_rank


# ------------------------------------------------------------------------------------------------
# reference arm / CPU baseline: the eager decoder layer on the host cores
# ------------------------------------------------------------------------------------------------
def _cpu_layer_and_inputs(seq: int):
    from xpu_graph_b200.workloads import make_llama_layer

    return make_llama_layer(seed=3, batch=1, seq=seq, hidden=HIDDEN, heads=HEADS, ffn=FFN, dtype=torch.bfloat16)


def _use_all_host_threads() -> int:
    """torch.distributed.run exports OMP_NUM_THREADS=1; the CPU arms are meant to use every core this process may run on."""
    try:
        n = len(os.sched_getaffinity(0))
    except AttributeError:
        n = os.cpu_count() or 1
    torch.set_num_threads(max(n, 1))
    return torch.get_num_threads()


def _time_cpu(layer, inputs, steps: int, warmup: int) -> float:
    with torch.no_grad():
        for _ in range(warmup):
            layer(*inputs)
        t0 = time.perf_counter()
        for _ in range(steps):
            layer(*inputs)
        return (time.perf_counter() - t0) / max(steps, 1)


def _pick_cpu_seq(budget_s: float, total_steps: int) -> int:
    """Choose the sample length so that total_steps passes fit the budget (calibrated on seq 128)."""
    layer, inp = _cpu_layer_and_inputs(128)
    per = _time_cpu(layer, inp, 1, 1)
    for seq in (2048, 1024, 512, 256):
        if per * (seq / 128.0) * 1.15 * total_steps <= budget_s:
            return seq
    return 128


def run_reference(args) -> dict:
    from oracle import ref_ops  # noqa: F401  (the oracle package is the reference path's restatement)

    steps, warmup = args.steps, max(args.warmup, 1)
    _use_all_host_threads()
    seq = _pick_cpu_seq(150.0, steps + warmup)
    layer, inp = _cpu_layer_and_inputs(seq)
    sec = _time_cpu(layer, inp, steps, warmup)
    # one pass = seq tokens of one sequence; a full sample is SEQ tokens
    value = (seq / SEQ) / sec
    cores = torch.get_num_threads()
    sample = f"eager decoder layer on CPU, batch 1 x seq {seq} per step (value scaled to {SEQ}-token samples)"
    return {
        "impl": "reference",
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": steps, "warmup": warmup,
        "ms_per_step": sec * 1e3, "higher_is_better": True, "scaling": "strong" if args.global_batch > 0 else "weak",
        "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic",
        "config": {"workload": WORKLOAD, "l2": "inputs_exceed_l2"},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }


# ------------------------------------------------------------------------------------------------
# our arm
# ------------------------------------------------------------------------------------------------
def _pci_bus_id(dev) -> str:
    """domain:bus:device.function of a CUDA device, as sysfs names it."""
    pr = torch.cuda.get_device_properties(dev)
    return f"{pr.pci_domain_id:04x}:{pr.pci_bus_id:02x}:{pr.pci_device_id:02x}.0"


def run_ours(args) -> dict | None:
    import torch.distributed as dist

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device; the cuda_sm100 target has no CPU path")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)

    from xpu_graph_b200 import lib, ops
    from xpu_graph_b200.fused_graphs import FusedLlamaDecoderLayer
    from xpu_graph_b200.replicas import shard_batch
    from xpu_graph_b200.workloads import make_llama_layer

    lib.load()
    # Weak scaling (default): every replica takes BATCH samples per step. --global-batch G: strong scaling, the G
    # samples of a step are split evenly over the replicas.
    strong = args.global_batch > 0
    if strong and args.global_batch % world != 0:
        raise SystemExit(f"--global-batch {args.global_batch} is not divisible by {world} GPUs")
    per_gpu = args.global_batch // world if strong else BATCH
    # Replica r owns samples [r*per_gpu, (r+1)*per_gpu) of the global batch: seeds differ per rank, weights do not.
    lo, hi = shard_batch(world * per_gpu, world, rank)
    assert hi - lo == per_gpu
    layer, (x, cos, sin) = make_llama_layer(seed=3, batch=per_gpu, seq=SEQ, hidden=HIDDEN, heads=HEADS, ffn=FFN,
                                            dtype=torch.bfloat16, device="cpu")
    if rank > 0:
        g = torch.Generator().manual_seed(3 + 1000 * rank)
        x = torch.randn(x.shape, generator=g).to(torch.bfloat16)
    layer = layer.to(dev)
    fused = FusedLlamaDecoderLayer(layer)
    via = "fused_graphs.FusedLlamaDecoderLayer (the post-rewrite op sequence assembled from the target's modules)"
    if not args.no_xpu_graph:
        # The real path when the xpu_graph package is importable on this box: torch.compile through the xpu_graph
        # pass pipeline with the cuda_sm100 target; it must reproduce the assembled sequence bit for bit.
        try:
            import logging

            from xpu_graph_b200.target.compat import reference_available

            # xpu_graph attaches a stdout handler to its logger unless one exists: give it a stderr one first,
            # this program's stdout carries exactly one JSON line
            xlog = logging.getLogger("xpu_graph")
            if not xlog.handlers:
                xlog.addHandler(logging.StreamHandler(sys.stderr))
                xlog.propagate = False
            if reference_available():
                from xpu_graph_b200 import target

                import contextlib

                probe = x[:1].to(dev)
                with torch.no_grad(), contextlib.redirect_stdout(sys.stderr):
                    compiled = torch.compile(layer, backend=target.backend(target.make_config()), dynamic=False)
                    same = torch.equal(compiled(probe, cos.to(dev), sin.to(dev)), fused(probe, cos.to(dev), sin.to(dev)))
                    if same:
                        compiled(x.to(dev), cos.to(dev), sin.to(dev))  # compile for the benchmark batch size
                if same:
                    assembled = fused

                    def fused(*a, _c=compiled):  # noqa: F811
                        with torch.no_grad():
                            return _c(*a)

                    via = "torch.compile(backend = xpu_graph pass pipeline + cuda_sm100 target)"
                else:
                    via += " [xpu_graph-compiled output differed from the assembled sequence: not used]"
        except Exception as e:  # keep the benchmark alive on any integration problem
            via += f" [xpu_graph path unavailable: {type(e).__name__}]"
    # With several replicas on one host, each keeps its pinned buffers (first touch) and copy threads next to its own GPU.
    if world > 1:
        from xpu_graph_b200.replicas import bind_to_device_numa_node
        try:
            bind_to_device_numa_node(_pci_bus_id(dev))
        except Exception:  # placement is an optimisation only
            pass
    x_host = x.pin_memory()
    out_host = torch.empty_like(x_host).pin_memory()
    x_dev, cos, sin = x_host.to(dev), cos.to(dev), sin.to(dev)

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(ms: float) -> float:
        if world == 1:
            return ms
        t = torch.tensor([ms], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    steps, warmup = args.steps, max(args.warmup, 3)
    stream = torch.cuda.current_stream()

    # ---- device-resident throughput -------------------------------------------------------
    for _ in range(warmup):
        fused(x_dev, cos, sin)
    sampler = ClockSampler(_physical_gpu_index(local_rank))
    sampler.start()
    ops.reset_counters()
    ops.GEMM_EVENTS = []
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for _ in range(steps):
        fused(x_dev, cos, sin)
    e1.record(stream)
    barrier()
    sampler.stop()
    ms_total = max_over_ranks(e0.elapsed_time(e1))
    launches = ops.launch_count()
    gemm_events, ops.GEMM_EVENTS = ops.GEMM_EVENTS, None
    ms_step = ms_total / steps
    value = world * per_gpu / (ms_step * 1e-3)

    # dominant kernel: the tcgen05 GEMM; algorithmic FLOPs per launch / mean launch duration (CUDA events)
    gemm_ms = sum(a.elapsed_time(b) for a, b, _ in gemm_events)
    gemm_flops = sum(f for _, _, f in gemm_events)
    peaks = _peaks()
    achieved = gemm_flops / (gemm_ms * 1e-3) / 1e12 if gemm_ms > 0 else 0.0
    # DRAM traffic per launch: from the ncu capture of the 8192 x 4096 x 11008 case, scaled by the FLOPs of the
    # launches timed here (traffic grows with the tiles processed)
    traffic = None
    tpath = os.path.join(ROOT, "profiles", "gemm_tc_pair_kernel_8192x4096x11008.md")
    if os.path.exists(tpath) and gemm_events:
        import re

        txt = open(tpath).read()
        m1 = re.search(r"traffic_bytes_per_launch\s*=\s*([0-9.e+]+)", txt)
        m2 = re.search(r"flops_per_launch\s*=\s*([0-9.e+]+)", txt)
        if m1 and m2:
            traffic = float(m1.group(1)) * (gemm_flops / len(gemm_events)) / float(m2.group(1))
    roofline = {"bound": "tensor", "achieved": achieved, "peak": peaks["tflops"], "unit": "TFLOP/s",
                "frac": achieved / peaks["tflops"], "traffic": traffic, "kernel": "gemm_tc_pair_kernel (tcgen05 cta_group::2 dense layers)",
                "launches_timed": len(gemm_events), "peak_source": peaks["source"],
                "gemm_share_of_step": gemm_ms / ms_total if ms_total > 0 else None}

    # ---- end to end: host buffers in, host buffers out, copies inside the timed region --------
    # Every step uploads its input from pinned host memory and downloads its output; the three stages
    # run on separate streams (HostPipeline), so uploads/downloads of neighbouring steps overlap compute.
    from xpu_graph_b200.pipeline import HostPipeline

    pipe = HostPipeline(fused, dev)
    out_hosts = [out_host, torch.empty_like(out_host).pin_memory()]
    for i in range(3):
        pipe.submit([x_host], out_hosts[i % 2], extra=(cos, sin))
    pipe.drain()
    barrier()
    e0 = pipe.record_start()
    for i in range(steps):
        pipe.submit([x_host], out_hosts[i % 2], extra=(cos, sin))
    e1 = pipe.record_end()
    pipe.drain()
    barrier()
    e2e_ms = max_over_ranks(e0.elapsed_time(e1)) / steps
    nbytes = x_host.numel() * x_host.element_size()
    e2e = {"value": world * per_gpu / (e2e_ms * 1e-3), "unit": UNIT, "h2d_bytes_per_step": nbytes, "d2h_bytes_per_step": nbytes,
           "ms_per_step": e2e_ms, "overlap": "3-stream pipeline: H2D(i+1) | compute(i) | D2H(i-1)"}

    status = lib.tc_status()
    if status != 0:
        raise SystemExit(f"bench.py: tensor-core kernel status word {status:#x} (a bounded wait expired); result invalid")

    # ---- CPU baseline (rank 0, N = 1 only): the oracle's eager layer on a bounded sample --------
    cpu_baseline = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        _use_all_host_threads()
        seq = _pick_cpu_seq(25.0, 2)
        cl, ci = _cpu_layer_and_inputs(seq)
        sec = _time_cpu(cl, ci, 1, 1)
        cpu_baseline = {"value": (seq / SEQ) / sec, "unit": UNIT, "cores": torch.get_num_threads(), "kind": "port",
                        "sample": f"eager decoder layer on CPU, 1 pass of batch 1 x seq {seq} (value scaled to {SEQ}-token samples)"}

    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    if rank != 0:
        return None
    return {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": steps, "warmup": warmup,
        "ms_per_step": ms_step, "higher_is_better": True, "scaling": "strong" if strong else "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic",
        "config": {"workload": WORKLOAD, "per_gpu_batch": per_gpu, "global_batch": world * per_gpu, "seq_len": SEQ,
                   "parallelism": f"replicas x{world} (no collectives)", "l2": "inputs_exceed_l2", "graph": via,
                   "tokens_per_s": value * SEQ},
        "clocks": sampler.summary(),
        "e2e": e2e,
        "gpu_launches": launches,
        "roofline": roofline,
        "cpu_baseline": cpu_baseline,
    }


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--global-batch", type=int, default=0,
                    help="strong scaling: split this many samples per step over the GPUs (default: 8 samples per GPU, weak scaling)")
    ap.add_argument("--no-xpu-graph", action="store_true", help="time the assembled op sequence even if xpu_graph is importable")
    args = ap.parse_args()
    if args.impl == "reference":
        if int(os.environ.get("RANK", "0")) != 0:
            return
        print(json.dumps(run_reference(args)), flush=True)
        return
    res = run_ours(args)
    if res is not None:
        print(json.dumps(res), flush=True)


if __name__ == "__main__":
    main()
