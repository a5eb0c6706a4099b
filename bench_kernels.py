#!/usr/bin/env python
"""Small stand-alone cases of each kernel, for profiling and quick timing (the per-kernel companion of bench.py).

    python bench_kernels.py <case> [--iters N]

Each case holds well under a few GB on the device and launches the named kernel ``iters`` times
(default 3) after one warm-up, then prints the mean device time measured with CUDA events. Sizes are
larger than L2 so that DRAM counters mean something.
"""
from __future__ import annotations

import argparse
import os
import sys

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import torch  # noqa: E402


def _time(fn, iters):
    fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters


def _time_graphed(fn, reps=10, iters=5):
    """Device time per call with the host out of the picture: `reps` calls are captured in one CUDA graph."""
    fn()
    torch.cuda.synchronize()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        fn()
    torch.cuda.current_stream().wait_stream(side)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=side):
        for _ in range(reps):
            fn()
    graph.replay()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        graph.replay()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / (iters * reps)


def sweep():
    """Stand-alone sweeps of the norm and dense-layer kernels (the shapes of benchmark configs 2 and 3),
    printed as markdown tables with the achieved fraction of the measured peaks."""
    import json
    import os

    from xpu_graph_b200 import workloads as W

    X = torch.ops.xg_sm100
    dev = torch.device("cuda")
    root = ROOT
    peaks = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}
    pk = os.path.join(root, "MEASURED_PEAKS.json")
    if os.path.exists(pk):
        peaks = json.load(open(pk))
    print(f"peaks: HBM {peaks['hbm_gbs']:.0f} GB/s, bf16 {peaks['bf16_tflops']:.0f} TFLOP/s (burst)\n")
    print("| rows | hidden | pattern | us | GB/s | of measured HBM |")
    print("|---:|---:|---|---:|---:|---:|")
    for hidden in W.NORM_SWEEP_HIDDEN:
        for rows in W.NORM_SWEEP_ROWS:
            x, r, gamma, beta = W.make_norm_inputs(rows, hidden, device=dev)
            cases = [
                ("add+RMSNorm (1 out)", lambda: X.add_rms_norm_y(x, r, gamma, 1e-6), 6),
                ("add+RMSNorm (2 out)", lambda: X.add_rms_norm(x, r, gamma, 1e-6), 8),
                ("add+LayerNorm (1 out)", lambda: X.add_layer_norm_y(x, r, gamma, beta, 1e-5), 6),
                ("add+LayerNorm (2 out)", lambda: X.add_layer_norm(x, r, gamma, beta, 1e-5), 8),
            ]
            for name, fn, bpe in cases:
                ms = _time_graphed(fn)
                gbs = bpe * rows * hidden / ms / 1e6
                print(f"| {rows} | {hidden} | {name} | {ms * 1e3:.1f} | {gbs:.0f} | {gbs / peaks['hbm_gbs']:.2f} |")
            del x, r
    print()
    print("| M | K | N | epilogue | us | TFLOP/s | of measured bf16 | GB/s (A+W+out) |")
    print("|---:|---:|---:|---|---:|---:|---:|---:|")
    for (M, K, N) in W.GEMM_SWEEP:
        a, w, b = W.make_gemm_inputs(M, K, N, device=dev)
        for act in ("gelu", "silu"):
            # 20 calls per graph for the cells of a few microseconds (the gap between graph replays would be 5-10 % of a
            # 5-call graph there), 5 for the long ones
            ms = _time_graphed(lambda: X.dense(a, w, True, b, None, act), reps=20 if M <= 256 else 5)
            tf = 2 * M * N * K / ms / 1e9
            gbs = 2 * (M * K + N * K + M * N) / ms / 1e6
            print(f"| {M} | {K} | {N} | bias+{act} | {ms * 1e3:.1f} | {tf:.0f} | {tf / peaks['bf16_tflops']:.2f} | {gbs:.0f} |")
        del a, w
    return 0


def graphs(iters: int) -> int:
    """The two fp32 configurations that are not the benchmark line: the small encoder block (config 1, batch 2 x seq 128,
    launch-bound: also timed as one replayed CUDA graph) and the recsys graph (config 5, batch 16384), each as the fused op
    sequence of this target and as the same model in eager CUDA PyTorch (TF32 off)."""
    from xpu_graph_b200.fused_graphs import FusedEncoderBlock, FusedRecsysGraph
    from xpu_graph_b200.graph_runner import CUDAGraphRunner
    from xpu_graph_b200.workloads import make_encoder, make_recsys

    dev = torch.device("cuda")
    torch.backends.cuda.matmul.allow_tf32 = False
    for name, make, fused_cls in (("encoder block (config 1)", make_encoder, FusedEncoderBlock), ("recsys graph (config 5)", make_recsys, FusedRecsysGraph)):
        model, inputs = make()
        model = model.to(dev).eval()
        inputs = [t.to(dev) for t in (inputs if isinstance(inputs, (list, tuple)) else [inputs])]
        fused = fused_cls(model)
        with torch.no_grad():
            want, got = model(*inputs), fused(*inputs)
            err = (got - want).abs().max().item() / max(want.abs().max().item(), 1e-30)
            ms_eager = _time(lambda: model(*inputs), iters)
            ms_fused = _time(lambda: fused(*inputs), iters)
            runner = CUDAGraphRunner(fused)
            runner.capture(*inputs)
            ms_graph = _time(lambda: runner(*inputs), iters)
        n = inputs[0].shape[0]
        print(f"{name}: batch {n}: fused {ms_fused:.4f} ms ({n / ms_fused * 1e3:.0f} samples/s), as one CUDA graph {ms_graph:.4f} ms "
              f"({n / ms_graph * 1e3:.0f} samples/s), eager CUDA {ms_eager:.4f} ms; max |diff| / scale vs eager {err:.1e}")
    return 0


def main(argv=None):
    from xpu_graph_b200 import lib, ops  # noqa: F401

    X = torch.ops.xg_sm100
    ap = argparse.ArgumentParser()
    ap.add_argument("case", choices=["sweep", "gemm_splitk", "gemm", "gemm_swiglu", "gemm_small_m", "add_rms_norm", "layer_norm", "sdpa", "rope", "swiglu",
                                     "gather", "slice_cat", "gemm_f32", "slice_sum_cat", "mul_sum_cat", "batch_dense", "graphs", "layer_gemms",
                                     "gemm_m256", "gemm_m64", "gemm_small_sweep", "layer_norm_small", "sdpa_full", "sdpa_simt", "gemm_f32_small",
                                     "mlp2", "mlp_small"])
    ap.add_argument("--iters", type=int, default=3)
    args = ap.parse_args(argv)
    if args.case == "sweep":
        return sweep()
    if args.case == "graphs":
        return graphs(args.iters)
    dev = torch.device("cuda")
    bf = torch.bfloat16
    g = torch.Generator(device=dev).manual_seed(0)

    def rn(*shape, dtype=bf, std=1.0):
        return (torch.randn(*shape, generator=g, device=dev) * std).to(dtype)

    if args.case == "gemm":
        M, K, N = 8192, 4096, 11008
        a, w, b = rn(M, K), rn(N, K, std=0.02), rn(N, std=0.02)
        ms = _time(lambda: X.dense(a, w, True, b, None, "gelu"), args.iters)
        print(f"gemm {M}x{K}x{N} gelu: {ms:.4f} ms, {2 * M * N * K / ms / 1e9:.1f} TFLOP/s")
    elif args.case == "gemm_small_m":
        M, K, N = 256, 4096, 11008
        a, w, b = rn(M, K), rn(N, K, std=0.02), rn(N, std=0.02)
        ms = _time(lambda: X.dense(a, w, True, b, None, "silu"), args.iters)
        print(f"gemm {M}x{K}x{N} silu: {ms:.4f} ms, {2 * M * N * K / ms / 1e9:.1f} TFLOP/s")
    elif args.case == "gemm_splitk":
        # small-M dense layers: split-K with scratch (what the op does) against the same kernel without scratch
        import ctypes

        L = lib.load()
        K, N = 4096, 11008
        w, b = rn(N, K, std=0.02), rn(N, std=0.02)
        for M in (16, 64, 128, 256):
            a = rn(M, K)
            out = torch.empty(M, N, device=dev, dtype=bf)
            st = torch.cuda.current_stream().cuda_stream

            def plain():
                L.xg_gemm_bias_act(a.data_ptr(), w.data_ptr(), b.data_ptr(), None, out.data_ptr(), M, N, K, K, K, N, 0, 1, 1, 1,
                                   torch.cuda.current_stream().cuda_stream)

            ms0 = _time_graphed(plain)
            ms1 = _time_graphed(lambda: X.dense(a, w, True, b, None, "gelu"))
            ws = L.xg_gemm_workspace_bytes(M, N, K, 1)
            print(f"M={M}: no scratch {ms0 * 1e3:.1f} us, op (scratch {ws / 1e6:.1f} MB) {ms1 * 1e3:.1f} us, "
                  f"weights at {2 * N * K / min(ms0, ms1) / 1e6:.0f} GB/s")
    elif args.case == "layer_gemms":
        # the six dense launches of one benchmark step (Llama-style layer, 8 x 2048 tokens, hidden 4096, FFN 11008)
        T, Hd, F, S, D = 16384, 4096, 11008, 2048, 128
        x, res = rn(T, Hd), rn(T, Hd)
        wq, wv, wo = rn(Hd, Hd, std=0.02), rn(Hd, Hd, std=0.02), rn(Hd, Hd, std=0.02)
        wg, wu, wd = rn(F, Hd, std=0.02), rn(F, Hd, std=0.02), rn(Hd, F, std=0.02)
        cos, sin = rn(S, D), rn(S, D)
        h = rn(T, F)
        ops_ = [("q/k projection + RoPE (xg_gemm_rope)", 2 * T * Hd * Hd, lambda: X.dense_rope(x, wq, cos, sin, S, D)),
                ("v projection (xg_gemm_bias_act)", 2 * T * Hd * Hd, lambda: X.dense(x, wv, True, None, None, "none")),
                ("o projection + residual", 2 * T * Hd * Hd, lambda: X.dense(x, wo, True, None, res, "none")),
                ("gate/up dual GEMM + SwiGLU (xg_gemm_swiglu)", 4 * T * F * Hd, lambda: X.dense_swiglu(x, wg, wu)),
                ("down projection + residual", 2 * T * Hd * F, lambda: X.dense(h, wd, True, None, res, "none"))]
        for name, flops, fn in ops_:
            ms = _time(fn, args.iters)
            print(f"{name}: {ms:.4f} ms, {flops / ms / 1e9:.1f} TFLOP/s")
    elif args.case == "gemm_m256":
        M, K, N = 256, 4096, 4096
        a, w, b = rn(M, K), rn(N, K, std=0.02), rn(N, std=0.02)
        ms = _time_graphed(lambda: X.dense(a, w, True, b, None, "gelu"))
        print(f"gemm {M}x{K}x{N} gelu: {ms * 1e3:.1f} us, {2 * M * N * K / ms / 1e9:.1f} TFLOP/s, "
              f"{2 * (M * K + N * K + M * N) / ms / 1e6:.0f} GB/s (A + W + out)")
    elif args.case == "gemm_m64":
        # split-K through scratch memory (the op allocates the fp32 partial sums) followed by the reduction pass
        M, K, N = 64, 4096, 4096
        a, w, b = rn(M, K), rn(N, K, std=0.02), rn(N, std=0.02)
        ms = _time_graphed(lambda: X.dense(a, w, True, b, None, "gelu"))
        print(f"gemm {M}x{K}x{N} gelu (split-K + reduce): {ms * 1e3:.1f} us, {2 * (M * K + N * K + M * N) / ms / 1e6:.0f} GB/s (A + W + out)")
    elif args.case == "gemm_small_sweep":
        # dense layers with few output tiles against torch's (cuBLAS) linear on the same inputs, device time per call
        import torch.nn.functional as F_

        for (M, K, N) in [(16, 4096, 4096), (64, 4096, 4096), (128, 4096, 4096), (256, 4096, 4096), (512, 4096, 4096),
                          (1024, 4096, 4096), (16, 4096, 11008), (128, 4096, 11008), (256, 4096, 11008), (512, 4096, 11008)]:
            a, w, b = rn(M, K), rn(N, K, std=0.02), rn(N, std=0.02)
            ms = _time_graphed(lambda: X.dense(a, w, True, b, None, "none"))
            ms2 = _time_graphed(lambda: F_.linear(a, w, b))
            gbs = 2 * (M * K + N * K + M * N) / ms / 1e6
            print(f"| {M} | {K} | {N} | {ms * 1e3:.1f} | {2 * M * N * K / ms / 1e9:.0f} | {gbs:.0f} | {ms2 * 1e3:.1f} |")
    elif args.case == "layer_norm_small":
        rows, hidden = 8192, 4096
        x, r, w, b = rn(rows, hidden), rn(rows, hidden), rn(hidden), rn(hidden)
        ms = _time_graphed(lambda: X.add_layer_norm_y(x, r, w, b, 1e-5))
        print(f"add_layer_norm (1 output) {rows}x{hidden}: {ms * 1e3:.1f} us, {6 * rows * hidden / ms / 1e6:.0f} GB/s")
    elif args.case == "sdpa_full":
        B, H, S, D = 8, 32, 2048, 128
        q, k, v = rn(B, H, S, D), rn(B, H, S, D), rn(B, H, S, D)
        for causal in (True, False):
            ms = _time_graphed(lambda: X.sdpa(q, k, v, None, D ** -0.5, causal), reps=5)
            flops = 4 * B * H * S * S * D / (2 if causal else 1)
            print(f"sdpa {'causal' if causal else 'full'} {B}x{H}x{S}x{D}: {ms:.4f} ms, {flops / ms / 1e9:.1f} TFLOP/s")
    elif args.case == "sdpa_simt":
        # the encoder block's attention (fp32, [1, 8, 128, 64] after the batch is folded into the heads)
        B, H, S, D = 1, 8, 128, 64
        q, k, v = (rn(B, H, S, D, dtype=torch.float32) for _ in range(3))
        ms = _time_graphed(lambda: X.sdpa(q, k, v, None, 0.125, False))
        print(f"sdpa fp32 {B}x{H}x{S}x{D}: {ms * 1e3:.1f} us, {4 * B * H * S * S * D / ms / 1e6:.1f} GFLOP/s")
    elif args.case == "gemm_f32_small":
        # the encoder block's dense layers (fp32 FMA kernel): 256 rows, K / N of the four layers
        for (M, K, N) in [(256, 256, 768), (256, 256, 256), (256, 256, 1024), (256, 1024, 256)]:
            a, w, b = rn(M, K, dtype=torch.float32), rn(N, K, dtype=torch.float32, std=0.02), rn(N, dtype=torch.float32, std=0.02)
            ms = _time_graphed(lambda: X.dense(a, w, True, b, None, "gelu"))
            print(f"gemm_f32 {M}x{K}x{N} gelu: {ms * 1e3:.1f} us, {2 * M * N * K / ms / 1e9:.2f} TFLOP/s")
    elif args.case == "mlp2":
        # two / three narrow 16-bit dense layers as one kernel (hidden activations on chip) against the same layers as one
        # launch each of this library and as eager torch (cuBLAS + elementwise kernels), device time per call
        import torch.nn.functional as F_

        print("| rows | layer widths | one kernel (us) | one launch per layer (us) | eager torch (us) | hidden bytes kept on chip (MB) |")
        print("|---:|---|---:|---:|---:|---:|")
        for (M, K1, N1, N2) in [(16384, 512, 256, 256), (65536, 256, 256, 128), (16384, 256, 128, 64), (4096, 1024, 256, 40),
                                (300, 256, 128, 64)]:
            x, w1, b1 = rn(M, K1), rn(N1, K1, std=K1 ** -0.5), rn(N1, std=0.1)
            w2, b2 = rn(N2, N1, std=N1 ** -0.5), rn(N2, std=0.1)
            ms = _time_graphed(lambda: X.mlp2(x, w1, b1, w2, b2, "relu", "none"))
            ms2 = _time_graphed(lambda: X.dense(X.dense(x, w1, True, b1, None, "relu"), w2, True, b2, None, "none"))
            ms3 = _time_graphed(lambda: F_.linear(torch.relu(F_.linear(x, w1, b1)), w2, b2))
            print(f"| {M} | {K1} -> {N1} -> {N2} | {ms * 1e3:.1f} | {ms2 * 1e3:.1f} | {ms3 * 1e3:.1f} | {4 * M * N1 / 1e6:.1f} |")
        for (M, K1, N1, N2, N3) in [(16384, 512, 256, 256, 128), (65536, 256, 256, 128, 64), (16384, 256, 128, 64, 32)]:
            x, w1, b1 = rn(M, K1), rn(N1, K1, std=K1 ** -0.5), rn(N1, std=0.1)
            w2, b2 = rn(N2, N1, std=N1 ** -0.5), rn(N2, std=0.1)
            w3, b3 = rn(N3, N2, std=N2 ** -0.5), rn(N3, std=0.1)
            ms = _time_graphed(lambda: X.mlp3(x, w1, b1, w2, b2, w3, b3, "relu", "relu", "none"))
            ms2 = _time_graphed(lambda: X.dense(X.dense(X.dense(x, w1, True, b1, None, "relu"), w2, True, b2, None, "relu"),
                                                w3, True, b3, None, "none"))
            ms3 = _time_graphed(lambda: F_.linear(torch.relu(F_.linear(torch.relu(F_.linear(x, w1, b1)), w2, b2)), w3, b3))
            print(f"| {M} | {K1} -> {N1} -> {N2} -> {N3} | {ms * 1e3:.1f} | {ms2 * 1e3:.1f} | {ms3 * 1e3:.1f} | {4 * M * (N1 + N2) / 1e6:.1f} |")
    elif args.case == "mlp_small":
        # narrow towers with the weights resident in shared memory (one launch, FMA arithmetic) against one launch per
        # layer of this library and eager torch, device time per call; and small fp32 / full-bias groups in one launch
        import torch.nn.functional as F_

        print("| dtype | rows | layer widths | one kernel (us) | one launch per layer (us) | eager torch (us) |")
        print("|---|---:|---|---:|---:|---:|")
        for dtype, M, dims in [(torch.float16, 16, (20, 32, 16, 1)), (torch.float32, 16384, (64, 32, 16, 1)),
                               (torch.float32, 16384, (128, 64, 32)), (torch.bfloat16, 16384, (100, 64, 16)),
                               (torch.float32, 65536, (26, 128, 64, 8))]:
            x = rn(M, dims[0], dtype=dtype)
            ws = [rn(dims[i + 1], dims[i], dtype=dtype, std=dims[i] ** -0.5) for i in range(len(dims) - 1)]
            bs = [rn(dims[i + 1], dtype=dtype, std=0.1) for i in range(len(dims) - 1)]
            acts = ["relu"] * (len(ws) - 1) + ["none"]

            def layers(x=x, ws=ws, bs=bs, acts=acts):
                y = x
                for w, b, a in zip(ws, bs, acts):
                    y = X.dense(y, w, True, b, None, a)
                return y

            def eager(x=x, ws=ws, bs=bs, acts=acts):
                y = x
                for w, b, a in zip(ws, bs, acts):
                    y = F_.linear(y, w, b)
                    y = torch.relu(y) if a == "relu" else y
                return y

            ms = _time_graphed(lambda: X.mlp_small(x, ws, bs, ",".join(acts), 0))
            ms2 = _time_graphed(layers)
            ms3 = _time_graphed(eager)
            print(f"| {str(dtype)[6:]} | {M} | {' -> '.join(map(str, dims))} | {ms * 1e3:.1f} | {ms2 * 1e3:.1f} | {ms3 * 1e3:.1f} |")
        print("| dtype | layers x (M x K x N) | bias | one grouped launch (us) | one launch per layer (us) | eager torch (us) |")
        print("|---|---|---|---:|---:|---:|")
        for dtype, T, M, K, N, full in [(torch.float32, 8, 5, 8, 7, True), (torch.float32, 16, 512, 64, 64, False),
                                        (torch.bfloat16, 8, 512, 64, 64, True)]:
            xs = [rn(M, K, dtype=dtype) for _ in range(T)]
            ws = [rn(N, K, dtype=dtype, std=K ** -0.5) for _ in range(T)]
            bs = [rn(M, N, dtype=dtype) if full else rn(N, dtype=dtype) for _ in range(T)]
            ms = _time_graphed(lambda: X.combo_dense(xs, ws, True, bs, "relu"))
            ms2 = _time_graphed(lambda: [X.dense(x, w, True, None if full else b, b if full else None, "relu") for x, w, b in zip(xs, ws, bs)])
            ms3 = _time_graphed(lambda: [torch.relu(F_.linear(x, w) + b) for x, w, b in zip(xs, ws, bs)])
            print(f"| {str(dtype)[6:]} | {T} x ({M} x {K} x {N}) | {'[M, N]' if full else '[N]'} | {ms * 1e3:.1f} | {ms2 * 1e3:.1f} | {ms3 * 1e3:.1f} |")
    elif args.case == "gemm_swiglu":
        M, K, N = 8192, 4096, 11008
        a, wg, wu = rn(M, K), rn(N, K, std=0.02), rn(N, K, std=0.02)
        ms = _time(lambda: X.dense_swiglu(a, wg, wu), args.iters)
        print(f"gemm_swiglu {M}x{K}x{N}: {ms:.4f} ms, {4 * M * N * K / ms / 1e9:.1f} TFLOP/s")
    elif args.case == "gemm_f32":
        M, K, N = 16384, 1728, 1024
        a, w, b = rn(M, K, dtype=torch.float32), rn(N, K, dtype=torch.float32, std=0.02), rn(N, dtype=torch.float32, std=0.02)
        ms = _time(lambda: X.dense(a, w, True, b, None, "relu"), args.iters)
        print(f"gemm_f32 {M}x{K}x{N} relu: {ms:.4f} ms, {2 * M * N * K / ms / 1e9:.1f} TFLOP/s")
    elif args.case == "add_rms_norm":
        rows, hidden = 16384, 8192
        x, r, w = rn(rows, hidden), rn(rows, hidden), rn(hidden)
        ms = _time(lambda: X.add_rms_norm(x, r, w, 1e-6), args.iters)
        print(f"add_rms_norm (2 outputs) {rows}x{hidden}: {ms:.4f} ms, {8 * rows * hidden / ms / 1e6:.0f} GB/s")
    elif args.case == "layer_norm":
        rows, hidden = 32768, 4096
        x, r, w, b = rn(rows, hidden), rn(rows, hidden), rn(hidden), rn(hidden)
        ms = _time(lambda: X.add_layer_norm_y(x, r, w, b, 1e-5), args.iters)
        print(f"add_layer_norm (1 output) {rows}x{hidden}: {ms:.4f} ms, {6 * rows * hidden / ms / 1e6:.0f} GB/s")
    elif args.case == "sdpa":
        B, H, S, D = 4, 32, 2048, 128
        q, k, v = rn(B, H, S, D), rn(B, H, S, D), rn(B, H, S, D)
        ms = _time(lambda: X.sdpa(q, k, v, None, D ** -0.5, True), args.iters)
        print(f"sdpa causal {B}x{H}x{S}x{D}: {ms:.4f} ms, {2 * B * H * S * S * D / ms / 1e9:.1f} TFLOP/s")
    elif args.case == "rope":
        B, H, S, D = 8, 32, 2048, 128
        x, cos, sin = rn(B, H, S, D), rn(S, D), rn(S, D)
        ms = _time(lambda: X.rope(x, cos, sin), args.iters)
        print(f"rope {B}x{H}x{S}x{D}: {ms:.4f} ms, {4 * x.numel() / ms / 1e6:.0f} GB/s")
    elif args.case == "swiglu":
        rows, cols = 16384, 11008
        a, b = rn(rows, cols), rn(rows, cols)
        ms = _time(lambda: X.swiglu(a, b), args.iters)
        print(f"swiglu {rows}x{cols}: {ms:.4f} ms, {6 * rows * cols / ms / 1e6:.0f} GB/s")
    elif args.case == "gather":
        rows, F, D, T = 65536, 26, 64, 100000
        tables = [rn(T, D, dtype=torch.float32, std=0.01) for _ in range(F)]
        idx = torch.randint(0, T, (rows, F), generator=g, device=dev)
        mask = torch.rand(rows, 1, generator=g, device=dev) < 0.3
        ms = _time(lambda: X.gather_stack(tables, idx, mask, True), args.iters)
        print(f"gather_stack {rows}x{F}x{D}: {ms:.4f} ms, {(2 * rows * F * D * 4 + rows * F * 8) / ms / 1e6:.0f} GB/s")
    elif args.case == "batch_dense":
        b, M, K, N = 64, 256, 512, 512
        x, w = rn(b, M, K), rn(b, N, K, std=0.02)
        bias = rn(b, 1, N, std=0.02)
        ms = _time(lambda: X.batch_dense(x, w, True, bias, None, "relu"), args.iters)
        ms2 = _time(lambda: torch.relu(torch.baddbmm(bias, x, w.transpose(1, 2))), args.iters)
        print(f"batch_dense {b} x {M}x{K}x{N} bf16: {ms:.4f} ms, {2 * b * M * N * K / ms / 1e9:.1f} TFLOP/s (torch baddbmm+relu {ms2:.4f} ms)")
    elif args.case == "slice_sum_cat":
        B, R, C = 65536, 50, 64
        x = rn(B, R, C, dtype=torch.float32)
        starts, ends = [0, 0, 0, 0], [10, 25, 50, 4]
        ms = _time(lambda: X.slice_sum_cat(x, starts, ends), args.iters)
        print(f"slice_sum_cat {B}x{R}x{C} fp32, 4 prefix ranges: {ms:.4f} ms, {(B * R * C + B * 4 * C) * 4 / ms / 1e6:.0f} GB/s")
    elif args.case == "mul_sum_cat":
        B, R, C, n = 65536, 10, 64, 4
        lhs = [rn(B, R, C, dtype=torch.float32) for _ in range(n)]
        rhs = [rn(B, R, C, dtype=torch.float32) for _ in range(n)]
        ms = _time(lambda: X.mul_sum_cat(lhs, rhs), args.iters)
        print(f"mul_sum_cat {n} x {B}x{R}x{C} fp32: {ms:.4f} ms, {(2 * n * B * R * C + B * n * C) * 4 / ms / 1e6:.0f} GB/s")
    elif args.case == "slice_cat":
        rows, width = 65536, 4310
        src = rn(rows, width, dtype=torch.float32)
        starts = [64 * i for i in range(50)]
        ends = [s + 64 for s in starts]
        ms = _time(lambda: X.slice_cat(src, starts, ends, None, False), args.iters)
        print(f"slice_cat {rows}x{width} -> 50x64: {ms:.4f} ms, {2 * rows * 50 * 64 * 4 / ms / 1e6:.0f} GB/s")
    if lib.tc_status() != 0:
        print("WARNING: tensor-core status word is non-zero", file=sys.stderr)
        return 1
    return 0


if __name__ == "__main__":
    sys.exit(main())
