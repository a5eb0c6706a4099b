"""The real thing on the GPU: eager models compiled by torch.compile through the xpu_graph pass pipeline with
the cuda_sm100 target, executed on sm_100a kernels, compared with the eager (pattern-disabled) models on CPU.

Needs the xpu_graph package importable on the GPU box (an offline install under baseline/_ref, or XPU_GRAPH_SRC);
skipped otherwise. The graph rewrites themselves are covered without a GPU in tests/test_target_patterns.py.
"""
import logging
import time

import pytest
import torch

from tests.helpers import assert_parity
from xpu_graph_b200.target.compat import reference_available

pytestmark = [pytest.mark.gpu, pytest.mark.skipif(not reference_available(), reason="xpu_graph package not importable")]


@pytest.fixture(autouse=True)
def _reset_dynamo():
    torch._dynamo.reset()
    yield
    torch._dynamo.reset()


def _compile_run(model, inputs, **cfg):
    from xpu_graph_b200 import target

    cap = {}
    be = target.backend(target.make_config(**cfg), capture=cap)
    compiled = torch.compile(model, backend=be, dynamic=False)
    with torch.no_grad():
        out = compiled(*inputs)
    torch.cuda.synchronize()
    gm = cap["gm"]
    graph = getattr(gm, "gm", gm).graph if not hasattr(gm, "graph") else gm.graph
    mods = [n.target for n in graph.nodes if n.op == "call_module"]
    atens = [str(n.target) for n in graph.nodes if n.op == "call_function"]
    return compiled, out, mods, atens


def test_llama_layer_compiled_on_gpu(cuda_device):
    from xpu_graph_b200 import lib
    from xpu_graph_b200.workloads import make_llama_layer

    model, (x, cos, sin) = make_llama_layer(seed=3, batch=2, seq=320, hidden=512, heads=4, ffn=1376)
    with torch.no_grad():
        want = model(x, cos, sin)
    model = model.to(cuda_device)
    inputs = (x.to(cuda_device), cos.to(cuda_device), sin.to(cuda_device))
    compiled, got, mods, atens = _compile_run(model, inputs)
    assert lib.tc_status() == 0
    assert_parity(got, want, "compiled llama layer")
    assert sorted(mods) == sorted(["custom_rms_norm", "xg_dense_rope", "xg_dense_rope", "custom_dense_layer_replacement",
                                   "xg_sdpa", "xg_dense_residual", "custom_rms_norm", "xg_dense_swiglu",
                                   "xg_dense_residual"]), mods
    assert all(("reshape" in a or "transpose" in a or "view" in a) for a in atens), atens


def test_llama_layer_benchmark_size_compiled_on_gpu(cuda_device):
    """The graph whose throughput is the headline number: the hidden-4096 / FFN-11008 decoder layer (seed 3) on one
    2048-token sequence, compiled by torch.compile through the xpu_graph pipeline with this target. The compiled graph
    must be the nine-op sequence whose ops tests/test_gpu_graphs.py::test_llama_layer_benchmark_size checks one by one
    at this size, its result must equal that sequence's bit for bit, and end to end it must be at least as close to
    the layer in fp32 as the eager bf16 layer on CPU is (max-abs and mean-rel against the eager result are printed)."""
    from tests.test_gpu_graphs import _end_to_end_gate
    from xpu_graph_b200 import lib
    from xpu_graph_b200.fused_graphs import FusedLlamaDecoderLayer
    from xpu_graph_b200.workloads import make_llama_layer

    model, (x, cos, sin) = make_llama_layer(seed=3, batch=1, seq=2048, hidden=4096, heads=32, ffn=11008)
    with torch.no_grad():
        want = model(x, cos, sin)
        exact = model.float()(x.float(), cos.float(), sin.float())
    model = model.to(torch.bfloat16).to(cuda_device)
    inputs = (x.to(cuda_device), cos.to(cuda_device), sin.to(cuda_device))
    compiled, got, mods, atens = _compile_run(model, inputs)
    assert lib.tc_status() == 0
    assert sorted(mods) == sorted(["custom_rms_norm", "xg_dense_rope", "xg_dense_rope", "custom_dense_layer_replacement",
                                   "xg_sdpa", "xg_dense_residual", "custom_rms_norm", "xg_dense_swiglu",
                                   "xg_dense_residual"]), mods
    assert torch.equal(got, FusedLlamaDecoderLayer(model)(*inputs)), "compiled graph and assembled op sequence must agree bitwise"
    _end_to_end_gate(got, want, exact, "compiled llama layer 1x2048x4096 bf16")


def test_encoder_block_compiled_on_gpu(cuda_device):
    from xpu_graph_b200.workloads import make_encoder

    model, x = make_encoder(seed=0)
    with torch.no_grad():
        want = model(x)
    compiled, got, mods, atens = _compile_run(model.to(cuda_device), (x.to(cuda_device),))
    assert_parity(got, want, "compiled encoder block")
    assert mods.count("xg_layer_norm") == 2 and "xg_sdpa" in mods and mods.count("xg_dense_residual") == 2, mods


def test_recsys_graph_compiled_on_gpu(cuda_device):
    from xpu_graph_b200.workloads import make_recsys

    model, (dense, idx, mask) = make_recsys(seed=4, batch=2048, table_rows=5000)
    with torch.no_grad():
        want = model(dense, idx, mask)
    compiled, got, mods, atens = _compile_run(model.to(cuda_device), (dense.to(cuda_device), idx.to(cuda_device), mask.to(cuda_device)))
    assert_parity(got, want, "compiled recsys graph")
    assert mods == ["xg_gather_stack", "fuse_slice_cat", "xg_cat_lastdim", "custom_dense_layer_replacement",
                    "custom_dense_layer_replacement", "custom_dense_layer_replacement"], mods


def test_recsys_graph_full_size_compiled_on_gpu(cuda_device):
    """At the benchmark's batch of 16384 the three dense layers collapse into one dense-tower call."""
    from xpu_graph_b200.workloads import make_recsys

    model, (dense, idx, mask) = make_recsys(seed=4)
    with torch.no_grad():
        want = model(dense, idx, mask)
    compiled, got, mods, atens = _compile_run(model.to(cuda_device), (dense.to(cuda_device), idx.to(cuda_device), mask.to(cuda_device)))
    assert_parity(got, want, "compiled recsys graph, full size")
    assert mods == ["xg_gather_stack", "fuse_slice_cat", "xg_cat_lastdim", "xg_dense_tower"], mods


def test_device_graph_vendor_compiler(cuda_device):
    """vendor_compiler_config={"compiler": "device_graph"}: the rewritten encoder graph goes through the reference's
    device_graph_compiler (backends/device_graph.py:54-130) with this target's GraphRunner subclass, is captured into
    one CUDA graph and replayed; results stay equal to eager on new inputs and replay is faster than launch by
    launch (the protocol of the reference's tests/mlu/test_mlu_graph.py:31-117)."""
    from xpu_graph_b200.workloads import make_encoder

    model, x = make_encoder(seed=0)
    cpu_model, _ = make_encoder(seed=0)
    model = model.to(cuda_device)
    compiled, got, mods, atens = _compile_run(model, (x.to(cuda_device),), vendor_compiler_config={"compiler": "device_graph"})
    # the reference's capability partitioner ran: what is left at the top level are its fused partitions, each a lazily
    # captured GraphRunner[Target.cuda] (every node of this graph lives on the device, so there is exactly one)
    assert mods == ["fused_0"], mods
    with torch.no_grad():
        assert_parity(got, cpu_model(x), "device_graph first call")
        g = torch.Generator().manual_seed(123)
        for _ in range(2):
            x2 = torch.randn(x.shape, generator=g)
            assert_parity(compiled(x2.to(cuda_device)), cpu_model(x2), "device_graph replay")
        plain, *_ = _compile_run(model, (x.to(cuda_device),))
        xd = x.to(cuda_device)

        def clock(fn):
            for _ in range(5):
                fn(xd)
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            for _ in range(50):
                fn(xd)
            torch.cuda.synchronize()
            return (time.perf_counter() - t0) / 50

        t_graph, t_plain = clock(compiled), clock(plain)
    print(f"encoder block: captured {t_graph * 1e6:.0f} us, launch-by-launch {t_plain * 1e6:.0f} us per call")
    assert t_graph < t_plain


def test_interceptor_on_gpu(cuda_device, caplog):
    """enable_interceptor="rtol=...,atol=...": the reference's interceptor (interceptor.py:93-179) runs the Dynamo graph
    (eager CUDA aten) beside the graph compiled for this target on every call; with the kernels in order it stays silent."""
    from xpu_graph_b200.workloads import make_encoder, make_llama_layer

    lg = logging.getLogger("xpu_graph")
    old = lg.propagate
    lg.propagate = True
    caplog.set_level(logging.INFO, logger="xpu_graph")
    try:
        model, x = make_encoder(seed=0)
        model = model.to(cuda_device)
        compiled, got, mods, atens = _compile_run(model, (x.to(cuda_device),), enable_interceptor="rtol=1e-4,atol=1e-5")
        layer, (lx, cos, sin) = make_llama_layer(seed=3, batch=1, seq=256, hidden=512, heads=4, ffn=1376)
        layer = layer.to(cuda_device)
        _compile_run(layer, (lx.to(cuda_device), cos.to(cuda_device), sin.to(cuda_device)), enable_interceptor="rtol=2e-2,atol=2e-2")
    finally:
        lg.propagate = old
    assert caplog.text.count("Monitored inference") >= 2
    assert "diverges" not in caplog.text, caplog.text[-2000:]


def test_reference_front_end_on_gpu(cuda_device):
    """torch.compile(model, backend=XpuGraph(config)) - the reference's own entry point (compiler.py:196-237, graph
    dispatch by fx_utils.dispatch_graph) - with this target: the same kernels run (same launch sequence as through
    target.backend()) and the results are bit-equal."""
    from tests.helpers import LaunchCounter
    from xpu_graph_b200 import lib, target
    from xpu_graph_b200.workloads import make_llama_layer, make_recsys

    layer, (x, cos, sin) = make_llama_layer(seed=3, batch=2, seq=320, hidden=512, heads=4, ffn=1376)
    layer = layer.to(cuda_device)
    cases = [(layer, (x.to(cuda_device), cos.to(cuda_device), sin.to(cuda_device)))]
    model, inputs = make_recsys(seed=5, batch=512)
    cases.append((model.to(cuda_device), tuple(t.to(cuda_device) for t in inputs)))
    for model, inputs in cases:
        through_backend, want, _, _ = _compile_run(model, inputs)
        with LaunchCounter() as ours:
            with torch.no_grad():
                through_backend(*inputs)
        torch._dynamo.reset()
        compiled = torch.compile(model, backend=target.reference_backend(), dynamic=False)
        with torch.no_grad():
            compiled(*inputs)  # compiles
            with LaunchCounter() as theirs:
                got = compiled(*inputs)
        torch.cuda.synchronize()
        assert lib.tc_status() == 0
        outs_w = want if isinstance(want, (tuple, list)) else (want,)
        outs_g = got if isinstance(got, (tuple, list)) else (got,)
        for a, b in zip(outs_g, outs_w):
            assert torch.equal(a, b)
        assert theirs.names and theirs.names == ours.names, (theirs.names, ours.names)


def test_decomposed_attention_on_gpu(cuda_device):
    """The decomposed attention graph of the reference's tests (tests/common/test_fuse_sdpa.py:14-25, fp16, 32 heads,
    S = 38, E = 64, and a tensor-core shape) compiled for this target: one attention launch, no operand copies."""
    import math

    from oracle import ref_ops
    from tests.helpers import LaunchCounter

    def fn(query, key, value):
        return torch.matmul(query, key.transpose(-2, -1)).div(math.sqrt(query.shape[-1])).softmax(dim=-1).matmul(value)

    for B, H, S, E in ((2, 32, 38, 64), (2, 8, 256, 128)):
        g = torch.Generator().manual_seed(14)
        q, k, v = (torch.randn(B, H, S, E, generator=g).to(torch.float16) for _ in range(3))
        compiled, got, mods, atens = _compile_run(fn, (q.to(cuda_device), k.to(cuda_device), v.to(cuda_device)))
        assert mods == ["xg_sdpa"] and not any("clone" in a for a in atens), (mods, atens)
        with LaunchCounter() as c:
            with torch.no_grad():
                got = compiled(q.to(cuda_device), k.to(cuda_device), v.to(cuda_device))
        torch.cuda.synchronize()
        assert c.names == ["xg_sdpa_fwd"], c.names
        assert_parity(got, ref_ops.sdpa(q, k, v, None, None, False), f"decomposed attention {B}x{H}x{S}x{E}")
        torch._dynamo.reset()



def test_combo_matmul_forms_on_gpu(cuda_device):
    """The reference's combo test at its own dtype and sizes (tests/mlu/test_combo_matmul.py:33-39, 57-79, 90-100: fp32,
    eight 5 x 8 x 7 layers with full-matrix addends over one shared input, and relu(F.linear(x_i, w_i.T)) over eight
    split inputs) compiled for this target: one grouped launch each, compared with fp64 math."""
    from tests.helpers import LaunchCounter

    T, M, K, N = 8, 5, 8, 7
    g = torch.Generator().manual_seed(15)
    shared, split = torch.randn(1, M, K, generator=g), torch.randn(T, M, K, generator=g)
    ws = [torch.randn(K, N, generator=g) for _ in range(T)]
    mats = [torch.randn(M, N, generator=g) for _ in range(T)]

    def shared_bias_relu(x, *wb):
        x = x.squeeze(0)
        return tuple(torch.relu(x @ wi + bi) for wi, bi in zip(wb[:T], wb[T:]))

    def split_linear_t(x, *w):
        xs = [i.squeeze(0) for i in x.split(x.shape[0] // T, dim=0)]
        return tuple(torch.relu(torch.nn.functional.linear(xi, wi.T)) for xi, wi in zip(xs, w))

    for fn, args in ((shared_bias_relu, (shared, *ws, *mats)), (split_linear_t, (split, *ws))):
        dev_args = tuple(a.to(cuda_device) for a in args)
        compiled, got, mods, atens = _compile_run(fn, dev_args)
        assert mods.count("xg_combo_dense") == 1 and "custom_dense_layer_replacement" not in mods, mods
        with LaunchCounter() as c:
            with torch.no_grad():
                got = compiled(*dev_args)
        torch.cuda.synchronize()
        assert c.names == ["xg_gemm_group_bias_act"], c.names
        want = fn(*(a.double() for a in args))
        for o, w in zip(got, want):
            assert_parity(o, w.float(), f"combo {fn.__name__}")
        torch._dynamo.reset()


def test_dynamic_batch_on_gpu(cuda_device):
    """One compilation with a symbolic batch dimension (mark_dynamic) serves several batch sizes on the GPU: the grouped
    launch, the narrow tower and the residual-add LayerNorm run with the actual row count of each call."""
    from tests.helpers import LaunchCounter
    from xpu_graph_b200 import target

    torch.manual_seed(16)

    class Towers(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.layers = torch.nn.ModuleList(torch.nn.Linear(64, 48) for _ in range(5))
            self.chain = torch.nn.Sequential(torch.nn.Linear(20, 32), torch.nn.ReLU(), torch.nn.Linear(32, 16), torch.nn.ReLU(),
                                             torch.nn.Linear(16, 1))
            self.ln = torch.nn.LayerNorm(64)

        def forward(self, x, z, r):
            return tuple(torch.relu(layer(x)) for layer in self.layers) + (self.chain(z), self.ln(x + r))

    model = Towers().eval().to(cuda_device)
    compiled = torch.compile(model, backend=target.backend(target.make_config()), dynamic=None)
    for m in (6, 50, 300):
        args = (torch.randn(m, 64, device=cuda_device), torch.randn(m, 20, device=cuda_device), torch.randn(m, 64, device=cuda_device))
        for a in args:
            torch._dynamo.mark_dynamic(a, 0)
        with torch.no_grad():
            with LaunchCounter() as c:
                got = compiled(*args)
            want = model.double()(*(a.double() for a in args))
            model.float()
        torch.cuda.synchronize()
        assert sorted(c.names) == sorted(["xg_gemm_group_bias_act", "xg_mlp_small_bias_act", "xg_layernorm"]), c.names
        for o, w in zip(got, want):
            assert_parity(o, w.float(), f"dynamic batch {m}")


def test_dynamic_batch_recsys_graph_on_gpu(cuda_device):
    """The recsys graph compiled once with a symbolic batch dimension and run at two batch sizes on the GPU: lookups +
    mask + stack, slice-cat, the concatenation and the dense layers run fused, results equal eager CUDA."""
    from tests.helpers import LaunchCounter
    from xpu_graph_b200 import target
    from xpu_graph_b200.workloads import make_recsys

    model = None
    compiled = None
    for batch in (512, 1536):
        m, inputs = make_recsys(seed=5, batch=batch)
        if model is None:
            model = m.to(cuda_device)
            compiled = torch.compile(model, backend=target.backend(target.make_config()), dynamic=None)
        args = tuple(t.to(cuda_device) for t in inputs)
        for a in args:
            torch._dynamo.mark_dynamic(a, 0)
        with torch.no_grad():
            with LaunchCounter() as c:
                got = compiled(*args)
            want = model(*args)
        torch.cuda.synchronize()
        assert "xg_gather_rows" in c.names and "xg_seg_copy" in c.names, c.names
        assert_parity(got, want, f"recsys graph, dynamic batch {batch}")


def test_dynamic_batch_llama_layer_on_gpu(cuda_device):
    """The Llama-style layer (bf16, reduced size) compiled once with a symbolic batch dimension and run at two batch
    sizes: the nine launches of the static graph (RoPE in the q / k projections' epilogues, the residual adds in theirs,
    the dual GEMM with SwiGLU), results within the 16-bit bar of eager CUDA."""
    from tests.helpers import LaunchCounter
    from xpu_graph_b200 import lib, target
    from xpu_graph_b200.workloads import make_llama_layer

    layer, (x, cos, sin) = make_llama_layer(seed=3, batch=2, seq=320, hidden=512, heads=4, ffn=1376)
    layer = layer.to(cuda_device)
    cos, sin = cos.to(cuda_device), sin.to(cuda_device)
    compiled = torch.compile(layer, backend=target.backend(target.make_config()), dynamic=None)
    g = torch.Generator().manual_seed(17)
    for batch in (2, 5):
        xb = torch.randn(batch, 320, 512, generator=g).to(torch.bfloat16).to(cuda_device)
        torch._dynamo.mark_dynamic(xb, 0)
        with torch.no_grad():
            with LaunchCounter() as c:
                got = compiled(xb, cos, sin)
            want = layer(xb, cos, sin)
        torch.cuda.synchronize()
        assert lib.tc_status() == 0
        assert len(c.names) == 9 and c.names.count("xg_gemm_rope") == 2 and "xg_gemm_swiglu" in c.names, c.names
        assert_parity(got, want, f"Llama layer, dynamic batch {batch}", magnitude=xb)


def test_dynamic_batch_row_sums_on_gpu(cuda_device):
    """slice -> sum -> cat and sum -> cat compiled once with a symbolic batch dimension, run at three batch sizes on the GPU."""
    from tests.helpers import LaunchCounter
    from xpu_graph_b200 import target

    def fn(x, y0, y1, y2):
        s = torch.cat([x[:, 0:10, :].sum(dim=1), x[:, 0:25, :].sum(dim=1), x[:, 8:40, :].sum(dim=1)], dim=-1)
        t = torch.cat([y0.sum(dim=1), y1.sum(dim=1), y2.sum(dim=1)], dim=-1)
        return s, t

    compiled = torch.compile(fn, backend=target.backend(target.make_config()), dynamic=None)
    g = torch.Generator().manual_seed(18)
    for b in (6, 200, 33):
        args = tuple(torch.randn(b, r, c, generator=g).to(cuda_device) for r, c in ((40, 16), (3, 8), (7, 8), (4, 8)))
        for a in args:
            torch._dynamo.mark_dynamic(a, 0)
        with torch.no_grad():
            with LaunchCounter() as c:
                got = compiled(*args)
            want = fn(*(a.double() for a in args))
        torch.cuda.synchronize()
        assert c.names == ["xg_rowsum_cat", "xg_rowsum_cat"], c.names
        for o, w in zip(got, want):
            assert_parity(o, w.float(), f"row sums, dynamic batch {b}")
