"""The cuda_sm100 target inside the xpu_graph pass pipeline (host side, CPU graphs).

Style follows the reference's pattern tests (e.g. tests/common/test_fuse_layernorm.py:58-134,
tests/mlu/test_custom_denselayer.py:109-179): compile a small eager function through
``torch.compile(backend=XpuGraph-based)``, compare with eager, and assert on the
"Pattern.<Class> changed graph" log lines. The fused ops run on CPU through test doubles
(tests/cpu_doubles.py), so this checks the graph rewrites, not the kernels.

Skipped when the xpu_graph package is not importable.
"""
import logging

import pytest
import torch
import torch.nn.functional as F

from xpu_graph_b200.target.compat import reference_available

pytestmark = pytest.mark.skipif(not reference_available(), reason="xpu_graph reference package not importable")

MAX_INT64 = 9223372036854775807


@pytest.fixture(autouse=True)
def _reset_dynamo():
    torch._dynamo.reset()
    yield
    torch._dynamo.reset()


@pytest.fixture(scope="module")
def tgt():
    from tests import cpu_doubles

    cpu_doubles.register()
    from xpu_graph_b200 import target

    target.install()
    return target


def _compile(tgt, fn, *inputs, **cfg):
    cap = {}
    be = tgt.backend(tgt.make_config(debug=True, **cfg), capture=cap)
    with torch.no_grad():
        want = fn(*inputs)
        got = torch.compile(fn, backend=be, dynamic=False)(*inputs)
    mods = [n.target for n in cap["gm"].graph.nodes if n.op == "call_module"]
    atens = [str(n.target) for n in cap["gm"].graph.nodes if n.op == "call_function"]
    return want, got, mods, atens


@pytest.fixture()
def xlog(caplog):
    lg = logging.getLogger("xpu_graph")
    old = lg.propagate
    lg.propagate = True
    caplog.set_level(logging.DEBUG, logger="xpu_graph")
    yield caplog
    lg.propagate = old


def _same(a, b, tol=1e-5):
    assert a.shape == b.shape and a.dtype == b.dtype
    scale = max(b.float().abs().max().item(), 1e-6)
    assert (a.float() - b.float()).abs().max().item() <= tol * scale


def test_target_is_installed(tgt):
    from xpu_graph.config import Target
    from xpu_graph.passes.patterns.targets import get_all_patterns, get_structure_replacements

    assert Target.cuda_sm100.value == "cuda_sm100" and Target("cuda_sm100") is Target.cuda_sm100
    cfg = tgt.make_config()
    reps = get_structure_replacements(cfg)
    for name in ("CustomRMSNorm", "CustomLayerNorm", "CustomDenseLayer", "CustomBatchDenseLayer", "FusedSlice",
                 "FusedCatSlice", "FusedSliceStackSum", "FusedMultipleSliceCat"):
        assert name in reps and "target_mod" in reps[name]
    pats = get_all_patterns(cfg)
    names = {type(p).__name__ for group in pats.values() for p in group}
    assert {"FusedNativeLayerNorm", "FusedSdpa", "FusedRoPE", "FusedSwiGLU", "FusedDenseResidual", "FusedAddNorm",
            "FusedEmbeddingStack", "FusedCatLastDim"} <= names
    # skip_patterns is honoured through Pattern.filter
    pats = get_all_patterns(tgt.make_config(skip_patterns=["FusedRoPE"]))
    assert "FusedRoPE" not in {type(p).__name__ for group in pats.values() for p in group}


def test_graph_runner_is_registered_for_the_target(tgt):
    """GraphRunner[Target.cuda_sm100] (device_graph_runner.py:146-191 shows the NPU / MLU registrations) resolves to the
    CUDA subclass, also under the device-type alias that backends/device_graph.py:72 looks it up by; the vendor
    compiler hook is published where backends/__init__.py:19-25 imports it from."""
    import importlib

    from xpu_graph.config import Target
    from xpu_graph.device_graph_runner import GraphRunner
    from xpu_graph_b200.graph_runner import CUDAGraphRunner

    assert GraphRunner[Target.cuda_sm100] is CUDAGraphRunner and GraphRunner[Target("cuda")] is CUDAGraphRunner
    assert issubclass(CUDAGraphRunner, GraphRunner)
    runner = CUDAGraphRunner(lambda x: x + 1)
    assert runner.captured is False and type(runner.clone()) is CUDAGraphRunner
    hook = importlib.import_module("xpu_graph.backends.cuda_sm100").cuda_sm100_compile
    gm = torch.fx.symbolic_trace(torch.nn.Linear(4, 4))
    assert hook(gm, [torch.empty(2, 4)], is_inference=True) is gm                           # no capture asked for
    assert hook(gm, [torch.empty(2, 4)], is_inference=True, compiler="device_graph") is gm  # host tensors: nothing to capture


def test_llama_layer_graph(tgt, xlog):
    from xpu_graph_b200.workloads import make_llama_layer

    m, inp = make_llama_layer(seed=3, batch=2, seq=32, hidden=256, heads=2, ffn=384)
    want, got, mods, atens = _compile(tgt, m, *inp)
    _same(got, want, 1e-2)
    assert sorted(mods) == sorted(["custom_rms_norm", "xg_dense_rope", "xg_dense_rope", "custom_dense_layer_replacement",
                                   "xg_sdpa", "xg_dense_residual", "custom_rms_norm", "xg_dense_swiglu", "xg_dense_residual"])
    assert mods[0] == "custom_rms_norm" and mods[-1] == "xg_dense_residual" and mods.index("xg_sdpa") == 4
    assert all(("reshape" in a or "transpose" in a) for a in atens), atens  # only views are left
    for cls in ("CustomRMSNorm", "CustomDenseLayer", "FusedRoPE", "FusedDenseRope", "FusedSdpa", "FusedSwiGLU",
                "FusedDenseResidual"):
        assert f"Pattern.{cls} changed graph" in xlog.text


def test_encoder_block_graph(tgt, xlog):
    from xpu_graph_b200.workloads import make_encoder

    m, x = make_encoder(seed=0, batch=2, seq=16, hidden=64, heads=4, ffn=128)
    want, got, mods, atens = _compile(tgt, m, x)
    _same(got, want)
    assert mods == ["xg_layer_norm", "custom_dense_layer_replacement", "xg_sdpa", "xg_dense_residual", "xg_layer_norm",
                    "custom_dense_layer_replacement", "xg_dense_residual"]
    for cls in ("FusedNativeLayerNorm", "CustomDenseLayer", "FusedSdpa", "FusedDenseResidual"):
        assert f"Pattern.{cls} changed graph" in xlog.text


def test_recsys_graph(tgt, xlog):
    from xpu_graph_b200.workloads import make_recsys

    m, inp = make_recsys(seed=4, batch=32, table_rows=50)
    want, got, mods, atens = _compile(tgt, m, *inp)
    _same(got, want)
    assert mods == ["xg_gather_stack", "fuse_slice_cat", "xg_cat_lastdim", "custom_dense_layer_replacement",
                    "custom_dense_layer_replacement", "custom_dense_layer_replacement"]
    assert not any("embedding" in a or "where" in a or "slice" in a for a in atens)
    for cls in ("FusedEmbeddingStack", "FusedCatSlice", "FusedCatLastDim", "CustomDenseLayer"):
        assert f"Pattern.{cls} changed graph" in xlog.text


@pytest.mark.parametrize("reuse_sum", [False, True])
@pytest.mark.parametrize("kind", ["rms", "ln"])
def test_add_norm(tgt, xlog, kind, reuse_sum):
    g = torch.Generator().manual_seed(0)
    x, r = torch.randn(6, 64, generator=g), torch.randn(6, 64, generator=g)
    w, b = torch.randn(64, generator=g), torch.randn(64, generator=g)

    def fn(x, r, w, b):
        s = x + r
        if kind == "rms":
            y = s * torch.rsqrt(s.pow(2).mean(-1, keepdim=True) + 1e-6) * w
        else:
            y = F.layer_norm(s, s.shape[-1:], w, b, 1e-5)
        return (y, s * 2.0) if reuse_sum else y

    want, got, mods, atens = _compile(tgt, fn, x, r, w, b)
    if reuse_sum:
        _same(got[0], want[0])
        _same(got[1], want[1])
    else:
        _same(got, want)
    expect = {("rms", False): "xg_add_rms_norm_y", ("rms", True): "xg_add_rms_norm", ("ln", False): "xg_add_layer_norm_y",
              ("ln", True): "xg_add_layer_norm"}[(kind, reuse_sum)]
    assert mods == [expect], mods
    assert "Pattern.FusedAddNorm changed graph" in xlog.text
    assert not any("add.Tensor" in a for a in atens)


@pytest.mark.parametrize("kind", ["rms", "ln"])
def test_add_norm_with_an_earlier_user_of_the_sum(tgt, xlog, kind):
    """A consumer of the sum that sits before the norm in the graph must still find its operand defined: the fused
    call (whose second output replaces the sum) then takes the add's place instead of the norm's."""
    g = torch.Generator().manual_seed(0)
    x, r = torch.randn(6, 64, generator=g), torch.randn(6, 64, generator=g)
    w, b = torch.randn(64, generator=g), torch.randn(64, generator=g)

    def fn(x, r, w, b):
        s = x + r
        early = s * 2.0  # defined before the norm chain
        if kind == "rms":
            y = s * torch.rsqrt(s.pow(2).mean(-1, keepdim=True) + 1e-6) * w
        else:
            y = F.layer_norm(s, s.shape[-1:], w, b, 1e-5)
        return y, early

    want, got, mods, atens = _compile(tgt, fn, x, r, w, b)
    _same(got[0], want[0])
    _same(got[1], want[1])
    assert mods == ["xg_add_rms_norm" if kind == "rms" else "xg_add_layer_norm"], mods
    assert not any("add.Tensor" in a for a in atens)


def test_add_norm_keeps_the_add_when_the_fused_call_cannot_move():
    """Hand-built graph: the sum has a user before the norm AND the norm's weight is defined after the add, so the
    fused call can neither stay at the norm (its second output would be used before it exists) nor move to the add.
    The pattern then fuses without the second output and leaves the add in place; the graph must lint."""
    from torch import fx

    from xpu_graph_b200 import modules as M
    from xpu_graph_b200.target.patterns import FusedAddNorm

    graph = fx.Graph()
    a, b = graph.placeholder("a"), graph.placeholder("b")
    add = graph.call_function(torch.ops.aten.add.Tensor, (a, b))
    early = graph.call_function(torch.ops.aten.mul.Tensor, (add, 2.0))
    w = graph.placeholder("w")  # placeholders normally lead the graph; any late-defined operand behaves like this one
    norm = graph.call_module("custom_rms_norm", (add, w, 1e-6))
    graph.output((norm, early))
    root = torch.nn.Module()
    root.add_module("custom_rms_norm", M.RMSNormModule())
    gm = fx.GraphModule(root, graph)
    t = torch.empty(4, 8)
    for n, v in ((a, t), (b, t), (add, t), (early, t), (w, torch.empty(8)), (norm, t)):
        n.meta["val"] = v
    M.ALLOWED_DEVICE_TYPES.add("cpu")
    assert FusedAddNorm().process(gm) is True
    gm.graph.lint()
    mods = [n.target for n in gm.graph.nodes if n.op == "call_module"]
    assert mods == ["xg_add_rms_norm_y"]
    assert any(n.op == "call_function" and n.target is torch.ops.aten.add.Tensor for n in gm.graph.nodes)


def test_rope_with_tables_of_another_dtype_is_left_alone(tgt):
    """bf16 x with fp32 cos / sin: eager promotes the result to fp32; the kernel would return bf16 and round the
    tables, so the chain must stay as it is."""
    from xpu_graph_b200.workloads import rotate_half

    g = torch.Generator().manual_seed(5)
    x = torch.randn(2, 3, 10, 16, generator=g).to(torch.bfloat16)
    c, s = torch.randn(10, 16, generator=g), torch.randn(10, 16, generator=g)
    want, got, mods, atens = _compile(tgt, lambda x, c, s: x * c + rotate_half(x) * s, x, c, s)
    assert got.dtype == torch.float32 == want.dtype
    _same(got, want)
    assert "xg_rope" not in mods


@pytest.mark.parametrize("act", ["none", "gelu", "relu", "silu"])
@pytest.mark.parametrize("bias", [False, True])
def test_dense_layer(tgt, xlog, act, bias):
    g = torch.Generator().manual_seed(1)
    x, w, b = torch.randn(10, 24, generator=g), torch.randn(40, 24, generator=g), torch.randn(40, generator=g)
    f = {"none": lambda t: t, "gelu": F.gelu, "relu": F.relu, "silu": F.silu}[act]
    fn = (lambda x, w, b: f(F.linear(x, w, b))) if bias else (lambda x, w, b: f(F.linear(x, w)))
    want, got, mods, atens = _compile(tgt, fn, x, w, b)
    _same(got, want)
    assert mods == ["custom_dense_layer_replacement"]
    assert "Pattern.CustomDenseLayer changed graph" in xlog.text


def test_bf16_dense_with_rows_no_tensor_map_addresses(tgt):
    """bf16 x @ W with rows that are not multiples of 16 bytes has no tensor-core kernel; the dense layer is fused all
    the same (the library runs such shapes on its FMA kernel), as are aligned [K, N] weights."""
    g = torch.Generator().manual_seed(2)
    x = torch.randn(8, 16, generator=g).to(torch.bfloat16)
    for n in (20, 24):
        w = torch.randn(16, n, generator=g).to(torch.bfloat16)
        want, got, mods, atens = _compile(tgt, lambda x, w: F.relu(x @ w), x, w)
        _same(got, want, 3e-2)
        assert mods == ["custom_dense_layer_replacement"] and not any("mm" in a for a in atens), (n, mods, atens)
        torch._dynamo.reset()


def test_decomposed_attention_goes_through_fused_sdpa(tgt, xlog):
    g = torch.Generator().manual_seed(3)
    q, k, v = (torch.randn(4, 20, 32, generator=g) for _ in range(3))

    def fn(q, k, v):
        s = torch.bmm(q, k.transpose(1, 2)) * 0.25
        return torch.bmm(torch.softmax(s, dim=-1), v)

    want, got, mods, atens = _compile(tgt, fn, q, k, v)
    _same(got, want)
    assert "xg_sdpa" in mods
    assert "Pattern.FusedSDPA changed graph" in xlog.text and "Pattern.FusedSdpa changed graph" in xlog.text


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("form", ["functional", "module", "residual"])
def test_rms_norm_as_lowered_from_torch(tgt, xlog, dtype, form):
    """F.rms_norm / nn.RMSNorm reach the compiler as a pow-mean-add.Scalar-rsqrt chain (with an fp32 detour for 16-bit
    inputs), which the reference's FusedRMSNorm does not match (check_ops.py:88-89 wants add.Tensor): the target's own
    matcher turns it into the fused norm, and a preceding residual add is folded in as for the hand-written form."""
    g = torch.Generator().manual_seed(11)
    x, r = torch.randn(6, 64, generator=g).to(dtype), torch.randn(6, 64, generator=g).to(dtype)
    if form == "module":
        m = torch.nn.RMSNorm(64, eps=1e-6).to(dtype)
        with torch.no_grad():
            m.weight.copy_(torch.randn(64, generator=g))
        want, got, mods, atens = _compile(tgt, m, x)
        expect = ["xg_rms_norm"]
    else:
        w = torch.randn(64, generator=g).to(dtype)
        if form == "functional":
            want, got, mods, atens = _compile(tgt, lambda x, w: F.rms_norm(x, (64,), w, 1e-6), x, w)
            expect = ["xg_rms_norm"]
        else:
            want, got, mods, atens = _compile(tgt, lambda x, r, w: F.rms_norm(x + r, (64,), w, 1e-6), x, r, w)
            expect = ["xg_add_rms_norm_y"]
    _same(got, want, 1e-5 if dtype == torch.float32 else 1e-2)
    assert mods == expect, mods
    assert "Pattern.FusedRmsNormLowered changed graph" in xlog.text
    assert not any("rsqrt" in a or "pow" in a or "mean" in a for a in atens), atens


def test_attention_with_a_tensor_scale(tgt, xlog):
    """A tensor-valued softmax scale: the reference's FusedSDPA wraps it (SDPAWrappedScale,
    default_replacements.py:39-55) instead of emitting the aten call; the target folds the scale into q and runs the
    fused attention with scale 1."""
    g = torch.Generator().manual_seed(3)
    q, k, v = (torch.randn(4, 20, 32, generator=g) for _ in range(3))
    scale = torch.tensor(0.3)

    def fn(q, k, v, scale):
        s = torch.bmm(q, k.transpose(1, 2)) * scale
        return torch.bmm(torch.softmax(s, dim=-1), v)

    want, got, mods, atens = _compile(tgt, fn, q, k, v, scale)
    _same(got, want)
    assert mods == ["xg_sdpa"], mods
    assert "Pattern.FusedSDPA changed graph" in xlog.text and "Pattern.FusedSdpaTensorScale changed graph" in xlog.text


def test_single_row_gathers(tgt, xlog):
    """table[idx] in its three graph forms (embedding, advanced indexing on dim 0, index_select) -> the gather kernel;
    negative indices of the indexing forms count from the end as in eager."""
    g = torch.Generator().manual_seed(6)
    table = torch.randn(50, 16, generator=g)
    idx = torch.randint(0, 50, (7, 3), generator=g)
    neg = torch.tensor([0, -1, 49, -50, 3])

    def fn(table, idx, neg):
        return F.embedding(idx, table) * 2.0, table[neg] + 1.0, torch.index_select(table, 0, idx[:, 0]) - 1.0

    want, got, mods, atens = _compile(tgt, fn, table, idx, neg)
    for a, b in zip(got, want):
        _same(a, b)
    assert sorted(mods) == ["xg_row_gather", "xg_row_gather", "xg_row_gather_wrap"], mods
    assert "Pattern.FusedRowGather changed graph" in xlog.text
    assert not any("embedding" in a or "index" in a for a in atens), atens


def test_gather_with_a_repeated_index_uses_expand(tgt, xlog):
    """gather(x, 1, idx.unsqueeze(-1).repeat(1, 1, C)): the repeat becomes an expand
    (targets/mlu/repeat_to_expand.py:25-56 does the same for the MLU target)."""
    g = torch.Generator().manual_seed(7)
    x = torch.randn(4, 9, 8, generator=g)
    idx = torch.randint(0, 9, (4, 5), generator=g)
    want, got, mods, atens = _compile(tgt, lambda x, idx: torch.gather(x, 1, idx.unsqueeze(-1).repeat(1, 1, 8)) * 1.0, x, idx)
    assert torch.equal(got, want)
    assert "Pattern.GatherIndexRepeatToExpand changed graph" in xlog.text
    assert not any("repeat" in a for a in atens) and any("expand" in a for a in atens), atens


def test_masked_slice_cat(tgt, xlog):
    """cat of where(mask, 0, slice) over one source: the common passes merge the per-slice where nodes, FusedCatSlice
    fuses the slices, and the target folds the remaining where into the copy (MaskedSliceCatModule)."""
    g = torch.Generator().manual_seed(8)
    src = torch.randn(12, 200, generator=g)
    mask = torch.rand(12, 1, generator=g) < 0.4

    def fn(src, mask):
        parts = [src[:, 0:32], src[:, 64:96], src[:, 100:132], src[:, 10:42]]
        zero = torch.zeros_like(parts[0])
        return torch.cat([torch.where(mask, zero, p) for p in parts], dim=-1)

    want, got, mods, atens = _compile(tgt, fn, src, mask)
    assert torch.equal(got, want)
    assert mods == ["xg_masked_slice_cat"], (mods, atens)
    assert not any("where" in a or "slice" in a for a in atens), atens


def test_masked_slice_cat_reference_test_forms(tgt, xlog):
    """The two graphs of the reference's own test (tests/mlu/test_fuse_slice_where_cat.py:19-76, fp16, a 35149-wide
    source): an unmasked slice followed by where-masked slices, concatenated along the last dim or stacked along a new
    leading one, the unmasked slice being a second output. Each becomes one module call; the plain slice stays a view."""
    g = torch.Generator().manual_seed(9)
    B = 96
    src = torch.randn(B, 35149, generator=g).to(torch.float16)
    mask = (torch.rand(B, generator=g) < 0.5).unsqueeze(-1)

    def cat_form(mask, src):
        zeros = torch.zeros([B, 32], dtype=torch.float16)
        first = src[:, 0:32]
        rest = [src[:, a:a + 32] for a in (10118, 10579, 11032, 11445)]
        return torch.cat([first] + [torch.where(mask, zeros, r) for r in rest], dim=-1), first

    def stack_form(mask, src):
        zeros = torch.zeros([B, 4], dtype=torch.float16)
        first = src[:, 0:4]
        rest = [src[:, a:a + 4] for a in (11984, 11562, 9782, 9727, 9745, 9763, 9773, 9805, 9822, 10283, 10736)]
        return torch.stack([first] + [torch.where(mask, zeros, r) for r in rest], dim=0), first

    for fn, module in ((cat_form, "xg_masked_slice_cat"), (stack_form, "xg_masked_slice_stack")):
        want, got, mods, atens = _compile(tgt, fn, mask, src)
        assert torch.equal(got[0], want[0]) and torch.equal(got[1], want[1])
        assert mods == [module], (mods, atens)
        assert not any("where" in a or "unbind" in a or "transpose" in a for a in atens), atens
        torch._dynamo.reset()


def test_slice_fusions_use_target_modules(tgt, xlog):
    g = torch.Generator().manual_seed(4)
    src = torch.randn(12, 200, generator=g)

    def cat_fn(s):
        return torch.cat([s[:, 0:32], s[:, 64:96], s[:, 100:MAX_INT64], s[:, 10:-150]], dim=-1) * 2.0

    want, got, mods, atens = _compile(tgt, cat_fn, src)
    assert torch.equal(got, want)
    assert mods == ["fuse_slice_cat"]
    assert "Pattern.FusedCatSlice changed graph" in xlog.text

    def slice_fn(s):
        a, b, c, d = s[:, 0:16], s[:, 40:56], s[:, 100:116], s[:, 7:23]
        return a * 1.0 + b * 2.0 + c * 3.0 + d * 4.0

    torch._dynamo.reset()
    want, got, mods, atens = _compile(tgt, slice_fn, src)
    _same(got, want)
    assert any(m.startswith("fused_triton_slice") for m in mods)
    assert "Pattern.FusedSlice changed graph" in xlog.text


def test_rope_and_swiglu_standalone(tgt, xlog):
    from xpu_graph_b200.workloads import rotate_half

    g = torch.Generator().manual_seed(5)
    x, c, s = torch.randn(2, 3, 10, 16, generator=g), torch.randn(10, 16, generator=g), torch.randn(10, 16, generator=g)
    want, got, mods, atens = _compile(tgt, lambda x, c, s: x * c + rotate_half(x) * s, x, c, s)
    _same(got, want)
    assert mods == ["xg_rope"] and not any("cat" in a or "neg" in a for a in atens)
    torch._dynamo.reset()
    a, b = torch.randn(7, 48, generator=g), torch.randn(7, 48, generator=g)
    want, got, mods, atens = _compile(tgt, lambda a, b: F.silu(a) * b, a, b)
    _same(got, want)
    assert mods == ["xg_swiglu"]


def test_replacement_modules_are_picklable(tgt):
    """The compile cache pickles graphs with their sub-modules (cache.py:113-179)."""
    import pickle

    from xpu_graph_b200 import modules as M

    for mod in (M.RMSNormModule(), M.LayerNormModule(), M.DenseLayerModule(False), M.FuseSliceModule([0, 4, 8]),
                M.FuseSliceCatSameInputModule(), M.FuseSliceCatSameInputModule_v2([[(0, 2)], [(2, 4), (6, 8)]]),
                M.AddRMSNormModule(True), M.SDPAModule(), M.GatherStackModule()):
        clone = pickle.loads(pickle.dumps(mod))
        assert type(clone) is type(mod)


def test_module_signatures_match_reference_call_sites(tgt):
    """forward() parameter counts equal what the reference's structure patterns pass."""
    import inspect

    from xpu_graph_b200 import modules as M

    def nparams(cls):
        return len(inspect.signature(cls.forward).parameters) - 1

    assert nparams(M.RMSNormModule) == 3       # (inputs, weight, eps)      custom_rmsnorm.py:28
    assert nparams(M.LayerNormModule) == 4     # (inputs, weight, bias, eps) custom_layernorm.py:28
    assert nparams(M.DenseLayerModule) == 5    # custom_denselayer.py:87-88
    assert nparams(M.BatchDenseLayerModule) == 5
    assert nparams(M.FuseSliceModule) == 2     # (src, slice_len)           fuse_slice.py:104-106
    assert nparams(M.FuseSliceCatSameInputModule) == 2
    assert nparams(M.FuseSliceCatSameInputModule_v2) == 2
    assert len(inspect.signature(M.DenseLayerModule.__init__).parameters) == 2   # M(fast_act)
    assert len(inspect.signature(M.FuseSliceModule.__init__).parameters) == 2    # M(start_indices)


def test_combo_sum_after_multi_slice_cat(tgt, xlog):
    """Two slice+cat groups of one source (merged by FusedMultipleSliceCat) reshaped to 3-D and summed:
    ComboSum3dInp batches the sums into the target's ComboSumModule."""
    g = torch.Generator().manual_seed(6)
    src = torch.randn(12, 200, generator=g)

    def fn(s):
        a = torch.cat([s[:, 0:16], s[:, 32:48]], dim=-1).view(12, 2, 16).sum(dim=1)
        b = torch.cat([s[:, 64:80], s[:, 100:116], s[:, 120:136]], dim=-1).view(12, 3, 16).sum(dim=1)
        return a * 2.0, b * 3.0

    want, got, mods, atens = _compile(tgt, fn, src)
    _same(got[0], want[0])
    _same(got[1], want[1])
    assert "Pattern.FusedMultipleSliceCat changed graph" in xlog.text
    assert any(m.startswith("fuse_slice_cat_v2") for m in mods)
    assert "Pattern.ComboSum3dInp changed graph" in xlog.text
    assert "combo_sum" in mods and not any("sum" in a for a in atens)


def test_add_layer_norm_without_bias(tgt, xlog):
    """The reference's residual-add LayerNorm test (tests/mlu/test_fuse_addlayernorm.py:17-43): torch.layer_norm with a
    weight and bias=None on [8, 1024], the sum returned or not."""
    g = torch.Generator().manual_seed(12)
    x, r, w = torch.randn(8, 1024, generator=g), torch.randn(8, 1024, generator=g), torch.randn(1024, generator=g)

    def fn0(inputs, residual, weight):
        return torch.layer_norm(inputs + residual, normalized_shape=[1024], weight=weight, bias=None, eps=1e-5)

    def fn1(inputs, residual, weight):
        s = inputs + residual
        return torch.layer_norm(s, normalized_shape=[1024], weight=weight, bias=None, eps=1e-5), s

    want, got, mods, atens = _compile(tgt, fn0, x, r, w)
    _same(got, want)
    assert mods == ["xg_add_layer_norm_y"], (mods, atens)
    torch._dynamo.reset()
    want, got, mods, atens = _compile(tgt, fn1, x, r, w)
    _same(got[0], want[0])
    assert torch.equal(got[1], want[1])
    assert mods == ["xg_add_layer_norm"], (mods, atens)


def test_decomposed_attention_operands_stay_views(tgt, xlog):
    """matmul(q, k^T) / s -> softmax -> matmul(v) (the first form of the reference's attention tests,
    tests/common/test_fuse_sdpa.py:14-25): FusedSDPA rewrites it with contiguous copies of q, k and v in front of the
    attention call; the target replaces the copies by views, because its kernels address the operands by strides."""
    import math

    g = torch.Generator().manual_seed(13)
    q, k, v = (torch.randn(2, 8, 38, 64, generator=g).to(torch.float16) for _ in range(3))

    def fn(query, key, value):
        return torch.matmul(query, key.transpose(-2, -1)).div(math.sqrt(64)).softmax(dim=-1).matmul(value)

    want, got, mods, atens = _compile(tgt, fn, q, k, v)
    _same(got, want, 5e-3)
    assert mods == ["xg_sdpa"], mods
    assert "Pattern.SdpaOperandViews changed graph" in xlog.text
    assert not any("clone" in a for a in atens), atens


def test_dense_tower(tgt, xlog):
    """Three chained fp32 Linear+ReLU layers, each large enough for the tensor-core path, collapse into one
    DenseTowerModule call; so does a narrow chain (the weights-in-shared-memory kernel's case); a chain that is neither
    (too few FLOP for the tensor-core path, too wide for shared memory) is left as separate dense layers."""
    torch.manual_seed(9)
    big = torch.nn.Sequential(torch.nn.Linear(512, 512), torch.nn.ReLU(), torch.nn.Linear(512, 512), torch.nn.ReLU(),
                              torch.nn.Linear(512, 256)).eval()
    x = torch.randn(4096, 512)
    want, got, mods, atens = _compile(tgt, big, x)
    _same(got, want, 1e-4)
    assert "Pattern.FusedDenseTower changed graph" in xlog.text
    assert "xg_dense_tower" in mods and "custom_dense_layer_replacement" not in mods

    small = torch.nn.Sequential(torch.nn.Linear(64, 64), torch.nn.ReLU(), torch.nn.Linear(64, 32)).eval()
    want, got, mods, atens = _compile(tgt, small, torch.randn(128, 64))
    _same(got, want, 1e-4)
    assert mods == ["xg_dense_tower"], mods

    middle = torch.nn.Sequential(torch.nn.Linear(64, 192), torch.nn.ReLU(), torch.nn.Linear(192, 160)).eval()
    want, got, mods, atens = _compile(tgt, middle, torch.randn(128, 64))
    _same(got, want, 1e-4)
    assert "xg_dense_tower" not in mods


def test_dense_tower_16bit_pairs(tgt, xlog):
    """bf16 Linear+ReLU -> Linear whose widths fit the two-layer kernel (N <= 256) become one DenseTowerModule call (the
    graph form of targets/mlu/fuse_densetower.py:272-316); a chain whose hidden layer is too wide stays as it is."""
    torch.manual_seed(10)
    narrow = torch.nn.Sequential(torch.nn.Linear(192, 256), torch.nn.ReLU(), torch.nn.Linear(256, 64)).eval().to(torch.bfloat16)
    x = torch.randn(512, 192).to(torch.bfloat16)
    want, got, mods, atens = _compile(tgt, narrow, x)
    _same(got, want, 2e-2)
    assert "Pattern.FusedDenseTower changed graph" in xlog.text
    assert mods == ["xg_dense_tower"], mods

    three = torch.nn.Sequential(torch.nn.Linear(64, 128), torch.nn.GELU(), torch.nn.Linear(128, 128), torch.nn.Sigmoid(),
                                torch.nn.Linear(128, 24)).eval().to(torch.bfloat16)
    want, got, mods, atens = _compile(tgt, three, torch.randn(300, 64).to(torch.bfloat16))
    _same(got, want, 2e-2)
    assert mods == ["xg_dense_tower"], mods

    wide = torch.nn.Sequential(torch.nn.Linear(64, 512), torch.nn.ReLU(), torch.nn.Linear(512, 512)).eval().to(torch.bfloat16)
    want, got, mods, atens = _compile(tgt, wide, torch.randn(256, 64).to(torch.bfloat16))
    assert "xg_dense_tower" not in mods


def test_dense_tower_matmul_form(tgt, xlog):
    """The graph of the reference's own dense-tower test (tests/mlu/test_fuse_densetower.py:18-35): fp16
    matmul(x, W) + bias (+ relu) three times with weights stored [K, N] becomes one DenseTowerModule call, with widths
    the tensor-core chained-layer kernel can take and with the reference's exact sizes (20 -> 32 -> 16 -> 1: a 40-byte
    row stride and a one-column [K, N] weight, which no TMA descriptor addresses: the weights-in-shared-memory kernel's
    case), in fp16 as in the test and in fp32."""
    import torch.nn.functional as F

    def fn0(x, w1, w2, w3, b1, b2, b3):
        out = F.relu(torch.matmul(x, w1) + b1)
        out = F.relu(torch.matmul(out, w2) + b2)
        return torch.matmul(out, w3) + b3

    g = torch.Generator().manual_seed(11)
    for sizes, dtype in (((24, 32, 16, 8), torch.float16), ((20, 32, 16, 1), torch.float16), ((20, 32, 16, 1), torch.float32)):
        x = torch.randn(16, sizes[0], generator=g).to(dtype)
        ws = [(torch.randn(sizes[i], sizes[i + 1], generator=g) * sizes[i] ** -0.5).to(dtype) for i in range(3)]
        bs = [torch.randn(sizes[i + 1], generator=g).to(dtype) for i in range(3)]
        want, got, mods, atens = _compile(tgt, fn0, x, *ws, *bs)
        _same(got, want, 2e-2 if dtype == torch.float16 else 1e-5)
        assert mods == ["xg_dense_tower"], (sizes, dtype, mods)
        assert not any(a in ("mm", "addmm", "matmul", "relu") for a in atens), atens
        torch._dynamo.reset()


def test_combo_dense(tgt, xlog):
    """Five parallel bf16 Linear+ReLU layers of one shape over different inputs -> one ComboDenseModule call;
    three of them are too few (the reference's width of 4) and stay separate."""
    torch.manual_seed(10)

    class Towers(torch.nn.Module):
        def __init__(self, n):
            super().__init__()
            self.layers = torch.nn.ModuleList(torch.nn.Linear(64, 48) for _ in range(n))

        def forward(self, *xs):
            return tuple(torch.relu(layer(x)) for layer, x in zip(self.layers, xs))

    class TwoLevels(torch.nn.Module):  # the second level's operands are the first level's results
        def __init__(self):
            super().__init__()
            self.l1 = torch.nn.ModuleList(torch.nn.Linear(64, 64) for _ in range(4))
            self.l2 = torch.nn.ModuleList(torch.nn.Linear(64, 48) for _ in range(4))

        def forward(self, *xs):
            hs = [torch.relu(layer(x)) for layer, x in zip(self.l1, xs)]
            return tuple(layer(h) for layer, h in zip(self.l2, hs))

    m = TwoLevels().to(torch.bfloat16).eval()
    xs = [torch.randn(32, 64).to(torch.bfloat16) for _ in range(4)]
    want, got, mods, atens = _compile(tgt, m, *xs)
    for w, o in zip(want, got):
        _same(o, w, 3e-2)
    assert "xg_combo_dense" in mods and "custom_dense_layer_replacement" not in mods

    for n, fused in ((5, True), (3, False)):
        m = Towers(n).to(torch.bfloat16).eval()
        xs = [torch.randn(32, 64).to(torch.bfloat16) for _ in range(n)]
        want, got, mods, atens = _compile(tgt, m, *xs)
        for w, o in zip(want, got):
            _same(o, w, 2e-2)
        assert ("xg_combo_dense" in mods) == fused
        if fused:
            assert "Pattern.FusedComboDense changed graph" in xlog.text and "custom_dense_layer_replacement" not in mods


def test_combo_dense_reference_forms_fp32(tgt, xlog):
    """The graphs of the reference's combo test at its own dtype and sizes (tests/mlu/test_combo_matmul.py:17-100:
    fp32, T = 8, one shared or eight split inputs of 5 x 8, [K, N] weights of 8 x 7, no bias / a row of 7 / a full
    5 x 7 addend per layer, with and without relu) end in one grouped call each."""
    g = torch.Generator().manual_seed(12)
    T, M, K, N = 8, 5, 8, 7
    shared = torch.randn(1, M, K, generator=g)
    split = torch.randn(T, M, K, generator=g)
    ws = [torch.randn(K, N, generator=g) for _ in range(T)]
    rows = [torch.randn(N, generator=g) for _ in range(T)]
    mats = [torch.randn(M, N, generator=g) for _ in range(T)]

    def shared_plain(x, *w):
        x = x.squeeze(0)
        return tuple(x @ wi for wi in w)

    def shared_bias(x, *wb):
        x = x.squeeze(0)
        return tuple(x @ wi + bi for wi, bi in zip(wb[:T], wb[T:]))

    def shared_bias_relu(x, *wb):
        x = x.squeeze(0)
        return tuple(torch.relu(x @ wi + bi) for wi, bi in zip(wb[:T], wb[T:]))

    def split_relu(x, *w):
        xs = [i.squeeze(0) for i in x.split(x.shape[0] // T, dim=0)]
        return tuple(torch.relu(xi @ wi) for xi, wi in zip(xs, w))

    def split_linear_t(x, *w):
        xs = [i.squeeze(0) for i in x.split(x.shape[0] // T, dim=0)]
        return tuple(torch.relu(torch.nn.functional.linear(xi, wi.T)) for xi, wi in zip(xs, w))

    cases = [("fn0", shared_plain, (shared, *ws)), ("fn2", shared_bias, (shared, *ws, *mats)), ("fn4", shared_bias, (shared, *ws, *rows)),
             ("fn5", shared_bias_relu, (shared, *ws, *mats)), ("fn6", split_relu, (split, *ws)), ("fn7", split_linear_t, (split, *ws))]
    for name, fn, args in cases:
        want, got, mods, atens = _compile(tgt, fn, *args)
        for w, o in zip(want, got):
            _same(o, w, 1e-5)
        assert mods.count("xg_combo_dense") == 1 and "custom_dense_layer_replacement" not in mods, (name, mods)
        assert not any(a in ("mm", "addmm", "matmul", "relu") for a in atens), (name, atens)
        torch._dynamo.reset()


def test_combo_batch_dense_reference_forms(tgt, xlog):
    """Lists of bmm over one shared input (tests/mlu/test_combo_matmul.py:25-30, 41-46, 102-109: fp32, T = 8, S = 3,
    5 x 6 x 7, without and with full [S, M, K] addends) -> one grouped call over the T * S products."""
    g = torch.Generator().manual_seed(13)
    T, S, M, K, N = 8, 3, 5, 6, 7
    x = torch.randn(S, M, K, generator=g)
    ws = [torch.randn(S, K, N, generator=g) for _ in range(T)]
    bs = [torch.randn(S, M, N, generator=g) for _ in range(T)]

    def plain(x, *w):
        return tuple(torch.bmm(x, wi) for wi in w)

    def with_addend(x, *wb):
        return tuple(x @ wi + bi for wi, bi in zip(wb[:T], wb[T:]))

    for name, fn, args in (("fn1", plain, (x, *ws)), ("fn3", with_addend, (x, *ws, *bs))):
        want, got, mods, atens = _compile(tgt, fn, *args)
        for w, o in zip(want, got):
            _same(o, w, 1e-5)
        assert mods.count("xg_combo_batch_dense") == 1 and "custom_batch_dense_layer_replacement" not in mods, (name, mods)
        assert not any(a in ("bmm", "baddbmm", "matmul") for a in atens), (name, atens)
        torch._dynamo.reset()


def test_dynamic_batch_keeps_the_fusions(tgt):
    """A symbolic row count (torch._dynamo.mark_dynamic on the batch dimension, parameters static - the way the reference's
    tests compile with dynamic=True) does not cost the grouped launch, the dense tower or the residual-add norm: one
    compilation serves three batch sizes and ends in the same modules as the static graph."""
    torch.manual_seed(14)

    class Towers(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.layers = torch.nn.ModuleList(torch.nn.Linear(64, 48) for _ in range(5))

        def forward(self, x):
            return tuple(torch.relu(layer(x)) for layer in self.layers)

    class Chain(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.a, self.b, self.c = torch.nn.Linear(20, 32), torch.nn.Linear(32, 16), torch.nn.Linear(16, 1)

        def forward(self, x):
            return self.c(torch.relu(self.b(torch.relu(self.a(x)))))

    class AddNorm(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.ln = torch.nn.LayerNorm(64)

        def forward(self, x, r):
            return self.ln(x + r)

    cases = ((Towers().eval(), lambda m: (torch.randn(m, 64),), ["xg_combo_dense"]),
             (Chain().eval(), lambda m: (torch.randn(m, 20),), ["xg_dense_tower"]),
             (AddNorm().eval(), lambda m: (torch.randn(m, 64), torch.randn(m, 64)), ["xg_add_layer_norm_y"]))
    for mod, make, expect in cases:
        torch._dynamo.reset()
        cap, graphs = {}, []
        inner = tgt.backend(tgt.make_config(), capture=cap)

        def counting(gm, example_inputs, inner=inner, graphs=graphs):
            graphs.append(1)
            return inner(gm, example_inputs)

        compiled = torch.compile(mod, backend=counting, dynamic=None)
        for m in (5, 9, 13):
            args = make(m)
            for a in args:
                torch._dynamo.mark_dynamic(a, 0)
            with torch.no_grad():
                got, want = compiled(*args), mod(*args)
            for o, w in zip(got if isinstance(got, tuple) else (got,), want if isinstance(want, tuple) else (want,)):
                _same(o, w, 1e-5)
        assert [n.target for n in cap["gm"].graph.nodes if n.op == "call_module"] == expect
        assert len(graphs) == 1, "one compilation for all three batch sizes"
    torch._dynamo.reset()


def test_dynamic_batch_row_sums(tgt):
    """slice -> sum -> cat, sum -> cat and mul -> sum -> cat with a symbolic batch dimension: one module call each, as in
    the static graph."""
    def fn(x, y0, y1, y2):
        s = torch.cat([x[:, 0:10, :].sum(dim=1), x[:, 0:25, :].sum(dim=1), x[:, 8:40, :].sum(dim=1)], dim=-1)
        t = torch.cat([y0.sum(dim=1), y1.sum(dim=1), y2.sum(dim=1)], dim=-1)
        return s, t

    torch._dynamo.reset()
    cap = {}
    compiled = torch.compile(fn, backend=tgt.backend(tgt.make_config(), capture=cap), dynamic=None)
    g = torch.Generator().manual_seed(16)
    for b in (6, 9, 4):
        args = (torch.randn(b, 40, 16, generator=g), torch.randn(b, 3, 8, generator=g), torch.randn(b, 7, 8, generator=g),
                torch.randn(b, 4, 8, generator=g))
        for a in args:
            torch._dynamo.mark_dynamic(a, 0)
        with torch.no_grad():
            got, want = compiled(*args), fn(*args)
        for o, w in zip(got, want):
            _same(o, w, 1e-5)
    mods = [n.target for n in cap["gm"].graph.nodes if n.op == "call_module"]
    assert mods == ["xg_slice_sum_cat_0", "xg_sum_cat"], mods
    assert not [n for n in cap["gm"].graph.nodes if n.op == "call_function"]

    def products(a0, a1, a2, b0, b1, b2):  # the middle pair's second operand broadcasts over the batch
        return torch.cat([(a0 * b0).sum(dim=1), (a1 * b1).sum(dim=1), (a2 * b2).sum(dim=1)], dim=-1)

    torch._dynamo.reset()
    cap = {}
    compiled = torch.compile(products, backend=tgt.backend(tgt.make_config(), capture=cap), dynamic=None)
    for b in (6, 9, 4):
        a = [torch.randn(b, 5, 8, generator=g) for _ in range(3)]
        bb = [torch.randn(1 if i == 1 else b, 5, 8, generator=g) for i in range(3)]
        for t in a + [bb[0], bb[2]]:
            torch._dynamo.mark_dynamic(t, 0)
        with torch.no_grad():
            _same(compiled(*a, *bb), products(*a, *bb), 1e-5)
    assert [n.target for n in cap["gm"].graph.nodes if n.op == "call_module"] == ["xg_mul_sum_cat"]
    torch._dynamo.reset()


def test_dynamic_batch_row_gathers(tgt):
    """The three single-lookup forms (embedding, table[idx] with negative indices, index_select) with a symbolic number
    of lookups: one RowGatherModule call each, as in the static graph."""
    torch.manual_seed(17)

    class Lookups(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.emb = torch.nn.Embedding(1000, 32)
            self.table = torch.nn.Parameter(torch.randn(500, 16))

        def forward(self, i, j, k):
            return self.emb(i), self.table[j], torch.index_select(self.table, 0, k)

    model = Lookups().eval()
    torch._dynamo.reset()
    cap = {}
    compiled = torch.compile(model, backend=tgt.backend(tgt.make_config(), capture=cap), dynamic=None)
    for b in (7, 19, 4):
        i, j, k = torch.randint(0, 1000, (b, 3)), torch.randint(-500, 500, (b,)), torch.randint(0, 500, (b,))
        for t in (i, j, k):
            torch._dynamo.mark_dynamic(t, 0)
        with torch.no_grad():
            got, want = compiled(i, j, k), model(i, j, k)
        for o, w in zip(got, want):
            assert torch.equal(o, w)
    mods = [n.target for n in cap["gm"].graph.nodes if n.op == "call_module"]
    assert mods == ["xg_row_gather", "xg_row_gather_wrap", "xg_row_gather"], mods
    torch._dynamo.reset()


def test_automatic_dynamic_batch(tgt):
    """The reference's own dynamic-shape test style (tests/common/test_dynamic_shape.py:17-31: dynamic=None, the batch size
    walking up and down): the first call compiles a static graph, the second a symbolic one, both with the grouped launch
    and the add + LayerNorm module, and every result equals eager."""
    torch.manual_seed(15)

    class Block(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.layers = torch.nn.ModuleList(torch.nn.Linear(16, 24) for _ in range(4))
            self.ln = torch.nn.LayerNorm(16)

        def forward(self, x, r):
            h = self.ln(x + r)
            return tuple(torch.relu(layer(h)) for layer in self.layers)

    model = Block().eval()
    torch._dynamo.reset()
    cap = {}
    compiled = torch.compile(model, backend=tgt.backend(tgt.make_config(), capture=cap), dynamic=None)
    seen = []
    for bs in list(range(2, 7)) + list(range(7, 2, -1)):
        x, r = torch.randn(bs, 16), torch.randn(bs, 16)
        with torch.no_grad():
            got, want = compiled(x, r), model(x, r)
        for o, w in zip(got, want):
            _same(o, w, 1e-5)
        seen.append([n.target for n in cap["gm"].graph.nodes if n.op == "call_module"])
    assert all(m == ["xg_add_layer_norm_y", "xg_combo_dense"] for m in seen), seen
    torch._dynamo.reset()


def test_dynamic_batch_on_the_benchmark_graphs(tgt):
    """The recsys graph, the encoder block and the Llama-style layer (reduced sizes) compiled with a symbolic batch dimension: same results
    as eager; the recsys graph ends in the same modules as its static compilation (lookups + mask + stack, slice-cat, the
    concatenation, three dense layers), the layer keeps its norms, RoPE, attention and residual-in-epilogue modules."""
    from xpu_graph_b200.workloads import make_llama_layer, make_recsys

    def run(model, inputs, dynamic_args):
        torch._dynamo.reset()
        cap = {}
        compiled = torch.compile(model, backend=tgt.backend(tgt.make_config(), capture=cap), dynamic=None)
        args = tuple(t.clone() for t in inputs)
        for i in dynamic_args:
            torch._dynamo.mark_dynamic(args[i], 0)
        with torch.no_grad():
            got, want = compiled(*args), model(*args)
        for o, w in zip(got if isinstance(got, (tuple, list)) else (got,), want if isinstance(want, (tuple, list)) else (want,)):
            _same(o, w, 1e-5)
        return [n.target for n in cap["gm"].graph.nodes if n.op == "call_module"]

    model, inputs = make_recsys(seed=5, batch=64)
    mods = run(model, inputs, range(len(inputs)))
    assert mods == ["xg_gather_stack", "fuse_slice_cat", "xg_cat_lastdim"] + ["custom_dense_layer_replacement"] * 3, mods
    layer, (x, cos, sin) = make_llama_layer(seed=3, batch=2, seq=64, hidden=256, heads=4, ffn=512)
    mods = run(layer.float(), (x.float(), cos.float(), sin.float()), [0])
    assert mods.count("xg_rope") == 2 and "xg_sdpa" in mods and mods.count("custom_rms_norm") == 2, mods
    assert mods.count("xg_dense_residual") == 2, mods  # both residual adds ride in their projection's epilogue
    from xpu_graph_b200.workloads import make_encoder

    made = make_encoder(seed=1, batch=2, seq=32)
    enc, enc_in = made[0], made[1] if isinstance(made[1], (tuple, list)) else (made[1],)
    mods = run(enc, enc_in, range(len(enc_in)))
    assert mods == ["xg_layer_norm", "custom_dense_layer_replacement", "xg_sdpa", "xg_dense_residual", "xg_layer_norm",
                    "custom_dense_layer_replacement", "xg_dense_residual"], mods  # as the static encoder block
    # in bf16 (the benchmark's dtype) the symbolic batch costs nothing: the same nine modules as the static graph
    layer16, (x16, cos16, sin16) = make_llama_layer(seed=3, batch=2, seq=64, hidden=256, heads=4, ffn=512)
    torch._dynamo.reset()
    cap = {}
    compiled = torch.compile(layer16, backend=tgt.backend(tgt.make_config(), capture=cap), dynamic=None)
    xd = x16.clone()
    torch._dynamo.mark_dynamic(xd, 0)
    with torch.no_grad():
        compiled(xd, cos16, sin16)
    mods = [n.target for n in cap["gm"].graph.nodes if n.op == "call_module"]
    assert mods == ["custom_rms_norm", "custom_dense_layer_replacement", "xg_dense_rope", "xg_dense_rope", "xg_sdpa", "xg_dense_residual",
                    "custom_rms_norm", "xg_dense_swiglu", "xg_dense_residual"], mods
    torch._dynamo.reset()


def test_sum_cat_fusions(tgt, xlog):
    """slice -> sum -> cat, mul -> sum -> cat and sum -> cat along the last dim become one module call each
    (graph forms of targets/mlu/fuse_sum_cat.py and fuse_mul_sum_cat.py; the reference's tests
    tests/mlu/test_fuse_sum_cat.py / test_mul_sum_cat.py compare compiled vs eager the same way)."""
    g = torch.Generator().manual_seed(8)
    x = torch.randn(6, 40, 16, generator=g)
    a = [torch.randn(6, 5, 8, generator=g) for _ in range(3)]
    b = [torch.randn(1 if i == 1 else 6, 5, 8, generator=g) for i in range(3)]
    y = [torch.randn(6, r, 8, generator=g) for r in (3, 7, 4)]

    def fn(x, a0, a1, a2, b0, b1, b2, y0, y1, y2):
        s = torch.cat([x[:, 0:10, :].sum(dim=1), x[:, 0:25, :].sum(dim=1), x[:, 0:4, :].sum(dim=1), x[:, 8:40, :].sum(dim=1)], dim=-1)
        m = torch.cat([(a0 * b0).sum(dim=1), (a1 * b1).sum(dim=1), (a2 * b2).sum(dim=1)], dim=-1)
        c = torch.cat([y0.sum(dim=1), y1.sum(dim=1), y2.sum(dim=1)], dim=-1)
        return s * 2.0, m + 1.0, c - 1.0

    want, got, mods, atens = _compile(tgt, fn, x, *a, *b, *y)
    for w, o in zip(want, got):
        _same(o, w, 1e-5)
    assert "Pattern.FusedSliceSumCat changed graph" in xlog.text
    assert "Pattern.FusedMulSumCat changed graph" in xlog.text
    assert "Pattern.FusedSumCat changed graph" in xlog.text
    assert any(m.startswith("xg_slice_sum_cat") for m in mods) and "xg_mul_sum_cat" in mods and "xg_sum_cat" in mods
    assert not any("sum" in t or "cat" in t or "slice" in t for t in atens)


def test_compile_cache_round_trip(tgt, xlog, tmp_path):
    """The compile cache (cache.py:113-179, 270-326) pickles the rewritten graph with the target's sub-modules and
    custom-op nodes; a second compilation of the same graph loads the artifact instead of re-running the passes
    (the log-line protocol of the reference's tests/common/test_cache.py:13-56)."""
    from xpu_graph import XpuGraphLocalCache
    from xpu_graph_b200.workloads import make_llama_layer

    m, inp = make_llama_layer(seed=3, batch=1, seq=16, hidden=128, heads=1, ffn=256)
    cache = XpuGraphLocalCache(str(tmp_path))
    outs = []
    for _ in range(2):
        torch._dynamo.reset()
        be = tgt.backend(tgt.make_config(enable_cache=True, debug=True), cache=cache)
        with torch.no_grad():
            outs.append(torch.compile(m, backend=be, dynamic=False)(*inp))
    assert xlog.text.count("Save cache in location") == 1
    assert xlog.text.count("Use cache in location") == 1
    assert torch.equal(outs[0], outs[1])
    with torch.no_grad():
        _same(outs[1], m(*inp), 1e-2)


def test_interceptor_monitors_the_target(tgt, xlog, monkeypatch):
    """enable_interceptor runs the original graph beside the compiled one on every call (interceptor.py:93-179); through
    the target's backend() the reference's interceptor monitors the fused graph: agreement stays silent, a wrong
    kernel is reported and dumped."""
    from xpu_graph_b200 import modules as M
    from xpu_graph_b200.workloads import make_encoder

    if torch._utils._get_available_device_type() is None:
        # the interceptor forks the RNG state of "the available device type" (interceptor.py:127); a host without any
        # accelerator has none, which torch.random.fork_rng rejects: name the CUDA module (zero devices to fork here)
        monkeypatch.setattr(torch._utils, "_get_available_device_type", lambda: "cuda")
    m, x = make_encoder(seed=0, batch=2, seq=16, hidden=64, heads=4, ffn=128)
    cfg = tgt.make_config(enable_interceptor="rtol=1e-3,atol=1e-4")
    with torch.no_grad():
        compiled = torch.compile(m, backend=tgt.backend(cfg), dynamic=False)
        got = compiled(x)
        _same(got, m(x), 1e-4)
        assert "Monitored inference" in xlog.text and "diverges" not in xlog.text
        # a broken replacement is caught: make the fused LayerNorm return something else for one call
        keep = M.LayerNormModule.forward
        try:
            M.LayerNormModule.forward = lambda self, inputs, weights, bias, epsilon: keep(self, inputs, weights, bias, epsilon) + 1.0
            compiled(x)
        finally:
            M.LayerNormModule.forward = keep
    assert "The inference pass diverges" in xlog.text


def test_reference_front_end_runs_the_target(tgt, xlog, monkeypatch):
    """torch.compile(model, backend=XpuGraph(config)) - the reference's own entry (compiler.py:196-237): graph dispatch
    through fx_utils.dispatch_graph (repaired for this PyTorch by target/compat.py), the pass manager with this target's
    patterns, the runtime artifact, and the interceptor fed with the forward metadata."""
    from xpu_graph import XpuGraph
    from xpu_graph_b200.workloads import make_encoder

    if torch._utils._get_available_device_type() is None:
        monkeypatch.setattr(torch._utils, "_get_available_device_type", lambda: "cuda")
    m, x = make_encoder(seed=0, batch=2, seq=16, hidden=64, heads=4, ffn=128)
    be = tgt.reference_backend(tgt.make_config(debug=True))
    assert isinstance(be, XpuGraph)
    with torch.no_grad():
        got = torch.compile(m, backend=be, dynamic=False)(x)
        _same(got, m(x), 1e-4)
    assert "decompose graph complete" in xlog.text            # compiler.py:187: the dispatch_graph branch ran
    for name in ("FusedNativeLayerNorm", "FusedSdpa"):
        assert name in xlog.text, f"{name} did not fire through the reference front-end"
    torch._dynamo.reset()
    cfg = tgt.make_config(enable_interceptor="rtol=1e-3,atol=1e-4")
    with torch.no_grad():
        got = torch.compile(m, backend=tgt.reference_backend(cfg), dynamic=False)(x)
        _same(got, m(x), 1e-4)
    assert "Monitored inference" in xlog.text and "diverges" not in xlog.text

