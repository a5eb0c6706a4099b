"""GPU parity: dense layers (matmul + bias + activation) through the C ABI vs the CPU oracle.

The 21 bias / activation / transpose variants of the reference's tests/mlu/test_custom_denselayer.py
(fn0-fn20) reduce to: act in {none, gelu, relu, silu, sigmoid} x bias in {none, [N], [1,N], [M,N]} x
weight given as [K,N] or [N,K]; the cases below cover that grid at ragged and tile-aligned sizes.
"""
import pytest
import torch

from oracle import ref_ops
from tests.helpers import LaunchCounter, assert_parity, error_stats

pytestmark = pytest.mark.gpu


def _mk(M, K, N, dtype, seed, weight_trans=True):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(M, K, generator=g).to(dtype)
    w = (0.02 * torch.randn(N, K, generator=g)).to(dtype)
    if not weight_trans:
        w = w.t().contiguous()
    b = (0.02 * torch.randn(N, generator=g)).to(dtype)
    return x, w, b


@pytest.mark.parametrize("act", ["none", "gelu", "silu", "relu", "sigmoid"])
@pytest.mark.parametrize(
    "M,K,N",
    [(128, 64, 256), (256, 4096, 512), (200, 200, 136), (1, 8, 8), (384, 1024, 1000), (130, 72, 264), (512, 512, 11008 // 8)],
)
def test_dense_bf16(cuda_device, M, K, N, act):
    from xpu_graph_b200 import lib
    from xpu_graph_b200.modules import DenseLayerModule

    x, w, b = _mk(M, K, N, torch.bfloat16, 20)
    got = DenseLayerModule(False)(x.to(cuda_device), w.to(cuda_device), True, b.to(cuda_device), act)
    torch.cuda.synchronize()
    assert lib.tc_status() == 0, "a bounded wait expired inside the tensor-core kernel"
    want = ref_ops.dense(x, w, True, b, act)
    assert_parity(got, want, f"dense bf16 {M}x{K}x{N} {act}")
    # report against exact fp32 math as well
    exact = ref_ops.dense(x.float(), w.float(), True, b.float(), act)
    max_abs, mean_rel = error_stats(got, exact)
    print(f"dense bf16 {M}x{K}x{N} {act}: max_abs={max_abs:.3g} mean_rel={mean_rel:.3g} vs fp32 math")


@pytest.mark.parametrize("bias_form", ["none", "row", "full"])
def test_dense_bias_forms(cuda_device, bias_form):
    from xpu_graph_b200.modules import DenseLayerModule

    M, K, N = 260, 320, 392
    x, w, b = _mk(M, K, N, torch.bfloat16, 21)
    g = torch.Generator().manual_seed(22)
    bias = {"none": None, "row": b.view(1, N), "full": torch.randn(M, N, generator=g).to(torch.bfloat16)}[bias_form]
    got = DenseLayerModule(False)(x.to(cuda_device), w.to(cuda_device), True, bias.to(cuda_device) if bias is not None else None, "gelu")
    assert_parity(got, ref_ops.dense(x, w, True, bias, "gelu"), f"dense bias {bias_form}")


@pytest.mark.parametrize("act", ["none", "gelu"])
@pytest.mark.parametrize("M,K,N", [(128, 64, 256), (300, 512, 1000), (130, 72, 264), (64, 4096, 128)])
def test_dense_bf16_kn_weights(cuda_device, M, K, N, act):
    """Weights given as [K, N] (x @ W without a transpose): consumed MN-major by the tensor cores."""
    from xpu_graph_b200 import lib
    from xpu_graph_b200.modules import DenseLayerModule

    x, w, b = _mk(M, K, N, torch.bfloat16, 27, weight_trans=False)
    got = DenseLayerModule(False)(x.to(cuda_device), w.to(cuda_device), False, b.to(cuda_device), act)
    torch.cuda.synchronize()
    assert lib.tc_status() == 0
    assert_parity(got, ref_ops.dense(x, w, False, b, act), f"dense bf16 [K,N] {M}x{K}x{N} {act}")


@pytest.mark.parametrize("M,K,N,act,with_res", [(64, 4096, 4096, "gelu", False), (32, 4096, 11008, "silu", False),
                                                (16, 4096, 11008, "silu", False), (128, 4096, 2048, "gelu", False),
                                                (128, 4096, 1000, "none", True), (100, 2048, 1002, "relu", True),
                                                (16, 1024, 512, "gelu", True), (1, 4096, 4096, "none", False)])
def test_dense_split_k(cuda_device, M, K, N, act, with_res):
    """Small-M shapes: the kernel splits K across CTAs and reduces fp32 partial sums from scratch memory
    (allocated by the op). Checked against the oracle and for run-to-run bit equality."""
    from xpu_graph_b200 import lib
    from xpu_graph_b200.modules import DenseResidualModule

    if (M, K, N) in ((64, 4096, 4096), (16, 4096, 11008), (128, 4096, 2048), (1, 4096, 4096)):
        assert lib.load().xg_gemm_workspace_bytes(M, N, K, lib.XG_BF16) > 0, "shape expected to use split-K"
    x, w, b = _mk(M, K, N, torch.bfloat16, 28)
    g = torch.Generator().manual_seed(29)
    r = torch.randn(M, N, generator=g).to(torch.bfloat16) if with_res else None
    args = (x.to(cuda_device), w.to(cuda_device), True, b.to(cuda_device), r.to(cuda_device) if with_res else None, act)
    got = DenseResidualModule()(*args)
    again = DenseResidualModule()(*args)
    torch.cuda.synchronize()
    assert lib.tc_status() == 0
    want = ref_ops.dense(x, w, True, b, "none")
    if with_res:
        want = want + r
    want = ref_ops._ACTS[act](want)
    assert_parity(got, want, f"split-K dense {M}x{K}x{N}", magnitude=r)
    assert torch.equal(got, again), "split-K reduction must be deterministic"


def _cluster_dense(L, lib, x, w, b, r, act, out, splits, tile_n):
    M, K = x.shape
    N = w.shape[0]
    return L.xg_gemm_bias_act_cluster(x.data_ptr(), w.data_ptr(), b.data_ptr() if b is not None else None,
                                      r.data_ptr() if r is not None else None, out.data_ptr(), M, N, K, x.stride(0),
                                      w.stride(0), out.stride(0), r.stride(0) if r is not None else 0, lib.ACT_CODES[act],
                                      lib.XG_BF16 if x.dtype == torch.bfloat16 else lib.XG_F16, splits, tile_n,
                                      torch.cuda.current_stream().cuda_stream)


@pytest.mark.parametrize("splits,tile_n", [(1, 64), (1, 160), (1, 256), (2, 64), (2, 128), (2, 256), (3, 96), (3, 256),
                                           (4, 128), (4, 256)])
@pytest.mark.parametrize("M,K,N,act,with_res", [(256, 4096, 1024, "gelu", False), (300, 1032, 520, "none", True),
                                                (77, 512, 1000, "silu", True), (512, 2048, 264, "relu", False)])
def test_dense_cluster_kernel(cuda_device, splits, tile_n, M, K, N, act, with_res):
    """The cluster kernel at every decomposition (k-splits 1..4 x tile widths incl. the uneven column shares of 3
    pairs), tile-aligned and ragged M / N / K, with bias, residual and activation: against the oracle, and bit-equal
    from run to run (the partial tiles are added in split order)."""
    from xpu_graph_b200 import lib

    L = lib.load()
    x, w, b = _mk(M, K, N, torch.bfloat16, 41)
    g = torch.Generator().manual_seed(42)
    r = torch.randn(M, N, generator=g).to(torch.bfloat16) if with_res else None
    xd, wd, bd = x.to(cuda_device), w.to(cuda_device), b.to(cuda_device)
    rd = r.to(cuda_device) if with_res else None
    outs = []
    for _ in range(2):
        out = torch.full((M, N), float("nan"), device=cuda_device, dtype=torch.bfloat16)
        lib.check(_cluster_dense(L, lib, xd, wd, bd, rd, act, out, splits, tile_n), "xg_gemm_bias_act_cluster")
        outs.append(out)
    torch.cuda.synchronize()
    assert lib.tc_status() == 0, "a bounded wait expired inside the cluster kernel"
    want = ref_ops.dense(x, w, True, b, "none")
    if with_res:
        want = want + r
    want = ref_ops._ACTS[act](want)
    assert_parity(outs[0], want, f"cluster dense {M}x{K}x{N} splits={splits} tile_n={tile_n}", magnitude=r)
    assert torch.equal(outs[0], outs[1]), "the exchange must add the partial tiles in a fixed order"


def test_dense_cluster_kernel_matches_unsplit_bitwise_inputs(cuda_device):
    """fp16 and an odd leading dimension of the output (scalar store path), plus the argument checks of the entry point."""
    from xpu_graph_b200 import lib

    L = lib.load()
    M, K, N = 260, 768, 328
    x, w, b = _mk(M, K, N, torch.float16, 43)
    xd, wd, bd = x.to(cuda_device), w.to(cuda_device), b.to(cuda_device)
    wide = torch.zeros(M, N + 3, device=cuda_device, dtype=torch.float16)
    out = wide[:, :N]  # row stride N + 3: not 16-byte addressable
    lib.check(_cluster_dense(L, lib, xd, wd, bd, None, "gelu", out, 3, 128), "xg_gemm_bias_act_cluster")
    torch.cuda.synchronize()
    assert lib.tc_status() == 0
    assert_parity(out.contiguous(), ref_ops.dense(x, w, True, b, "gelu"), "cluster dense fp16, odd ldc")
    assert float(wide[:, N:].abs().max()) == 0.0, "columns beyond N must stay untouched"
    good = torch.empty(M, N, device=cuda_device, dtype=torch.float16)
    assert _cluster_dense(L, lib, xd, wd, bd, None, "none", good, 5, 256) == -1      # splits out of range
    assert _cluster_dense(L, lib, xd, wd, bd, None, "none", good, 3, 64) == -1       # fewer 32-column chunks than pairs
    assert _cluster_dense(L, lib, xd, wd, bd, None, "none", good, 2, 100) == -1      # tile width not a multiple of 32
    short = torch.zeros(M, 64, device=cuda_device, dtype=torch.float16)
    assert L.xg_gemm_bias_act_cluster(short.data_ptr(), wd.data_ptr(), None, None, good.data_ptr(), M, N, 64, 64, K, N, 0, 0,
                                      lib.XG_F16, 2, 128, torch.cuda.current_stream().cuda_stream) == -1  # one k-block, two pairs


def test_dense_picks_the_cluster_kernel_for_few_tiles(cuda_device):
    """The planner's choice for the weight-streaming cells of the matmul sweep, and that the op needs no scratch there."""
    import ctypes

    from xpu_graph_b200 import lib

    L = lib.load()
    s, t = ctypes.c_int(0), ctypes.c_int(0)
    for (M, N, K) in ((256, 4096, 4096), (256, 11008, 4096), (512, 4096, 4096)):
        assert L.xg_gemm_cluster_plan(M, N, K, lib.XG_BF16, ctypes.byref(s), ctypes.byref(t)) == 1, (M, N, K)
        assert 1 <= s.value <= 4 and 64 <= t.value <= 256 and t.value % 32 == 0
        assert L.xg_gemm_workspace_bytes(M, N, K, lib.XG_BF16) == 0
    for (M, N, K) in ((16384, 4096, 4096), (64, 4096, 4096)):  # the persistent pair kernel / split-K through scratch
        assert L.xg_gemm_cluster_plan(M, N, K, lib.XG_BF16, ctypes.byref(s), ctypes.byref(t)) == 0, (M, N, K)


def test_dense_fp16(cuda_device):
    from xpu_graph_b200.modules import DenseLayerModule

    x, w, b = _mk(300, 256, 520, torch.float16, 23)
    got = DenseLayerModule(False)(x.to(cuda_device), w.to(cuda_device), True, b.to(cuda_device), "silu")
    assert_parity(got, ref_ops.dense(x, w, True, b, "silu"), "dense fp16")


@pytest.mark.parametrize("weight_trans", [True, False])
@pytest.mark.parametrize("act", ["none", "gelu", "relu"])
@pytest.mark.parametrize("M,K,N", [(256, 256, 768), (256, 1024, 256), (100, 37, 53), (1024, 1728, 1024)])
def test_dense_fp32(cuda_device, M, K, N, act, weight_trans):
    from xpu_graph_b200.modules import DenseLayerModule

    x, w, b = _mk(M, K, N, torch.float32, 24, weight_trans)
    got = DenseLayerModule(False)(x.to(cuda_device), w.to(cuda_device), weight_trans, b.to(cuda_device), act)
    # fp64 math is the yardstick for the fp32 path: both aten and this kernel are within 1e-5 of it
    want = ref_ops.dense(x.double(), w.double(), weight_trans, b.double(), act).float()
    assert_parity(got, want, f"dense fp32 {M}x{K}x{N} {act}")


@pytest.mark.parametrize("weight_trans", [True, False])
@pytest.mark.parametrize("M,K,N,act,with_res", [(2048, 512, 1024, "relu", False), (1100, 1000, 520, "gelu", True),
                                                (4096, 1728, 1024, "none", False), (300, 4100, 450, "sigmoid", True)])
def test_dense_fp32_on_tensor_cores(cuda_device, M, K, N, act, with_res, weight_trans):
    """fp32 dense layers of at least 2^30 FLOPs run from three bf16 planes per operand on the tensor cores: the result
    must stay within the fp32 tolerance of fp64 math (ragged M / N / K, both weight layouts, bias + residual + act)."""
    from xpu_graph_b200 import lib, ops

    assert ops._f32_on_tensor_cores(M, N, K)
    x, w, b = _mk(M, K, N, torch.float32, 26, weight_trans)
    r = torch.randn(M, N, generator=torch.Generator().manual_seed(27)) if with_res else None
    with LaunchCounter() as calls:
        got = torch.ops.xg_sm100.dense(x.to(cuda_device), w.to(cuda_device), weight_trans, b.to(cuda_device),
                                       r.to(cuda_device) if with_res else None, act)
    torch.cuda.synchronize()
    assert calls.n >= 2 and "xg_gemm_f32x3" in calls.names  # operand split(s) and the tensor-core GEMM
    assert lib.tc_status() == 0
    y = x.double() @ (w.double().t() if weight_trans else w.double()) + b.double()
    if with_res:
        y = y + r.double()
    want = ref_ops._ACTS[act](y).float()
    assert_parity(got, want, f"dense fp32 (bf16 planes) {M}x{K}x{N} {act}")


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("M,K1,N1,N2,acts,with_bias", [
    (300, 256, 128, 64, ("relu", "none"), (True, True)),
    (1000, 520, 200, 100, ("gelu", "sigmoid"), (True, False)),   # ragged K1 (not a multiple of 64), N1, N2
    (16384, 512, 256, 256, ("relu", "relu"), (True, True)),      # the widest layers the kernel takes; one block per SM and more
    (128, 64, 16, 1, ("silu", "none"), (False, True)),
    (4100, 1024, 256, 40, ("none", "gelu"), (False, False)),
    (40000, 72, 96, 136, ("relu", "silu"), (True, True)),        # several blocks per CTA
])
def test_mlp2(cuda_device, M, K1, N1, N2, acts, with_bias, dtype):
    """Two chained dense layers in one kernel (the hidden activation handed over through shared memory) vs the two
    layers one after the other on CPU, the hidden tensor rounded to the 16-bit dtype in between as eager does."""
    from xpu_graph_b200 import lib, ops  # noqa: F401  (ops registers torch.ops.xg_sm100.*)

    g = torch.Generator().manual_seed(41)
    x = torch.randn(M, K1, generator=g).to(dtype)
    w1 = (torch.randn(N1, K1, generator=g) * K1 ** -0.5).to(dtype)
    w2 = (torch.randn(N2, N1, generator=g) * N1 ** -0.5).to(dtype)
    b1 = (0.1 * torch.randn(N1, generator=g)).to(dtype) if with_bias[0] else None
    b2 = (0.1 * torch.randn(N2, generator=g)).to(dtype) if with_bias[1] else None
    dev = lambda t: t.to(cuda_device) if t is not None else None
    got = torch.ops.xg_sm100.mlp2(dev(x), dev(w1), dev(b1), dev(w2), dev(b2), acts[0], acts[1])
    torch.cuda.synchronize()
    assert lib.tc_status() == 0, "a bounded wait expired inside the two-layer kernel"
    # (a) the kernel's own arithmetic: fp32 through the first layer and its activation, ONE rounding of the hidden
    #     tensor to the 16-bit dtype, fp32 through the second layer
    f = lambda t: t.float() if t is not None else None
    h = ref_ops.dense(f(x), f(w1), True, f(b1), acts[0]).to(dtype)
    once = ref_ops.dense(f(h), f(w2), True, f(b2), acts[1]).to(dtype)
    assert_parity(got, once, f"mlp2 {M}x{K1}->{N1}->{N2} {acts} {dtype} (hidden rounded once)")
    # (b) the eager chain, which rounds the hidden tensor after the linear and again after the activation: its hidden
    #     elements can sit one rounding step (2^-8 relative for bf16, 2^-11 for f16) away from the kernel's, so the
    #     outputs may differ by that step times the sum of |h w| over the hidden width
    want = ref_ops.dense(ref_ops.dense(x, w1, True, b1, acts[0]), w2, True, b2, acts[1])
    step = 2.0 ** -8 if dtype == torch.bfloat16 else 2.0 ** -11
    from tests.helpers import BF16_RTOL
    assert_parity(got, want, f"mlp2 {M}x{K1}->{N1}->{N2} {acts} {dtype} (eager chain)",
                  magnitude=(h.float().abs() @ w2.float().abs().t()) * (step / BF16_RTOL))


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("M,dims,acts", [
    (5000, [256, 256, 128, 64], ("relu", "relu", "none")),
    (700, [72, 200, 104, 30], ("gelu", "silu", "sigmoid")),       # ragged everywhere
    (30000, [512, 256, 256, 256], ("relu", "relu", "relu")),      # widest; several blocks per CTA
])
def test_mlp3(cuda_device, M, dims, acts, dtype):
    """Three chained dense layers in one kernel vs the kernel's own arithmetic on CPU (fp32 through each layer, one
    rounding of each hidden tensor to the 16-bit dtype)."""
    from xpu_graph_b200 import lib, ops  # noqa: F401

    g = torch.Generator().manual_seed(43)
    x = torch.randn(M, dims[0], generator=g).to(dtype)
    ws = [(torch.randn(dims[i + 1], dims[i], generator=g) * dims[i] ** -0.5).to(dtype) for i in range(3)]
    bs = [(0.1 * torch.randn(dims[i + 1], generator=g)).to(dtype) for i in range(3)]
    bs[1] = None
    dev = lambda t: t.to(cuda_device) if t is not None else None
    got = torch.ops.xg_sm100.mlp3(dev(x), dev(ws[0]), dev(bs[0]), dev(ws[1]), dev(bs[1]), dev(ws[2]), dev(bs[2]), *acts)
    torch.cuda.synchronize()
    assert lib.tc_status() == 0, "a bounded wait expired inside the chained-layer kernel"
    f = lambda t: t.float() if t is not None else None
    y = x
    for w, b, a in zip(ws, bs, acts):
        y = ref_ops.dense(f(y), f(w), True, f(b), a).to(dtype)
    assert_parity(got, y, f"mlp3 {M}x{dims} {acts} {dtype}")


@pytest.mark.parametrize("tag", ["bf16", "f16"])
@pytest.mark.parametrize("name", ["two", "three"])
def test_mlp_against_reference_fixtures(cuda_device, name, tag):
    """The chained-layer kernel (through DenseTowerModule, one launch) on the inputs of tests/golden/golden_v3.pt vs the
    outputs the reference pipeline recorded for them."""
    import os

    from tests.helpers import LaunchCounter
    from xpu_graph_b200 import lib
    from xpu_graph_b200.modules import DenseTowerModule

    c = torch.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "golden_v3.pt"))[f"tower_{name}_{tag}"]
    dev = lambda t: t.to(cuda_device)
    with LaunchCounter() as launches:
        got = DenseTowerModule()(dev(c["x"]), [dev(w) for w in c["ws"]], [True] * len(c["ws"]), [dev(b) for b in c["bs"]], c["acts"])
    torch.cuda.synchronize()
    assert lib.tc_status() == 0
    assert launches.names == ["xg_mlp2_bias_act" if name == "two" else "xg_mlp3_bias_act"], launches.names
    assert_parity(got, c["y"], f"chained-layer kernel vs reference fixture ({name}, {tag})")


def test_grouped_tower_and_unaligned_kernels_against_reference_fixtures(cuda_device):
    """The grouped fp32 launches, the batched-list form, the weights-in-shared-memory tower and the 16-bit FMA path on
    the inputs of tests/golden/golden_v4.pt (the reference's combo and dense-tower test graphs at their own sizes) vs
    the outputs the reference pipeline recorded for them; one launch each."""
    import os

    from tests.helpers import LaunchCounter
    from xpu_graph_b200.modules import ComboBatchDenseModule, ComboDenseModule, DenseLayerModule, DenseTowerModule

    G4 = torch.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "golden_v4.pt"))
    dev = lambda t: None if t is None else t.to(cuda_device)  # noqa: E731
    for name in ("combo_plain", "combo_matrix_bias", "combo_row_bias", "combo_matrix_bias_relu", "combo_split_linear_t"):
        c = G4[name]
        x = dev(c["x"])
        xs = [x[0]] * len(c["ws"]) if c["shared"] else list(x.unbind(0))
        with LaunchCounter() as launches:
            got = ComboDenseModule()(xs, [dev(w) for w in c["ws"]], [dev(b) for b in c["bs"]], c["act"], False)
        assert launches.names == ["xg_gemm_group_bias_act"], (name, launches.names)
        assert_parity(got, torch.stack(list(c["y"])), f"{name} vs reference fixture")
    for name in ("combo_bmm_plain", "combo_bmm_addend"):
        c = G4[name]
        with LaunchCounter() as launches:
            got = ComboBatchDenseModule()([dev(c["x"])] * len(c["ws"]), [dev(w) for w in c["ws"]], [dev(b) for b in c["bs"]], "none", False)
        assert launches.names == ["xg_gemm_group_bias_act"], (name, launches.names)
        assert_parity(got, torch.stack(list(c["y"])), f"{name} vs reference fixture")
    c = G4["tower_kn_f16"]
    with LaunchCounter() as launches:
        got = DenseTowerModule()(dev(c["x"]), [dev(w) for w in c["ws"]], [False] * 3, [dev(b) for b in c["bs"]], c["acts"])
    assert launches.names == ["xg_mlp_small_bias_act"], launches.names
    assert_parity(got, c["y"], "narrow tower vs reference fixture")
    c = G4["dense_unaligned_bf16"]
    got = DenseLayerModule(False)(dev(c["x"]), dev(c["w"]), True, dev(c["b"]), c["act"])
    torch.cuda.synchronize()
    assert_parity(got, c["y"], "bf16 layer with K = 444 vs reference fixture")


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_mlp_kn_weights(cuda_device, dtype):
    """Weights stored [K, N] (the operand of torch.matmul(x, W), the form of the reference's dense-tower test) are
    consumed MN-major as TMA leaves them: all layers [K, N], and a mix of both layouts."""
    from xpu_graph_b200 import lib, ops  # noqa: F401

    g = torch.Generator().manual_seed(44)
    M, dims = 1500, [200, 256, 104, 48]
    x = torch.randn(M, dims[0], generator=g).to(dtype)
    ws_nk = [(torch.randn(dims[i + 1], dims[i], generator=g) * dims[i] ** -0.5).to(dtype) for i in range(3)]
    bs = [(0.1 * torch.randn(dims[i + 1], generator=g)).to(dtype) for i in range(3)]
    acts = ("relu", "gelu", "none")
    dev = lambda t: t.to(cuda_device)
    f = lambda t: t.float()
    y = x
    for w, b, a in zip(ws_nk, bs, acts):
        y = ref_ops.dense(f(y), f(w), True, f(b), a).to(dtype)
    for mask in (0b111, 0b101, 0b010):
        ws = [w.t().contiguous() if (mask >> l) & 1 else w for l, w in enumerate(ws_nk)]
        got = torch.ops.xg_sm100.mlp3(dev(x), dev(ws[0]), dev(bs[0]), dev(ws[1]), dev(bs[1]), dev(ws[2]), dev(bs[2]), *acts, mask)
        torch.cuda.synchronize()
        assert lib.tc_status() == 0
        assert_parity(got, y, f"mlp3 with weight layout mask {mask:03b} {dtype}")
    y2 = ref_ops.dense(ref_ops.dense(f(x), f(ws_nk[0]), True, f(bs[0]), "silu").to(dtype).float(), f(ws_nk[1]), True, None, "none").to(dtype)
    got = torch.ops.xg_sm100.mlp2(dev(x), dev(ws_nk[0].t().contiguous()), dev(bs[0]), dev(ws_nk[1].t().contiguous()), None, "silu", "none", 3)
    assert_parity(got, y2, f"mlp2 with [K, N] weights {dtype}")


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_transposed_view_weights(cuda_device, dtype):
    """Weights handed over as transposed views (w.T of a contiguous matrix, what F.linear(x, w.T) and x @ w.t() produce)
    are read through their base in the other orientation: dense layers in both orientations, and the grouped launch of
    the reference's combo test form (tests/mlu/test_combo_matmul.py:73-79: relu(F.linear(x_i, w_i.T)))."""
    from tests.helpers import LaunchCounter
    from xpu_graph_b200 import lib, ops  # noqa: F401
    from xpu_graph_b200.modules import ComboDenseModule, DenseLayerModule

    g = torch.Generator().manual_seed(45)
    M, K, N = 200, 128, 72
    x = torch.randn(M, K, generator=g).to(dtype)
    w_kn = (torch.randn(K, N, generator=g) * K ** -0.5).to(dtype)   # contiguous [K, N]
    w_nk = w_kn.t().contiguous()                                     # contiguous [N, K]
    b = (0.1 * torch.randn(N, generator=g)).to(dtype)
    want = ref_ops.dense(x, w_nk, True, b, "gelu")
    xd, bd = x.to(cuda_device), b.to(cuda_device)
    # [N, K] given as the transposed view of a contiguous [K, N] matrix, and the other way round
    got = DenseLayerModule(False)(xd, w_kn.to(cuda_device).t(), True, bd, "gelu")
    assert_parity(got, want, f"dense, weight = (K,N).T view {dtype}")
    got = DenseLayerModule(False)(xd, w_nk.to(cuda_device).t(), False, bd, "gelu")
    assert_parity(got, want, f"dense, weight = (N,K).T view {dtype}")
    if dtype == torch.float32:
        return
    T = 6
    xs = [torch.randn(M, K, generator=g).to(dtype) for _ in range(T)]
    ws = [(torch.randn(K, N, generator=g) * K ** -0.5).to(dtype) for _ in range(T)]
    with LaunchCounter() as c:
        got = ComboDenseModule()([t.to(cuda_device) for t in xs], [w.to(cuda_device).t() for w in ws], [None] * T, "relu", True)
    torch.cuda.synchronize()
    assert lib.tc_status() == 0 and c.names == ["xg_gemm_group_bias_act"], c.names
    for i in range(T):
        assert_parity(got[i], ref_ops.dense(xs[i], ws[i], False, None, "relu"), f"combo member {i}, transposed-view weights")


def test_mlp2_strided_input_and_limits(cuda_device):
    """A row-strided x (a column slice of a wider tensor) is read in place; shapes outside the kernel's limits are
    refused with XG_ERR_UNSUPPORTED, and the tower op then runs the layers one by one."""
    from xpu_graph_b200 import lib, ops  # noqa: F401
    from xpu_graph_b200.modules import DenseTowerModule

    g = torch.Generator().manual_seed(42)
    wide = torch.randn(700, 384, generator=g).to(torch.bfloat16)
    x = wide[:, 64:320]
    w1 = (torch.randn(64, 256, generator=g) / 16).to(torch.bfloat16)
    w2 = (torch.randn(32, 64, generator=g) / 8).to(torch.bfloat16)
    got = torch.ops.xg_sm100.mlp2(wide.to(cuda_device)[:, 64:320], w1.to(cuda_device), None, w2.to(cuda_device), None, "relu", "none")
    assert_parity(got, ref_ops.dense(ref_ops.dense(x, w1, True, None, "relu"), w2, True, None, "none"), "mlp2 strided x")
    L = lib.load()
    assert L.xg_mlp2_supported(128, 64, 512, 64, lib.XG_BF16) == 0      # hidden layer too wide
    assert L.xg_mlp2_supported(128, 64, 100, 64, lib.XG_BF16) == 0      # N1 not a multiple of 8
    assert L.xg_mlp2_supported(128, 64, 128, 64, lib.XG_F32) == 0
    assert L.xg_mlp2_supported(128, 64, 128, 64, lib.XG_F16) == 1
    # a three-layer 16-bit tower: the first two layers as one launch, the third (too wide to pair) on its own
    w3 = (torch.randn(512, 32, generator=g) / 6).to(torch.bfloat16)
    from tests.helpers import LaunchCounter
    with LaunchCounter() as c:
        got = DenseTowerModule()(x.to(cuda_device), [w1.to(cuda_device), w2.to(cuda_device), w3.to(cuda_device)],
                                 [True, True, True], [None, None, None], ["relu", "relu", "none"])
    torch.cuda.synchronize()
    assert lib.tc_status() == 0
    assert len(c.names) == 2 and c.names[0] == "xg_mlp2_bias_act" and c.names[1].startswith("xg_gemm_bias_act"), c.names
    want = ref_ops.dense(ref_ops.dense(ref_ops.dense(x, w1, True, None, "relu"), w2, True, None, "relu"), w3, True, None, "none")
    assert_parity(got, want, "16-bit dense tower")
    # all three layers narrow: one launch
    w3n = (torch.randn(48, 32, generator=g) / 6).to(torch.bfloat16)
    with LaunchCounter() as c:
        got = DenseTowerModule()(x.to(cuda_device), [w1.to(cuda_device), w2.to(cuda_device), w3n.to(cuda_device)],
                                 [True, True, True], [None, None, None], ["relu", "relu", "none"])
    torch.cuda.synchronize()
    assert lib.tc_status() == 0 and c.names == ["xg_mlp3_bias_act"], c.names
    want = ref_ops.dense(ref_ops.dense(ref_ops.dense(x, w1, True, None, "relu"), w2, True, None, "relu"), w3n, True, None, "none")
    assert_parity(got, want, "16-bit dense tower, three narrow layers")


def test_dense_tower_fp32(cuda_device):
    """Recsys MLP sizes (1728 -> 1024 -> 512 -> 256 over 16384 rows, ReLU between): the inner results travel as bf16
    planes; the result must stay within the fp32 tolerance of fp64 math. A ragged tower checks the zero padding."""
    from xpu_graph_b200 import lib
    from xpu_graph_b200.modules import DenseTowerModule

    for M, dims, acts in [(16384, [1728, 1024, 512, 256], ["relu", "relu", "none"]), (3000, [600, 1000, 420], ["gelu", "sigmoid"])]:
        g = torch.Generator().manual_seed(31)
        x = torch.randn(M, dims[0], generator=g)
        ws = [0.05 * torch.randn(dims[i + 1], dims[i], generator=g) for i in range(len(dims) - 1)]
        bs = [0.05 * torch.randn(dims[i + 1], generator=g) for i in range(len(dims) - 1)]
        bs[-1] = None
        got = DenseTowerModule()(x.to(cuda_device), [w.to(cuda_device) for w in ws], [True] * len(ws),
                                 [b.to(cuda_device) if b is not None else None for b in bs], acts)
        torch.cuda.synchronize()
        assert lib.tc_status() == 0
        y = x.double()
        for w, b, a in zip(ws, bs, acts):
            y = y @ w.double().t()
            if b is not None:
                y = y + b.double()
            y = ref_ops._ACTS[a](y)
        assert_parity(got, y.float(), f"dense tower {dims}")


def test_split_bf16x3_planes_add_up(cuda_device):
    """x0 + x1 + x2 reproduces x to 2^-24 relative; padding columns are zero; the transposed form agrees."""
    from xpu_graph_b200 import lib

    L = lib.load()
    g = torch.Generator().manual_seed(28)
    x = (torch.randn(37, 100, generator=g) * torch.logspace(-20, 20, 100)).to(cuda_device)
    Kp = int(L.xg_gemm_f32x3_padded_k(100))
    assert Kp == 128
    out = torch.full((37, 3 * Kp), 7.0, dtype=torch.bfloat16, device=cuda_device)
    assert L.xg_split_bf16x3(x.data_ptr(), 37, 100, 100, 0, out.data_ptr(), None) == 0
    planes = out.view(37, 3, Kp).float()
    assert torch.all(planes[:, :, 100:] == 0)
    back = planes[:, 0, :100].double() + planes[:, 1, :100].double() + planes[:, 2, :100].double()
    assert ((back - x.double()).abs() <= x.double().abs() * 2.0 ** -24).all()
    xt = x.t().contiguous()  # [K, rows]
    out_t = torch.empty_like(out)
    assert L.xg_split_bf16x3(xt.data_ptr(), 37, 100, 37, 1, out_t.data_ptr(), None) == 0
    assert torch.equal(out_t, out)


def test_dense_fp32_weight_planes_follow_the_weight(cuda_device):
    """The bf16 planes of a weight are kept between calls; an in-place update of the weight must not reuse them."""
    x, w, b = _mk(2048, 512, 1024, torch.float32, 29)
    x, w = x.to(cuda_device), w.to(cuda_device)
    y1 = torch.ops.xg_sm100.dense(x, w, True, None, None, "none")
    w.mul_(2.0)
    y2 = torch.ops.xg_sm100.dense(x, w, True, None, None, "none")
    assert_parity(y2, (y1 * 2.0), "dense fp32 after an in-place weight update")


def test_dense_swiglu(cuda_device):
    from xpu_graph_b200 import lib
    from xpu_graph_b200.modules import DenseSwiGLUModule

    g = torch.Generator().manual_seed(25)
    M, K, N = 300, 512, 1376
    x = torch.randn(M, K, generator=g).to(torch.bfloat16)
    wg = (0.02 * torch.randn(N, K, generator=g)).to(torch.bfloat16)
    wu = (0.02 * torch.randn(N, K, generator=g)).to(torch.bfloat16)
    got = DenseSwiGLUModule()(x.to(cuda_device), wg.to(cuda_device), wu.to(cuda_device))
    torch.cuda.synchronize()
    assert lib.tc_status() == 0
    assert_parity(got, ref_ops.dense_swiglu(x, wg, wu), "dense_swiglu")


@pytest.mark.parametrize("B,S,H,D,K", [(2, 64, 2, 128, 256), (1, 200, 3, 64, 128), (2, 320, 4, 128, 512), (3, 33, 1, 64, 64)])
def test_dense_rope(cuda_device, B, S, H, D, K):
    """Projection with the rotary embedding in the epilogue == dense layer followed by the RoPE kernel (bit for
    bit: both round the projection to bf16 and rotate in fp32), and within tolerance of the eager chain."""
    from xpu_graph_b200 import lib
    from xpu_graph_b200.modules import DenseLayerModule, DenseRopeModule, RopeModule

    g = torch.Generator().manual_seed(41)
    x = torch.randn(B * S, K, generator=g).to(torch.bfloat16)
    w = (0.05 * torch.randn(H * D, K, generator=g)).to(torch.bfloat16)
    inv = 1.0 / (10000.0 ** (torch.arange(0, D, 2).float() / D))
    ang = torch.outer(torch.arange(S).float(), inv)
    emb = torch.cat((ang, ang), dim=-1)
    cos, sin = emb.cos().to(torch.bfloat16), emb.sin().to(torch.bfloat16)
    xd, wd, cd, sd = (t.to(cuda_device) for t in (x, w, cos, sin))
    got = DenseRopeModule()(xd, wd, cd, sd, B, S, H, D)
    two_step = RopeModule()(DenseLayerModule(False)(xd, wd, True, None, "none").view(B, S, H, D).transpose(1, 2), cd, sd)
    torch.cuda.synchronize()
    assert lib.tc_status() == 0
    assert got.shape == (B, H, S, D)
    assert torch.equal(got, two_step), "fused epilogue must equal dense + rope kernels bit for bit"
    want = ref_ops.rope(ref_ops.dense(x, w, True, None, "none").view(B, S, H, D).transpose(1, 2), cos, sin)
    assert_parity(got, want, f"dense_rope {B}x{S}x{H}x{D}")


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
@pytest.mark.parametrize("b,M,K,N,weight_trans,act,with_bias", [
    (3, 130, 64, 72, True, "gelu", True),      # ragged rows and columns
    (16, 256, 512, 384, True, "relu", True),   # many entries, one launch
    (5, 100, 200, 136, False, "none", True),   # weights given as [b, K, N]
    (2, 64, 4096, 128, True, "silu", False),   # deep K
    (1, 77, 64, 64, True, "none", True),       # a batch of one takes the 2-D path
])
def test_batch_dense(cuda_device, b, M, K, N, weight_trans, act, with_bias, dtype):
    from xpu_graph_b200 import lib, ops
    from xpu_graph_b200.modules import BatchDenseLayerModule

    g = torch.Generator().manual_seed(26)
    x = torch.randn(b, M, K, generator=g).to(dtype)
    w = (0.05 * torch.randn(b, N, K, generator=g)).to(dtype)
    if not weight_trans:
        w = w.transpose(1, 2).contiguous()
    bias = (0.05 * torch.randn(b, 1, N, generator=g)).to(dtype) if with_bias else None
    with LaunchCounter() as calls:
        got = BatchDenseLayerModule()(x.to(cuda_device), w.to(cuda_device), weight_trans,
                                      bias.to(cuda_device) if with_bias else None, act)
    torch.cuda.synchronize()
    assert calls.names == ["xg_bgemm_bias_act"]
    assert lib.tc_status() == 0
    if dtype == torch.float32:
        want = ref_ops.batch_dense(x.double(), w.double(), weight_trans, bias.double() if with_bias else None, act).float()
    else:
        want = ref_ops.batch_dense(x, w, weight_trans, bias, act)
    assert_parity(got, want, f"batch_dense {b}x{M}x{K}x{N} {dtype}")


@pytest.mark.parametrize("T,M,K,N,weight_trans,with_bias", [(6, 96, 128, 200, True, True), (14, 130, 264, 72, True, False),
                                                            (5, 256, 512, 384, False, True), (4, 64, 64, 1000, True, True)])
def test_combo_dense(cuda_device, T, M, K, N, weight_trans, with_bias):
    """T same-shape dense layers on separate tensors in one grouped launch (a pointer per layer: nothing is stacked or
    copied; 14 layers need two launches of at most 12 entries), both weight layouts, against the per-layer oracle."""
    from xpu_graph_b200 import lib
    from xpu_graph_b200.modules import ComboDenseModule

    g = torch.Generator().manual_seed(33)
    xs = [torch.randn(M, K, generator=g).to(torch.bfloat16) for _ in range(T)]
    ws = [(0.05 * torch.randn(N, K, generator=g)).to(torch.bfloat16) for _ in range(T)]
    if not weight_trans:
        ws = [w.t().contiguous() for w in ws]
    bs = [(0.05 * torch.randn(N, generator=g)).to(torch.bfloat16) if with_bias else None for _ in range(T)]
    want = torch.stack([ref_ops.dense(x, w, weight_trans, b, "relu") for x, w, b in zip(xs, ws, bs)])
    with LaunchCounter() as calls:
        got = ComboDenseModule()([x.to(cuda_device) for x in xs], [w.to(cuda_device) for w in ws],
                                 [b.to(cuda_device) if b is not None else None for b in bs], "relu", weight_trans)
    torch.cuda.synchronize()
    assert calls.names == ["xg_gemm_group_bias_act"], calls.names  # no stacking copy, no per-layer calls
    assert lib.tc_status() == 0
    assert_parity(got, want, f"combo_dense grouped T={T} {M}x{K}x{N}")


@pytest.mark.parametrize("T,M,K,N,weight_trans,bias_kind", [(8, 5, 8, 7, False, "matrix"), (8, 5, 8, 7, False, "row"),
                                                             (8, 5, 8, 7, True, "none"), (6, 40, 64, 48, True, "row"),
                                                             (30, 33, 100, 70, True, "matrix"), (5, 300, 256, 520, False, "row"),
                                                             (4, 1024, 192, 1024, True, "matrix"), (8, 256, 64, 256, True, "row"),
                                                             (5, 1024, 64, 1100, False, "matrix")])
def test_combo_dense_fp32(cuda_device, T, M, K, N, weight_trans, bias_kind):
    """fp32 layers in one grouped launch of the FMA kernels (the entry is the grid's third dimension; 30 layers need two
    launches of at most 24): the reference's own sizes (tests/mlu/test_combo_matmul.py:90-100: T = 8, 5 x 8 x 7, [K, N]
    weights, full-matrix or row biases) and sizes that reach each of the four kernel choices (two panel tiles, two tiled
    kernels), against fp64 math."""
    from xpu_graph_b200.modules import ComboDenseModule

    g = torch.Generator().manual_seed(34)
    xs = [torch.randn(M, K, generator=g) for _ in range(T)]
    ws = [0.05 * torch.randn(N, K, generator=g) for _ in range(T)]
    if not weight_trans:
        ws = [w.t().contiguous() for w in ws]
    if bias_kind == "none":
        bs = [None] * T
    else:
        bs = [0.05 * torch.randn((M, N) if bias_kind == "matrix" else (N,), generator=g) for _ in range(T)]
    want = []
    for x, w, b in zip(xs, ws, bs):
        y = x.double() @ (w.double().t() if weight_trans else w.double())
        want.append(torch.relu(y if b is None else y + b.double()).float())
    with LaunchCounter() as calls:
        got = ComboDenseModule()([x.to(cuda_device) for x in xs], [w.to(cuda_device) for w in ws],
                                 [b.to(cuda_device) if b is not None else None for b in bs], "relu", weight_trans)
    torch.cuda.synchronize()
    assert calls.names == ["xg_gemm_group_bias_act"], calls.names
    assert_parity(got, torch.stack(want), f"combo_dense fp32 grouped T={T} {M}x{K}x{N} {bias_kind}")


def test_combo_dense_full_matrix_biases_16bit(cuda_device):
    """Full [M, N] addends per layer (the addmm(bias, x, w) form of tests/mlu/test_combo_matmul.py:33-39) ride in the
    grouped tensor-core kernel's epilogue as per-entry residuals; layers may mix them with none."""
    from xpu_graph_b200 import lib
    from xpu_graph_b200.modules import ComboDenseModule

    g = torch.Generator().manual_seed(35)
    T, M, K, N = 13, 130, 264, 200
    xs = [torch.randn(M, K, generator=g).to(torch.bfloat16) for _ in range(T)]
    ws = [(0.05 * torch.randn(N, K, generator=g)).to(torch.bfloat16) for _ in range(T)]
    bs = [torch.randn(M, N, generator=g).to(torch.bfloat16) for _ in range(T)]
    want = torch.stack([torch.relu(x.float() @ w.float().t() + b.float()) for x, w, b in zip(xs, ws, bs)]).to(torch.bfloat16)
    with LaunchCounter() as calls:
        got = ComboDenseModule()([x.to(cuda_device) for x in xs], [w.to(cuda_device) for w in ws], [b.to(cuda_device) for b in bs],
                                 "relu", True)
    torch.cuda.synchronize()
    assert calls.names == ["xg_gemm_group_bias_act"] and lib.tc_status() == 0
    assert_parity(got, want, "combo_dense bf16 with [M, N] addends", magnitude=torch.stack(bs))


def _chain_reference(x, ws, bs, acts, kn, dtype):
    """Layer by layer in fp64 with the hidden activation rounded to `dtype` once per layer (what the chained kernels do)."""
    y = x.double()
    for i, (w, b, a) in enumerate(zip(ws, bs, acts)):
        y = y @ (w.double() if kn[i] else w.double().t())
        if b is not None:
            y = y + b.double()
        y = ref_ops._ACTS[a](y.float()).double()
        y = y.to(dtype).double()
    return y.to(dtype)


@pytest.mark.parametrize("dtype,M,dims,kn,acts", [
    (torch.float16, 16, (20, 32, 16, 1), (True, True, True), ("relu", "relu", "none")),
    (torch.float32, 1000, (64, 128, 32, 8), (False, False, False), ("relu", "gelu", "none")),
    (torch.bfloat16, 4097, (100, 128, 64), (False, True), ("silu", "sigmoid")),
    (torch.float32, 33, (7, 5, 3), (True, False), ("none", "relu")),
    (torch.bfloat16, 300, (13, 50), (False,), ("gelu",)),
    (torch.float32, 70000, (128, 128, 64), (False, False), ("relu", "none"))])
def test_mlp_small(cuda_device, dtype, M, dims, kn, acts):
    """One to three narrow layers with the weights resident in shared memory: the reference's own tower (16 rows of
    20 -> 32 -> 16 -> 1 in fp16 with [K, N] weights, tests/mlu/test_fuse_densetower.py:36-53), both weight layouts,
    widths that are no multiple of anything, the widest case the kernel takes, more row blocks than CTAs."""
    from xpu_graph_b200 import ops  # noqa: F401  (registers the ops)

    g = torch.Generator().manual_seed(37)
    x = torch.randn(M, dims[0], generator=g).to(dtype)
    ws, bs = [], []
    for i in range(len(dims) - 1):
        w = (torch.randn(dims[i + 1], dims[i], generator=g) * dims[i] ** -0.5).to(dtype)
        ws.append(w.t().contiguous() if kn[i] else w)
        bs.append(None if i == 1 else (0.3 * torch.randn(dims[i + 1], generator=g)).to(dtype))
    want = _chain_reference(x, ws, bs, acts, kn, dtype)
    kn_bits = sum(1 << i for i, f in enumerate(kn) if f)
    with LaunchCounter() as calls:
        got = torch.ops.xg_sm100.mlp_small(x.to(cuda_device), [w.to(cuda_device) for w in ws],
                                           [b.to(cuda_device) if b is not None else None for b in bs], ",".join(acts), kn_bits)
    torch.cuda.synchronize()
    assert calls.names == ["xg_mlp_small_bias_act"], calls.names
    assert_parity(got, want, f"mlp_small {dtype} M={M} {dims}")


def test_dense_tower_module_takes_the_small_kernel(cuda_device):
    """DenseTowerModule on the reference's tower: one launch, for fp16 as in its test and for fp32."""
    from xpu_graph_b200.modules import DenseTowerModule

    g = torch.Generator().manual_seed(38)
    dims = (20, 32, 16, 1)
    for dtype in (torch.float16, torch.float32):
        x = torch.randn(16, dims[0], generator=g).to(dtype)
        ws = [(torch.randn(dims[i], dims[i + 1], generator=g) * dims[i] ** -0.5).to(dtype) for i in range(3)]
        bs = [torch.randn(dims[i + 1], generator=g).to(dtype) for i in range(3)]
        acts = ["relu", "relu", "none"]
        with LaunchCounter() as calls:
            got = DenseTowerModule()(x.to(cuda_device), [w.to(cuda_device) for w in ws], [False] * 3, [b.to(cuda_device) for b in bs], acts)
        torch.cuda.synchronize()
        assert calls.names == ["xg_mlp_small_bias_act"], calls.names
        assert_parity(got, _chain_reference(x, ws, bs, acts, (True, True, True), dtype), f"dense tower {dtype} {dims}")


@pytest.mark.parametrize("M,K,N,weight_trans,act", [(128, 5897, 5897, True, "gelu"), (50, 444, 300, False, "relu"), (7, 20, 1, False, "none"),
                                                    (2048, 100, 2564, True, "silu"), (2100, 36, 2564, False, "none")])
def test_dense_16bit_rows_no_tensor_map_addresses(cuda_device, M, K, N, weight_trans, act):
    """16-bit dense layers whose rows are not multiples of 16 bytes (the sizes of tests/mlu/test_custom_denselayer.py run
    in 16-bit: K = 5897, 444) run on the library's FMA kernel: bias, residual and activation fused as everywhere else."""
    from xpu_graph_b200.modules import DenseLayerModule, can_fuse_custom_denselayer

    x, w, b = _mk(M, K, N, torch.bfloat16, 39)
    if not weight_trans:
        w = w.t().contiguous()
    # the pattern's constraint sends only small layers of this kind here (a large one is left to the vendor matmul);
    # the module itself takes either
    assert can_fuse_custom_denselayer(x.to(cuda_device), w.to(cuda_device), weight_trans, b.to(cuda_device), act) == (2 * M * K * N <= 1 << 26)
    with LaunchCounter() as calls:
        got = DenseLayerModule(False)(x.to(cuda_device), w.to(cuda_device), weight_trans, b.to(cuda_device), act)
    torch.cuda.synchronize()
    assert calls.names == ["xg_gemm_bias_act_ws"] or calls.names == ["xg_gemm_bias_act"], calls.names
    assert_parity(got, ref_ops.dense(x, w, weight_trans, b, act), f"dense bf16 unaligned {M}x{K}x{N}")


@pytest.mark.parametrize("dtype,T,S,M,K,N,weight_trans,bias_kind", [
    (torch.float32, 8, 3, 5, 6, 7, False, "full"), (torch.float32, 8, 3, 5, 6, 7, False, "none"),
    (torch.float32, 5, 4, 33, 64, 48, True, "row"), (torch.bfloat16, 6, 4, 64, 128, 96, True, "full"),
    (torch.bfloat16, 4, 5, 40, 64, 200, False, "row")])
def test_combo_batch_dense(cuda_device, dtype, T, S, M, K, N, weight_trans, bias_kind):
    """Lists of bmm in one grouped launch over the T * S products (a pointer per product; the shared input of the
    reference's form, tests/mlu/test_combo_matmul.py:25-30 and 102-109, is read in place by every member), against
    fp64 math."""
    from xpu_graph_b200 import lib
    from xpu_graph_b200.modules import ComboBatchDenseModule

    g = torch.Generator().manual_seed(36)
    x = torch.randn(S, M, K, generator=g).to(dtype)
    ws = [(0.1 * torch.randn(S, N, K, generator=g)).to(dtype) for _ in range(T)]
    if not weight_trans:
        ws = [w.transpose(1, 2).contiguous() for w in ws]
    shape = {"full": (S, M, N), "row": (S, 1, N)}.get(bias_kind)
    bs = [torch.randn(shape, generator=g).to(dtype) if shape else None for _ in range(T)]
    want = []
    for w, b in zip(ws, bs):
        y = torch.bmm(x.double(), w.double().transpose(1, 2) if weight_trans else w.double())
        want.append(torch.relu(y if b is None else y + b.double()).to(dtype))
    xd = x.to(cuda_device)
    with LaunchCounter() as calls:
        got = ComboBatchDenseModule()([xd] * T, [w.to(cuda_device) for w in ws],
                                      [b.to(cuda_device) if b is not None else None for b in bs], "relu", weight_trans)
    torch.cuda.synchronize()
    assert set(calls.names) == {"xg_gemm_group_bias_act"} and lib.tc_status() == 0, calls.names
    mag = torch.stack([b.broadcast_to((S, M, N)) for b in bs]) if shape else None
    assert_parity(got, torch.stack(want), f"combo_batch_dense {dtype} T={T} S={S} {M}x{K}x{N} {bias_kind}", magnitude=mag)


def test_combo_dense_fallback_to_the_batched_form(cuda_device):
    """Layers the grouped kernels cannot address (16-bit rows that are not multiples of 16 bytes) go through the batched
    entry point: separate tensors are stacked, slabs of one buffer are used in place."""
    from xpu_graph_b200 import ops
    from xpu_graph_b200.modules import ComboDenseModule

    g = torch.Generator().manual_seed(34)
    T, M, K, N = 4, 40, 64, 48
    xs = [torch.randn(M, K, generator=g) for _ in range(T)]
    xcat = torch.stack(xs).to(cuda_device)
    assert ops._stack_or_view(list(xcat.unbind(0))).data_ptr() == xcat.data_ptr()  # no copy for slabs of one buffer
    xs16 = [x.to(torch.bfloat16) for x in xs]
    ws16 = [(0.05 * torch.randn(N, K, generator=g)).to(torch.bfloat16) for _ in range(T)]
    bs16 = [(0.05 * torch.randn(N, generator=g)).to(torch.bfloat16) for _ in range(T)]
    want = torch.stack([ref_ops.dense(x, w, True, b, "relu") for x, w, b in zip(xs16, ws16, bs16)])
    pad = torch.zeros(T, M, K + 4, dtype=torch.bfloat16, device=cuda_device)  # rows of 136 bytes: no tensor map for them
    pad[:, :, :K] = torch.stack(xs16).to(cuda_device)
    with LaunchCounter() as calls:
        got = ComboDenseModule()([pad[i, :, :K] for i in range(T)], [w.to(cuda_device) for w in ws16],
                                 [b.to(cuda_device) for b in bs16], "relu", True)
    assert "xg_gemm_group_bias_act" not in calls.names, calls.names
    assert_parity(got, want, "combo_dense (batched form)")


@pytest.mark.parametrize("act", ["gelu", "silu"])
@pytest.mark.parametrize("N", [4096, 11008])
@pytest.mark.parametrize("M", [256, 4096, 16384])
def test_config3_cell(cuda_device, M, N, act):
    """Every full-size cell of the matmul sweep (M in {256, 4096, 16384} x K = 4096 x N in {4096, 11008}, GELU and
    SiLU, seed 2): sampled rows against the oracle (first / last row, both sides of every kind of tile edge) plus
    linearity in the bias (out(b) - out(0) == b before the activation). The M = 256 cells run the cluster kernel
    that splits K, the others the CTA-pair kernel."""
    from xpu_graph_b200 import lib
    from xpu_graph_b200.modules import DenseLayerModule

    K = 4096
    g = torch.Generator(device=cuda_device).manual_seed(2)
    x = torch.randn(M, K, generator=g, device=cuda_device, dtype=torch.bfloat16)
    w = (0.02 * torch.randn(N, K, generator=g, device=cuda_device)).to(torch.bfloat16)
    b = (0.02 * torch.randn(N, generator=g, device=cuda_device)).to(torch.bfloat16)
    got = DenseLayerModule(False)(x, w, True, b, act)
    torch.cuda.synchronize()
    assert lib.tc_status() == 0
    rows = sorted({0, 1, 127, 128, 255, M // 2 + 1, M - 129, M - 1} & set(range(M)))
    sel = torch.tensor(rows, device=cuda_device)
    want = ref_ops.dense(x[sel].cpu(), w.cpu(), True, b.cpu(), act)
    assert_parity(got[sel], want, f"config-3 cell {M}x{K}x{N} {act}")
    exact = ref_ops.dense(x[sel].cpu().float(), w.cpu().float(), True, b.cpu().float(), act)
    max_abs, mean_rel = error_stats(got[sel], exact)
    print(f"config-3 cell {M}x{K}x{N} {act}: max_abs={max_abs:.3g} mean_rel={mean_rel:.3g} vs fp32 math")
    if act == "gelu":
        lin = DenseLayerModule(False)(x, w, True, None, "none")
        lin_b = DenseLayerModule(False)(x, w, True, b, "none")
        assert ((lin_b.float() - lin.float()) - b.float()).abs().max().item() < 0.05
