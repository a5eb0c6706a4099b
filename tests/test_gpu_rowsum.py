"""GPU parity: slice -> sum -> cat, sum -> cat and mul -> sum -> cat through the C ABI (xg_rowsum_cat) vs the oracle.

Shapes follow the reference's tests (tests/mlu/test_fuse_sum_cat.py, test_mul_sum_cat.py): a [batch, rows, C]
source cut into row ranges that start at row 0, pairs of equally shaped operands with a broadcast batch, and the
recsys sizes of the benchmark graph (batch 16384, 64-wide rows). fp32 within 1e-5 (the summation order differs
from eager's), 16-bit types within the bf16 tolerance; sums that cancel are judged against the summed magnitudes.
"""
import pytest
import torch

from oracle import ref_ops
from tests.helpers import assert_parity

pytestmark = pytest.mark.gpu


def _rand(shape, dtype, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randn(*shape, generator=g).to(dtype)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
@pytest.mark.parametrize(
    "shape,slices",
    [
        ((64, 50, 64), [(0, 10), (0, 25), (0, 50), (0, 4)]),           # prefix ranges, unsorted ends: one walk
        ((64, 50, 64), [(3, 10), (0, 25), (12, 50)]),                  # different first rows: one segment per range
        ((16384, 26, 64), [(0, 13), (0, 26)]),                         # benchmark batch
        ((33, 17, 5), [(0, 17), (0, 1), (0, 9)]),                      # row length without a 16-byte vector
        ((2, 300, 8), [(0, i + 1) for i in range(70)]),                # more ranges than one launch carries
        ((5, 12, 16), [(0, 0), (0, 12), (4, 4)]),                      # empty ranges give zeros
        ((0, 12, 16), [(0, 6), (0, 12)]),                              # empty batch
    ],
)
def test_slice_sum_cat(cuda_device, shape, slices, dtype):
    from xpu_graph_b200.modules import SliceSumCatModule

    x = _rand(shape, dtype, 21)
    got = SliceSumCatModule(slices)(x.to(cuda_device))
    want = ref_ops.slice_sum_cat(x.float(), slices).to(dtype)
    mag = ref_ops.slice_sum_cat(x.float().abs(), slices)
    assert_parity(got, want, f"slice_sum_cat {shape} {dtype}", magnitude=mag * (1e-2 if dtype != torch.float32 else 1e-3))


def test_slice_sum_cat_negative_and_open_ends(cuda_device):
    from xpu_graph_b200.modules import SliceSumCatModule

    x = _rand((7, 20, 16), torch.float32, 22)
    slices = [(0, 9223372036854775807), (0, -3), (-5, 20)]
    got = SliceSumCatModule(slices)(x.to(cuda_device))
    want = ref_ops.slice_sum_cat(x, slices)
    assert_parity(got, want, "slice_sum_cat open ends")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("batch,rows,C,n,bcast", [(64, 5, 8, 2, ()), (16384, 10, 64, 3, (1,)), (9, 7, 3, 5, (0, 4)), (1, 4, 16, 2, ())])
def test_mul_sum_cat(cuda_device, batch, rows, C, n, bcast, dtype):
    from xpu_graph_b200.modules import MulSumCatModule

    ml = []
    for k in range(n):
        ml.append(_rand((batch, rows, C), dtype, 30 + k))
        ml.append(_rand((1 if k in bcast else batch, rows, C), dtype, 40 + k))
    got = MulSumCatModule()([t.to(cuda_device) for t in ml])
    want = ref_ops.mul_sum_cat([t.float() for t in ml]).to(dtype)
    mag = ref_ops.mul_sum_cat([t.float().abs() for t in ml])
    assert_parity(got, want, f"mul_sum_cat {batch}x{rows}x{C} n={n} {dtype}", magnitude=mag * (1e-2 if dtype != torch.float32 else 1e-3))


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16])
def test_sum_cat(cuda_device, dtype):
    from xpu_graph_b200.modules import SumCatModule

    xs = [_rand((128, r, 32), dtype, 50 + r) for r in (3, 1, 40, 7)]
    got = SumCatModule()([t.to(cuda_device) for t in xs])
    want = ref_ops.sum_cat([t.float() for t in xs]).to(dtype)
    mag = ref_ops.sum_cat([t.float().abs() for t in xs])
    assert_parity(got, want, f"sum_cat {dtype}", magnitude=mag * (1e-2 if dtype != torch.float32 else 1e-3))


def test_rowsum_cat_rejects_bad_arguments(cuda_device):
    import ctypes

    from xpu_graph_b200 import lib

    L = lib.load()
    x = torch.zeros(2, 4, 8, device=cuda_device)
    out = torch.zeros(2, 8, device=cuda_device)
    a = lib.ptr_array([x.data_ptr()])
    bs = lib.i64_array([32])
    assert L.xg_rowsum_cat(a, None, bs, None, lib.i64_array([3, 2]), 1, 2, 8, out.data_ptr(), 8, 0, None) == -1  # r1 < r0
    assert L.xg_rowsum_cat(a, None, bs, None, lib.i64_array([0, 4]), 1, 2, 8, out.data_ptr(), 4, 0, None) == -1  # out_ld < n*C
    assert L.xg_rowsum_cat(a, a, bs, None, lib.i64_array([0, 4]), 1, 2, 8, out.data_ptr(), 8, 0, None) == -1      # strides missing
    assert L.xg_rowsum_cat(a, None, bs, None, lib.i64_array([0, 4]), 1, 2, 8, out.data_ptr(), 8, 9, None) == -1   # dtype
    assert b"xg_rowsum_cat" in ctypes.c_char_p(L.xg_last_error()).value


@pytest.mark.parametrize("tag", ["f32", "bf16"])
def test_against_reference_fixtures(cuda_device, tag):
    """The same graphs as recorded from the reference's own pipeline (tests/golden/golden_v2.pt)."""
    import os

    from xpu_graph_b200.modules import MulSumCatModule, SliceSumCatModule, SumCatModule

    G = torch.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "golden_v2.pt"))
    for name in ("prefix", "general"):
        c = G[f"slice_sum_cat_{name}_{tag}"]
        got = SliceSumCatModule(c["slices"])(c["x"].to(cuda_device))
        mag = ref_ops.slice_sum_cat(c["x"].float().abs(), c["slices"]) * (1e-2 if tag == "bf16" else 1e-3)
        assert_parity(got, c["y"], f"fixture slice_sum_cat {name} {tag}", magnitude=mag)
    c = G[f"mul_sum_cat_{tag}"]
    ml = []
    for a, b in zip(c["a"], c["b"]):
        ml += [a.to(cuda_device), b.to(cuda_device)]
    mag = ref_ops.mul_sum_cat([t.float().abs().cpu() for t in ml]) * (1e-2 if tag == "bf16" else 1e-3)
    assert_parity(MulSumCatModule()(ml), c["y"], f"fixture mul_sum_cat {tag}", magnitude=mag)
    c = G[f"sum_cat_{tag}"]
    mag = ref_ops.sum_cat([t.float().abs() for t in c["xs"]]) * (1e-2 if tag == "bf16" else 1e-3)
    assert_parity(SumCatModule()([t.to(cuda_device) for t in c["xs"]]), c["y"], f"fixture sum_cat {tag}", magnitude=mag)
