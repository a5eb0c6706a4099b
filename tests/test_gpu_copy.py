"""GPU parity (bit-exact): slice/cat/stack/gather/where copy fusions through the C ABI vs the numpy oracle.

Cases follow the reference's slice-fusion tests (tests/mlu/test_fuse_slice.py, test_fuse_slice_cat.py,
test_fuse_slice_where_cat.py): many equal slices of a wide 2-D source, INT64_MAX and negative ends,
ragged widths, N-D sources for the multi-slice form.
"""
import pytest
import torch

from oracle import ref_ops
from tests.helpers import assert_bit_exact

pytestmark = pytest.mark.gpu

MAX_INT64 = 9223372036854775807


def _src(rows, width, dtype, seed=10):
    g = torch.Generator().manual_seed(seed)
    if dtype in (torch.int64, torch.int32):
        return torch.randint(-1000, 1000, (rows, width), generator=g, dtype=dtype)
    return torch.randn(rows, width, generator=g).to(dtype)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.int64])
@pytest.mark.parametrize(
    "rows,width,slices",
    [
        (16384 // 64, 64, [(4 * ((5 * i) % 16), 4 * ((5 * i) % 16) + 4) for i in range(16)]),  # config-5 shape, permuted groups
        (512, 4310, [(32 * i + 3, 32 * i + 35) for i in range(25)]),  # odd starts: 4-byte units
        (512, 4310, [(64 * i, 64 * i + 64) for i in range(13)]),
        (7, 100, [(0, 1), (99, 100), (10, 57)]),
        (5, 40, [(0, MAX_INT64), (10, -3), (0, 40)]),
        (1, 9000, [(0, 9000), (1, 8999)]),  # wider than one look-up table
        (3, 1, [(0, 1)] * 70),  # more segments than one launch carries
        (0, 16, [(0, 8), (8, 16)]),  # empty
    ],
)
def test_slice_cat(cuda_device, rows, width, slices, dtype):
    from xpu_graph_b200.modules import FuseSliceCatSameInputModule

    src = _src(rows, width, dtype)
    got = FuseSliceCatSameInputModule()(src.to(cuda_device), slices)
    assert_bit_exact(got, ref_ops.slice_cat(src, slices), f"slice_cat {rows}x{width}")


def test_slice_cat_rejects_non_2d(cuda_device):
    from xpu_graph_b200.modules import FuseSliceCatSameInputModule

    with pytest.raises(NotImplementedError):
        FuseSliceCatSameInputModule()(torch.zeros(2, 3, 4, device=cuda_device), [(0, 1), (1, 2)])


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("shape,starts,length", [((86, 1000), [0, 100, 37, 900], 64), ((4, 9, 128), [0, 16, 32, 3], 16), ((16384, 64), list(range(0, 64, 4)), 4)])
def test_multi_slice(cuda_device, shape, starts, length, dtype):
    from xpu_graph_b200.modules import FuseSliceModule

    g = torch.Generator().manual_seed(11)
    src = torch.randn(*shape, generator=g).to(dtype)
    got = FuseSliceModule(starts)(src.to(cuda_device), length)
    assert_bit_exact(got, ref_ops.multi_slice(src, starts, length), f"multi_slice {shape}")


def test_slice_cat_multi(cuda_device):
    from xpu_graph_b200.modules import FuseSliceCatSameInputModule_v2

    src = _src(300, 777, torch.float32)
    many = [[(0, 32), (100, 164)], [(5, 6)], [(700, 777), (0, 16), (300, 420)]]
    got = FuseSliceCatSameInputModule_v2(many)(src.to(cuda_device), many)
    want = ref_ops.slice_cat_multi(src, many)
    assert len(got) == len(want)
    for k, (a, b) in enumerate(zip(got, want)):
        assert_bit_exact(a, b, f"slice_cat_multi output {k}")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_masked_slice_cat(cuda_device, dtype):
    from xpu_graph_b200.modules import MaskedSliceCatModule

    src = _src(257, 640, dtype)
    g = torch.Generator().manual_seed(12)
    mask = torch.rand(257, 1, generator=g) < 0.3
    slices = [(64 * i, 64 * i + 32) for i in range(10)]
    got = MaskedSliceCatModule()(src.to(cuda_device), mask.to(cuda_device), slices)
    assert_bit_exact(got, ref_ops.masked_slice_cat(src, mask, slices), "masked slice_cat")


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16])
def test_partly_masked_slice_cat_and_stack(cuda_device, dtype):
    """Slices of one source where only some take the row mask, concatenated (MaskedSliceCatModule with flags) or stacked
    along a new leading dim (MaskedSliceStackModule): bit-exact against slicing, masking and joining on CPU."""
    from xpu_graph_b200.modules import MaskedSliceCatModule, MaskedSliceStackModule

    src = _src(513, 1200, dtype)
    g = torch.Generator().manual_seed(14)
    mask = torch.rand(513, 1, generator=g) < 0.4
    slices = [(0, 32), (700, 731), (64, 96), (1100, 1200), (5, 6)]
    flags = [False, True, True, False, True]
    want = torch.cat([torch.where(mask, torch.zeros((), dtype=dtype), src[:, a:b]) if f else src[:, a:b] for (a, b), f in zip(slices, flags)], dim=-1)
    got = MaskedSliceCatModule()(src.to(cuda_device), mask.to(cuda_device), slices, flags)
    assert_bit_exact(got, want, "partly masked slice_cat")
    starts, L = [0, 1001, 37, 640], 24
    sflags = [False, True, True, True]
    want = torch.stack([torch.where(mask, torch.zeros((), dtype=dtype), src[:, a:a + L]) if f else src[:, a:a + L] for a, f in zip(starts, sflags)], dim=0)
    got = MaskedSliceStackModule()(src.to(cuda_device), mask.to(cuda_device), starts, L, sflags)
    assert_bit_exact(got, want, "partly masked slice stack")


def test_cat_and_stack(cuda_device):
    from xpu_graph_b200.modules import CatLastDimModule

    g = torch.Generator().manual_seed(13)
    xs = [torch.randn(129, w, generator=g) for w in (64, 3, 1000, 64)]
    got = CatLastDimModule()([x.to(cuda_device) for x in xs])
    assert_bit_exact(got, ref_ops.cat_lastdim(xs), "cat")
    es = [torch.randn(200, 64, generator=g).to(torch.bfloat16) for _ in range(26)]
    got = CatLastDimModule()([e.to(cuda_device) for e in es]).view(200, 26, 64)
    assert_bit_exact(got, torch.stack(es, dim=1), "stack dim 1")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("rows,F,D,table_rows,masked", [(1000, 26, 64, 5000, True), (33, 3, 7, 11, False), (16384, 26, 64, 100000, True), (0, 2, 8, 4, False)])
def test_gather_stack(cuda_device, rows, F, D, table_rows, masked, dtype):
    from xpu_graph_b200.modules import GatherStackModule

    g = torch.Generator().manual_seed(14)
    tables = [(0.01 * torch.randn(table_rows, D, generator=g)).to(dtype) for _ in range(F)]
    idx = torch.randint(0, table_rows, (rows, F), generator=g, dtype=torch.int64)
    mask = (torch.rand(rows, 1, generator=g) < 0.3) if masked else None
    got = GatherStackModule()([t.to(cuda_device) for t in tables], idx.to(cuda_device), mask.to(cuda_device) if masked else None)
    assert_bit_exact(got, ref_ops.gather_stack(tables, idx, mask), f"gather_stack {rows}x{F}x{D}")


def test_gather_strided_index(cuda_device):
    """Index matrix given as a transposed view (column-major strides)."""
    from xpu_graph_b200.modules import GatherStackModule

    g = torch.Generator().manual_seed(15)
    tables = [torch.randn(50, 16, generator=g) for _ in range(4)]
    idx_t = torch.randint(0, 50, (4, 300), generator=g, dtype=torch.int64)
    got = GatherStackModule()([t.to(cuda_device) for t in tables], idx_t.to(cuda_device).t())
    assert_bit_exact(got, ref_ops.gather_stack(tables, idx_t.t().contiguous(), None), "gather strided idx")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("dim", [0, 1, 2])
def test_combo_sum(cuda_device, dim, dtype):
    """Batched sum over one dim of several 3-D tensors (ComboSum3dInp), ragged shapes incl. an empty one."""
    from tests.helpers import assert_parity
    from xpu_graph_b200.modules import ComboSumModule

    g = torch.Generator().manual_seed(16)
    shapes = [(300, 26, 64), (7, 3, 5), (129, 64, 8), (1, 1, 1), (50, 33, 100), (0, 4, 4)]
    xs = [torch.randn(*s, generator=g).to(dtype) for s in shapes]
    got = ComboSumModule()([x.to(cuda_device) for x in xs], [dim])
    want = ref_ops.combo_sum([x.float() for x in xs], [dim])
    assert len(got) == len(want)
    for a, e in zip(got, want):
        assert_parity(a, e.to(dtype), f"combo_sum dim {dim}")
