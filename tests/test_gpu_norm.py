"""GPU parity: fused (residual +) RMSNorm / LayerNorm through the C ABI vs the CPU oracle."""
import pytest
import torch

from oracle import ref_ops
from tests.helpers import assert_bit_exact, assert_parity

pytestmark = pytest.mark.gpu

SHAPES = [(1, 8), (3, 24), (33, 1000), (32, 1024), (31, 1032), (64, 4096), (17, 8192), (5, 16384), (2, 40000), (7, 250)]


def _mk(rows, hidden, dtype, seed):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(rows, hidden, generator=g).to(dtype)
    r = torch.randn(rows, hidden, generator=g).to(dtype)
    w = (1.0 + 0.1 * torch.randn(hidden, generator=g)).to(dtype)
    b = (0.1 * torch.randn(hidden, generator=g)).to(dtype)
    return x, r, w, b


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32, torch.float16])
@pytest.mark.parametrize("rows,hidden", SHAPES)
def test_rms_norm(cuda_device, rows, hidden, dtype):
    from xpu_graph_b200.modules import RMSNormModule

    x, _, w, _ = _mk(rows, hidden, dtype, 1)
    got = RMSNormModule()(x.to(cuda_device), w.to(cuda_device), 1e-6)
    assert_parity(got, ref_ops.rms_norm(x, w, 1e-6), f"rms_norm {rows}x{hidden} {dtype}")


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("rows,hidden", SHAPES)
def test_layer_norm(cuda_device, rows, hidden, dtype):
    from xpu_graph_b200.modules import LayerNormModule

    x, _, w, b = _mk(rows, hidden, dtype, 2)
    got = LayerNormModule()(x.to(cuda_device), w.to(cuda_device), b.to(cuda_device), 1e-5)
    assert_parity(got, ref_ops.layer_norm(x, w, b, 1e-5), f"layer_norm {rows}x{hidden} {dtype}")


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
@pytest.mark.parametrize("rows,hidden", [(8, 1024), (33, 1000), (5, 8192)])
def test_layer_norm_without_bias(cuda_device, rows, hidden, dtype):
    """layer_norm(x, weight, bias=None), alone and behind a residual add with one and two outputs: the configuration of
    the reference's residual-add test (tests/mlu/test_fuse_addlayernorm.py:39-43: [8, 1024], bias = None)."""
    from xpu_graph_b200.modules import AddLayerNormModule, LayerNormModule

    x, r, w, _ = _mk(rows, hidden, dtype, 6)
    xd, rd, wd = (t.to(cuda_device) for t in (x, r, w))
    assert_parity(LayerNormModule()(xd, wd, None, 1e-5), ref_ops.layer_norm(x, w, None, 1e-5), "layer_norm, no bias")
    want_y, want_s = ref_ops.add_layer_norm(x, r, w, None, 1e-5)
    assert_parity(AddLayerNormModule(False)(xd, rd, wd, None, 1e-5), want_y, "add_layer_norm, no bias")
    y, s = AddLayerNormModule(True)(xd, rd, wd, None, 1e-5)
    assert_parity(y, want_y, "add_layer_norm (2 outputs), no bias")
    assert_bit_exact(s, want_s, "add_layer_norm sum, no bias")


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("rows,hidden", [(4, 64), (33, 1000), (64, 4096), (9, 8192), (3, 16384)])
@pytest.mark.parametrize("store_sum", [False, True])
def test_add_norms(cuda_device, rows, hidden, dtype, store_sum):
    from xpu_graph_b200.modules import AddLayerNormModule, AddRMSNormModule

    x, r, w, b = _mk(rows, hidden, dtype, 3)
    xd, rd, wd, bd = (t.to(cuda_device) for t in (x, r, w, b))
    want_y, want_s = ref_ops.add_rms_norm(x, r, w, 1e-6)
    got = AddRMSNormModule(store_sum)(xd, rd, wd, 1e-6)
    if store_sum:
        assert_parity(got[0], want_y, "add_rms_norm y")
        assert_bit_exact(got[1], want_s, "add_rms_norm sum")  # the sum is a plain rounded add
    else:
        assert_parity(got, want_y, "add_rms_norm y")
    want_y, want_s = ref_ops.add_layer_norm(x, r, w, b, 1e-5)
    got = AddLayerNormModule(store_sum)(xd, rd, wd, bd, 1e-5)
    if store_sum:
        assert_parity(got[0], want_y, "add_layer_norm y")
        assert_bit_exact(got[1], want_s, "add_layer_norm sum")
    else:
        assert_parity(got, want_y, "add_layer_norm y")


def test_fp32_weights_and_strided_rows(cuda_device):
    """bf16 activations with fp32 affine parameters, and a row-strided (sliced) input."""
    from xpu_graph_b200.modules import LayerNormModule, RMSNormModule

    g = torch.Generator().manual_seed(4)
    big = torch.randn(40, 2048 + 64, generator=g).to(torch.bfloat16)
    x = big[:, :2048]  # row stride 2112, last dim contiguous
    w = 1.0 + 0.1 * torch.randn(2048, generator=g)
    b = 0.1 * torch.randn(2048, generator=g)
    got = RMSNormModule()(big.to(cuda_device)[:, :2048], w.to(cuda_device), 1e-6)
    assert_parity(got, ref_ops.rms_norm(x, w, 1e-6), "rms_norm fp32 weight strided")
    got = LayerNormModule()(big.to(cuda_device)[:, :2048], w.to(cuda_device), b.to(cuda_device), 1e-5)
    assert_parity(got, ref_ops.layer_norm(x, w, b, 1e-5), "layer_norm fp32 weight strided")


def test_3d_input_and_determinism(cuda_device):
    from xpu_graph_b200.modules import RMSNormModule

    g = torch.Generator().manual_seed(5)
    x = torch.randn(2, 37, 4096, generator=g).to(torch.bfloat16)
    w = (1.0 + 0.1 * torch.randn(4096, generator=g)).to(torch.bfloat16)
    xd, wd = x.to(cuda_device), w.to(cuda_device)
    outs = [RMSNormModule()(xd, wd, 1e-6) for _ in range(3)]
    assert outs[0].shape == x.shape
    assert_parity(outs[0], ref_ops.rms_norm(x, w, 1e-6), "rms_norm 3d")
    assert_bit_exact(outs[1], outs[0], "determinism")
    assert_bit_exact(outs[2], outs[0], "determinism")


def test_config2_full_size_properties(cuda_device):
    """Full-size cell of the norm sweep (65536 x 8192 bf16): checked through size-independent
    properties — per-row RMS of y/w is 1, and a sampled set of rows matches the oracle."""
    from xpu_graph_b200.modules import AddRMSNormModule

    rows, hidden = 65536, 8192
    g = torch.Generator(device=cuda_device).manual_seed(1)
    x = torch.randn(rows, hidden, generator=g, device=cuda_device, dtype=torch.bfloat16)
    r = torch.randn(rows, hidden, generator=g, device=cuda_device, dtype=torch.bfloat16)
    w = (1.0 + 0.1 * torch.randn(hidden, generator=g, device=cuda_device)).to(torch.bfloat16)
    y, s = AddRMSNormModule(True)(x, r, w, 1e-6)
    sel = torch.tensor([0, 1, 4095, 32768, 65535], device=cuda_device)
    want_y, want_s = ref_ops.add_rms_norm(x[sel].cpu(), r[sel].cpu(), w.cpu(), 1e-6)
    assert_parity(y[sel], want_y, "full-size rows")
    assert_bit_exact(s[sel], want_s, "full-size sum rows")
    rms = (y.float() / w.float()).pow(2).mean(dim=1).sqrt()
    assert (rms - 1.0).abs().max().item() < 2e-2


@pytest.mark.parametrize("store_sum", [False, True])
def test_config2_full_size_layer_norm(cuda_device, store_sum):
    """Full-size LayerNorm + residual cell of the norm sweep (65536 x 8192 bf16, seed 1), with one output and with
    the sum as second output: sampled rows against the oracle (the sum bit-exact) and, over the whole tensor, the
    property that (y - beta) / gamma has zero mean and unit variance per row."""
    from xpu_graph_b200.modules import AddLayerNormModule

    rows, hidden = 65536, 8192
    g = torch.Generator(device=cuda_device).manual_seed(1)
    x = torch.randn(rows, hidden, generator=g, device=cuda_device, dtype=torch.bfloat16)
    r = torch.randn(rows, hidden, generator=g, device=cuda_device, dtype=torch.bfloat16)
    w = (1.0 + 0.1 * torch.randn(hidden, generator=g, device=cuda_device)).to(torch.bfloat16)
    b = (0.1 * torch.randn(hidden, generator=g, device=cuda_device)).to(torch.bfloat16)
    out = AddLayerNormModule(store_sum)(x, r, w, b, 1e-5)
    y, s = (out[0], out[1]) if store_sum else (out, None)
    sel = torch.tensor([0, 1, 4095, 32768, 65535], device=cuda_device)
    want_y, want_s = ref_ops.add_layer_norm(x[sel].cpu(), r[sel].cpu(), w.cpu(), b.cpu(), 1e-5)
    assert_parity(y[sel], want_y, "full-size LayerNorm rows")
    if store_sum:
        assert_bit_exact(s[sel], want_s, "full-size LayerNorm sum rows")
    for lo in range(0, rows, 16384):  # in slabs: the fp32 copy of the whole tensor would be 2 GiB
        z = (y[lo:lo + 16384].float() - b.float()) / w.float()
        assert z.mean(dim=1).abs().max().item() < 2e-2
        assert (z.var(dim=1, unbiased=False) - 1.0).abs().max().item() < 3e-2
