"""GPU parity: RoPE and SwiGLU through the C ABI vs the CPU oracle."""
import pytest
import torch

from oracle import ref_ops
from tests.helpers import assert_parity

pytestmark = pytest.mark.gpu


def _rope_tables(S, D, dtype, theta=10000.0):
    inv = 1.0 / (theta ** (torch.arange(0, D, 2).float() / D))
    ang = torch.outer(torch.arange(S).float(), inv)
    emb = torch.cat((ang, ang), dim=-1)
    return emb.cos().to(dtype), emb.sin().to(dtype)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("B,H,S,D", [(1, 1, 1, 2), (2, 3, 17, 64), (2, 4, 33, 128), (1, 2, 5, 6), (1, 32, 256, 128)])
def test_rope(cuda_device, B, H, S, D, dtype):
    from xpu_graph_b200.modules import RopeModule

    g = torch.Generator().manual_seed(6)
    x = torch.randn(B, H, S, D, generator=g).to(dtype)
    cos, sin = _rope_tables(S, D, dtype)
    got = RopeModule()(x.to(cuda_device), cos.to(cuda_device)[None, None], sin.to(cuda_device)[None, None])
    assert_parity(got, ref_ops.rope(x, cos[None, None], sin[None, None]), f"rope {B}x{H}x{S}x{D}")


def test_rope_transposed_input(cuda_device):
    """q as it leaves the projection: [B, S, H*D] viewed [B, S, H, D] and transposed to [B, H, S, D]."""
    from xpu_graph_b200.modules import RopeModule

    g = torch.Generator().manual_seed(7)
    B, S, H, D = 2, 40, 4, 128
    base = torch.randn(B, S, H * D, generator=g).to(torch.bfloat16)
    x = base.view(B, S, H, D).transpose(1, 2)
    cos, sin = _rope_tables(S, D, torch.bfloat16)
    xd = base.to(cuda_device).view(B, S, H, D).transpose(1, 2)
    got = RopeModule()(xd, cos.to(cuda_device), sin.to(cuda_device))
    assert got.stride() == xd.stride()  # the output keeps the [B, S, H, D] memory layout
    assert_parity(got, ref_ops.rope(x, cos, sin), "rope transposed")


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("rows,cols", [(1, 1), (7, 24), (33, 1000), (64, 11008), (5, 333)])
def test_swiglu(cuda_device, rows, cols, dtype):
    from xpu_graph_b200.modules import SwiGLUModule

    g = torch.Generator().manual_seed(8)
    gate = torch.randn(rows, cols, generator=g).to(dtype)
    up = torch.randn(rows, cols, generator=g).to(dtype)
    got = SwiGLUModule()(gate.to(cuda_device), up.to(cuda_device))
    assert_parity(got, ref_ops.swiglu(gate, up), f"swiglu {rows}x{cols}")


def test_swiglu_packed(cuda_device):
    """gate and up as the two halves of one packed [rows, 2d] tensor (row stride 2d)."""
    from xpu_graph_b200.modules import SwiGLUModule

    g = torch.Generator().manual_seed(9)
    packed = torch.randn(19, 2 * 512, generator=g).to(torch.bfloat16)
    pd = packed.to(cuda_device)
    got = SwiGLUModule()(pd[:, :512], pd[:, 512:])
    assert_parity(got, ref_ops.swiglu(packed[:, :512], packed[:, 512:]), "swiglu packed")
