"""GPU parity: fused scaled-dot-product attention through the C ABI vs the CPU oracle.

Shapes follow the reference's SDPA tests (tests/common/test_fuse_sdpa.py:553-561: B in {1,2,4}, 32 heads,
S=38, E=64, fp16) plus the two benchmark shapes (encoder block fp32 [1,8,128,64]; Llama prefill bf16
[8,32,2048,128] causal). The reference's own test drops its comparison result; these pin it.
"""
import pytest
import torch

from oracle import ref_ops
from tests.helpers import assert_parity, error_stats

pytestmark = pytest.mark.gpu


def _qkv(B, H, Sq, Skv, D, dtype, seed):
    g = torch.Generator().manual_seed(seed)
    q = torch.randn(B, H, Sq, D, generator=g).to(dtype)
    k = torch.randn(B, H, Skv, D, generator=g).to(dtype)
    v = torch.randn(B, H, Skv, D, generator=g).to(dtype)
    return q, k, v


def _run(cuda_device, q, k, v, mask, scale, causal):
    from xpu_graph_b200 import lib
    from xpu_graph_b200.modules import SDPAModule

    out = SDPAModule()(q.to(cuda_device), k.to(cuda_device), v.to(cuda_device), mask.to(cuda_device) if mask is not None else None, scale, causal)
    torch.cuda.synchronize()
    assert lib.tc_status() == 0, "a bounded wait expired inside the attention kernel"
    return out


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("B,H,S,D", [(1, 1, 128, 128), (2, 3, 256, 128), (1, 2, 300, 128), (2, 2, 38, 64), (1, 4, 512, 64), (1, 1, 1, 128)])
def test_flash_tc(cuda_device, B, H, S, D, causal, dtype):
    q, k, v = _qkv(B, H, S, S, D, dtype, 30)
    got = _run(cuda_device, q, k, v, None, None, causal)
    want = ref_ops.sdpa(q, k, v, None, None, causal)
    assert_parity(got, want, f"sdpa {B}x{H}x{S}x{D} causal={causal} {dtype}")
    exact = ref_ops.sdpa_math(q, k, v, None, None, causal)
    max_abs, mean_rel = error_stats(got, exact)
    assert max_abs < 2e-2, f"max abs error vs fp32 math {max_abs}"


@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("D", [64, 128])
@pytest.mark.parametrize("shape", ["ramp", "jump", "masked_tail"])
def test_flash_tc_growing_row_maximum(cuda_device, shape, D, causal):
    """Scores whose row maximum grows by far more than the lazy-rescale threshold in later key blocks: the kernel
    forms a block's probabilities against the running maximum first and must rescale O and redo the block."""
    B, H, S = 1, 2, 640
    q, k, v = _qkv(B, H, S, S, D, torch.bfloat16, 33)
    q = (q.float().abs() + 0.5).to(torch.bfloat16)  # positive queries: a key's scale sets the sign and size of its scores
    mask = None
    if shape == "ramp":      # every 64-key block is about 25 (natural units, after scaling) above the previous one
        gain = torch.linspace(0.0, 8.0, S).view(1, 1, S, 1)
        k = (k.float().abs() * gain).to(torch.bfloat16)
    elif shape == "jump":    # small scores, then one block far above everything before it
        k = (k.float() * 0.05).to(torch.bfloat16)
        k[:, :, 400:420] = (k[:, :, 400:420].float().abs() * 400.0 + 4.0).to(torch.bfloat16)
    else:                    # the general-mask variant of the kernel: additive mask, large scores late
        gain = torch.linspace(0.0, 6.0, S).view(1, 1, S, 1)
        k = (k.float().abs() * gain).to(torch.bfloat16)
        g = torch.Generator().manual_seed(34)
        mask = (torch.randn(B, 1, S, S, generator=g) * 2.0).to(torch.bfloat16)
    got = _run(cuda_device, q, k, v, mask, None, causal)
    want = ref_ops.sdpa(q, k, v, mask, None, causal)
    assert torch.isfinite(got.float()).all()
    assert_parity(got, want, f"sdpa growing maximum ({shape}) D={D} causal={causal}")


def test_flash_tc_mask_and_cross_lengths(cuda_device):
    q, k, v = _qkv(2, 2, 130, 200, 64, torch.bfloat16, 31)
    g = torch.Generator().manual_seed(32)
    mask = torch.randn(2, 1, 130, 200, generator=g).to(torch.bfloat16)
    got = _run(cuda_device, q, k, v, mask, 0.2, False)
    assert_parity(got, ref_ops.sdpa(q, k, v, mask, 0.2, False), "sdpa additive mask")
    keep = torch.rand(1, 1, 130, 200, generator=g) > 0.3
    keep[..., 0] = True  # no fully masked row
    got = _run(cuda_device, q, k, v, keep, None, False)
    assert_parity(got, ref_ops.sdpa(q, k, v, keep, None, False), "sdpa boolean mask")


@pytest.mark.parametrize("Sq,Skv,D", [(384, 384, 128), (640, 1024, 128), (1152, 1152, 64), (130, 192, 128), (256, 64, 64),
                                       (1024, 1000, 128), (200, 513, 64)])
def test_flash_tc_causal_diagonal_paths(cuda_device, Sq, Skv, D):
    """Causal attention over several query tiles and key counts: blocks cut by the diagonal are handled per warp (all,
    some or no keys visible), key counts that are not a multiple of the key block take the kernel variant with the
    general masking code, and every output row leaves through the staged epilogue. The mask is top-left aligned as in
    aten (row i sees keys 0..i), also when the lengths differ."""
    q, k, v = _qkv(2, 3, Sq, Skv, D, torch.bfloat16, 40 + Sq)
    got = _run(cuda_device, q, k, v, None, None, True)
    assert_parity(got, ref_ops.sdpa(q, k, v, None, None, True), f"causal sdpa {Sq}x{Skv}x{D}")
    max_abs, mean_rel = error_stats(got, ref_ops.sdpa_math(q, k, v, None, None, True))
    print(f"causal sdpa {Sq}x{Skv}x{D}: max_abs={max_abs:.3g} mean_rel={mean_rel:.3g} vs fp32 math")
    assert torch.isfinite(got.float()).all()


def test_flash_tc_strided_output_rows(cuda_device):
    """The output written as [B, S, H, D] (row stride H*D): the staged epilogue addresses rows by the caller's strides."""
    from xpu_graph_b200 import ops  # noqa: F401

    B, H, S, D = 2, 4, 320, 128
    q, k, v = _qkv(B, H, S, S, D, torch.bfloat16, 77)
    qd, kd, vd = (t.to(cuda_device).transpose(1, 2).contiguous().transpose(1, 2) for t in (q, k, v))  # [B,H,S,D] views of [B,S,H,D]
    got = torch.ops.xg_sm100.sdpa(qd, kd, vd, None, D ** -0.5, True)
    assert_parity(got, ref_ops.sdpa(q, k, v, None, None, True), "sdpa with [B, S, H, D] output rows")
    max_abs, mean_rel = error_stats(got, ref_ops.sdpa_math(q, k, v, None, None, True))
    print(f"sdpa strided output: max_abs={max_abs:.3g} mean_rel={mean_rel:.3g} vs fp32 math")


def test_flash_tc_transposed_views(cuda_device):
    """q/k/v as they leave the projections: [B, S, H*D] viewed and transposed to [B, H, S, D]."""
    B, S, H, D = 2, 260, 4, 128
    g = torch.Generator().manual_seed(33)
    base = [torch.randn(B, S, H * D, generator=g).to(torch.bfloat16) for _ in range(3)]
    q, k, v = (t.view(B, S, H, D).transpose(1, 2) for t in base)
    from xpu_graph_b200.modules import SDPAModule

    dq, dk, dv = (t.to(cuda_device).view(B, S, H, D).transpose(1, 2) for t in base)
    got = SDPAModule()(dq, dk, dv, None, None, True)
    assert_parity(got, ref_ops.sdpa(q, k, v, None, None, True), "sdpa transposed views")


@pytest.mark.parametrize("causal", [False, True])
def test_simt_fp32_encoder_shape(cuda_device, causal):
    q, k, v = _qkv(1, 8, 128, 128, 64, torch.float32, 34)
    got = _run(cuda_device, q, k, v, None, 0.125, causal)
    want = ref_ops.sdpa_math(q.double(), k.double(), v.double(), None, 0.125, causal).float()
    assert_parity(got, want, "sdpa fp32")


@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("B,H,Sq,Skv,D", [(2, 3, 77, 91, 64), (1, 2, 300, 300, 32), (1, 2, 130, 517, 128), (2, 2, 16, 1, 64),
                                          (1, 1, 1, 260, 64)])
def test_tiled_fp32(cuda_device, B, H, Sq, Skv, D, causal):
    """fp32 attention without a mask at head dims 32 / 64 / 128 runs on the shared-memory tiled kernel: ragged row and
    key counts, several key chunks, rows that see a single key."""
    q, k, v = _qkv(B, H, Sq, Skv, D, torch.float32, 37)
    got = _run(cuda_device, q, k, v, None, None, causal)
    want = ref_ops.sdpa_math(q.double(), k.double(), v.double(), None, None, causal).float()
    assert_parity(got, want, f"sdpa fp32 tiled {B}x{H}x{Sq}x{Skv}x{D} causal={causal}")


def test_tiled_fp32_strided_views_and_mask_fallback(cuda_device):
    """q / k / v as transposed views of [B, S, H, D] buffers go through the tiled kernel in place; with an additive mask
    the same shape runs on the row-per-warp kernel. Both against fp64 math."""
    B, H, S, D = 2, 4, 100, 64
    g = torch.Generator().manual_seed(38)
    qb, kb, vb = (torch.randn(B, S, H, D, generator=g) for _ in range(3))
    q, k, v = qb.transpose(1, 2), kb.transpose(1, 2), vb.transpose(1, 2)
    got = _run(cuda_device, q, k, v, None, None, True)
    assert_parity(got, ref_ops.sdpa_math(q.double(), k.double(), v.double(), None, None, True).float(), "sdpa fp32 tiled, strided views")
    mask = torch.randn(S, S, generator=g)
    got = _run(cuda_device, q, k, v, mask, None, False)
    assert_parity(got, ref_ops.sdpa_math(q.double(), k.double(), v.double(), mask.double(), None, False).float(), "sdpa fp32 with mask")


def test_simt_other_head_dims(cuda_device):
    q, k, v = _qkv(2, 2, 77, 91, 96, torch.bfloat16, 35)
    g = torch.Generator().manual_seed(36)
    mask = torch.randn(77, 91, generator=g).to(torch.bfloat16)
    got = _run(cuda_device, q, k, v, mask, None, False)
    assert_parity(got, ref_ops.sdpa(q, k, v, mask, None, False), "sdpa D=96")


def test_config4_prefill_shape(cuda_device):
    """Llama prefill shape [8, 32, 2048, 128] bf16 causal: sampled (batch, head) pairs against the oracle,
    plus the row-stochastic property (attention over an all-ones V returns ones)."""
    B, H, S, D = 8, 32, 2048, 128
    g = torch.Generator(device=cuda_device).manual_seed(3)
    q = torch.randn(B, H, S, D, generator=g, device=cuda_device, dtype=torch.bfloat16)
    k = torch.randn(B, H, S, D, generator=g, device=cuda_device, dtype=torch.bfloat16)
    v = torch.randn(B, H, S, D, generator=g, device=cuda_device, dtype=torch.bfloat16)
    from xpu_graph_b200 import lib
    from xpu_graph_b200.modules import SDPAModule

    got = SDPAModule()(q, k, v, None, None, True)
    torch.cuda.synchronize()
    assert lib.tc_status() == 0
    for b, h in [(0, 0), (7, 31), (3, 17)]:
        want = ref_ops.sdpa(q[b:b + 1, h:h + 1].cpu(), k[b:b + 1, h:h + 1].cpu(), v[b:b + 1, h:h + 1].cpu(), None, None, True)
        assert_parity(got[b:b + 1, h:h + 1], want, f"prefill pair ({b},{h})")
    ones = SDPAModule()(q, k, torch.ones_like(v), None, None, True)
    assert (ones.float() - 1.0).abs().max().item() < 1e-2
