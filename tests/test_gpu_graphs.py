"""GPU parity of whole fused graphs against the eager (pattern-disabled) models on CPU."""
import pytest
import torch

from tests.helpers import assert_parity, error_stats

pytestmark = pytest.mark.gpu


def test_encoder_block_fp32(cuda_device):
    """Config 1: encoder block fp32, batch 2 x seq 128 x hidden 256, 4 heads, FFN 1024 GELU, seed 0."""
    from xpu_graph_b200.fused_graphs import FusedEncoderBlock
    from xpu_graph_b200.workloads import make_encoder

    model, x = make_encoder(seed=0)
    with torch.no_grad():
        want = model(x)
    got = FusedEncoderBlock(model.to(cuda_device))(x.to(cuda_device))
    assert_parity(got, want, "encoder block fp32")


@pytest.mark.parametrize("fuse_swiglu_gemm", [True, False])
def test_llama_layer_small(cuda_device, fuse_swiglu_gemm):
    """Config 4 at reduced size (hidden 512, 4 heads x 128, FFN 1376, batch 2 x seq 320), bf16, causal."""
    from xpu_graph_b200 import lib
    from xpu_graph_b200.fused_graphs import FusedLlamaDecoderLayer
    from xpu_graph_b200.workloads import make_llama_layer

    model, (x, cos, sin) = make_llama_layer(seed=3, batch=2, seq=320, hidden=512, heads=4, ffn=1376)
    with torch.no_grad():
        want = model(x, cos, sin)
        exact = model.float()(x.float(), cos.float(), sin.float())
    model = model.to(torch.bfloat16).to(cuda_device)
    got = FusedLlamaDecoderLayer(model, fuse_swiglu_gemm)(x.to(cuda_device), cos.to(cuda_device), sin.to(cuda_device))
    torch.cuda.synchronize()
    assert lib.tc_status() == 0
    assert_parity(got, want, "llama layer bf16")
    ours, theirs = error_stats(got, exact)[0], error_stats(want, exact)[0]
    print(f"max abs error vs fp32 math: fused {ours:.4g}, eager bf16 {theirs:.4g}")
    assert ours <= 2.0 * theirs + 1e-2


def test_recsys_graph(cuda_device):
    """Config 5 at reduced size (batch 2048, tables of 5000 rows), fp32 values / int64 indices."""
    from xpu_graph_b200.fused_graphs import FusedRecsysGraph
    from xpu_graph_b200.workloads import make_recsys

    model, (dense, idx, mask) = make_recsys(seed=4, batch=2048, table_rows=5000)
    with torch.no_grad():
        want = model(dense, idx, mask)
    got = FusedRecsysGraph(model.to(cuda_device))(dense.to(cuda_device), idx.to(cuda_device), mask.to(cuda_device))
    assert_parity(got, want, "recsys graph fp32")


def test_recsys_graph_full_size(cuda_device):
    """Config 5 at its full size (batch 16384, 26 tables of 1e5 rows): here all three MLP layers are large enough for the
    fp32 tensor-core path, so the graph ends in one dense-tower call; checked against the eager model on the CPU."""
    from xpu_graph_b200 import ops
    from xpu_graph_b200.fused_graphs import FusedRecsysGraph
    from xpu_graph_b200.workloads import make_recsys

    model, (dense, idx, mask) = make_recsys(seed=4)
    assert dense.shape[0] == 16384
    with torch.no_grad():
        want = model(dense, idx, mask)
    assert ops.dense_tower_eligible(16384, [64 + 26 * 64, 1024, 512, 256])
    got = FusedRecsysGraph(model.to(cuda_device))(dense.to(cuda_device), idx.to(cuda_device), mask.to(cuda_device))
    assert_parity(got, want, "recsys graph fp32, full size")


def test_cuda_graph_replay_encoder(cuda_device):
    """Capture the fused encoder block once, replay it on new inputs (the reference's GraphRunner contract)."""
    from xpu_graph_b200.fused_graphs import FusedEncoderBlock
    from xpu_graph_b200.graph_runner import CUDAGraphRunner
    from xpu_graph_b200.workloads import make_encoder

    model, x = make_encoder(seed=0)
    cpu_model, _ = make_encoder(seed=0)  # same seed: an identical copy that stays on the CPU
    fused = FusedEncoderBlock(model.to(cuda_device))
    runner = CUDAGraphRunner(fused)
    xd = x.to(cuda_device)
    runner.capture(xd, clone_args=True)
    g = torch.Generator().manual_seed(99)
    for _ in range(2):
        x2 = torch.randn(x.shape, generator=g)
        with torch.no_grad():
            want = cpu_model(x2)
        got = runner(x2.to(cuda_device)).clone()
        assert_parity(got, want, "graph replay")


def test_cuda_graph_replay_llama_small(cuda_device):
    from xpu_graph_b200 import lib
    from xpu_graph_b200.fused_graphs import FusedLlamaDecoderLayer
    from xpu_graph_b200.graph_runner import CUDAGraphRunner
    from xpu_graph_b200.workloads import make_llama_layer

    model, (x, cos, sin) = make_llama_layer(seed=3, batch=1, seq=256, hidden=512, heads=4, ffn=1376)
    with torch.no_grad():
        want = model(x, cos, sin)
    fused = FusedLlamaDecoderLayer(model.to(cuda_device))
    runner = CUDAGraphRunner(fused)
    args = (x.to(cuda_device), cos.to(cuda_device), sin.to(cuda_device))
    runner.capture(*args, clone_args=True)
    got = runner(*args).clone()
    torch.cuda.synchronize()
    assert lib.tc_status() == 0
    assert_parity(got, want, "llama graph replay")
