"""GPU test of xg_gemm_bias_act_static: the split-K dense layer for callers that cannot allocate.

Who needs it: code that runs where device allocation is off limits — a plugin inside another framework's
memory pool, a runtime with a fixed start-up memory budget, a latency-critical serving loop that must not hit
cudaMalloc's implicit synchronisation. The entry point keeps its fp32 partial sums in a 32 MiB array that
ships inside the library instead of a caller workspace.

The test calls the entry point through the C ABI (ctypes, raw pointers) and checks it against the existing
workspace-based entry point on the same inputs, twice in a row (the second call finds the array full of
the first call's partial sums), plus the size limit. It is named to be collected last so that a run that
stops at the first failure has already run every other test; it does not depend on them.
"""
import pytest
import torch

from tests.helpers import assert_parity

pytestmark = pytest.mark.gpu


def _dense_static(L, lib, x, w, b, r, act, out):
    M, K = x.shape
    N = w.shape[0]
    return L.xg_gemm_bias_act_static(x.data_ptr(), w.data_ptr(), b.data_ptr() if b is not None else None,
                                     r.data_ptr() if r is not None else None, out.data_ptr(), M, N, K, K, K, N,
                                     N if r is not None else 0, 1, lib.ACT_CODES[act], lib.XG_BF16,
                                     torch.cuda.current_stream().cuda_stream)


def _dense_ws(L, lib, x, w, b, r, act, out, ws):
    M, K = x.shape
    N = w.shape[0]
    return L.xg_gemm_bias_act_ws(x.data_ptr(), w.data_ptr(), b.data_ptr() if b is not None else None,
                                 r.data_ptr() if r is not None else None, out.data_ptr(), M, N, K, K, K, N,
                                 N if r is not None else 0, 1, lib.ACT_CODES[act], lib.XG_BF16,
                                 ws.data_ptr() if ws is not None else None, ws.numel() if ws is not None else 0,
                                 torch.cuda.current_stream().cuda_stream)


@pytest.mark.parametrize("M,K,N,act", [(256, 4096, 4096, "gelu"), (200, 1024, 1000, "none"), (4096, 256, 256, "silu"),
                                       (64, 8192, 4096, "gelu")])
def test_static_scratch_matches_workspace_entry(cuda_device, M, K, N, act):
    from xpu_graph_b200 import lib

    L = lib.load()
    assert L.xg_gemm_static_scratch_bytes() == 32 << 20
    g = torch.Generator(device=cuda_device).manual_seed(40)
    x = torch.randn(M, K, generator=g, device=cuda_device, dtype=torch.bfloat16)
    w = (0.02 * torch.randn(N, K, generator=g, device=cuda_device)).to(torch.bfloat16)
    b = (0.02 * torch.randn(N, generator=g, device=cuda_device)).to(torch.bfloat16)
    r = torch.randn(M, N, generator=g, device=cuda_device).to(torch.bfloat16)
    # the existing entry point with a caller workspace is the yardstick
    want = torch.empty(M, N, device=cuda_device, dtype=torch.bfloat16)
    need = L.xg_gemm_workspace_bytes(M, N, K, lib.XG_BF16)
    ws = torch.empty(max(need, 16), device=cuda_device, dtype=torch.uint8)
    lib.check(_dense_ws(L, lib, x, w, b, r, act, want, ws), "xg_gemm_bias_act_ws")
    torch.cuda.synchronize()

    outs = []
    before = torch.cuda.memory_allocated()
    for _ in range(2):  # two calls in a row on the shared array
        out = torch.full((M, N), float("nan"), device=cuda_device, dtype=torch.bfloat16)
        lib.check(_dense_static(L, lib, x, w, b, r, act, out), "xg_gemm_bias_act_static")
        torch.cuda.synchronize()
        outs.append(out)
    assert lib.tc_status() == 0
    # the same arithmetic restated on the CPU: act(x @ w^T + b + r)
    from oracle import ref_ops

    pre = ref_ops.dense(x.cpu(), w.cpu(), True, b.cpu(), "none") + r.cpu()
    oracle = ref_ops._ACTS[act](pre)
    for out in outs:
        assert_parity(out, want, f"static-scratch dense {M}x{K}x{N} {act}", magnitude=r)
        assert_parity(out, oracle, f"static-scratch dense {M}x{K}x{N} {act} vs the CPU oracle", magnitude=r)
    assert torch.equal(outs[0], outs[1]), "the second call must not see the first call's leftovers"
    # nothing but the two output tensors was allocated while the entry point ran
    grown = torch.cuda.memory_allocated() - before
    assert 2 * M * N * 2 <= grown <= 2 * (M * N * 2 + 1024)


def test_static_scratch_rejects_oversize(cuda_device):
    from xpu_graph_b200 import lib

    L = lib.load()
    M, K, N = 4096, 128, 2048  # 2*M*N*4 = 64 MiB > 32 MiB
    x = torch.zeros(M, K, device=cuda_device, dtype=torch.bfloat16)
    w = torch.zeros(N, K, device=cuda_device, dtype=torch.bfloat16)
    out = torch.zeros(M, N, device=cuda_device, dtype=torch.bfloat16)
    rc = _dense_static(L, lib, x, w, None, None, "none", out)
    assert rc == -5, lib.last_error()  # XG_ERR_TOO_LARGE
    assert "xg_gemm_bias_act_ws" in lib.last_error()
    # a single k-block cannot be split
    x1 = torch.zeros(64, 64, device=cuda_device, dtype=torch.bfloat16)
    w1 = torch.zeros(64, 64, device=cuda_device, dtype=torch.bfloat16)
    o1 = torch.zeros(64, 64, device=cuda_device, dtype=torch.bfloat16)
    assert _dense_static(L, lib, x1, w1, None, None, "none", o1) == -2  # XG_ERR_UNSUPPORTED
    # fp32 has no scratch-using kernel
    xf = torch.zeros(64, 128, device=cuda_device)
    rc = L.xg_gemm_bias_act_static(xf.data_ptr(), xf.data_ptr(), None, None, xf.data_ptr(), 64, 64, 128, 128, 128, 64, 0, 1,
                                   0, lib.XG_F32, torch.cuda.current_stream().cuda_stream)
    assert rc == -2
