"""Host-side checks of the C ABI: the library loads, exports every symbol the header declares, and
rejects bad arguments with an error code before anything touches a GPU."""
import ctypes
import os
import re

import pytest
import torch

from xpu_graph_b200 import lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "xg_sm100.h")


def _declared_functions():
    src = open(HEADER).read()
    src = re.sub(r"/\*.*?\*/", "", src, flags=re.S)
    return sorted(set(re.findall(r"\b(xg_[a-z0-9_]+)\s*\(", src)))


def test_library_exports_every_declared_symbol():
    names = _declared_functions()
    assert len(names) >= 14
    L = lib.load()
    for n in names:
        assert hasattr(L, n), f"{n} declared in include/xg_sm100.h but not exported"
    assert set(names) == set(lib.SIGNATURES), "ctypes signature table and header disagree"
    assert L.xg_version() >= 1000


def test_missing_library_fails_loudly(tmp_path):
    with pytest.raises(lib.XgLibraryError):
        lib.load(str(tmp_path / "libxg_sm100.so"))
    bogus = tmp_path / "bogus.so"
    bogus.write_bytes(b"not an ELF file")
    with pytest.raises(lib.XgLibraryError):
        lib.load(str(bogus))


def test_argument_validation_without_gpu():
    L = lib.load()
    # null pointers
    assert L.xg_rmsnorm(None, None, None, None, None, 4, 8, 8, 0, 1e-6, lib.XG_BF16, lib.XG_BF16, None) == -1
    assert "null" in lib.last_error()
    buf = ctypes.create_string_buffer(4096)
    p = ctypes.cast(buf, ctypes.c_void_p)
    # bad extents / dtypes / strides
    assert L.xg_rmsnorm(p, None, p, p, None, -1, 8, 8, 0, 1e-6, lib.XG_BF16, lib.XG_BF16, None) == -1
    assert L.xg_rmsnorm(p, None, p, p, None, 4, 8, 4, 0, 1e-6, lib.XG_BF16, lib.XG_BF16, None) == -1
    assert L.xg_rmsnorm(p, None, p, p, None, 4, 8, 8, 0, 1e-6, 7, 7, None) == -1
    assert L.xg_rmsnorm(p, None, p, p, p, 4, 8, 8, 0, 1e-6, lib.XG_BF16, lib.XG_BF16, None) == -1  # sum_out without residual
    assert L.xg_layernorm(p, None, None, None, p, None, 4, 8, 8, 0, 1e-5, lib.XG_F32, lib.XG_F32, None) == -1  # weight required (bias is not)
    assert L.xg_rope(p, p, p, p, 1, 1, 4, 7, 28, 28, 7, 28, 28, 7, lib.XG_F32, None) == -1  # odd head dim
    assert L.xg_swiglu(p, p, p, 4, 8, 4, 8, 8, lib.XG_F32, None) == -1
    assert L.xg_gemm_bias_act(p, p, None, None, p, 4, 4, 0, 4, 4, 4, 0, 1, 0, lib.XG_F32, None) == -1  # K == 0
    assert L.xg_gemm_bias_act(p, p, None, None, p, 4, 4, 8, 4, 8, 4, 0, 1, 0, lib.XG_F32, None) == -1  # lda < K
    assert L.xg_gemm_bias_act(p, p, None, None, p, 4, 4, 8, 8, 8, 4, 0, 1, 9, lib.XG_F32, None) == -1  # bad act
    # rows a tensor map cannot address: the cluster kernel refuses them (the plain entry runs them on the FMA kernel)
    assert L.xg_gemm_bias_act_cluster(p, p, None, None, p, 8, 8, 8, 12, 8, 8, 0, 0, lib.XG_BF16, 1, 64, None) == -2
    assert "16-byte" in lib.last_error()
    # small tower: limits answered without a device
    dims_ok, dims_wide = lib.i64_array([20, 32, 16, 1]), lib.i64_array([20, 256, 16, 1])
    assert L.xg_mlp_small_supported(dims_ok, 3, lib.XG_F16) == 1 and L.xg_mlp_small_supported(dims_wide, 3, lib.XG_F16) == 0
    assert L.xg_mlp_small_supported(lib.i64_array([128, 128, 128, 128]), 3, lib.XG_F32) == 0  # 49152 weight elements
    assert L.xg_mlp_small_supported(dims_ok, 4, lib.XG_F16) == 0
    ws, ld, acts = lib.ptr_array([p.value] * 3), lib.i64_array([32, 16, 1]), (ctypes.c_int * 3)(1, 1, 0)
    assert L.xg_mlp_small_bias_act(p, ws, None, p, 16, dims_wide, 3, 20, ld, 1, acts, 7, lib.XG_F16, None) == -2
    assert L.xg_mlp_small_bias_act(None, ws, None, p, 16, dims_ok, 3, 20, ld, 1, acts, 7, lib.XG_F16, None) == -1
    assert L.xg_mlp_small_bias_act(p, ws, None, p, 16, dims_ok, 3, 8, ld, 1, acts, 7, lib.XG_F16, None) == -1  # lda < K
    assert L.xg_gemm_swiglu(p, p, p, p, 8, 8, 8, 8, 8, 8, lib.XG_F32, None) == -2
    assert L.xg_sdpa_fwd(None, None, None, None, None, 1, 1, 1, 1, 8, None, None, None, None, None, 1.0, 0, lib.XG_BF16, None) == -1
    assert L.xg_gather_rows(None, None, 2, None, 2, 1, None, 1, None, 4, 8, 16, 4, None) == -1
    assert L.xg_gather_rows(None, None, 2, None, 2, 1, None, 1, None, 4, 8, 16, 3, None) == -1  # elem_size
    assert L.xg_seg_copy(None, None, None, None, None, 3, 4, None, 1, None) == -1
    assert L.xg_tc_status(None, 0) == -1
    # the fp32-on-tensor-core entry points, the batched dense layer, the row-sum fusions
    assert L.xg_gemm_f32x3_padded_k(1) == 64 and L.xg_gemm_f32x3_padded_k(64) == 64 and L.xg_gemm_f32x3_padded_k(65) == 128
    assert L.xg_gemm_f32x3_padded_k(0) == 0
    assert L.xg_split_bf16x3(None, 4, 8, 8, 0, p, None) == -1
    assert L.xg_split_bf16x3(p, 4, 8, 4, 0, p, None) == -1  # ld < K
    assert L.xg_split_bf16x3(p, -1, 8, 8, 0, p, None) == -1
    assert L.xg_split_bf16x3(p, 0, 8, 8, 0, p, None) == 0
    assert L.xg_gemm_f32x3(None, p, None, None, p, 4, 4, 8, 4, 0, 0, 0, None) == -1
    assert L.xg_gemm_f32x3(p, p, None, None, p, 4, 4, 0, 4, 0, 0, 0, None) == -1  # K == 0
    assert L.xg_gemm_f32x3(p, p, None, None, p, 4, 4, 8, 2, 0, 0, 0, None) == -1  # ldc < N
    assert L.xg_gemm_f32x3(p, p, None, None, p, 4, 4, 8, 4, 0, 7, 0, None) == -1  # bad activation
    assert L.xg_gemm_f32x3(p, p, None, p, p, 4, 4, 8, 4, 4, 0, 1, None) == -2     # plane output takes no residual
    assert L.xg_bgemm_bias_act(p, p, None, None, p, -1, 4, 4, 8, 8, 8, 4, 0, 32, 32, 0, 0, 16, 1, 0, lib.XG_BF16, None) == -1
    assert L.xg_bgemm_bias_act(p, p, None, None, p, 0, 4, 4, 8, 8, 8, 4, 0, 32, 32, 0, 0, 16, 1, 0, lib.XG_BF16, None) == 0
    a1 = lib.ptr_array([p.value])
    assert L.xg_rowsum_cat(a1, None, lib.i64_array([32]), None, lib.i64_array([0, 4]), 1, -2, 8, p, 8, lib.XG_F32, None) == -1
    assert L.xg_rowsum_cat(a1, None, lib.i64_array([32]), None, lib.i64_array([0, 4]), 0, 2, 8, p, 8, lib.XG_F32, None) == 0
    assert L.xg_sum3d(None, None, None, 2, 1, lib.XG_F32, None) == -1
    assert L.xg_sum3d(None, None, None, 1, 5, lib.XG_F32, None) == -1  # dim
    # empty problems succeed without a launch
    assert L.xg_seg_copy(None, None, None, None, None, 0, 4, None, 1, None) == 0
    assert L.xg_swiglu(p, p, p, 0, 8, 8, 8, 8, lib.XG_F32, None) == 0
    assert L.xg_rmsnorm(p, None, p, p, None, 0, 8, 8, 0, 1e-6, lib.XG_BF16, lib.XG_BF16, None) == 0


def test_ops_have_no_cpu_kernel():
    """The target has no CPU fallback: calling an op on CPU tensors raises instead of computing."""
    import torch

    from xpu_graph_b200 import ops  # noqa: F401

    if "cpu" in getattr(__import__("xpu_graph_b200.modules", fromlist=["x"]), "ALLOWED_DEVICE_TYPES"):
        pytest.skip("CPU test doubles already registered in this process")
    with pytest.raises((NotImplementedError, RuntimeError)):
        torch.ops.xg_sm100.rms_norm(torch.zeros(2, 8), torch.ones(8), 1e-6)


def test_stack_or_view_reuses_slabs_of_one_buffer():
    """Operands of a combo dense call that are consecutive slabs of one buffer are used in place; anything else is
    stacked (host logic only, no GPU needed)."""
    import torch

    from xpu_graph_b200 import ops

    base = torch.arange(4 * 6 * 8, dtype=torch.float32).reshape(4, 6, 8)
    v = ops._stack_or_view(list(base.unbind(0)))
    assert v.data_ptr() == base.data_ptr() and torch.equal(v, base)
    mid = ops._stack_or_view(list(base[1:3].unbind(0)))
    assert mid.data_ptr() == base[1].data_ptr() and torch.equal(mid, base[1:3])
    separate = [base[i].clone() for i in range(4)]
    w = ops._stack_or_view(separate)
    assert w.data_ptr() not in {t.data_ptr() for t in separate} and torch.equal(w, base)
    shuffled = [base[2], base[0], base[1]]
    assert torch.equal(ops._stack_or_view(shuffled), torch.stack(shuffled))
    strided = [base[:, i, :] for i in range(3)]  # not contiguous slabs
    assert torch.equal(ops._stack_or_view(strided), torch.stack(strided))


def test_multi_slice_refuses_slices_outside_the_row():
    """FusedSlice passes end - start of the raw aten.slice arguments as the slice length (structure/fuse_slice.py:28);
    a slice that aten would have clamped must be refused on the host, not read past the row on the device."""
    import pytest

    from xpu_graph_b200 import ops

    assert ops._checked_starts(64, [0, 60, -4], 4) == [0, 60, 60]
    for starts, length in (([62], 4), ([-70], 4), ([0], 65), ([0], 9223372036854775807), ([0], -1)):
        with pytest.raises(ValueError):
            ops._checked_starts(64, starts, length)
    # the fake implementation (shape propagation in the compiler) refuses the same slices
    from torch._subclasses.fake_tensor import FakeTensorMode

    with FakeTensorMode():
        src = torch.empty(8, 64)
        assert tuple(torch.ops.xg_sm100.multi_slice(src, [0, 8], 8).shape) == (2, 8, 8)
        with pytest.raises(Exception):
            torch.ops.xg_sm100.multi_slice(src, [60], 8)


def test_weight_plane_cache_key_with_untracked_tensors():
    """Tensors made under torch.inference_mode() have no version counter: their planes are not cached (the key is
    None) instead of raising; ordinary tensors are keyed on version, address, layout and orientation."""
    from xpu_graph_b200 import ops

    with torch.inference_mode():
        w_inf = torch.randn(4, 8)
    assert ops._planes_tag(w_inf, True) is None
    w = torch.randn(4, 8)
    t0 = ops._planes_tag(w, True)
    assert t0 is not None and t0 != ops._planes_tag(w, False)
    w.add_(1.0)
    assert ops._planes_tag(w, True) != t0  # an in-place update moves the version counter
    w.data.mul_(2.0)  # through .data it does not: that is what invalidate_weight_planes is for
    w._xg_bf16_planes = ("stale", None)
    ops.invalidate_weight_planes(w)
    assert not hasattr(w, "_xg_bf16_planes")
    ops.invalidate_weight_planes(w)  # idempotent


def test_small_m_plan_and_tower_routing_without_gpu():
    """Host-side decisions that need no device: the split-K plan of dense layers with M <= 128 (scratch size = splits x
    M x N x 4 bytes; the measured best choices of the sweep it was fitted to) and the routing of narrow towers."""
    import torch

    from xpu_graph_b200 import ops

    L = lib.load()
    splits = lambda M, N, K: L.xg_gemm_workspace_bytes(M, N, K, lib.XG_BF16) // (M * N * 4)  # noqa: E731
    assert [splits(M, 4096, 4096) for M in (16, 64, 128)] == [4, 4, 4]      # 128-wide tiles x 4 splits = 128 CTAs
    assert splits(128, 2048, 4096) == 4 and splits(128, 1024, 4096) == 8    # 64-wide tiles for narrow outputs
    assert splits(16, 11008, 4096) == 3                                     # 43 tiles of 256 x 3 = 129 CTAs
    assert splits(128, 11008, 4096) == 0 and splits(64, 11008, 4096) == 0   # 86 tiles of 128, unsplit: partial sums would leave L2
    assert splits(256, 4096, 4096) == 0 and splits(4096, 4096, 4096) == 0   # the cluster / pair kernels need none
    # narrow towers: every width <= 128 and <= 24576 weight elements fit the kernel; it is used for few rows or tiny layers
    assert ops.mlp_small_eligible((20, 32, 16, 1), torch.float16) and not ops.mlp_small_eligible((20, 256, 16), torch.float16)
    assert not ops.mlp_small_eligible((128, 128, 128, 128), torch.float32)
    assert ops.mlp_small_worth_it(16, (20, 32, 16, 1), torch.float16) and ops.mlp_small_worth_it(16384, (64, 32, 16, 1), torch.float32)
    assert not ops.mlp_small_worth_it(16384, (128, 64, 32), torch.float32) and ops.mlp_small_worth_it(2048, (128, 64, 32), torch.float32)
    assert ops._small_run((20, 32, 16, 1), 0, 3, torch.float16, 16) == 3 and ops._small_run((512, 32, 16, 1), 0, 3, torch.float16, 16) == 1
    assert ops._small_run((512, 32, 16, 1), 1, 3, torch.float16, 16) == 2
