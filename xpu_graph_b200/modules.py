"""Replacement modules of the ``cuda_sm100`` target.

These are the ``nn.Module`` classes that xpu_graph's structure patterns instantiate and call
(``target_mod(...)``); names, constructor arguments, ``forward`` signatures and error behaviour mirror
the Cambricon target's (passes/patterns/targets/mlu/structure_replacements/__init__.py:21-179,
dense_layer_modules.py:4-128, norm_modules.py:4-21) so that the reference's structure patterns can use
them unchanged. Every ``forward`` ends in a ``torch.ops.xg_sm100.*`` custom op; the modules hold no
tensors and no library handles, so compiled graphs stay picklable for the compile cache
(cache.py:113-179 of the reference).
"""
from __future__ import annotations

from typing import List, Optional, Sequence, Tuple

import torch

from . import ops  # noqa: F401  (registers torch.ops.xg_sm100.*)

_X = torch.ops.xg_sm100

_SUPPORTED = (torch.float32, torch.bfloat16, torch.float16)
# Device types on which the fusions are applied. The kernels exist for CUDA only; the host-side test
# suite adds "cpu" together with CPU stand-ins for the ops so that the graph rewrites can be exercised
# without a GPU.
ALLOWED_DEVICE_TYPES = {"cuda"}


# ---- normalisation -------------------------------------------------------------------------
class RMSNormModule(torch.nn.Module):
    """CustomRMSNorm target (structure/custom_rmsnorm.py:21-29): forward(inputs, weights, epsilon)."""

    def forward(self, inputs, weights, epsilon):
        return _X.rms_norm(inputs, weights, float(epsilon))


class LayerNormModule(torch.nn.Module):
    """CustomLayerNorm target (structure/custom_layernorm.py:21-29): forward(inputs, weights, bias, epsilon)."""

    def forward(self, inputs, weights, bias, epsilon):
        return _X.layer_norm(inputs, weights, bias, float(epsilon))


class AddRMSNormModule(torch.nn.Module):
    """Residual add fused into RMSNorm. ``store_sum`` mirrors store_output_before_norm of
    targets/mlu/fuse_add_norm.py:118-121: with it the module returns (normed, x + residual)."""

    def __init__(self, store_sum: bool):
        super().__init__()
        self.store_sum = bool(store_sum)

    def forward(self, inputs, residual, weights, epsilon):
        if self.store_sum:
            y, s = _X.add_rms_norm(inputs, residual, weights, float(epsilon))
            return y, s
        return _X.add_rms_norm_y(inputs, residual, weights, float(epsilon))


class AddLayerNormModule(torch.nn.Module):
    """Residual add fused into LayerNorm (see AddRMSNormModule)."""

    def __init__(self, store_sum: bool):
        super().__init__()
        self.store_sum = bool(store_sum)

    def forward(self, inputs, residual, weights, bias, epsilon):
        if self.store_sum:
            y, s = _X.add_layer_norm(inputs, residual, weights, bias, float(epsilon))
            return y, s
        return _X.add_layer_norm_y(inputs, residual, weights, bias, float(epsilon))


# ---- dense layers --------------------------------------------------------------------------
UNALIGNED_16BIT_MAX_FLOPS = 1 << 26


class DenseLayerModule(torch.nn.Module):
    """CustomDenseLayer target (structure/custom_denselayer.py:80-88):
    ``M(fast_act)``; forward(inputs, weight, weight_trans, bias, act). Bias handling follows
    dense_layer_modules.py:22-57: a 1-D (or [1, N]) bias is a per-column bias, anything else is a
    full [M, N] addend."""

    def __init__(self, fast_act):
        super().__init__()
        self.fast_act = fast_act

    def forward(self, inputs, weight, weight_trans, bias, act):
        m = inputs.shape[0]
        n = weight.shape[-1] if not weight_trans else weight.shape[-2]
        col_bias, full_bias = None, None
        if bias is not None:
            bshape = bias.shape
            if len(bshape) == 2 and bshape[0] == 1:
                bias = bias.view(-1)
                bshape = bias.shape
            if len(bshape) == 1:
                col_bias = bias if bias.shape[0] == n else bias.broadcast_to((n,)).contiguous()
            else:
                full_bias = bias if bias.shape == torch.Size([m, n]) else bias.broadcast_to((m, n)).contiguous()
        return _X.dense(inputs, weight, bool(weight_trans), col_bias, full_bias, act)


def can_fuse_custom_denselayer(inputs, weight, weight_trans, bias, act_str):
    """constraint_fn of CustomDenseLayer, evaluated on FakeTensors (custom_denselayer.py:86)."""
    if act_str not in ["gelu", "relu", "silu", "sigmoid", "none"]:
        return False
    if inputs.dim() != 2 or weight.dim() != 2:
        return False
    if inputs.dtype not in _SUPPORTED or weight.dtype != inputs.dtype:
        return False
    if bias is not None and bias.dtype != inputs.dtype:
        return False
    if inputs.device.type not in ALLOWED_DEVICE_TYPES:
        return False
    if inputs.dtype != torch.float32:
        # 16-bit rows a tensor map cannot address (not multiples of 16 bytes: K for the activations and [N, K] weights,
        # N for weights given as [K, N]) run on the library's FMA kernel. That wins while the layer is mostly launches
        # (one fused launch against matmul + add + activation); beyond about 64 MFLOP the vendor matmul is the faster
        # home for such a shape, and the layer is left to it.
        unaligned = inputs.shape[1] % 8 != 0 or (not weight_trans and weight.shape[1] % 8 != 0)
        if unaligned:
            try:
                flops = 2 * int(inputs.shape[0]) * int(weight.shape[0]) * int(weight.shape[1])
            except (TypeError, RuntimeError):  # symbolic extents: size unknown at compile time
                return False
            if flops > UNALIGNED_16BIT_MAX_FLOPS:
                return False
    return True


class BatchDenseLayerModule(torch.nn.Module):
    """CustomBatchDenseLayer target (custom_denselayer.py:111-117); bias forms as
    dense_layer_modules.py:82-93: [b, M, N] is a residual, anything else broadcasts to [b, 1, N]."""

    def forward(self, inputs, weight, weight_trans, bias, act):
        b, m, _ = inputs.shape
        n = weight.shape[-1] if not weight_trans else weight.shape[-2]
        col_bias, residual = None, None
        if bias is not None:
            if bias.shape == torch.Size([b, m, n]):
                residual = bias
            else:
                col_bias = bias.broadcast_to((b, 1, n))
        return _X.batch_dense(inputs, weight, bool(weight_trans), col_bias, residual, act)


def can_fuse_custom_batch_denselayer(inputs, weight, weight_trans, bias, act_str):
    if act_str not in ["gelu", "silu", "none"]:
        return False
    if inputs.dim() != 3 or weight.dim() != 3 or inputs.device.type not in ALLOWED_DEVICE_TYPES:
        return False
    if inputs.dtype not in _SUPPORTED or weight.dtype != inputs.dtype:
        return False
    if inputs.dtype != torch.float32 and (inputs.shape[2] % 8 != 0 or (not weight_trans and weight.shape[2] % 8 != 0)):
        return False
    return True


class DenseResidualModule(torch.nn.Module):
    """Dense layer with both a per-column bias and a full [M, N] addend (a residual) in one epilogue:
    act(inputs @ W + bias + residual)."""

    def forward(self, inputs, weight, weight_trans, bias, residual, act):
        if bias is not None and bias.dim() != 1:
            bias = bias.reshape(-1)
        return _X.dense(inputs, weight, bool(weight_trans), bias, residual, act)


class DenseSwiGLUModule(torch.nn.Module):
    """mul(silu(x @ Wg^T), x @ Wu^T) as one dual GEMM with the SwiGLU epilogue."""

    def forward(self, inputs, w_gate, w_up):
        return _X.dense_swiglu(inputs, w_gate, w_up)


class DenseRopeModule(torch.nn.Module):
    """q/k projection with the rotary embedding applied in the GEMM epilogue:
    forward(inputs [B*S, K], weight [H*D, K], cos, sin, B, S, H, D) -> [B, H, S, D] (a view of the [B, S, H*D]
    result, i.e. exactly what reshape + transpose + RopeModule returned). B = -1: inferred from the rows (a graph
    compiled with a symbolic batch size)."""

    def forward(self, inputs, weight, cos, sin, B, S, H, D):
        y = _X.dense_rope(inputs, weight, cos, sin, int(S), int(D))
        return y.view(B, S, H, D).transpose(1, 2)


class SwiGLUModule(torch.nn.Module):
    """silu(gate) * up (targets/npu/fuse_silu_mul.py:21-69 applies the same fusion to a packed tensor)."""

    def forward(self, gate, up):
        return _X.swiglu(gate, up)


class RopeModule(torch.nn.Module):
    """x*cos + rotate_half(x)*sin on [B, H, S, D]."""

    def forward(self, x, cos, sin):
        return _X.rope(x, cos, sin)


class SDPAModule(torch.nn.Module):
    """aten.scaled_dot_product_attention as produced by FusedSDPA
    (common/fuse_scaled_dot_product_attention.py:230-234)."""

    def forward(self, q, k, v, attn_mask, scale, is_causal):
        if scale is None:
            scale = q.shape[-1] ** -0.5
        return _X.sdpa(q, k, v, attn_mask, float(scale), bool(is_causal))


# ---- copy fusions --------------------------------------------------------------------------
class FuseSliceModule(torch.nn.Module):
    """FusedSlice target (structure/fuse_slice.py:96-106): ``M(start_indices)``;
    forward(src, slice_len) -> [num, *src.shape[:-1], slice_len]."""

    def __init__(self, slices_index):
        super().__init__()
        self.slices_index = [int(s) for s in slices_index]

    def forward(self, input_tensor, slice_len):
        return _X.multi_slice(input_tensor, self.slices_index, int(slice_len))


class FuseSliceCatSameInputModule(torch.nn.Module):
    """FusedCatSlice / FusedSliceStackSum target (structure/fuse_slice_cat.py:72-75):
    forward(src_2d, [(start, end), ...]) -> [rows, sum(len)]."""

    def forward(self, input_tensor, slices):
        if len(input_tensor.shape) != 2:
            raise NotImplementedError("input must be 2d")
        starts = [int(s) for s, _ in slices]
        ends = [int(e) for _, e in slices]
        return _X.slice_cat(input_tensor, starts, ends, None, False)


class FuseSliceCatSameInputModule_v2(torch.nn.Module):
    """FusedMultipleSliceCat target (structure/fuse_multiple_slice_cat.py:29-39):
    ``M(many_slices)``; forward(src, many_slices) -> list of [rows, sum(len_k)]."""

    def __init__(self, many_slices):
        super().__init__()
        self.starts = [int(s) for group in many_slices for s, _ in group]
        self.ends = [int(e) for group in many_slices for _, e in group]
        self.counts = [len(group) for group in many_slices]

    def forward(self, input_tensor, many_slices):
        return _X.slice_cat_multi(input_tensor, self.starts, self.ends, self.counts)


class MaskedSliceCatModule(torch.nn.Module):
    """cat([where(mask[B,1], 0, x[:, s:e]) ...], -1) — the computation of the reference's
    fuse_slice_where_cat kernel (targets/mlu/triton_kernel/fused_slice_where_cat.py:12-73)."""

    def forward(self, input_tensor, mask, slices, masked=None):
        """`masked`: optional flag per slice; slices flagged False are copied as they are (the form
        cat([x[:, a:b], where(m, 0, x[:, c:d]), ...]) of the reference's test, tests/mlu/test_fuse_slice_where_cat.py:19-31)."""
        starts = [int(s) for s, _ in slices]
        ends = [int(e) for _, e in slices]
        if masked is None or all(masked):
            return _X.slice_cat(input_tensor, starts, ends, mask, True)
        return _X.slice_cat_partly_masked(input_tensor, starts, ends, [bool(m) for m in masked], mask, True)


class MaskedSliceStackModule(torch.nn.Module):
    """stack([x[:, a:a+L], where(mask[B,1], 0, x[:, b:b+L]), ...], 0) -> [num, B, L]: forward(x, mask, starts, slice_len,
    masked) with a flag per slice (the stack form of the reference's test, tests/mlu/test_fuse_slice_where_cat.py:34-76)."""

    def forward(self, input_tensor, mask, starts, slice_len, masked):
        return _X.multi_slice_masked(input_tensor, [int(s) for s in starts], int(slice_len), [bool(m) for m in masked], mask, True)


class CatLastDimModule(torch.nn.Module):
    """cat / stack of several tensors along the last dim in one pass."""

    def forward(self, tensors, row_mask=None, zero_when=True):
        return _X.cat_lastdim(list(tensors), row_mask, bool(zero_when))


class GatherStackModule(torch.nn.Module):
    """F embedding lookups + where-mask + stack in one pass: forward(tables, idx[rows, F], mask)."""

    def forward(self, tables, idx, row_mask=None, zero_when=True):
        return _X.gather_stack(list(tables), idx, row_mask, bool(zero_when))


class RowGatherModule(torch.nn.Module):
    """table[idx] for a 2-D table and an integer index tensor of any shape -> [*idx.shape, D] (the single-lookup forms
    aten.embedding, aten.index.Tensor with one index on dim 0, aten.index_select on dim 0). ``wrap_negative``: indices
    below zero count from the end, as aten.index does (aten.embedding does not allow them)."""

    def __init__(self, wrap_negative: bool = False):
        super().__init__()
        self.wrap_negative = bool(wrap_negative)

    def forward(self, table, idx):
        shape = list(idx.shape)
        flat = idx.reshape(-1, 1).to(torch.int64)
        if self.wrap_negative:
            flat = torch.where(flat < 0, flat + table.shape[0], flat)
        return _X.gather_stack([table], flat, None, True).view(shape + [table.shape[1]])


class ComboSumModule(torch.nn.Module):
    """ComboSum3dInp target (structure/fuse_combosum.py:82-98): forward(input_list, dim) -> list of
    sum(x, dim[0]); one launch for the whole list (the MLU module splits by size,
    targets/mlu/structure_replacements/__init__.py:147-165)."""

    def forward(self, input_list, dim):
        d = dim[0] if isinstance(dim, (list, tuple)) else dim
        if d < 0:
            d += 3
        return _X.sum3d(list(input_list), int(d))


class ComboDenseModule(torch.nn.Module):
    """Many same-shape dense layers in one batched launch: forward(input_list, weight_list, bias_list, act,
    weight_trans) -> stacked [T, M, N] (callers unbind it). The place of FusedCombineBmm,
    targets/mlu/combo_matmul.py:22-113 (stacked bmm / grouped GEMM)."""

    def forward(self, input_list, weight_list, bias_list, act, weight_trans):
        return _X.combo_dense(list(input_list), list(weight_list), bool(weight_trans), list(bias_list), str(act))


class ComboBatchDenseModule(torch.nn.Module):
    """Many same-shape batched dense layers (lists of bmm) in one grouped launch: forward(input_list, weight_list,
    bias_list, act, weight_trans) -> [T, S, M, N] (callers unbind it). The place of FusedCombineBmm's stacked-bmm form,
    targets/mlu/combo_matmul.py:22-86."""

    def forward(self, input_list, weight_list, bias_list, act, weight_trans):
        return _X.combo_batch_dense(list(input_list), list(weight_list), bool(weight_trans), list(bias_list), str(act))


class DenseTowerModule(torch.nn.Module):
    """A chain of dense layers in one call: forward(x, weights, weight_trans, biases, acts) with one entry per layer.
    Stands where the reference fuses serial matmuls into one kernel (targets/mlu/fuse_densetower.py:272-316,
    triton_kernel/fused_serial_mm_2dot.py / _3dot.py). 16-bit towers: neighbouring narrow layers (N <= 256) run as one
    kernel per pair with the hidden activation kept on chip (xg_mlp2_bias_act). fp32 towers: the layers stay separate
    tensor-core GEMMs and the activations travel between them as bf16 planes. Towers of any dtype whose widths are all
    <= 128: runs of up to three layers in one kernel with the weights resident in shared memory (xg_mlp_small_bias_act)."""

    def forward(self, x, weights, weight_trans, biases, acts):
        return _X.dense_tower(x, list(weights), [bool(t) for t in weight_trans], list(biases), ",".join(str(a) for a in acts))


class SliceSumCatModule(torch.nn.Module):
    """slice(dim 1) -> sum(dim 1) -> cat(dim -1) of one [B, R, C] tensor in one pass: M(slice_param)(input) with
    slice_param = [(start, end), ...], the interface of targets/mlu/fuse_sum_cat.py:76-115 (SliceSumCatOperation)."""

    def __init__(self, slice_param):
        super().__init__()
        self.starts = [int(s) for s, _ in slice_param]
        self.ends = [int(e) for _, e in slice_param]

    def forward(self, input):
        return _X.slice_sum_cat(input, self.starts, self.ends)


class SumCatModule(torch.nn.Module):
    """sum(dim 1) -> cat(dim -1) of several [B, R_k, C] tensors (targets/mlu/fuse_sum_cat.py:20-43,
    ConcatenateSumOperation2): forward(inputs)."""

    def forward(self, inputs):
        return _X.sum_cat(list(inputs))


class MulSumCatModule(torch.nn.Module):
    """cat([sum(a_i * b_i, dim 1)], dim -1): forward(mul_list) with mul_list = [a_0, b_0, a_1, b_1, ...], the interface
    of targets/mlu/fuse_mul_sum_cat.py:16-50 (FusedMulSumCatReplacement); operands may broadcast over the batch."""

    def forward(self, mul_list):
        return _X.mul_sum_cat(list(mul_list[0::2]), list(mul_list[1::2]))


def get_structure_replacements(config=None) -> dict:
    """Structure-pattern name -> module (or (module, constraint_fn)), the dict that
    passes/patterns/targets/__init__.py:13-27 normalises."""
    return {
        "CustomRMSNorm": RMSNormModule,
        "CustomLayerNorm": LayerNormModule,
        "FusedSlice": FuseSliceModule,
        "FusedCatSlice": FuseSliceCatSameInputModule,
        "FusedSliceStackSum": FuseSliceCatSameInputModule,
        "FusedMultipleSliceCat": FuseSliceCatSameInputModule_v2,
        "ComboSum3dInp": ComboSumModule,
        "CustomDenseLayer": (DenseLayerModule, can_fuse_custom_denselayer),
        "CustomBatchDenseLayer": (BatchDenseLayerModule, can_fuse_custom_batch_denselayer),
    }
