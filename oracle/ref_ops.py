"""CPU oracle for the cuda_sm100 hot path — TEST INFRASTRUCTURE ONLY.

A restatement, in plain torch-on-CPU and numpy, of what the reference computes for each fused
pattern when its pattern pass is disabled and the graph runs as eager aten (the correctness bar of
the target). Only tests/, ``__graft_entry__.smoke()`` and the ``cpu_baseline`` / ``--impl reference``
legs of bench.py may import this module; the product package never does.

Parity status: pinned. tests/golden/ holds input/output fixtures produced by running the reference's
own modules and pass pipeline (tests/golden/gen_golden.py, executed where the reference is
importable); tests/test_oracle_golden.py checks every function below against them.

File:line citations are relative to the reference's src/xpu_graph/.
"""
from __future__ import annotations

from typing import List, Optional, Sequence, Tuple

import numpy as np
import torch
import torch.nn.functional as F

MAX_INT64 = 9223372036854775807


# ---- normalisation -------------------------------------------------------------------------
def rms_norm(x: torch.Tensor, weight: Optional[torch.Tensor], eps: float) -> torch.Tensor:
    """passes/patterns/utils/default_replacements.py:19-25 (DefaultRMSNorm.forward): upcast to fp32,
    F.rms_norm over the last dim, cast back."""
    w = weight.to(torch.float32) if weight is not None else None
    return F.rms_norm(x.to(torch.float32), x.shape[-1:], weight=w, eps=eps).to(x.dtype)


def layer_norm(x: torch.Tensor, weight: Optional[torch.Tensor], bias: Optional[torch.Tensor], eps: float) -> torch.Tensor:
    """passes/patterns/utils/default_replacements.py:28-36 (DefaultLayerNorm.forward)."""
    w = weight.to(torch.float32) if weight is not None else None
    b = bias.to(torch.float32) if bias is not None else None
    return F.layer_norm(x.to(torch.float32), x.shape[-1:], weight=w, bias=b, eps=eps).to(x.dtype)


def add_rms_norm(x, residual, weight, eps) -> Tuple[torch.Tensor, torch.Tensor]:
    """Eager form of the add + RMSNorm sub-graph: the sum is an aten.add in the promoted dtype
    (targets/mlu/fuse_add_norm.py:36-38), the norm then sees that rounded sum. Returns (normed, sum);
    the second result is the store_output_before_norm output (fuse_add_norm.py:118-121)."""
    dtype = torch.promote_types(x.dtype, residual.dtype)
    s = x.to(dtype) + residual.to(dtype)
    return rms_norm(s, weight, eps), s


def add_layer_norm(x, residual, weight, bias, eps) -> Tuple[torch.Tensor, torch.Tensor]:
    """See add_rms_norm; LayerNorm variant (targets/mlu/fuse_add_norm.py:40-48)."""
    dtype = torch.promote_types(x.dtype, residual.dtype)
    s = x.to(dtype) + residual.to(dtype)
    return layer_norm(s, weight, bias, eps), s


# ---- elementwise ---------------------------------------------------------------------------
def rotate_half(x: torch.Tensor) -> torch.Tensor:
    h = x.shape[-1] // 2
    return torch.cat((-x[..., h:], x[..., :h]), dim=-1)


def rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """The reference has no RoPE op; this is the aten chain the graph carries (2x slice, neg, cat,
    2x mul, add), evaluated op by op in the tensor dtype exactly as eager does."""
    return x * cos + rotate_half(x) * sin


def swiglu(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    """targets/npu/triton_kernel/fused_silu_mul.py:19-29 computes silu(x1) * x2; the eager graph is
    aten.silu followed by aten.mul in the tensor dtype."""
    return F.silu(gate) * up


# ---- dense layers --------------------------------------------------------------------------
_ACTS = {
    "none": lambda t: t,
    "gelu": lambda t: F.gelu(t),  # erf form: passes/patterns/common/gelu.py:29 emits aten.gelu
    "relu": F.relu,
    "silu": F.silu,
    "sigmoid": torch.sigmoid,
}


def dense(x, weight, weight_trans: bool, bias, act: str) -> torch.Tensor:
    """passes/patterns/structure/custom_denselayer.py:31-48 (match_mm_act): act(mm | addmm) with an
    optional transposed weight; bias forms as targets/mlu/structure_replacements/dense_layer_modules.py:22-57."""
    w = weight.t() if weight_trans else weight
    y = x @ w
    if bias is not None:
        y = y + bias
    return _ACTS[act](y)


def batch_dense(x, weight, weight_trans: bool, bias, act: str) -> torch.Tensor:
    """custom_denselayer.py:51-68 (match_bmm_act) / dense_layer_modules.py:71-120."""
    w = weight.transpose(-1, -2) if weight_trans else weight
    y = torch.bmm(x, w)
    if bias is not None:
        y = y + bias
    return _ACTS[act](y)


def dense_swiglu(x, w_gate, w_up) -> torch.Tensor:
    return F.silu(x @ w_gate.t()) * (x @ w_up.t())


# ---- attention -----------------------------------------------------------------------------
def sdpa(q, k, v, attn_mask=None, scale: Optional[float] = None, is_causal: bool = False) -> torch.Tensor:
    """passes/patterns/common/fuse_scaled_dot_product_attention.py:230-234: the fused node is
    aten.scaled_dot_product_attention(q, k, v, attn_mask=..., scale=...)."""
    return F.scaled_dot_product_attention(q, k, v, attn_mask=attn_mask, scale=scale, is_causal=is_causal)


def sdpa_math(q, k, v, attn_mask=None, scale: Optional[float] = None, is_causal: bool = False) -> torch.Tensor:
    """The un-fused sub-graph FusedSDPA matches (fuse_scaled_dot_product_attention.py:63-117):
    bmm(softmax(bmm(q, k^T) * scale + mask), v), in fp32. Used as the high-precision check."""
    qf, kf, vf = q.float(), k.float(), v.float()
    sc = scale if scale is not None else q.shape[-1] ** -0.5
    s = torch.matmul(qf, kf.transpose(-1, -2)) * sc
    if attn_mask is not None:
        s = s + attn_mask.float()
    if is_causal:
        sq, skv = s.shape[-2:]
        keep = torch.ones(sq, skv, dtype=torch.bool).tril(diagonal=0)  # top-left aligned, as aten
        s = s.masked_fill(~keep, float("-inf"))
    return torch.matmul(torch.softmax(s, dim=-1), vf)


# ---- copy fusions (numpy, bit-exact) ------------------------------------------------------
def _np(t):
    if isinstance(t, torch.Tensor):
        if t.dtype == torch.bfloat16:
            return t.view(torch.int16).numpy()
        return t.numpy()
    return np.asarray(t)


def _like(arr: np.ndarray, ref) -> torch.Tensor:
    out = torch.from_numpy(np.ascontiguousarray(arr))
    if isinstance(ref, torch.Tensor) and ref.dtype == torch.bfloat16:
        out = out.view(torch.bfloat16)
    return out


def normalise_slices(width: int, slices: Sequence[Tuple[int, int]]) -> List[Tuple[int, int]]:
    """passes/patterns/structure/fuse_slice_cat.py:39-44: an end of INT64_MAX means "to the end of the
    row", a negative end counts from the end."""
    out = []
    for s, e in slices:
        if e == MAX_INT64:
            e = width
        elif e < 0:
            e = width - (-e)
        out.append((s, min(e, width)))
    return out


def slice_cat(src, slices: Sequence[Tuple[int, int]]):
    """targets/mlu/structure_replacements/__init__.py:50-63 (FuseSliceCatSameInputModule): gather the
    columns [start, end) of every slice of a 2-D source, in order."""
    a = _np(src)
    if a.ndim != 2:
        raise NotImplementedError("input must be 2d")
    cols = [i for s, e in normalise_slices(a.shape[1], slices) for i in range(s, e)]
    return _like(a[:, cols], src)


def multi_slice(src, starts: Sequence[int], slice_len: int):
    """targets/mlu/structure_replacements/__init__.py:21-47 (FuseSliceModule): equal-length last-dim
    slices stacked on a new leading dim -> [num, *src.shape[:-1], slice_len]."""
    a = _np(src)
    return _like(np.stack([a[..., s:s + slice_len] for s in starts], axis=0), src)


def slice_cat_multi(src, many_slices: Sequence[Sequence[Tuple[int, int]]]):
    """targets/mlu/structure_replacements/__init__.py:66-144 (FuseSliceCatSameInputModule_v2): one
    slice_cat per group."""
    return [slice_cat(src, group) for group in many_slices]


def masked_slice_cat(src, mask, slices: Sequence[Tuple[int, int]]):
    """targets/mlu/triton_kernel/fused_slice_where_cat.py:62: where(mask[row], 0, value)."""
    out = _np(slice_cat(src, slices)).copy()
    m = _np(mask).reshape(-1).astype(bool)
    out[m, :] = 0
    return _like(out, src)


def cat_lastdim(tensors):
    return torch.cat(list(tensors), dim=-1)


def gather_stack(tables, idx, mask=None):
    """F aten.embedding lookups, where(mask[:, None], 0, e) and the stack/cat along the feature dim,
    as the recsys graph carries them after the common passes."""
    idx_np = _np(idx)
    parts = [_np(t)[idx_np[:, f]] for f, t in enumerate(tables)]
    out = np.concatenate(parts, axis=1)
    if mask is not None:
        out = out.copy()
        out[_np(mask).reshape(-1).astype(bool), :] = 0
    return _like(out, tables[0])


def combo_sum(inputs, dim):
    """targets/mlu/structure_replacements/__init__.py:147-165 (ComboSumModule): sum(x, dim[0]) for each
    3-D tensor of the list, i.e. the aten.sum.dim_IntList nodes that ComboSum3dInp batches
    (passes/patterns/structure/fuse_combosum.py:82-98)."""
    d = dim[0] if isinstance(dim, (list, tuple)) else dim
    return [x.sum(dim=d) for x in inputs]


def slice_sum_cat(src, slices):
    """cat([src[:, s:e, :].sum(1)], -1): the eager graph that targets/mlu/fuse_sum_cat.py:120-252 rewrites (and the
    fallback branch of SliceSumCatOperation.forward, :104-111)."""
    return torch.cat([src[:, s:e, :].sum(dim=1) for s, e in slices], dim=-1)


def sum_cat(inputs):
    """cat([x.sum(1)], -1) over different tensors (targets/mlu/fuse_sum_cat.py:20-43)."""
    return torch.cat([x.sum(dim=1) for x in inputs], dim=-1)


def mul_sum_cat(mul_list):
    """cat([(a_i * b_i).sum(1)], -1) with mul_list = [a_0, b_0, a_1, b_1, ...], batch broadcast allowed
    (targets/mlu/fuse_mul_sum_cat.py:16-50)."""
    return torch.cat([(mul_list[i] * mul_list[i + 1]).sum(dim=1) for i in range(0, len(mul_list), 2)], dim=-1)
