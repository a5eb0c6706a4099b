"""torch.library custom ops of the ``cuda_sm100`` target (namespace ``xg_sm100``).

PyTorch appears here only at the Python boundary: each op validates its tensors, allocates the
outputs with ``torch.empty`` on the input's device and hands raw pointers, extents and the current
CUDA stream to the C ABI of libxg_sm100.so. Ops are functional (``mutates_args=()``), registered for
the ``cuda`` device only (there is no CPU implementation on purpose) and carry fake implementations
so that the graph compiler can propagate shapes through them.

Registration pattern follows passes/patterns/targets/mlu/triton_kernel/fused_slice_where_cat.py:75,132
(``custom_op`` + ``register_fake``) of the reference.
"""
from __future__ import annotations

import ctypes
import os
from typing import List, Optional, Sequence

import torch

from . import lib as _lib

NS = "xg_sm100"

_DTYPE_CODE = {torch.float32: _lib.XG_F32, torch.bfloat16: _lib.XG_BF16, torch.float16: _lib.XG_F16}


def _code(dtype: torch.dtype) -> int:
    try:
        return _DTYPE_CODE[dtype]
    except KeyError:
        raise TypeError(f"xg_sm100: unsupported dtype {dtype}") from None


def _stream(t: torch.Tensor) -> int:
    return torch.cuda.current_stream(t.device).cuda_stream


def _ptr(t: Optional[torch.Tensor]):
    return None if t is None else t.data_ptr()


def _rows_view(x: torch.Tensor) -> torch.Tensor:
    """View x as [rows, hidden] with a contiguous last dim; copies only when strides do not allow it."""
    h = x.shape[-1]
    if x.dim() == 2 and x.stride(1) == 1:
        return x
    if x.is_contiguous():
        return x.view(-1, h)
    return x.contiguous().view(-1, h)


def _row_stride(x2: torch.Tensor) -> int:
    return x2.stride(0) if x2.shape[0] > 1 else max(x2.stride(0), x2.shape[1])


def _empty_like_layout(x: torch.Tensor) -> torch.Tensor:
    """[B, H, S, D] output that keeps x's memory layout when x is a [B, S, H, D] buffer viewed with
    dims 1 and 2 swapped (so that the transpose + reshape after attention stays a view); contiguous
    otherwise."""
    B, H, S, D = x.shape
    if x.stride(3) == 1 and x.stride(1) == D and x.stride(2) == H * D and x.stride(0) == S * H * D and H > 1 and S > 1:
        return torch.empty((B, S, H, D), dtype=x.dtype, device=x.device).transpose(1, 2)
    return torch.empty((B, H, S, D), dtype=x.dtype, device=x.device)


def _coef(w: torch.Tensor, dtype: torch.dtype) -> torch.Tensor:
    """Affine coefficients are passed as fp32 or as the activation dtype."""
    if w.dtype not in (torch.float32, dtype):
        w = w.to(torch.float32)
    return w.contiguous()


# --------------------------------------------------------------------------------------------
# normalisation
# --------------------------------------------------------------------------------------------
def _norm_call(kind: str, x, residual, weight, bias, eps: float, want_sum: bool):
    L = _lib.load()
    x2 = _rows_view(x)
    rows, hidden = x2.shape
    r2 = None
    if residual is not None:
        if residual.shape != x.shape or residual.dtype != x.dtype:
            raise ValueError("xg_sm100 norm: residual must match x in shape and dtype")
        r2 = _rows_view(residual)
    w = _coef(weight, x.dtype)
    b = _coef(bias, x.dtype).to(w.dtype) if bias is not None else None
    y = torch.empty((rows, hidden), dtype=x.dtype, device=x.device)
    s = torch.empty((rows, hidden), dtype=x.dtype, device=x.device) if want_sum else None
    code, wcode = _code(x.dtype), _code(w.dtype)
    if kind == "rms":
        rc = L.xg_rmsnorm(_ptr(x2), _ptr(r2), _ptr(w), _ptr(y), _ptr(s), rows, hidden, _row_stride(x2),
                          _row_stride(r2) if r2 is not None else 0, float(eps), code, wcode, _stream(x))
        _lib.check(rc, "xg_rmsnorm")
    else:
        rc = L.xg_layernorm(_ptr(x2), _ptr(r2), _ptr(w), _ptr(b), _ptr(y), _ptr(s), rows, hidden, _row_stride(x2),
                            _row_stride(r2) if r2 is not None else 0, float(eps), code, wcode, _stream(x))
        _lib.check(rc, "xg_layernorm")
    y = y.view(x.shape)
    if want_sum:
        return y, s.view(x.shape)
    return y


@torch.library.custom_op(f"{NS}::rms_norm", mutates_args=(), device_types="cuda")
def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    return _norm_call("rms", x, None, weight, None, eps, False)


@rms_norm.register_fake
def _(x, weight, eps):
    return torch.empty(x.shape, dtype=x.dtype, device=x.device)


@torch.library.custom_op(f"{NS}::add_rms_norm", mutates_args=(), device_types="cuda")
def add_rms_norm(x: torch.Tensor, residual: torch.Tensor, weight: torch.Tensor, eps: float) -> List[torch.Tensor]:
    y, s = _norm_call("rms", x, residual, weight, None, eps, True)
    return [y, s]


@add_rms_norm.register_fake
def _(x, residual, weight, eps):
    return [torch.empty(x.shape, dtype=x.dtype, device=x.device), torch.empty(x.shape, dtype=x.dtype, device=x.device)]


@torch.library.custom_op(f"{NS}::add_rms_norm_y", mutates_args=(), device_types="cuda")
def add_rms_norm_y(x: torch.Tensor, residual: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    return _norm_call("rms", x, residual, weight, None, eps, False)


@add_rms_norm_y.register_fake
def _(x, residual, weight, eps):
    return torch.empty(x.shape, dtype=x.dtype, device=x.device)


@torch.library.custom_op(f"{NS}::layer_norm", mutates_args=(), device_types="cuda")
def layer_norm(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor], eps: float) -> torch.Tensor:
    return _norm_call("ln", x, None, weight, bias, eps, False)


@layer_norm.register_fake
def _(x, weight, bias, eps):
    return torch.empty(x.shape, dtype=x.dtype, device=x.device)


@torch.library.custom_op(f"{NS}::add_layer_norm", mutates_args=(), device_types="cuda")
def add_layer_norm(x: torch.Tensor, residual: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor],
                   eps: float) -> List[torch.Tensor]:
    y, s = _norm_call("ln", x, residual, weight, bias, eps, True)
    return [y, s]


@add_layer_norm.register_fake
def _(x, residual, weight, bias, eps):
    return [torch.empty(x.shape, dtype=x.dtype, device=x.device), torch.empty(x.shape, dtype=x.dtype, device=x.device)]


@torch.library.custom_op(f"{NS}::add_layer_norm_y", mutates_args=(), device_types="cuda")
def add_layer_norm_y(x: torch.Tensor, residual: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor],
                     eps: float) -> torch.Tensor:
    return _norm_call("ln", x, residual, weight, bias, eps, False)


@add_layer_norm_y.register_fake
def _(x, residual, weight, bias, eps):
    return torch.empty(x.shape, dtype=x.dtype, device=x.device)


# --------------------------------------------------------------------------------------------
# elementwise
# --------------------------------------------------------------------------------------------
@torch.library.custom_op(f"{NS}::rope", mutates_args=(), device_types="cuda")
def rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """x: [B, H, S, D] (any strides with D contiguous); cos/sin broadcastable from [S, D]."""
    if x.dim() != 4:
        raise ValueError("xg_sm100::rope expects [B, H, S, D]")
    B, H, S, D = x.shape
    if x.stride(3) != 1:
        x = x.contiguous()
    cos2 = cos.reshape(S, D).to(x.dtype).contiguous()
    sin2 = sin.reshape(S, D).to(x.dtype).contiguous()
    y = _empty_like_layout(x)
    rc = _lib.load().xg_rope(_ptr(x), _ptr(cos2), _ptr(sin2), _ptr(y), B, H, S, D, x.stride(0), x.stride(1), x.stride(2),
                             y.stride(0), y.stride(1), y.stride(2), _code(x.dtype), _stream(x))
    _lib.check(rc, "xg_rope")
    return y


@rope.register_fake
def _(x, cos, sin):
    return _empty_like_layout(x)


@torch.library.custom_op(f"{NS}::swiglu", mutates_args=(), device_types="cuda")
def swiglu(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    if gate.shape != up.shape or gate.dtype != up.dtype:
        raise ValueError("xg_sm100::swiglu: gate and up must match")
    g2, u2 = _rows_view(gate), _rows_view(up)
    rows, cols = g2.shape
    out = torch.empty((rows, cols), dtype=gate.dtype, device=gate.device)
    rc = _lib.load().xg_swiglu(_ptr(g2), _ptr(u2), _ptr(out), rows, cols, _row_stride(g2), _row_stride(u2), cols,
                               _code(gate.dtype), _stream(gate))
    _lib.check(rc, "xg_swiglu")
    return out.view(gate.shape)


@swiglu.register_fake
def _(gate, up):
    return torch.empty(gate.shape, dtype=gate.dtype, device=gate.device)


# --------------------------------------------------------------------------------------------
# dense layers
# --------------------------------------------------------------------------------------------
def _mat(t: torch.Tensor) -> torch.Tensor:
    return t if t.stride(-1) == 1 else t.contiguous()


def _weight_rows(w: torch.Tensor, weight_trans: bool):
    """A 2-D weight with contiguous rows and the orientation flag that goes with it. A transposed view of a contiguous
    matrix (``w.T``, what F.linear(x, w.T) or x @ w.t() hand over) is read through its base in the other orientation -
    the kernels take both [N, K] and [K, N] - instead of being copied on every call."""
    if w.dim() == 2 and w.stride(-1) != 1 and w.stride(0) == 1 and w.shape[0] > 1:
        return w.t(), not weight_trans
    return _mat(w), weight_trans


# fp32 dense layers above this many FLOPs run on the bf16 tensor cores from three bf16 planes per operand
# (fp32-grade results at several times the FMA rate); smaller ones stay on the FMA kernel, whose launch is cheaper.
F32_TENSOR_MIN_FLOPS = int(os.environ.get("XG_F32_TENSOR_MIN_FLOPS", str(1 << 30)))
F32_TENSOR_MAX_K = 8192  # measured error vs fp64 grows from 2e-6 (K = 1728) to 6e-6 (K = 4096) of the output scale


def _f32_on_tensor_cores(M: int, N: int, K: int) -> bool:
    if os.environ.get("XG_F32_TENSOR", "1") == "0":
        return False
    return 2 * M * N * K >= F32_TENSOR_MIN_FLOPS and K <= F32_TENSOR_MAX_K


def _planes_tag(weight: torch.Tensor, weight_trans: bool):
    """Key under which a weight's bf16 planes are kept, or None when the tensor cannot be tracked: tensors made under
    torch.inference_mode() have no version counter, so their planes are rebuilt on every call."""
    try:
        version = weight._version
    except RuntimeError:
        return None
    return (version, weight.data_ptr(), tuple(weight.shape), tuple(weight.stride()), bool(weight_trans))


def invalidate_weight_planes(weight: torch.Tensor) -> None:
    """Drop the bf16 planes kept for an fp32 weight. Needed after the weight was rewritten through ``.data`` (or any
    other route that does not bump its version counter): the planes are keyed on the counter and would go stale."""
    try:
        del weight._xg_bf16_planes
    except AttributeError:
        pass


def _weight_planes(L, weight: torch.Tensor, weight_trans: bool, N: int, K: int) -> torch.Tensor:
    """The three bf16 planes of an fp32 weight, [N, 3*Kp]. They ride on the weight tensor object itself and are
    rebuilt when its version counter, layout or orientation changes, so a dense layer's weight is split once in
    inference and the planes go away with the tensor; a fresh view of a weight is simply split again. In-place
    updates through ``weight.data`` do not move the counter: call ``invalidate_weight_planes`` after those. A
    captured CUDA graph replays with the planes that existed at capture."""
    tag = _planes_tag(weight, weight_trans)
    kept = getattr(weight, "_xg_bf16_planes", None) if tag is not None else None
    if kept is not None and kept[0] == tag:
        return kept[1]
    Kp = int(L.xg_gemm_f32x3_padded_k(K))
    w3 = torch.empty((N, 3 * Kp), dtype=torch.bfloat16, device=weight.device)
    rc = L.xg_split_bf16x3(_ptr(weight), N, K, _row_stride(weight), 0 if weight_trans else 1, _ptr(w3), _stream(weight))
    _lib.check(rc, "xg_split_bf16x3")
    if tag is not None:
        try:
            weight._xg_bf16_planes = (tag, w3)
        except (AttributeError, RuntimeError):  # a tensor type without instance attributes: no reuse
            pass
    return w3


def _dense_f32x3(L, x, weight, weight_trans, bias, residual, ldr, act, out, M, N, K):
    Kp = int(L.xg_gemm_f32x3_padded_k(K))
    w3 = _weight_planes(L, weight, weight_trans, N, K)
    a3 = torch.empty((M, 3 * Kp), dtype=torch.bfloat16, device=x.device)
    rc = L.xg_split_bf16x3(_ptr(x), M, K, _row_stride(x), 0, _ptr(a3), _stream(x))
    _lib.check(rc, "xg_split_bf16x3")
    rc = L.xg_gemm_f32x3(_ptr(a3), _ptr(w3), _ptr(bias), _ptr(residual), _ptr(out), M, N, K, N, ldr,
                         _lib.ACT_CODES[act], 0, _stream(x))
    _lib.check(rc, "xg_gemm_f32x3")
    return out


def dense_tower_eligible(M: int, dims: Sequence[int]) -> bool:
    """Every layer of an fp32 tower [K0 -> K1 -> ... -> Kn] over M rows qualifies for the tensor-core path."""
    return all(_f32_on_tensor_cores(M, dims[i + 1], dims[i]) for i in range(len(dims) - 1))


def mlp2_eligible(M: int, K1: int, N1: int, N2: int, dtype: torch.dtype, trans1: bool = True, trans2: bool = True) -> bool:
    """Two chained 16-bit dense layers [K1 -> N1 -> N2] fit the single-kernel form: 16 <= N1 <= 256 with N1 % 8 == 0,
    N2 <= 256, K1 % 8 == 0 (the limits of xg_mlp2_supported); a weight stored [K, N] (not transposed) needs N % 8 == 0."""
    return (dtype in (torch.bfloat16, torch.float16) and M > 0 and K1 >= 8 and K1 % 8 == 0
            and 16 <= N1 <= 256 and N1 % 8 == 0 and 1 <= N2 <= 256 and (bool(trans2) or N2 % 8 == 0))


def _mlp_dims(x, ws, weights_kn, who):
    """Layer widths of a chain; weight l is [N, K] unless bit l of weights_kn says [K, N]."""
    k = x.shape[1]
    dims = []
    for l, w in enumerate(ws):
        kn = (weights_kn >> l) & 1
        wk, wn = (w.shape[0], w.shape[1]) if kn else (w.shape[1], w.shape[0])
        if wk != k:
            raise ValueError(f"xg_sm100::{who}: inner dimensions differ")
        if w.dtype != x.dtype:
            raise ValueError(f"xg_sm100::{who}: x and the weights must share a dtype")
        dims.append(wn)
        k = wn
    return dims


@torch.library.custom_op(f"{NS}::mlp2", mutates_args=(), device_types="cuda")
def mlp2(x: torch.Tensor, w1: torch.Tensor, b1: Optional[torch.Tensor], w2: torch.Tensor, b2: Optional[torch.Tensor],
         act1: str, act2: str, weights_kn: int = 0) -> torch.Tensor:
    """act2(act1(x @ W1 + b1) @ W2 + b2) in one kernel; weight l is given as [N, K] (nn.Linear's layout) or, if bit l of
    weights_kn is set, as [K, N]; the hidden activation stays on chip (rounded to the tensors' 16-bit dtype between the
    layers, as the unfused graph does)."""
    if x.dim() != 2 or w1.dim() != 2 or w2.dim() != 2:
        raise ValueError("xg_sm100::mlp2 expects 2-D x, w1 and w2")
    x, w1, w2 = _mat(x), _mat(w1), _mat(w2)
    M, K1 = x.shape
    N1, N2 = _mlp_dims(x, (w1, w2), weights_kn, "mlp2")
    b1 = b1.to(x.dtype).contiguous() if b1 is not None else None
    b2 = b2.to(x.dtype).contiguous() if b2 is not None else None
    if (b1 is not None and b1.numel() != N1) or (b2 is not None and b2.numel() != N2):
        raise ValueError("xg_sm100::mlp2: a bias does not match its layer's width")
    out = torch.empty((M, N2), dtype=x.dtype, device=x.device)
    if M == 0:
        return out
    L = _lib.load()
    rc = L.xg_mlp2_bias_act(_ptr(x), _ptr(w1), _ptr(b1), _ptr(w2), _ptr(b2), _ptr(out), M, K1, N1, N2, _row_stride(x),
                            _row_stride(w1), _row_stride(w2), N2, _lib.ACT_CODES[act1], _lib.ACT_CODES[act2], weights_kn,
                            _code(x.dtype), _stream(x))
    _lib.check(rc, "xg_mlp2_bias_act")
    return out


@mlp2.register_fake
def _(x, w1, b1, w2, b2, act1, act2, weights_kn=0):
    return torch.empty((x.shape[0], w2.shape[1] if (weights_kn >> 1) & 1 else w2.shape[0]), dtype=x.dtype, device=x.device)


def mlp3_eligible(M: int, K1: int, N1: int, N2: int, N3: int, dtype: torch.dtype, trans=(True, True, True)) -> bool:
    """Three chained 16-bit dense layers fit the single-kernel form (the limits of xg_mlp3_supported)."""
    return (mlp2_eligible(M, K1, N1, N2, dtype, trans[0], trans[1]) and 16 <= N2 and N2 % 8 == 0
            and 1 <= N3 <= 256 and (bool(trans[2]) or N3 % 8 == 0))


@torch.library.custom_op(f"{NS}::mlp3", mutates_args=(), device_types="cuda")
def mlp3(x: torch.Tensor, w1: torch.Tensor, b1: Optional[torch.Tensor], w2: torch.Tensor, b2: Optional[torch.Tensor],
         w3: torch.Tensor, b3: Optional[torch.Tensor], act1: str, act2: str, act3: str, weights_kn: int = 0) -> torch.Tensor:
    """Three chained dense layers in one kernel (see mlp2)."""
    if x.dim() != 2 or w1.dim() != 2 or w2.dim() != 2 or w3.dim() != 2:
        raise ValueError("xg_sm100::mlp3 expects 2-D x and weights")
    x, w1, w2, w3 = _mat(x), _mat(w1), _mat(w2), _mat(w3)
    M, K1 = x.shape
    N1, N2, N3 = _mlp_dims(x, (w1, w2, w3), weights_kn, "mlp3")
    bs = [b.to(x.dtype).contiguous() if b is not None else None for b in (b1, b2, b3)]
    if any(b is not None and b.numel() != n for b, n in zip(bs, (N1, N2, N3))):
        raise ValueError("xg_sm100::mlp3: a bias does not match its layer's width")
    out = torch.empty((M, N3), dtype=x.dtype, device=x.device)
    if M == 0:
        return out
    L = _lib.load()
    rc = L.xg_mlp3_bias_act(_ptr(x), _ptr(w1), _ptr(bs[0]), _ptr(w2), _ptr(bs[1]), _ptr(w3), _ptr(bs[2]), _ptr(out), M, K1, N1,
                            N2, N3, _row_stride(x), _row_stride(w1), _row_stride(w2), _row_stride(w3), N3, _lib.ACT_CODES[act1],
                            _lib.ACT_CODES[act2], _lib.ACT_CODES[act3], weights_kn, _code(x.dtype), _stream(x))
    _lib.check(rc, "xg_mlp3_bias_act")
    return out


@mlp3.register_fake
def _(x, w1, b1, w2, b2, w3, b3, act1, act2, act3, weights_kn=0):
    return torch.empty((x.shape[0], w3.shape[1] if (weights_kn >> 2) & 1 else w3.shape[0]), dtype=x.dtype, device=x.device)


MLP_SMALL_MAX_DIM = 128
MLP_SMALL_MAX_WEIGHTS = 24576


def _small_run(dims: Sequence[int], i: int, n: int, dtype: torch.dtype, M: int) -> int:
    """How many layers starting at layer i (at most three) run together on the weights-in-shared-memory kernel."""
    for run in (3, 2):
        if i + run <= n and mlp_small_worth_it(M, dims[i:i + run + 1], dtype):
            return run
    return 1


def mlp_small_worth_it(M: int, dims: Sequence[int], dtype: torch.dtype) -> bool:
    """The one-launch FMA tower is the faster form where a launch per layer is mostly launch and latency: few rows, or
    very narrow layers. Measured on B200 (us, one kernel / a launch per layer): 16 rows of 20 -> 32 -> 16 -> 1 fp16
    8.3 / 26.5; 16384 rows of 64 -> 32 -> 16 -> 1 fp32 20.5 / 21.7; 16384 rows of 128 -> 64 -> 32 fp32 43.5 / 24.6."""
    if not mlp_small_eligible(dims, dtype):
        return False
    weights = sum(((dims[i] + 3) // 4 * 4) * dims[i + 1] for i in range(len(dims) - 1))
    return M <= 2048 or weights <= 4096


def mlp_small_eligible(dims: Sequence[int], dtype: torch.dtype) -> bool:
    """A tower [K0 -> N1 -> ... ] of one to three layers fits the weights-in-shared-memory kernel (the limits of
    xg_mlp_small_supported: every width <= 128, at most 24576 weight elements with K padded to a multiple of 4)."""
    n = len(dims) - 1
    if dtype not in (torch.float32, torch.bfloat16, torch.float16) or not 1 <= n <= 3:
        return False
    if any(d < 1 or d > MLP_SMALL_MAX_DIM for d in dims):
        return False
    return sum(((dims[i] + 3) // 4 * 4) * dims[i + 1] for i in range(n)) <= MLP_SMALL_MAX_WEIGHTS


@torch.library.custom_op(f"{NS}::mlp_small", mutates_args=(), device_types="cuda")
def mlp_small(x: torch.Tensor, weights: List[torch.Tensor], biases: List[Optional[torch.Tensor]], act_names: str,
              weights_kn: int) -> torch.Tensor:
    """One to three chained narrow dense layers in one launch with every weight resident in shared memory (FMA
    arithmetic, fp32 accumulation, any row length); weight l is [N, K] unless bit l of weights_kn says [K, N]."""
    acts = act_names.split(",")
    n = len(weights)
    if x.dim() != 2 or len(biases) != n or len(acts) != n or any(w.dim() != 2 for w in weights):
        raise ValueError("xg_sm100::mlp_small expects a 2-D x and one 2-D weight, bias and activation per layer")
    x = _mat(x)
    ws = [_mat(w) for w in weights]
    dims = [x.shape[1]] + _mlp_dims(x, ws, weights_kn, "mlp_small")
    bs = [None if b is None else b.reshape(-1).to(x.dtype).contiguous() for b in biases]
    if any(b is not None and b.numel() != dims[i + 1] for i, b in enumerate(bs)):
        raise ValueError("xg_sm100::mlp_small: a bias does not match its layer's width")
    M = x.shape[0]
    out = torch.empty((M, dims[-1]), dtype=x.dtype, device=x.device)
    if M == 0:
        return out
    rc = _lib.load().xg_mlp_small_bias_act(
        _ptr(x), _lib.ptr_array([w.data_ptr() for w in ws]), _lib.ptr_array([0 if b is None else b.data_ptr() for b in bs]),
        _ptr(out), M, _lib.i64_array(dims), n, _row_stride(x), _lib.i64_array([_row_stride(w) for w in ws]), dims[-1],
        (ctypes.c_int * n)(*[_lib.ACT_CODES[a] for a in acts]), weights_kn, _code(x.dtype), _stream(x))
    _lib.check(rc, "xg_mlp_small_bias_act")
    return out


@mlp_small.register_fake
def _(x, weights, biases, act_names, weights_kn):
    w = weights[-1]
    last = len(weights) - 1
    return torch.empty((x.shape[0], w.shape[1] if (weights_kn >> last) & 1 else w.shape[0]), dtype=x.dtype, device=x.device)


@torch.library.custom_op(f"{NS}::dense_tower", mutates_args=(), device_types="cuda")
def dense_tower(x: torch.Tensor, weights: List[torch.Tensor], weight_trans: List[bool], biases: List[Optional[torch.Tensor]],
                act_names: str) -> torch.Tensor:
    """A chain of fp32 dense layers y_i = act_i(y_{i-1} @ W_i + b_i); act_names = "relu,relu,none" (one per layer).
    On the tensor-core path every inner layer's epilogue writes its result straight as the next layer's three bf16
    planes, so no fp32 activation is stored or re-read between layers; the last layer stores fp32."""
    acts = act_names.split(",")
    if not (len(acts) == len(weights) == len(weight_trans) == len(biases)):
        raise ValueError("xg_sm100::dense_tower: one weight, orientation, bias and activation per layer")
    if x.dim() != 2 or x.dtype not in (torch.float32, torch.bfloat16, torch.float16):
        raise ValueError("xg_sm100::dense_tower expects a 2-D floating-point input")
    n = len(weights)
    M = x.shape[0]
    dims = [x.shape[1]] + [(w.shape[0] if t else w.shape[1]) for w, t in zip(weights, weight_trans)]
    if x.dtype != torch.float32:
        rows = [_weight_rows(w, t) for w, t in zip(weights, weight_trans)]
        weights, weight_trans = [r[0] for r in rows], [r[1] for r in rows]
        # 16-bit towers: runs of three or two neighbouring layers that fit the chained-layer kernel run as one launch
        # each, the rest layer by layer
        y, i = x, 0
        while i < n:
            kn = lambda a, b: sum((0 if weight_trans[i + l] else 1) << l for l in range(a, b))  # noqa: E731
            if i + 2 < n and mlp3_eligible(M, dims[i], dims[i + 1], dims[i + 2], dims[i + 3], x.dtype, weight_trans[i:i + 3]):
                y = mlp3(y, weights[i], biases[i], weights[i + 1], biases[i + 1], weights[i + 2], biases[i + 2],
                         acts[i], acts[i + 1], acts[i + 2], kn(0, 3))
                i += 3
            elif i + 1 < n and mlp2_eligible(M, dims[i], dims[i + 1], dims[i + 2], x.dtype, weight_trans[i], weight_trans[i + 1]):
                y = mlp2(y, weights[i], biases[i], weights[i + 1], biases[i + 1], acts[i], acts[i + 1], kn(0, 2))
                i += 2
            else:
                run = _small_run(dims, i, n, x.dtype, M)
                if run >= 2:  # narrow layers no tensor map addresses (or too narrow for a tile): weights in shared memory
                    y = mlp_small(y, weights[i:i + run], biases[i:i + run], ",".join(acts[i:i + run]), kn(0, run))
                    i += run
                else:
                    y = dense(y, weights[i], weight_trans[i], biases[i], None, acts[i])
                    i += 1
        return y
    if not dense_tower_eligible(M, dims):
        y, i = x, 0
        while i < n:
            run = _small_run(dims, i, n, x.dtype, M)
            if run >= 2:
                kn_bits = sum((0 if weight_trans[i + l] else 1) << l for l in range(run))
                y = mlp_small(y, weights[i:i + run], biases[i:i + run], ",".join(acts[i:i + run]), kn_bits)
                i += run
            else:
                y = dense(y, weights[i], weight_trans[i], biases[i], None, acts[i])
                i += 1
        return y
    L = _lib.load()
    x = _mat(x)
    a3 = torch.empty((M, 3 * int(L.xg_gemm_f32x3_padded_k(dims[0]))), dtype=torch.bfloat16, device=x.device)
    rc = L.xg_split_bf16x3(_ptr(x), M, dims[0], _row_stride(x), 0, _ptr(a3), _stream(x))
    _lib.check(rc, "xg_split_bf16x3")
    for i in range(n):
        K, N = dims[i], dims[i + 1]
        w = _mat(weights[i])
        if (w.shape[1] if weight_trans[i] else w.shape[0]) != K:
            raise ValueError("xg_sm100::dense_tower: inner dimensions differ")
        w3 = _weight_planes(L, w, weight_trans[i], N, K)
        b = biases[i].to(torch.float32).contiguous() if biases[i] is not None else None
        last = i == n - 1
        if last:
            out = torch.empty((M, N), dtype=torch.float32, device=x.device)
        else:
            out = torch.empty((M, 3 * int(L.xg_gemm_f32x3_padded_k(N))), dtype=torch.bfloat16, device=x.device)
        rc = L.xg_gemm_f32x3(_ptr(a3), _ptr(w3), _ptr(b), None, _ptr(out), M, N, K, N, 0, _lib.ACT_CODES[acts[i]],
                             0 if last else 1, _stream(x))
        _lib.check(rc, "xg_gemm_f32x3")
        a3 = out
    return a3


@dense_tower.register_fake
def _(x, weights, weight_trans, biases, act_names):
    N = weights[-1].shape[0] if weight_trans[-1] else weights[-1].shape[1]
    return torch.empty((x.shape[0], N), dtype=x.dtype, device=x.device)


@torch.library.custom_op(f"{NS}::dense", mutates_args=(), device_types="cuda")
def dense(x: torch.Tensor, weight: torch.Tensor, weight_trans: bool, bias: Optional[torch.Tensor],
          residual: Optional[torch.Tensor], act: str) -> torch.Tensor:
    """act(x @ W + bias + residual); W = weight ([K, N]) or weight^T (weight is [N, K], weight_trans)."""
    if x.dim() != 2 or weight.dim() != 2:
        raise ValueError("xg_sm100::dense expects 2-D x and weight")
    x = _mat(x)
    weight, weight_trans = _weight_rows(weight, weight_trans)
    M, K = x.shape
    N = weight.shape[0] if weight_trans else weight.shape[1]
    if (weight.shape[1] if weight_trans else weight.shape[0]) != K:
        raise ValueError("xg_sm100::dense: inner dimensions differ")
    if bias is not None:
        bias = bias.to(x.dtype).contiguous()
    ldr = 0
    if residual is not None:
        residual = _mat(residual.to(x.dtype))
        ldr = _row_stride(residual)
    out = torch.empty((M, N), dtype=x.dtype, device=x.device)
    L = _lib.load()
    if x.dtype == torch.float32 and _f32_on_tensor_cores(M, N, K):
        return _dense_f32x3(L, x, weight, weight_trans, bias, residual, ldr, act, out, M, N, K)
    ws, ws_bytes = None, 0
    if x.dtype != torch.float32 and M <= 128:
        ws_bytes = int(L.xg_gemm_workspace_bytes(M, N, K, _code(x.dtype)))
        if ws_bytes > 0:  # split-K scratch for weight-streaming shapes (small M)
            ws = torch.empty(ws_bytes, dtype=torch.uint8, device=x.device)
    rc = L.xg_gemm_bias_act_ws(_ptr(x), _ptr(weight), _ptr(bias), _ptr(residual), _ptr(out), M, N, K,
                               _row_stride(x), _row_stride(weight), N, ldr, 1 if weight_trans else 0,
                               _lib.ACT_CODES[act], _code(x.dtype), _ptr(ws), ws_bytes, _stream(x))
    _lib.check(rc, "xg_gemm_bias_act")
    return out


@dense.register_fake
def _(x, weight, weight_trans, bias, residual, act):
    N = weight.shape[0] if weight_trans else weight.shape[1]
    return torch.empty((x.shape[0], N), dtype=x.dtype, device=x.device)


@torch.library.custom_op(f"{NS}::batch_dense", mutates_args=(), device_types="cuda")
def batch_dense(x: torch.Tensor, weight: torch.Tensor, weight_trans: bool, bias: Optional[torch.Tensor],
                residual: Optional[torch.Tensor], act: str) -> torch.Tensor:
    """Batched dense: x [b, M, K], weight [b, K, N] or [b, N, K]; bias [b, 1, N] / [b, N]; residual [b, M, N]."""
    x = x.contiguous()
    weight = weight.contiguous()
    b, M, K = x.shape
    N = weight.shape[1] if weight_trans else weight.shape[2]
    sbias = 0
    if bias is not None:
        bias = bias.to(x.dtype).broadcast_to((b, 1, N)).contiguous()
        sbias = N
    sr = 0
    if residual is not None:
        residual = residual.to(x.dtype).broadcast_to((b, M, N)).contiguous()
        sr = M * N
    out = torch.empty((b, M, N), dtype=x.dtype, device=x.device)
    rc = _lib.load().xg_bgemm_bias_act(_ptr(x), _ptr(weight), _ptr(bias), _ptr(residual), _ptr(out), b, M, N, K, K,
                                       weight.shape[2], N, N, M * K, weight.shape[1] * weight.shape[2], sbias, sr, M * N,
                                       1 if weight_trans else 0, _lib.ACT_CODES[act], _code(x.dtype), _stream(x))
    _lib.check(rc, "xg_bgemm_bias_act")
    return out


@batch_dense.register_fake
def _(x, weight, weight_trans, bias, residual, act):
    N = weight.shape[1] if weight_trans else weight.shape[2]
    return torch.empty((x.shape[0], x.shape[1], N), dtype=x.dtype, device=x.device)


@torch.library.custom_op(f"{NS}::combo_dense", mutates_args=(), device_types="cuda")
def combo_dense(inputs: List[torch.Tensor], weights: List[torch.Tensor], weight_trans: bool,
                biases: List[Optional[torch.Tensor]], act: str) -> torch.Tensor:
    """T same-shape dense layers act(x_t @ W_t + b_t) in one launch; returns the stacked [T, M, N] result. Operands are
    used in place through the grouped kernels (a pointer per layer, no stacking copy: tensor-core kernel for 16-bit,
    FMA kernel for fp32); what those cannot address goes through the batched form, for which operands that are not
    consecutive slabs of one buffer are stacked first. b_t: None, a row of N, or a full [M, N] addend."""
    T = len(inputs)
    if T == 0 or len(weights) != T or len(biases) != T:
        raise ValueError("xg_sm100::combo_dense: one input, weight and bias entry per layer")
    grouped = _combo_dense_grouped(inputs, weights, weight_trans, biases, act)
    if grouped is not None:
        return grouped
    x = _stack_or_view(inputs)
    w = _stack_or_view(weights)
    M = inputs[0].shape[0]
    N = weights[0].shape[0] if weight_trans else weights[0].shape[1]
    kinds = {_bias_kind(b, M, N) for b in biases}
    if len(kinds) != 1:
        raise ValueError("xg_sm100::combo_dense: the layers' biases must be of one kind (none, a row of N, or [M, N])")
    kind = kinds.pop()
    b = torch.stack([bi.reshape(1, -1) for bi in biases]) if kind == 1 else None  # [T, 1, N]
    r = torch.stack([bi.reshape(M, N) for bi in biases]) if kind == 2 else None   # [T, M, N]
    return batch_dense(x, w, weight_trans, b, r, act)


def _bias_kind(b: Optional[torch.Tensor], M: int, N: int) -> int:
    """0: none; 1: a per-column bias ([N] or [1, N]); 2: a full [M, N] addend (dense_layer_modules.py:22-57)."""
    if b is None:
        return 0
    if b.numel() == N and (b.dim() == 1 or (b.dim() == 2 and b.shape[0] == 1)):
        return 1
    if b.dim() == 2 and tuple(b.shape) == (M, N):
        return 2
    raise ValueError(f"xg_sm100::combo_dense: bias of shape {tuple(b.shape)} for an [{M}, {N}] result")


def _combo_dense_grouped(inputs, weights, weight_trans: bool, biases, act: str) -> Optional[torch.Tensor]:
    """The grouped launch: every layer's operands are used where they are (a pointer per entry), the results land side
    by side in one [T, M, N] tensor. A bias is a row of N or a full [M, N] addend, layer by layer. Returns None when
    the operands do not qualify (shapes that differ; 16-bit rows a tensor map cannot address), and the caller falls back
    to the stacked batched form."""
    x0, w0 = inputs[0], weights[0]
    if x0.dtype not in (torch.bfloat16, torch.float16, torch.float32) or x0.dim() != 2 or w0.dim() != 2:
        return None
    tc = x0.dtype != torch.float32
    xs = [_mat(t) for t in inputs]
    rows = [_weight_rows(t, weight_trans) for t in weights]
    if any(r[1] != rows[0][1] for r in rows):
        return None
    ws, weight_trans = [r[0] for r in rows], rows[0][1]
    M, K = xs[0].shape
    N = ws[0].shape[0] if weight_trans else ws[0].shape[1]
    lda, ldw = _row_stride(xs[0]), _row_stride(ws[0])
    for x, w in zip(xs, ws):
        if (x.shape != xs[0].shape or w.shape != ws[0].shape or x.dtype != x0.dtype or w.dtype != x0.dtype
                or _row_stride(x) != lda or _row_stride(w) != ldw or (tc and (x.data_ptr() % 16 or w.data_ptr() % 16))):
            return None
    if (ws[0].shape[1] if weight_trans else ws[0].shape[0]) != K or (tc and (lda % 8 or ldw % 8)):
        return None
    kinds = [_bias_kind(b, M, N) for b in biases]
    bs = [b.reshape(-1).to(x0.dtype).contiguous() if k == 1 else None for b, k in zip(biases, kinds)]
    rs = [_mat(b.to(x0.dtype)) if k == 2 else None for b, k in zip(biases, kinds)]
    ldr = 0
    if any(r is not None for r in rs):
        strides = {_row_stride(r) for r in rs if r is not None}
        if len(strides) != 1:
            rs = [None if r is None else r.contiguous() for r in rs]
            strides = {N}
        ldr = strides.pop()
    out = torch.empty((len(xs), M, N), dtype=x0.dtype, device=x0.device)
    step = M * N * out.element_size()
    rc = _lib.load().xg_gemm_group_bias_act(
        _lib.ptr_array([x.data_ptr() for x in xs]), _lib.ptr_array([w.data_ptr() for w in ws]),
        _lib.ptr_array([0 if b is None else b.data_ptr() for b in bs]), _lib.ptr_array([0 if r is None else r.data_ptr() for r in rs]),
        _lib.ptr_array([out.data_ptr() + i * step for i in range(len(xs))]),
        len(xs), M, N, K, lda, ldw, N, ldr, 1 if weight_trans else 0, _lib.ACT_CODES[act], _code(x0.dtype), _stream(x0))
    _lib.check(rc, "xg_gemm_group_bias_act")
    return out


def _stack_or_view(ts: Sequence[torch.Tensor]) -> torch.Tensor:
    """[T, ...] tensor of the list's members: a view when they are equally spaced contiguous slabs of one storage
    (the outputs of an unbind / split), else a stacked copy."""
    t0 = ts[0]
    if len(ts) > 1 and all(t.is_contiguous() and t.shape == t0.shape and t.dtype == t0.dtype for t in ts):
        step = ts[1].data_ptr() - t0.data_ptr()
        same_store = all(t.untyped_storage().data_ptr() == t0.untyped_storage().data_ptr() for t in ts)
        if same_store and step == t0.numel() * t0.element_size() and all(
                ts[i].data_ptr() - t0.data_ptr() == i * step for i in range(len(ts))):
            return t0.as_strided((len(ts),) + tuple(t0.shape), (t0.numel(),) + tuple(t0.stride()), t0.storage_offset())
    return torch.stack(list(ts))


@combo_dense.register_fake
def _(inputs, weights, weight_trans, biases, act):
    N = weights[0].shape[0] if weight_trans else weights[0].shape[1]
    return torch.empty((len(inputs), inputs[0].shape[0], N), dtype=inputs[0].dtype, device=inputs[0].device)


@torch.library.custom_op(f"{NS}::combo_batch_dense", mutates_args=(), device_types="cuda")
def combo_batch_dense(inputs: List[torch.Tensor], weights: List[torch.Tensor], weight_trans: bool,
                      biases: List[Optional[torch.Tensor]], act: str) -> torch.Tensor:
    """T same-shape batched dense layers act(bmm(x_t, W_t) + b_t), x_t [S, M, K], W_t [S, K, N] (or [S, N, K]), in one
    grouped launch over the T * S matrix products (a pointer per product: batch entries of a member, also broadcast
    ones, are addressed where they lie); returns [T, S, M, N]. b_t: None, a full [S, M, N] addend, or anything that
    broadcasts to [S, 1, N]."""
    T = len(inputs)
    if T == 0 or len(weights) != T or len(biases) != T:
        raise ValueError("xg_sm100::combo_batch_dense: one input, weight and bias entry per layer")
    S, M, _ = inputs[0].shape
    N = weights[0].shape[1] if weight_trans else weights[0].shape[2]
    xs, ws, bs = [], [], []
    for x, w, b in zip(inputs, weights, biases):
        if x.dim() != 3 or w.dim() != 3 or x.shape[0] != S or w.shape[0] != S:
            raise ValueError("xg_sm100::combo_batch_dense: every member is [S, M, K] x [S, K, N] with one S")
        if b is not None:
            b = b if tuple(b.shape) == (S, M, N) else b.broadcast_to((S, 1, N))
        for i in range(S):
            xs.append(x[i])
            ws.append(w[i])
            bs.append(None if b is None else b[i])
    return combo_dense(xs, ws, weight_trans, bs, act).view(T, S, M, N)


@combo_batch_dense.register_fake
def _(inputs, weights, weight_trans, biases, act):
    S, M, _ = inputs[0].shape
    N = weights[0].shape[1] if weight_trans else weights[0].shape[2]
    return torch.empty((len(inputs), S, M, N), dtype=inputs[0].dtype, device=inputs[0].device)


@torch.library.custom_op(f"{NS}::dense_swiglu", mutates_args=(), device_types="cuda")
def dense_swiglu(x: torch.Tensor, w_gate: torch.Tensor, w_up: torch.Tensor) -> torch.Tensor:
    """silu(x @ w_gate^T) * (x @ w_up^T); weights in Linear layout [N, K]."""
    x = _mat(x)
    w_gate, w_up = _mat(w_gate), _mat(w_up)
    if _row_stride(w_gate) != _row_stride(w_up):
        w_gate, w_up = w_gate.contiguous(), w_up.contiguous()
    M, K = x.shape
    N = w_gate.shape[0]
    out = torch.empty((M, N), dtype=x.dtype, device=x.device)
    rc = _lib.load().xg_gemm_swiglu(_ptr(x), _ptr(w_gate), _ptr(w_up), _ptr(out), M, N, K, _row_stride(x),
                                    _row_stride(w_gate), N, _code(x.dtype), _stream(x))
    _lib.check(rc, "xg_gemm_swiglu")
    return out


@dense_swiglu.register_fake
def _(x, w_gate, w_up):
    return torch.empty((x.shape[0], w_gate.shape[0]), dtype=x.dtype, device=x.device)


@torch.library.custom_op(f"{NS}::dense_rope", mutates_args=(), device_types="cuda")
def dense_rope(x: torch.Tensor, weight: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, seq_len: int,
               head_dim: int) -> torch.Tensor:
    """rope(x @ weight^T) with the rotation in the GEMM epilogue. x: [B*S, K] (row r is token r % seq_len of its
    sequence), weight: [H*D, K]; cos/sin broadcastable from [S, D]. Returns [B*S, H*D]."""
    x = _mat(x)
    weight = _mat(weight)
    M, K = x.shape
    N = weight.shape[0]
    cos2 = cos.reshape(seq_len, head_dim).to(x.dtype).contiguous()
    sin2 = sin.reshape(seq_len, head_dim).to(x.dtype).contiguous()
    out = torch.empty((M, N), dtype=x.dtype, device=x.device)
    rc = _lib.load().xg_gemm_rope(_ptr(x), _ptr(weight), _ptr(cos2), _ptr(sin2), _ptr(out), M, N, K, _row_stride(x),
                                  _row_stride(weight), N, seq_len, head_dim, _code(x.dtype), _stream(x))
    _lib.check(rc, "xg_gemm_rope")
    return out


@dense_rope.register_fake
def _(x, weight, cos, sin, seq_len, head_dim):
    return torch.empty((x.shape[0], weight.shape[0]), dtype=x.dtype, device=x.device)


# --------------------------------------------------------------------------------------------
# attention
# --------------------------------------------------------------------------------------------
@torch.library.custom_op(f"{NS}::sdpa", mutates_args=(), device_types="cuda")
def sdpa(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, attn_mask: Optional[torch.Tensor], scale: float,
         is_causal: bool) -> torch.Tensor:
    """q [B,H,Sq,D], k/v [B,H,Skv,D]; attn_mask: additive (same dtype) or boolean, broadcastable to [B,H,Sq,Skv]."""
    if q.dim() != 4:
        raise ValueError("xg_sm100::sdpa expects 4-D q/k/v")
    B, H, Sq, D = q.shape
    Skv = k.shape[2]
    q, k, v = (t if t.stride(3) == 1 else t.contiguous() for t in (q, k, v))
    mstr = None
    if attn_mask is not None:
        m = attn_mask
        if m.dtype == torch.bool:
            m = torch.zeros(m.shape, dtype=q.dtype, device=q.device).masked_fill_(~m, float("-inf"))
        m = m.to(q.dtype)
        while m.dim() < 4:
            m = m.unsqueeze(0)
        m = m.expand(B, H, Sq, Skv)
        attn_mask = m
        mstr = _lib.i64_array(m.stride())
    out = _empty_like_layout(q)
    rc = _lib.load().xg_sdpa_fwd(_ptr(q), _ptr(k), _ptr(v), _ptr(attn_mask), _ptr(out), B, H, Sq, Skv, D,
                                 _lib.i64_array(q.stride()[:3]), _lib.i64_array(k.stride()[:3]),
                                 _lib.i64_array(v.stride()[:3]), _lib.i64_array(out.stride()[:3]), mstr, float(scale),
                                 1 if is_causal else 0, _code(q.dtype), _stream(q))
    _lib.check(rc, "xg_sdpa_fwd")
    return out


@sdpa.register_fake
def _(q, k, v, attn_mask, scale, is_causal):
    return _empty_like_layout(q if q.stride(3) == 1 else q.contiguous())


# --------------------------------------------------------------------------------------------
# copy fusions (bit-exact)
# --------------------------------------------------------------------------------------------
def _seg_copy(srcs: Sequence[int], dsts: Sequence[int], src_ld: Sequence[int], dst_ld: Sequence[int],
              lens: Sequence[int], rows: int, mask: Optional[torch.Tensor], zero_when: bool, ref: torch.Tensor) -> None:
    n = len(srcs)
    rc = _lib.load().xg_seg_copy(_lib.ptr_array(srcs), _lib.ptr_array(dsts), _lib.i64_array(src_ld), _lib.i64_array(dst_ld),
                                 _lib.i64_array(lens), n, rows, _ptr(mask), 1 if zero_when else 0, _stream(ref))
    _lib.check(rc, "xg_seg_copy")


def _norm_slices(width: int, starts: Sequence[int], ends: Sequence[int]):
    out = []
    for s, e in zip(starts, ends):
        s = s + width if s < 0 else s
        e = e + width if e < 0 else e
        s = min(max(s, 0), width)
        e = min(max(e, s), width)
        out.append((s, e))
    return out


def _mask_bytes(mask: Optional[torch.Tensor], rows: int) -> Optional[torch.Tensor]:
    if mask is None:
        return None
    m = mask.reshape(-1)
    if m.numel() != rows:
        raise ValueError("xg_sm100: row mask must have one entry per row")
    return m.to(torch.uint8) if m.dtype != torch.uint8 else m.contiguous()


@torch.library.custom_op(f"{NS}::slice_cat", mutates_args=(), device_types="cuda")
def slice_cat(src: torch.Tensor, starts: List[int], ends: List[int], row_mask: Optional[torch.Tensor],
              zero_when: bool) -> torch.Tensor:
    """cat([src[:, s:e] for s, e in zip(starts, ends)], -1) of a 2-D src; rows where
    (row_mask != 0) == zero_when are written as zeros."""
    if src.dim() != 2:
        raise NotImplementedError("input must be 2d")
    if src.stride(1) != 1:
        src = src.contiguous()
    rows, width = src.shape
    segs = _norm_slices(width, starts, ends)
    total = sum(e - s for s, e in segs)
    out = torch.empty((rows, total), dtype=src.dtype, device=src.device)
    es = src.element_size()
    srcs, dsts, lens = [], [], []
    off = 0
    for s, e in segs:
        srcs.append(src.data_ptr() + s * es)
        dsts.append(out.data_ptr() + off * es)
        lens.append((e - s) * es)
        off += e - s
    n = len(segs)
    _seg_copy(srcs, dsts, [_row_stride(src) * es] * n, [total * es] * n, lens, rows, _mask_bytes(row_mask, rows), zero_when, src)
    return out


@slice_cat.register_fake
def _(src, starts, ends, row_mask, zero_when):
    segs = _norm_slices(src.shape[1], starts, ends)
    return torch.empty((src.shape[0], sum(e - s for s, e in segs)), dtype=src.dtype, device=src.device)


@torch.library.custom_op(f"{NS}::slice_cat_partly_masked", mutates_args=(), device_types="cuda")
def slice_cat_partly_masked(src: torch.Tensor, starts: List[int], ends: List[int], masked: List[bool], row_mask: torch.Tensor,
                            zero_when: bool) -> torch.Tensor:
    """slice_cat where the row mask applies to the slices flagged in `masked` only (cat([x[:, a:b], where(m, 0, x[:, c:d]),
    ...], -1)): the masked and the unmasked slices are two passes of the segmented copy into one output buffer."""
    if src.dim() != 2:
        raise NotImplementedError("input must be 2d")
    if len(masked) != len(starts):
        raise ValueError("xg_sm100::slice_cat_partly_masked: one flag per slice")
    if src.stride(1) != 1:
        src = src.contiguous()
    rows, width = src.shape
    segs = _norm_slices(width, starts, ends)
    total = sum(e - s for s, e in segs)
    out = torch.empty((rows, total), dtype=src.dtype, device=src.device)
    es = src.element_size()
    off = 0
    groups = {False: ([], [], []), True: ([], [], [])}
    for (s, e), m in zip(segs, masked):
        srcs, dsts, lens = groups[bool(m)]
        srcs.append(src.data_ptr() + s * es)
        dsts.append(out.data_ptr() + off * es)
        lens.append((e - s) * es)
        off += e - s
    for m, (srcs, dsts, lens) in groups.items():
        n = len(srcs)
        if n:
            _seg_copy(srcs, dsts, [_row_stride(src) * es] * n, [total * es] * n, lens, rows,
                      _mask_bytes(row_mask, rows) if m else None, zero_when, src)
    return out


@slice_cat_partly_masked.register_fake
def _(src, starts, ends, masked, row_mask, zero_when):
    segs = _norm_slices(src.shape[1], starts, ends)
    return torch.empty((src.shape[0], sum(e - s for s, e in segs)), dtype=src.dtype, device=src.device)


def _checked_starts(width: int, starts: Sequence[int], slice_len: int) -> List[int]:
    """Slice starts with negative values wrapped; every slice [s, s + slice_len) has to lie inside the row. The
    reference derives slice_len as end - start of the raw aten.slice arguments (structure/fuse_slice.py:28), so a slice
    that aten would have clamped (an end past the width, INT64_MAX) arrives here with a length the row does not
    have: that is refused instead of read past the row."""
    if slice_len < 0:
        raise ValueError(f"xg_sm100::multi_slice: negative slice length {slice_len}")
    out = []
    for s in starts:
        s = s + width if s < 0 else s
        if s < 0 or s + slice_len > width:
            raise ValueError(f"xg_sm100::multi_slice: slice [{s}, {s + slice_len}) is outside a row of {width} elements")
        out.append(s)
    return out


@torch.library.custom_op(f"{NS}::multi_slice", mutates_args=(), device_types="cuda")
def multi_slice(src: torch.Tensor, starts: List[int], slice_len: int) -> torch.Tensor:
    """stack([src[..., s:s+slice_len] for s in starts], 0) -> [num, *src.shape[:-1], slice_len]."""
    lead = list(src.shape[:-1])
    starts = _checked_starts(src.shape[-1], starts, slice_len)
    s2 = _rows_view(src)
    rows, width = s2.shape
    num = len(starts)
    out = torch.empty((num, rows, slice_len), dtype=src.dtype, device=src.device)
    es = src.element_size()
    srcs = [s2.data_ptr() + s * es for s in starts]
    dsts = [out.data_ptr() + k * rows * slice_len * es for k in range(num)]
    _seg_copy(srcs, dsts, [_row_stride(s2) * es] * num, [slice_len * es] * num, [slice_len * es] * num, rows, None, False, src)
    return out.view([num] + lead + [slice_len])


@multi_slice.register_fake
def _(src, starts, slice_len):
    _checked_starts(src.shape[-1], starts, slice_len)
    return torch.empty([len(starts)] + list(src.shape[:-1]) + [slice_len], dtype=src.dtype, device=src.device)


@torch.library.custom_op(f"{NS}::multi_slice_masked", mutates_args=(), device_types="cuda")
def multi_slice_masked(src: torch.Tensor, starts: List[int], slice_len: int, masked: List[bool], row_mask: torch.Tensor,
                       zero_when: bool) -> torch.Tensor:
    """multi_slice of a 2-D src where the slices flagged in `masked` are written as zeros in the rows where
    (row_mask != 0) == zero_when: stack([x[:, a:a+L], where(m, 0, x[:, b:b+L]), ...], 0) -> [num, rows, L]."""
    if src.dim() != 2:
        raise NotImplementedError("input must be 2d")
    if len(masked) != len(starts):
        raise ValueError("xg_sm100::multi_slice_masked: one flag per slice")
    starts = _checked_starts(src.shape[-1], starts, slice_len)
    s2 = _rows_view(src)
    rows = s2.shape[0]
    num = len(starts)
    out = torch.empty((num, rows, slice_len), dtype=src.dtype, device=src.device)
    es = src.element_size()
    for flag in (False, True):
        ks = [k for k in range(num) if bool(masked[k]) == flag]
        if ks:
            n = len(ks)
            _seg_copy([s2.data_ptr() + starts[k] * es for k in ks], [out.data_ptr() + k * rows * slice_len * es for k in ks],
                      [_row_stride(s2) * es] * n, [slice_len * es] * n, [slice_len * es] * n, rows,
                      _mask_bytes(row_mask, rows) if flag else None, zero_when, src)
    return out


@multi_slice_masked.register_fake
def _(src, starts, slice_len, masked, row_mask, zero_when):
    _checked_starts(src.shape[-1], starts, slice_len)
    return torch.empty((len(starts), src.shape[0], slice_len), dtype=src.dtype, device=src.device)


@torch.library.custom_op(f"{NS}::slice_cat_multi", mutates_args=(), device_types="cuda")
def slice_cat_multi(src: torch.Tensor, starts: List[int], ends: List[int], counts: List[int]) -> List[torch.Tensor]:
    """Several slice_cat results of one 2-D src in one pass: output k concatenates the next
    counts[k] (start, end) pairs."""
    if src.dim() != 2:
        raise NotImplementedError("input must be 2d")
    if src.stride(1) != 1:
        src = src.contiguous()
    rows, width = src.shape
    segs = _norm_slices(width, starts, ends)
    es = src.element_size()
    outs, srcs, dsts, slds, dlds, lens = [], [], [], [], [], []
    pos = 0
    for c in counts:
        group = segs[pos:pos + c]
        pos += c
        total = sum(e - s for s, e in group)
        o = torch.empty((rows, total), dtype=src.dtype, device=src.device)
        outs.append(o)
        off = 0
        for s, e in group:
            srcs.append(src.data_ptr() + s * es)
            dsts.append(o.data_ptr() + off * es)
            slds.append(_row_stride(src) * es)
            dlds.append(total * es)
            lens.append((e - s) * es)
            off += e - s
    _seg_copy(srcs, dsts, slds, dlds, lens, rows, None, False, src)
    return outs


@slice_cat_multi.register_fake
def _(src, starts, ends, counts):
    segs = _norm_slices(src.shape[1], starts, ends)
    outs, pos = [], 0
    for c in counts:
        outs.append(torch.empty((src.shape[0], sum(e - s for s, e in segs[pos:pos + c])), dtype=src.dtype, device=src.device))
        pos += c
    return outs


@torch.library.custom_op(f"{NS}::cat_lastdim", mutates_args=(), device_types="cuda")
def cat_lastdim(xs: List[torch.Tensor], row_mask: Optional[torch.Tensor], zero_when: bool) -> torch.Tensor:
    """cat(xs, -1) for tensors that agree on every leading dim (stack along a new trailing-but-one
    dim is the same copy followed by a view)."""
    lead = list(xs[0].shape[:-1])
    xs2 = [_rows_view(x) for x in xs]
    rows = xs2[0].shape[0]
    total = sum(x.shape[1] for x in xs2)
    out = torch.empty((rows, total), dtype=xs[0].dtype, device=xs[0].device)
    es = out.element_size()
    srcs, dsts, slds, lens = [], [], [], []
    off = 0
    for x in xs2:
        if x.dtype != out.dtype or x.shape[0] != rows:
            raise ValueError("xg_sm100::cat_lastdim: inputs must agree in dtype and leading dims")
        srcs.append(x.data_ptr())
        dsts.append(out.data_ptr() + off * es)
        slds.append(_row_stride(x) * es)
        lens.append(x.shape[1] * es)
        off += x.shape[1]
    _seg_copy(srcs, dsts, slds, [total * es] * len(xs2), lens, rows, _mask_bytes(row_mask, rows), zero_when, out)
    return out.view(lead + [total])


@cat_lastdim.register_fake
def _(xs, row_mask, zero_when):
    return torch.empty(list(xs[0].shape[:-1]) + [sum(x.shape[-1] for x in xs)], dtype=xs[0].dtype, device=xs[0].device)


@torch.library.custom_op(f"{NS}::gather_stack", mutates_args=(), device_types="cuda")
def gather_stack(tables: List[torch.Tensor], idx: torch.Tensor, row_mask: Optional[torch.Tensor],
                 zero_when: bool) -> torch.Tensor:
    """out[r, f*D:(f+1)*D] = tables[f][idx[r, f]] (zeros where the row mask says so): F embedding
    lookups, the where-mask and the stack in one pass. idx: int64 [rows, F]."""
    F = len(tables)
    if idx.dim() != 2 or idx.shape[1] != F or idx.dtype != torch.int64:
        raise ValueError("xg_sm100::gather_stack: idx must be int64 [rows, F]")
    D = tables[0].shape[1]
    tabs = []
    for t in tables:
        if t.dim() != 2 or t.shape[1] != D or t.dtype != tables[0].dtype:
            raise ValueError("xg_sm100::gather_stack: tables must be 2-D with one embedding dim and dtype")
        tabs.append(t if t.is_contiguous() else t.contiguous())
    rows = idx.shape[0]
    out = torch.empty((rows, F * D), dtype=tables[0].dtype, device=idx.device)
    rc = _lib.load().xg_gather_rows(_lib.ptr_array([t.data_ptr() for t in tabs]), _lib.i64_array([t.shape[0] for t in tabs]),
                                    F, _ptr(idx), idx.stride(0), idx.stride(1), _ptr(_mask_bytes(row_mask, rows)),
                                    1 if zero_when else 0, _ptr(out), rows, D, F * D, out.element_size(), _stream(idx))
    _lib.check(rc, "xg_gather_rows")
    # keep the contiguous copies alive until the launch is enqueued (stream-ordered frees make this safe)
    del tabs
    return out


@gather_stack.register_fake
def _(tables, idx, row_mask, zero_when):
    return torch.empty((idx.shape[0], len(tables) * tables[0].shape[1]), dtype=tables[0].dtype, device=idx.device)


@torch.library.custom_op(f"{NS}::sum3d", mutates_args=(), device_types="cuda")
def sum3d(inputs: List[torch.Tensor], dim: int) -> List[torch.Tensor]:
    """[sum(x, dim) for x in inputs] for 3-D tensors, one launch for the whole list."""
    xs, outs, shapes = [], [], []
    for x in inputs:
        if x.dim() != 3:
            raise ValueError("xg_sm100::sum3d expects 3-D tensors")
        if x.dtype != inputs[0].dtype:
            raise ValueError("xg_sm100::sum3d: inputs must share a dtype")
        x = x.contiguous()
        xs.append(x)
        s0, s1, s2 = x.shape
        shapes += [s0, s1, s2]
        oshape = (s1, s2) if dim == 0 else ((s0, s2) if dim == 1 else (s0, s1))
        outs.append(torch.empty(oshape, dtype=x.dtype, device=x.device))
    if xs:
        rc = _lib.load().xg_sum3d(_lib.ptr_array([x.data_ptr() for x in xs]), _lib.ptr_array([o.data_ptr() for o in outs]),
                                  _lib.i64_array(shapes), len(xs), int(dim), _code(xs[0].dtype), _stream(xs[0]))
        _lib.check(rc, "xg_sum3d")
    return outs


@sum3d.register_fake
def _(inputs, dim):
    outs = []
    for x in inputs:
        s0, s1, s2 = x.shape
        oshape = (s1, s2) if dim == 0 else ((s0, s2) if dim == 1 else (s0, s1))
        outs.append(torch.empty(oshape, dtype=x.dtype, device=x.device))
    return outs


# ---- row sums written side by side -----------------------------------------------------------------
def _rowsum_cat_impl(a_list, b_list, ranges, batch):
    a0 = a_list[0]
    C = a0.shape[-1]
    n = len(a_list)
    xs, ys, a_bs, b_bs = [], [], [], []
    for k in range(n):
        a = a_list[k].contiguous()
        if a.dim() != 3 or a.shape[-1] != C or a.dtype != a0.dtype or a.shape[0] not in (1, batch):
            raise ValueError("xg_sm100::rowsum_cat: operands must be [batch or 1, rows, C] tensors of one dtype")
        xs.append(a)
        a_bs.append(0 if a.shape[0] == 1 and batch != 1 else a.shape[1] * C)
        if b_list is not None:
            b = b_list[k].contiguous()
            if b.dim() != 3 or b.shape[1:] != a.shape[1:] or b.dtype != a0.dtype or b.shape[0] not in (1, batch):
                raise ValueError("xg_sm100::rowsum_cat: second operands must match the first in rows, C and dtype")
            ys.append(b)
            b_bs.append(0 if b.shape[0] == 1 and batch != 1 else b.shape[1] * C)
        r0, r1 = ranges[2 * k], ranges[2 * k + 1]
        if not (0 <= r0 <= r1 <= a.shape[1]):
            raise ValueError("xg_sm100::rowsum_cat: row range outside the operand")
    out = torch.empty((batch, n * C), dtype=a0.dtype, device=a0.device)
    rc = _lib.load().xg_rowsum_cat(
        _lib.ptr_array([x.data_ptr() for x in xs]), _lib.ptr_array([y.data_ptr() for y in ys]) if b_list is not None else None,
        _lib.i64_array(a_bs), _lib.i64_array(b_bs) if b_list is not None else None, _lib.i64_array(list(ranges)), n,
        batch, C, out.data_ptr(), n * C, _code(a0.dtype), _stream(a0))
    _lib.check(rc, "xg_rowsum_cat")
    return out


@torch.library.custom_op(f"{NS}::slice_sum_cat", mutates_args=(), device_types="cuda")
def slice_sum_cat(src: torch.Tensor, starts: List[int], ends: List[int]) -> torch.Tensor:
    """cat([src[:, s:e, :].sum(1) for s, e in zip(starts, ends)], -1) for a [B, R, C] tensor."""
    if src.dim() != 3:
        raise ValueError("xg_sm100::slice_sum_cat expects a 3-D tensor")
    R = src.shape[1]
    ranges = []
    for s0, e0 in zip(starts, ends):  # aten.slice clamping
        s1 = min(max(s0 + R if s0 < 0 else s0, 0), R)
        e1 = min(max(e0 + R if e0 < 0 else e0, 0), R)
        ranges += [s1, max(e1, s1)]
    return _rowsum_cat_impl([src] * len(starts), None, ranges, src.shape[0])


@slice_sum_cat.register_fake
def _(src, starts, ends):
    return torch.empty((src.shape[0], len(starts) * src.shape[2]), dtype=src.dtype, device=src.device)


@torch.library.custom_op(f"{NS}::sum_cat", mutates_args=(), device_types="cuda")
def sum_cat(inputs: List[torch.Tensor]) -> torch.Tensor:
    """cat([x.sum(1) for x in inputs], -1) for [B, R_k, C] tensors."""
    ranges = []
    for x in inputs:
        ranges += [0, x.shape[1]]
    return _rowsum_cat_impl(list(inputs), None, ranges, inputs[0].shape[0])


@sum_cat.register_fake
def _(inputs):
    return torch.empty((inputs[0].shape[0], len(inputs) * inputs[0].shape[2]), dtype=inputs[0].dtype, device=inputs[0].device)


@torch.library.custom_op(f"{NS}::mul_sum_cat", mutates_args=(), device_types="cuda")
def mul_sum_cat(lhs: List[torch.Tensor], rhs: List[torch.Tensor]) -> torch.Tensor:
    """cat([(a * b).sum(1) for a, b in zip(lhs, rhs)], -1) for [B or 1, R, C] tensors (batch broadcast)."""
    batch = max(max(a.shape[0], b.shape[0]) for a, b in zip(lhs, rhs))
    ranges = []
    for a in lhs:
        ranges += [0, a.shape[1]]
    return _rowsum_cat_impl(list(lhs), list(rhs), ranges, batch)


@mul_sum_cat.register_fake
def _(lhs, rhs):
    batch = max(max(a.shape[0], b.shape[0]) for a, b in zip(lhs, rhs))
    return torch.empty((batch, len(lhs) * lhs[0].shape[2]), dtype=lhs[0].dtype, device=lhs[0].device)
