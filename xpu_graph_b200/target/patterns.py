"""Target patterns of ``cuda_sm100``: FX rewrites that xpu_graph's own patterns do not perform.

xpu_graph's structure patterns (CustomRMSNorm, CustomLayerNorm, CustomDenseLayer, FusedSlice, ...)
already route to this target's modules through ``get_structure_replacements``. The classes below
cover the graph forms that reach the target un-matched on current PyTorch releases
(``aten.native_layer_norm`` from ``nn.LayerNorm``, pre-fused ``_scaled_dot_product_*`` ops, the
rotate-half RoPE chain, ``mul(silu(mm), mm)``, residual adds next to a dense layer or a norm, and
embedding + where + stack). Each is a ``Pattern`` subclass (passes/patterns/pattern.py:26-49) so it is
run, linted, recompiled and logged ("Pattern.<Class> changed graph") by the pass manager like any
built-in pattern; each rewrites aten nodes into ``call_module`` nodes only, so no pattern can match
its own output and the fix-point loop (passes/pass_manager.py:62-82) terminates.
"""
from __future__ import annotations

import operator
from typing import Optional

import torch
from torch import fx
from xpu_graph.config import OptLevel
from xpu_graph.passes.patterns.pattern import Pattern, PatternGroup

from .. import modules as M

aten = torch.ops.aten
INT64_MAX = 9223372036854775807
DENSE_NAME = "custom_dense_layer_replacement"  # sub-module name used by structure/custom_denselayer.py:82
BATCH_DENSE_NAME = "custom_batch_dense_layer_replacement"  # ... and by structure/custom_denselayer.py:108-115
_RESHAPES = (aten.reshape.default, aten.view.default, aten._unsafe_view.default)


# ---- helpers ---------------------------------------------------------------------------------
def _val(node):
    return node.meta.get("val") if isinstance(node, fx.Node) else None


def _is(node, *targets) -> bool:
    return isinstance(node, fx.Node) and node.op == "call_function" and node.target in targets


def _tensor_ok(v, dims: Optional[int] = None) -> bool:
    if not isinstance(v, torch.Tensor):
        return False
    if v.dtype not in M._SUPPORTED or v.device.type not in M.ALLOWED_DEVICE_TYPES:
        return False
    return dims is None or v.dim() == dims


def _broadcasts_to(shape, target) -> bool:
    try:
        return tuple(torch.broadcast_shapes(tuple(shape), tuple(target))) == tuple(target)
    except RuntimeError:
        return False


def _static(shape) -> bool:
    return all(isinstance(s, int) for s in shape)


def _static_but_rows(shape) -> bool:
    """Every extent but the first is a plain int; the first (the row / batch count) may be symbolic (dynamic=True)."""
    return len(shape) >= 1 and _static(tuple(shape)[1:]) and (isinstance(shape[0], int) or isinstance(shape[0], torch.SymInt))


def _rows_hint(n) -> int:
    """A row count as a number: itself, or the example value a symbolic one was traced with (0 if it has none)."""
    if isinstance(n, int):
        return n
    from torch.fx.experimental import symbolic_shapes as ss

    if hasattr(ss, "size_hint"):  # the name on current releases; hint_int is its older spelling
        return int(ss.size_hint(n, fallback=0))
    return int(ss.hint_int(n)) if ss.has_hint(n) else 0


def _shape_key(shape) -> tuple:
    """Hashable stand-in for a shape that may hold symbolic extents (equal expressions give equal keys)."""
    return tuple(s if isinstance(s, int) else str(s) for s in shape)


def _only_user(node: fx.Node, user: fx.Node) -> bool:
    return len(node.users) == 1 and next(iter(node.users)) is user


def _module_call(gm: fx.GraphModule, node, cls) -> bool:
    if not (isinstance(node, fx.Node) and node.op == "call_module"):
        return False
    try:
        return isinstance(gm.get_submodule(node.target), cls)
    except AttributeError:
        return False


def _ensure(gm: fx.GraphModule, name: str, factory) -> str:
    if not hasattr(gm, name):
        gm.add_submodule(name, factory())
    return name


def _unique(gm: fx.GraphModule, stem: str) -> str:
    """A sub-module name not yet used by `gm` (for modules that carry per-site parameters)."""
    i = 0
    while hasattr(gm, f"{stem}_{i}"):
        i += 1
    return f"{stem}_{i}"


def _fill_meta(gm: fx.GraphModule, node: fx.Node) -> None:
    """Give a freshly inserted node its fake value right away (the pass runs under the compiler's fake
    mode), so that later patterns of the same sweep can inspect it; on any problem the value is left
    for the next FakeTensorProp (passes/fake_tensor_prop.py:39-69)."""
    try:
        args = fx.map_arg(node.args, lambda n: n.meta["val"])
        if node.op == "call_module":
            node.meta["val"] = gm.get_submodule(node.target)(*args)
        elif node.op == "call_function":
            node.meta["val"] = node.target(*args, **node.kwargs)
    except Exception:
        node.meta.pop("val", None)


# ---- LayerNorm as lowered from nn.LayerNorm ---------------------------------------------------------
class FusedNativeLayerNorm(Pattern):
    """aten.native_layer_norm(x, [H], w, b, eps)[0] -> LayerNormModule. The reference's FusedLayerNorm
    (common/fuse_layernorm.py:153-212) only matches the decomposed mean/var chain."""

    _opt_level = OptLevel.level2

    def process(self, gm: fx.GraphModule) -> bool:
        changed = False
        for node in list(gm.graph.nodes):
            if not _is(node, aten.native_layer_norm.default) or len(node.args) != 5:
                continue
            x, shape, w, b, eps = node.args
            xv = _val(x)
            if w is None or not _tensor_ok(xv) or xv.dim() < 1 or list(shape) != [xv.shape[-1]]:
                continue  # (a missing bias is fine: the kernel takes none)
            users = list(node.users)
            if not all(_is(u, operator.getitem) for u in users):
                continue
            if any(u.args[1] != 0 and len(u.users) > 0 for u in users):
                continue  # mean / rstd are consumed: leave it alone
            _ensure(gm, "xg_layer_norm", M.LayerNormModule)
            with gm.graph.inserting_before(node):
                new = gm.graph.call_module("xg_layer_norm", (x, w, b, eps))
            _fill_meta(gm, new)
            for u in users:
                if u.args[1] == 0:
                    u.replace_all_uses_with(new)
                gm.graph.erase_node(u)
            gm.graph.erase_node(node)
            changed = True
        return changed


# ---- RMSNorm as lowered from F.rms_norm / nn.RMSNorm -----------------------------------------------------------
class FusedRmsNormLowered(Pattern):
    """The two forms that ``F.rms_norm`` / ``nn.RMSNorm`` reach the compiler in on current PyTorch releases, neither of
    which the reference's FusedRMSNorm matches (its chain matcher asks for ``aten.add.Tensor``,
    passes/patterns/utils/check_ops.py:88-89 through common/fuse_rmsnorm.py:29-114):

      * the decomposition  [to fp32] -> pow 2 -> mean(last dim, keepdim) -> add.Scalar(eps) -> rsqrt -> mul -> mul(weight)
        [-> back to the input dtype];
      * ``aten._fused_rms_norm(x, [H], weight, eps)`` whose second output (the reciprocal rms) is unused.

    Both become an RMSNormModule call, after which the residual-add fusion applies as for the hand-written form."""

    _opt_level = OptLevel.level2

    @staticmethod
    def _fp32_view_of(node):
        """(source, cast) when `node` is `_to_copy(source, dtype=float32)` of a 16-bit tensor, else (node, None)."""
        if _is(node, aten._to_copy.default) and node.kwargs.get("dtype") == torch.float32:
            src = node.args[0]
            sv = _val(src)
            if isinstance(sv, torch.Tensor) and sv.dtype in (torch.bfloat16, torch.float16):
                return src, node
        return node, None

    def _match_chain(self, gm, out):
        """out = mul(mul(X, rsqrt(add.Scalar(mean(pow(X, 2), [last], True), eps))), W)"""
        if not _is(out, aten.mul.Tensor) or len(out.args) != 2:
            return None
        for inner, w in ((out.args[0], out.args[1]), (out.args[1], out.args[0])):
            if not (_is(inner, aten.mul.Tensor) and isinstance(w, fx.Node) and _only_user(inner, out)):
                continue
            for X, rs in ((inner.args[0], inner.args[1]), (inner.args[1], inner.args[0])):
                if not (isinstance(X, fx.Node) and _is(rs, aten.rsqrt.default) and _only_user(rs, inner)):
                    continue
                add = rs.args[0]
                if not (_is(add, aten.add.Scalar, aten.add.Tensor) and _only_user(add, rs)):
                    continue
                mean, eps = add.args[0], add.args[1]
                if not isinstance(eps, (int, float)) or not (_is(mean, aten.mean.dim) and _only_user(mean, add)):
                    continue
                pw = mean.args[0]
                if not (_is(pw, aten.pow.Tensor_Scalar) and pw.args[1] == 2 and pw.args[0] is X and _only_user(pw, mean)):
                    continue
                xv = _val(X)
                if not _tensor_ok(xv) or xv.dim() < 1:
                    continue
                dims = list(mean.args[1]) if isinstance(mean.args[1], (list, tuple)) else [mean.args[1]]
                keep = mean.args[2] if len(mean.args) > 2 else False
                if len(dims) != 1 or dims[0] not in (-1, xv.dim() - 1) or not keep:
                    continue
                wv = _val(w)
                if not (isinstance(wv, torch.Tensor) and wv.dim() == 1 and wv.shape[0] == xv.shape[-1]):
                    continue
                return X, w, float(eps), [out, inner, rs, add, mean, pw]
        return None

    def process(self, gm: fx.GraphModule) -> bool:
        changed = False
        for node in list(gm.graph.nodes):
            fused = getattr(aten, "_fused_rms_norm", None)
            if fused is not None and _is(node, fused.default) and len(node.args) >= 4:
                x, shape, w, eps = node.args[:4]
                xv = _val(x)
                users = list(node.users)
                if (w is not None and eps is not None and _tensor_ok(xv) and list(shape) == [xv.shape[-1]]
                        and all(_is(u, operator.getitem) for u in users)
                        and not any(u.args[1] != 0 and len(u.users) > 0 for u in users)):
                    _ensure(gm, "xg_rms_norm", M.RMSNormModule)
                    with gm.graph.inserting_before(node):
                        new = gm.graph.call_module("xg_rms_norm", (x, w, float(eps)))
                    _fill_meta(gm, new)
                    for u in users:
                        if u.args[1] == 0:
                            u.replace_all_uses_with(new)
                        gm.graph.erase_node(u)
                    gm.graph.erase_node(node)
                    changed = True
                continue
            m = self._match_chain(gm, node)
            if m is None:
                continue
            X, w, eps, chain = m
            src, cast_in = self._fp32_view_of(X)
            out = node
            if cast_in is not None:
                # 16-bit input computed in fp32: the chain's only consumer has to be the cast back to the input dtype
                if len(node.users) != 1:
                    continue
                back = next(iter(node.users))
                if not (_is(back, aten._to_copy.default) and back.kwargs.get("dtype") == _val(src).dtype):
                    continue
                out = back
            elif _val(X).dtype != torch.float32:
                continue  # a 16-bit chain without the fp32 detour rounds after every step: not what the kernel computes
            _ensure(gm, "xg_rms_norm", M.RMSNormModule)
            with gm.graph.inserting_before(out):
                new = gm.graph.call_module("xg_rms_norm", (src, w, eps))
            _fill_meta(gm, new)
            out.replace_all_uses_with(new)
            for dead in ([out] if out is not node else []) + chain + ([cast_in] if cast_in is not None else []):
                if len(dead.users) == 0:
                    gm.graph.erase_node(dead)
            changed = True
        return changed


# ---- scaled dot product attention ----------------------------------------------------------------------
def _sdpa_targets():
    names = ["scaled_dot_product_attention", "_scaled_dot_product_flash_attention_for_cpu",
             "_scaled_dot_product_flash_attention", "_scaled_dot_product_efficient_attention",
             "_scaled_dot_product_cudnn_attention"]
    out = {}
    for n in names:
        pkt = getattr(aten, n, None)
        if pkt is not None and hasattr(pkt, "default"):
            out[pkt.default] = (n == "scaled_dot_product_attention")
    return out


class FusedSdpa(Pattern):
    """aten.scaled_dot_product_attention (as emitted by common/fuse_scaled_dot_product_attention.py:230-234)
    and the pre-fused _scaled_dot_product_* forms that F.scaled_dot_product_attention lowers to
    -> SDPAModule. Dropout, GQA and consumed log-sum-exp outputs are left untouched."""

    _opt_level = OptLevel.level2

    def process(self, gm: fx.GraphModule) -> bool:
        from torch.fx.operator_schemas import normalize_function

        targets = _sdpa_targets()
        changed = False
        for node in list(gm.graph.nodes):
            if not (isinstance(node, fx.Node) and node.op == "call_function" and node.target in targets):
                continue
            single_output = targets[node.target]
            try:
                norm = normalize_function(node.target, node.args, node.kwargs, normalize_to_only_use_kwargs=True)
            except Exception:
                norm = None
            if norm is None:
                continue
            kw = norm.kwargs
            q, k, v = kw.get("query"), kw.get("key"), kw.get("value")
            mask = kw.get("attn_mask", kw.get("attn_bias"))
            scale = kw.get("scale")
            if kw.get("dropout_p", 0.0) != 0.0 or kw.get("enable_gqa", False) or isinstance(scale, fx.Node):
                continue
            causal = bool(kw.get("is_causal", False))
            qv, kv, vv = _val(q), _val(k), _val(v)
            if not (_tensor_ok(qv, 4) and _tensor_ok(kv, 4) and _tensor_ok(vv, 4)):
                continue
            if not (qv.dtype == kv.dtype == vv.dtype) or qv.shape[1] != kv.shape[1] or qv.shape[-1] > 256:
                continue
            if qv.shape[-1] != vv.shape[-1] or (mask is not None and causal):
                continue
            if single_output:
                outs = [node]
            else:
                users = list(node.users)
                if not all(_is(u, operator.getitem) for u in users):
                    continue
                if any(u.args[1] != 0 and len(u.users) > 0 for u in users):
                    continue
                outs = [u for u in users if u.args[1] == 0]
            _ensure(gm, "xg_sdpa", M.SDPAModule)
            with gm.graph.inserting_before(node):
                new = gm.graph.call_module("xg_sdpa", (q, k, v, mask, scale, causal))
            _fill_meta(gm, new)
            for o in outs:
                o.replace_all_uses_with(new)
            if not single_output:
                for u in list(node.users):
                    gm.graph.erase_node(u)
            gm.graph.erase_node(node)
            changed = True
        return changed


class SdpaOperandViews(Pattern):
    """The reference's FusedSDPA hands q, k, v to the attention call as  reshape(clone(x3, contiguous), [1, B*H, S, E])
    (common/fuse_scaled_dot_product_attention.py:205-221): three materialised copies per call. The kernels behind
    SDPAModule address q / k / v by strides, so a copy of a [B*H, S, E] operand whose last dim is contiguous is replaced
    by unsqueeze(x3, 0), a view."""

    _opt_level = OptLevel.level2
    _pattern_group = PatternGroup.GROUP2

    def process(self, gm: fx.GraphModule) -> bool:
        changed = False
        for node in list(gm.graph.nodes):
            if not _module_call(gm, node, M.SDPAModule) or len(node.args) < 3:
                continue
            for i in range(3):
                rs = node.args[i]
                if not (_is(rs, *_RESHAPES) and _only_user(rs, node)):
                    continue
                cl = rs.args[0]
                if not (_is(cl, aten.clone.default) and _only_user(cl, rs)):
                    continue
                x = cl.args[0]
                xv, rv = _val(x), _val(rs)
                if not (isinstance(xv, torch.Tensor) and isinstance(rv, torch.Tensor) and xv.dim() == 3 and rv.dim() == 4):
                    continue
                if not _static(xv.shape) or tuple(rv.shape) != (1,) + tuple(xv.shape) or xv.stride(-1) != 1:
                    continue
                if xv.dtype != torch.float32 and any(st % 8 for st in xv.stride()[:-1]):
                    continue  # the tensor-core path wants 16-byte aligned rows: keep the copy
                with gm.graph.inserting_before(node):
                    view = gm.graph.call_function(aten.unsqueeze.default, (x, 0))
                _fill_meta(gm, view)
                node.replace_input_with(rs, view)
                gm.graph.erase_node(rs)
                gm.graph.erase_node(cl)
                changed = True
        return changed


class FusedSdpaTensorScale(Pattern):
    """The reference's FusedSDPA keeps a tensor-valued softmax scale out of the aten call: at OptLevel.level2 it emits
    a ``SDPAWrappedScale`` module whose op reads the scalar on the host (default_replacements.py:39-55,
    common/fuse_scaled_dot_product_attention.py:149-161, 222-229), at level3 it folds the scale into q (:151-156). Here
    the wrapped call becomes  q * scale  (the level-3 form: no host read, so the graph stays capturable) followed by
    the flash kernel with scale 1."""

    _opt_level = OptLevel.level2

    def process(self, gm: fx.GraphModule) -> bool:
        changed = False
        for node in list(gm.graph.nodes):
            if node.op != "call_module" or len(node.args) != 5:
                continue
            try:
                sub = gm.get_submodule(node.target)
            except AttributeError:
                continue
            if type(sub).__name__ != "SDPAWrappedScale":
                continue
            q, k, v, mask, scale = node.args
            qv, kv, vv, sv = _val(q), _val(k), _val(v), _val(scale)
            if not (_tensor_ok(qv, 4) and _tensor_ok(kv, 4) and _tensor_ok(vv, 4) and isinstance(sv, torch.Tensor)):
                continue
            if not (qv.dtype == kv.dtype == vv.dtype) or qv.shape[1] != kv.shape[1] or qv.shape[-1] > 256 or sv.numel() != 1:
                continue
            _ensure(gm, "xg_sdpa", M.SDPAModule)
            with gm.graph.inserting_before(node):
                qs = gm.graph.call_function(aten.mul.Tensor, (q, scale))
                _fill_meta(gm, qs)
                if _val(qs) is not None and _val(qs).dtype != qv.dtype:  # an fp32 scale promotes the product
                    qs = gm.graph.call_function(aten._to_copy.default, (qs,), {"dtype": qv.dtype})
                    _fill_meta(gm, qs)
                new = gm.graph.call_module("xg_sdpa", (qs, k, v, mask, 1.0, False))
            _fill_meta(gm, new)
            node.replace_all_uses_with(new)
            gm.graph.erase_node(node)
            changed = True
        return changed


# ---- rotate-half RoPE --------------------------------------------------------------------------------------
class FusedRoPE(Pattern):
    """x*cos + cat(-x[..., D/2:], x[..., :D/2])*sin on a 4-D x -> RopeModule (one pass instead of seven)."""

    _opt_level = OptLevel.level2

    @staticmethod
    def _match_rotate_half(cat: fx.Node):
        if not _is(cat, aten.cat.default):
            return None
        parts = cat.args[0]
        dim = cat.args[1] if len(cat.args) > 1 else 0
        if len(parts) != 2 or not _is(parts[0], aten.neg.default):
            return None
        hi, lo = parts[0].args[0], parts[1]
        if not (_is(hi, aten.slice.Tensor) and _is(lo, aten.slice.Tensor)) or hi.args[0] is not lo.args[0]:
            return None
        x = hi.args[0]
        xv = _val(x)
        if not _tensor_ok(xv, 4) or not _static_but_rows(xv.shape):  # (the batch extent may be symbolic)
            return None
        D = xv.shape[-1]
        if D % 2 or dim not in (-1, 3):
            return None

        def sl(n):
            a = list(n.args) + [None] * (5 - len(n.args))
            d = a[1] if a[1] is not None else 0
            start = a[2] if a[2] is not None else 0
            end = a[3] if a[3] is not None else INT64_MAX
            step = a[4] if a[4] is not None else 1
            return d, start, min(end, D) if isinstance(end, int) else end, step

        if sl(hi) != (dim if dim == 3 else -1, D // 2, D, 1) and sl(hi) != (3, D // 2, D, 1) and sl(hi) != (-1, D // 2, D, 1):
            return None
        if sl(lo)[1:] != (0, D // 2, 1) or sl(lo)[0] not in (-1, 3):
            return None
        if not (_only_user(hi, parts[0]) and _only_user(parts[0], cat) and _only_user(lo, cat)):
            return None
        return x

    def process(self, gm: fx.GraphModule) -> bool:
        changed = False
        for node in list(gm.graph.nodes):
            if not _is(node, aten.add.Tensor) or node.kwargs:
                continue
            m1, m2 = node.args
            if not (_is(m1, aten.mul.Tensor) and _is(m2, aten.mul.Tensor)):
                continue
            found = None
            for ma, mb in ((m1, m2), (m2, m1)):
                for cat, sin in ((mb.args[0], mb.args[1]), (mb.args[1], mb.args[0])):
                    x = self._match_rotate_half(cat) if isinstance(cat, fx.Node) else None
                    if x is None:
                        continue
                    for xa, cos in ((ma.args[0], ma.args[1]), (ma.args[1], ma.args[0])):
                        if xa is x and isinstance(cos, fx.Node) and isinstance(sin, fx.Node):
                            found = (x, cos, sin, ma, mb, cat)
                if found:
                    break
            if not found:
                continue
            x, cos, sin, ma, mb, cat = found
            xv, cv, sv = _val(x), _val(cos), _val(sin)
            S, D = xv.shape[2], xv.shape[3]
            if not (isinstance(cv, torch.Tensor) and isinstance(sv, torch.Tensor)):
                continue
            # tables of another dtype (fp32 tables next to a 16-bit x) promote the eager result: the kernel computes and
            # returns x's dtype, so such a chain is left alone
            nv = _val(node)
            if not (cv.dtype == sv.dtype == xv.dtype and isinstance(nv, torch.Tensor) and nv.dtype == xv.dtype):
                continue
            if cv.numel() != S * D or sv.numel() != S * D or tuple(cv.shape[-2:]) != (S, D) or tuple(sv.shape[-2:]) != (S, D):
                continue
            if not (_only_user(ma, node) and _only_user(mb, node) and _only_user(cat, mb)):
                continue
            _ensure(gm, "xg_rope", M.RopeModule)
            with gm.graph.inserting_before(node):
                new = gm.graph.call_module("xg_rope", (x, cos, sin))
            _fill_meta(gm, new)
            node.replace_all_uses_with(new)
            # erase the dead chain, consumers first
            neg = cat.args[0][0]
            hi, lo = neg.args[0], cat.args[0][1]
            for dead in (node, ma, mb, cat, neg, hi, lo):
                if len(dead.users) == 0:
                    gm.graph.erase_node(dead)
            changed = True
        return changed


# ---- SwiGLU ------------------------------------------------------------------------------------------------
class FusedSwiGLU(Pattern):
    """mul(silu(x @ Wg^T), x @ Wu^T) -> one dual GEMM with the SwiGLU epilogue (DenseSwiGLUModule);
    mul(silu(g), u) otherwise -> SwiGLUModule (the NPU target fuses the packed form,
    targets/npu/fuse_silu_mul.py:21-69)."""

    _opt_level = OptLevel.level2
    _pattern_group = PatternGroup.GROUP1

    def process(self, gm: fx.GraphModule) -> bool:
        changed = False
        for node in list(gm.graph.nodes):
            if not _is(node, aten.mul.Tensor) or len(node.args) != 2:
                continue
            a, b = node.args
            if not (isinstance(a, fx.Node) and isinstance(b, fx.Node)):
                continue
            done = False
            for g0, u0 in ((a, b), (b, a)):
                # the two dense outputs may each sit behind an identical reshape ([M, N] -> [B, S, N])
                g, u, via_g, via_u = g0, u0, None, None
                if (_is(g0, *_RESHAPES) and _is(u0, *_RESHAPES) and list(g0.args[1]) == list(u0.args[1])
                        and _only_user(g0, node) and _only_user(u0, node)):
                    g, u, via_g, via_u = g0.args[0], u0.args[0], g0, u0
                if (_module_call(gm, g, M.DenseLayerModule) and _module_call(gm, u, M.DenseLayerModule)
                        and g.target == DENSE_NAME and u.target == DENSE_NAME):
                    gx, gw, gt, gb, gact = g.args
                    ux, uw, ut, ub, uact = u.args
                    wv, uv, xv = _val(gw), _val(uw), _val(gx)
                    if (gact == "silu" and uact == "none" and gx is ux and gt and ut and gb is None and ub is None
                            and _only_user(g, via_g if via_g is not None else node)
                            and _only_user(u, via_u if via_u is not None else node) and _tensor_ok(xv, 2)
                            and xv.dtype in (torch.bfloat16, torch.float16) and isinstance(wv, torch.Tensor)
                            and isinstance(uv, torch.Tensor) and wv.shape == uv.shape and xv.shape[1] % 8 == 0):
                        _ensure(gm, "xg_dense_swiglu", M.DenseSwiGLUModule)
                        with gm.graph.inserting_before(node):
                            new = gm.graph.call_module("xg_dense_swiglu", (gx, gw, uw))
                            _fill_meta(gm, new)
                            out = new
                            if via_g is not None:
                                out = gm.graph.call_function(aten.reshape.default, (new, list(via_g.args[1])))
                                _fill_meta(gm, out)
                        node.replace_all_uses_with(out)
                        for dead in (node, via_g, via_u, g, u):
                            if dead is not None:
                                gm.graph.erase_node(dead)
                        changed = done = True
                        break
                if _is(g0, aten.silu.default) and _only_user(g0, node):
                    gv, uv = _val(g0.args[0]), _val(u0)
                    if _tensor_ok(gv) and _tensor_ok(uv) and gv.shape == uv.shape and gv.dtype == uv.dtype and gv.dim() >= 1:
                        _ensure(gm, "xg_swiglu", M.SwiGLUModule)
                        with gm.graph.inserting_before(node):
                            new = gm.graph.call_module("xg_swiglu", (g0.args[0], u0))
                        _fill_meta(gm, new)
                        node.replace_all_uses_with(new)
                        gm.graph.erase_node(node)
                        gm.graph.erase_node(g0)
                        changed = done = True
                        break
            if done:
                continue
        return changed


# ---- residual add folded into the dense layer's epilogue ----------------------------------------------------
class FusedDenseResidual(Pattern):
    """add(dense(x, W, bias), r) (optionally through a reshape of the dense output) -> the dense layer
    with r as its full [M, N] addend; the MLU dense module takes the same addend as a 2-D bias
    (dense_layer_modules.py:43-56)."""

    _opt_level = OptLevel.level2
    _pattern_group = PatternGroup.GROUP1

    def process(self, gm: fx.GraphModule) -> bool:
        changed = False
        for node in list(gm.graph.nodes):
            if not _is(node, aten.add.Tensor) or node.kwargs or len(node.args) != 2:
                continue
            for d_side, other in ((node.args[0], node.args[1]), (node.args[1], node.args[0])):
                if not (isinstance(d_side, fx.Node) and isinstance(other, fx.Node)):
                    continue
                dense, via = d_side, None
                if _is(d_side, *_RESHAPES) and _only_user(d_side, node):
                    dense, via = d_side.args[0], d_side
                if not (_module_call(gm, dense, M.DenseLayerModule) and dense.target == DENSE_NAME):
                    continue
                if not _only_user(dense, via if via is not None else node):
                    continue
                x, w, wt, bias, act = dense.args
                dv, ov, av, bv = _val(dense), _val(other), _val(node), _val(bias)
                if act != "none" or not (_tensor_ok(dv, 2) and _tensor_ok(ov) and isinstance(av, torch.Tensor)):
                    continue
                Mr, N = dv.shape
                if ov.dtype != dv.dtype or ov.dim() < 1 or not isinstance(N, int):
                    continue
                if _static(dv.shape) and _static(ov.shape):
                    if ov.numel() != Mr * N or ov.shape[-1] != N or av.numel() != Mr * N:
                        continue
                    back = None if list(av.shape) == [Mr, N] else list(av.shape)
                else:
                    # symbolic extents (a dynamic batch): the addend must have the sum's shape expression for expression,
                    # ending in N; the way back to that shape is the size list of the reshape the dense output went through
                    if ov.shape[-1] != N or _shape_key(ov.shape) != _shape_key(av.shape):
                        continue
                    if via is None and _shape_key(av.shape) != _shape_key(dv.shape):
                        continue
                    if via is not None and _shape_key(_val(via).shape) != _shape_key(av.shape):
                        continue
                    back = None if via is None else list(via.args[1])
                if bias is not None and not (isinstance(bv, torch.Tensor) and bv.numel() == N and bv.dim() <= 2):
                    continue
                _ensure(gm, "xg_dense_residual", M.DenseResidualModule)
                with gm.graph.inserting_before(node):
                    r2 = other if ov.dim() == 2 else gm.graph.call_function(aten.reshape.default, (other, [-1, N]))
                    if r2 is not other:
                        _fill_meta(gm, r2)
                    new = gm.graph.call_module("xg_dense_residual", (x, w, wt, bias, r2, "none"))
                    _fill_meta(gm, new)
                    out = new if back is None else gm.graph.call_function(aten.reshape.default, (new, back))
                    if out is not new:
                        _fill_meta(gm, out)
                node.replace_all_uses_with(out)
                gm.graph.erase_node(node)
                if via is not None:
                    gm.graph.erase_node(via)
                gm.graph.erase_node(dense)
                changed = True
                break
        return changed


# ---- residual add folded into the norm ---------------------------------------------------------------------
class FusedAddNorm(Pattern):
    """norm(a + b) -> one kernel that also returns the sum when it has other users
    (store_output_before_norm, targets/mlu/fuse_add_norm.py:118-121, 150-180; NPU form
    targets/npu/fuse_add_rmsnorm.py:28-115)."""

    _opt_level = OptLevel.level2
    _pattern_group = PatternGroup.GROUP2

    def process(self, gm: fx.GraphModule) -> bool:
        changed = False
        for node in list(gm.graph.nodes):
            is_rms = _module_call(gm, node, M.RMSNormModule)
            is_ln = _module_call(gm, node, M.LayerNormModule)
            if not (is_rms or is_ln):
                continue
            add = node.args[0]
            if not _is(add, aten.add.Tensor) or add.kwargs or len(add.args) != 2:
                continue
            a, b = add.args
            av, bv, sv = _val(a), _val(b), _val(add)
            if not (_tensor_ok(av) and _tensor_ok(bv) and isinstance(sv, torch.Tensor)):
                continue
            if av.shape != bv.shape or av.dtype != bv.dtype or av.dtype != sv.dtype:
                continue
            store = len(add.users) > 1
            anchor = node
            if store:
                # The sum's other users read the fused call's second output, so the call has to be defined before the
                # earliest of them. When one precedes the norm, the call takes the add's place if the norm's remaining
                # operands (weight, bias) are already defined there; otherwise the add stays for its other users.
                order = {n: i for i, n in enumerate(gm.graph.nodes)}
                if any(order[u] < order[node] for u in add.users if u is not node):
                    if all(order[x] < order[add] for x in node.args[1:] if isinstance(x, fx.Node)):
                        anchor = add.next
                    else:
                        store = False
            if is_rms:
                name = _ensure(gm, "xg_add_rms_norm" if store else "xg_add_rms_norm_y", lambda: M.AddRMSNormModule(store))
                args = (a, b) + tuple(node.args[1:])
            else:
                name = _ensure(gm, "xg_add_layer_norm" if store else "xg_add_layer_norm_y", lambda: M.AddLayerNormModule(store))
                args = (a, b) + tuple(node.args[1:])
            with gm.graph.inserting_before(anchor):
                new = gm.graph.call_module(name, args)
                _fill_meta(gm, new)
                if store:
                    y = gm.graph.call_function(operator.getitem, (new, 0))
                    s = gm.graph.call_function(operator.getitem, (new, 1))
                    _fill_meta(gm, y)
                    _fill_meta(gm, s)
                else:
                    y, s = new, None
            node.replace_all_uses_with(y)
            gm.graph.erase_node(node)
            if store:
                add.replace_all_uses_with(s, delete_user_cb=lambda u: u is not new)
            if len(add.users) == 0:
                gm.graph.erase_node(add)
            changed = True
        return changed


# ---- embedding lookups + where + stack -------------------------------------------------------------------------
class FusedEmbeddingStack(Pattern):
    """stack([embedding(T_f, idx[:, f]) ...]) with the optional where(mask, 0, .) that the common
    CombinePointwiseSink pass (common/combine_pointwise_sink.py:21-95) hoists above the un-bind/re-stack
    -> GatherStackModule. The reference leaves the F lookups un-fused; its nearest relative is
    torch_mlu.emb_concat (targets/mlu/structure_replacements/__init__.py:136)."""

    _opt_level = OptLevel.level1

    @staticmethod
    def _match_lookups(stack0: fx.Node):
        if not _is(stack0, aten.stack.default):
            return None
        embs = stack0.args[0]
        dim = stack0.args[1] if len(stack0.args) > 1 else 0
        if dim != 0 or len(embs) < 2:
            return None
        tables, idx = [], None
        for f, e in enumerate(embs):
            if not _is(e, aten.embedding.default) or len(e.args) != 2 or e.kwargs or not _only_user(e, stack0):
                return None
            t, sel = e.args
            if not _is(sel, aten.select.int) or sel.args[1] != 1 or sel.args[2] != f:
                return None
            if idx is None:
                idx = sel.args[0]
            if sel.args[0] is not idx:
                return None
            tables.append(t)
        iv = _val(idx)
        tv = [_val(t) for t in tables]
        if not isinstance(iv, torch.Tensor) or iv.dim() != 2 or iv.dtype != torch.int64 or iv.shape[1] != len(embs):
            return None
        if not all(_tensor_ok(t, 2) and t.shape[1] == tv[0].shape[1] and t.dtype == tv[0].dtype for t in tv):
            return None
        return tables, idx

    @staticmethod
    def _is_zero_const(gm: fx.GraphModule, n) -> bool:
        if isinstance(n, (int, float)):
            return n == 0
        if isinstance(n, fx.Node) and n.op == "get_attr":
            t = gm
            try:
                for part in n.target.split("."):
                    t = getattr(t, part)
            except AttributeError:
                return False
            return isinstance(t, torch.Tensor) and not bool(t.ne(0).any())
        if _is(n, aten.zeros_like.default, aten.zeros.default):
            return True
        if _is(n, aten.full.default, aten.full_like.default):
            return n.args[1] == 0
        return False

    def process(self, gm: fx.GraphModule) -> bool:
        changed = False
        for stack0 in list(gm.graph.nodes):
            m = self._match_lookups(stack0)
            if m is None:
                continue
            tables, idx = m
            F = len(tables)
            mask, top = None, stack0
            if len(stack0.users) == 1:
                w = next(iter(stack0.users))
                if _is(w, aten.where.self) and w.args[2] is stack0 and self._is_zero_const(gm, w.args[1]):
                    mv, iv = _val(w.args[0]), _val(idx)
                    if isinstance(mv, torch.Tensor) and mv.dtype == torch.bool and tuple(mv.shape) == (iv.shape[0], 1):
                        mask, top = w.args[0], w
            # consumer A: unbind -> getitem(i) -> stack(dim=1) in order  => [B, F, D]
            target, layout = None, None
            if len(top.users) == 1:
                ub = next(iter(top.users))
                if _is(ub, aten.unbind.int) and (len(ub.args) == 1 or ub.args[1] == 0):
                    gets = list(ub.users)
                    if len(gets) == F and all(_is(g, operator.getitem) for g in gets):
                        finals = {next(iter(g.users)) for g in gets if len(g.users) == 1}
                        if len(finals) == 1 and all(len(g.users) == 1 for g in gets):
                            fin = next(iter(finals))
                            if _is(fin, aten.stack.default) and len(fin.args) > 1 and fin.args[1] == 1:
                                order = [g.args[1] for g in fin.args[0] if _is(g, operator.getitem) and g.args[0] is ub]
                                if order == list(range(F)):
                                    target, layout = fin, "bfd"
            if target is None:
                # consumer B: the [F, B, D] stack (or masked stack) is used directly
                target, layout = top, "fbd"
            tv = _val(tables[0])
            D = tv.shape[1]
            _ensure(gm, "xg_gather_stack", M.GatherStackModule)
            with gm.graph.inserting_before(target):
                new = gm.graph.call_module("xg_gather_stack", (list(tables), idx, mask, True))
                _fill_meta(gm, new)
                B = _val(idx).shape[0]
                # (a symbolic batch size must not be written into the graph as a literal: let reshape infer it)
                out = gm.graph.call_function(aten.reshape.default, (new, [B if isinstance(B, int) else -1, F, D]))
                _fill_meta(gm, out)
                if layout == "fbd":
                    out = gm.graph.call_function(aten.transpose.int, (out, 0, 1))
                    _fill_meta(gm, out)
            target.replace_all_uses_with(out)
            # sweep the dead chain from the consumer side
            dead = [target]
            while dead:
                n = dead.pop()
                if len(n.users) == 0 and n.op in ("call_function", "call_module"):
                    ins = [a for a in n.all_input_nodes]
                    gm.graph.erase_node(n)
                    dead.extend(i for i in ins if len(i.users) == 0 and i.op == "call_function")
            changed = True
        return changed


# ---- single row gathers -------------------------------------------------------------------------------------------
class FusedRowGather(Pattern):
    """table[idx] on dim 0 of a 2-D table in its three graph forms - ``aten.embedding(table, idx)``,
    ``aten.index.Tensor(table, [idx])`` and ``aten.index_select(table, 0, idx)`` - -> RowGatherModule (one pass of the
    gather kernel). Lookups that feed a stack are taken by FusedEmbeddingStack first (this pattern runs in a later
    group)."""

    _opt_level = OptLevel.level1
    _pattern_group = PatternGroup.GROUP2

    def process(self, gm: fx.GraphModule) -> bool:
        changed = False
        for node in list(gm.graph.nodes):
            table = idx = None
            wrap = False
            if _is(node, aten.embedding.default) and len(node.args) == 2 and not node.kwargs:
                table, idx = node.args
            elif _is(node, aten.index.Tensor) and len(node.args) == 2 and len(node.args[1]) == 1 and node.args[1][0] is not None:
                table, idx, wrap = node.args[0], node.args[1][0], True
            elif _is(node, aten.index_select.default) and len(node.args) == 3 and node.args[1] == 0:
                table, idx = node.args[0], node.args[2]  # like embedding, index_select takes no negative indices
            if table is None:
                continue
            tv, iv = _val(table), _val(idx)
            if not (_tensor_ok(tv, 2) and isinstance(iv, torch.Tensor) and iv.dtype in (torch.int64, torch.int32)):
                continue
            # (the index tensor's extents may be symbolic - a dynamic batch of lookups; the module reads them at run time)
            if not _static(tv.shape) or iv.dim() < 1 or iv.device.type not in M.ALLOWED_DEVICE_TYPES:
                continue
            name = _ensure(gm, "xg_row_gather_wrap" if wrap else "xg_row_gather", lambda: M.RowGatherModule(wrap))
            with gm.graph.inserting_before(node):
                new = gm.graph.call_module(name, (table, idx))
            _fill_meta(gm, new)
            node.replace_all_uses_with(new)
            gm.graph.erase_node(node)
            changed = True
        return changed


class GatherIndexRepeatToExpand(Pattern):
    """gather(x, dim, repeat(idx, reps)) -> gather(x, dim, expand(idx, ...)): the repeated index tensor is never
    materialised (the reference's FusedGatherToCopy, targets/mlu/repeat_to_expand.py:25-56)."""

    _opt_level = OptLevel.level1

    def process(self, gm: fx.GraphModule) -> bool:
        changed = False
        for node in list(gm.graph.nodes):
            if not _is(node, aten.gather.default) or len(node.args) < 3:
                continue
            rep = node.args[2]
            if not (_is(rep, aten.repeat.default) and _only_user(rep, node)):
                continue
            src, reps = rep.args[0], list(rep.args[1])
            sv = _val(src)
            if not isinstance(sv, torch.Tensor) or len(reps) != sv.dim() or not _static(sv.shape):
                continue
            # a dim may be repeated only where the source has extent 1: that is exactly what expand can express
            if any(r != 1 and sv.shape[i] != 1 for i, r in enumerate(reps)):
                continue
            with gm.graph.inserting_before(rep):
                new = gm.graph.call_function(aten.expand.default, (src, [-1 if r == 1 else r for r in reps]))
            _fill_meta(gm, new)
            rep.replace_all_uses_with(new)
            gm.graph.erase_node(rep)
            changed = True
        return changed


# ---- where(mask, 0, slice-cat) --------------------------------------------------------------------------------------
class FusedMaskedSliceCat(Pattern):
    """cat([where(mask[B, 1], 0, src[:, s_i:e_i]) ...], -1) -> MaskedSliceCatModule: the row mask is applied while the
    slices are copied (the computation of the reference's slice-where-cat kernel,
    targets/mlu/triton_kernel/fused_slice_where_cat.py:12-73; its matcher, targets/mlu/fuse_slice_where_cat.py:147-216,
    is switched off upstream). By the time target patterns run, the common passes have merged the per-slice ``where``
    nodes into one (common/combine_pointwise_sink.py:21-95) and the slice fusions have replaced the slices, so the
    graph arrives as

        where(mask, 0, fuse_slice_cat(src, slices))                                       or, for equal-length slices,
        cat(unbind(where(mask, 0, transpose(reshape(fuse_slice_cat(src, slices), [B, n, L]), 0, 1))), -1)

    and both forms are matched here; in the second one the members may stand between plain (unmasked) slices of the same
    source, and may be stacked along a new leading dim instead of concatenated (-> MaskedSliceStackModule): the two
    graphs of the reference's own test, tests/mlu/test_fuse_slice_where_cat.py:19-76."""

    _opt_level = OptLevel.level1
    _pattern_group = PatternGroup.GROUP2

    @staticmethod
    def _mask_ok(gm, where, rows, dtype):
        if not _is(where, aten.where.self) or len(where.args) != 3:
            return False
        mv = _val(where.args[0])
        if not (isinstance(mv, torch.Tensor) and mv.dtype == torch.bool and tuple(mv.shape) == (rows, 1)):
            return False
        wv = _val(where)
        return FusedEmbeddingStack._is_zero_const(gm, where.args[1]) and isinstance(wv, torch.Tensor) and wv.dtype == dtype

    def _stacked_form(self, gm, node):
        """node = cat / CatLastDimModule over getitem(unbind(where(mask, 0, transpose(reshape(slice_cat))))) in order."""
        stacked = False
        if _is(node, aten.cat.default):
            parts = node.args[0]
            dim = node.args[1] if len(node.args) > 1 else 0
            if dim not in (-1, 1):
                return None
        elif _is(node, aten.stack.default) and (len(node.args) == 1 or node.args[1] == 0):
            parts, stacked = node.args[0], True  # the members side by side along a new leading dim instead
        elif _module_call(gm, node, M.CatLastDimModule) and len(node.args) == 1:
            parts = node.args[0]
        else:
            return None
        # the masked members are getitem(unbind(...), i) in order; plain slices of the same source (dim 1) may stand
        # between them: they are copied unmasked (the form of tests/mlu/test_fuse_slice_where_cat.py:19-31)
        items = [q for q in parts if _is(q, operator.getitem)]
        plain = [q for q in parts if not _is(q, operator.getitem)]
        if len(items) < 2 or not all(_only_user(q, node) for q in items):
            return None
        parts_all, parts = parts, items
        ub = parts[0].args[0]
        if not (_is(ub, aten.unbind.int) and (len(ub.args) == 1 or ub.args[1] == 0) and len(ub.users) == len(parts)):
            return None
        if [q.args[0] for q in parts] != [ub] * len(parts) or [q.args[1] for q in parts] != list(range(len(parts))):
            return None
        where = ub.args[0]
        if not (isinstance(where, fx.Node) and _only_user(where, ub)):
            return None
        tr = where.args[2] if _is(where, aten.where.self) and len(where.args) == 3 else None
        if not (_is(tr, aten.transpose.int) and sorted(tr.args[1:3]) == [0, 1] and _only_user(tr, where)):
            return None
        rs = tr.args[0]
        if not (_is(rs, *_RESHAPES) and _only_user(rs, tr)):
            return None
        sc = rs.args[0]
        if not (_module_call(gm, sc, M.FuseSliceCatSameInputModule) and len(sc.args) == 2):
            return None
        ov, rv = _val(sc), _val(rs)
        if not (isinstance(ov, torch.Tensor) and ov.dim() == 2 and isinstance(rv, torch.Tensor) and rv.dim() == 3):
            return None
        if rv.shape[0] != ov.shape[0] or rv.shape[1] != len(parts) or not self._mask_ok(gm, where, ov.shape[0], ov.dtype):
            return None
        # the slice-cat result may also feed the `size` node that the reshape takes its batch extent from
        others = [u for u in sc.users if u is not rs]
        if any(not (u.op == "call_method" and u.target == "size" and _only_user(u, rs)) for u in others):
            return None
        # the slices of the combined copy, in the order of the cat, with a flag per slice
        src, width = sc.args[0], _val(sc.args[0]).shape[1] if isinstance(_val(sc.args[0]), torch.Tensor) else None
        slices, masked = [], []
        for q in parts_all:
            if _is(q, operator.getitem):
                slices.append(tuple(sc.args[1][q.args[1]]))
                masked.append(True)
                continue
            if not (_is(q, aten.slice.Tensor) and q.args[0] is src and width is not None and len(q.args) >= 2 and q.args[1] in (1, -1)
                    and (len(q.args) < 5 or q.args[4] == 1)):
                return None
            lo = q.args[2] if len(q.args) > 2 and q.args[2] is not None else 0
            hi = q.args[3] if len(q.args) > 3 and q.args[3] is not None else width
            if not (isinstance(lo, int) and isinstance(hi, int)):
                return None
            slices.append((lo, hi))
            masked.append(False)
        if stacked:
            lens = {hi - lo for lo, hi in slices}
            if len(lens) != 1 or min(lo for lo, _ in slices) < 0:
                return None
            return where.args[0], sc, [ub, where, tr, rs] + others, ("stack", [lo for lo, _ in slices], lens.pop(), masked)
        return where.args[0], sc, [ub, where, tr, rs] + others, (slices, masked) if plain else None

    def process(self, gm: fx.GraphModule) -> bool:
        changed = False
        for node in list(gm.graph.nodes):
            mask = sc = mixed = None
            dead = []
            if _is(node, aten.where.self) and len(node.args) == 3:
                cand = node.args[2]
                if (_module_call(gm, cand, M.FuseSliceCatSameInputModule) and _only_user(cand, node) and len(cand.args) == 2
                        and isinstance(_val(cand), torch.Tensor) and _val(cand).dim() == 2
                        and self._mask_ok(gm, node, _val(cand).shape[0], _val(cand).dtype)):
                    mask, sc = node.args[0], cand
            else:
                m = self._stacked_form(gm, node)
                if m is not None:
                    mask, sc, dead, mixed = m
                    dead = [q for q in node.args[0] if _is(q, operator.getitem)] + dead
            if sc is None:
                continue
            _ensure(gm, "xg_masked_slice_cat", M.MaskedSliceCatModule)
            with gm.graph.inserting_before(node):
                if mixed is not None and mixed[0] == "stack":
                    _ensure(gm, "xg_masked_slice_stack", M.MaskedSliceStackModule)
                    new = gm.graph.call_module("xg_masked_slice_stack", (sc.args[0], mask, mixed[1], mixed[2], mixed[3]))
                elif mixed is None:
                    new = gm.graph.call_module("xg_masked_slice_cat", (sc.args[0], mask, sc.args[1]))
                else:
                    new = gm.graph.call_module("xg_masked_slice_cat", (sc.args[0], mask, mixed[0], mixed[1]))
            _fill_meta(gm, new)
            node.replace_all_uses_with(new)
            gm.graph.erase_node(node)
            for d in dead + [sc]:
                if len(d.users) == 0:
                    gm.graph.erase_node(d)
            changed = True
        return changed


# ---- RoPE folded into the projection's epilogue ------------------------------------------------------------------
class FusedDenseRope(Pattern):
    """rope(transpose(reshape(dense(x, W), [B, S, H, D]), 1, 2)) -> DenseRopeModule: the rotation runs in the GEMM
    epilogue, which saves one full read and write of q / k. Runs after FusedRoPE and CustomDenseLayer."""

    _opt_level = OptLevel.level2
    _pattern_group = PatternGroup.GROUP2

    def process(self, gm: fx.GraphModule) -> bool:
        changed = False
        for node in list(gm.graph.nodes):
            if not _module_call(gm, node, M.RopeModule):
                continue
            tr, cos, sin = node.args
            if not (_is(tr, aten.transpose.int) and set(tr.args[1:3]) == {1, 2} and _only_user(tr, node)):
                continue
            rs = tr.args[0]
            if not (_is(rs, *_RESHAPES) and _only_user(rs, tr)):
                continue
            dense = rs.args[0]
            if not (_module_call(gm, dense, M.DenseLayerModule) and dense.target == DENSE_NAME and _only_user(dense, rs)):
                continue
            x, w, wt, bias, act = dense.args
            xv, rv = _val(x), _val(rs)
            if not (wt and bias is None and act == "none" and _tensor_ok(xv, 2) and isinstance(rv, torch.Tensor)):
                continue
            if xv.dtype not in (torch.bfloat16, torch.float16) or rv.dim() != 4 or not _static_but_rows(rv.shape):
                continue
            B, S, H, D = rv.shape
            if D not in (64, 128) or xv.shape[1] % 8 != 0:
                continue
            if isinstance(B, int) and isinstance(xv.shape[0], int):
                if xv.shape[0] != B * S:
                    continue
            else:
                # a symbolic batch: the rows must be B * S as expressions; the module infers B (view(-1, S, H, D))
                from torch.fx.experimental.symbolic_shapes import statically_known_true

                if not statically_known_true(xv.shape[0] == B * S):
                    continue
                B = -1
            _ensure(gm, "xg_dense_rope", M.DenseRopeModule)
            with gm.graph.inserting_before(node):
                new = gm.graph.call_module("xg_dense_rope", (x, w, cos, sin, B, S, H, D))
            _fill_meta(gm, new)
            node.replace_all_uses_with(new)
            for dead in (node, tr, rs, dense):
                gm.graph.erase_node(dead)
            changed = True
        return changed


# ---- cat along the last dim -------------------------------------------------------------------------------------
class FusedCatLastDim(Pattern):
    """aten.cat of >= 2 tensors along the last dim -> one segmented copy (CatLastDimModule). Runs after
    the slice fusions (structure/fuse_slice_cat.py:52-95 re-emits a cat of the fused slices and the
    remaining inputs), so what is left is a plain concatenation."""

    _opt_level = OptLevel.level1
    _pattern_group = PatternGroup.GROUP2

    def process(self, gm: fx.GraphModule) -> bool:
        changed = False
        for node in list(gm.graph.nodes):
            if not _is(node, aten.cat.default):
                continue
            parts = node.args[0]
            dim = node.args[1] if len(node.args) > 1 else 0
            vals = [_val(p) for p in parts]
            if len(parts) < 2 or not all(isinstance(v, torch.Tensor) for v in vals):
                continue
            nd = vals[0].dim()
            if nd < 2 or dim not in (-1, nd - 1):
                continue
            if any(_is(p, aten.slice.Tensor) for p in parts):
                continue  # leave slices to the slice-cat fusion
            # (the leading extent may be symbolic - a dynamic batch - as long as it is the same expression in every part)
            if not all(v.dim() == nd and v.dtype == vals[0].dtype and _shape_key(v.shape[:-1]) == _shape_key(vals[0].shape[:-1])
                       and v.device.type in M.ALLOWED_DEVICE_TYPES and _static_but_rows(v.shape) for v in vals):
                continue
            _ensure(gm, "xg_cat_lastdim", M.CatLastDimModule)
            with gm.graph.inserting_before(node):
                new = gm.graph.call_module("xg_cat_lastdim", (list(parts),))
            _fill_meta(gm, new)
            node.replace_all_uses_with(new)
            gm.graph.erase_node(node)
            changed = True
        return changed


# ---- row sums written side by side ------------------------------------------------------------------------------
def _sum_dim1(node) -> bool:
    """aten.sum.dim_IntList(x, [1]) of a 3-D tensor without keepdim."""
    if not _is(node, aten.sum.dim_IntList) or len(node.args) < 2 or len(node.args) > 2 or node.kwargs:
        return False
    v = _val(node.args[0])
    return list(node.args[1]) == [1] and _tensor_ok(v, 3) and _static_but_rows(v.shape)  # (the batch may be symbolic)


def _replace_run(gm: fx.GraphModule, cat: fx.Node, lo: int, hi: int, new: fx.Node) -> None:
    """Inputs lo..hi (inclusive) of the last-dim cat are replaced by `new`; a cat of one input disappears."""
    parts = list(cat.args[0])
    rest = parts[:lo] + [new] + parts[hi + 1:]
    if len(rest) == 1:
        cat.replace_all_uses_with(new)
    else:
        with gm.graph.inserting_before(cat):
            new_cat = gm.graph.call_function(aten.cat.default, (rest, -1))
        _fill_meta(gm, new_cat)
        cat.replace_all_uses_with(new_cat)
    gm.graph.erase_node(cat)
    for old in parts[lo:hi + 1]:
        chain = [old]
        while chain:
            n = chain.pop()
            if isinstance(n, fx.Node) and len(n.users) == 0 and n.op == "call_function":
                chain.extend(a for a in n.args if isinstance(a, fx.Node))
                gm.graph.erase_node(n)


def _last_dim_cat(node):
    if not _is(node, aten.cat.default):
        return None
    parts = node.args[0]
    dim = node.args[1] if len(node.args) > 1 else 0
    vals = [_val(q) for q in parts]
    if len(parts) < 2 or not all(isinstance(v, torch.Tensor) and v.dim() == 2 for v in vals) or dim not in (-1, 1):
        return None
    return list(parts)


class FusedSliceSumCat(Pattern):
    """cat([x[:, s_k:e_k, :].sum(1) ...], -1) over one 3-D tensor -> SliceSumCatModule: every row of x is read once
    (the graph form of targets/mlu/fuse_sum_cat.py:120-252; any start row, two or more slices)."""

    _opt_level = OptLevel.level2
    _pattern_group = PatternGroup.GROUP0

    def process(self, gm: fx.GraphModule) -> bool:
        changed = False
        for cat in list(gm.graph.nodes):
            parts = _last_dim_cat(cat)
            if parts is None:
                continue

            def src_of(q):
                if not (_sum_dim1(q) and _only_user(q, cat)):
                    return None
                sl = q.args[0]
                if not (_is(sl, aten.slice.Tensor) and _only_user(sl, q) and len(sl.args) >= 4 and sl.args[1] == 1):
                    return None
                if len(sl.args) > 4 and sl.args[4] != 1:
                    return None
                if not (isinstance(sl.args[2], int) and isinstance(sl.args[3], int)):
                    return None
                v = _val(sl.args[0])
                return sl.args[0] if _tensor_ok(v, 3) and _static_but_rows(v.shape) else None

            i = 0
            while i < len(parts):
                src = src_of(parts[i])
                j = i
                while src is not None and j + 1 < len(parts) and src_of(parts[j + 1]) is src:
                    j += 1
                if src is None or j == i:
                    i += 1
                    continue
                params = [(q.args[0].args[2], q.args[0].args[3]) for q in parts[i:j + 1]]
                name = _unique(gm, "xg_slice_sum_cat")
                gm.add_submodule(name, M.SliceSumCatModule(params))
                with gm.graph.inserting_before(cat):
                    new = gm.graph.call_module(name, (src,))
                _fill_meta(gm, new)
                _replace_run(gm, cat, i, j, new)
                changed = True
                break  # the cat node is gone; later runs are found on the next sweep
        return changed


class FusedSumCat(Pattern):
    """cat([x_k.sum(1) ...], -1) over different [B, R_k, C] tensors -> SumCatModule (the graph form served by
    ConcatenateSumOperation2, targets/mlu/fuse_sum_cat.py:20-43)."""

    _opt_level = OptLevel.level2
    _pattern_group = PatternGroup.GROUP0

    def process(self, gm: fx.GraphModule) -> bool:
        changed = False
        for cat in list(gm.graph.nodes):
            parts = _last_dim_cat(cat)
            if parts is None:
                continue

            def ok(q, ref):
                if not (_sum_dim1(q) and _only_user(q, cat)) or _is(q.args[0], aten.slice.Tensor, aten.mul.Tensor):
                    return False
                v = _val(q.args[0])
                return ref is None or (_shape_key(v.shape[:1]) == _shape_key(ref.shape[:1]) and v.shape[2] == ref.shape[2] and v.dtype == ref.dtype)

            i = 0
            while i < len(parts):
                if not ok(parts[i], None):
                    i += 1
                    continue
                ref = _val(parts[i].args[0])
                j = i
                while j + 1 < len(parts) and ok(parts[j + 1], ref):
                    j += 1
                if j == i:
                    i += 1
                    continue
                _ensure(gm, "xg_sum_cat", M.SumCatModule)
                with gm.graph.inserting_before(cat):
                    new = gm.graph.call_module("xg_sum_cat", ([q.args[0] for q in parts[i:j + 1]],))
                _fill_meta(gm, new)
                _replace_run(gm, cat, i, j, new)
                changed = True
                break
        return changed


class FusedMulSumCat(Pattern):
    """cat([(a_k * b_k).sum(1) ...], -1) -> MulSumCatModule (the graph form of targets/mlu/fuse_mul_sum_cat.py:53-123);
    a_k / b_k are [B or 1, R, C] tensors of one shape apart from the batch (B may be symbolic)."""

    _opt_level = OptLevel.level2
    _pattern_group = PatternGroup.GROUP0

    @staticmethod
    def _common_batch(a0, b0):
        """The batch extent two operands broadcast to: both equal (as numbers or as symbolic expressions), or one is 1."""
        one = lambda d: isinstance(d, int) and d == 1  # noqa: E731
        if one(a0):
            return b0
        if one(b0) or _shape_key((a0,)) == _shape_key((b0,)):
            return a0
        return None

    def process(self, gm: fx.GraphModule) -> bool:
        changed = False
        for cat in list(gm.graph.nodes):
            parts = _last_dim_cat(cat)
            if parts is None:
                continue

            def ok(q, ref):
                if not (_is(q, aten.sum.dim_IntList) and len(q.args) == 2 and list(q.args[1]) == [1] and _only_user(q, cat)):
                    return False
                mul = q.args[0]
                if not (_is(mul, aten.mul.Tensor) and _only_user(mul, q)):
                    return False
                va, vb = _val(mul.args[0]), _val(mul.args[1])
                if not (_tensor_ok(va, 3) and _tensor_ok(vb, 3) and _static_but_rows(va.shape) and _static_but_rows(vb.shape)):
                    return False
                if va.shape[1:] != vb.shape[1:] or va.dtype != vb.dtype:
                    return False
                batch = self._common_batch(va.shape[0], vb.shape[0])
                if batch is None:
                    return False
                return ref is None or (_shape_key((batch,)) == _shape_key((ref[0],)) and va.shape[2] == ref[1] and va.dtype == ref[2])

            i = 0
            while i < len(parts):
                if not ok(parts[i], None):
                    i += 1
                    continue
                va, vb = (_val(a) for a in parts[i].args[0].args[:2])
                ref = (self._common_batch(va.shape[0], vb.shape[0]), va.shape[2], va.dtype)
                j = i
                while j + 1 < len(parts) and ok(parts[j + 1], ref):
                    j += 1
                if j == i:
                    i += 1
                    continue
                mul_list = []
                for q in parts[i:j + 1]:
                    mul_list += [q.args[0].args[0], q.args[0].args[1]]
                _ensure(gm, "xg_mul_sum_cat", M.MulSumCatModule)
                with gm.graph.inserting_before(cat):
                    new = gm.graph.call_module("xg_mul_sum_cat", (mul_list,))
                _fill_meta(gm, new)
                _replace_run(gm, cat, i, j, new)
                changed = True
                break
        return changed


# ---- many same-shape dense layers -------------------------------------------------------------------------------------
COMBO_MIN_WIDTH = 4  # the reference's default width (utils/combo_utils.py:40-41)


class FusedComboDense(Pattern):
    """>= 4 independent dense layers of one shape, dtype, orientation, bias kind (none, a row, a full addend) and
    activation -> one ComboDenseModule call (a grouped launch: tensor-core kernel for 16-bit, FMA kernel for small fp32
    members) + unbind; the same for batched dense layers (lists of bmm) -> ComboBatchDenseModule. The graph form of
    targets/mlu/combo_matmul.py:116-232, restricted to groups whose operands are all defined before the group's first
    member, or whose results are all used after its last member, so that the combined node can take that member's
    place without reordering the graph."""

    _opt_level = OptLevel.level2
    _pattern_group = PatternGroup.GROUP2

    def process(self, gm: fx.GraphModule) -> bool:
        return (self._combine(gm, M.DenseLayerModule, DENSE_NAME, 2, "xg_combo_dense", M.ComboDenseModule)
                or self._combine(gm, M.BatchDenseLayerModule, BATCH_DENSE_NAME, 3, "xg_combo_batch_dense", M.ComboBatchDenseModule))

    def _combine(self, gm, member_cls, member_name, rank, combo_name, combo_cls) -> bool:
        from .. import ops as _ops

        order = {n: i for i, n in enumerate(gm.graph.nodes)}
        groups = {}
        for n in gm.graph.nodes:
            if not (_module_call(gm, n, member_cls) and n.target == member_name and len(n.args) == 5):
                continue
            x, w, wt, bias, act = n.args
            xv, wv, bv, v = _val(x), _val(w), _val(bias), _val(n)
            # (2-D members may have a symbolic row count, the same expression in all of them; batched ones are static)
            x_ok = _static_but_rows(xv.shape) if (rank == 2 and isinstance(xv, torch.Tensor)) else _static(xv.shape) if isinstance(xv, torch.Tensor) else False
            if not (_tensor_ok(xv, rank) and _tensor_ok(wv, rank) and _tensor_ok(v, rank) and x_ok and _static(wv.shape)):
                continue
            if xv.dtype not in (torch.bfloat16, torch.float16, torch.float32) or wv.dtype != xv.dtype:
                continue
            if rank == 3 and xv.shape[0] != wv.shape[0]:
                continue
            rows, k, cols = v.shape[-2], xv.shape[-1], v.shape[-1]
            if xv.dtype == torch.float32:
                # the grouped fp32 launch is the FMA kernel; members large enough for the tensor-core path stay single
                if 2 * _rows_hint(rows) * k * cols >= _ops.F32_TENSOR_MIN_FLOPS:
                    continue
            elif k % 8 != 0 or wv.shape[-1] % 8 != 0 or (rank == 3 and (rows * k) % 8 != 0):  # (rank 3: static extents)
                continue  # 16-bit rows (and the batch entries' first rows) must be addressable by a tensor map
            kind = 0
            if bias is not None:
                if not (isinstance(bv, torch.Tensor) and bv.dtype == xv.dtype and (_static(bv.shape) or (rank == 2 and bv.dim() == 2 and _static_but_rows(bv.shape)))):
                    continue
                if _shape_key(bv.shape) == _shape_key(v.shape) and _shape_key(v.shape)[-2] != 1:
                    kind = 2  # a full addend
                elif bv.numel() == cols and rank == 2 and (bv.dim() == 1 or (bv.dim() == 2 and bv.shape[0] == 1)):
                    kind = 1  # a row of N
                elif rank == 3 and _broadcasts_to(bv.shape, (v.shape[0], 1, cols)):
                    kind = 1  # a row of N per batch entry
                else:
                    continue
            key = (_shape_key(xv.shape), tuple(wv.shape), bool(wt), kind, act, xv.dtype)
            groups.setdefault(key, []).append(n)
        for key, nodes in groups.items():
            if len(nodes) < COMBO_MIN_WIDTH:
                continue
            first, last = order[nodes[0]], order[nodes[-1]]
            # either every operand of every member precedes the first member (the combined node then takes that member's
            # place), or every user of every member follows the last member (it takes the last member's place; the form of
            # weights that are each produced right before their layer, e.g. F.linear(x_i, w_i.T)): the members are mutually
            # independent in both cases
            anchor = nodes[0]
            members = [n for n in nodes if all(not isinstance(a, fx.Node) or order[a] < first for a in n.args)]
            if len(members) < COMBO_MIN_WIDTH:
                anchor = nodes[-1]
                members = [n for n in nodes if all(order[u] > last for u in n.users)]
            if len(members) < COMBO_MIN_WIDTH:
                continue
            _ensure(gm, combo_name, combo_cls)
            with gm.graph.inserting_before(anchor):
                new = gm.graph.call_module(combo_name, ([n.args[0] for n in members], [n.args[1] for n in members],
                                                        [n.args[3] for n in members], key[4], key[2]))
                _fill_meta(gm, new)
                parts = gm.graph.call_function(aten.unbind.int, (new,))
                _fill_meta(gm, parts)
                for i, n in enumerate(members):
                    item = gm.graph.call_function(operator.getitem, (parts, i))
                    _fill_meta(gm, item)
                    n.replace_all_uses_with(item)
            for n in members:
                gm.graph.erase_node(n)
            return True  # one group per sweep: the node order used above is stale now; the pass manager calls again
        return False


# ---- chains of fp32 dense layers ---------------------------------------------------------------------------------
class FusedDenseTower(Pattern):
    """dense(dense(dense(x))), each inner result used only by the next layer -> DenseTowerModule. fp32 chains of any
    depth >= 2 when every layer is large enough for the tensor-core path (ops.dense_tower_eligible); 16-bit chains when
    at least one pair of neighbouring layers fits the two-layer kernel (ops.mlp2_eligible: narrow layers whose hidden
    activation then never leaves the SM); chains of any dtype when a pair of neighbours is narrow enough for the
    weights-in-shared-memory kernel and the rows are few or the layers very narrow (ops.mlp_small_worth_it). The graph form of targets/mlu/fuse_densetower.py:272-316
    (FusedDenseTower2 / 3)."""

    _opt_level = OptLevel.level2
    _pattern_group = PatternGroup.GROUP2

    def process(self, gm: fx.GraphModule) -> bool:
        from .. import ops as _ops

        def is_dense(n, dtype=None):
            if not (_module_call(gm, n, M.DenseLayerModule) and n.target == DENSE_NAME and len(n.args) == 5):
                return False
            v, xv, bv = _val(n), _val(n.args[0]), _val(n.args[3])
            if not (_tensor_ok(v, 2) and _tensor_ok(xv, 2) and _static_but_rows(v.shape) and _static_but_rows(xv.shape)):
                return False  # (the row count may be symbolic: the op chooses its kernels from the actual one)
            if v.dtype not in (torch.float32, torch.bfloat16, torch.float16) or xv.dtype != v.dtype:
                return False
            if dtype is not None and v.dtype != dtype:
                return False
            if not isinstance(n.args[2], bool) or not isinstance(n.args[4], str):
                return False
            return n.args[3] is None or (isinstance(bv, torch.Tensor) and bv.dim() == 1 and bv.numel() == v.shape[1])

        def worth_it(x, chain):
            rows = _rows_hint(_val(x).shape[0])
            dims = [_val(x).shape[1]] + [_val(n).shape[1] for n in chain]
            dtype = _val(chain[0]).dtype
            # narrow neighbours whose weights fit in shared memory together (any dtype, any row length)
            small = any(_ops.mlp_small_worth_it(rows, dims[i:i + 3], dtype) for i in range(len(chain) - 1))
            if dtype == torch.float32:
                return small or _ops.dense_tower_eligible(rows, dims)
            # four or more independent layers of one shape are FusedComboDense's (one grouped launch for all of them)
            head = chain[0]
            alike = [m for m in gm.graph.nodes
                     if is_dense(m, dtype) and m.args[2] == head.args[2] and m.args[4] == head.args[4]
                     and _val(m.args[1]).shape == _val(head.args[1]).shape
                     and _shape_key(_val(m.args[0]).shape) == _shape_key(_val(x).shape)]
            if len(alike) >= 4:
                return False
            return small or any(_ops.mlp2_eligible(rows, dims[i], dims[i + 1], dims[i + 2], dtype, chain[i].args[2], chain[i + 1].args[2])
                                for i in range(len(chain) - 1))

        changed = False
        for tail in reversed(list(gm.graph.nodes)):
            if getattr(tail, "_erased", False):
                continue  # an inner layer of a chain that this sweep has already replaced
            if not is_dense(tail):
                continue
            dtype = _val(tail).dtype
            if any(is_dense(u, dtype) and u.args[0] is tail and _only_user(tail, u) for u in tail.users):
                continue  # not the last layer of its chain
            chain = [tail]
            while is_dense(chain[0].args[0], dtype) and _only_user(chain[0].args[0], chain[0]):
                chain.insert(0, chain[0].args[0])
            if len(chain) < 2:
                continue
            x = chain[0].args[0]
            if not worth_it(x, chain):
                continue
            _ensure(gm, "xg_dense_tower", M.DenseTowerModule)
            with gm.graph.inserting_before(tail):
                new = gm.graph.call_module("xg_dense_tower", (x, [n.args[1] for n in chain], [n.args[2] for n in chain],
                                                              [n.args[3] for n in chain], [n.args[4] for n in chain]))
            _fill_meta(gm, new)
            tail.replace_all_uses_with(new)
            for n in reversed(chain):
                gm.graph.erase_node(n)
            changed = True
        return changed


ALL_PATTERNS = [FusedDenseTower, FusedComboDense, FusedSliceSumCat, FusedMulSumCat, FusedSumCat, FusedNativeLayerNorm,
                FusedRmsNormLowered, FusedSdpa, FusedSdpaTensorScale, SdpaOperandViews, FusedRoPE, FusedEmbeddingStack, FusedSwiGLU,
                FusedDenseResidual, FusedAddNorm, FusedCatLastDim, FusedDenseRope, FusedRowGather, GatherIndexRepeatToExpand,
                FusedMaskedSliceCat]


def get_all_patterns(config) -> dict:
    """Target patterns keyed by group, filtered by the config (template: targets/mlu/__init__.py:8-29)."""
    groups = {PatternGroup.GROUP0: [], PatternGroup.GROUP1: [], PatternGroup.GROUP2: []}
    for cls in ALL_PATTERNS:
        if cls.filter(config):
            groups[cls._pattern_group].append(cls())
    return groups
