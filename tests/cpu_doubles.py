"""CPU stand-ins for the xg_sm100 ops — test doubles, registered only by the host-side test suite.

They let FX graphs rewritten by the cuda_sm100 patterns run on CPU tensors so that the rewrites can be
checked where there is no GPU. They call the oracle; the product package never imports this file.
"""
import torch

from oracle import ref_ops

_DONE = False


def register():
    global _DONE
    if _DONE:
        return
    from xpu_graph_b200 import modules, ops

    modules.ALLOWED_DEVICE_TYPES.add("cpu")

    def k(op):
        return op.register_kernel("cpu")

    k(ops.rms_norm)(lambda x, weight, eps: ref_ops.rms_norm(x, weight, eps))
    k(ops.layer_norm)(lambda x, weight, bias, eps: ref_ops.layer_norm(x, weight, bias, eps))
    k(ops.add_rms_norm)(lambda x, residual, weight, eps: list(ref_ops.add_rms_norm(x, residual, weight, eps)))
    k(ops.add_rms_norm_y)(lambda x, residual, weight, eps: ref_ops.add_rms_norm(x, residual, weight, eps)[0])
    k(ops.add_layer_norm)(lambda x, residual, weight, bias, eps: list(ref_ops.add_layer_norm(x, residual, weight, bias, eps)))
    k(ops.add_layer_norm_y)(lambda x, residual, weight, bias, eps: ref_ops.add_layer_norm(x, residual, weight, bias, eps)[0])
    k(ops.rope)(lambda x, cos, sin: ref_ops.rope(x, cos.reshape(x.shape[2], x.shape[3]), sin.reshape(x.shape[2], x.shape[3])).contiguous())
    k(ops.swiglu)(lambda gate, up: ref_ops.swiglu(gate, up))

    def dense(x, weight, weight_trans, bias, residual, act):
        y = x @ (weight.t() if weight_trans else weight)
        if bias is not None:
            y = y + bias
        if residual is not None:
            y = y + residual
        return ref_ops._ACTS[act](y)

    k(ops.dense)(dense)
    k(ops.batch_dense)(lambda x, weight, weight_trans, bias, residual, act: ref_ops.batch_dense(
        x, weight, weight_trans, bias if residual is None else residual, act))
    def dense_rope(x, weight, cos, sin, seq_len, head_dim):
        y = x @ weight.t()
        M, N = y.shape
        y4 = y.view(M // seq_len, seq_len, N // head_dim, head_dim).transpose(1, 2)
        r = ref_ops.rope(y4, cos.reshape(seq_len, head_dim), sin.reshape(seq_len, head_dim))
        return r.transpose(1, 2).reshape(M, N).contiguous()

    k(ops.dense_rope)(dense_rope)
    k(ops.dense_swiglu)(lambda x, w_gate, w_up: ref_ops.dense_swiglu(x, w_gate, w_up))
    k(ops.sdpa)(lambda q, k_, v, attn_mask, scale, is_causal: ref_ops.sdpa(q, k_, v, attn_mask, scale, is_causal).contiguous())

    def slice_cat(src, starts, ends, row_mask, zero_when):
        out = ref_ops.slice_cat(src, list(zip(starts, ends)))
        if row_mask is not None:
            out = out.clone()
            out[(row_mask.reshape(-1) != 0) == zero_when] = 0
        return out

    k(ops.slice_cat)(slice_cat)

    def slice_cat_partly_masked(src, starts, ends, masked, row_mask, zero_when):
        parts = []
        for s_, e_, m in zip(starts, ends, masked):
            part = ref_ops.slice_cat(src, [(s_, e_)])
            if m:
                part = part.clone()
                part[(row_mask.reshape(-1) != 0) == zero_when] = 0
            parts.append(part)
        return torch.cat(parts, dim=-1)

    k(ops.slice_cat_partly_masked)(slice_cat_partly_masked)
    def multi_slice_masked(src, starts, slice_len, masked, row_mask, zero_when):
        parts = []
        for s_, m in zip(starts, masked):
            part = ref_ops.slice_cat(src, [(s_, s_ + slice_len)])
            if m:
                part = part.clone()
                part[(row_mask.reshape(-1) != 0) == zero_when] = 0
            parts.append(part)
        return torch.stack(parts, dim=0)

    k(ops.multi_slice_masked)(multi_slice_masked)
    k(ops.multi_slice)(lambda src, starts, slice_len: ref_ops.multi_slice(src, starts, slice_len))

    def slice_cat_multi(src, starts, ends, counts):
        pairs, groups, pos = list(zip(starts, ends)), [], 0
        for c in counts:
            groups.append(pairs[pos:pos + c])
            pos += c
        return ref_ops.slice_cat_multi(src, groups)

    k(ops.slice_cat_multi)(slice_cat_multi)

    def cat_lastdim(xs, row_mask, zero_when):
        out = torch.cat(xs, dim=-1)
        if row_mask is not None:
            out = out.clone()
            out.view(-1, out.shape[-1])[(row_mask.reshape(-1) != 0) == zero_when] = 0
        return out

    k(ops.cat_lastdim)(cat_lastdim)

    def gather_stack(tables, idx, row_mask, zero_when):
        m = None
        if row_mask is not None:
            m = (row_mask.reshape(-1) != 0) == zero_when
        return ref_ops.gather_stack(tables, idx, m)

    k(ops.gather_stack)(gather_stack)
    k(ops.sum3d)(lambda inputs, dim: ref_ops.combo_sum(inputs, dim))
    k(ops.slice_sum_cat)(lambda src, starts, ends: ref_ops.slice_sum_cat(src, list(zip(starts, ends))))
    k(ops.sum_cat)(lambda inputs: ref_ops.sum_cat(inputs))

    def mul_sum_cat(lhs, rhs):
        ml = []
        for a, b in zip(lhs, rhs):
            ml += [a, b]
        return ref_ops.mul_sum_cat(ml)

    k(ops.mul_sum_cat)(mul_sum_cat)

    def dense_tower(x, weights, weight_trans, biases, act_names):
        y = x
        for w, t, b, a in zip(weights, weight_trans, biases, act_names.split(",")):
            y = dense(y, w, t, b, None, a)
        return y

    k(ops.dense_tower)(dense_tower)
    def mlp_chain(x, ws, bs, acts, weights_kn):
        y = x
        for l, (w, b, a) in enumerate(zip(ws, bs, acts)):
            y = dense(y, w, not ((weights_kn >> l) & 1), b, None, a)
        return y

    k(ops.mlp_small)(lambda x, weights, biases, act_names, weights_kn: mlp_chain(x, weights, biases, act_names.split(","), weights_kn))
    k(ops.mlp3)(lambda x, w1, b1, w2, b2, w3, b3, a1, a2, a3, weights_kn=0: mlp_chain(x, (w1, w2, w3), (b1, b2, b3), (a1, a2, a3), weights_kn))
    k(ops.mlp2)(lambda x, w1, b1, w2, b2, a1, a2, weights_kn=0: mlp_chain(x, (w1, w2), (b1, b2), (a1, a2), weights_kn))

    def combo_dense(inputs, weights, weight_trans, biases, act):
        return torch.stack([dense(x, w, weight_trans, b, None, act) for x, w, b in zip(inputs, weights, biases)])

    k(ops.combo_dense)(combo_dense)

    def combo_batch_dense(inputs, weights, weight_trans, biases, act):
        outs = []
        for x, w, b in zip(inputs, weights, biases):
            y = torch.bmm(x, w.transpose(1, 2) if weight_trans else w)
            outs.append(ref_ops._ACTS[act](y if b is None else y + b))
        return torch.stack(outs)

    k(ops.combo_batch_dense)(combo_batch_dense)
    _DONE = True
