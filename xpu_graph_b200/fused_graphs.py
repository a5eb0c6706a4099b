"""The benchmark graphs after the ``cuda_sm100`` rewrite, assembled directly from the target's
replacement modules.

Each class takes the eager model from ``workloads.py``, shares its parameters (no copies except the
stated re-layouts) and issues, in ``forward``, exactly the fused-op sequence that xpu_graph's pattern
pass produces for that model with this target. They let the fused path run (and be measured) where
the xpu_graph package itself is not installed; tests/test_target_patterns.py checks, where it is,
that compiling the eager model through XpuGraph yields the same op sequence.
"""
from __future__ import annotations

import torch
import torch.nn as nn

from . import modules as M
from . import ops
from .workloads import EncoderBlock, LlamaDecoderLayer, RecsysGraph


class FusedLlamaDecoderLayer(nn.Module):
    """RMSNorm | 2x dense with the RoPE epilogue (q, k) | dense (v) | flash SDPA | dense(+residual) | RMSNorm |
    dual-GEMM SwiGLU | dense(+residual). The two residual adds ride in the GEMM epilogues (the [M, N] addend
    form of the dense layer) and RoPE in the q/k projections' epilogues, so the block is 9 kernels."""

    def __init__(self, layer: LlamaDecoderLayer, fuse_swiglu_gemm: bool = True, fuse_rope_gemm: bool = True):
        super().__init__()
        self.layer = layer
        self.fuse_rope_gemm = fuse_rope_gemm and layer.head_dim in (64, 128)
        self.dense_rope = M.DenseRopeModule()
        self.heads, self.head_dim = layer.heads, layer.head_dim
        self.eps1, self.eps2 = layer.input_norm.eps, layer.post_norm.eps
        self.fuse_swiglu_gemm = fuse_swiglu_gemm
        self.norm = M.RMSNormModule()
        self.dense = M.DenseLayerModule(False)
        self.rope = M.RopeModule()
        self.sdpa = M.SDPAModule()
        self.dense_swiglu = M.DenseSwiGLUModule()
        self.swiglu = M.SwiGLUModule()

    @torch.no_grad()
    def forward(self, x, cos, sin):
        L = self.layer
        B, S, Hd = x.shape
        x2 = x.reshape(B * S, Hd)
        h = self.norm(x2, L.input_norm.weight, self.eps1)
        if self.fuse_rope_gemm:
            q = self.dense_rope(h, L.q_proj.weight, cos, sin, B, S, self.heads, self.head_dim)
            k = self.dense_rope(h, L.k_proj.weight, cos, sin, B, S, self.heads, self.head_dim)
        else:
            q = self.dense(h, L.q_proj.weight, True, None, "none").view(B, S, self.heads, self.head_dim).transpose(1, 2)
            k = self.dense(h, L.k_proj.weight, True, None, "none").view(B, S, self.heads, self.head_dim).transpose(1, 2)
            q = self.rope(q, cos, sin)
            k = self.rope(k, cos, sin)
        v = self.dense(h, L.v_proj.weight, True, None, "none").view(B, S, self.heads, self.head_dim).transpose(1, 2)
        a = self.sdpa(q, k, v, None, None, True)  # [B, H, S, D]
        a2 = a.transpose(1, 2).reshape(B * S, Hd)
        x2 = self.dense(a2, L.o_proj.weight, True, x2, "none")  # residual as the full [M, N] addend
        h = self.norm(x2, L.post_norm.weight, self.eps2)
        if self.fuse_swiglu_gemm:
            g = self.dense_swiglu(h, L.gate_proj.weight, L.up_proj.weight)
        else:
            g = self.swiglu(self.dense(h, L.gate_proj.weight, True, None, "none"),
                            self.dense(h, L.up_proj.weight, True, None, "none"))
        out = self.dense(g, L.down_proj.weight, True, x2, "none")
        return out.view(B, S, Hd)


class FusedEncoderBlock(nn.Module):
    """LayerNorm | dense+bias | SDPA | dense+bias(+residual) | LayerNorm | dense+bias+GELU | dense+bias(+residual)."""

    def __init__(self, block: EncoderBlock):
        super().__init__()
        self.block = block
        self.ln = M.LayerNormModule()
        self.dense = M.DenseLayerModule(False)
        self.sdpa = M.SDPAModule()
        self.cat = M.CatLastDimModule()

    @torch.no_grad()
    def forward(self, x):
        Bk = self.block
        B, S, Hd = x.shape
        heads = Bk.heads
        x2 = x.reshape(B * S, Hd)
        h = self.ln(x2, Bk.ln1.weight, Bk.ln1.bias, Bk.ln1.eps)
        qkv = self.dense(h, Bk.qkv.weight, True, Bk.qkv.bias, "none").view(B, S, 3, heads, Hd // heads)
        q, k, v = (qkv[:, :, i].transpose(1, 2) for i in range(3))
        a = self.sdpa(q, k, v, None, None, False)
        a2 = a.transpose(1, 2).reshape(B * S, Hd)
        # bias and residual in one epilogue: bias as the column bias, x as the full addend
        x2 = torch.ops.xg_sm100.dense(a2, Bk.proj.weight, True, Bk.proj.bias, x2, "none")
        h = self.ln(x2, Bk.ln2.weight, Bk.ln2.bias, Bk.ln2.eps)
        h = self.dense(h, Bk.fc1.weight, True, Bk.fc1.bias, "gelu")
        out = torch.ops.xg_sm100.dense(h, Bk.fc2.weight, True, Bk.fc2.bias, x2, "none")
        return out.view(B, S, Hd)


class FusedRecsysGraph(nn.Module):
    """slice+cat of the dense features (one copy kernel) | 26 embedding lookups + where + stack (one
    gather kernel) | cat | 3x dense+bias+ReLU (one dense-tower call when the layers are large enough for the fp32
    tensor-core path)."""

    def __init__(self, graph: RecsysGraph):
        super().__init__()
        self.graph = graph
        w = graph.n_dense // graph.n_groups
        self.slices = [(g * w, (g + 1) * w) for g in graph.perm]
        self.slice_cat = M.FuseSliceCatSameInputModule()
        self.gather = M.GatherStackModule()
        self.cat = M.CatLastDimModule()
        self.dense = M.DenseLayerModule(False)
        self.tower = M.DenseTowerModule()

    @torch.no_grad()
    def forward(self, dense, idx, mask):
        G = self.graph
        d = self.slice_cat(dense, self.slices)
        s = self.gather(list(G.tables), idx, mask, True)
        h = self.cat([d, s])
        dims = [h.shape[1]] + [layer.weight.shape[0] for layer in G.layers]
        if h.dtype == torch.float32 and ops.dense_tower_eligible(h.shape[0], dims):
            return self.tower(h, [layer.weight for layer in G.layers], [True] * len(G.layers),
                              [layer.bias for layer in G.layers], ["relu"] * len(G.layers))
        for layer in G.layers:
            h = self.dense(h, layer.weight, True, layer.bias, "relu")
        return h
