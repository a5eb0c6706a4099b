"""The five benchmark graphs as plain eager ``nn.Module``s plus their seeded synthetic inputs.

These are the *user models*: what one hands to ``torch.compile(model, backend=...)``. They contain no
fused op; run eagerly on CPU they are the pattern-disabled reference path, compiled through xpu_graph
with the ``cuda_sm100`` target they become the fused graphs in ``fused_graphs.py``.

Inputs are synthetic (no dataset is involved anywhere): shapes, seeds and distributions as stated per
config below.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Dict, List, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F


def _normal_(module: nn.Module, std: float, gen: torch.Generator) -> None:
    with torch.no_grad():
        for prm in module.parameters():
            prm.copy_(torch.randn(prm.shape, generator=gen) * std)


# ---- config 1: small transformer encoder block (fp32) ------------------------------------------
class EncoderBlock(nn.Module):
    """LayerNorm -> QKV Linear -> SDPA -> out-proj + residual -> LayerNorm -> MLP(GELU) + residual."""

    def __init__(self, hidden=256, heads=4, ffn=1024):
        super().__init__()
        self.hidden, self.heads = hidden, heads
        self.ln1 = nn.LayerNorm(hidden)
        self.qkv = nn.Linear(hidden, 3 * hidden)
        self.proj = nn.Linear(hidden, hidden)
        self.ln2 = nn.LayerNorm(hidden)
        self.fc1 = nn.Linear(hidden, ffn)
        self.fc2 = nn.Linear(ffn, hidden)

    def forward(self, x):
        B, S, Hd = x.shape
        h = self.ln1(x)
        qkv = self.qkv(h).view(B, S, 3, self.heads, Hd // self.heads)
        q, k, v = (qkv[:, :, i].transpose(1, 2) for i in range(3))
        a = F.scaled_dot_product_attention(q, k, v)
        a = a.transpose(1, 2).reshape(B, S, Hd)
        x = x + self.proj(a)
        h = self.ln2(x)
        return x + self.fc2(F.gelu(self.fc1(h)))


def make_encoder(seed=0, batch=2, seq=128, hidden=256, heads=4, ffn=1024, dtype=torch.float32):
    g = torch.Generator().manual_seed(seed)
    m = EncoderBlock(hidden, heads, ffn)
    _normal_(m, 0.02, g)
    with torch.no_grad():  # keep the norms' affine parameters near identity
        for ln in (m.ln1, m.ln2):
            ln.weight.copy_(1.0 + 0.02 * torch.randn(hidden, generator=g))
    x = torch.randn(batch, seq, hidden, generator=g)
    return m.to(dtype).eval(), x.to(dtype)


# ---- config 4: Llama-style decoder layer (bf16) -------------------------------------------------
def rope_tables(seq: int, head_dim: int, theta: float = 10000.0) -> Tuple[torch.Tensor, torch.Tensor]:
    inv = 1.0 / (theta ** (torch.arange(0, head_dim, 2, dtype=torch.float32) / head_dim))
    ang = torch.outer(torch.arange(seq, dtype=torch.float32), inv)
    emb = torch.cat((ang, ang), dim=-1)
    return emb.cos(), emb.sin()


def rotate_half(x):
    h = x.shape[-1] // 2
    return torch.cat((-x[..., h:], x[..., :h]), dim=-1)


class RMSNorm(nn.Module):
    def __init__(self, hidden, eps=1e-6):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(hidden))
        self.eps = eps

    def forward(self, x):
        dt = x.dtype
        xf = x.to(torch.float32)
        xf = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + self.eps)
        return (xf * self.weight.to(torch.float32)).to(dt)


class LlamaDecoderLayer(nn.Module):
    """RMSNorm -> q/k/v proj -> RoPE -> causal SDPA -> o proj + residual -> RMSNorm -> SwiGLU FFN + residual."""

    def __init__(self, hidden=4096, heads=32, ffn=11008, eps=1e-6):
        super().__init__()
        self.hidden, self.heads, self.head_dim = hidden, heads, hidden // heads
        self.input_norm = RMSNorm(hidden, eps)
        self.q_proj = nn.Linear(hidden, hidden, bias=False)
        self.k_proj = nn.Linear(hidden, hidden, bias=False)
        self.v_proj = nn.Linear(hidden, hidden, bias=False)
        self.o_proj = nn.Linear(hidden, hidden, bias=False)
        self.post_norm = RMSNorm(hidden, eps)
        self.gate_proj = nn.Linear(hidden, ffn, bias=False)
        self.up_proj = nn.Linear(hidden, ffn, bias=False)
        self.down_proj = nn.Linear(ffn, hidden, bias=False)

    def forward(self, x, cos, sin):
        B, S, Hd = x.shape
        h = self.input_norm(x)
        q = self.q_proj(h).view(B, S, self.heads, self.head_dim).transpose(1, 2)
        k = self.k_proj(h).view(B, S, self.heads, self.head_dim).transpose(1, 2)
        v = self.v_proj(h).view(B, S, self.heads, self.head_dim).transpose(1, 2)
        q = q * cos + rotate_half(q) * sin
        k = k * cos + rotate_half(k) * sin
        a = F.scaled_dot_product_attention(q, k, v, is_causal=True)
        a = a.transpose(1, 2).reshape(B, S, Hd)
        x = x + self.o_proj(a)
        h = self.post_norm(x)
        return x + self.down_proj(F.silu(self.gate_proj(h)) * self.up_proj(h))


def llama_layer_stages(layer: LlamaDecoderLayer, x, cos, sin) -> dict:
    """The eager layer, stage by stage: every intermediate tensor that a fused op of the rewritten graph consumes or
    produces (same arithmetic as LlamaDecoderLayer.forward, in the layer's dtype). Lets a test feed each fused op
    with exactly the inputs its eager counterpart saw, so that the comparison sees the rounding of that op alone."""
    B, S, Hd = x.shape
    H, D = layer.heads, layer.head_dim
    st = {}
    with torch.no_grad():
        st["h1"] = layer.input_norm(x)
        for name, proj in (("q", layer.q_proj), ("k", layer.k_proj), ("v", layer.v_proj)):
            st[name + "_proj"] = proj(st["h1"]).view(B, S, H, D).transpose(1, 2)
        st["q"] = st["q_proj"] * cos + rotate_half(st["q_proj"]) * sin
        st["k"] = st["k_proj"] * cos + rotate_half(st["k_proj"]) * sin
        st["attn"] = F.scaled_dot_product_attention(st["q"], st["k"], st["v_proj"], is_causal=True)
        st["attn_rows"] = st["attn"].transpose(1, 2).reshape(B, S, Hd)
        st["o"] = layer.o_proj(st["attn_rows"])
        st["x1"] = x + st["o"]
        st["h2"] = layer.post_norm(st["x1"])
        st["gate"], st["up"] = layer.gate_proj(st["h2"]), layer.up_proj(st["h2"])
        st["ffn_h"] = F.silu(st["gate"]) * st["up"]
        st["down"] = layer.down_proj(st["ffn_h"])
        st["out"] = st["x1"] + st["down"]
    return st


def make_llama_layer(seed=3, batch=8, seq=2048, hidden=4096, heads=32, ffn=11008, dtype=torch.bfloat16, device="cpu"):
    """Random-init weights ~N(0, 0.02) (norm weights 1), input ~N(0, 1), RoPE theta 10000."""
    g = torch.Generator().manual_seed(seed)
    m = LlamaDecoderLayer(hidden, heads, ffn)
    with torch.no_grad():
        for name, prm in m.named_parameters():
            if prm.dim() == 2:
                # filled block-wise so that the big matrices do not need a second full-size fp32 temporary
                for r0 in range(0, prm.shape[0], 1024):
                    blk = prm[r0:r0 + 1024]
                    blk.copy_(torch.randn(blk.shape, generator=g) * 0.02)
    x = torch.randn(batch, seq, hidden, generator=g)
    cos, sin = rope_tables(seq, hidden // heads)
    m = m.to(dtype).eval().to(device)
    return m, (x.to(dtype).to(device), cos.to(dtype).to(device), sin.to(dtype).to(device))


# ---- config 5: recsys feature-processing graph (fp32 values, int64 indices) -----------------------
class RecsysGraph(nn.Module):
    """64 dense features sliced into 16 groups and re-concatenated (permuted), 26 embedding lookups
    masked with where() and stacked, then a 3-layer ReLU MLP."""

    def __init__(self, n_dense=64, n_groups=16, n_sparse=26, emb_dim=64, table_rows=100000, mlp=(1024, 512, 256)):
        super().__init__()
        self.n_dense, self.n_groups, self.n_sparse, self.emb_dim = n_dense, n_groups, n_sparse, emb_dim
        self.perm = [(5 * i) % n_groups for i in range(n_groups)]
        self.tables = nn.ParameterList([nn.Parameter(torch.empty(table_rows, emb_dim)) for _ in range(n_sparse)])
        d_in = n_dense + n_sparse * emb_dim
        dims = (d_in,) + tuple(mlp)
        self.layers = nn.ModuleList([nn.Linear(dims[i], dims[i + 1]) for i in range(len(mlp))])

    def forward(self, dense, idx, mask):
        w = self.n_dense // self.n_groups
        groups = [dense[:, g * w:(g + 1) * w] for g in self.perm]
        d = torch.cat(groups, dim=1)
        embs = []
        for f in range(self.n_sparse):
            e = F.embedding(idx[:, f], self.tables[f])
            embs.append(torch.where(mask, torch.zeros_like(e), e))
        s = torch.stack(embs, dim=1).reshape(dense.shape[0], -1)
        h = torch.cat([d, s], dim=1)
        for layer in self.layers:
            h = F.relu(layer(h))
        return h


def make_recsys(seed=4, batch=16384, table_rows=100000, device="cpu"):
    g = torch.Generator().manual_seed(seed)
    m = RecsysGraph(table_rows=table_rows)
    with torch.no_grad():
        for t in m.tables:
            t.copy_(torch.randn(t.shape, generator=g) * 0.01)
        for layer in m.layers:
            layer.weight.copy_(torch.randn(layer.weight.shape, generator=g) * 0.02)
            layer.bias.copy_(torch.randn(layer.bias.shape, generator=g) * 0.02)
    dense = torch.randn(batch, 64, generator=g)
    idx = torch.randint(0, table_rows, (batch, 26), generator=g, dtype=torch.int64)
    mask = torch.rand(batch, 1, generator=g) < 0.3
    return m.eval().to(device), (dense.to(device), idx.to(device), mask.to(device))


# ---- configs 2 and 3: stand-alone kernel sweeps ---------------------------------------------------
NORM_SWEEP_ROWS = (4096, 8192, 16384, 32768, 65536)
NORM_SWEEP_HIDDEN = (1024, 4096, 8192)
GEMM_SWEEP = [(m, 4096, n) for m in (256, 4096, 16384) for n in (4096, 11008)]


def make_norm_inputs(rows, hidden, seed=1, dtype=torch.bfloat16, device="cpu"):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(rows, hidden, generator=g)
    r = torch.randn(rows, hidden, generator=g)
    gamma = 1.0 + 0.1 * torch.randn(hidden, generator=g)
    beta = 0.1 * torch.randn(hidden, generator=g)
    return tuple(t.to(dtype).to(device) for t in (x, r, gamma, beta))


def make_gemm_inputs(M, K, N, seed=2, dtype=torch.bfloat16, device="cpu"):
    g = torch.Generator().manual_seed(seed)
    a = torch.randn(M, K, generator=g)
    w = torch.randn(N, K, generator=g) * 0.02
    b = torch.randn(N, generator=g) * 0.02
    return tuple(t.to(dtype).to(device) for t in (a, w, b))
