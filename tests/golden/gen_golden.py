"""Generates tests/golden/golden_v1.pt by running the xpu_graph reference itself.

Run where the xpu_graph source is importable (set XPU_GRAPH_SRC or keep it beside the repository):

    python tests/golden/gen_golden.py

What is recorded (inputs and outputs, all seeded, all small):
  * the reference's own DefaultRMSNorm / DefaultLayerNorm modules
    (passes/patterns/utils/default_replacements.py:19-36) on bf16 and fp32 rows;
  * the reference's pass pipeline (target none, OptLevel.level2) compiling and running
      - residual add + RMSNorm / LayerNorm graphs,
      - Linear (+bias) + activation graphs (the dense-layer pattern's input),
      - the decomposed bmm-softmax-bmm attention graph that FusedSDPA rewrites
        (common/fuse_scaled_dot_product_attention.py:120-242), with and without an additive mask,
      - slice + cat graphs incl. the INT64_MAX / negative-end cases of tests/mlu/test_fuse_slice_cat.py:293-323,
      - multi-slice + stack, embedding + where + stack, RoPE and SwiGLU chains,
      - the three benchmark graphs at reduced size (encoder block, Llama-style layer, recsys graph).
`python tests/golden/gen_golden.py v4` writes tests/golden/golden_v4.pt: the graph forms of the reference's combo
and dense-tower tests at their own sizes (tests/mlu/test_combo_matmul.py:17-109, test_fuse_densetower.py:17-53: eight
layers of 5 x 8 x 7 in fp32 over a shared or split input with no bias, a row or a full [M, N] addend; lists of bmm;
16 rows of 20 -> 32 -> 16 -> 1 in fp16 with [K, N] weights) and a bf16 layer whose rows no tensor map addresses;
`python tests/golden/gen_golden.py v3` writes tests/golden/golden_v3.pt (16-bit towers of narrow dense layers);
`python tests/golden/gen_golden.py v2` writes tests/golden/golden_v2.pt the same way: slice -> sum -> cat,
mul -> sum -> cat and sum -> cat graphs (targets/mlu/fuse_sum_cat.py, fuse_mul_sum_cat.py), a chain of three dense
layers, four parallel dense layers of one shape, and a bmm + bias + GELU graph.
The torch-version shims of xpu_graph_b200/target/compat.py are the only thing between this script and
the unmodified reference.
"""
import os
import sys

import torch
import torch.nn.functional as F

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)

from xpu_graph_b200.target.compat import import_xpu_graph  # noqa: E402

import_xpu_graph()
from torch._dynamo.backends.common import aot_autograd  # noqa: E402
from xpu_graph import OptLevel, Target, XpuGraph, XpuGraphConfig  # noqa: E402
from xpu_graph.fx_utils import FxStage  # noqa: E402
from xpu_graph.passes.patterns.utils.default_replacements import DefaultLayerNorm, DefaultRMSNorm  # noqa: E402

from xpu_graph_b200.workloads import make_encoder, make_llama_layer, make_recsys, rotate_half  # noqa: E402

MAX_INT64 = 9223372036854775807


def ref_backend():
    cfg = XpuGraphConfig(is_training=False, target=Target.none, opt_level=OptLevel.level2, enable_cache=False)
    return aot_autograd(fw_compiler=XpuGraph(cfg)._get_compiler(FxStage.inference), keep_inference_input_mutations=True)


def run_ref(fn, *inputs):
    torch._dynamo.reset()
    with torch.no_grad():
        out = torch.compile(fn, backend=ref_backend(), dynamic=False)(*inputs)
    return out


def main():
    G = {}
    g = torch.Generator().manual_seed(1234)

    def rn(*shape, dtype=torch.float32, std=1.0):
        return (torch.randn(*shape, generator=g) * std).to(dtype)

    # ---- the reference's own default norm modules -------------------------------------------------
    for dt, tag in ((torch.bfloat16, "bf16"), (torch.float32, "f32")):
        x, w, b = rn(6, 96, dtype=dt), (1 + 0.1 * rn(96)).to(dt), (0.1 * rn(96)).to(dt)
        with torch.no_grad():
            G[f"default_rms_{tag}"] = dict(x=x, w=w, eps=1e-6, y=DefaultRMSNorm()(x, w, 1e-6))
            G[f"default_ln_{tag}"] = dict(x=x, w=w, b=b, eps=1e-5, y=DefaultLayerNorm()(x, w, b, 1e-5))

    # ---- add + norm through the pipeline -----------------------------------------------------------
    def add_rms(x, r, w):
        s = x + r
        sf = s.float()
        y = (sf * torch.rsqrt(sf.pow(2).mean(-1, keepdim=True) + 1e-6) * w.float()).to(x.dtype)
        return y, s

    def add_ln(x, r, w, b):
        s = x + r
        return F.layer_norm(s.float(), s.shape[-1:], w.float(), b.float(), 1e-5).to(x.dtype), s

    for dt, tag in ((torch.bfloat16, "bf16"), (torch.float32, "f32")):
        x, r = rn(5, 128, dtype=dt), rn(5, 128, dtype=dt)
        w, b = (1 + 0.1 * rn(128)).to(dt), (0.1 * rn(128)).to(dt)
        y, s = run_ref(add_rms, x, r, w)
        G[f"add_rms_{tag}"] = dict(x=x, r=r, w=w, eps=1e-6, y=y, s=s)
        y, s = run_ref(add_ln, x, r, w, b)
        G[f"add_ln_{tag}"] = dict(x=x, r=r, w=w, b=b, eps=1e-5, y=y, s=s)

    # ---- dense layers --------------------------------------------------------------------------------
    for act in ("none", "gelu", "relu", "silu", "sigmoid"):
        fn = {"none": lambda t: t, "gelu": F.gelu, "relu": F.relu, "silu": F.silu, "sigmoid": torch.sigmoid}[act]
        x, w, b = rn(24, 40), rn(56, 40, std=0.1), rn(56, std=0.1)
        G[f"dense_{act}_f32"] = dict(x=x, w=w, b=b, act=act, y=run_ref(lambda x, w, b: fn(F.linear(x, w, b)), x, w, b))
    x, w = rn(24, 40, dtype=torch.bfloat16), rn(56, 40, dtype=torch.bfloat16, std=0.1)
    G["dense_nobias_bf16"] = dict(x=x, w=w, b=None, act="gelu", y=run_ref(lambda x, w: F.gelu(F.linear(x, w)), x, w))
    x, w, r = rn(24, 40), rn(40, 56, std=0.1), rn(24, 56)
    G["dense_kn_residual_f32"] = dict(x=x, w=w, r=r, y=run_ref(lambda x, w, r: torch.addmm(r, x, w), x, w, r))

    # ---- attention: the decomposed form FusedSDPA matches -----------------------------------------------
    def attn(q, k, v):
        s = torch.bmm(q, k.transpose(1, 2)) * 0.125
        return torch.bmm(torch.softmax(s, dim=-1), v)

    def attn_mask(q, k, v, m):
        s = torch.bmm(q, k.transpose(1, 2)) * 0.125 + m
        return torch.bmm(torch.softmax(s, dim=-1), v)

    q, k, v = rn(6, 38, 64), rn(6, 38, 64), rn(6, 38, 64)
    G["sdpa_f32"] = dict(q=q, k=k, v=v, scale=0.125, y=run_ref(attn, q, k, v))
    m = rn(6, 38, 38)
    G["sdpa_mask_f32"] = dict(q=q, k=k, v=v, m=m, scale=0.125, y=run_ref(attn_mask, q, k, v, m))
    qb, kb, vb = (t.to(torch.bfloat16) for t in (q, k, v))
    G["sdpa_bf16"] = dict(q=qb, k=kb, v=vb, scale=0.125, y=run_ref(attn, qb, kb, vb))
    q4, k4, v4 = rn(2, 3, 40, 32, dtype=torch.bfloat16), rn(2, 3, 40, 32, dtype=torch.bfloat16), rn(2, 3, 40, 32, dtype=torch.bfloat16)
    G["sdpa_causal_bf16"] = dict(q=q4, k=k4, v=v4, y=run_ref(lambda q, k, v: F.scaled_dot_product_attention(q, k, v, is_causal=True), q4, k4, v4))

    # ---- copy fusions ------------------------------------------------------------------------------------
    src = rn(9, 120)
    cases = {
        "even": [(0, 32), (64, 96), (32, 64)],
        "ragged": [(3, 10), (100, 119), (50, 51)],
        "int64max": [(8, MAX_INT64), (0, 8)],
        "negative_end": [(0, -100), (10, -3)],
    }
    for name, sl in cases.items():
        fn = lambda s, sl=sl: torch.cat([s[:, a:b] for a, b in sl], dim=-1) + 0  # noqa: E731
        G[f"slice_cat_{name}"] = dict(src=src, slices=sl, y=run_ref(fn, src))
    srcb = src.to(torch.bfloat16)
    G["slice_cat_bf16"] = dict(src=srcb, slices=cases["even"], y=run_ref(lambda s: torch.cat([s[:, a:b] for a, b in cases["even"]], dim=-1) + 0, srcb))
    starts = [0, 40, 16, 100]
    G["multi_slice"] = dict(src=src, starts=starts, length=12, y=run_ref(lambda s: torch.stack([s[:, a:a + 12] for a in starts], 0) + 0, src))
    mask = torch.rand(9, 1, generator=g) < 0.4
    G["masked_slice_cat"] = dict(src=src, mask=mask, slices=cases["even"],
                                 y=run_ref(lambda s, m: torch.cat([torch.where(m, torch.zeros_like(s[:, a:b]), s[:, a:b]) for a, b in cases["even"]], -1), src, mask))
    tables = [rn(20, 8, std=0.01) for _ in range(3)]
    idx = torch.randint(0, 20, (9, 3), generator=g)

    def emb(t0, t1, t2, idx, m):
        es = [F.embedding(idx[:, f], t) for f, t in enumerate((t0, t1, t2))]
        return torch.stack([torch.where(m, torch.zeros_like(e), e) for e in es], dim=1).reshape(idx.shape[0], -1)

    G["gather_stack"] = dict(tables=tables, idx=idx, mask=mask, y=run_ref(emb, *tables, idx, mask))

    # ---- RoPE and SwiGLU ---------------------------------------------------------------------------------------
    for dt, tag in ((torch.bfloat16, "bf16"), (torch.float32, "f32")):
        x, c, s = rn(2, 3, 10, 16, dtype=dt), rn(10, 16, dtype=dt), rn(10, 16, dtype=dt)
        G[f"rope_{tag}"] = dict(x=x, cos=c, sin=s, y=run_ref(lambda x, c, s: x * c + rotate_half(x) * s, x, c, s))
        a, b = rn(7, 48, dtype=dt), rn(7, 48, dtype=dt)
        G[f"swiglu_{tag}"] = dict(gate=a, up=b, y=run_ref(lambda a, b: F.silu(a) * b, a, b))

    # ---- the benchmark graphs at reduced size -----------------------------------------------------------------------
    m, x = make_encoder(seed=0, batch=2, seq=16, hidden=64, heads=4, ffn=128)
    G["encoder_small"] = dict(args=dict(seed=0, batch=2, seq=16, hidden=64, heads=4, ffn=128), y=run_ref(m, x))
    m, inp = make_llama_layer(seed=3, batch=2, seq=24, hidden=128, heads=2, ffn=192)
    G["llama_small"] = dict(args=dict(seed=3, batch=2, seq=24, hidden=128, heads=2, ffn=192), y=run_ref(m, *inp))
    m, inp = make_recsys(seed=4, batch=32, table_rows=50)
    G["recsys_small"] = dict(args=dict(seed=4, batch=32, table_rows=50), y=run_ref(m, *inp))

    def compact(o):  # detach views from their (possibly larger) storages
        if isinstance(o, torch.Tensor):
            return o.detach().clone().contiguous()
        if isinstance(o, dict):
            return {k: compact(v) for k, v in o.items()}
        if isinstance(o, (list, tuple)):
            return type(o)(compact(v) for v in o)
        return o

    out = os.path.join(HERE, "golden_v1.pt")
    torch.save(compact(G), out)
    print(f"wrote {out}: {len(G)} cases, {os.path.getsize(out) / 1024:.0f} KiB")


def main_v2():
    """Second fixture file: the row-sum fusions, chained / parallel / batched dense layers (added after golden_v1.pt;
    a separate file and generator so that the first one is never rewritten)."""
    G = {}
    g = torch.Generator().manual_seed(4321)

    def rn(*shape, dtype=torch.float32, std=1.0):
        return (torch.randn(*shape, generator=g) * std).to(dtype)

    for dt, tag in ((torch.float32, "f32"), (torch.bfloat16, "bf16")):
        x = rn(6, 40, 16, dtype=dt)
        for name, sl in (("prefix", [(0, 10), (0, 25), (0, 40), (0, 4)]), ("general", [(3, 10), (0, 25), (12, 40)])):
            G[f"slice_sum_cat_{name}_{tag}"] = dict(x=x, slices=sl, y=run_ref(
                lambda t, sl=sl: torch.cat([t[:, a:b, :].sum(dim=1) for a, b in sl], dim=-1) + 0, x))
        a = [rn(6, 5, 8, dtype=dt) for _ in range(3)]
        b = [rn(1 if i == 1 else 6, 5, 8, dtype=dt) for i in range(3)]
        G[f"mul_sum_cat_{tag}"] = dict(a=a, b=b, y=run_ref(
            lambda a0, a1, a2, b0, b1, b2: torch.cat([(a0 * b0).sum(dim=1), (a1 * b1).sum(dim=1), (a2 * b2).sum(dim=1)], dim=-1) + 0, *a, *b))
        ys = [rn(6, r, 8, dtype=dt) for r in (3, 7, 4)]
        G[f"sum_cat_{tag}"] = dict(xs=ys, y=run_ref(lambda y0, y1, y2: torch.cat([y0.sum(dim=1), y1.sum(dim=1), y2.sum(dim=1)], dim=-1) + 0, *ys))

    # chained dense layers (the dense tower) and parallel same-shape ones (the combo dense layer), fp32 / bf16
    x = rn(12, 24)
    ws = [rn(32, 24, std=0.2), rn(16, 32, std=0.2), rn(8, 16, std=0.2)]
    bs = [rn(32, std=0.1), rn(16, std=0.1), rn(8, std=0.1)]

    def tower(x, w0, w1, w2, b0, b1, b2):
        h = torch.relu(F.linear(x, w0, b0))
        h = torch.relu(F.linear(h, w1, b1))
        return F.linear(h, w2, b2)

    G["dense_tower_f32"] = dict(x=x, ws=ws, bs=bs, acts=["relu", "relu", "none"], y=run_ref(tower, x, *ws, *bs))
    xs = [rn(10, 16, dtype=torch.bfloat16) for _ in range(4)]
    wc = [rn(24, 16, dtype=torch.bfloat16, std=0.2) for _ in range(4)]
    bc = [rn(24, dtype=torch.bfloat16, std=0.1) for _ in range(4)]

    def combo(*t):
        return tuple(torch.relu(F.linear(t[i], t[4 + i], t[8 + i])) for i in range(4))

    G["combo_dense_bf16"] = dict(xs=xs, ws=wc, bs=bc, act="relu", y=list(run_ref(combo, *xs, *wc, *bc)))
    xb, wb, bb = rn(3, 10, 16), rn(3, 16, 12, std=0.2), rn(3, 1, 12, std=0.1)
    G["batch_dense_f32"] = dict(x=xb, w=wb, b=bb, act="gelu", y=run_ref(lambda x, w, b: F.gelu(torch.bmm(x, w) + b), xb, wb, bb))

    def compact(o):
        if isinstance(o, torch.Tensor):
            return o.detach().clone().contiguous()
        if isinstance(o, dict):
            return {k: compact(v) for k, v in o.items()}
        if isinstance(o, (list, tuple)):
            return type(o)(compact(v) for v in o)
        return o

    out = os.path.join(HERE, "golden_v2.pt")
    torch.save(compact(G), out)
    print(f"wrote {out}: {len(G)} cases, {os.path.getsize(out) / 1024:.0f} KiB")


def main_v3():
    """Third fixture file: 16-bit towers of two and three narrow dense layers (the shapes the chained-layer kernel
    takes), run through the reference pipeline like the others."""
    G = {}
    g = torch.Generator().manual_seed(8765)

    def rn(*shape, dtype=torch.float32, std=1.0):
        return (torch.randn(*shape, generator=g) * std).to(dtype)

    for dt, tag in ((torch.bfloat16, "bf16"), (torch.float16, "f16")):
        for name, M, dims, acts in (("two", 200, [72, 96, 40], ["relu", "none"]),
                                    ("three", 150, [64, 128, 64, 24], ["gelu", "relu", "sigmoid"])):
            x = rn(M, dims[0], dtype=dt)
            ws = [rn(dims[i + 1], dims[i], dtype=dt, std=dims[i] ** -0.5) for i in range(len(dims) - 1)]
            bs = [rn(dims[i + 1], dtype=dt, std=0.1) for i in range(len(dims) - 1)]
            fns = {"relu": torch.relu, "gelu": F.gelu, "sigmoid": torch.sigmoid, "none": lambda t: t}

            def tower(x, *wb, acts=acts, n=len(ws)):
                h = x
                for i in range(n):
                    h = fns[acts[i]](F.linear(h, wb[i], wb[n + i]))
                return h + 0

            G[f"tower_{name}_{tag}"] = dict(x=x, ws=ws, bs=bs, acts=acts, y=run_ref(tower, x, *ws, *bs))

    def compact(o):
        if isinstance(o, torch.Tensor):
            return o.detach().clone().contiguous()
        if isinstance(o, dict):
            return {k: compact(v) for k, v in o.items()}
        if isinstance(o, (list, tuple)):
            return type(o)(compact(v) for v in o)
        return o

    out = os.path.join(HERE, "golden_v3.pt")
    torch.save(compact(G), out)
    print(f"wrote {out}: {len(G)} cases, {os.path.getsize(out) / 1024:.0f} KiB")


def main_v4():
    """Fourth fixture file: see the module docstring."""
    G = {}
    g = torch.Generator().manual_seed(4321)

    def rn(*shape, dtype=torch.float32, std=1.0):
        return (torch.randn(*shape, generator=g) * std).to(dtype)

    T, M, K, N = 8, 5, 8, 7
    shared, split = rn(1, M, K), rn(T, M, K)
    ws = [rn(K, N) for _ in range(T)]
    rows, mats = [rn(N) for _ in range(T)], [rn(M, N) for _ in range(T)]

    def shared_plain(x, *w):
        x = x.squeeze(0)
        return tuple(x @ wi for wi in w)

    def shared_bias(x, *wb):
        x = x.squeeze(0)
        return tuple(x @ wi + bi for wi, bi in zip(wb[:T], wb[T:]))

    def shared_bias_relu(x, *wb):
        x = x.squeeze(0)
        return tuple(torch.relu(x @ wi + bi) for wi, bi in zip(wb[:T], wb[T:]))

    def split_linear_t(x, *w):
        xs = [i.squeeze(0) for i in x.split(x.shape[0] // T, dim=0)]
        return tuple(torch.relu(F.linear(xi, wi.T)) for xi, wi in zip(xs, w))

    G["combo_plain"] = dict(x=shared, ws=ws, bs=[None] * T, act="none", shared=True, y=list(run_ref(shared_plain, shared, *ws)))
    G["combo_matrix_bias"] = dict(x=shared, ws=ws, bs=mats, act="none", shared=True, y=list(run_ref(shared_bias, shared, *ws, *mats)))
    G["combo_row_bias"] = dict(x=shared, ws=ws, bs=rows, act="none", shared=True, y=list(run_ref(shared_bias, shared, *ws, *rows)))
    G["combo_matrix_bias_relu"] = dict(x=shared, ws=ws, bs=mats, act="relu", shared=True, y=list(run_ref(shared_bias_relu, shared, *ws, *mats)))
    G["combo_split_linear_t"] = dict(x=split, ws=ws, bs=[None] * T, act="relu", shared=False, y=list(run_ref(split_linear_t, split, *ws)))

    S, Mb, Kb, Nb = 3, 5, 6, 7
    xb = rn(S, Mb, Kb)
    wbs = [rn(S, Kb, Nb) for _ in range(T)]
    bbs = [rn(S, Mb, Nb) for _ in range(T)]

    def bmm_plain(x, *w):
        return tuple(torch.bmm(x, wi) for wi in w)

    def bmm_addend(x, *wb):
        return tuple(x @ wi + bi for wi, bi in zip(wb[:T], wb[T:]))

    G["combo_bmm_plain"] = dict(x=xb, ws=wbs, bs=[None] * T, y=list(run_ref(bmm_plain, xb, *wbs)))
    G["combo_bmm_addend"] = dict(x=xb, ws=wbs, bs=bbs, y=list(run_ref(bmm_addend, xb, *wbs, *bbs)))

    dims = (20, 32, 16, 1)
    x = rn(16, dims[0], dtype=torch.float16)
    tw = [rn(dims[i], dims[i + 1], dtype=torch.float16, std=dims[i] ** -0.5) for i in range(3)]
    tb = [rn(dims[i + 1], dtype=torch.float16) for i in range(3)]

    def tower(x, w1, w2, w3, b1, b2, b3):
        out = F.relu(torch.matmul(x, w1) + b1)
        out = F.relu(torch.matmul(out, w2) + b2)
        return torch.matmul(out, w3) + b3

    G["tower_kn_f16"] = dict(x=x, ws=tw, bs=tb, acts=["relu", "relu", "none"], y=run_ref(tower, x, *tw, *tb))

    xa, wa, ba = rn(50, 444, dtype=torch.bfloat16), rn(300, 444, dtype=torch.bfloat16, std=444 ** -0.5), rn(300, dtype=torch.bfloat16)
    G["dense_unaligned_bf16"] = dict(x=xa, w=wa, b=ba, act="gelu", y=run_ref(lambda x, w, b: F.gelu(F.linear(x, w, b)), xa, wa, ba))

    def compact(o):
        if isinstance(o, torch.Tensor):
            return o.detach().clone().contiguous()
        if isinstance(o, dict):
            return {k: compact(v) for k, v in o.items()}
        if isinstance(o, (list, tuple)):
            return type(o)(compact(v) for v in o)
        return o

    out = os.path.join(HERE, "golden_v4.pt")
    torch.save(compact(G), out)
    print(f"wrote {out}: {len(G)} cases, {os.path.getsize(out) / 1024:.0f} KiB")


if __name__ == "__main__":
    if len(sys.argv) > 1 and sys.argv[1] == "v2":
        main_v2()
    elif len(sys.argv) > 1 and sys.argv[1] == "v3":
        main_v3()
    elif len(sys.argv) > 1 and sys.argv[1] == "v4":
        main_v4()
    else:
        main()
