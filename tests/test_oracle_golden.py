"""The CPU oracle against the golden fixtures recorded from the xpu_graph reference itself
(tests/golden/gen_golden.py). This is what pins the oracle: every restated function must reproduce the
reference's outputs on the reference's inputs."""
import os

import pytest
import torch

from oracle import ref_ops
from tests.helpers import assert_bit_exact, assert_parity

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "golden_v1.pt")


@pytest.fixture(scope="module")
def G():
    return torch.load(GOLDEN)


def _close(a, e, what):
    # same machine arithmetic on both sides: fp32 within 1e-5 relative, 16-bit within one rounding
    assert_parity(a, e, what)


@pytest.mark.parametrize("tag", ["bf16", "f32"])
def test_default_norm_modules(G, tag):
    c = G[f"default_rms_{tag}"]
    assert_bit_exact(ref_ops.rms_norm(c["x"], c["w"], c["eps"]), c["y"], "DefaultRMSNorm")
    c = G[f"default_ln_{tag}"]
    assert_bit_exact(ref_ops.layer_norm(c["x"], c["w"], c["b"], c["eps"]), c["y"], "DefaultLayerNorm")


@pytest.mark.parametrize("tag", ["bf16", "f32"])
def test_add_norms(G, tag):
    c = G[f"add_rms_{tag}"]
    y, s = ref_ops.add_rms_norm(c["x"], c["r"], c["w"], c["eps"])
    assert_bit_exact(s, c["s"], "add_rms sum")
    _close(y, c["y"], "add_rms y")
    c = G[f"add_ln_{tag}"]
    y, s = ref_ops.add_layer_norm(c["x"], c["r"], c["w"], c["b"], c["eps"])
    assert_bit_exact(s, c["s"], "add_ln sum")
    _close(y, c["y"], "add_ln y")


@pytest.mark.parametrize("act", ["none", "gelu", "relu", "silu", "sigmoid"])
def test_dense(G, act):
    c = G[f"dense_{act}_f32"]
    _close(ref_ops.dense(c["x"], c["w"], True, c["b"], act), c["y"], f"dense {act}")


def test_dense_variants(G):
    c = G["dense_nobias_bf16"]
    _close(ref_ops.dense(c["x"], c["w"], True, None, "gelu"), c["y"], "dense bf16 no bias")
    c = G["dense_kn_residual_f32"]
    _close(ref_ops.dense(c["x"], c["w"], False, c["r"], "none"), c["y"], "dense [K,N] + residual")


def test_sdpa(G):
    c = G["sdpa_f32"]
    q, k, v = (t.unsqueeze(0) for t in (c["q"], c["k"], c["v"]))
    _close(ref_ops.sdpa(q, k, v, None, c["scale"]).squeeze(0), c["y"], "sdpa f32")
    _close(ref_ops.sdpa_math(q, k, v, None, c["scale"]).squeeze(0), c["y"], "sdpa_math f32")
    c = G["sdpa_mask_f32"]
    q, k, v, m = (t.unsqueeze(0) for t in (c["q"], c["k"], c["v"], c["m"]))
    _close(ref_ops.sdpa(q, k, v, m, c["scale"]).squeeze(0), c["y"], "sdpa mask f32")
    c = G["sdpa_bf16"]
    q, k, v = (t.unsqueeze(0) for t in (c["q"], c["k"], c["v"]))
    _close(ref_ops.sdpa(q, k, v, None, c["scale"]).squeeze(0), c["y"], "sdpa bf16")
    c = G["sdpa_causal_bf16"]
    _close(ref_ops.sdpa(c["q"], c["k"], c["v"], None, None, True), c["y"], "sdpa causal bf16")
    _close(ref_ops.sdpa_math(c["q"], c["k"], c["v"], None, None, True).to(torch.bfloat16), c["y"], "sdpa_math causal")


@pytest.mark.parametrize("name", ["even", "ragged", "int64max", "negative_end", "bf16"])
def test_slice_cat(G, name):
    c = G[f"slice_cat_{name}"]
    assert_bit_exact(ref_ops.slice_cat(c["src"], c["slices"]), c["y"], f"slice_cat {name}")


def test_other_copy_fusions(G):
    c = G["multi_slice"]
    assert_bit_exact(ref_ops.multi_slice(c["src"], c["starts"], c["length"]), c["y"], "multi_slice")
    c = G["masked_slice_cat"]
    assert_bit_exact(ref_ops.masked_slice_cat(c["src"], c["mask"], c["slices"]), c["y"], "masked slice_cat")
    c = G["gather_stack"]
    assert_bit_exact(ref_ops.gather_stack(c["tables"], c["idx"], c["mask"]), c["y"], "gather_stack")
    many = [G["slice_cat_even"]["slices"], G["slice_cat_ragged"]["slices"]]
    outs = ref_ops.slice_cat_multi(G["slice_cat_even"]["src"], many)
    assert_bit_exact(outs[0], G["slice_cat_even"]["y"], "slice_cat_multi 0")
    assert_bit_exact(outs[1], G["slice_cat_ragged"]["y"], "slice_cat_multi 1")


@pytest.mark.parametrize("tag", ["bf16", "f32"])
def test_rope_swiglu(G, tag):
    c = G[f"rope_{tag}"]
    assert_bit_exact(ref_ops.rope(c["x"], c["cos"], c["sin"]), c["y"], "rope")
    c = G[f"swiglu_{tag}"]
    assert_bit_exact(ref_ops.swiglu(c["gate"], c["up"]), c["y"], "swiglu")


def test_benchmark_graphs_small(G):
    """The eager workload models reproduce what the reference pipeline returned for them."""
    from xpu_graph_b200.workloads import make_encoder, make_llama_layer, make_recsys

    c = G["encoder_small"]
    m, x = make_encoder(**c["args"])
    with torch.no_grad():
        _close(m(x), c["y"], "encoder")
    c = G["llama_small"]
    m, inp = make_llama_layer(**c["args"])
    with torch.no_grad():
        _close(m(*inp), c["y"], "llama layer")
    c = G["recsys_small"]
    m, inp = make_recsys(**c["args"])
    with torch.no_grad():
        _close(m(*inp), c["y"], "recsys")


# ---- second fixture file: row-sum fusions, chained / parallel / batched dense layers ------------------------------
GOLDEN2 = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "golden_v2.pt")


@pytest.fixture(scope="module")
def G2():
    return torch.load(GOLDEN2)


@pytest.mark.parametrize("tag", ["f32", "bf16"])
def test_row_sum_fusions(G2, tag):
    for name in ("prefix", "general"):
        c = G2[f"slice_sum_cat_{name}_{tag}"]
        assert_bit_exact(ref_ops.slice_sum_cat(c["x"], c["slices"]), c["y"], f"slice_sum_cat {name}")
    c = G2[f"mul_sum_cat_{tag}"]
    ml = []
    for a, b in zip(c["a"], c["b"]):
        ml += [a, b]
    assert_bit_exact(ref_ops.mul_sum_cat(ml), c["y"], "mul_sum_cat")
    c = G2[f"sum_cat_{tag}"]
    assert_bit_exact(ref_ops.sum_cat(c["xs"]), c["y"], "sum_cat")


def test_dense_chains(G2):
    c = G2["dense_tower_f32"]
    y = c["x"]
    for w, b, a in zip(c["ws"], c["bs"], c["acts"]):
        y = ref_ops.dense(y, w, True, b, a)
    _close(y, c["y"], "dense tower")
    c = G2["combo_dense_bf16"]
    for x, w, b, want in zip(c["xs"], c["ws"], c["bs"], c["y"]):
        _close(ref_ops.dense(x, w, True, b, c["act"]), want, "combo dense member")
    c = G2["batch_dense_f32"]
    _close(ref_ops.batch_dense(c["x"], c["w"], False, c["b"], c["act"]), c["y"], "batch dense")


GOLDEN3 = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "golden_v3.pt")


@pytest.mark.parametrize("tag", ["bf16", "f16"])
@pytest.mark.parametrize("name", ["two", "three"])
def test_narrow_towers(name, tag):
    """16-bit towers of two / three narrow dense layers as the reference pipeline computes them (golden_v3.pt): the
    oracle's layer-by-layer chain reproduces them."""
    c = torch.load(GOLDEN3)[f"tower_{name}_{tag}"]
    y = c["x"]
    for w, b, a in zip(c["ws"], c["bs"], c["acts"]):
        y = ref_ops.dense(y, w, True, b, a)
    _close(y, c["y"], f"tower {name} {tag}")



GOLDEN4 = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "golden_v4.pt")


def test_combo_tower_and_unaligned_forms():
    """The reference's combo and dense-tower test graphs at their own sizes, and a bf16 layer with 888-byte rows, as the
    reference pipeline computes them (golden_v4.pt): the oracle's per-layer functions reproduce them."""
    G4 = torch.load(GOLDEN4)
    for name in ("combo_plain", "combo_matrix_bias", "combo_row_bias", "combo_matrix_bias_relu", "combo_split_linear_t"):
        c = G4[name]
        xs = [c["x"][0]] * len(c["ws"]) if c["shared"] else list(c["x"].unbind(0))
        for x, w, b, want in zip(xs, c["ws"], c["bs"], c["y"]):
            _close(ref_ops.dense(x, w, False, b, c["act"]), want, name)
    for name in ("combo_bmm_plain", "combo_bmm_addend"):
        c = G4[name]
        for w, b, want in zip(c["ws"], c["bs"], c["y"]):
            _close(ref_ops.batch_dense(c["x"], w, False, b, "none"), want, name)
    c = G4["tower_kn_f16"]
    y = c["x"]
    for w, b, a in zip(c["ws"], c["bs"], c["acts"]):
        y = ref_ops.dense(y, w, False, b, a)
    _close(y, c["y"], "tower with [K, N] weights, fp16")
    c = G4["dense_unaligned_bf16"]
    _close(ref_ops.dense(c["x"], c["w"], True, c["b"], c["act"]), c["y"], "bf16 layer with K = 444")
