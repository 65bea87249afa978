"""The plain implementation against the reference's own recorded test vectors.

The expected arrays are parsed out of the reference's Rust sources at run time (nothing is copied
here); the tests skip when that tree is not mounted.  The reference re-initialises every float
parameter with `arange(n) * 5 / n` in burn's `[d_in, d_out]` layout
(crates/burn-lm-llama/src/lib.rs:142-148,199-205), so the plain functions, which take `[out, in]`
matrices, get the transposes.
"""
import ast
import os
import re

import numpy as np
import pytest

from plain import llama_plain as P

# the reference's tree: where BURN_LM_REFERENCE says, else a folder `reference` beside this repository
REF = os.environ.get("BURN_LM_REFERENCE") or os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))), "reference")
LLAMA = os.path.join(REF, "crates", "burn-lm-llama", "src")

pytestmark = pytest.mark.skipif(not os.path.isdir(LLAMA), reason="reference tree not mounted")


def rust_array(path, fn_name, which):
    """The `which`-th bracketed float array literal inside `fn fn_name`."""
    src = open(os.path.join(LLAMA, path)).read()
    start = src.index(f"fn {fn_name}(")
    nxt = src.find("#[test]", start)
    body = src[start: nxt if nxt > 0 else len(src)]
    found = []
    for m in re.finditer(r"(?:from|TensorData::from)\(\s*(\[)", body):
        i = m.start(1)
        depth = 0
        for j in range(i, len(body)):
            if body[j] == "[":
                depth += 1
            elif body[j] == "]":
                depth -= 1
                if depth == 0:
                    break
        lit = body[i: j + 1]
        lit = re.sub(r",\s*\]", "]", lit)
        # the text comes from outside this repository: numbers, brackets and commas only, and never evaluated as code
        assert re.fullmatch(r"[\s\d.,eE+\-\[\]]+", lit), f"not a plain array literal in {path}::{fn_name}: {lit[:60]!r}"
        found.append(np.array(ast.literal_eval(lit), dtype=np.float64))
    return found[which]


def ramp(shape):
    n = int(np.prod(shape))
    return (np.arange(n, dtype=np.float64) * (5.0 / n)).reshape(shape)


def test_rms_norm_vector():
    x = rust_array("nn/transformer.rs", "test_rms_norm", 0)
    want = rust_array("nn/transformer.rs", "test_rms_norm", 1)
    got = P.rms_norm(x, np.ones(4), 1e-5)
    np.testing.assert_allclose(got, want, rtol=2e-3)  # recorded in half precision


def test_feed_forward_vector():
    want = rust_array("nn/fftn.rs", "test_fftn", 0)
    x = np.arange(16, dtype=np.float64).reshape(2, 2, 4)
    got = P.feed_forward(x, ramp((4, 8)).T, ramp((4, 8)).T, ramp((8, 4)).T)
    np.testing.assert_allclose(got, want, rtol=1e-6)


def test_rope_vector():
    x = rust_array("nn/pos_encoding.rs", "test_rope", 0)
    want = rust_array("nn/pos_encoding.rs", "test_rope", 1)
    inv = P.llama3_frequency_scaling(P.rope_inverse_frequencies(2, 500000.0), 32.0, 1.0, 4.0, 8192.0)
    for pairing in ("interleaved", "half"):  # one pair: both layouts are the same
        got = P.rope_apply(x, np.arange(2), inv, pairing)
        # recorded from a bfloat16 run (8 mantissa bits); the reference itself allows 5 %
        np.testing.assert_allclose(got, want, rtol=8e-3)


def test_temperature_softmax_vector():
    logits = rust_array("generation/generate.rs", "test_temperature_softmax", 0)
    want = rust_array("generation/generate.rs", "test_temperature_softmax", 1)
    got = P.temperature_softmax(logits, 0.6)
    np.testing.assert_allclose(got, want, rtol=0.05)  # the reference's own tolerance


def test_whole_transformer_vector():
    """TransformerConfig::new(8, 2, 8, 16, 2, 1): vocab 8, 2 layers, width 8, inner 16, 2 heads,
    1 kv head; tokens [[0,1],[2,3]]; theta 10000 (transformer.rs:299-349)."""
    want = rust_array("nn/transformer.rs", "test_transformer", 0)
    V, L, D, I, H, KV = 8, 2, 8, 16, 2, 1
    hd = D // H
    cfg = dict(hidden_size=D, intermediate_size=I, num_hidden_layers=L, num_attention_heads=H,
               num_key_value_heads=KV, vocab_size=V, rms_norm_eps=1e-5, rope_theta=10000.0,
               tie_word_embeddings=False)
    t = {"model.embed_tokens.weight": ramp((V, D)), "model.norm.weight": ramp((D,)),
         "lm_head.weight": ramp((D, V)).T}
    for n in range(L):
        p = f"model.layers.{n}."
        t[p + "self_attn.q_proj.weight"] = ramp((D, H * hd)).T
        t[p + "self_attn.k_proj.weight"] = ramp((D, KV * hd)).T
        t[p + "self_attn.v_proj.weight"] = ramp((D, KV * hd)).T
        t[p + "self_attn.o_proj.weight"] = ramp((H * hd, D)).T
        t[p + "mlp.gate_proj.weight"] = ramp((D, I)).T
        t[p + "mlp.up_proj.weight"] = ramp((D, I)).T
        t[p + "mlp.down_proj.weight"] = ramp((I, D)).T
        t[p + "input_layernorm.weight"] = ramp((D,))
        t[p + "post_attention_layernorm.weight"] = ramp((D,))
    for b, toks in enumerate(([0, 1], [2, 3])):
        got = P.forward(cfg, t, toks, pairing="interleaved")
        np.testing.assert_allclose(got, want[b], rtol=1e-6)


def test_pairings_agree_after_permuting_rows():
    """The two lane pairings give the same logits when q/k rows are permuted between the layouts
    (llama/import.rs:95-126: reshape [.., heads, 2, hd/2] and swap the last two)."""
    rng = np.random.default_rng(0)
    D, H, KV, hd, I, V = 24, 3, 1, 8, 40, 19
    cfg = dict(hidden_size=D, intermediate_size=I, num_hidden_layers=1, num_attention_heads=H,
               num_key_value_heads=KV, head_dim=hd, vocab_size=V, rms_norm_eps=1e-6,
               rope_theta=100.0, tie_word_embeddings=True)
    t = {"model.embed_tokens.weight": rng.normal(size=(V, D)), "model.norm.weight": np.ones(D)}
    p = "model.layers.0."
    shapes = {"self_attn.q_proj": (H * hd, D), "self_attn.k_proj": (KV * hd, D),
              "self_attn.v_proj": (KV * hd, D), "self_attn.o_proj": (D, H * hd),
              "mlp.gate_proj": (I, D), "mlp.up_proj": (I, D), "mlp.down_proj": (D, I)}
    for k, s in shapes.items():
        t[p + k + ".weight"] = rng.normal(size=s) * 0.3
    t[p + "input_layernorm.weight"] = np.ones(D)
    t[p + "post_attention_layernorm.weight"] = np.ones(D)
    toks = [3, 1, 4, 1, 5, 9, 2, 6]
    half = P.forward(cfg, t, toks, pairing="half")

    def to_interleaved(w, heads):
        return w.reshape(heads, 2, hd // 2, -1).transpose(0, 2, 1, 3).reshape(heads * hd, -1)

    t2 = dict(t)
    t2[p + "self_attn.q_proj.weight"] = to_interleaved(t[p + "self_attn.q_proj.weight"], H)
    t2[p + "self_attn.k_proj.weight"] = to_interleaved(t[p + "self_attn.k_proj.weight"], KV)
    inter = P.forward(cfg, t2, toks, pairing="interleaved")
    np.testing.assert_allclose(inter, half, rtol=1e-9, atol=1e-12)
