"""Plain, slow implementation of the dense Llama decoder: whole sequences, no cache.

It rests on the formulas of tracel-ai/burn-lm (the reference is Rust on top of the external
`burn` crate and cannot be imported or compiled here: there is no Rust toolchain), tightened by
the reference's own recorded unit-test vectors, which `tests/test_plain_anchor.py` parses out of
the reference's source files and reproduces with these functions.

One function for each part, numpy float64 throughout (or float32 on request), and no code shared
with the product package: it even reads model folders with the `safetensors` package instead of the
product's reader.  Every function cites the reference file:line whose formula it restates.
"""
from __future__ import annotations

import json
import math
import os

import numpy as np


# --------------------------------------------------------------------------------------------
# model folder -> plain dict
# --------------------------------------------------------------------------------------------
def read_model_folder(folder):
    """config.json as a dict and every tensor as float64, keyed by its stored name."""
    import torch
    from safetensors.torch import load_file

    with open(os.path.join(folder, "config.json")) as f:
        cfg = json.load(f)
    raw = load_file(os.path.join(folder, "model.safetensors"))
    tensors = {k: v.to(torch.float64).numpy() for k, v in raw.items()}
    return cfg, tensors


# --------------------------------------------------------------------------------------------
# parts
# --------------------------------------------------------------------------------------------
def embedding(table, tokens):
    """Row gather, no scale.  crates/burn-lm-llama/src/nn/transformer.rs:95"""
    return table[np.asarray(tokens, dtype=np.int64)]


def rms_norm(x, gamma, eps):
    """x / sqrt(mean(x^2) + eps) * gamma.  crates/burn-lm-llama/src/nn/transformer.rs:60-62,
    211-216 (construction with epsilon), checked by test_rms_norm at :278-297."""
    ms = (x * x).mean(axis=-1, keepdims=True)
    return x / np.sqrt(ms + eps) * gamma


def rope_inverse_frequencies(head_dim, theta):
    """theta^(-2i/head_dim) for each pair i.  The reference hands theta to burn's
    RotaryEncodingConfig: crates/burn-lm-llama/src/nn/llama/base.rs:269-277."""
    i = np.arange(0, head_dim, 2, dtype=np.float64)
    return 1.0 / (float(theta) ** (i / head_dim))


def llama3_frequency_scaling(freqs, factor, low_freq_factor, high_freq_factor, original_len):
    """Llama-3 scaling "by parts" of the inverse frequencies.
    crates/burn-lm-llama/src/nn/pos_encoding.rs:107-138: three masked passes whose net effect is
    wavelen < high_wavelen: unchanged; wavelen > low_wavelen: divided by the factor; between:
    interpolated with smooth = (original/wavelen - low) / (high - low)."""
    low_wavelen = original_len / low_freq_factor
    high_wavelen = original_len / high_freq_factor
    out = np.empty_like(freqs)
    for n, f in enumerate(freqs):
        wavelen = 2.0 * math.pi / f
        if wavelen < high_wavelen:
            out[n] = f
        elif wavelen > low_wavelen:
            out[n] = f / factor
        else:
            smooth = (original_len / wavelen - low_freq_factor) / (high_freq_factor - low_freq_factor)
            out[n] = (1.0 - smooth) * f / factor + smooth * f
    return out


def rope_apply(x, positions, inv_freq, pairing):
    """Rotate pairs of lanes of x [..., T, head_dim] by positions[t] * inv_freq[i].
    crates/burn-lm-llama/src/nn/attention/mha.rs:91-92 and pos_encoding.rs:60-62 (applied to q and
    k after projection, at the sequence's absolute positions).  `interleaved` pairs lanes
    (2i, 2i+1), the reference's layout; `half` pairs lanes (i, i + head_dim/2), the layout of
    weights stored under Hugging Face names (llama/import.rs:95-126 is the permutation between
    the two)."""
    ang = np.outer(np.asarray(positions, dtype=np.float64), inv_freq)  # [T, hd/2]
    c, s = np.cos(ang), np.sin(ang)
    out = np.empty_like(x)
    half = x.shape[-1] // 2
    if pairing == "interleaved":
        a, b = x[..., 0::2], x[..., 1::2]
        out[..., 0::2] = a * c - b * s
        out[..., 1::2] = a * s + b * c
    elif pairing == "half":
        a, b = x[..., :half], x[..., half:]
        out[..., :half] = a * c - b * s
        out[..., half:] = a * s + b * c
    else:
        raise ValueError(pairing)
    return out


def softmax(x, axis=-1):
    m = x.max(axis=axis, keepdims=True)
    e = np.exp(x - m)
    return e / e.sum(axis=axis, keepdims=True)


def attention(xn, wq, wk, wv, wo, n_heads, n_kv_heads, head_dim, inv_freq, pairing,
              window=None, positions=None):
    """Causal grouped-query attention of one whole sequence xn [T, D]; weights are [out, in].
    crates/burn-lm-llama/src/nn/attention/mha.rs:121-140 (projections, head split), :91-92
    (rotation of q and k), :174-185 (a query head h reads kv head h // group), :157-166
    (scores / sqrt(head_dim), mask to -inf, softmax, times v), :168-170 and :118 (merge, wo)."""
    T = xn.shape[0]
    if positions is None:
        positions = np.arange(T)
    q = (xn @ wq.T).reshape(T, n_heads, head_dim).transpose(1, 0, 2)
    k = (xn @ wk.T).reshape(T, n_kv_heads, head_dim).transpose(1, 0, 2)
    v = (xn @ wv.T).reshape(T, n_kv_heads, head_dim).transpose(1, 0, 2)
    if inv_freq is not None:
        q = rope_apply(q, positions, inv_freq, pairing)
        k = rope_apply(k, positions, inv_freq, pairing)
    group = n_heads // n_kv_heads
    k = np.repeat(k, group, axis=0)
    v = np.repeat(v, group, axis=0)
    scores = q @ k.transpose(0, 2, 1) / math.sqrt(head_dim)
    i = np.arange(T)[:, None]
    j = np.arange(T)[None, :]
    hidden = j > i
    if window is not None:
        hidden = hidden | (j <= i - window)
    scores = np.where(hidden[None], -np.inf, scores)
    p = softmax(scores, axis=-1)
    o = (p @ v).transpose(1, 0, 2).reshape(T, n_heads * head_dim)
    return o @ wo.T


def silu(z):
    return z / (1.0 + np.exp(-z))


def feed_forward(xn, w_gate, w_up, w_down):
    """(silu(x Wgate) * (x Wup)) Wdown, no biases; weights are [out, in].
    crates/burn-lm-llama/src/nn/fftn.rs:26-36,44-46, checked by test_fftn at :57-92."""
    return (silu(xn @ w_gate.T) * (xn @ w_up.T)) @ w_down.T


def block(h, lw, cfg, inv_freq, pairing):
    """Pre-norm residual block.  crates/burn-lm-llama/src/nn/transformer.rs:241-256."""
    a = attention(rms_norm(h, lw["input_layernorm"], cfg["rms_norm_eps"]),
                  lw["q_proj"], lw["k_proj"], lw["v_proj"], lw["o_proj"],
                  cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"],
                  inv_freq, pairing)
    h = h + a
    f = feed_forward(rms_norm(h, lw["post_attention_layernorm"], cfg["rms_norm_eps"]),
                     lw["gate_proj"], lw["up_proj"], lw["down_proj"])
    return h + f


# --------------------------------------------------------------------------------------------
# whole model
# --------------------------------------------------------------------------------------------
def complete_config(cfg):
    """Fill the defaults the reference uses: kv heads = heads (llama/base.rs:254), head_dim =
    width / heads (attention/mha.rs:191), eps 1e-5 (transformer.rs:39-40), theta 10000
    (llama/base.rs:61-62)."""
    c = dict(cfg)
    c.setdefault("num_key_value_heads", c["num_attention_heads"])
    if c.get("head_dim") is None:
        c["head_dim"] = c["hidden_size"] // c["num_attention_heads"]
    c.setdefault("rms_norm_eps", 1e-5)
    c.setdefault("rope_theta", 10000.0)
    c.setdefault("tie_word_embeddings", False)
    return c


def model_inverse_frequencies(cfg):
    inv = rope_inverse_frequencies(cfg["head_dim"], cfg["rope_theta"])
    rs = cfg.get("rope_scaling")
    if rs:
        kind = rs.get("rope_type", rs.get("type"))
        if kind != "llama3":
            raise ValueError(f"plain implementation knows llama3 scaling only, not {kind}")
        inv = llama3_frequency_scaling(inv, rs["factor"], rs["low_freq_factor"],
                                       rs["high_freq_factor"],
                                       rs["original_max_position_embeddings"])
    return inv


def layer_weights(tensors, n):
    p = f"model.layers.{n}."
    return {
        "input_layernorm": tensors[p + "input_layernorm.weight"],
        "post_attention_layernorm": tensors[p + "post_attention_layernorm.weight"],
        "q_proj": tensors[p + "self_attn.q_proj.weight"],
        "k_proj": tensors[p + "self_attn.k_proj.weight"],
        "v_proj": tensors[p + "self_attn.v_proj.weight"],
        "o_proj": tensors[p + "self_attn.o_proj.weight"],
        "gate_proj": tensors[p + "mlp.gate_proj.weight"],
        "up_proj": tensors[p + "mlp.up_proj.weight"],
        "down_proj": tensors[p + "mlp.down_proj.weight"],
    }


def forward(cfg, tensors, tokens, pairing="half"):
    """Logits [T, V] at every position of one whole sequence.
    crates/burn-lm-llama/src/nn/transformer.rs:88-103: embed, the blocks in order, final norm,
    output projection (the embedding table when tie_word_embeddings)."""
    cfg = complete_config(cfg)
    inv_freq = model_inverse_frequencies(cfg)
    h = embedding(tensors["model.embed_tokens.weight"], tokens)
    for n in range(cfg["num_hidden_layers"]):
        h = block(h, layer_weights(tensors, n), cfg, inv_freq, pairing)
    h = rms_norm(h, tensors["model.norm.weight"], cfg["rms_norm_eps"])
    head = (tensors["model.embed_tokens.weight"] if cfg["tie_word_embeddings"]
            else tensors["lm_head.weight"])
    return h @ head.T


# --------------------------------------------------------------------------------------------
# sampling
# --------------------------------------------------------------------------------------------
def greedy(logits):
    """argmax over raw logits; the lowest index wins a tie.
    crates/burn-lm-llama/src/generation/sampling.rs:15-20."""
    return int(np.argmax(logits))


def temperature_softmax(logits, temperature):
    """softmax(logits / temperature).  crates/burn-lm-llama/src/generation/generate.rs:8-10."""
    return softmax(np.asarray(logits, dtype=np.float64) / temperature, axis=-1)


def top_p_keep(probs, p):
    """The nucleus: in descending order a token is kept while the mass before it is < p.
    crates/burn-lm-llama/src/generation/sampling.rs:44-70.  Equal probabilities are ordered by
    index (the reference leaves their order to its sort).  Returns a boolean mask."""
    order = np.lexsort((np.arange(len(probs)), -probs))
    keep = np.zeros(len(probs), dtype=bool)
    cum = 0.0
    for idx in order:
        if cum >= p:
            break
        keep[idx] = True
        cum += probs[idx]
    return keep


def top_p_draw(probs, p, u):
    """Draw from the kept tokens in proportion to their probability: the first token, in
    vocabulary order, at which the running kept mass exceeds u * (kept mass)."""
    keep = top_p_keep(probs, p)
    kept = np.where(keep, probs, 0.0)
    target = u * kept.sum()
    run = 0.0
    last = -1
    for i, w in enumerate(kept):
        if w <= 0.0:
            continue
        run += w
        last = i
        if run > target:
            return i
    return last


def greedy_generate(cfg, tensors, prompt, n_new, stop_ids=(), pairing="half"):
    """Whole-sequence greedy generation: every new token recomputes the whole sequence.
    crates/burn-lm-llama/src/generation/generate.rs:61-98 (loop), stop ids end a sequence and
    are not part of the output (generation/context.rs:142-170)."""
    seq = list(prompt)
    out = []
    for _ in range(n_new):
        tok = greedy(forward(cfg, tensors, seq, pairing)[-1])
        if tok in stop_ids:
            break
        out.append(tok)
        seq.append(tok)
    return out
