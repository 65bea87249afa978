"""Anchors for the Llama-3 frequency scaling and for the `half` pairing that do not rest on the loop
that the plain implementation and the product's position part both carry.

The reference's own test of the scaling (crates/burn-lm-llama/src/nn/pos_encoding.rs:150-178) has one
pair whose frequency stays unchanged, so the two other branches need anchors of their own:

1. the reference's code itself is three masked passes over the whole vector, in an order that matters
   (pos_encoding.rs:107-138); `three_passes` below restates those passes one tensor operation at a time,
   which is another form than an if / elif over single frequencies;
2. values worked out by hand from the same lines for frequencies whose wavelengths are round numbers.

The `half` pairing rests on the reference's weight permutation between the two layouts
(crates/burn-lm-llama/src/nn/llama/import.rs:95-126): a model whose q and k rows are permuted that way
and rotated in adjacent pairs must give the logits of the stored model rotated in halves.

No installed package's model code is imported here: the reference's files are the only source.
"""
import math

import numpy as np
import pytest

from plain import llama_plain as P
from tiny import TINY_B, TINY_C, TINY_D, make_folder, random_tokens


def three_passes(freqs, scale_factor, low_freq_factor, high_freq_factor, old_context_len):
    """pos_encoding.rs:107-138, statement by statement."""
    freqs = np.asarray(freqs, dtype=np.float64)
    low_freq_wavelen = old_context_len / low_freq_factor                          # :108
    high_freq_wavelen = old_context_len / high_freq_factor                        # :109
    wavelen = (1.0 / freqs) * (2.0 * math.pi)                                     # :111
    cond = wavelen >= high_freq_wavelen                                           # :114
    smooth = ((1.0 / wavelen) * old_context_len - low_freq_factor) / (high_freq_factor - low_freq_factor)   # :115-120
    new_freqs = (-smooth + 1.0) * (freqs / scale_factor) + smooth * freqs         # :122-127
    new_freqs = np.where(cond, new_freqs, freqs)                                  # :128  mask_where(cond, value)
    cond = wavelen > low_freq_wavelen                                             # :131
    new_freqs = np.where(cond, freqs / scale_factor, new_freqs)                   # :132
    cond = wavelen < high_freq_wavelen                                            # :135
    return np.where(cond, freqs, new_freqs)                                       # :137


def product_frequencies(head_dim, theta, scaling):
    from burn_lm_b200.parts.position import Llama3Scaling, RotarySpec, rotary_inverse_frequencies
    s = Llama3Scaling(*scaling) if scaling else None
    return np.array(rotary_inverse_frequencies(RotarySpec(head_dim=head_dim, theta=theta, scaling=s)))


SCALINGS = [(8.0, 1.0, 4.0, 64), (32.0, 1.0, 4.0, 8192), (4.0, 1.0, 2.0, 128), (32.0, 1.0, 4.0, 256), (8.0, 2.0, 8.0, 1000)]


@pytest.mark.parametrize("head_dim,theta", [(32, 500000.0), (64, 500000.0), (128, 500000.0), (48, 50000.0), (16, 10000.0)])
@pytest.mark.parametrize("scaling", SCALINGS)
def test_plain_and_product_equal_the_three_passes(head_dim, theta, scaling):
    base = P.rope_inverse_frequencies(head_dim, theta)
    want = three_passes(base, *scaling)
    np.testing.assert_allclose(P.llama3_frequency_scaling(base, *scaling), want, rtol=1e-14)
    np.testing.assert_allclose(product_frequencies(head_dim, theta, scaling), want, rtol=1e-13)
    np.testing.assert_allclose(product_frequencies(head_dim, theta, None), base, rtol=1e-13)


def test_the_edges_between_the_branches():
    """Wavelengths exactly at the two limits: at the high-frequency limit the interpolation gives the
    frequency itself (smooth = 1), at the low-frequency limit the divided one (smooth = 0), so the passes
    and the loop agree there as well, whichever side takes the equality."""
    factor, low, high, old = 8.0, 1.0, 4.0, 64
    freqs = np.array([2 * math.pi / 16.0, 2 * math.pi / 64.0, 2 * math.pi / 15.999, 2 * math.pi / 64.001])
    want = three_passes(freqs, factor, low, high, old)
    np.testing.assert_allclose(P.llama3_frequency_scaling(freqs, factor, low, high, old), want, rtol=1e-12)
    np.testing.assert_allclose(want / freqs, [1.0, 1 / 8, 1.0, 1 / 8], rtol=1e-4)


def test_values_worked_out_by_hand():
    """old_context_len 64, low 1, high 4, factor 8: the limits are wavelengths 64 and 16.
    wavelength 2 pi (f = 1): below 16, unchanged.  wavelength 32: smooth = (64 / 32 - 1) / 3 = 1 / 3, so
    f' = (2/3) f / 8 + (1/3) f = (5 / 12) f.  wavelength 24: smooth = (64 / 24 - 1) / 3 = 5 / 9, so
    f' = (4/9) f / 8 + (5/9) f = (11 / 18) f.  wavelength 128: above 64, f / 8."""
    f = np.array([1.0, 2 * math.pi / 32, 2 * math.pi / 24, 2 * math.pi / 128])
    want = f * np.array([1.0, 5.0 / 12.0, 11.0 / 18.0, 1.0 / 8.0])
    np.testing.assert_allclose(three_passes(f, 8.0, 1.0, 4.0, 64), want, rtol=1e-14)
    np.testing.assert_allclose(P.llama3_frequency_scaling(f, 8.0, 1.0, 4.0, 64), want, rtol=1e-14)
    from burn_lm_b200.parts.position import Llama3Scaling, RotarySpec, rotary_inverse_frequencies
    # the product's function builds its own base frequencies: theta 1, so that every pair has f = 1 (unchanged) ...
    got = rotary_inverse_frequencies(RotarySpec(head_dim=8, theta=1.0, scaling=Llama3Scaling(8.0, 1.0, 4.0, 64)))
    np.testing.assert_allclose(got, [1.0] * 4, rtol=1e-14)
    # ... and theta chosen so that pair 1 of 2 has the wavelength 32, 24 or 128: f_1 = theta^(-1/2)
    for wavelen, ratio in ((32.0, 5.0 / 12.0), (24.0, 11.0 / 18.0), (128.0, 1.0 / 8.0)):
        theta = (wavelen / (2 * math.pi)) ** 2
        got = rotary_inverse_frequencies(RotarySpec(head_dim=4, theta=theta, scaling=Llama3Scaling(8.0, 1.0, 4.0, 64)))
        np.testing.assert_allclose(got, [1.0, 2 * math.pi / wavelen * ratio], rtol=1e-12)


def permute_rows_to_adjacent_pairs(w, n_heads):
    """import.rs:103-109 on a weight stored [out, in]: the reference's matrices are [in, out], and it regroups
    the out axis of every head from (2, head_dim / 2) to (head_dim / 2, 2): lane i of the first half and lane i
    of the second half become neighbours."""
    out, width = w.shape
    hd = out // n_heads
    return w.reshape(n_heads, 2, hd // 2, width).swapaxes(1, 2).reshape(out, width)


@pytest.mark.parametrize("name", ["tiny_b", "tiny_c", "tiny_d"])
def test_half_pairing_equals_adjacent_pairs_on_permuted_weights(tmp_path, name):
    cfg, tensors = P.read_model_folder(make_folder(tmp_path, name, seed=4, dtype="float32"))
    toks = random_tokens(7, 50, cfg["vocab_size"])
    want = P.forward(cfg, tensors, toks, pairing="half")
    permuted = dict(tensors)
    for n in range(cfg["num_hidden_layers"]):
        p = f"model.layers.{n}.self_attn."
        permuted[p + "q_proj.weight"] = permute_rows_to_adjacent_pairs(tensors[p + "q_proj.weight"], cfg["num_attention_heads"])
        permuted[p + "k_proj.weight"] = permute_rows_to_adjacent_pairs(tensors[p + "k_proj.weight"], cfg["num_key_value_heads"])
    got = P.forward(cfg, permuted, toks, pairing="interleaved")
    np.testing.assert_allclose(got, want, rtol=1e-9, atol=1e-11)
    # and the pairing matters: the stored weights rotated in adjacent pairs give other logits
    assert np.abs(P.forward(cfg, tensors, toks, pairing="interleaved") - want).max() > 1e-3 * np.abs(want).max()
