"""The plain implementation checked against itself: properties that do not need the engine."""
import numpy as np

from plain import llama_plain as P
from tiny import TINY_B, make_folder, random_tokens


def test_prefix_logits_do_not_depend_on_what_follows(tmp_path):
    cfg, t = P.read_model_folder(make_folder(tmp_path, "tiny_b", seed=1, dtype="float32"))
    toks = random_tokens(0, 40, cfg["vocab_size"])
    full = P.forward(cfg, t, toks)
    part = P.forward(cfg, t, toks[:17])
    np.testing.assert_allclose(full[:17], part, rtol=1e-10, atol=1e-12)


def test_llama3_scaling_hits_all_three_branches():
    cfg = P.complete_config(TINY_B)
    base = P.rope_inverse_frequencies(cfg["head_dim"], cfg["rope_theta"])
    scaled = P.model_inverse_frequencies(cfg)
    ratio = scaled / base
    assert np.isclose(ratio, 1.0).any() and np.isclose(ratio, 1 / 8).any()
    assert ((ratio > 1 / 8 + 1e-6) & (ratio < 1 - 1e-6)).any()


def test_window_hides_old_keys():
    rng = np.random.default_rng(0)
    D, H, hd, T = 16, 2, 8, 12
    x = rng.normal(size=(T, D))
    w = [rng.normal(size=s) for s in ((H * hd, D), (H * hd, D), (H * hd, D), (D, H * hd))]
    inv = P.rope_inverse_frequencies(hd, 10000.0)
    a = P.attention(x, *w, H, H, hd, inv, "half", window=4)
    x2 = x.copy()
    x2[:3] += 5.0                                    # keys older than the window of the last rows
    b = P.attention(x2, *w, H, H, hd, inv, "half", window=4)
    np.testing.assert_allclose(a[7:], b[7:], rtol=1e-10)
    assert not np.allclose(a[:5], b[:5])


def test_top_p_keeps_while_mass_before_is_below_p():
    probs = np.array([0.5, 0.2, 0.2, 0.05, 0.05])
    assert P.top_p_keep(probs, 0.5).tolist() == [True, False, False, False, False]
    assert P.top_p_keep(probs, 0.51).tolist() == [True, True, False, False, False]      # ties: lower index first
    assert P.top_p_keep(probs, 0.75).tolist() == [True, True, True, False, False]
    assert P.top_p_keep(probs, 1.0).all()
    assert P.top_p_draw(probs, 0.75, 0.0) == 0 and P.top_p_draw(probs, 0.75, 0.99) == 2
    assert P.greedy(np.array([1.0, 3.0, 3.0])) == 1
