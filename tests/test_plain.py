"""The plain implementation against hand-checkable anchors lifted from the reference's own
unit tests, and against itself (no GPU)."""
import math

import numpy as np
import pytest

import plain_llama as P
from conftest import TINY_A, TINY_B


def test_rms_norm_anchor():
    """crates/kernels/src/tests.rs:170-176."""
    out = P.rms_norm(np.array([[3.0, 4.0]]), np.array([2.0, 0.5]), 0.0)
    inv = 1 / math.sqrt(12.5)
    assert np.allclose(out, [[6 * inv, 2 * inv]])


def test_softmax_anchors():
    """crates/kernels/src/tests.rs:178-193."""
    e = np.exp([1.0, 2.0, 3.0])
    assert np.allclose(P.softmax(np.array([1.0, 2.0, 3.0])), e / e.sum())
    assert np.allclose(P.softmax(np.array([5.0])), [1.0])


def test_silu_anchor():
    """crates/kernels/src/tests.rs:142-168: v / (1 + exp(-v))."""
    for v in (-3.0, 0.0, 0.5, 4.0):
        assert P.silu(np.array(v)) == pytest.approx(v / (1 + math.exp(-v)))


def test_rope_anchors():
    """crates/kernels/src/tests.rs:197-238: position 0 is the identity, pairs are (0,1),(2,3),
    and a tail beyond the rotated dimensions is untouched."""
    x = np.arange(1.0, 9.0).reshape(1, 1, 8)
    inv = np.array([1.0, 0.1])
    assert np.array_equal(P.rope(x[..., :4], np.array([0]), inv, "adjacent"), x[..., :4])
    y = P.rope(x[..., :4], np.array([3]), inv, "adjacent")[0, 0]
    c, s = math.cos(3.0), math.sin(3.0)
    assert np.allclose(y[:2], [1 * c - 2 * s, 1 * s + 2 * c])
    c, s = math.cos(0.3), math.sin(0.3)
    assert np.allclose(y[2:], [3 * c - 4 * s, 3 * s + 4 * c])
    z = P.rope(x[..., :4], np.array([3]), inv, "half")[0, 0]          # pairs (0,2),(1,3)
    c, s = math.cos(3.0), math.sin(3.0)
    assert np.allclose([z[0], z[2]], [1 * c - 3 * s, 1 * s + 3 * c])


def test_the_two_pairings_agree_after_permuting_rows():
    """A checkpoint with HF-ordered q/k rows under "half" equals the same checkpoint with rows
    permuted to the GGUF order under "adjacent": scores only see q.k."""
    rng = np.random.default_rng(0)
    T, H, D = 6, 2, 8
    q, k = rng.normal(size=(T, H, D)), rng.normal(size=(T, H, D))
    inv = P.rope_inv_freq({"head_dim": D, "hidden_size": 16, "num_attention_heads": 2, "rope_theta": 100.0})
    pos = np.arange(T)
    perm = np.array([i // 2 + (i % 2) * (D // 2) for i in range(D)])    # new[2i] = old[i], new[2i+1] = old[i + D/2]
    s1 = np.einsum("thd,shd->hts", P.rope(q, pos, inv, "half"), P.rope(k, pos, inv, "half"))
    s2 = np.einsum("thd,shd->hts", P.rope(q[..., perm], pos, inv, "adjacent"), P.rope(k[..., perm], pos, inv, "adjacent"))
    assert np.allclose(s1, s2)


def test_llama3_scaling_takes_all_three_branches():
    """theta 5e5, R 32, original 64, factors (8, 1, 4): pairs 0-1 unchanged, pair 2 blended,
    pairs >= 3 divided by the factor."""
    f = P.rope_inv_freq(TINY_B)
    base = 500000.0 ** (-2.0 * np.arange(16) / 32)
    assert np.allclose(f[:2], base[:2])
    assert base[2] / 8 < f[2] < base[2]
    assert np.allclose(f[3:], base[3:] / 8)


def test_llama3_scaling_against_numbers_worked_by_hand():
    """The blended branch, worked on paper (40-digit decimal arithmetic, independent of both
    implementations).  Rule: f = theta^(-2i/R); wavelength = 2 pi / f; between original/high and
    original/low, s = (original / wavelength - low) / (high - low) and f' = ((1 - s) / factor + s) f.

    Second tiny configuration (theta 5e5, R 32, original 64, factor 8, low 1, high 4), pair 2:
      f = 5e5^(-4/32) = 0.19392274474868577...; wavelength = 32.400455734691059... (between 16 and 64)
      s = (64 / 32.4004557... - 1) / 3 = 0.32509361930029289...
      f' = ((1 - s) / 8 + s) f = 0.079403009179208206...
    Pair 1 (wavelength 14.268 < 16) keeps f = 0.44036660267178047...; pair 3 (73.576 > 64) gives f / 8 =
    0.08539710028576561... / 8 = 0.010674637535720701...
    Fourth tiny configuration (theta 1e5, R 64, original 32, factor 4, low 1, high 2), pair 3:
      f = 1e5^(-6/64) = 0.33982083289425593...; wavelength = 18.489700156596233... (between 16 and 32)
      s = (32 / 18.4897001... - 1) / 1 = 0.73069329026322490...
      f' = ((1 - s) / 4 + s) f = 0.27118381008918403...
    and pair 4: f = 0.23713737056616552..., s = 0.20773071095743265..., f' = 0.096229878578255677...
    The product's table is checked against the same numbers."""
    from conftest import TINY_D
    from ferrum_b200.config import LlamaConfig
    from ferrum_b200.parts.rope import inverse_frequencies
    want_b = {1: 0.4403666026717804735919833, 2: 0.07940300917920820642694930, 3: 0.08539710028576561128014966 / 8}
    want_d = {2: 0.4869675251658631149352974, 3: 0.2711838100891840334453061, 4: 0.09622987857825567756248523,
              5: 0.1654817099943181422945613 / 4}
    for cfg, want in ((TINY_B, want_b), (TINY_D, want_d)):
        plain = P.rope_inv_freq(cfg)
        c = LlamaConfig.from_dict(cfg)
        product = inverse_frequencies(c.rope_dim, c.rope_freq_base, c.rope_scaling)
        for i, v in want.items():
            assert plain[i] == pytest.approx(v, rel=1e-12), (i, plain[i], v)
            assert product[i] == pytest.approx(v, rel=1e-12), (i, product[i], v)


def test_argmax_anchor():
    """crates/core-types/src/model.rs:304-309."""
    assert P.argmax([1.0, 3.0, 3.0, float("nan")]) == 1
    with pytest.raises(ValueError):
        P.argmax([float("nan")])


def test_gqa_attention_is_causal_and_groups_heads():
    rng = np.random.default_rng(1)
    T, Hq, Hkv, D = 5, 4, 2, 4
    q, k, v = rng.normal(size=(T, Hq, D)), rng.normal(size=(T, Hkv, D)), rng.normal(size=(T, Hkv, D))
    o = P.attention(q, k, v)
    assert np.allclose(o[0, :, :], v[0, [0, 0, 1, 1], :])                 # the first token sees itself only
    k2, v2 = k.copy(), v.copy()
    k2[3:], v2[3:] = 9.0, -9.0                                              # the future does not matter
    assert np.allclose(P.attention(q, k2, v2)[:3], o[:3])
    w = P.attention(q, k, v, window=2)
    s = (q[4, 0] @ k[3:5, 0].T) / 2.0
    p = np.exp(s - s.max()); p /= p.sum()
    assert np.allclose(w[4, 0], p @ v[3:5, 0])


def test_reference_mock_model_shape(tmp_path):
    """The reference's MockModel (crates/model/src/tests.rs:36-128): 1 layer, width 4, 2 heads,
    1 KV head, F 8, vocab 4, every weight 0.01: logits are finite and equal for every token."""
    cfg = {"hidden_size": 4, "num_hidden_layers": 1, "num_attention_heads": 2, "num_key_value_heads": 1,
           "intermediate_size": 8, "vocab_size": 4, "rms_norm_eps": 1e-5, "rope_theta": 10000.0}
    names = ["model.embed_tokens.weight", "model.norm.weight", "model.layers.0.input_layernorm.weight",
             "model.layers.0.post_attention_layernorm.weight"]
    w = {"model.embed_tokens.weight": np.full((4, 4), 0.01), "model.norm.weight": np.full(4, 0.01),
         "model.layers.0.input_layernorm.weight": np.full(4, 0.01),
         "model.layers.0.post_attention_layernorm.weight": np.full(4, 0.01),
         "model.layers.0.self_attn.q_proj.weight": np.full((4, 4), 0.01),
         "model.layers.0.self_attn.k_proj.weight": np.full((2, 4), 0.01),
         "model.layers.0.self_attn.v_proj.weight": np.full((2, 4), 0.01),
         "model.layers.0.self_attn.o_proj.weight": np.full((4, 4), 0.01),
         "model.layers.0.mlp.gate_proj.weight": np.full((8, 4), 0.01),
         "model.layers.0.mlp.up_proj.weight": np.full((8, 4), 0.01),
         "model.layers.0.mlp.down_proj.weight": np.full((4, 8), 0.01)}
    logits = P.forward(cfg, w, [0, 1])
    assert logits.shape == (2, 4) and np.isfinite(logits).all()
    assert np.allclose(logits, logits[0, 0])


def test_sampling_is_a_pure_function_of_seed_and_counter():
    row = np.linspace(-2, 2, 50)
    a = [P.sample(row, 0.8, 1, n) for n in range(20)]
    assert a == [P.sample(row, 0.8, 1, n) for n in range(20)]
    assert a != [P.sample(row, 0.8, 2, n) for n in range(20)]
    assert len(set(a)) > 3
    u = P.gumbel_uniform(3, 4, 1000)
    assert (u > 0).all() and (u < 1).all() and abs(u.mean() - 0.5) < 0.05
    assert P.sample(row, 0.0, 1, 0) == 49
