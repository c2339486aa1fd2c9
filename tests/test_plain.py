"""The plain implementation checked against itself: properties that its
formulas must have whatever the weights are."""
import numpy as np
import pytest

import plain_hunyuan as ph
import tiny_configs
from crane_b200.weights.random_init import write_model_folder


@pytest.fixture(scope="module")
def model_b(tmp_path_factory):
    d = tmp_path_factory.mktemp("plain_b")
    write_model_folder(str(d), tiny_configs.B, 1, "float32", std=0.08, norm_std=0.05)
    return ph.load_folder(str(d))


def test_inv_freq_formula():
    f = ph.rope_inv_freq(32, 1e6, 0.0)
    assert f.dtype == np.float32 and f.shape == (16,)
    assert f[0] == 1.0 and np.isclose(f[1], 1e6 ** (-2 / 32), rtol=1e-6)
    # alpha scales the base by alpha^(d/(d-2)) (modeling.rs:202-205)
    g = ph.rope_inv_freq(32, 1e6, 1000.0)
    base = 1e6 * 1000.0 ** (32 / 30)
    assert np.isclose(g[5], base ** (-10 / 32), rtol=1e-6)
    assert np.array_equal(ph.rope_inv_freq(32, 1e6, -1.0), f)


def test_rope_depends_on_relative_position_only():
    rng = np.random.default_rng(0)
    q, k = rng.normal(size=(1, 1, 32)), rng.normal(size=(1, 1, 32))
    f = ph.rope_inv_freq(32, 10000.0, 0.0)

    def dot(pq, pk):
        a = ph.apply_rope(q, ph.rope_angles(np.array([pq]), f))
        b = ph.apply_rope(k, ph.rope_angles(np.array([pk]), f))
        return float((a * b).sum())
    assert np.isclose(dot(7, 3), dot(107, 103), atol=1e-4)
    assert not np.isclose(dot(7, 3), dot(7, 4), atol=1e-3)
    # half-split convention: position 0 leaves x unchanged, pairs are (j, j + d/2)
    x = rng.normal(size=(1, 1, 32))
    assert np.allclose(ph.apply_rope(x, ph.rope_angles(np.array([0]), f)), x)
    y = ph.apply_rope(x, ph.rope_angles(np.array([5]), f))
    assert np.allclose(y[..., 3] ** 2 + y[..., 19] ** 2, x[..., 3] ** 2 + x[..., 19] ** 2)


def test_rope_of_a_head_of_two_elements_with_alpha():
    """d / (d - 2) divides by zero: the reference's float arithmetic gives an
    infinite exponent and a frequency of 1 (modeling.rs:203-208); the engine's
    position part and the plain function follow it, neither raises."""
    from crane_b200.config import PartSpec
    from crane_b200.parts import build_part
    assert ph.rope_inv_freq(2, 10000.0, 1000.0).tolist() == [1.0]
    assert ph.rope_inv_freq(2, 10000.0, 0.5).tolist() == [1.0]
    rope = build_part(PartSpec("position", "rope", {"head_dim": 2, "theta": 10000.0, "alpha": 1000.0,
                                                    "max_positions": 16}))
    assert rope.inv_freq().tolist() == [1.0]
    for d in (4, 6, 128):
        rope = build_part(PartSpec("position", "rope", {"head_dim": d, "theta": 1e4, "alpha": 7.0, "max_positions": 16}))
        assert np.array_equal(rope.inv_freq(), ph.rope_inv_freq(d, 1e4, 7.0))


def test_rms_norm_formula():
    x = np.array([[3.0, 4.0]])
    w = np.array([2.0, 0.5])
    got = ph.rms_norm(x, w, 1e-5)
    rms = np.sqrt((9 + 16) / 2 + 1e-5)
    assert np.allclose(got, [[3 / rms * 2, 4 / rms * 0.5]])


def test_attention_is_causal_and_grouped():
    rng = np.random.default_rng(1)
    q, k, v = rng.normal(size=(6, 4, 8)), rng.normal(size=(6, 2, 8)), rng.normal(size=(6, 2, 8))
    full = ph.causal_attention(q, k, v)
    k2, v2 = k.copy(), v.copy()
    k2[4:], v2[4:] = 9.0, -9.0                       # later positions must not matter
    assert np.allclose(ph.causal_attention(q, k2, v2)[:4], full[:4])
    assert np.allclose(full[0].reshape(4, 8)[1], v[0, 0])      # heads 0,1 read kv head 0
    assert np.allclose(full[0].reshape(4, 8)[2], v[0, 1])      # heads 2,3 read kv head 1
    win = ph.causal_attention(q, k, v, window=2)
    assert np.allclose(win[:2], full[:2]) and not np.allclose(win[5], full[5])


def test_silu_and_swiglu():
    assert np.isclose(ph.silu(np.array(0.0)), 0.0) and np.isclose(ph.silu(np.array(2.0)), 2 / (1 + np.exp(-2)))
    h = np.array([[1.0, -1.0]])
    eye = np.eye(2)
    assert np.allclose(ph.swiglu(h, eye, 2 * eye, eye), ph.silu(h) * 2 * h)


def test_logits_at_a_position_ignore_later_tokens(model_b):
    cfg, w = model_b
    a = ph.logits_all(cfg, w, [5, 9, 200, 31, 7, 8])
    b = ph.logits_all(cfg, w, [5, 9, 200, 31])
    assert np.allclose(a[:4], b, atol=1e-10)
    assert a.shape == (6, 384) and np.abs(a).max() > 0.5


def test_greedy_generation_stops_on_eos(model_b):
    cfg, w = model_b
    out = ph.greedy_generate(cfg, w, [1, 2, 3], 6)
    assert len(out) == 9 and out[:3] == [1, 2, 3]
    eos = out[4]
    cut = ph.greedy_generate(cfg, w, [1, 2, 3], 6, eos=eos)
    assert cut == out[:out.index(eos, 3) + 1]


def test_sampling_helpers():
    l = np.array([2.0, -1.0, 0.5, 3.0])
    p = ph.apply_repetition_penalty(l, 2.0, [0, 1, 1, 9])
    assert np.allclose(p, [1.0, -2.0, 0.5, 3.0])
    u = ph.uniform_noise(1024, 3, 50)
    assert u.min() >= 1e-7 and u.max() < 0.999 and len(set(u.tolist())) > 40
    assert np.array_equal(u, ph.uniform_noise(1024, 3, 50))
    assert not np.array_equal(u, ph.uniform_noise(1024, 4, 50))
    logits = np.log(np.array([0.5, 0.3, 0.15, 0.05]))
    assert list(ph.top_k_top_p_keep(logits, 1.0, 2, 1.0)) == [0, 1]
    assert list(ph.top_k_top_p_keep(logits, 1.0, 0, 0.6)) == [0, 1]     # 0.5 <= 0.6, and the one after
    assert list(ph.top_k_top_p_keep(logits, 1.0, 0, 0.4)) == [0]        # the first always stays
    assert list(ph.top_k_top_p_keep(logits, 1.0, 3, 0.85)) == [0, 1, 2]
