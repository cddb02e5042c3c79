"""The plain implementation against the reference's own unit facts and against properties
every decoder of this architecture has (no GPU)."""
import numpy as np
import pytest
import torch

import helpers
import plain_qwen3 as P


def test_rms_norm_fact_of_the_reference():
    # src/engine/ops.zig:227-234: [2,-2,2,-2] with unit weight and eps 0 -> [1,-1,1,-1]
    out = P.rms_norm(np.array([[2.0, -2.0, 2.0, -2.0]]), np.ones(4), 0.0)
    assert np.allclose(out, [[1, -1, 1, -1]], atol=1e-12)


def test_rotate_half_fact_of_the_reference():
    # src/engine/ops.zig:236-252: 90 degrees, neox pairs (x0,x2),(x1,x3): [1,0,0,1] -> [0,-1,1,0]
    x = np.array([[1.0, 0.0, 0.0, 1.0]])
    out = P.rope_rotate_half(x, 4, np.zeros((1, 2)), np.ones((1, 2)))
    assert np.allclose(out, [[0, -1, 1, 0]], atol=1e-12)


def test_inv_freq_facts_of_the_reference():
    # src/engine/ops.zig:326-329: theta 1e4, 64 dims: inv_freq[0] = 1, inv_freq[31] = 4 * 3.333803761e-05
    f = P.rope_inv_freq(10000.0, 64)
    assert f.dtype == np.float32 and f[0] == 1.0
    assert abs(f[31] / (4.0 * 3.333803761e-05) - 1) < 1e-5


# Numbers the reference's own tests carry, exported from Transformers (src/engine/ops.zig:303-329): (index, inv_freq)
LLAMA3 = [(0, 1.0), (1, 6.636012793e-01), (7, 5.666961893e-02), (8, 3.760603070e-02), (12, 7.292665076e-03),
          (16, 5.248460220e-04), (20, 3.428102355e-05), (24, 6.647869668e-06), (31, 3.767322596e-07)]
YARN = [(0, 1.0), (1, 7.498942018e-01), (7, 1.333521456e-01), (8, 1.000000015e-01), (12, 2.797399648e-02),
        (16, 6.538461894e-03), (20, 1.337886788e-03), (24, 2.500000119e-04), (31, 3.333803761e-05)]
LINEAR = [(0, 0.25), (1, 1.874735504e-01), (16, 2.499999944e-03), (31, 3.333803761e-05)]


def test_rope_scaling_numbers_of_the_reference():
    """Plain restatement and the engine's rotary part against the values the reference pins (relative 2e-6, as there)."""
    from hk_b200.parts import RopeScaling, RotaryEmbedding
    cases = [
        (LLAMA3, 500000.0, dict(kind="llama3", factor=8.0, orig_ctx=8192, low_freq_factor=1.0, high_freq_factor=4.0)),
        (YARN, 10000.0, dict(kind="yarn", factor=4.0, orig_ctx=4096)),
        (LINEAR, 10000.0, dict(kind="linear", factor=4.0)),
    ]
    for probes, theta, kw in cases:
        plain = P.rope_inv_freq_scaled(theta, 64, **kw)
        part = RotaryEmbedding(theta, 64, 8, scaling=RopeScaling(**kw)).inv_freq().numpy()
        for i, want in probes:
            assert abs(plain[i] / want - 1) < 2e-6, (kw["kind"], i)
            assert abs(part[i] / want - 1) < 2e-6, (kw["kind"], i)
        assert np.array_equal(plain, part)
    # magnitude: only yarn changes it (src/engine/ops.zig:318-319)
    assert abs(P.rope_mscale("yarn", 4.0) / 1.138629436 - 1) < 1e-6
    assert abs(RotaryEmbedding(10000.0, 64, 8, scaling=RopeScaling("yarn", 4.0, 4096)).mscale() / 1.138629436 - 1) < 1e-6
    assert P.rope_mscale("llama3", 8.0) == 1.0 and RotaryEmbedding(5e5, 64, 8, scaling=RopeScaling("llama3", 8.0, 8192)).mscale() == 1.0
    assert np.array_equal(P.rope_inv_freq_scaled(1e4, 64, "none"), P.rope_inv_freq(1e4, 64))


def test_adjacent_rotation_fact_of_the_reference():
    # src/engine/ops.zig:236-252 with style .norm: pairs (x0,x1),(x2,x3) by 90 degrees: [1,0,0,1] -> [0,1,-1,0]
    out = P.rope_rotate_adjacent(np.array([[1.0, 0.0, 0.0, 1.0]]), 4, np.zeros((1, 2)), np.ones((1, 2)))
    assert np.allclose(out, [[0, 1, -1, 0]], atol=1e-12)


def test_head_norm_shares_one_weight_across_heads():
    rng = np.random.default_rng(0)
    x = rng.standard_normal((3, 8))
    w = rng.standard_normal(4)
    out = P.head_norm(x, w, 4, 1e-6)
    assert np.allclose(out[:, :4], P.rms_norm(x[:, :4], w, 1e-6))
    assert np.allclose(out[:, 4:], P.rms_norm(x[:, 4:], w, 1e-6))


def test_attention_is_causal_grouped_and_scaled():
    rng = np.random.default_rng(1)
    t, H, G, hd = 6, 4, 2, 8
    q, k, v = rng.standard_normal((t, H * hd)), rng.standard_normal((t, G * hd)), rng.standard_normal((t, G * hd))
    out = P.causal_gqa_attention(q, k, v, H, G, hd)
    # the first token sees only itself
    assert np.allclose(out[0].reshape(H, hd), v[0].reshape(G, hd)[[0, 0, 1, 1]])
    # by hand for one (token, head): consecutive q heads share a kv head (h // (H/G))
    h, p = 3, 4
    s = (q[p].reshape(H, hd)[h] / np.sqrt(hd)) @ k[:p + 1].reshape(p + 1, G, hd)[:, 1].T
    w = np.exp(s - s.max())
    w /= w.sum()
    assert np.allclose(out[p].reshape(H, hd)[h], w @ v[:p + 1].reshape(p + 1, G, hd)[:, 1])
    # changing a later token changes nothing earlier
    k2, v2 = k.copy(), v.copy()
    k2[5] += 1
    v2[5] -= 1
    out2 = P.causal_gqa_attention(q, k2, v2, H, G, hd)
    assert np.array_equal(out[:5], out2[:5]) and not np.allclose(out[5], out2[5])


def test_window_limits_the_keys():
    rng = np.random.default_rng(2)
    t, H, G, hd = 9, 2, 1, 4
    q, k, v = rng.standard_normal((t, H * hd)), rng.standard_normal((t, hd)), rng.standard_normal((t, hd))
    out = P.causal_gqa_attention(q, k, v, H, G, hd, window=3)
    full = P.causal_gqa_attention(q, k, v, H, G, hd)
    assert np.allclose(out[:3], full[:3]) and not np.allclose(out[3], full[3])
    # position 8 with window 3 reads exactly keys 6, 7, 8
    alone = P.causal_gqa_attention(q[6:], k[6:], v[6:], H, G, hd)
    assert np.allclose(out[8], alone[2])


def test_swiglu_and_linear():
    g, u = np.array([[0.0, 1.0, -2.0]]), np.array([[3.0, 2.0, 1.0]])
    assert np.allclose(P.swiglu(g, u), [[0.0, 2.0 / (1 + np.exp(-1.0)), -2.0 / (1 + np.exp(2.0))]])
    assert np.allclose(P.linear(np.array([[1.0, 2.0]]), np.array([[1.0, 0.0], [0.5, 0.5], [0.0, -1.0]])), [[1.0, 1.5, -2.0]])


@pytest.mark.parametrize("which", ["A", "B", "C"])
def test_forward_is_causal_and_prefix_stable(tmp_path, which):
    d = helpers.make_model_dir(tmp_path, which, torch.float32)
    cfg, w = helpers.load_plain(d)
    rng = np.random.default_rng(3)
    ids = rng.integers(0, cfg["vocab_size"], 40).tolist()
    full = P.forward(cfg, w, ids)
    assert full.shape == (40, cfg["vocab_size"]) and np.isfinite(full).all()
    part = P.forward(cfg, w, ids[:23])
    assert np.allclose(full[:23], part, atol=1e-12)
    f32 = P.forward(cfg, w, ids, dtype=np.float32)
    assert np.abs(f32 - full).max() < 2e-5 * np.abs(full).max()


def test_tied_head_uses_the_embedding(tmp_path):
    d = helpers.make_model_dir(tmp_path, "A", torch.float32)
    cfg, w = helpers.load_plain(d)
    assert "lm_head.weight" not in w
    ids = [1, 2, 3]
    a = P.forward(cfg, w, ids)
    w2 = dict(w, **{"lm_head.weight": w["model.embed_tokens.weight"]})
    assert np.array_equal(a, P.forward(dict(cfg, tie_word_embeddings=False), w2, ids))
    with pytest.raises(KeyError):
        P.forward(dict(cfg, tie_word_embeddings=False), w, ids)


def test_sampling_chain_of_the_reference():
    # src/sampler.zig:220-299 restated: top-k 1 is argmax; top-p and min-p cut the tail
    logits = np.log(np.array([0.5, 0.3, 0.15, 0.05]))
    assert P.greedy(np.array([1.0, 3.0, 3.0, 2.0])) == 1           # first maximum wins
    ids, p = P.candidate_distribution(logits, 1.0, 1, 1.0)
    assert ids.tolist() == [0] and np.allclose(p, [1.0])
    ids, p = P.candidate_distribution(logits, 1.0, 0, 0.7)          # 0.5 + 0.3 reaches 0.7
    assert ids.tolist() == [0, 1] and np.allclose(p, [0.625, 0.375])
    ids, p = P.candidate_distribution(logits, 1.0, 0, 1.0, min_p=0.5)   # floor 0.25
    assert ids.tolist() == [0, 1]
    ids, p = P.candidate_distribution(logits, 0.5, 3, 1.0)          # temperature sharpens the survivors
    assert ids.tolist() == [0, 1, 2] and np.allclose(p, np.array([0.25, 0.09, 0.0225]) / 0.3625)
    ids, _ = P.candidate_distribution(np.array([0.0, 1.0, 1.0, -np.inf]), 1.0, 2, 1.0)
    assert ids.tolist() == [1, 2]                                    # ties by id, non-finite dropped
