"""The plain implementation itself (CPU): properties its formulas must have."""
import numpy as np

import plain_qwen3 as P
from helpers import TINY, random_tokens


def small_weights(cfg, seed=0):
    rng = np.random.default_rng(seed)
    e, h, hk, d, i, v = (cfg[k] for k in ("hidden_size", "num_attention_heads", "num_key_value_heads", "head_dim",
                                           "intermediate_size", "vocab_size"))
    w = {"model.embed_tokens.weight": rng.normal(0, 0.02, (v, e)), "model.norm.weight": 1 + rng.normal(0, 0.05, e)}
    if not cfg["tie_word_embeddings"]:
        w["lm_head.weight"] = rng.normal(0, 0.02, (v, e))
    for l in range(cfg["num_hidden_layers"]):
        p = "model.layers.%d." % l
        for n, shape in (("q_proj", (h * d, e)), ("k_proj", (hk * d, e)), ("v_proj", (hk * d, e)), ("o_proj", (e, h * d))):
            w[p + "self_attn." + n + ".weight"] = rng.normal(0, 0.02, shape)
            if cfg["attention_bias"]:
                w[p + "self_attn." + n + ".bias"] = rng.normal(0, 0.02, shape[0])
        w[p + "self_attn.q_norm.weight"] = 1 + rng.normal(0, 0.05, d)
        w[p + "self_attn.k_norm.weight"] = 1 + rng.normal(0, 0.05, d)
        w[p + "input_layernorm.weight"] = 1 + rng.normal(0, 0.05, e)
        w[p + "post_attention_layernorm.weight"] = 1 + rng.normal(0, 0.05, e)
        w[p + "mlp.gate_proj.weight"] = rng.normal(0, 0.02, (i, e))
        w[p + "mlp.up_proj.weight"] = rng.normal(0, 0.02, (i, e))
        w[p + "mlp.down_proj.weight"] = rng.normal(0, 0.02, (e, i))
    return w


def test_rms_norm():
    x = np.random.default_rng(0).normal(size=(3, 8))
    y = P.rms_norm(x, np.ones(8), 0.0)
    assert np.allclose((y * y).mean(-1), 1.0)
    assert np.allclose(P.rms_norm(x, 2 * np.ones(8), 1e-6), 2 * P.rms_norm(x, np.ones(8), 1e-6))


def test_rope_keeps_norms_and_depends_on_relative_position():
    rng = np.random.default_rng(1)
    q, k = rng.normal(size=(1, 1, 16)), rng.normal(size=(1, 1, 16))
    for theta in (1e4, 1e6):
        a = (P.rope(q, [7], theta) * P.rope(k, [3], theta)).sum()
        b = (P.rope(q, [107], theta) * P.rope(k, [103], theta)).sum()
        assert abs(a - b) < 1e-4  # angles are float32 products, so not exact
        assert np.allclose(np.linalg.norm(P.rope(q, [55], theta)), np.linalg.norm(q))
    assert np.allclose(P.rope(q, [0], 1e4), q)
    # half-split pairs (d, d + D/2): the first pair turns by the full position angle
    x = np.zeros((1, 1, 16)); x[0, 0, 0] = 1.0
    y = P.rope(x, [1], 1e4)
    assert np.allclose(y[0, 0, 0], np.cos(1.0), atol=1e-6) and np.allclose(y[0, 0, 8], np.sin(1.0), atol=1e-6)


def test_attention_is_causal_grouped_and_windowed():
    rng = np.random.default_rng(2)
    q, k, v = rng.normal(size=(9, 4, 8)), rng.normal(size=(9, 2, 8)), rng.normal(size=(9, 2, 8))
    full = P.causal_attention(q, k, v)
    k2, v2 = k.copy(), v.copy()
    k2[6:], v2[6:] = 0, 0
    assert np.allclose(P.causal_attention(q, k2, v2)[:6], full[:6])  # later keys do not matter
    assert np.allclose(full[0], v[0][[0, 0, 1, 1]])  # first token sees itself only; heads 0,1 -> kv 0; 2,3 -> kv 1
    assert np.allclose(P.causal_attention(q, k, v, window=9), full)
    w3 = P.causal_attention(q, k, v, window=3)
    assert np.allclose(w3[:3], full[:3]) and not np.allclose(w3[5], full[5])
    k3, v3 = k.copy(), v.copy()
    k3[:6], v3[:6] = 99, 99
    assert np.allclose(P.causal_attention(q, k3, v3, window=3)[8], w3[8])  # query 8 sees keys 6, 7, 8 only


def test_prefix_logits_do_not_depend_on_what_follows():
    for name in TINY:
        cfg = dict(TINY[name]["config"])
        w = small_weights(cfg)
        ids = random_tokens(cfg["vocab_size"], 30, 3)
        whole = P.forward_logits(cfg, w, ids)
        part = P.forward_logits(cfg, w, ids[:17])
        assert np.allclose(whole[:17], part, atol=1e-12)
        assert whole.shape == (30, cfg["vocab_size"])


def test_window_layers_follow_the_configuration():
    cfg = dict(TINY["tiny_b"]["config"])
    assert [P.layer_window(cfg, i) for i in range(3)] == [0, 20, 20]
    w = small_weights(cfg)
    ids = random_tokens(cfg["vocab_size"], 40, 4)
    windowed = P.forward_logits(cfg, w, ids)
    free = P.forward_logits(dict(cfg, use_sliding_window=False), w, ids)
    assert np.allclose(windowed[:20], free[:20], atol=1e-12) and not np.allclose(windowed[30:], free[30:], atol=1e-9)


def test_sampling():
    logits = np.array([0.1, 2.0, 2.0, -1.0, 1.5])
    assert P.greedy(logits) == 1  # first maximum
    p = P.probabilities(logits, 0.8)
    assert abs(p.sum() - 1) < 1e-12 and p[1] == p[2] > p[4]
    n = P.probabilities(logits, 1.0, top_p=0.5)  # the two tied tokens cross 0.5 together
    assert (n > 0).tolist() == [False, True, True, False, False] and abs(n.sum() - 1) < 1e-12
    assert P.sample_from(p, 0.0) == 0 and P.sample_from(p, 0.999999) == 4
    c = np.cumsum(p)
    assert P.sample_from(p, float(c[1] - 1e-9)) == 1 and P.sample_from(p, float(c[1] + 1e-9)) == 2


def test_store_bfloat16_rounds_to_nearest_even():
    import torch
    x = np.random.default_rng(5).standard_normal(4096).astype(np.float32) * 3
    x[:4] = [1.0, 1.00390625, 1.01171875, -0.0]   # exact; a tie that goes down to even; a tie that goes up
    want = torch.from_numpy(x).to(torch.bfloat16).to(torch.float32).numpy()
    assert (P.store_bfloat16(x) == want).all()
    assert P.store_bfloat16(x.astype(np.float64)).dtype == np.float64
