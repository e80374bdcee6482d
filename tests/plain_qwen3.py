"""Plain, slow Qwen3 decoder in numpy: the oracle of the test-suite.

Whole sequences, no cache, no pages, one function for each part.  It shares no
code with the product path (`velox_b200/`): it reads `config.json` with `json`
and `model.safetensors` with the `safetensors` package, and every formula is
restated here from the reference's own files (cited as file:line inside the
reference project).

The reference (a Rust project whose tensor operations come from crates that
are not in its tree) cannot be compiled or imported in this environment: there
is no Rust toolchain and its dependencies are not vendored.  This
implementation therefore rests on the reference's formulas, not on outputs of
the reference's code.

All arithmetic is float64 unless `dtype=np.float32` is asked for; weights are
whatever the file holds, widened exactly.
"""
from __future__ import annotations

import json
import math
import os

import numpy as np


# ----------------------------------------------------------------------------
# files
# ----------------------------------------------------------------------------
def load_model_folder(folder, dtype="float64"):
    """(config dict, {name: float64 array}) of a folder with config.json and
    model.safetensors.  bfloat16 is widened exactly through its bit pattern.
    `dtype="float32"` holds the arrays in 32-bit, for models of many gigabytes."""
    from safetensors import safe_open

    with open(os.path.join(folder, "config.json")) as f:
        config = json.load(f)
    weights = {}
    import torch  # only as the container that safetensors hands bfloat16 in

    with safe_open(os.path.join(folder, "model.safetensors"), framework="pt") as f:
        for name in f.keys():
            weights[name] = f.get_tensor(name).to(getattr(torch, dtype)).numpy()
    return config, weights


# ----------------------------------------------------------------------------
# parts (one function each)
# ----------------------------------------------------------------------------
def embedding(ids, table):
    """x[t,:] = embed_tokens.weight[ids[t],:]  (src/paged/qwen3.rs:958, 998)."""
    return table[np.asarray(ids, dtype=np.int64)]


def rms_norm(x, weight, eps):
    """h = x * rsqrt(mean(x^2) + eps) * w over the last axis; the weight
    multiplies, without a +1 offset (src/paged/qwen3.rs:923, 933: the call of
    the library's rms_norm with `rms_norm_eps`)."""
    var = np.mean(x * x, axis=-1, keepdims=True)
    return x / np.sqrt(var + eps) * weight


def linear(x, weight, bias=None):
    """y = x W^T (+ b), weight stored [out, in] (src/paged/qwen3.rs:120-132,
    226-239)."""
    y = x @ weight.T
    if bias is not None:
        y = y + bias
    return y


def rope_inverse_frequencies(head_dim, theta):
    """inv_freq[i] = 1 / theta^(2i/D), the power in float64, the result rounded
    to float32 (src/paged/qwen3.rs:281-284)."""
    return np.array(
        [np.float32(1.0) / np.float32(theta ** (i / head_dim)) for i in range(0, head_dim, 2)],
        dtype=np.float32,
    )


def rope(x, positions, theta):
    """Half-split rotation of x [T, heads, D] at absolute positions [T]
    (src/paged/metal_kernels.rs:199-202, 230-236; the test reference at
    tests/metal_batched_kernels_parity.rs:65-72): for d < D/2
        y[d]       = x[d] cos - x[d + D/2] sin
        y[d + D/2] = x[d] sin + x[d + D/2] cos
    with angle[p, i] = p * inv_freq[i] formed in float32
    (src/paged/qwen3.rs:287-290)."""
    d = x.shape[-1]
    inv = rope_inverse_frequencies(d, theta)
    ang = (np.asarray(positions, dtype=np.float32)[:, None] * inv[None, :]).astype(np.float32)
    ang = ang.astype(np.float64)
    cos = np.cos(ang)[:, None, :]
    sin = np.sin(ang)[:, None, :]
    lo, hi = x[..., : d // 2], x[..., d // 2 :]
    return np.concatenate([lo * cos - hi * sin, lo * sin + hi * cos], axis=-1)


def causal_attention(q, k, v, window=0):
    """q [T,H,D], k,v [T,Hk,D] of ONE whole sequence starting at position 0.
    Query i sees keys j <= i (src/paged/metal_kernels.rs:333-336;
    src/paged/qwen3.rs:868-884), and with a window W only the W most recent of
    them, j >= i + 1 - W (src/paged/metal_kernels.rs:339-341).  q-head h reads
    kv-head h // (H/Hk) (src/paged/metal_kernels.rs:130-131).  Scores are scaled
    by 1/sqrt(D) (src/paged/qwen3.rs:488); softmax over the visible keys, then
    the weighted sum of V (src/paged/metal_kernels.rs:171-185)."""
    t, h, d = q.shape
    hk = k.shape[1]
    group = h // hk
    scale = 1.0 / math.sqrt(d)
    out = np.zeros_like(q)
    idx = np.arange(t)
    visible = idx[None, :] <= idx[:, None]
    if window and window > 0:
        visible &= idx[None, :] >= (idx[:, None] + 1 - window)
    for head in range(h):
        kh = head // group
        s = (q[:, head, :] @ k[:, kh, :].T) * scale
        s = np.where(visible, s, -np.inf)
        s = s - s.max(axis=-1, keepdims=True)
        p = np.exp(s)
        p = p / p.sum(axis=-1, keepdims=True)
        out[:, head, :] = p @ v[:, kh, :]
    return out


def silu(z):
    """silu(z) = z / (1 + exp(-z)): `hidden_act` of Qwen3
    (src/paged/qwen3.rs:50, 317)."""
    return z / (1.0 + np.exp(-z))


def keep(x):
    """Activations held as computed (the default `store`)."""
    return x


def store_bfloat16(x):
    """x rounded to bfloat16 (nearest, ties to even) and widened again: what is
    left of an activation that a bfloat16 model holds between two operations,
    as the reference does with its bfloat16 weights and activations
    (src/paged/qwen3.rs:226-239: the matmul's output takes the input's dtype)."""
    b = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    b = (b + np.uint32(0x7FFF) + ((b >> np.uint32(16)) & np.uint32(1))) & np.uint32(0xFFFF0000)
    return b.view(np.float32).astype(np.asarray(x).dtype)


def gated_mlp(x, w_gate, w_up, w_down, store=keep):
    """down(act(gate(x)) * up(x)), never biased (src/paged/qwen3.rs:324-326,
    333-339)."""
    return store(linear(store(silu(linear(x, w_gate)) * linear(x, w_up)), w_down))


def attention_block(x, positions, w, prefix, cfg, window, store=keep):
    """q/k/v projections, per-head RMSNorm of q and k before the rotation, the
    rotation, attention, output projection (src/paged/qwen3.rs:428-448,
    506-544).  The output projection's input width is H*D, not the hidden size
    (src/paged/qwen3.rs:390, 395)."""
    t = x.shape[0]
    h, hk, d = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    eps = cfg["rms_norm_eps"]
    bias = (lambda n: w[prefix + n + ".bias"]) if cfg["attention_bias"] else (lambda n: None)
    q = store(linear(x, w[prefix + "q_proj.weight"], bias("q_proj"))).reshape(t, h, d)
    k = store(linear(x, w[prefix + "k_proj.weight"], bias("k_proj"))).reshape(t, hk, d)
    v = store(linear(x, w[prefix + "v_proj.weight"], bias("v_proj"))).reshape(t, hk, d)
    q = rms_norm(q, w[prefix + "q_norm.weight"], eps)
    k = rms_norm(k, w[prefix + "k_norm.weight"], eps)
    q = store(rope(q, positions, cfg["rope_theta"]))
    k = store(rope(k, positions, cfg["rope_theta"]))
    a = store(causal_attention(q, k, v, window)).reshape(t, h * d)
    return store(linear(a, w[prefix + "o_proj.weight"], bias("o_proj")))


def layer_window(cfg, layer):
    """The window of a layer, 0 for none.  The reference applies
    `sliding_window` to every layer when `use_sliding_window` is set
    (src/paged/qwen3.rs:373-381) and reads `max_window_layers` without using it
    (src/paged/qwen3.rs:43-44; default 0).  Here the first `max_window_layers`
    layers attend to everything and the later ones use the window, which is the
    reference's behaviour at its default of 0."""
    if not cfg.get("use_sliding_window", False):
        return 0
    w = cfg.get("sliding_window") or 0
    return w if layer >= cfg.get("max_window_layers", 0) else 0


def decoder_layer(x, positions, w, layer, cfg, store=keep):
    """Pre-norm residual block (src/paged/qwen3.rs:932-939).  `store` is applied
    to what a model would hold between operations; the residual sum is not."""
    p = "model.layers.%d." % layer
    eps = cfg["rms_norm_eps"]
    h = store(rms_norm(x, w[p + "input_layernorm.weight"], eps))
    x = x + attention_block(h, positions, w, p + "self_attn.", cfg, layer_window(cfg, layer), store)
    h = store(rms_norm(x, w[p + "post_attention_layernorm.weight"], eps))
    x = x + gated_mlp(
        h, w[p + "mlp.gate_proj.weight"], w[p + "mlp.up_proj.weight"], w[p + "mlp.down_proj.weight"], store
    )
    return x


def forward_logits(cfg, w, ids, dtype=np.float64, store=keep, rows=None):
    """Logits [T, V] at every position of one whole sequence (at `rows` only,
    if given) (src/paged/qwen3.rs:1019-1036: embed, the layers, final norm,
    output head; the head is the embedding table when `tie_word_embeddings`,
    :966-976).  With `store=store_bfloat16` every activation between two
    operations is rounded to bfloat16, the residual sum and the logits are not:
    the distance of that result from the exact one is what bfloat16 costs."""
    w = {k: v.astype(dtype, copy=False) for k, v in w.items()}
    positions = np.arange(len(ids))
    x = embedding(ids, w["model.embed_tokens.weight"])
    for layer in range(cfg["num_hidden_layers"]):
        x = decoder_layer(x, positions, w, layer, cfg, store)
    if rows is not None:
        x = x[np.asarray(rows, dtype=np.int64)]
    x = store(rms_norm(x, w["model.norm.weight"], cfg["rms_norm_eps"]))
    head = w["model.embed_tokens.weight"] if cfg["tie_word_embeddings"] else w["lm_head.weight"]
    return linear(x, head)


# ----------------------------------------------------------------------------
# sampling
# ----------------------------------------------------------------------------
def greedy(logits_row):
    """argmax, the first maximum winning (src/paged/spec.rs:356-365 keeps the
    first with a strict `>`)."""
    return int(np.argmax(logits_row))


def probabilities(logits_row, temperature, top_p=1.0):
    """softmax(logits / T); with 0 < top_p < 1 only the most probable tokens
    whose mass reaches top_p stay (the one that crosses it included, ties of
    the last one included), renormalised (src/paged/scheduler.rs:545-553: All
    when top_p <= 0 or >= 1, else TopP)."""
    z = np.asarray(logits_row, dtype=np.float64) / temperature
    z = z - z.max()
    p = np.exp(z)
    p = p / p.sum()
    if 0.0 < top_p < 1.0:
        order = np.argsort(-p, kind="stable")
        csum = np.cumsum(p[order])
        last = int(np.searchsorted(csum, top_p, side="left"))
        last = min(last, len(p) - 1)
        threshold = p[order[last]]
        p = np.where(p >= threshold, p, 0.0)
        p = p / p.sum()
    return p


def sample_from(p, u):
    """First index whose cumulative probability (in index order) exceeds u."""
    c = np.cumsum(p)
    return int(min(np.searchsorted(c, u * c[-1], side="right"), len(p) - 1))


def greedy_generate(cfg, w, prompt, new_tokens, dtype=np.float64):
    """Greedy continuation by recomputing the whole sequence for every token."""
    ids = list(prompt)
    for _ in range(new_tokens):
        ids.append(greedy(forward_logits(cfg, w, ids, dtype)[-1]))
    return ids[len(prompt):]
