"""Each part of a layer alone against its plain counterpart, at sizes that are
neither tiny configuration's."""
import math

import numpy as np
import pytest
import torch

import plain_qwen3 as P
from helpers import RoundingJudge

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda:0")
DTYPES = [torch.float32, torch.bfloat16]


def runtime(dtype):
    from velox_b200.parts import Runtime
    return Runtime(dtype, DEV)


def make(part, dtype, seed=0):
    """Random tensors for a part (rounded to bfloat16 so both precisions see the same numbers)."""
    from velox_b200.weights.loader import held_dtype
    from velox_b200.weights.random_init import random_tensor
    rt = runtime(dtype)
    host = {s.name: random_tensor(s, seed, torch.bfloat16) for s in part.tensor_specs()}
    part.bind({s.name: host[s.name].to(DEV, held_dtype(s.role, torch.bfloat16, rt)) for s in part.tensor_specs()}, rt)
    return {k: v.double().numpy() for k, v in host.items()}


def close(got, want, dtype, what="", rounded=None):
    """float32: 2e-5 + 1e-5 |x|.  bfloat16: `rounded` is the plain part with what it stores
    rounded to bfloat16; its distance from `want` is what rounding costs, and the engine's
    part is held to that (helpers.assert_close)."""
    got = got.detach().double().cpu().numpy()
    if dtype == torch.float32:
        err = np.abs(got - want)
        assert got.shape == want.shape and np.isfinite(got).all() and (err <= 2e-5 + 1e-5 * np.abs(want)).all(), \
            "%s: max err %.3g" % (what, err.max())
        return
    cost = np.sqrt(np.mean(np.square(rounded - want), axis=1))
    judge = RoundingJudge("part: " + what, np.sqrt(np.mean(cost * cost)))
    judge.check(got, want, cost, what)
    judge.finish()


def act(shape, dtype, seed):
    x = torch.randn(shape, generator=torch.Generator().manual_seed(seed)).to(dtype)
    return x.to(DEV), x.double().numpy()


@pytest.mark.parametrize("dtype", DTYPES)
def test_rms_norm_part(dtype):
    from velox_b200.parts import RMSNorm
    n = RMSNorm("x.", 72, 1e-5)
    w = make(n, dtype)
    res = torch.randn(5, 72, generator=torch.Generator().manual_seed(1)).to(DEV)
    delta, dn = act((5, 72), dtype, 2)
    total = res.double().cpu().numpy() + dn
    out = n.add_norm(res, delta)
    want = P.rms_norm(total, w["x.weight"], 1e-5)
    close(out, want, dtype, "add_norm", P.store_bfloat16(want))
    assert np.allclose(res.double().cpu().numpy(), total, atol=1e-6)
    x, xn = act((3, 72), dtype, 3)
    want = P.rms_norm(xn, w["x.weight"], 1e-5)
    close(n.forward(x), want, dtype, "norm", P.store_bfloat16(want))


def test_rotary_position_frequencies():
    from velox_b200.parts import RotaryPosition
    for d, theta in ((16, 1e4), (48, 1e6), (128, 5e5)):
        r = RotaryPosition(head_dim=d, theta=theta)
        inv, rot = r.rotary_table(DEV)
        assert rot == d and inv.dtype == torch.float32
        assert np.array_equal(inv.cpu().numpy(), P.rope_inverse_frequencies(d, theta))
    half = RotaryPosition(head_dim=64, theta=1e4, rotary_dim=32)
    assert half.rotary_table(DEV)[0].numel() == 16


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("activation", ["silu", "gelu_pytorch_tanh"])
def test_gated_mlp_part(dtype, activation):
    from velox_b200.parts import GatedMLP
    m = GatedMLP("m.", 72, 200, activation)
    w = make(m, dtype)
    x, xn = act((6, 72), dtype, 4)
    g = xn @ w["m.gate_proj.weight"].T
    a = P.silu(g) if activation == "silu" else 0.5 * g * (1 + np.tanh(math.sqrt(2 / math.pi) * (g + 0.044715 * g ** 3)))
    want = (a * (xn @ w["m.up_proj.weight"].T)) @ w["m.down_proj.weight"].T
    sb = P.store_bfloat16
    close(m.forward(x), want, dtype, "gated mlp", sb(sb(a * (xn @ w["m.up_proj.weight"].T)) @ w["m.down_proj.weight"].T))


@pytest.mark.parametrize("dtype", DTYPES)
def test_embedding_and_head(dtype):
    from velox_b200.parts import OutputHead, TokenEmbedding
    emb, head, tied = TokenEmbedding("e.", 300, 40), OutputHead("h.", 300, 40), OutputHead("h.", 300, 40, tied=True)
    we, wh = make(emb, dtype), make(head, dtype, seed=1)
    ids = torch.tensor([5, 299, 0, 5], dtype=torch.int32, device=DEV)
    from types import SimpleNamespace
    out = emb.forward(SimpleNamespace(token_ids=ids))   # (an embedding is handed the step's context)
    assert out.dtype == torch.float32 and np.array_equal(out.double().cpu().numpy(), we["e.weight"][[5, 299, 0, 5]])
    x, xn = act((4, 40), dtype, 5)
    logits = head.forward(x)
    assert logits.dtype == torch.float32
    close(logits, xn @ wh["h.weight"].T, torch.float32)   # (float32 logits from bfloat16 operands: nothing is rounded)
    tied.bind({}, runtime(dtype))
    tied.tie(emb.weight)
    assert tied.tensor_specs() == [] and tied.ignored_tensors() == ["h.weight"]
    close(tied.forward(x), xn @ we["e.weight"].T, torch.float32)


def step_context(cache, requests, device):
    """requests: [(id, tokens)] -> reserved cache + context"""
    from velox_b200.engine.batch import StepEntry, build_step_context
    entries = [StepEntry(i, t, []) for i, t in requests]
    for e in entries:
        if not cache.has_request(e.request_id):
            cache.add_request(e.request_id)
        assert cache.reserve(e.request_id, len(e.tokens))
    return entries, build_step_context(entries, cache, device)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("window,bias,qk_norm", [(0, False, True), (9, True, True), (0, True, False)])
def test_attention_part_in_two_portions(dtype, window, bias, qk_norm):
    """The mixer alone with its own cache: a sequence in two steps equals the
    plain attention block on the whole sequence."""
    from velox_b200.cache import CacheManager
    from velox_b200.parts import PagedAttention, PartSpec
    E, H, Hk, D, T = 72, 6, 3, 48, 29
    att = PagedAttention("a.", E, H, Hk, D, bias=bias, qk_norm=qk_norm, eps=1e-5, window=window,
                         position=PartSpec("rotary", "", dict(head_dim=D, theta=1e4)))
    w = make(att, dtype)
    cfg = dict(num_attention_heads=H, num_key_value_heads=Hk, head_dim=D, rms_norm_eps=1e-5, attention_bias=bias,
               rope_theta=1e4)
    x, xn = act((T, E), dtype, 6)
    if not qk_norm:  # the plain block always norms: a unit weight and a huge eps would not be the same; restate
        def plain_block(xn, st=P.keep):
            q = st(P.linear(xn, w["a.q_proj.weight"], w.get("a.q_proj.bias"))).reshape(T, H, D)
            k = st(P.linear(xn, w["a.k_proj.weight"], w.get("a.k_proj.bias"))).reshape(T, Hk, D)
            v = st(P.linear(xn, w["a.v_proj.weight"], w.get("a.v_proj.bias"))).reshape(T, Hk, D)
            q, k = st(P.rope(q, np.arange(T), 1e4)), st(P.rope(k, np.arange(T), 1e4))
            a = st(P.causal_attention(q, k, v, window)).reshape(T, H * D)
            return st(P.linear(a, w["a.o_proj.weight"], w.get("a.o_proj.bias")))
        want, rounded = plain_block(xn), plain_block(xn, P.store_bfloat16)
    else:
        want = P.attention_block(xn, np.arange(T), w, "a.", cfg, window)
        rounded = P.attention_block(xn, np.arange(T), w, "a.", cfg, window, P.store_bfloat16)
    cache = CacheManager([att.cache_spec()], [None], 8, 12, 2, 8, dtype, DEV, poison=True)
    got = []
    for lo, hi in ((0, 18), (18, T)):
        entries, ctx = step_context(cache, [("r", list(range(lo, hi)))], DEV)
        got.append(att.forward(x[lo:hi].contiguous(), ctx, cache.layer(0)))
        cache.commit("r", hi - lo)
    close(torch.cat(got), want, dtype, "attention part", rounded)


@pytest.mark.parametrize("dtype", DTYPES)
def test_pre_norm_block(dtype):
    from velox_b200.cache import CacheManager
    from velox_b200.parts import GatedMLP, PagedAttention, PartSpec, PreNormBlock, RMSNorm
    E, H, Hk, D, I, T, eps = 80, 4, 2, 32, 144, 21, 1e-6
    p = "model.layers.0."
    att = PagedAttention(p + "self_attn.", E, H, Hk, D, eps=eps, position=PartSpec("rotary", "", dict(head_dim=D, theta=1e6)))
    mlp = GatedMLP(p + "mlp.", E, I)
    n1, n2 = RMSNorm(p + "input_layernorm.", E, eps), RMSNorm(p + "post_attention_layernorm.", E, eps)
    w = {}
    for part in (att, mlp, n1, n2):
        w.update(make(part, dtype))
    block = PreNormBlock(att, mlp, {"mixer": n1, "feed_forward": n2})
    cfg = dict(num_attention_heads=H, num_key_value_heads=Hk, head_dim=D, rms_norm_eps=eps, attention_bias=False,
               rope_theta=1e6)
    res = torch.randn(T, E, generator=torch.Generator().manual_seed(7)).to(DEV)
    want = P.decoder_layer(res.double().cpu().numpy(), np.arange(T), w, 0, cfg)
    rounded = P.decoder_layer(res.double().cpu().numpy(), np.arange(T), w, 0, cfg, P.store_bfloat16)
    cache = CacheManager([att.cache_spec()], [None], 16, 4, 1, 4, dtype, DEV, poison=True)
    entries, ctx = step_context(cache, [("r", list(range(T)))], DEV)
    residual, delta = block.forward(res, None, ctx, cache.layer(0))
    close(residual.double() + delta.double(), want, dtype, "block", rounded)   # (the block updated `res` in place)
