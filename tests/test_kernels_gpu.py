"""Each kernel alone against its plain reference, at sizes other than the models'."""
import math

import numpy as np
import pytest
import torch

import plain_qwen3 as P

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
DTYPES = [torch.float32, torch.bfloat16]


def ops():
    from velox_b200.csrc import ops as o
    return o


def close(got, want, dtype, atol32=2e-5, what=""):
    """A kernel against the plain operation on the SAME inputs (already rounded to the
    kernel's element type).  float32: atol32 + 1e-5 |x|.  bfloat16: all that separates the
    two is the rounding of the result (and, in attention, of the probabilities) to
    bfloat16, 2^-9 relative each: a value may be off by 2^-7 of the largest value of its
    row, plus 2^-10 for rows near zero."""
    got = got.detach().double().cpu().numpy()
    want = np.asarray(want, np.float64)
    assert got.shape == want.shape, (got.shape, want.shape)
    assert np.isfinite(got).all(), what + ": non-finite output"
    err = np.abs(got - want)
    if dtype == torch.float32:
        bound = atol32 + 1e-5 * np.abs(want)
    else:
        flat = np.abs(want).reshape(-1, want.shape[-1])
        bound = (2.0 ** -7 * flat.max(axis=1, keepdims=True) + 2.0 ** -10).reshape(want.shape[:-1] + (1,))
    assert (err <= bound).all(), "%s: max err %.3g at %s" % (what, err.max(), np.unravel_index((err - bound).argmax(), err.shape))


def rnd(shape, dtype, seed, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(shape, generator=g) * scale).to(dtype).to(DEV)


def f64(t):
    return t.detach().double().cpu().numpy()


# ----------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", DTYPES)
def test_embedding(dtype):
    table = rnd((37, 50), dtype, 0)
    ids = torch.tensor([0, 36, 5, 5, 17], dtype=torch.int32, device=DEV)
    out = ops().embedding(ids, table)
    assert out.dtype == torch.float32
    assert torch.equal(out, table.float()[ids.long()])
    bad = ops().embedding(torch.tensor([3, 37], dtype=torch.int32, device=DEV), table)
    assert torch.isnan(bad[1]).all() and torch.equal(bad[0], table.float()[3])


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("width", [48, 1000, 4100])
def test_add_rmsnorm(dtype, width):
    rows, eps = 7, 1e-5
    res = rnd((rows, width), torch.float32, 1)
    delta = rnd((rows, width), dtype, 2)
    w = (1 + 0.05 * torch.randn(width)).to(DEV)
    want_sum = f64(res) + f64(delta)
    want = P.rms_norm(want_sum, f64(w), eps)
    r = res.clone()
    out = ops().add_rmsnorm(r, delta, w, eps, dtype)
    close(out, want, dtype, what="normed")
    assert np.allclose(f64(r), want_sum, atol=1e-6)  # the residual holds the float32 sum
    # no delta: residual untouched
    r2 = res.clone()
    out2 = ops().add_rmsnorm(r2, None, w, eps, dtype)
    close(out2, P.rms_norm(f64(res), f64(w), eps), dtype)
    assert torch.equal(r2, res)
    # gathered rows: only those are normed, the residual stays
    idx = torch.tensor([6, 0, 3], dtype=torch.int32, device=DEV)
    r3 = res.clone()
    out3 = ops().add_rmsnorm(r3, delta, w, eps, dtype, rows=idx)
    close(out3, want[[6, 0, 3]], dtype)
    assert torch.equal(r3, res)


@pytest.mark.parametrize("dtype", DTYPES)
def test_rmsnorm_rows(dtype):
    x = rnd((11, 80), dtype, 3)
    w = (1 + 0.05 * torch.randn(80)).to(DEV)
    close(ops().rmsnorm(x, w, 1e-6), P.rms_norm(f64(x), f64(w), 1e-6), dtype)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("act", ["silu", "gelu", "gelu_pytorch_tanh", "relu"])
def test_gated_act(dtype, act):
    x = rnd((9, 2 * 75), dtype, 4, 2.0)
    g, u = f64(x)[:, :75], f64(x)[:, 75:]
    if act == "silu":
        a = P.silu(g)
    elif act == "gelu":
        a = 0.5 * g * (1 + np.vectorize(math.erf)(g / math.sqrt(2)))
    elif act == "gelu_pytorch_tanh":
        a = 0.5 * g * (1 + np.tanh(math.sqrt(2 / math.pi) * (g + 0.044715 * g ** 3)))
    else:
        a = np.maximum(g, 0)
    close(ops().gated_act(x, act), a * u, dtype)
    # the same values laid out in tiles of 5 gates followed by their 5 ups
    tiled = torch.stack([x[:, :75].reshape(9, 15, 5), x[:, 75:].reshape(9, 15, 5)], 2).reshape(9, 150).contiguous()
    assert torch.equal(ops().gated_act(tiled, act, block=5), ops().gated_act(x, act))


# ----------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H,Hk,D,rot,S", [(6, 3, 48, 48, 8), (5, 1, 16, 8, 4), (8, 2, 128, 128, 16), (2, 2, 80, 0, 2)])
def test_qk_norm_rope_kv(dtype, H, Hk, D, rot, S):
    T, pages, eps, theta = 13, 9, 1e-5, 1e6
    qkv = rnd((T, (H + 2 * Hk) * D), dtype, 5)
    qw = (1 + 0.05 * torch.randn(D)).to(DEV)
    kw = (1 + 0.05 * torch.randn(D)).to(DEV)
    positions = torch.tensor([0, 1, 2, 77, 78, 5000, 5001, 31, 32, 33, 3, 40000, 9], dtype=torch.int32, device=DEV)
    slots = torch.randperm(pages * S)[:T].to(torch.int32).to(DEV)
    k_pool = torch.full((pages, Hk, S, D), float("nan"), dtype=dtype, device=DEV)
    v_pool = torch.full((pages, Hk, S, D), float("nan"), dtype=dtype, device=DEV)
    inv = None
    if rot:
        inv = torch.tensor([np.float32(1.0) / np.float32(theta ** (i / rot)) for i in range(0, rot, 2)],
                           dtype=torch.float32, device=DEV)
    x = f64(qkv)
    q = x[:, : H * D].reshape(T, H, D)
    k = x[:, H * D : (H + Hk) * D].reshape(T, Hk, D)
    v = x[:, (H + Hk) * D :].reshape(T, Hk, D)
    qn, kn = P.rms_norm(q, f64(qw), eps), P.rms_norm(k, f64(kw), eps)
    if rot:
        pos = positions.cpu().numpy()
        qn = np.concatenate([P.rope(qn[..., :rot], pos, theta), qn[..., rot:]], -1)
        kn = np.concatenate([P.rope(kn[..., :rot], pos, theta), kn[..., rot:]], -1)
    work = qkv.clone()
    ops().qk_norm_rope_kv(work, qw, kw, eps, inv, rot, positions, slots, k_pool, v_pool, H, Hk, D)
    close(work[:, : H * D].reshape(T, H, D), qn, dtype, what="q")
    sl = slots.cpu().numpy()
    got_k = k_pool[sl // S, :, sl % S, :]
    got_v = v_pool[sl // S, :, sl % S, :]
    close(got_k, kn, dtype, what="k in the pool")
    assert torch.equal(got_v, qkv[:, (H + Hk) * D :].reshape(T, Hk, D))  # values are copied bit for bit
    untouched = torch.ones(pages * S, dtype=torch.bool)
    untouched[sl] = False
    assert torch.isnan(k_pool.reshape(pages, Hk, S, D).permute(0, 2, 1, 3).reshape(pages * S, -1)[untouched]).all()
    # without a slot mapping nothing is written and keys are treated in place
    work2 = qkv.clone()
    ops().qk_norm_rope_kv(work2, qw, kw, eps, inv, rot, positions, None, None, None, H, Hk, D)
    close(work2[:, H * D : (H + Hk) * D].reshape(T, Hk, D), kn, dtype, what="k in place")
    assert torch.equal(work2[:, (H + Hk) * D :], qkv[:, (H + Hk) * D :])


def test_qk_norm_rope_kv_for_many_tokens_gives_the_same_bits():
    """From 64 tokens on the bfloat16 kernel for heads of 128 works row by row with the
    token's cosines and sines shared by all heads; the result is the one of the
    kernel for few tokens, bit for bit."""
    H, Hk, D, S, T, pages, eps = 6, 2, 128, 16, 150, 12, 1e-6
    qkv = rnd((T, (H + 2 * Hk) * D), torch.bfloat16, 6, 2.0)
    qw, kw = (1 + 0.05 * torch.randn(D)).to(DEV), (1 + 0.05 * torch.randn(D)).to(DEV)
    positions = torch.randint(0, 40000, (T,), dtype=torch.int32).to(DEV)
    slots = torch.randperm(pages * S)[:T].to(torch.int32)
    slots[17] = -1                                            # a row that writes nothing
    slots = slots.to(DEV)
    inv = torch.from_numpy(P.rope_inverse_frequencies(D, 1e6)).to(DEV)
    outs = []
    for step in (T, 50):                                      # all at once; in slices below 64 tokens
        work = qkv.clone()
        kp = torch.full((pages, Hk, S, D), float("nan"), dtype=torch.bfloat16, device=DEV)
        vp = torch.full_like(kp, float("nan"))
        for a in range(0, T, step):
            part = work[a:a + step].contiguous()
            ops().qk_norm_rope_kv(part, qw, kw, eps, inv, D, positions[a:a + step].contiguous(),
                                  slots[a:a + step].contiguous(), kp, vp, H, Hk, D)
            work[a:a + step] = part
        outs.append((work, kp, vp))
    for x, y in zip(*outs):
        assert torch.equal(torch.nan_to_num(x.float(), nan=-7.0), torch.nan_to_num(y.float(), nan=-7.0))
    assert int(torch.isnan(outs[0][1].float()).sum()) == (pages * S - (T - 1)) * Hk * D


# ----------------------------------------------------------------------------
def paged_case(dtype, seqs, H, Hk, D, S, window, seed, spike=None):
    """seqs: list of (kv_offset, new_tokens).  Builds whole sequences, scatters
    keys/values into scattered pages, and returns kernel inputs + the plain answer."""
    rng = np.random.default_rng(seed)
    total_pages = sum(-(-(o + n) // S) for o, n in seqs) + 5
    perm = rng.permutation(total_pages)
    k_pool = torch.full((total_pages, Hk, S, D), float("nan"), dtype=dtype, device=DEV)
    v_pool = torch.full((total_pages, Hk, S, D), float("nan"), dtype=dtype, device=DEV)
    max_blocks = max(-(-(o + n) // S) for o, n in seqs) + 2
    bt = np.full((len(seqs), max_blocks), -1, np.int32)
    qs, pos, sot, want = [], [], [], []
    used = 0
    for i, (off, n) in enumerate(seqs):
        L = off + n
        q = torch.randn(L, H, D, generator=torch.Generator().manual_seed(seed * 100 + i)).to(dtype)
        k = torch.randn(L, Hk, D, generator=torch.Generator().manual_seed(seed * 100 + 50 + i)).to(dtype)
        v = torch.randn(L, Hk, D, generator=torch.Generator().manual_seed(seed * 100 + 70 + i)).to(dtype)
        if spike is not None and L > spike:
            # one far key that every late query of head 0 must find: its score
            # towers over the others, so the output is that key's value
            j = spike
            q[-1, 0] = 0; q[-1, 0, 0] = 12.0
            k[j, 0] = 0; k[j, 0, 0] = 12.0
        npg = -(-L // S)
        pages = perm[used:used + npg]
        used += npg
        bt[i, :npg] = pages
        for p in range(L):
            k_pool[pages[p // S], :, p % S] = k[p].to(DEV)
            v_pool[pages[p // S], :, p % S] = v[p].to(DEV)
        ref = P.causal_attention(f64(q), f64(k), f64(v), window)
        qs.append(q[off:])
        want.append(ref[off:])
        pos += list(range(off, L))
        sot += [i] * n
    q_all = torch.cat(qs).reshape(-1, H * D).contiguous().to(DEV)
    return (q_all, k_pool, v_pool, torch.from_numpy(bt).to(DEV), torch.tensor(sot, dtype=torch.int32, device=DEV),
            torch.tensor(pos, dtype=torch.int32, device=DEV), np.concatenate(want).reshape(-1, H * D))


ATT_CASES = [
    # (seqs, H, Hk, D, S, window)
    ([(0, 1)], 4, 2, 16, 4, 0),                              # a sequence's first token
    ([(0, 3), (0, 2), (0, 1)], 4, 4, 32, 8, 0),              # first tokens, no grouping
    ([(0, 8), (20, 4), (10, 1)], 8, 2, 64, 4, 0),            # the reference's mixed batch: cold 8, warm 4 @20, decode 1 @10
    ([(239, 1)] * 8, 8, 2, 128, 16, 0),                      # 8 decodes over 240 keys
    ([(0, 37)], 6, 3, 48, 8, 0),                             # head size 48, 3 groups, a partial last page
    ([(0, 50), (45, 5), (63, 1)], 4, 1, 80, 16, 13),         # a window that is no multiple of the page
    ([(300, 2)], 2, 1, 256, 16, 0),                          # the largest head size
    ([(31, 1), (32, 1), (33, 1)], 4, 2, 16, 16, 0),          # around a page's edge
    ([(0, 21), (40, 3)], 6, 2, 40, 4, 0),                    # a head size that is even and no multiple of 16
]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("case", range(len(ATT_CASES)))
def test_paged_attention_generic(dtype, case):
    seqs, H, Hk, D, S, window = ATT_CASES[case]
    q, kp, vp, bt, sot, pos, want = paged_case(dtype, seqs, H, Hk, D, S, window, seed=case)
    out = ops().paged_attention_generic(q, H * D, kp, vp, bt, sot, pos, 1 / math.sqrt(D), window, H, Hk, D, q.shape[0])
    close(out, want, dtype, atol32=1e-5, what="attention case %d" % case)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("far", [0, 3, 250, 511])
def test_attention_finds_one_far_key_among_hundreds(dtype, far):
    H, Hk, D, S = 4, 2, 64, 16
    q, kp, vp, bt, sot, pos, want = paged_case(dtype, [(599, 1)], H, Hk, D, S, 0, seed=11, spike=far)
    out = ops().paged_attention_generic(q, H * D, kp, vp, bt, sot, pos, 1 / math.sqrt(D), 0, H, Hk, D, 1)
    close(out, want, dtype, atol32=1e-5)
    # the spike dominates: head 0's output is (nearly) the far key's value
    page, off = int(bt[0, far // S]), far % S
    assert torch.allclose(out[0, :D].float(), vp[page, 0, off].float(), atol=5e-2)


# ----------------------------------------------------------------------------
@pytest.mark.parametrize("M,N,K", [(1, 53, 71), (37, 64, 16), (130, 129, 100), (5, 384, 96)])
def test_gemm_simt_fp32(M, N, K):
    a, w = rnd((M, K), torch.float32, 6), rnd((N, K), torch.float32, 7)
    bias = rnd((N,), torch.float32, 8)
    close(ops().gemm_nt_simt(a, w), f64(a) @ f64(w).T, torch.float32)
    close(ops().gemm_nt_simt(a, w, bias), f64(a) @ f64(w).T + f64(bias), torch.float32)
    # a row's result does not depend on the rows beside it: bit-identical
    alone = ops().gemm_nt_simt(a[M - 1 :].contiguous(), w)
    assert torch.equal(alone[0], ops().gemm_nt_simt(a, w)[M - 1])


@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("M,N,K", [(1, 53, 72), (37, 64, 16), (130, 136, 104), (64, 384, 96), (8, 4096, 4096)])
def test_gemm_bf16(M, N, K, out_dtype):
    a, w = rnd((M, K), torch.bfloat16, 6), rnd((N, K), torch.bfloat16, 7, 0.05)
    want = f64(a) @ f64(w).T
    close(ops().gemm_bf16(a, w, None, out_dtype), want, torch.bfloat16)
    close(ops().gemm_nt_simt(a, w, None, out_dtype), want, torch.bfloat16)  # the plain product takes bfloat16 too
    bias = rnd((N,), torch.float32, 8)
    close(ops().gemm_bf16(a, w, bias, out_dtype), want + f64(bias), torch.bfloat16)


# ----------------------------------------------------------------------------
def test_sample_greedy_ties_and_rows():
    x = torch.randn(5, 1000, generator=torch.Generator().manual_seed(0)).to(DEV)
    x[2, 77] = x[2, 400] = 9.0  # the first maximum wins
    got = ops().sample(x).tolist()
    assert got == [P.greedy(r) for r in f64(x)] and got[2] == 77
    wide = torch.randn(3, 151936, generator=torch.Generator().manual_seed(1)).to(DEV)
    assert ops().sample(wide).tolist() == wide.argmax(-1).tolist()


@pytest.mark.parametrize("vocab", [384, 5000, 151936])
def test_sample_temperature_and_top_p(vocab):
    from velox_b200.sampling.rng import uniform
    rows = 12
    x = (torch.randn(rows, vocab, generator=torch.Generator().manual_seed(2)) * 2.0).to(DEV)
    temps = [0.0, 0.8, 1.0, 0.5, 1.3, 0.8, 0.8, 1.0, 0.0, 0.7, 2.0, 0.8]
    tops = [1.0, 1.0, 0.9, 0.5, 1.0, 0.3, 0.95, 0.0, 0.5, 0.999, 0.8, 1.0]
    us = [uniform(5, 0, i) for i in range(rows)]
    t = lambda v: torch.tensor(v, dtype=torch.float32, device=DEV)
    got = ops().sample(x, t(temps), t(tops), t(us)).tolist()
    xs = f64(x)
    for r in range(rows):
        if temps[r] <= 1e-7:
            assert got[r] == P.greedy(xs[r])
            continue
        p = P.probabilities(xs[r], temps[r], tops[r])
        want = P.sample_from(p, us[r])
        if got[r] != want:
            # float32 against float64 may disagree only where u falls on a boundary of the
            # cumulative distribution, or where the nucleus' edge is a near-tie
            c = np.cumsum(p)
            lo, hi = sorted((got[r], want))
            assert p[got[r]] > 0 and abs(c[lo] - us[r]) < 1e-5 * max(1, hi - lo), (r, got[r], want)
    # the same inputs give the same tokens
    assert ops().sample(x, t(temps), t(tops), t(us)).tolist() == got


def test_sample_top_p_keeps_only_the_nucleus():
    x = torch.full((1, 300), -5.0, device=DEV)
    x[0, [10, 20, 30]] = torch.tensor([3.0, 2.0, 1.0], device=DEV)
    t = lambda v: torch.tensor([v], dtype=torch.float32, device=DEV)
    seen = set()
    for i in range(64):
        seen.add(ops().sample(x, t(1.0), t(0.85), t(i / 64.0)).item())
    assert seen == {10, 20}  # p = .66, .24, .09: the first two reach 0.85
    assert {ops().sample(x, t(1.0), t(0.5), t(i / 64.0)).item() for i in range(64)} == {10}
    # ties at the nucleus' edge stay together: p = .475, .175 x 3, the rest 0.002 in all; 0.6 is crossed inside the tie
    y = torch.full((1, 5000), -12.0, device=DEV)
    y[0, [7, 4000, 4500, 4999]] = torch.tensor([3.0, 2.0, 2.0, 2.0], device=DEV)
    seen = {ops().sample(y, t(1.0), t(0.6), t(i / 256.0)).item() for i in range(256)}
    assert seen == {7, 4000, 4500, 4999}
    p = P.probabilities(f64(y)[0], 1.0, 0.6)
    assert set(np.nonzero(p)[0].tolist()) == seen


# ----------------------------------------------------------------------------
DECODE_CASES = [
    # (kv lengths, H, Hk, D, S, window)
    ([1, 2, 15, 16, 17], 8, 2, 128, 16, 0),          # first tokens, around a page's edge
    ([255, 256, 257, 600, 1600], 8, 2, 128, 16, 0),   # around a piece's edge (256 keys), several pieces
    ([700, 33, 300], 6, 6, 64, 32, 0),               # no grouping, head size 64, pages of 32
    ([900, 64, 257], 16, 1, 64, 16, 0),              # 16 query heads share one kv head
    ([1300, 40, 590, 5], 4, 2, 128, 16, 540),        # a window that crosses split boundaries
    ([3000], 32, 8, 128, 16, 0),                     # the flagship's head layout, 12 pieces
    # the kernel's other block shapes, chosen from requests x kv heads x pieces against 148 SMs:
    ([1000] + [(i * 97) % 1000 + 1 for i in range(19)], 16, 8, 128, 16, 0),   # 640 pieces: blocks of 5 warps
    ([1000] + [(i * 61) % 1000 + 1 for i in range(25)], 16, 8, 128, 16, 0),   # 832 pieces: blocks of 6 warps
    ([1000] + [(i * 43) % 1000 + 1 for i in range(29)], 16, 8, 64, 16, 0),    # 960 pieces: blocks of 4 warps, two an SM
]


@pytest.mark.parametrize("case", range(len(DECODE_CASES)))
def test_paged_decode_attention(case):
    lens, H, Hk, D, S, window = DECODE_CASES[case]
    seqs = [(n - 1, 1) for n in lens]
    q, kp, vp, bt, sot, pos, want = paged_case(torch.bfloat16, seqs, H, Hk, D, S, window, seed=40 + case)
    out = ops().paged_decode_attention(q, H * D, kp, vp, bt, sot, pos, 1 / math.sqrt(D), window, H, Hk, D,
                                       len(lens), max(lens))
    close(out, want, torch.bfloat16, what="decode attention case %d" % case)
    # and it agrees with the general kernel far more closely than with the bound
    gen = ops().paged_attention_generic(q, H * D, kp, vp, bt, sot, pos, 1 / math.sqrt(D), window, H, Hk, D, len(lens))
    assert (out.float() - gen.float()).abs().max() < 2e-2


@pytest.mark.parametrize("far", [0, 17, 255, 256, 700, 1023])
def test_decode_attention_finds_one_far_key(far):
    H, Hk, D, S = 8, 2, 128, 16
    q, kp, vp, bt, sot, pos, want = paged_case(torch.bfloat16, [(1099, 1)], H, Hk, D, S, 0, seed=12, spike=far)
    out = ops().paged_decode_attention(q, H * D, kp, vp, bt, sot, pos, 1 / math.sqrt(D), 0, H, Hk, D, 1, 1100)
    close(out, want, torch.bfloat16)
    page, off = int(bt[0, far // S]), far % S
    assert torch.allclose(out[0, :D].float(), vp[page, 0, off].float(), atol=5e-2)


def test_decode_attention_token_rows_and_batch_independence():
    """Requests picked out of a larger batch by row; a request's output does not
    depend on which others are beside it."""
    H, Hk, D, S = 8, 2, 128, 16
    seqs = [(0, 5), (499, 1), (0, 3), (299, 1), (1200, 1)]
    q, kp, vp, bt, sot, pos, want = paged_case(torch.bfloat16, seqs, H, Hk, D, S, 0, seed=13)
    rows = torch.tensor([5, 9, 10], dtype=torch.int32, device=DEV)  # the three single-token requests
    out = torch.zeros((11, H * D), dtype=torch.bfloat16, device=DEV)
    ops().paged_decode_attention(q, H * D, kp, vp, bt, sot, pos, 1 / math.sqrt(D), 0, H, Hk, D, 3, 1201,
                                 token_rows=rows, out=out)
    close(out[rows.long()], want[[5, 9, 10]], torch.bfloat16)
    assert (out[:5] == 0).all()
    alone = torch.zeros_like(out)
    ops().paged_decode_attention(q, H * D, kp, vp, bt, sot, pos, 1 / math.sqrt(D), 0, H, Hk, D, 1, 500,
                                 token_rows=rows[:1], out=alone)
    assert torch.equal(alone[5], out[5])  # bit-identical alone and in company


def test_decode_attention_gives_the_same_bits_in_every_block_shape():
    """The kernel picks warps per block and stages from the step's size; a request's
    output must not notice (1, 20, 26 and 30 requests reach its four shapes on 148 SMs)."""
    H, Hk, D, S = 16, 8, 128, 16
    lens = [1000] + [(i * 43) % 1000 + 1 for i in range(29)]
    q, kp, vp, bt, sot, pos, want = paged_case(torch.bfloat16, [(n - 1, 1) for n in lens], H, Hk, D, S, 0, seed=15)
    full = ops().paged_decode_attention(q, H * D, kp, vp, bt, sot, pos, 1 / math.sqrt(D), 0, H, Hk, D, 30, 1000)
    close(full, want, torch.bfloat16)
    for n in (1, 20, 26):
        part = ops().paged_decode_attention(q, H * D, kp, vp, bt, sot, pos, 1 / math.sqrt(D), 0, H, Hk, D, n, 1000)
        assert torch.equal(part[:n], full[:n]), n


def test_decode_attention_refuses_what_it_cannot_do():
    from velox_b200.csrc.ops import KernelError
    q, kp, vp, bt, sot, pos, _ = paged_case(torch.bfloat16, [(9, 1)], 4, 2, 48, 16, 0, seed=14)
    with pytest.raises(KernelError, match="size"):
        ops().paged_decode_attention(q, 4 * 48, kp, vp, bt, sot, pos, 0.1, 0, 4, 2, 48, 1, 10)
    assert not ops().decode_attention_supported(torch.bfloat16, 48, 16, 2)
    assert not ops().decode_attention_supported(torch.bfloat16, 128, 8, 2)
    assert not ops().decode_attention_supported(torch.float32, 128, 16, 2)


# ----------------------------------------------------------------------------
@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("M,N,K", [(1, 48, 64), (3, 50, 96), (8, 4096, 4096), (7, 136, 160), (8, 333, 1024), (5, 16, 12288)])
def test_gemm_skinny(M, N, K, out_dtype):
    a, w = rnd((M, K), torch.bfloat16, 20), rnd((N, K), torch.bfloat16, 21, 0.05)
    bias = rnd((N,), torch.float32, 22)
    want = f64(a) @ f64(w).T
    close(ops().gemm_skinny(a, w, None, out_dtype), want, torch.bfloat16, what="skinny")
    close(ops().gemm_skinny(a, w, bias, out_dtype), want + f64(bias), torch.bfloat16, what="skinny + bias")
    # against the plain product on the same bfloat16 inputs: only the order of additions differs
    ref = ops().gemm_nt_simt(a, w, None, torch.float32)
    got = ops().gemm_skinny(a, w, None, torch.float32)
    assert (got - ref).abs().max() <= 1e-3 * max(1.0, float(ref.abs().max()))
    # a row alone gives the same bits as in company
    alone = ops().gemm_skinny(a[:1].contiguous(), w, None, torch.float32)
    assert torch.equal(alone[0], got[0])


@pytest.mark.parametrize("act", ["silu", "gelu_pytorch_tanh"])
@pytest.mark.parametrize("M,I,K", [(2, 24, 64), (8, 200, 96), (5, 1024, 512)])
def test_gemm_skinny_gated(M, I, K, act):
    a = rnd((M, K), torch.bfloat16, 23)
    wg, wu = rnd((I, K), torch.bfloat16, 24, 0.1), rnd((I, K), torch.bfloat16, 25, 0.1)
    # tiles of 16 rows: 8 gate rows, then their 8 up rows
    w = torch.stack([wg.view(I // 8, 8, K), wu.view(I // 8, 8, K)], 1).reshape(2 * I, K).contiguous()
    g, u = f64(a) @ f64(wg).T, f64(a) @ f64(wu).T
    av = P.silu(g) if act == "silu" else 0.5 * g * (1 + np.tanh(math.sqrt(2 / math.pi) * (g + 0.044715 * g ** 3)))
    close(ops().gemm_skinny(a, w, None, torch.bfloat16, gated_activation=act), av * u, torch.bfloat16, what="gated")


def test_gemm_skinny_refuses_what_it_cannot_do():
    from velox_b200.csrc.ops import KernelError
    a, w = rnd((9, 64), torch.bfloat16, 1), rnd((32, 64), torch.bfloat16, 2)
    with pytest.raises(KernelError):
        ops().gemm_skinny(a, w)
    with pytest.raises(KernelError):
        ops().gemm_skinny(rnd((4, 40), torch.bfloat16, 1), rnd((32, 40), torch.bfloat16, 2))
    assert not ops().skinny_supported(4, 40, a, w) and not ops().skinny_supported(9, 64, a, w)


# ----------------------------------------------------------------------------
def prefill_inputs(seqs):
    cu = np.concatenate([[0], np.cumsum([n for _, n in seqs])]).astype(np.int32)
    offs = np.asarray([o for o, _ in seqs], np.int32)
    return torch.from_numpy(cu).to(DEV), torch.from_numpy(offs).to(DEV)


PREFILL_CASES = [
    # (seqs (kv_offset, new tokens), H, Hk, D, S, window)
    ([(0, 1)], 4, 2, 64, 16, 0),                               # a sequence's first token
    ([(0, 64)], 4, 2, 128, 16, 0),                             # exactly one tile
    ([(0, 65), (0, 3), (0, 127)], 4, 4, 128, 16, 0),           # one past a tile, a short one, one short of two tiles
    ([(0, 8), (20, 4), (10, 1)], 8, 2, 64, 16, 0),             # the reference's mixed batch: cold 8, warm 4 @20, decode 1 @10
    ([(100, 200), (63, 2), (64, 1), (300, 1)], 8, 2, 128, 16, 0),   # portions on top of cached keys, decodes beside them
    ([(0, 300)], 6, 3, 64, 32, 0),                             # pages of 32, 3 groups
    ([(0, 200), (150, 90), (400, 1)], 4, 1, 128, 16, 70),      # a window that is no multiple of the tile
    ([(7, 130)], 32, 8, 128, 16, 0),                           # the flagship's head layout
]


@pytest.mark.parametrize("case", range(len(PREFILL_CASES)))
def test_paged_prefill_attention(case):
    seqs, H, Hk, D, S, window = PREFILL_CASES[case]
    q, kp, vp, bt, sot, pos, want = paged_case(torch.bfloat16, seqs, H, Hk, D, S, window, seed=60 + case)
    cu, offs = prefill_inputs(seqs)
    out = ops().paged_prefill_attention(q, H * D, kp, vp, bt, cu, offs, 1 / math.sqrt(D), window, H, Hk, D,
                                        len(seqs), max(n for _, n in seqs), q.shape[0])
    close(out, want, torch.bfloat16, what="prefill attention case %d" % case)
    gen = ops().paged_attention_generic(q, H * D, kp, vp, bt, sot, pos, 1 / math.sqrt(D), window, H, Hk, D, q.shape[0])
    assert (out.float() - gen.float()).abs().max() < 2e-2


@pytest.mark.parametrize("far", [0, 63, 64, 500, 777])
def test_prefill_attention_finds_one_far_key(far):
    H, Hk, D, S = 8, 2, 128, 16
    seqs = [(700, 100)]
    q, kp, vp, bt, sot, pos, want = paged_case(torch.bfloat16, seqs, H, Hk, D, S, 0, seed=15, spike=far)
    cu, offs = prefill_inputs(seqs)
    out = ops().paged_prefill_attention(q, H * D, kp, vp, bt, cu, offs, 1 / math.sqrt(D), 0, H, Hk, D, 1, 100, 100)
    close(out, want, torch.bfloat16)
    page, off = int(bt[0, far // S]), far % S
    assert torch.allclose(out[-1, :D].float(), vp[page, 0, off].float(), atol=5e-2)  # the last query has the spike


# ----------------------------------------------------------------------------
TC_SHAPES = [(128, 256, 64), (128, 128, 128), (256, 512, 4096), (200, 384, 96), (77, 48, 72), (1000, 6144, 4096),
             (2048, 4096, 12288)]


TC_TILES = {"128x256": dict(wide=True), "128x128": dict(wide=False), "256x256 by a pair of blocks": dict(pair=True)}


@pytest.mark.parametrize("tiles", list(TC_TILES))
@pytest.mark.parametrize("M,N,K", TC_SHAPES)
def test_gemm_tcgen05(M, N, K, tiles):
    how = TC_TILES[tiles]
    a, w = rnd((M, K), torch.bfloat16, 30), rnd((N, K), torch.bfloat16, 31, 0.05)
    got = ops().gemm_tcgen05(a, w, None, **how)
    ops().check_device_errors()
    if M * N * K <= 1 << 28:
        close(got, f64(a) @ f64(w).T, torch.bfloat16, what="tcgen05")
    # against the library product on the same inputs (both accumulate in float32)
    ref = torch.mm(a, w.t())
    scale = max(1.0, float(ref.float().abs().max()))
    assert (got.float() - ref.float()).abs().max() <= 2e-2 * scale
    bias = rnd((N,), torch.float32, 32)
    got_b = ops().gemm_tcgen05(a, w, bias, **how)
    assert (got_b.float() - (ref.float() + bias)).abs().max() <= 2e-2 * scale + 2e-2


@pytest.mark.parametrize("tiles", list(TC_TILES))
@pytest.mark.parametrize("M,I,K", [(128, 128, 64), (300, 200, 96), (2048, 12288, 4096)])
def test_gemm_tcgen05_gated(M, I, K, tiles):
    a = rnd((M, K), torch.bfloat16, 33)
    wg, wu = rnd((I, K), torch.bfloat16, 34, 0.05), rnd((I, K), torch.bfloat16, 35, 0.05)
    w = torch.stack([wg.view(I // 8, 8, K), wu.view(I // 8, 8, K)], 1).reshape(2 * I, K).contiguous()
    got = ops().gemm_tcgen05(a, w, None, gated_activation="silu", **TC_TILES[tiles])
    ops().check_device_errors()
    g, u = torch.mm(a, wg.t()).float(), torch.mm(a, wu.t()).float()
    want = torch.nn.functional.silu(g) * u
    assert got.shape == (M, I)
    assert (got.float() - want).abs().max() <= 3e-2 + 3e-2 * float(want.abs().max())


# ----------------------------------------------------------------------------
TC_PREFILL_CASES = [
    ([(0, 1)], 4, 2, 128, 16, 0),                                  # a sequence's first token
    ([(0, 128)], 4, 1, 128, 16, 0),                                # 4 heads share a tile: 32 tokens each
    ([(0, 65), (0, 3), (0, 127)], 4, 4, 128, 16, 0),               # no sharing: 128 tokens a tile
    ([(100, 200), (63, 2), (64, 1), (300, 1)], 8, 2, 128, 16, 0),  # portions on top of cached keys, decodes beside them
    ([(0, 300)], 16, 2, 128, 32, 0),                               # 8 heads share, pages of 32
    ([(0, 400), (350, 90), (600, 1)], 4, 1, 128, 16, 170),         # a window that is no multiple of the tile
    ([(0, 300), (77, 41)], 10, 2, 128, 16, 0),                     # 5 heads a kv head (24 tokens of each in a tile, 8 rows idle)
    ([(130, 100), (0, 50)], 3, 1, 128, 32, 90),                    # 3 heads: 40 tokens each; a window
    ([(0, 200)], 14, 2, 128, 16, 0),                               # 7 heads: 16 tokens each, 16 rows idle
    ([(500, 64)], 6, 1, 128, 16, 0),                               # 6 heads
    ([(7, 333)], 32, 8, 128, 16, 0),                               # the flagship's head layout
    ([(0, 700)], 2, 1, 128, 16, 0),                                # two heads share: several tiles deep
]


@pytest.mark.parametrize("case", range(len(TC_PREFILL_CASES)))
def test_paged_prefill_attention_tc(case):
    seqs, H, Hk, D, S, window = TC_PREFILL_CASES[case]
    q, kp, vp, bt, sot, pos, want = paged_case(torch.bfloat16, seqs, H, Hk, D, S, window, seed=80 + case)
    cu, offs = prefill_inputs(seqs)
    out = ops().paged_prefill_attention_tc(q, H * D, kp, vp, bt, cu, offs, 1 / math.sqrt(D), window, H, Hk, D,
                                           len(seqs), max(n for _, n in seqs), q.shape[0])
    ops().check_device_errors()
    close(out, want, torch.bfloat16, what="tcgen05 prefill attention case %d" % case)
    gen = ops().paged_attention_generic(q, H * D, kp, vp, bt, sot, pos, 1 / math.sqrt(D), window, H, Hk, D, q.shape[0])
    assert (out.float() - gen.float()).abs().max() < 3e-2


@pytest.mark.parametrize("far", [0, 127, 128, 500, 777])
def test_prefill_attention_tc_finds_one_far_key(far):
    H, Hk, D, S = 8, 2, 128, 16
    seqs = [(700, 100)]
    q, kp, vp, bt, sot, pos, want = paged_case(torch.bfloat16, seqs, H, Hk, D, S, 0, seed=16, spike=far)
    cu, offs = prefill_inputs(seqs)
    out = ops().paged_prefill_attention_tc(q, H * D, kp, vp, bt, cu, offs, 1 / math.sqrt(D), 0, H, Hk, D, 1, 100, 100)
    ops().check_device_errors()
    close(out, want, torch.bfloat16)
    page, off = int(bt[0, far // S]), far % S
    assert torch.allclose(out[-1, :D].float(), vp[page, 0, off].float(), atol=5e-2)


# ----------------------------------------------------------------------------
def _attend(kernel, q, kp, vp, bt, sot, pos, seqs, H, Hk, D, window):
    scale = 1 / math.sqrt(D)
    if kernel == "generic":
        return ops().paged_attention_generic(q, H * D, kp, vp, bt, sot, pos, scale, window, H, Hk, D, q.shape[0])
    if kernel == "decode":
        return ops().paged_decode_attention(q, H * D, kp, vp, bt, sot, pos, scale, window, H, Hk, D, len(seqs),
                                            max(o + n for o, n in seqs))
    cu, offs = prefill_inputs(seqs)
    fn = ops().paged_prefill_attention_tc if kernel == "prefill_tc" else ops().paged_prefill_attention
    out = fn(q, H * D, kp, vp, bt, cu, offs, scale, window, H, Hk, D, len(seqs), max(n for _, n in seqs), q.shape[0])
    ops().check_device_errors()
    return out


@pytest.mark.parametrize("window,length", [(70, 400), (256, 1000), (33, 34), (129, 700)])
@pytest.mark.parametrize("kernel", ["generic", "decode", "prefill", "prefill_tc"])
def test_a_window_ends_where_it_should(kernel, window, length):
    """The query at position p sees the keys p + 1 - W to p (src/paged/metal_kernels.rs:135-137,
    339-341).  A key whose score towers over all others decides the output when it stands at
    p + 1 - W, and must leave no trace when it stands at p - W, one place further back."""
    H, Hk, D, S = 8, 2, 128, 16
    new = 1 if kernel == "decode" else min(40, length)      # the last query of a portion, or a decoded token
    seqs = [(length - new, new)]
    p = length - 1
    for inside in (True, False):
        j = p + 1 - window if inside else p - window
        q, kp, vp, bt, sot, pos, want = paged_case(torch.bfloat16, seqs, H, Hk, D, S, window, seed=17, spike=j)
        out = _attend(kernel, q, kp, vp, bt, sot, pos, seqs, H, Hk, D, window)
        close(out, want, torch.bfloat16, what="%s, spike %s the window" % (kernel, "inside" if inside else "behind"))
        value = vp[int(bt[0, j // S]), 0, j % S].float()
        near = torch.allclose(out[-1, :D].float(), value, atol=2e-2)
        assert near == inside, "%s: the key at %d (query at %d, window %d) %s" % (
            kernel, j, p, window, "was not seen" if inside else "was seen")


# ----------------------------------------------------------------------------
TC_SPLIT_CASES = [
    ([(3000, 64)], 8, 2, 128, 16, 0),                              # two query tiles on 24 key tiles: cut into 6 runs
    ([(1500, 40), (20, 33), (2500, 35), (0, 70)], 8, 2, 128, 16, 0),  # cut (3 runs), whole, cut (5 runs), whole, in one launch
    ([(2000, 100)], 32, 8, 128, 16, 0),                            # the flagship's head layout: 4 query tiles x 8 kv heads
    ([(4000, 50), (900, 60)], 4, 1, 128, 32, 600),                 # a window: the runs' tiles start far from key 0
    ([(1021, 130)], 4, 4, 128, 16, 0),                             # no sharing; the last tokens see one key tile more than the first
    ([(2100, 70), (1300, 33)], 10, 2, 128, 16, 0),                 # 5 heads a kv head, cut
]


@pytest.mark.parametrize("case", range(len(TC_SPLIT_CASES)))
def test_paged_prefill_attention_tc_cut_into_runs(case):
    """A short portion on top of many cached keys: its key tiles are cut into runs that several blocks take,
    and a second kernel adds the runs."""
    seqs, H, Hk, D, S, window = TC_SPLIT_CASES[case]
    q, kp, vp, bt, sot, pos, want = paged_case(torch.bfloat16, seqs, H, Hk, D, S, window, seed=120 + case)
    cu, offs = prefill_inputs(seqs)
    max_kv = max(o + n for o, n in seqs)
    out = ops().paged_prefill_attention_tc(q, H * D, kp, vp, bt, cu, offs, 1 / math.sqrt(D), window, H, Hk, D,
                                           len(seqs), max(n for _, n in seqs), q.shape[0], max_kv=max_kv)
    ops().check_device_errors()
    close(out, want, torch.bfloat16, what="tcgen05 prefill attention in runs, case %d" % case)
    whole = ops().paged_prefill_attention_tc(q, H * D, kp, vp, bt, cu, offs, 1 / math.sqrt(D), window, H, Hk, D,
                                             len(seqs), max(n for _, n in seqs), q.shape[0])
    assert not torch.equal(out, whole), "nothing was cut: the case lost its point"
    assert (out.float() - whole.float()).abs().max() < 2e-2
    # a request's result does not depend on what else is in the launch
    if len(seqs) > 1:
        alone_q, kp1, vp1, bt1, _, _, _ = paged_case(torch.bfloat16, seqs[:1], H, Hk, D, S, window, seed=120 + case)
        cu1, offs1 = prefill_inputs(seqs[:1])
        alone = ops().paged_prefill_attention_tc(alone_q, H * D, kp1, vp1, bt1, cu1, offs1, 1 / math.sqrt(D), window, H, Hk,
                                                 D, 1, seqs[0][1], alone_q.shape[0], max_kv=max_kv)
        assert torch.equal(alone, out[:seqs[0][1]])


@pytest.mark.parametrize("seed", range(10))
def test_paged_prefill_attention_tc_drawn_shapes(seed):
    """Drawn cases: one to four requests with portions of 1 to 400 tokens on 0 to 3,000 cached keys, every group size (1 to 8)
    and page size the kernel takes, with and without a window (of any length, so that the two query tiles of a block
    want different key tiles), cut into runs or not.  Never-written slots of the pools hold NaN."""
    rng = np.random.default_rng(900 + seed)
    G = int(rng.choice([1, 2, 3, 4, 5, 6, 7, 8]))
    Hk = int(rng.choice([1, 2, 3]))
    H, D = G * Hk, 128
    S = int(rng.choice([16, 32, 64]))
    window = int(rng.choice([0, 0, int(rng.integers(1, 700))]))
    seqs = []
    for _ in range(int(rng.integers(1, 5))):
        n = int(rng.choice([1, int(rng.integers(2, 40)), int(rng.integers(40, 400))]))
        off = int(rng.choice([0, int(rng.integers(1, 300)), int(rng.integers(300, 3000))]))
        seqs.append((off, n))
    q, kp, vp, bt, sot, pos, want = paged_case(torch.bfloat16, seqs, H, Hk, D, S, window, seed=950 + seed)
    cu, offs = prefill_inputs(seqs)
    max_kv = max(o + n for o, n in seqs) if seed % 2 == 0 else 0
    out = ops().paged_prefill_attention_tc(q, H * D, kp, vp, bt, cu, offs, 1 / math.sqrt(D), window, H, Hk, D,
                                           len(seqs), max(n for _, n in seqs), q.shape[0], max_kv=max_kv)
    ops().check_device_errors()
    close(out, want, torch.bfloat16, what="drawn case %d: %r, %d/%d heads, pages of %d, window %d" % (seed, seqs, H, Hk, S, window))


@pytest.mark.parametrize("far", [0, 500, 1023, 1024, 2900])
def test_prefill_attention_tc_in_runs_finds_one_far_key(far):
    H, Hk, D, S = 8, 2, 128, 16
    seqs = [(2960, 40)]
    q, kp, vp, bt, sot, pos, want = paged_case(torch.bfloat16, seqs, H, Hk, D, S, 0, seed=18, spike=far)
    cu, offs = prefill_inputs(seqs)
    out = ops().paged_prefill_attention_tc(q, H * D, kp, vp, bt, cu, offs, 1 / math.sqrt(D), 0, H, Hk, D, 1, 40, 40, max_kv=3000)
    ops().check_device_errors()
    close(out, want, torch.bfloat16)
    page, off = int(bt[0, far // S]), far % S
    value = vp[page, 0, off].float().cpu().numpy()
    scale = np.abs(value).max()
    assert np.abs(want[-1, :D] - value).max() < 0.03 * scale, "the far key does not decide the plain answer: the case lost its point"
    assert np.abs(f64(out)[-1, :D] - value).max() < 0.04 * scale
