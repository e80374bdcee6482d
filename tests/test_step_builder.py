"""The host library's step builders against a plain restatement in numpy: what
every kernel reads about a step (token rows, positions, block tables, slots)."""
import ctypes

import numpy as np
import pytest

from velox_b200 import native
from velox_b200.cache import CacheManager
from velox_b200.engine.batch import StepEntry, build_step_arrays
from velox_b200.parts.base import PagedKV


def manager(window=24):
    specs = [PagedKV(2, 16, 0), PagedKV(2, 16, window), PagedKV(2, 16, 0)]
    return CacheManager(specs, [None, None, None], 8, 64, 6, 32)


def plain(entries, cache, short_max=1):
    """The description built row by row from the request's books."""
    S, MB = cache.page_size, cache.max_blocks
    out = dict(token_ids=[], positions=[], seq_of_token=[], cu_seqlens=[0], kv_offsets=[], state_slots=[], wanted_rows=[],
               single_rows=[], portion_seqs=[])
    groups = [dict(bt=[], sm=[]) for _ in cache.groups]
    row = 0
    for i, e in enumerate(entries):
        rc = cache.requests[e.request_id]
        for j, t in enumerate(e.tokens):
            out["token_ids"].append(t)
            out["positions"].append(rc.length + j)
            out["seq_of_token"].append(i)
            for g, table in zip(groups, rc.tables):
                pos = rc.length + j
                g["sm"].append(table[pos // S] * S + pos % S)
        out["cu_seqlens"].append(row + len(e.tokens))
        out["kv_offsets"].append(rc.length)
        out["state_slots"].append(rc.slot)
        out["wanted_rows"] += [row + w for w in e.want]
        if len(e.tokens) <= short_max:
            out["single_rows"] += list(range(row, row + len(e.tokens)))
        else:
            out["portion_seqs"].append(i)
        for g, table in zip(groups, rc.tables):
            g["bt"].append(table + [-1] * (MB - len(table)))
        row += len(e.tokens)
    return out, groups


def test_a_mixed_step_is_described_as_the_books_say():
    rng = np.random.default_rng(0)
    m = manager()
    lens_before = {"a": 37, "b": 0, 7: 70, "d": 5}
    for rid, L in lens_before.items():
        m.add_request(rid)
        if L:
            assert m.reserve(rid, L)
            m.commit(rid, L)          # the windowed group has given back pages of request 7 by now
    entries = [StepEntry("a", [int(t) for t in rng.integers(0, 100, 11)], [0, 10]),
               StepEntry(7, [5], [0]),
               StepEntry("b", [int(t) for t in rng.integers(0, 100, 19)], []),
               StepEntry("d", [9, 8], [1])]
    for e in entries:
        assert m.reserve(e.request_id, len(e.tokens))
    buf, sizes, starts, summary = build_step_arrays(entries, m, vocab_size=100)
    want, groups = plain(entries, m)
    names = list(want)
    for k, name in enumerate(names):
        got = buf[starts[k]:starts[k] + sizes[k]]
        assert got.tolist()[:len(want[name])] == want[name], name   # (single_rows and portion_seqs: the filled part)
    for g, ref in enumerate(groups):
        bt = buf[starts[9 + 2 * g]:starts[9 + 2 * g] + sizes[9 + 2 * g]].reshape(len(entries), m.max_blocks)
        sm = buf[starts[10 + 2 * g]:starts[10 + 2 * g] + sizes[10 + 2 * g]]
        assert bt.tolist() == ref["bt"] and sm.tolist() == ref["sm"]
    assert -1 in groups[1]["bt"][1][:4]            # pages the window passed are gone from request 7's table
    assert summary == [33, 4, 19, 71, 1, 71, 3, 1]   # one request brings a single token (and has 71 keys then)
    # requests of up to 11 tokens listed token by token: a's 11, 7's one and d's two rows; b's 19 stay a portion
    buf, sizes, starts, summary = build_step_arrays(entries, m, vocab_size=100, short_max=11)
    want, _ = plain(entries, m, short_max=11)
    assert want["single_rows"] == list(range(0, 12)) + [31, 32] and want["portion_seqs"] == [2]
    for k, name in enumerate(want):
        assert buf[starts[k]:starts[k] + sizes[k]].tolist()[:len(want[name])] == want[name], name
    assert summary == [33, 4, 19, 71, 14, 71, 1, 11]
    assert all(s % 4 == 0 for s in starts)         # every section on a 16-byte boundary


def test_what_the_builder_refuses():
    m = manager()
    m.add_request("a")
    with pytest.raises(ValueError, match="block table too short"):
        build_step_arrays([StepEntry("a", [1, 2, 3], [])], m)          # nothing reserved
    assert m.reserve("a", 3)
    with pytest.raises(ValueError, match="token id outside"):
        build_step_arrays([StepEntry("a", [1, 200, 3], [])], m, vocab_size=100)
    with pytest.raises(ValueError, match="wanted place"):
        build_step_arrays([StepEntry("a", [1, 2, 3], [3])], m, vocab_size=100)
    with pytest.raises(KeyError):
        build_step_arrays([StepEntry("nobody", [1], [0])], m)


def test_a_decode_step_padded_to_its_bucket():
    m = manager()
    lengths = {"x": 41, "y": 8, "z": 15}
    for rid, L in lengths.items():
        m.add_request(rid)
        assert m.reserve(rid, L)
        m.commit(rid, L)
        assert m.reserve(rid, 1)
    n, B, MB, G = 3, 8, m.max_blocks, len(m.groups)
    sizes = [B, B, B, B + 1, B, B, B, B, B] + [B * MB, B] * G
    starts, cur = [], 0
    for s in sizes:
        starts.append(cur)
        cur += (s + 3) // 4 * 4
    buf = np.full(cur, 77, np.int32)
    max_kv = ctypes.c_int64(0)
    native.check(m._lib.vxh_fill_decode(m._book, n, B, m.handles(lengths), native.int_array([3, 4, 5]), 100,
                                        buf.ctypes.data_as(ctypes.c_void_p), native.int64_array(starts),
                                        ctypes.byref(max_kv)))
    sec = lambda k: buf[starts[k]:starts[k] + sizes[k]]
    assert sec(0).tolist() == [3, 4, 5, 0, 0, 0, 0, 0]
    assert sec(1).tolist() == [41, 8, 15, 0, 0, 0, 0, 0] and sec(4).tolist() == sec(1).tolist()
    assert sec(5).tolist()[:3] == [m.requests[r].slot for r in lengths] and sec(5).tolist()[3:] == [0] * 5
    assert all((sec(k) == 77).all() for k in (2, 3, 6, 7, 8))   # constant sections are left alone
    assert max_kv.value == 42
    cols = 41 // 8 + 1
    for g in range(G):
        bt = sec(9 + 2 * g).reshape(B, MB)
        sm = sec(10 + 2 * g)
        for i, rid in enumerate(lengths):
            table = m.requests[rid].tables[g]
            L = lengths[rid]
            assert bt[i, :cols].tolist() == (table + [-1] * MB)[:cols]
            assert sm[i] == table[L // 8] * 8 + L % 8
        assert (bt[n:, :cols] == 0).all() and (sm[n:] == -1).all()
        assert (bt[:, cols:] == 77).all()          # columns nobody can reach are not written
