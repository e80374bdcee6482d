"""The decode-attention entry point that allocates nothing, called through its
exported C symbol the way a caller without an allocator would, against the
ordinary entry point.

Such a caller (code inside someone else's stream capture, a real-time loop, a
host with a fixed memory budget) passes its own inputs and outputs and no
scratch; the library's built-in scratch array is shared by all calls and keeps
the last call's contents, so the check is made on two calls in a row with
different inputs.  This file is collected last on purpose."""
import ctypes
import gc
import math

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _inputs(seed, lens, H, Hk, D, S):
    g = torch.Generator().manual_seed(seed)
    pages_per = [-(-n // S) for n in lens]
    total = sum(pages_per) + 3
    kp = torch.randn(total, Hk, S, D, generator=g).to(torch.bfloat16).to(DEV)
    vp = torch.randn(total, Hk, S, D, generator=g).to(torch.bfloat16).to(DEV)
    perm = torch.randperm(total, generator=g).tolist()
    bt = torch.full((len(lens), max(pages_per) + 1), -1, dtype=torch.int32)
    at = 0
    for i, n in enumerate(pages_per):
        bt[i, :n] = torch.tensor(perm[at:at + n], dtype=torch.int32)
        at += n
    q = torch.randn(len(lens), H * D, generator=g).to(torch.bfloat16).to(DEV)
    pos = torch.tensor([n - 1 for n in lens], dtype=torch.int32, device=DEV)
    sot = torch.arange(len(lens), dtype=torch.int32, device=DEV)
    return q, kp, vp, bt.to(DEV), sot, pos


def test_no_alloc_entry_point_matches_the_ordinary_one_twice_in_a_row():
    from velox_b200.csrc import build, ops
    lib = ctypes.CDLL(build.build())
    P, I, F = ctypes.c_void_p, ctypes.c_int, ctypes.c_float
    fn = lib.vx_paged_decode_attention_static
    fn.argtypes = [P, I, P, P, P, I, P, P, P, I, P, I, F, I, I, I, I, I, I, I, P]
    fn.restype = I
    lib.vx_paged_decode_static_max_floats.restype = ctypes.c_longlong
    limit = lib.vx_paged_decode_static_max_floats()
    assert limit == 4 * 1024 * 1024

    H, Hk, D, S, chunk = 8, 2, 128, 16, ops.DECODE_CHUNK_TILES
    stream = torch.cuda.current_stream().cuda_stream
    for call, lens in enumerate(([900, 257, 40, 1300], [300, 1111, 5])):  # several pieces each, different shapes
        q, kp, vp, bt, sot, pos = _inputs(100 + call, lens, H, Hk, D, S)
        max_kv = max(lens)
        max_splits = -(-(-(-max_kv // 16)) // chunk)
        assert max_splits > 1 and len(lens) * H * max_splits * (D + 2) <= limit
        want = ops.paged_decode_attention(q, H * D, kp, vp, bt, sot, pos, 1 / math.sqrt(D), 0, H, Hk, D,
                                          len(lens), max_kv)
        got = torch.zeros_like(want)
        gc.collect()   # garbage of earlier tests must not be freed between the two readings
        torch.cuda.synchronize()
        before = torch.cuda.memory_allocated()
        rc = fn(q.data_ptr(), H * D, kp.data_ptr(), vp.data_ptr(), bt.data_ptr(), bt.shape[1], None,
                sot.data_ptr(), pos.data_ptr(), max_splits, got.data_ptr(), H * D, 1 / math.sqrt(D), 0,
                len(lens), H, Hk, D, S, chunk, stream)
        torch.cuda.synchronize()
        assert rc == 0, "call %d returned %d" % (call, rc)
        assert torch.cuda.memory_allocated() <= before, "the entry point made torch allocate"
        assert torch.isfinite(got.float()).all()
        # the tolerance of the kernel tests (2^-7 of the row's largest value + 2^-10); in fact the two are the same kernels
        bound = 2.0 ** -7 * want.float().abs().max(dim=1, keepdim=True).values + 2.0 ** -10
        assert ((got.float() - want.float()).abs() <= bound).all(), "call %d" % call
        assert torch.equal(got, want)

    # beyond the built-in scratch: refused with the limit's code, nothing written
    q, kp, vp, bt, sot, pos = _inputs(7, [50], H, Hk, D, S)
    out = torch.zeros(1, H * D, dtype=torch.bfloat16, device=DEV)
    too_many_splits = limit // (H * (D + 2)) + 1
    rc = fn(q.data_ptr(), H * D, kp.data_ptr(), vp.data_ptr(), bt.data_ptr(), bt.shape[1], None, sot.data_ptr(),
            pos.data_ptr(), too_many_splits, out.data_ptr(), H * D, 0.1, 0, 1, H, Hk, D, S, chunk, stream)
    torch.cuda.synchronize()
    assert rc == -4 and (out == 0).all()
