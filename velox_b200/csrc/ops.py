"""Python face of the kernel library: one function per C entry point.

The library is compiled on first use (`build.build`) and loaded with ctypes.
There is no other implementation behind these functions: if the library cannot
be built or loaded, or a kernel refuses a size, the call raises.  Every function
launches on torch's current CUDA stream and takes torch tensors only as holders
of device memory.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import c_float, c_int, c_void_p
from typing import Optional

import torch

from . import build as _build

_LIB = None

VX_F32, VX_BF16 = 0, 1
ACTIVATIONS = {"silu": 0, "gelu": 1, "gelu_pytorch_tanh": 2, "relu": 3}
_ERRORS = {
    -1: "a size the kernel does not take",
    -2: "an element type the kernel does not know",
    -3: "a pointer or stride that is not aligned as the kernel needs",
    -4: "a size beyond the kernel's stated maximum",
    -5: "the device or driver lacks what the kernel needs",
}


class KernelError(RuntimeError):
    pass


def library():
    """The loaded kernel library; built first if needed.  Raises if it cannot be had."""
    global _LIB
    if _LIB is None:
        path = _build.build()
        try:
            _LIB = ctypes.CDLL(path)
        except OSError as e:
            raise KernelError("the kernel library %s could not be loaded: %s" % (path, e))
        _declare(_LIB)
        if os.environ.get("VELOX_B200_PDL", "1") == "0":
            _LIB.vx_set_pdl(0)
        if os.environ.get("VELOX_B200_PDL_MASK"):
            _LIB.vx_set_pdl_mask(int(os.environ["VELOX_B200_PDL_MASK"], 0))
    return _LIB


def set_pdl(enabled: bool) -> None:
    """Programmatic dependent launch on or off for kernels launched from now on
    (on by default; VELOX_B200_PDL=0 in the environment starts with it off)."""
    library().vx_set_pdl(1 if enabled else 0)


def is_loaded() -> bool:
    return _LIB is not None


def _declare(lib) -> None:
    P, I, F = c_void_p, c_int, c_float
    sigs = {
        "vx_embedding": [P, P, P, I, I, I, I, P],
        "vx_add_rmsnorm": [P, P, P, P, P, P, I, I, F, I, P],
        "vx_rmsnorm": [P, P, P, I, I, F, I, P],
        "vx_gated_act": [P, P, I, I, I, I, I, I, P],
        "vx_add_bias": [P, P, P, I, I, I, P],
        "vx_qk_norm_rope_kv": [P, I, P, P, F, P, I, P, P, P, P, I, I, I, I, I, I, P],
        "vx_paged_attention_generic": [P, I, P, P, P, I, P, P, P, I, F, I, I, I, I, I, I, I, P],
        "vx_gemm_nt_simt": [P, P, P, P, I, I, I, I, I, I, I, I, P],
        "vx_gemm_tcgen05": [P, P, P, P, I, I, I, I, I, I, I, I, I, P, P],
        "vx_gemm_tcgen05_pair": [P, P, P, P, I, I, I, I, I, I, I, I, P, P],
        "vx_gemm_skinny": [P, P, P, P, I, I, I, I, I, I, I, I, I, I, P],
        "vx_paged_prefill_attention_tc": [P, I, I, P, P, I, P, I, P, P, P, P, I, F, I, I, I, I, I, I, I, P, I, P, P],
        "vx_paged_prefill_attention": [P, I, P, P, P, I, P, P, P, P, I, F, I, I, I, I, I, I, I, P],
        "vx_paged_decode_attention": [P, I, P, P, P, I, P, P, P, P, I, P, I, F, I, I, I, I, I, I, I, I, P],
        "vx_sample": [P, I, I, I, P, P, P, P, P],
    }
    lib.vx_set_pdl_mask.argtypes = [I]
    lib.vx_set_pdl_mask.restype = None
    lib.vx_set_pdl.argtypes = [I]
    lib.vx_set_pdl.restype = None
    for name, args in sigs.items():
        fn = getattr(lib, name)
        fn.argtypes = args
        fn.restype = c_int


_LAUNCHES = 0


def launch_count() -> int:
    """Calls of this library's kernels so far (library matrix products are not counted)."""
    return _LAUNCHES


def add_launches(n: int) -> None:
    """Kernels launched by replaying a captured graph (counted at capture)."""
    global _LAUNCHES
    _LAUNCHES += n


def _check(code: int, what: str) -> None:
    global _LAUNCHES
    _LAUNCHES += 1
    if code == 0:
        return
    if code < 0:
        raise KernelError("%s refused: %s (code %d)" % (what, _ERRORS.get(code, "unknown"), code))
    raise KernelError("%s: CUDA error %d at launch" % (what, code))


def _ptr(t: Optional[torch.Tensor]):
    return None if t is None else t.data_ptr()


_RAW_STREAM = getattr(torch._C, "_cuda_getCurrentRawStream", None)
_GET_DEVICE = getattr(torch._C, "_cuda_getDevice", None)


def _stream():
    """The current stream's handle (the capture stream while a graph is recorded).
    Asked of torch's C layer directly: the Python route costs 15 microseconds a call,
    and every kernel launch asks."""
    if _RAW_STREAM is not None and _GET_DEVICE is not None:
        return _RAW_STREAM(_GET_DEVICE())
    return torch.cuda.current_stream().cuda_stream


def dtype_code(dtype: torch.dtype) -> int:
    if dtype == torch.float32:
        return VX_F32
    if dtype == torch.bfloat16:
        return VX_BF16
    raise KernelError("element type %s has no kernels (float32 and bfloat16 have)" % dtype)


def _need(cond: bool, msg: str) -> None:
    if not cond:
        raise KernelError(msg)


def _dev(*tensors) -> None:
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise KernelError("kernels take CUDA tensors; got one on %s" % t.device)


# ----------------------------------------------------------------------------
def embedding(ids: torch.Tensor, table: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """float32 rows of `table` [V,E] at int32 `ids` [T]."""
    _dev(ids, table)
    _need(ids.dtype == torch.int32 and ids.is_contiguous() and table.is_contiguous(), "embedding: int32 ids, contiguous")
    t, (v, e) = ids.numel(), table.shape
    if out is None:
        out = torch.empty((t, e), dtype=torch.float32, device=table.device)
    _check(library().vx_embedding(_ptr(ids), _ptr(table), _ptr(out), t, e, v, dtype_code(table.dtype), _stream()),
           "embedding")
    return out


def add_rmsnorm(residual: torch.Tensor, delta: Optional[torch.Tensor], weight: torch.Tensor, eps: float,
                out_dtype: torch.dtype, rows: Optional[torch.Tensor] = None,
                residual_out: Optional[torch.Tensor] = None, update_residual: bool = True) -> torch.Tensor:
    """normed = rmsnorm(residual (+ delta)) rounded to `out_dtype`.

    With a delta, the residual must be older than the delta: not something the
    kernel launched just before this one writes (the kernel reads it before it
    waits for that kernel; in a decoder the delta is computed from the residual,
    so this holds by itself).

    Without `rows` the sum is written back into `residual` (if there is a delta
    and `update_residual`).  With `rows` (int32 indices) only those rows are
    read, and the sums go to `residual_out` if given."""
    _dev(residual, delta, weight, rows)
    _need(residual.dtype == torch.float32 and residual.is_contiguous(), "add_rmsnorm: float32 contiguous residual")
    _need(weight.dtype == torch.float32, "add_rmsnorm: float32 weight")
    width = residual.shape[-1]
    _need(weight.numel() == width, "add_rmsnorm: weight has %d elements, rows %d" % (weight.numel(), width))
    if delta is not None:
        _need(delta.dtype == out_dtype and delta.is_contiguous() and delta.shape == residual.shape,
              "add_rmsnorm: delta must match the residual's shape and the output's element type")
    n = residual.shape[0] if rows is None else rows.numel()
    out = torch.empty((n, width), dtype=out_dtype, device=residual.device)
    if rows is None:
        res_out = residual if (delta is not None and update_residual) else None
    else:
        _need(rows.dtype == torch.int32, "add_rmsnorm: int32 rows")
        res_out = residual_out
    _check(library().vx_add_rmsnorm(_ptr(residual), _ptr(delta), _ptr(rows), _ptr(res_out), _ptr(weight), _ptr(out),
                                    n, width, float(eps), dtype_code(out_dtype), _stream()), "add_rmsnorm")
    return out


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    _dev(x, weight)
    _need(x.is_contiguous() and weight.dtype == torch.float32, "rmsnorm: contiguous input, float32 weight")
    width = x.shape[-1]
    _need(weight.numel() == width, "rmsnorm: weight has %d elements, rows %d" % (weight.numel(), width))
    out = torch.empty_like(x)
    _check(library().vx_rmsnorm(_ptr(x), _ptr(weight), _ptr(out), x.numel() // width, width, float(eps),
                                dtype_code(x.dtype), _stream()), "rmsnorm")
    return out


def gated_act(gate_up: torch.Tensor, activation: str, block: int = 0,
              out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
    """act(gate) * up.  block == 0: rows are [all gates | all ups]; block > 0: rows
    are tiles of `block` gates followed by their `block` ups.  float32 input may give a
    bfloat16 result (`out_dtype`)."""
    _dev(gate_up)
    _need(gate_up.is_contiguous() and gate_up.shape[-1] % 2 == 0, "gated_act: contiguous rows of even width")
    _need(activation in ACTIVATIONS, "gated_act: activation %r is not one of %s" % (activation, sorted(ACTIVATIONS)))
    rows, inner = gate_up.shape[0], gate_up.shape[-1] // 2
    out = torch.empty((rows, inner), dtype=out_dtype or gate_up.dtype, device=gate_up.device)
    _check(library().vx_gated_act(_ptr(gate_up), _ptr(out), rows, inner, ACTIVATIONS[activation], int(block),
                                  dtype_code(gate_up.dtype), dtype_code(out.dtype), _stream()), "gated_act")
    return out


def qk_norm_rope_kv(qkv: torch.Tensor, q_weight, k_weight, eps: float, inv_freq, rot_dim: int,
                    positions: torch.Tensor, slot_mapping, k_pool, v_pool, num_heads: int, num_kv_heads: int,
                    head_dim: int) -> None:
    """In place on the packed projections `qkv` [T, (H+2Hk)D]; writes new keys
    and values into the pools [pages, Hk, S, D] when a slot mapping is given."""
    _dev(qkv, q_weight, k_weight, inv_freq, positions, slot_mapping, k_pool, v_pool)
    _need(qkv.is_contiguous() and positions.dtype == torch.int32, "qk_norm_rope_kv: contiguous qkv, int32 positions")
    page_size = 1
    if slot_mapping is not None:
        _need(k_pool is not None and v_pool is not None and k_pool.dtype == qkv.dtype and k_pool.is_contiguous()
              and v_pool.is_contiguous(), "qk_norm_rope_kv: pools of the activations' element type")
        _need(tuple(k_pool.shape[1:]) == (num_kv_heads, k_pool.shape[2], head_dim), "qk_norm_rope_kv: pool shape")
        page_size = k_pool.shape[2]
    if inv_freq is not None:
        _need(inv_freq.dtype == torch.float32 and inv_freq.numel() * 2 == rot_dim, "qk_norm_rope_kv: inv_freq size")
    for w in (q_weight, k_weight):
        if w is not None:
            _need(w.dtype == torch.float32 and w.numel() == head_dim, "qk_norm_rope_kv: norm weight size")
    _check(library().vx_qk_norm_rope_kv(
        _ptr(qkv), qkv.shape[-1], _ptr(q_weight), _ptr(k_weight), float(eps), _ptr(inv_freq), int(rot_dim),
        _ptr(positions), _ptr(slot_mapping), _ptr(k_pool), _ptr(v_pool), qkv.shape[0], num_heads, num_kv_heads,
        head_dim, page_size, dtype_code(qkv.dtype), _stream()), "qk_norm_rope_kv")


ATTENTION_MAX_HEAD_DIM = 256


def attention_head_dim_supported(head_dim: int) -> bool:
    """Head sizes some attention kernel of the library takes: even ones up to 256 (the general
    kernel; the tensor-core kernels take 64 and 128)."""
    return 0 < head_dim <= ATTENTION_MAX_HEAD_DIM and head_dim % 2 == 0


def paged_attention_generic(q: torch.Tensor, q_row_stride: int, k_pool, v_pool, block_table: torch.Tensor,
                            seq_of_token, positions, scale: float, window: int, num_heads: int,
                            num_kv_heads: int, head_dim: int, tokens: int) -> torch.Tensor:
    _dev(q, k_pool, v_pool, block_table, seq_of_token, positions)
    _need(block_table.dtype == torch.int32 and block_table.is_contiguous() and block_table.dim() == 2,
          "paged_attention: int32 block table [requests, blocks]")
    _need(k_pool.dtype == q.dtype and v_pool.dtype == q.dtype, "paged_attention: pools of the queries' element type")
    _need(attention_head_dim_supported(head_dim),
          "paged_attention: head size %d (the kernels take even sizes up to %d)" % (head_dim, ATTENTION_MAX_HEAD_DIM))
    out = torch.empty((tokens, num_heads * head_dim), dtype=q.dtype, device=q.device)
    _check(library().vx_paged_attention_generic(
        _ptr(q), q_row_stride, _ptr(k_pool), _ptr(v_pool), _ptr(block_table), block_table.shape[1],
        _ptr(seq_of_token), _ptr(positions), _ptr(out), num_heads * head_dim, float(scale), int(window), tokens,
        num_heads, num_kv_heads, head_dim, k_pool.shape[2], dtype_code(q.dtype), _stream()), "paged_attention_generic")
    return out


DECODE_CHUNK_TILES = 16  # keys per piece of the split decode kernel: 16 tiles of 16
_WORKSPACE = {}


def workspace(device, nfloats: int, which: str = "decode") -> torch.Tensor:
    """A float32 scratch buffer of at least `nfloats` on `device`, kept between calls
    (one per use: `which`).  While a CUDA graph is being captured the buffer is the
    graph's own."""
    if torch.cuda.is_current_stream_capturing():
        return torch.empty(max(nfloats, 1), dtype=torch.float32, device=device)
    key = (str(device), which)
    buf = _WORKSPACE.get(key)
    if buf is None or buf.numel() < nfloats:
        buf = torch.empty(max(nfloats, 1 << 16), dtype=torch.float32, device=device)
        _WORKSPACE[key] = buf
    return buf


def decode_attention_supported(dtype, head_dim: int, page_size: int, group: int) -> bool:
    return dtype == torch.bfloat16 and head_dim in (64, 128) and page_size % 16 == 0 and group <= 16


def paged_decode_attention(q: torch.Tensor, q_row_stride: int, k_pool, v_pool, block_table: torch.Tensor,
                           seq_of_token, positions, scale: float, window: int, num_heads: int, num_kv_heads: int,
                           head_dim: int, requests: int, max_kv: int, token_rows=None,
                           out: Optional[torch.Tensor] = None, out_rows: Optional[int] = None,
                           single_tokens: bool = True) -> torch.Tensor:
    """Attention of one query token per entry over its request's pages (bfloat16), the
    key range split over blocks of DECODE_CHUNK_TILES * 16 keys.  `max_kv` bounds
    every entry's number of keys (it sizes the grid and the scratch).  `token_rows`
    picks the entries' rows; `single_tokens=False` says that some of them are tokens of
    one request's portion (the kernel then waits for the step's cache writes before it
    reads any key)."""
    _dev(q, k_pool, v_pool, block_table, seq_of_token, positions, token_rows)
    _need(q.dtype == torch.bfloat16 and k_pool.dtype == torch.bfloat16 and v_pool.dtype == torch.bfloat16,
          "paged_decode_attention: bfloat16 only")
    _need(block_table.dtype == torch.int32 and block_table.is_contiguous() and block_table.dim() == 2,
          "paged_decode_attention: int32 block table [requests, blocks]")
    if out is None:
        out = torch.empty((out_rows if out_rows is not None else requests, num_heads * head_dim),
                          dtype=q.dtype, device=q.device)
    keys = max_kv if window <= 0 else min(max_kv, window + 15)
    max_splits = max(1, -(-(-(-keys // 16) + (1 if window > 0 else 0)) // DECODE_CHUNK_TILES))
    scratch = None
    if max_splits > 1:
        scratch = workspace(q.device, requests * num_heads * max_splits * (head_dim + 2))
    _check(library().vx_paged_decode_attention(
        _ptr(q), q_row_stride, _ptr(k_pool), _ptr(v_pool), _ptr(block_table), block_table.shape[1],
        _ptr(token_rows), _ptr(seq_of_token), _ptr(positions), _ptr(scratch), max_splits, _ptr(out),
        num_heads * head_dim, float(scale), int(window), requests, num_heads, num_kv_heads, head_dim,
        k_pool.shape[2], DECODE_CHUNK_TILES, 1 if single_tokens else 0, _stream()), "paged_decode_attention")
    return out


def prefill_attention_supported(dtype, head_dim: int, page_size: int) -> bool:
    return dtype == torch.bfloat16 and head_dim in (64, 128) and page_size % 16 == 0


def paged_prefill_attention(q: torch.Tensor, q_row_stride: int, k_pool, v_pool, block_table: torch.Tensor,
                            cu_seqlens, kv_offsets, scale: float, window: int, num_heads: int, num_kv_heads: int,
                            head_dim: int, requests: int, max_new: int, tokens: int, seq_list=None,
                            out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Causal attention of prompt portions over the pages (bfloat16, tensor cores):
    request i brings token rows [cu_seqlens[i], cu_seqlens[i+1]) at positions
    kv_offsets[i] onward; `max_new` bounds the tokens of any request.  With `seq_list`
    (int32, on the device) only its first `requests` entries' requests are worked on,
    and only their rows of `out` are written."""
    _dev(q, k_pool, v_pool, block_table, cu_seqlens, kv_offsets, seq_list, out)
    _need(q.dtype == torch.bfloat16 and k_pool.dtype == torch.bfloat16 and v_pool.dtype == torch.bfloat16,
          "paged_prefill_attention: bfloat16 only")
    _need(block_table.dtype == torch.int32 and block_table.is_contiguous() and block_table.dim() == 2,
          "paged_prefill_attention: int32 block table [requests, blocks]")
    if out is None:
        out = torch.empty((tokens, num_heads * head_dim), dtype=q.dtype, device=q.device)
    _check(library().vx_paged_prefill_attention(
        _ptr(q), q_row_stride, _ptr(k_pool), _ptr(v_pool), _ptr(block_table), block_table.shape[1],
        _ptr(cu_seqlens), _ptr(kv_offsets), _ptr(seq_list), _ptr(out), num_heads * head_dim, float(scale), int(window), requests,
        int(max_new), num_heads, num_kv_heads, head_dim, k_pool.shape[2], _stream()), "paged_prefill_attention")
    return out


PREFILL_MAX_SPLITS = 16


def prefill_attention_tc_supported(dtype, head_dim: int, page_size: int, group: int) -> bool:
    return dtype == torch.bfloat16 and head_dim == 128 and page_size % 16 == 0 and 1 <= group <= 8


def paged_prefill_attention_tc(q: torch.Tensor, q_row_stride: int, k_pool, v_pool, block_table: torch.Tensor,
                               cu_seqlens, kv_offsets, scale: float, window: int, num_heads: int, num_kv_heads: int,
                               head_dim: int, requests: int, max_new: int, tokens: int, seq_list=None,
                               out: Optional[torch.Tensor] = None, max_kv: int = 0) -> torch.Tensor:
    """The same as `paged_prefill_attention` on the tcgen05 tensor cores (head size
    128, accumulators in tensor memory, operands by TMA).  `max_kv` (a bound on any
    request's keys after the step) lets short portions on top of many keys be cut into
    runs of key tiles that several blocks share; 0: never."""
    _dev(q, k_pool, v_pool, block_table, cu_seqlens, kv_offsets, seq_list, out)
    _need(q.dtype == torch.bfloat16 and k_pool.dtype == torch.bfloat16 and v_pool.dtype == torch.bfloat16,
          "paged_prefill_attention_tc: bfloat16 only")
    _need(block_table.dtype == torch.int32 and block_table.is_contiguous() and block_table.dim() == 2,
          "paged_prefill_attention_tc: int32 block table [requests, blocks]")
    _need(k_pool.is_contiguous() and v_pool.is_contiguous(), "paged_prefill_attention_tc: contiguous pools")
    if out is None:
        out = torch.empty((tokens, num_heads * head_dim), dtype=q.dtype, device=q.device)
    # runs of key tiles: up to a quarter of the longest request's key tiles, 16 at most; only a step whose
    # portions are short can have a request that is cut (a long portion has query tiles enough)
    max_splits, scratch = 1, None
    toks_per_tile = (128 // (num_heads // num_kv_heads)) & ~7   # (as pt_toks_per_tile in the kernel)
    sms = _sm_count(q.device)
    if max_kv >= 8 * 128 and 2 * -(-max_new // (2 * toks_per_tile)) * num_kv_heads <= sms:   # (a block takes two query tiles)
        max_splits = max(1, min(PREFILL_MAX_SPLITS, -(-max_kv // 128) // 4, sms // num_kv_heads))
        scratch = workspace(q.device, tokens * num_heads * max_splits * (head_dim + 2), which="prefill")
    _check(library().vx_paged_prefill_attention_tc(
        _ptr(q), q_row_stride, tokens, _ptr(k_pool), _ptr(v_pool), k_pool.shape[0], _ptr(block_table),
        block_table.shape[1], _ptr(cu_seqlens), _ptr(kv_offsets), _ptr(seq_list), _ptr(out), num_heads * head_dim, float(scale),
        int(window), requests, int(max_new), num_heads, num_kv_heads, head_dim, k_pool.shape[2],
        _ptr(scratch), max_splits, _ptr(_error_word(q.device)), _stream()), "paged_prefill_attention_tc")
    note_bounded_wait()
    return out


def gemm_nt_simt(a: torch.Tensor, w: torch.Tensor, bias=None, out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
    """a [M,K] times w [N,K] transposed, float32 multiply-adds on the CUDA cores."""
    _dev(a, w, bias)
    _need(a.dim() == 2 and w.dim() == 2 and a.shape[1] == w.shape[1], "gemm: a [M,K], w [N,K]")
    _need(a.stride(1) == 1 and w.stride(1) == 1 and a.dtype == w.dtype, "gemm: rows contiguous, one element type")
    out_dtype = out_dtype or a.dtype
    m, k = a.shape
    n = w.shape[0]
    if bias is not None:
        _need(bias.dtype == torch.float32 and bias.numel() == n, "gemm: float32 bias of N elements")
    out = torch.empty((m, n), dtype=out_dtype, device=a.device)
    _check(library().vx_gemm_nt_simt(_ptr(a), _ptr(w), _ptr(bias), _ptr(out), m, n, k, a.stride(0), w.stride(0), n,
                                     dtype_code(a.dtype), dtype_code(out_dtype), _stream()), "gemm_nt_simt")
    return out


_SM_COUNTS = {}


def _sm_count(device) -> int:
    key = str(device)
    if key not in _SM_COUNTS:
        _SM_COUNTS[key] = torch.cuda.get_device_properties(device).multi_processor_count
    return _SM_COUNTS[key]


_ERROR_WORDS = {}


def _error_word(device) -> torch.Tensor:
    """The device int that kernels with bounded waits report into."""
    key = str(device)
    if key not in _ERROR_WORDS:
        _ERROR_WORDS[key] = torch.zeros(1, dtype=torch.int32, device=device)
    return _ERROR_WORDS[key]


_BOUNDED_WAIT_LAUNCHES = 0   # launches of kernels with bounded waits, ever
_BOUNDED_WAIT_CHECKED = 0    # ... at the last check of the error word


def bounded_wait_launches() -> int:
    return _BOUNDED_WAIT_LAUNCHES


def note_bounded_wait(n: int = 1) -> None:
    """A kernel whose waits are bounded was launched (by the wrappers below, or by
    the replay of a graph that holds such kernels): the error word has to be read
    before the step's results are trusted."""
    global _BOUNDED_WAIT_LAUNCHES
    _BOUNDED_WAIT_LAUNCHES += n


def bounded_wait_pending() -> bool:
    """True if a kernel with bounded waits was launched since the error word was last read."""
    return _BOUNDED_WAIT_LAUNCHES != _BOUNDED_WAIT_CHECKED


def check_pending_device_errors() -> None:
    """`check_device_errors()` if a kernel with bounded waits ran since the last check,
    else nothing (and no synchronisation).  What steps a model calls this before it
    hands out a step's results; it does not have to know which kernels a part chose."""
    if bounded_wait_pending():
        check_device_errors()


def check_device_errors() -> None:
    """Raises if a kernel has reported that one of its bounded waits ran out since
    the last check (its results are then missing).  Synchronises the device."""
    global _BOUNDED_WAIT_CHECKED
    _BOUNDED_WAIT_CHECKED = _BOUNDED_WAIT_LAUNCHES
    for key, word in _ERROR_WORDS.items():
        code = int(word.item())
        if code:
            word.zero_()
            raise KernelError("a kernel on %s gave up a wait on its asynchronous copies or tensor-core work "
                              "(code %d); its results are missing" % (key, code))


def tcgen05_supported(a: torch.Tensor, w: torch.Tensor) -> bool:
    return (a.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and a.shape[1] % 8 == 0 and w.shape[0] % 16 == 0
            and a.stride(1) == 1 and w.stride(1) == 1 and a.stride(0) % 8 == 0 and w.stride(0) % 8 == 0
            and a.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)


def tcgen05_pair_better(m: int, n: int, device) -> bool:
    """Whether 256 x 256 tiles by pairs of blocks beat 128 x 256 tiles by single blocks for
    an [m, n] result: both kinds of block spend the same time on a tile (a pair a little
    less: each SM reads half of W's tile from its shared memory), so the kind that needs
    fewer rounds of the GPU's SMs wins; padding rows count as work."""
    sms = _sm_count(device)
    cols = -(-n // 256)
    single = -(-(-(-m // 128) * cols) // sms)
    paired = -(-(-(-m // 256) * cols) // max(1, sms // 2))
    return paired * 0.97 < single


def gemm_tcgen05(a: torch.Tensor, w: torch.Tensor, bias=None, gated_activation: Optional[str] = None,
                 wide: bool = True, pair: bool = False) -> torch.Tensor:
    """a [M,K] times w [N,K] transposed on the tcgen05 tensor cores (bfloat16 in and
    out, float32 accumulation in tensor memory, operands by TMA).  With
    `gated_activation`, w's rows come in tiles of 8 gate rows followed by their 8 up
    rows and the result is act(gate) * up, [M, N/2].  `wide`: 128 x 256 tiles, else
    128 x 128; `pair`: 256 x 256 tiles, each formed by a pair of blocks."""
    _dev(a, w, bias)
    _need(a.dim() == 2 and w.dim() == 2 and a.shape[1] == w.shape[1], "gemm_tcgen05: a [M,K], w [N,K]")
    _need(tcgen05_supported(a, w), "gemm_tcgen05: bfloat16, K a multiple of 8, N a multiple of 16, 16-byte aligned rows")
    m, k = a.shape
    n = w.shape[0]
    cols = n // 2 if gated_activation else n
    if gated_activation is not None:
        _need(gated_activation in ACTIVATIONS, "gemm_tcgen05: unknown activation %r" % gated_activation)
    if bias is not None:
        _need(bias.dtype == torch.float32 and bias.numel() == n, "gemm_tcgen05: float32 bias of N elements")
    out = torch.empty((m, cols), dtype=torch.bfloat16, device=a.device)
    _need(cols % 8 == 0, "gemm_tcgen05: output rows must be 16-byte aligned")
    if pair:
        _check(library().vx_gemm_tcgen05_pair(_ptr(a), _ptr(w), _ptr(bias), _ptr(out), m, n, k, a.stride(0), w.stride(0),
                                              cols, 1 if gated_activation else 0, ACTIVATIONS.get(gated_activation, 0),
                                              _ptr(_error_word(a.device)), _stream()), "gemm_tcgen05_pair")
    else:
        _check(library().vx_gemm_tcgen05(_ptr(a), _ptr(w), _ptr(bias), _ptr(out), m, n, k, a.stride(0), w.stride(0), cols,
                                         1 if gated_activation else 0, ACTIVATIONS.get(gated_activation, 0),
                                         1 if wide else 0, _ptr(_error_word(a.device)), _stream()), "gemm_tcgen05")
    note_bounded_wait()
    return out


SKINNY_MAX_ROWS = 8
_MATMUL_SET = False


def skinny_supported(m: int, k: int, a: torch.Tensor, w: torch.Tensor) -> bool:
    return (0 < m <= SKINNY_MAX_ROWS and k % 32 == 0 and a.stride(1) == 1 and w.stride(1) == 1
            and a.stride(0) % 8 == 0 and w.stride(0) % 8 == 0 and a.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)


def gemm_skinny(a: torch.Tensor, w: torch.Tensor, bias=None, out_dtype: Optional[torch.dtype] = None,
                gated_activation: Optional[str] = None, variant: int = 0) -> torch.Tensor:
    """a [M<=8, K] times w [N,K] transposed, W streamed once (bfloat16).  With
    `gated_activation`, w's rows come in tiles of 8 gate rows followed by their 8 up
    rows and the result is act(gate) * up, [M, N/2]."""
    _dev(a, w, bias)
    _need(a.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and a.dim() == 2 and w.dim() == 2
          and a.shape[1] == w.shape[1], "gemm_skinny: bfloat16 a [M,K], w [N,K]")
    out_dtype = out_dtype or torch.bfloat16
    m, k = a.shape
    n = w.shape[0]
    cols = n // 2 if gated_activation else n
    if gated_activation is not None:
        _need(gated_activation in ACTIVATIONS, "gemm_skinny: unknown activation %r" % gated_activation)
    out = torch.empty((m, cols), dtype=out_dtype, device=a.device)
    _check(library().vx_gemm_skinny(_ptr(a), _ptr(w), _ptr(bias), _ptr(out), m, n, k, a.stride(0), w.stride(0), cols,
                                    1 if gated_activation else 0, ACTIVATIONS.get(gated_activation, 0),
                                    dtype_code(out_dtype), variant, _stream()), "gemm_skinny")
    return out


def gemm_bf16(a: torch.Tensor, w: torch.Tensor, bias=None, out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
    """a [M,K] times w [N,K] transposed on the tensor cores, float32 accumulation."""
    _dev(a, w, bias)
    _need(a.dtype == torch.bfloat16 and w.dtype == torch.bfloat16, "gemm_bf16: bfloat16 operands")
    out_dtype = out_dtype or torch.bfloat16
    if skinny_supported(a.shape[0], a.shape[1], a, w):
        return gemm_skinny(a, w, bias, out_dtype)
    # library product (cuBLAS through torch); reductions stay in float32
    global _MATMUL_SET
    if not _MATMUL_SET:
        torch.backends.cuda.matmul.allow_bf16_reduced_precision_reduction = False
        _MATMUL_SET = True
    if out_dtype == torch.float32 or bias is not None:
        out = torch.mm(a, w.t(), out_dtype=torch.float32)
    else:
        out = torch.mm(a, w.t())
    if bias is not None:
        # added to the float32 sums; the result is rounded once
        _need(bias.dtype == torch.float32 and bias.numel() == w.shape[0], "gemm_bf16: float32 bias of N elements")
        summed = out
        out = torch.empty(summed.shape, dtype=out_dtype, device=a.device)
        _check(library().vx_add_bias(_ptr(summed), _ptr(bias), _ptr(out), summed.shape[0], summed.shape[1],
                                     dtype_code(out_dtype), _stream()), "add_bias")
    return out


def sample(logits: torch.Tensor, temperature=None, top_p=None, uniform=None) -> torch.Tensor:
    """int32 token per row of float32 `logits` [R,V]; all greedy without `temperature`."""
    _dev(logits, temperature, top_p, uniform)
    _need(logits.dtype == torch.float32 and logits.dim() == 2 and logits.stride(1) == 1, "sample: float32 logits [R,V]")
    r, v = logits.shape
    for t in (temperature, top_p, uniform):
        if t is not None:
            _need(t.dtype == torch.float32 and t.numel() == r, "sample: float32 per-row parameters")
    out = torch.empty((r,), dtype=torch.int32, device=logits.device)
    _check(library().vx_sample(_ptr(logits), logits.stride(0), r, v, _ptr(temperature), _ptr(top_p), _ptr(uniform),
                               _ptr(out), _stream()), "sample")
    return out
