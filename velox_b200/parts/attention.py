"""Attention over a paged cache of keys and values: the mixer of Qwen3.

In the reference's order (src/paged/qwen3.rs:428-448, 584-642):
q/k/v projections -> RMSNorm of each q and k head over head_dim (before the
rotation, not on v) -> rotation at position kv_offset + t -> new k (normed,
rotated) and v (raw) written into the pages -> causal attention over the
request's pages, scale 1/sqrt(head_dim), grouped heads -> output projection
whose input width is heads * head_dim.  The three projections are one matrix
here ([Wq; Wk; Wv], rows in that order), which the reference keeps apart
(src/paged/qwen3.rs:428-430).

Everything is a parameter: head counts, head size, whether q/k are normed,
whether projections are biased, the window (0: all keys), the scale, and the
position encoding (a `PartSpec` of category "position").
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch

from ..csrc import ops
from .base import Mixer, PagedKV, Runtime, TensorSpec
from .linear import Linear
from .plan import PartSpec
from .registry import build_part


TC_PREFILL_MIN_TOKENS = 32   # longest portion of a step from which the tcgen05 kernel is used


class PagedAttention(Mixer):
    # Requests that bring fewer tokens than the tcgen05 kernel's shortest portion are listed token by
    # token in the step's description (`single_rows`): every token goes to the decode kernel as a query
    # of its own, its request's keys cut into pieces of 256 that many warps share.  A prompt kernel gives
    # such a portion one block per kv head that walks ALL the request's keys alone: 16 tokens on top of
    # 4,000 cached keys took 300 us a layer that way.
    short_rows_up_to = TC_PREFILL_MIN_TOKENS - 1

    @property
    def cuda_graph_safe(self) -> bool:
        # reads nothing of a step but device tensors and sizes fixed per graph; a position
        # encoding of its own kind has to say the same of itself
        return self.position is None or bool(self.position.cuda_graph_safe)

    def __init__(self, prefix: str, hidden_size: int, num_heads: int, num_kv_heads: int, head_dim: int,
                 bias: bool = False, qk_norm: bool = True, eps: float = 1e-6, window: int = 0,
                 position: Optional[PartSpec] = None, scale: Optional[float] = None):
        super().__init__(prefix)
        if num_heads % num_kv_heads:
            raise ValueError("num_heads %d is not a multiple of num_kv_heads %d" % (num_heads, num_kv_heads))
        if not ops.attention_head_dim_supported(int(head_dim)):
            raise ValueError("%shead_dim %d: the attention kernels take even head sizes up to %d"
                             % (prefix, head_dim, ops.ATTENTION_MAX_HEAD_DIM))
        self.hidden_size, self.num_heads, self.num_kv_heads = int(hidden_size), int(num_heads), int(num_kv_heads)
        self.head_dim, self.bias, self.qk_norm = int(head_dim), bool(bias), bool(qk_norm)
        self.eps, self.window = float(eps), int(window)
        self.scale = float(scale) if scale is not None else 1.0 / math.sqrt(self.head_dim)
        self.position = build_part("position", position) if position is not None else None
        self.qkv: Optional[Linear] = None
        self.out: Optional[Linear] = None
        self.q_norm_weight = self.k_norm_weight = None

    # -- weights -------------------------------------------------------------
    def _proj_rows(self):
        d = self.head_dim
        return {"q_proj": self.num_heads * d, "k_proj": self.num_kv_heads * d, "v_proj": self.num_kv_heads * d}

    def tensor_specs(self) -> List[TensorSpec]:
        p, specs = self.prefix, []
        for name, rows in self._proj_rows().items():
            specs.append(TensorSpec(p + name + ".weight", (rows, self.hidden_size), "matrix"))
            if self.bias:
                specs.append(TensorSpec(p + name + ".bias", (rows,), "bias"))
        specs.append(TensorSpec(p + "o_proj.weight", (self.hidden_size, self.num_heads * self.head_dim), "matrix"))
        if self.bias:
            specs.append(TensorSpec(p + "o_proj.bias", (self.hidden_size,), "bias"))
        if self.qk_norm:
            specs.append(TensorSpec(p + "q_norm.weight", (self.head_dim,), "norm"))
            specs.append(TensorSpec(p + "k_norm.weight", (self.head_dim,), "norm"))
        if self.position is not None:
            specs.extend(self.position.tensor_specs())
        return specs

    def ignored_tensors(self) -> List[str]:
        return self.position.ignored_tensors() if self.position is not None else []

    def bind(self, tensors: Dict[str, torch.Tensor], runtime: Runtime) -> None:
        super().bind(tensors, runtime)
        p = self.prefix
        w = torch.cat([tensors[p + n + ".weight"] for n in ("q_proj", "k_proj", "v_proj")], dim=0).contiguous()
        b = torch.cat([tensors[p + n + ".bias"] for n in ("q_proj", "k_proj", "v_proj")]).contiguous() if self.bias else None
        self.qkv = Linear(w, b)
        self.out = Linear(tensors[p + "o_proj.weight"], tensors[p + "o_proj.bias"] if self.bias else None)
        if self.qk_norm:
            self.q_norm_weight, self.k_norm_weight = tensors[p + "q_norm.weight"], tensors[p + "k_norm.weight"]
        if self.position is not None:
            self.position.bind(tensors, runtime)

    # -- cache ---------------------------------------------------------------
    def cache_spec(self):
        return PagedKV(self.num_kv_heads, self.head_dim, self.window)

    # -- step ----------------------------------------------------------------
    def forward(self, h: torch.Tensor, ctx, cache) -> torch.Tensor:
        H, Hk, D = self.num_heads, self.num_kv_heads, self.head_dim
        group = ctx.groups[cache.group]
        qkv = self.qkv(h)
        slots = group.slot_mapping if cache.writes else None
        rotary = self.position.rotary_table(h.device) if self.position is not None else None
        qw, kw = self.q_norm_weight, self.k_norm_weight
        if self.position is None or rotary is not None:
            inv_freq, rot = rotary if rotary is not None else (None, 0)
            ops.qk_norm_rope_kv(qkv, qw, kw, self.eps, inv_freq, rot, ctx.positions, slots,
                                cache.k_pool, cache.v_pool, H, Hk, D)
        else:
            # An encoding the fused kernel does not know: norm in place, let the
            # part encode q and k in place, then write the cache.
            t = qkv.shape[0]
            ops.qk_norm_rope_kv(qkv, qw, kw, self.eps, None, 0, ctx.positions, None, None, None, H, Hk, D)
            q, k = qkv[:, : H * D].view(t, H, D), qkv[:, H * D : (H + Hk) * D].view(t, Hk, D)
            q2, k2 = self.position.apply(q, k, ctx.positions)
            if q2 is not q:
                q.copy_(q2)
            if k2 is not k:
                k.copy_(k2)
            ops.qk_norm_rope_kv(qkv, None, None, self.eps, None, 0, ctx.positions, slots,
                                cache.k_pool, cache.v_pool, H, Hk, D)
        attn = self._attend(qkv, ctx, cache, group)
        return self.out(attn)

    def _attend(self, qkv, ctx, cache, group) -> torch.Tensor:
        H, Hk, D = self.num_heads, self.num_kv_heads, self.head_dim
        if ctx.decode_only and ops.decode_attention_supported(qkv.dtype, D, cache.k_pool.shape[2], H // Hk):
            # one token per request: token row i is request i
            return ops.paged_decode_attention(qkv, qkv.shape[1], cache.k_pool, cache.v_pool, group.block_table,
                                              ctx.seq_of_token, ctx.positions, self.scale, self.window, H, Hk, D,
                                              ctx.n_seqs, ctx.max_kv)
        page = cache.k_pool.shape[2]
        use_tc = ctx.max_new >= TC_PREFILL_MIN_TOKENS and ops.prefill_attention_tc_supported(qkv.dtype, D, page, H // Hk)
        if use_tc or ops.prefill_attention_supported(qkv.dtype, D, page):
            prefill = ops.paged_prefill_attention_tc if use_tc else ops.paged_prefill_attention  # tcgen05 | mma.sync
            out, seqs, n = None, None, ctx.n_seqs
            if ctx.n_single and ops.decode_attention_supported(qkv.dtype, D, page, H // Hk):
                # A mixed step: the tokens of requests that bring one token, or a few, go to the
                # decode kernel (a warp per 256 keys), not into a query tile of their own; the
                # kernels write disjoint rows.  A decoded token's result is then the same bits
                # whether or not prompt portions ride in its step.
                out = torch.empty((qkv.shape[0], H * D), dtype=qkv.dtype, device=qkv.device)
                ops.paged_decode_attention(qkv, qkv.shape[1], cache.k_pool, cache.v_pool, group.block_table,
                                           ctx.seq_of_token, ctx.positions, self.scale, self.window, H, Hk, D,
                                           ctx.n_single, ctx.max_kv_single, token_rows=ctx.single_rows, out=out,
                                           single_tokens=ctx.max_short <= 1)
                if ctx.n_portions == 0:
                    return out
                seqs, n = ctx.portion_seqs, ctx.n_portions
            more = dict(max_kv=ctx.max_kv) if use_tc else {}   # (short portions on many keys: cut into runs of key tiles)
            return prefill(qkv, qkv.shape[1], cache.k_pool, cache.v_pool, group.block_table, ctx.cu_seqlens,
                           ctx.kv_offsets, self.scale, self.window, H, Hk, D, n, ctx.max_new, qkv.shape[0],
                           seq_list=seqs, out=out, **more)
        return ops.paged_attention_generic(qkv, qkv.shape[1], cache.k_pool, cache.v_pool, group.block_table,
                                           ctx.seq_of_token, ctx.positions, self.scale, self.window, H, Hk, D,
                                           qkv.shape[0])
