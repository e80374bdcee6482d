"""Arrangements and kinds that the framework itself does not have, defined here,
registered, built and stepped without a change to the framework's files:

  * a block with four norms (one before and one after each sublayer), a block with a
    single norm shared by a mixer and a feed-forward that run side by side, and a
    block without a feed-forward;
  * an embedding that adds a learned vector per position at the input (it reads the
    step's positions, not only its token ids);
  * a mixer whose cache is neither a key/value pair nor a fixed-size state: one latent
    vector per position, kept in pages through a cache kind registered here.

They live in a toy architecture beside the framework's own attention, feed-forward,
norm and head.  Nothing of it is a model of anyone's."""
from dataclasses import dataclass
from typing import ClassVar

import numpy as np
import pytest
import torch

import plain_qwen3 as P

pytestmark = pytest.mark.gpu
E, INNER, LATENT, VOCAB, MAXPOS, EPS = 48, 64, 12, 110, 96, 1e-5


def register_toy():
    from velox_b200.cache import CacheKind, LayerCache, register_cache_kind
    from velox_b200.config import ModelConfig, register_architecture
    from velox_b200.config.model_config import _field
    from velox_b200.parts import (Block, Embedding, LayerSpec, Mixer, ModelPlan, PartSpec, TensorSpec, matmul,
                                  register_block, register_mixer, register_part)

    class SandwichBlock(Block):
        """x += post_mixer(mixer(pre_mixer(x))); x += post_ff(ff(pre_ff(x)))."""
        norm_names = ("pre_mixer", "post_mixer", "pre_ff", "post_ff")

        def forward(self, residual, delta, ctx, cache):
            h = self.norms["pre_mixer"].add_norm(residual, delta)
            a = self.norms["post_mixer"].forward(self.mixer.forward(h, ctx, cache))
            h = self.norms["pre_ff"].add_norm(residual, a)
            return residual, self.norms["post_ff"].forward(self.feed_forward.forward(h, ctx))

    class ParallelBlock(Block):
        """h = norm(x); x += mixer(h) + ff(h)."""
        norm_names = ("shared",)

        def forward(self, residual, delta, ctx, cache):
            h = self.norms["shared"].add_norm(residual, delta)
            return residual, self.mixer.forward(h, ctx, cache) + self.feed_forward.forward(h, ctx)

    class MixerOnlyBlock(Block):
        norm_names = ("mixer",)
        needs_feed_forward = False

        def forward(self, residual, delta, ctx, cache):
            return residual, self.mixer.forward(self.norms["mixer"].add_norm(residual, delta), ctx, cache)

    class PositionalEmbedding(Embedding):
        """x[t] = tokens[id[t]] + places[position[t]]: a position encoding at the input."""

        def __init__(self, prefix, vocab_size, hidden_size, max_positions):
            super().__init__(prefix)
            self.vocab_size, self.hidden_size, self.max_positions = vocab_size, hidden_size, max_positions

        def tensor_specs(self):
            return [TensorSpec(self.prefix + "tokens", (self.vocab_size, self.hidden_size), "table"),
                    TensorSpec(self.prefix + "places", (self.max_positions, self.hidden_size), "table")]

        def bind(self, tensors, runtime):
            super().bind(tensors, runtime)
            self.tokens, self.places = tensors[self.prefix + "tokens"], tensors[self.prefix + "places"]

        def forward(self, ctx):
            return self.tokens[ctx.token_ids.long()].float() + self.places[ctx.positions.long()].float()

    @dataclass(frozen=True)
    class PagedLatent:
        """One vector of `width` numbers per position, in pages."""
        width: int

    class PagedLatentKind(CacheKind):
        def page_bytes(self, spec, page_size, element_bytes):
            return spec.width * page_size * element_bytes

        def allocate(self, spec, layers, num_pages, page_size, dtype, device):
            return torch.empty((layers, num_pages, page_size, spec.width), dtype=dtype, device=device)

        def layer_cache(self, storage, index, group):
            return LayerCache(group, True, pages=None if storage is None else storage[index])

    class LatentAttention(Mixer):
        """Caches c = h Wc per position; keys and values are made from the cached latents
        (k = c Wk, v = c Wv), one head, causal; out = softmax(q k^T / sqrt(r)) v Wo."""

        def __init__(self, prefix, hidden_size, latent):
            super().__init__(prefix)
            self.hidden_size, self.latent = hidden_size, latent

        def tensor_specs(self):
            p, e, r = self.prefix, self.hidden_size, self.latent
            return [TensorSpec(p + "c.weight", (r, e)), TensorSpec(p + "q.weight", (r, e)),
                    TensorSpec(p + "k.weight", (r, r)), TensorSpec(p + "v.weight", (r, r)),
                    TensorSpec(p + "o.weight", (e, r))]

        def bind(self, tensors, runtime):
            super().bind(tensors, runtime)
            self.w = {n: tensors[self.prefix + n + ".weight"] for n in "cqkvo"}

        def cache_spec(self):
            return PagedLatent(self.latent)

        def forward(self, h, ctx, cache):
            g, r = ctx.groups[cache.group], self.latent
            c, q = matmul(h, self.w["c"]), matmul(h, self.w["q"])
            cache.pages.view(-1, r)[g.slot_mapping.long()] = c          # the new latents, into their pages
            page = cache.pages.shape[1]
            out = torch.empty_like(q)
            row = 0
            for i, (n, off) in enumerate(zip(ctx.new_lens, ctx.offsets)):   # (a toy: per request, on the host)
                held = off + n
                table = g.block_table[i, : -(-held // page)].long()
                lat = cache.pages[table].reshape(-1, r)[:held]
                k, v = matmul(lat, self.w["k"]).float(), matmul(lat, self.w["v"]).float()
                s = q[row:row + n].float() @ k.t() / r ** 0.5
                seen = torch.arange(held, device=h.device)[None, :] <= (off + torch.arange(n, device=h.device))[:, None]
                out[row:row + n] = (torch.softmax(s.masked_fill(~seen, float("-inf")), -1) @ v).to(h.dtype)
                row += n
            return matmul(out, self.w["o"])

    @dataclass(frozen=True)
    class ToyConfig(ModelConfig):
        architecture: ClassVar[str] = "ToyBlocksLM"
        model_type: ClassVar[str] = "toy_blocks"
        vocab_size: int = _field(int)

    def plan(cfg):
        norm = lambda p: PartSpec("rms_norm", p, dict(size=E, eps=EPS))
        ff = lambda p: PartSpec("gated_mlp", p, dict(hidden_size=E, intermediate_size=INNER))
        att = lambda p: PartSpec("paged_attention", p, dict(
            hidden_size=E, num_heads=2, num_kv_heads=1, head_dim=16, qk_norm=False, eps=EPS,
            position=PartSpec("none", "", {})))
        layers = [
            LayerSpec(att("toy.0.a."), ff("toy.0.ff."), {n: norm("toy.0.%s." % n) for n in SandwichBlock.norm_names},
                      block="toy_sandwich"),
            LayerSpec(att("toy.1.a."), ff("toy.1.ff."), {"shared": norm("toy.1.shared.")}, block="toy_parallel"),
            LayerSpec(PartSpec("toy_latent_attention", "toy.2.m.", dict(hidden_size=E, latent=LATENT)), None,
                      {"mixer": norm("toy.2.n.")}, block="toy_mixer_only"),
        ]
        return ModelPlan(cfg.vocab_size, E,
                         PartSpec("toy_positional_embedding", "toy.embed.",
                                  dict(vocab_size=cfg.vocab_size, hidden_size=E, max_positions=MAXPOS)),
                         layers, norm("toy.norm."),
                         PartSpec("linear_head", "toy.head.", dict(vocab_size=cfg.vocab_size, hidden_size=E)),
                         order=[0, 1, 2], max_positions=MAXPOS)

    register_block("toy_sandwich", SandwichBlock)
    register_block("toy_parallel", ParallelBlock)
    register_block("toy_mixer_only", MixerOnlyBlock)
    register_part("embedding", "toy_positional_embedding", PositionalEmbedding)
    register_mixer("toy_latent_attention", LatentAttention)
    register_cache_kind(PagedLatent, PagedLatentKind())
    register_architecture("ToyBlocksLM", "toy_blocks", ToyConfig, plan)
    return ToyConfig, PagedLatent


def plain_toy(w, ids):
    """The toy model on a whole sequence, in numpy."""
    T = len(ids)
    norm = lambda x, name: P.rms_norm(x, w[name + "weight"], EPS)
    mlp = lambda h, p: P.gated_mlp(h, w[p + "gate_proj.weight"], w[p + "up_proj.weight"], w[p + "down_proj.weight"])

    def att(h, p):
        q = (h @ w[p + "q_proj.weight"].T).reshape(T, 2, 16)
        k = (h @ w[p + "k_proj.weight"].T).reshape(T, 1, 16)
        v = (h @ w[p + "v_proj.weight"].T).reshape(T, 1, 16)
        return P.causal_attention(q, k, v).reshape(T, 32) @ w[p + "o_proj.weight"].T

    x = w["toy.embed.tokens"][ids] + w["toy.embed.places"][:T]
    x = x + norm(att(norm(x, "toy.0.pre_mixer."), "toy.0.a."), "toy.0.post_mixer.")
    x = x + norm(mlp(norm(x, "toy.0.pre_ff."), "toy.0.ff."), "toy.0.post_ff.")
    h = norm(x, "toy.1.shared.")
    x = x + att(h, "toy.1.a.") + mlp(h, "toy.1.ff.")
    h = norm(x, "toy.2.n.")
    m = "toy.2.m."
    c = h @ w[m + "c.weight"].T
    q, k, v = h @ w[m + "q.weight"].T, c @ w[m + "k.weight"].T, c @ w[m + "v.weight"].T
    a = P.causal_attention(q[:, None, :], k[:, None, :], v[:, None, :])[:, 0, :]   # (scores over sqrt(r))
    x = x + a @ w[m + "o.weight"].T
    return norm(x, "toy.norm.") @ w["toy.head.weight"].T


def test_toy_blocks_input_positions_and_latent_cache_run_in_the_engine(tmp_path):
    from velox_b200 import Engine, EngineConfig, SamplingParams
    from velox_b200.cache import unregister_cache_kind
    from velox_b200.config import unregister_architecture
    from velox_b200.engine import StepEntry
    from velox_b200.parts import LayerSpec, PartSpec, unregister_part
    from velox_b200.parts.registry import part_class
    from velox_b200.weights import write_random_model
    from velox_b200.weights.safetensors_io import SafetensorsFile, write_safetensors
    import os

    ToyConfig, PagedLatent = register_toy()
    try:
        cfg = ToyConfig.from_dict(dict(vocab_size=VOCAB))
        folder = write_random_model(str(tmp_path / "toy"), cfg, seed=9)
        # let the places and the latent path matter: random weights of 0.02 would leave both near nothing
        path = os.path.join(folder, "model.safetensors")
        f = SafetensorsFile(path)
        tensors, meta = {name: f.tensor(name).clone() for name in f.keys()}, dict(f.metadata)
        f.close()
        for name in list(tensors):
            if name.endswith("embed.places") or ".2.m." in name:
                tensors[name] = tensors[name] * 20
        write_safetensors(path, tensors, meta)
        raw, w = P.load_model_folder(folder)
        engine = Engine(folder, EngineConfig(dtype="float32", page_size=8, num_pages=12, max_model_len=MAXPOS,
                                             max_running_requests=3))
        # two groups of pages: keys and values (layers 0 and 1), latents (layer 2), each with storage of its kind
        kinds = [type(g.spec).__name__ for g in engine.cache.groups]
        assert kinds == ["PagedKV", "PagedLatent"] and engine.cache.groups[0].layers == [0, 1]
        assert tuple(engine.cache.groups[1].storage.shape) == (1, 12, 8, LATENT)
        assert engine.cache.layer(2).pages is not None and engine.cache.layer(2).k_pool is None
        assert len(engine.model.blocks[0].parts()) == 6 and len(engine.model.blocks[2].parts()) == 2
        ids = [int(t) for t in np.random.default_rng(4).integers(0, VOCAB, 41)]
        other = [int(t) for t in np.random.default_rng(5).integers(0, VOCAB, 30)]
        want, want_other = plain_toy(w, ids), plain_toy(w, other)
        assert np.abs(plain_toy(w, ids[1:])[:-1] - want[1:-1]).max() > 1e-3, "the positions at the input do not matter"
        engine.cache.add_request("whole")
        got = engine.run_step([StepEntry("whole", ids, list(range(41)))]).cpu().numpy()
        assert np.abs(got - want).max() < 1e-4
        engine.cache.release("whole")
        # in portions down to two tokens, beside another request, then token by token; the pool of 12 pages
        # of 8 is too small for both without the pages that "whole" gave back
        engine.cache.add_request("a")
        engine.cache.add_request("b")
        out_a, out_b = [], []
        for (a0, a1), (b0, b1) in (((0, 7), (0, 2)), ((7, 9), (2, 19)), ((9, 33), (19, 21))):
            r = engine.run_step([StepEntry("a", ids[a0:a1], list(range(a1 - a0))),
                                 StepEntry("b", other[b0:b1], list(range(b1 - b0)))]).cpu().numpy()
            out_a.append(r[:a1 - a0])
            out_b.append(r[a1 - a0:])
        for t in range(8):
            r = engine.run_step([StepEntry("a", [ids[33 + t]], [0]), StepEntry("b", [other[21 + t]], [0])]).cpu().numpy()
            out_a.append(r[:1])
            out_b.append(r[1:])
        assert np.abs(np.concatenate(out_a) - want).max() < 1e-4
        assert np.abs(np.concatenate(out_b) - want_other[:29]).max() < 1e-4
        engine.cache.release("a")
        engine.cache.release("b")
        engine.cache.check()
        assert engine.cache.free_pages() == [12, 12]
        assert len(engine.generate([ids[:5], other[:9]], SamplingParams(max_tokens=4))[1]) == 4
        # what a block refuses, by name
        with pytest.raises(ValueError, match="takes the norms"):
            part_class("block", "toy_sandwich")(None, None, {"mixer": None})
        with pytest.raises(ValueError, match="needs a feed-forward"):
            part_class("block", "pre_norm")(object(), None, {"mixer": None, "feed_forward": None})
    finally:
        unregister_architecture("ToyBlocksLM")
        unregister_cache_kind(PagedLatent)
        for cat, kind in (("block", "toy_sandwich"), ("block", "toy_parallel"), ("block", "toy_mixer_only"),
                          ("embedding", "toy_positional_embedding"), ("mixer", "toy_latent_attention")):
            unregister_part(cat, kind)
