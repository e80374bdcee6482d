"""Two more kinds of parts defined here, registered, built and stepped without a
change to the framework's files: a position encoding of another kind (a table of
learned vectors added to queries and keys, which the fused rotation kernel does
not know) and a feed-forward with routing (a router picks one of three small
experts per token).  They live in a toy architecture beside the framework's own
attention, norm, embedding and head.  Nothing of it is a model of anyone's."""
from dataclasses import dataclass
from typing import ClassVar

import numpy as np
import pytest
import torch

import plain_qwen3 as P

pytestmark = pytest.mark.gpu
HEADS, KV_HEADS, D, EXPERTS = 4, 2, 16, 3


def register_toy():
    from velox_b200.config import ModelConfig, register_architecture
    from velox_b200.config.model_config import _field
    from velox_b200.parts import (FeedForward, LayerSpec, ModelPlan, PartSpec, Position, TensorSpec, matmul,
                                  register_feed_forward, register_position)

    class LearnedOffsets(Position):
        """q and k of the token at position p get table[p] added (every head alike)."""
        cuda_graph_safe = True   # reads the step's positions on the device only

        def __init__(self, prefix, head_dim, max_positions):
            super().__init__(prefix)
            self.head_dim, self.max_positions = head_dim, max_positions

        def tensor_specs(self):
            return [TensorSpec(self.prefix + "offsets", (self.max_positions, self.head_dim), "matrix")]

        def bind(self, tensors, runtime):
            super().bind(tensors, runtime)
            self.table = tensors[self.prefix + "offsets"]

        def apply(self, q, k, positions):
            add = self.table[positions.long()][:, None, :]
            return q + add, k + add

    class RoutedFeedForward(FeedForward):
        """Router logits in float32; the best expert alone serves a token, weighted by
        its softmax probability: out = p_e * W_out[e] relu(W_in[e] h)."""

        def __init__(self, prefix, hidden_size, inner_size, experts):
            super().__init__(prefix)
            self.hidden_size, self.inner_size, self.experts = hidden_size, inner_size, experts

        def tensor_specs(self):
            p = self.prefix
            specs = [TensorSpec(p + "router.weight", (self.experts, self.hidden_size), "matrix")]
            for e in range(self.experts):
                specs.append(TensorSpec(p + "experts.%d.in.weight" % e, (self.inner_size, self.hidden_size), "matrix"))
                specs.append(TensorSpec(p + "experts.%d.out.weight" % e, (self.hidden_size, self.inner_size), "matrix"))
            return specs

        def bind(self, tensors, runtime):
            super().bind(tensors, runtime)
            p = self.prefix
            self.router = tensors[p + "router.weight"]
            self.w_in = [tensors[p + "experts.%d.in.weight" % e] for e in range(self.experts)]
            self.w_out = [tensors[p + "experts.%d.out.weight" % e] for e in range(self.experts)]

        def forward(self, h, ctx):
            logits = h.float() @ self.router.float().t()
            prob, best = torch.softmax(logits, -1).max(-1)
            out = torch.zeros_like(h)
            for e in range(self.experts):
                rows = torch.nonzero(best == e).flatten()   # (a toy: the routing is read on the host)
                if rows.numel():
                    inner = torch.relu(matmul(h[rows].contiguous(), self.w_in[e]))
                    out[rows] = (matmul(inner, self.w_out[e]).float() * prob[rows, None]).to(h.dtype)
            return out

    @dataclass(frozen=True)
    class ToyConfig(ModelConfig):
        architecture: ClassVar[str] = "ToyRoutedLM"
        model_type: ClassVar[str] = "toy_routed"
        vocab_size: int = _field(int)
        hidden_size: int = _field(int)
        inner_size: int = _field(int)
        layers: int = _field(int)
        eps: float = _field(float)

    def plan(cfg):
        E = cfg.hidden_size
        norm = lambda p: PartSpec("rms_norm", p, dict(size=E, eps=cfg.eps))
        layers = []
        for i in range(cfg.layers):
            p = "toy.%d." % i
            att = PartSpec("paged_attention", p + "a.", dict(
                hidden_size=E, num_heads=HEADS, num_kv_heads=KV_HEADS, head_dim=D, qk_norm=True, eps=cfg.eps,
                position=PartSpec("toy_learned_offsets", p + "a.pos.", dict(head_dim=D, max_positions=128))))
            ff = PartSpec("toy_routed", p + "ff.", dict(hidden_size=E, inner_size=cfg.inner_size, experts=EXPERTS))
            layers.append(LayerSpec(att, ff, {"mixer": norm(p + "n1."), "feed_forward": norm(p + "n2.")}))
        return ModelPlan(cfg.vocab_size, E, PartSpec("token_embedding", "toy.embed.", dict(vocab_size=cfg.vocab_size, hidden_size=E)),
                         layers, norm("toy.norm."), PartSpec("linear_head", "toy.head.", dict(vocab_size=cfg.vocab_size, hidden_size=E)),
                         order=list(range(cfg.layers)), max_positions=128)

    register_position("toy_learned_offsets", LearnedOffsets)
    register_feed_forward("toy_routed", RoutedFeedForward)
    register_architecture("ToyRoutedLM", "toy_routed", ToyConfig, plan)
    return ToyConfig


def plain_toy(cfg, w, ids):
    """The toy model on a whole sequence, in numpy."""
    eps, T = cfg["eps"], len(ids)
    x = w["toy.embed.weight"][ids]
    routes = []
    for i in range(cfg["layers"]):
        p = "toy.%d." % i
        a = p + "a."
        h = P.rms_norm(x, w[p + "n1.weight"], eps)
        q = P.rms_norm((h @ w[a + "q_proj.weight"].T).reshape(T, HEADS, D), w[a + "q_norm.weight"], eps)
        k = P.rms_norm((h @ w[a + "k_proj.weight"].T).reshape(T, KV_HEADS, D), w[a + "k_norm.weight"], eps)
        v = (h @ w[a + "v_proj.weight"].T).reshape(T, KV_HEADS, D)
        off = w[a + "pos.offsets"][:T][:, None, :]
        att = P.causal_attention(q + off, k + off, v).reshape(T, HEADS * D)
        x = x + att @ w[a + "o_proj.weight"].T
        h = P.rms_norm(x, w[p + "n2.weight"], eps)
        logits = h @ w[p + "ff.router.weight"].T
        prob = np.exp(logits - logits.max(-1, keepdims=True))
        prob /= prob.sum(-1, keepdims=True)
        best = prob.argmax(-1)
        routes.append(best)
        out = np.zeros_like(x)
        for t in range(T):
            e = best[t]
            inner = np.maximum(h[t] @ w[p + "ff.experts.%d.in.weight" % e].T, 0)
            out[t] = prob[t, e] * (inner @ w[p + "ff.experts.%d.out.weight" % e].T)
        x = x + out
    return P.rms_norm(x, w["toy.norm.weight"], eps) @ w["toy.head.weight"].T, routes


def test_toy_position_encoding_and_routed_feed_forward_run_in_the_engine(tmp_path):
    from velox_b200 import Engine, EngineConfig, SamplingParams
    from velox_b200.config import unregister_architecture
    from velox_b200.engine import StepEntry
    from velox_b200.parts import unregister_part
    from velox_b200.weights import write_random_model

    ToyConfig = register_toy()
    try:
        cfg = ToyConfig.from_dict(dict(vocab_size=90, hidden_size=40, inner_size=56, layers=2, eps=1e-5))
        folder = write_random_model(str(tmp_path / "toy"), cfg, seed=5)
        raw, w = P.load_model_folder(folder)
        # make the router decisive and the offsets matter: random weights of 0.02 would leave both near nothing
        from velox_b200.weights.safetensors_io import SafetensorsFile, write_safetensors
        import os
        path = os.path.join(folder, "model.safetensors")
        f = SafetensorsFile(path)
        tensors, meta = {name: f.tensor(name).clone() for name in f.keys()}, dict(f.metadata)
        f.close()
        for name in list(tensors):
            if name.endswith("router.weight"):
                tensors[name] = tensors[name] * 200
            if name.endswith("pos.offsets"):
                tensors[name] = tensors[name] * 40
        write_safetensors(path, tensors, meta)
        raw, w = P.load_model_folder(folder)
        engine = Engine(folder, EngineConfig(dtype="float32", page_size=8, num_pages=24, max_model_len=96,
                                             max_running_requests=3))
        ids = [int(t) for t in np.random.default_rng(1).integers(0, 90, 37)]
        want, routes = plain_toy(raw, w, ids)
        assert all(len(set(r.tolist())) > 1 for r in routes), "the test's router sends every token the same way"
        engine.cache.add_request("whole")
        got = engine.run_step([StepEntry("whole", ids, list(range(37)))]).cpu().numpy()
        assert np.abs(got - want).max() < 1e-4
        engine.cache.release("whole")
        # in portions, beside another request, then token by token
        other = [int(t) for t in np.random.default_rng(2).integers(0, 90, 20)]
        want_other, _ = plain_toy(raw, w, other)
        engine.cache.add_request("a")
        engine.cache.add_request("b")
        out_a, out_b = [], []
        for (a0, a1), (b0, b1) in (((0, 9), (0, 2)), ((9, 11), (2, 13)), ((11, 30), (13, 14))):
            r = engine.run_step([StepEntry("a", ids[a0:a1], list(range(a1 - a0))),
                                 StepEntry("b", other[b0:b1], list(range(b1 - b0)))]).cpu().numpy()
            out_a.append(r[:a1 - a0])
            out_b.append(r[a1 - a0:])
        for t in range(6):
            r = engine.run_step([StepEntry("a", [ids[30 + t]], [0]), StepEntry("b", [other[14 + t]], [0])]).cpu().numpy()
            out_a.append(r[:1])
            out_b.append(r[1:])
        assert np.abs(np.concatenate(out_a) - want[:36]).max() < 1e-4
        assert np.abs(np.concatenate(out_b) - want_other).max() < 1e-4
        engine.cache.release("a")
        engine.cache.release("b")
        assert len(engine.generate([ids[:5]], SamplingParams(max_tokens=4))[0]) == 4
    finally:
        unregister_architecture("ToyRoutedLM")
        unregister_part("position", "toy_learned_offsets")
        unregister_part("feed_forward", "toy_routed")
