"""A mixer with state of its own, defined here, registered, built and stepped
without a change to the framework's files.

The toy mixer keeps, per request, the running sum of its inputs (a fixed-size
state in a slot) and returns W (sum so far, this token included).  It lives in a
toy architecture whose layers alternate between it and paged attention, whose
running order names layer 0 twice, and whose last layer reads layer 1's cache.
Nothing of it is a model of anyone's."""
from dataclasses import dataclass
from typing import ClassVar

import numpy as np
import pytest
import torch

import plain_qwen3 as P

pytestmark = pytest.mark.gpu


def register_toy():
    from velox_b200.config import ModelConfig, register_architecture
    from velox_b200.config.model_config import _field
    from velox_b200.parts import (FixedState, LayerSpec, Mixer, ModelPlan, PartSpec, TensorSpec, matmul,
                                  register_mixer)

    class RunningSumMixer(Mixer):
        def __init__(self, prefix, hidden_size):
            super().__init__(prefix)
            self.hidden_size = hidden_size

        def tensor_specs(self):
            return [TensorSpec(self.prefix + "mix.weight", (self.hidden_size, self.hidden_size), "matrix")]

        def bind(self, tensors, runtime):
            super().bind(tensors, runtime)
            self.weight = tensors[self.prefix + "mix.weight"]

        def cache_spec(self):
            return FixedState((self.hidden_size,), "float32")

        def forward(self, h, ctx, cache):
            sums = torch.empty(h.shape, dtype=torch.float32, device=h.device)
            row = 0
            for slot, n in zip(ctx.slots, ctx.new_lens):
                c = torch.cumsum(h[row:row + n].float(), 0) + cache.state[slot]
                sums[row:row + n] = c
                cache.state[slot] = c[-1]
                row += n
            return matmul(sums.to(h.dtype), self.weight)

    @dataclass(frozen=True)
    class ToyConfig(ModelConfig):
        architecture: ClassVar[str] = "ToyStateLM"
        model_type: ClassVar[str] = "toy_state"
        vocab_size: int = _field(int)
        hidden_size: int = _field(int)
        inner_size: int = _field(int)
        eps: float = _field(float)

    def plan(cfg):
        E = cfg.hidden_size
        norm = lambda p: PartSpec("rms_norm", p, dict(size=E, eps=cfg.eps))
        ff = lambda p: PartSpec("gated_mlp", p, dict(hidden_size=E, intermediate_size=cfg.inner_size))
        att = lambda p: PartSpec("paged_attention", p, dict(
            hidden_size=E, num_heads=2, num_kv_heads=1, head_dim=16, qk_norm=False, eps=cfg.eps,
            position=PartSpec("rotary", "", dict(head_dim=16, theta=100.0))))
        layers = []
        for i, kind in enumerate(["sum", "att", "att_shared"]):
            p = "toy.%d." % i
            mixer = PartSpec("toy_running_sum", p, dict(hidden_size=E)) if kind == "sum" else att(p + "a.")
            layers.append(LayerSpec(mixer, ff(p + "ff."), {"mixer": norm(p + "n1."), "feed_forward": norm(p + "n2.")},
                                    cache_of=1 if kind == "att_shared" else None))
        return ModelPlan(cfg.vocab_size, E, PartSpec("token_embedding", "toy.embed.", dict(vocab_size=cfg.vocab_size, hidden_size=E)),
                         layers, norm("toy.norm."), PartSpec("linear_head", "toy.head.", dict(vocab_size=cfg.vocab_size, hidden_size=E)),
                         order=[0, 1, 0, 2], max_positions=256)

    register_mixer("toy_running_sum", RunningSumMixer)
    register_architecture("ToyStateLM", "toy_state", ToyConfig, plan)
    return ToyConfig


def plain_toy(cfg, w, ids):
    """The toy model on a whole sequence, in numpy."""
    E, eps, T = cfg["hidden_size"], cfg["eps"], len(ids)
    pos = np.arange(T)
    x = w["toy.embed.weight"][ids]
    kv = {}

    def ffn(x, p):
        h = P.rms_norm(x, w[p + "n2.weight"], eps)
        return x + P.gated_mlp(h, w[p + "ff.gate_proj.weight"], w[p + "ff.up_proj.weight"], w[p + "ff.down_proj.weight"])

    for i in [0, 1, 0, 2]:
        p = "toy.%d." % i
        h = P.rms_norm(x, w[p + "n1.weight"], eps)
        if i == 0:  # running sum; each of the two runs of layer 0 has a state of its own
            x = x + np.cumsum(h, 0) @ w[p + "mix.weight"].T
        else:
            a = p + "a."
            q = P.rope((h @ w[a + "q_proj.weight"].T).reshape(T, 2, 16), pos, 100.0)
            if i == 1:
                kv["k"] = P.rope((h @ w[a + "k_proj.weight"].T).reshape(T, 1, 16), pos, 100.0)
                kv["v"] = (h @ w[a + "v_proj.weight"].T).reshape(T, 1, 16)
            att = P.causal_attention(q, kv["k"], kv["v"]).reshape(T, 32)
            x = x + att @ w[a + "o_proj.weight"].T
        x = ffn(x, p)
    return P.rms_norm(x, w["toy.norm.weight"], eps) @ w["toy.head.weight"].T


def test_toy_mixer_with_state_runs_in_the_engine(tmp_path):
    from velox_b200 import Engine, EngineConfig
    from velox_b200.config import unregister_architecture
    from velox_b200.engine import StepEntry
    from velox_b200.parts import unregister_part
    from velox_b200.weights import write_random_model

    ToyConfig = register_toy()
    try:
        cfg = ToyConfig.from_dict(dict(vocab_size=120, hidden_size=48, inner_size=64, eps=1e-5))
        folder = write_random_model(str(tmp_path / "toy"), cfg, seed=3)
        raw, w = P.load_model_folder(folder)
        assert raw["architectures"] == ["ToyStateLM"]
        engine = Engine(folder, EngineConfig(dtype="float32", page_size=8, num_pages=16, max_model_len=64,
                                             max_running_requests=2))
        # places of the running order [0, 1, 0, 2]: two states for layer 0, one paged cache, one reader of it
        assert len(engine.cache.groups) == 1 and engine.cache.groups[0].layers == [1]
        assert engine.cache.layer(3).group == 0 and not engine.cache.layer(3).writes
        assert engine.cache.layer(0).state.shape == (2, 48)
        assert engine.cache.layer(2).state is not engine.cache.layer(0).state
        ids = [int(t) for t in np.random.default_rng(0).integers(0, 120, 23)]
        engine.cache.add_request("whole")
        got = engine.run_step([StepEntry("whole", ids, list(range(23)))]).cpu().numpy()
        want = plain_toy(raw, w, ids)
        assert np.abs(got - want).max() < 1e-4
        # a second request gets a zeroed slot of its own, also after the first one's is given back
        engine.cache.release("whole")
        engine.cache.add_request("again")
        got2 = [engine.run_step([StepEntry("again", ids[a:b], list(range(b - a)))]).cpu().numpy()
                for a, b in ((0, 9), (9, 11), (11, 12), (12, 23))]
        assert np.abs(np.concatenate(got2) - want).max() < 1e-4  # in portions: the state carries over
        # and it generates through the scheduler like any model
        from velox_b200 import SamplingParams
        engine.cache.release("again")
        out = engine.generate([ids[:5]], SamplingParams(max_tokens=4))
        assert len(out[0]) == 4
    finally:
        unregister_architecture("ToyStateLM")
        unregister_part("mixer", "toy_running_sum")


def register_graph_safe_toy():
    """The running sum again, written so that it reads nothing of a step but device
    tensors: such a mixer may say `cuda_graph_safe`, and decode steps of its model are
    then captured in CUDA graphs (never padded: a padding row would touch a real slot)."""
    from velox_b200.config import ModelConfig, register_architecture
    from velox_b200.config.model_config import _field
    from velox_b200.parts import FixedState, LayerSpec, Mixer, ModelPlan, PartSpec, TensorSpec, matmul, register_mixer

    class DeviceRunningSum(Mixer):
        cuda_graph_safe = True

        def __init__(self, prefix, hidden_size):
            super().__init__(prefix)
            self.hidden_size = hidden_size

        def tensor_specs(self):
            return [TensorSpec(self.prefix + "mix.weight", (self.hidden_size, self.hidden_size), "matrix")]

        def bind(self, tensors, runtime):
            super().bind(tensors, runtime)
            self.weight = tensors[self.prefix + "mix.weight"]

        def cache_spec(self):
            return FixedState((self.hidden_size,), "float32")

        def forward(self, h, ctx, cache):
            seq = ctx.seq_of_token.long()
            first = ctx.cu_seqlens[:-1].long()[seq]                    # first row of each token's request
            c = torch.cumsum(h.float(), 0)
            before = torch.where((first > 0)[:, None], c[(first - 1).clamp(min=0)], torch.zeros_like(c))
            slots = ctx.state_slots.long()
            sums = c - before + cache.state[slots[seq]]
            cache.state[slots] = sums[ctx.cu_seqlens[1:].long() - 1]    # each request's last row
            return matmul(sums.to(h.dtype), self.weight)

    @dataclass(frozen=True)
    class ToyConfig(ModelConfig):
        architecture: ClassVar[str] = "ToyGraphStateLM"
        model_type: ClassVar[str] = "toy_graph_state"
        vocab_size: int = _field(int)
        hidden_size: int = _field(int)

    def plan(cfg):
        E = cfg.hidden_size
        norm = lambda p: PartSpec("rms_norm", p, dict(size=E, eps=1e-5))
        layers = [LayerSpec(PartSpec("toy_device_running_sum", "toy.%d." % i, dict(hidden_size=E)),
                            PartSpec("gated_mlp", "toy.%d.ff." % i, dict(hidden_size=E, intermediate_size=2 * E)),
                            {"mixer": norm("toy.%d.n1." % i), "feed_forward": norm("toy.%d.n2." % i)}) for i in range(2)]
        return ModelPlan(cfg.vocab_size, E, PartSpec("token_embedding", "toy.embed.", dict(vocab_size=cfg.vocab_size, hidden_size=E)),
                         layers, norm("toy.norm."), PartSpec("linear_head", "toy.head.", dict(vocab_size=cfg.vocab_size, hidden_size=E)),
                         max_positions=128)

    register_mixer("toy_device_running_sum", DeviceRunningSum)
    register_architecture("ToyGraphStateLM", "toy_graph_state", ToyConfig, plan)
    return ToyConfig


def test_a_stateful_mixer_in_captured_decode_steps_advances_its_state_once(tmp_path):
    """With graphs on, the step that first needs a graph captures it: that step must run
    the model once, not once eagerly and once more as a replay, or every request's state
    would be advanced twice.  Tokens and logits equal those of an engine without graphs."""
    from velox_b200 import Engine, EngineConfig, SamplingParams
    from velox_b200.config import unregister_architecture
    from velox_b200.parts import unregister_part
    from velox_b200.weights import write_random_model

    ToyConfig = register_graph_safe_toy()
    try:
        cfg = ToyConfig.from_dict(dict(vocab_size=100, hidden_size=32))
        folder = write_random_model(str(tmp_path / "toy"), cfg, seed=4)
        rng = np.random.default_rng(8)
        prompts = [[int(t) for t in rng.integers(0, 100, n)] for n in (3, 9, 14)]
        runs = {}
        for graphs in (False, True):
            e = Engine(folder, EngineConfig(dtype="float32", page_size=8, num_pages=8, max_model_len=64,
                                            max_running_requests=4, cuda_graphs=graphs))
            rows = []
            e.on_logits = lambda ids, logits: rows.append((list(ids), logits.cpu().numpy().copy()))
            # different lengths: requests finish at different steps, so several batch sizes get a graph
            outs = e.generate(prompts, [SamplingParams(max_tokens=n, ignore_eos=True) for n in (12, 5, 9)])
            runs[graphs] = (outs, rows)
            if graphs:
                g = e.runner.graphs
                assert g.usable and g.has_state and len(g.graphs) >= 3, "no decode step was captured"
        (outs_a, rows_a), (outs_b, rows_b) = runs[False], runs[True]
        assert outs_a == outs_b
        assert len(rows_a) == len(rows_b)
        for (ids_a, la), (ids_b, lb) in zip(rows_a, rows_b):
            assert ids_a == ids_b and np.abs(la - lb).max() < 1e-5
    finally:
        unregister_architecture("ToyGraphStateLM")
        unregister_part("mixer", "toy_device_running_sum")
