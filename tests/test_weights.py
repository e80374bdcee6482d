"""Safetensors reading/writing, the loader's single error, random weights (CPU)."""
import json
import os

import pytest
import torch

from helpers import tiny_config, write_tiny
from velox_b200.models import DecoderModel
from velox_b200.models.qwen3 import qwen3_plan
from velox_b200.parts.base import Runtime
from velox_b200.weights import (SafetensorsError, SafetensorsFile, WeightError, load_weights, write_random_model,
                                write_safetensors)


class Recorder(DecoderModel):
    """A model that keeps what the loader binds, without touching kernels."""

    def bind(self, tensors, runtime):
        self.bound = dict(tensors)   # (tensors are made when looked up, and only while the files are open)


def test_own_reader_agrees_with_the_safetensors_package(tmp_path):
    from safetensors import safe_open
    from safetensors.torch import save_file

    tensors = {"a": torch.randn(3, 5), "b": torch.randn(7).to(torch.bfloat16), "c": torch.arange(6, dtype=torch.int32)}
    ours, theirs = str(tmp_path / "ours.safetensors"), str(tmp_path / "theirs.safetensors")
    write_safetensors(ours, tensors)
    save_file(tensors, theirs)
    with safe_open(ours, framework="pt") as f:
        for k, v in tensors.items():
            assert torch.equal(f.get_tensor(k), v)
    r = SafetensorsFile(theirs)
    assert sorted(r.keys()) == ["a", "b", "c"]
    for k, v in tensors.items():
        assert r.info(k) == (v.dtype, tuple(v.shape))
        assert torch.equal(r.tensor(k), v)


def test_broken_files_are_refused(tmp_path):
    p = tmp_path / "bad.safetensors"
    p.write_bytes(b"\x10\x00\x00\x00\x00\x00\x00\x00{not json")
    with pytest.raises(SafetensorsError):
        SafetensorsFile(str(p))
    p.write_bytes(b"\xff\xff\xff\xff\x00\x00\x00\x00{}")
    with pytest.raises(SafetensorsError):
        SafetensorsFile(str(p))


def test_random_model_is_seeded_and_name_keyed(tmp_path):
    a = write_tiny("tiny_a", str(tmp_path / "a"))
    b = write_tiny("tiny_a", str(tmp_path / "b"))
    fa, fb = SafetensorsFile(a + "/model.safetensors"), SafetensorsFile(b + "/model.safetensors")
    for k in fa.keys():
        assert torch.equal(fa.tensor(k), fb.tensor(k))
    other = write_random_model(str(tmp_path / "c"), tiny_config("tiny_a"), seed=5)
    fc = SafetensorsFile(other + "/model.safetensors")
    assert not torch.equal(fa.tensor("model.norm.weight"), fc.tensor("model.norm.weight"))
    # distributions: matrices N(0, 0.02), norms 1 + N(0, 0.05)
    w = fa.tensor("model.embed_tokens.weight").float()
    assert abs(float(w.std()) - 0.02) < 0.002 and abs(float(w.mean())) < 0.002
    n = fa.tensor("model.layers.0.input_layernorm.weight").float()
    assert abs(float(n.mean()) - 1.0) < 0.03
    # tied model stores no head; untied does
    assert "lm_head.weight" not in fa.keys()
    fb2 = SafetensorsFile(write_tiny("tiny_b", str(tmp_path / "d")) + "/model.safetensors")
    assert "lm_head.weight" in fb2.keys() and "model.layers.2.self_attn.q_proj.bias" in fb2.keys()
    cfg = json.load(open(a + "/config.json"))
    assert cfg["architectures"] == ["Qwen3ForCausalLM"] and cfg["model_type"] == "qwen3"


def _model(name):
    return Recorder(qwen3_plan(tiny_config(name)))


def test_loader_keeps_element_types(tmp_path):
    folder = write_tiny("tiny_b", str(tmp_path / "m"))
    for dt in (torch.bfloat16, torch.float32):
        m = _model("tiny_b")
        load_weights(m, folder, Runtime(dt, torch.device("cpu")))
        assert m.bound["model.layers.0.self_attn.q_proj.weight"].dtype == dt
        assert m.bound["model.embed_tokens.weight"].dtype == dt
        # small vectors are widened exactly to float32
        assert m.bound["model.norm.weight"].dtype == torch.float32
        assert m.bound["model.layers.1.self_attn.k_proj.bias"].dtype == torch.float32
    f = SafetensorsFile(folder + "/model.safetensors")
    assert torch.equal(m.bound["model.norm.weight"], f.tensor("model.norm.weight").float())


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    folder = write_tiny("tiny_a", str(tmp_path / "m"))
    f = SafetensorsFile(folder + "/model.safetensors")
    tensors = {k: f.tensor(k).clone() for k in f.keys()}
    f.close()
    del tensors["model.layers.1.self_attn.q_norm.weight"]
    del tensors["model.layers.0.mlp.up_proj.weight"]
    tensors["model.layers.0.mlp.extra.weight"] = torch.zeros(2, dtype=torch.bfloat16)
    tensors["model.norm.weight"] = torch.ones(65, dtype=torch.bfloat16)
    tensors["model.layers.0.self_attn.o_proj.weight"] = torch.zeros(64, 32, dtype=torch.bfloat16)
    write_safetensors(folder + "/model.safetensors", tensors)
    with pytest.raises(WeightError) as e:
        load_weights(_model("tiny_a"), folder, Runtime(torch.float32, torch.device("cpu")))
    err = e.value
    assert set(err.missing) == {"model.layers.1.self_attn.q_norm.weight", "model.layers.0.mlp.up_proj.weight"}
    assert err.unexpected == ["model.layers.0.mlp.extra.weight"]
    assert {w[0] for w in err.wrong_shape} == {"model.norm.weight", "model.layers.0.self_attn.o_proj.weight"}
    text = str(err)
    for piece in ("missing (2)", "unexpected (1)", "expected [64]", "file has [65]", "q_norm"):
        assert piece in text


def test_tied_model_tolerates_a_stored_head(tmp_path):
    folder = write_tiny("tiny_a", str(tmp_path / "m"))
    f = SafetensorsFile(folder + "/model.safetensors")
    tensors = {k: f.tensor(k).clone() for k in f.keys()}
    f.close()
    tensors["lm_head.weight"] = tensors["model.embed_tokens.weight"].clone()
    write_safetensors(folder + "/model.safetensors", tensors)
    load_weights(_model("tiny_a"), folder, Runtime(torch.float32, torch.device("cpu")))


def test_integer_tensor_for_a_matrix_is_an_error(tmp_path):
    folder = write_tiny("tiny_a", str(tmp_path / "m"))
    f = SafetensorsFile(folder + "/model.safetensors")
    tensors = {k: f.tensor(k).clone() for k in f.keys()}
    f.close()
    tensors["model.norm.weight"] = torch.ones(64, dtype=torch.int32)
    write_safetensors(folder + "/model.safetensors", tensors)
    with pytest.raises(WeightError, match="unusable element type"):
        load_weights(_model("tiny_a"), folder, Runtime(torch.float32, torch.device("cpu")))


def test_sharded_checkpoint(tmp_path):
    folder = write_tiny("tiny_a", str(tmp_path / "m"))
    f = SafetensorsFile(folder + "/model.safetensors")
    names = f.keys()
    half = len(names) // 2
    write_safetensors(folder + "/p1.safetensors", {k: f.tensor(k).clone() for k in names[:half]})
    write_safetensors(folder + "/p2.safetensors", {k: f.tensor(k).clone() for k in names[half:]})
    f.close()
    os.remove(folder + "/model.safetensors")
    wm = {k: ("p1.safetensors" if i < half else "p2.safetensors") for i, k in enumerate(names)}
    json.dump({"weight_map": wm}, open(folder + "/model.safetensors.index.json", "w"))
    m = _model("tiny_a")
    load_weights(m, folder, Runtime(torch.float32, torch.device("cpu")))
    assert len(m.bound) == len(names)
