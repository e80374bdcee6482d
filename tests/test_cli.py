"""The command line (`bin/velox`, `python -m velox_b200`): options that need no device
here, a model folder in and tokens out on the GPU box."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest

from helpers import ROOT, TINY, random_tokens

VELOX = [sys.executable, os.path.join(ROOT, "bin", "velox")]


def test_model_folder_resolution(tmp_path):
    from velox_b200.cli import _model_folder
    root = tmp_path / "models"
    (root / "a").mkdir(parents=True)
    (root / "a" / "config.json").write_text("{}")
    assert _model_folder(str(root), "a") == str(root / "a")       # --model names a folder of --model-dir
    assert _model_folder(str(root), None) == str(root / "a")      # the only model there
    assert _model_folder(str(root / "a"), None) == str(root / "a")  # --model-dir is a model folder itself
    with pytest.raises(SystemExit, match="no model 'b'"):
        _model_folder(str(root), "b")
    (root / "b").mkdir()
    (root / "b" / "config.json").write_text("{}")
    with pytest.raises(SystemExit, match="holds 2 models"):
        _model_folder(str(root), None)
    with pytest.raises(SystemExit, match="holds 0 models"):
        _model_folder(str(tmp_path / "nothing"), None)


def test_memory_sizes():
    # the reference's forms (src/main.rs:49-51): "auto", "32GB", a share of the memory
    from velox_b200.cli import _memory_bytes
    assert _memory_bytes("auto", None) is None
    assert _memory_bytes("32GB", None) == 32 << 30 and _memory_bytes(" 1.5gb ", None) == 3 << 29
    assert _memory_bytes("512MB", None) == 512 << 20 and _memory_bytes("2g", None) == 2 << 30
    assert _memory_bytes("12345", None) == 12345


def test_parser_has_the_reference_option_names():
    from velox_b200.cli import build_parser, _ints
    ap = build_parser()
    a = ap.parse_args(["generate", "--model-dir", "/m", "--max-model-memory", "80%", "--max-concurrent", "3",
                       "--prompt-tokens", "1,2,3", "--prompt-tokens", "4, 5", "--stop", "7,8", "--dump-logits", "x"])
    assert (a.model_dir, a.max_model_memory, a.max_concurrent) == ("/m", "80%", 3)
    assert [_ints(p) for p in a.prompt_tokens] == [[1, 2, 3], [4, 5]] and a.stop == ["7,8"] and a.dump_logits == "x"
    with pytest.raises(SystemExit):
        ap.parse_args(["serve"])


def test_random_model_writes_a_folder_without_a_device(tmp_path):
    cfg = tmp_path / "tiny_a.json"
    raw = dict(TINY["tiny_a"]["config"], architectures=["Qwen3ForCausalLM"], model_type="qwen3")
    cfg.write_text(json.dumps(raw))
    out = subprocess.run(VELOX + ["random-model", "--config", str(cfg), "--model-dir", str(tmp_path / "m"),
                                  "--model", "tiny_a", "--seed", "5"], capture_output=True, text=True, timeout=300)
    assert out.returncode == 0, out.stderr
    rec = json.loads(out.stdout.strip().splitlines()[-1])
    assert rec == {"model": str(tmp_path / "m" / "tiny_a"), "architecture": "Qwen3ForCausalLM", "seed": 5}
    folder = tmp_path / "m" / "tiny_a"
    assert json.loads((folder / "config.json").read_text())["hidden_size"] == 64
    assert (folder / "model.safetensors").stat().st_size > 0
    bad = subprocess.run(VELOX + ["random-model", "--config", str(cfg)[:-1], "--model-dir", str(tmp_path / "m")],
                         capture_output=True, text=True, timeout=300)
    assert bad.returncode != 0


def _generate(folder_root, model, *options):
    out = subprocess.run(VELOX + ["generate", "--model-dir", folder_root, "--model", model] + list(options),
                         capture_output=True, text=True, timeout=900)
    assert out.returncode == 0, out.stderr[-2000:]
    recs = [json.loads(line) for line in out.stdout.splitlines() if line.startswith("{")]
    return recs, out.stderr


def _write_model(tmp_path, name):
    cfg = tmp_path / (name + ".json")
    cfg.write_text(json.dumps(dict(TINY[name]["config"], architectures=["Qwen3ForCausalLM"], model_type="qwen3")))
    out = subprocess.run(VELOX + ["random-model", "--config", str(cfg), "--model-dir", str(tmp_path / "models"),
                                  "--model", name, "--seed", str(TINY[name]["seed"])],
                         capture_output=True, text=True, timeout=300)
    assert out.returncode == 0, out.stderr
    return str(tmp_path / "models"), str(tmp_path / "models" / name)


@pytest.mark.gpu
def test_generate_greedy_tiny_a_tokens_logits_and_stop(tmp_path):
    """BASELINE's tiny A workload through the command line: prompts of 5, 11 and 17
    tokens, 8 new tokens each, greedy, pages of 4, in 32-bit: the plain
    implementation's tokens exactly, and the dumped logits within 1e-4."""
    import plain_qwen3 as P
    root, folder = _write_model(tmp_path, "tiny_a")
    cfg, w = P.load_model_folder(folder)
    prompts = [random_tokens(cfg["vocab_size"], n, 40 + n) for n in (5, 11, 17)]
    want = [P.greedy_generate(cfg, w, p, 8) for p in prompts]
    dump = str(tmp_path / "logits.f32")
    opts = [x for p in prompts for x in ("--prompt-tokens", ",".join(map(str, p)))]
    recs, err = _generate(root, "tiny_a", *opts, "--dtype", "float32", "--max-tokens", "8", "--page-size", "4",
                          "--num-pages", "64", "--max-concurrent", "2", "--max-model-len", "64", "--ignore-eos",
                          "--dump-logits", dump, "--stats")
    assert [r["tokens"] for r in recs] == want
    assert [r["prompt_tokens"] for r in recs] == [5, 11, 17] and all(r["finish_reason"] == "length" for r in recs)
    stats = json.loads(err.strip().splitlines()[-1])
    assert stats["requests_completed"] == 3 and stats["tokens_generated"] == 24 and stats["free_pages"] == [64]
    assert stats["last_step_us"] > 0 and stats["running"] == 0
    index = json.load(open(dump + ".json"))
    rows = np.fromfile(dump, "<f4").reshape(index["rows"], cfg["vocab_size"])
    assert index["rows"] == 24 and sorted(set(index["request_of_row"])) == [0, 1, 2]
    seen = [0, 0, 0]
    for row, rid in zip(rows, index["request_of_row"]):
        exact = P.forward_logits(cfg, w, prompts[rid] + want[rid][:seen[rid]])[-1]
        assert np.abs(row - exact).max() <= 1e-4
        seen[rid] += 1
    # --stop: a run of generated tokens ends the request, and the run is kept
    recs, _ = _generate(root, "tiny_a", "--prompt-tokens", ",".join(map(str, prompts[1])), "--dtype", "float32",
                        "--max-tokens", "8", "--page-size", "4", "--num-pages", "64", "--max-model-len", "64",
                        "--ignore-eos", "--stop", "%d,%d" % (want[1][3], want[1][4]), "--stop", "9999")
    pair = want[1][3:5]
    first = next(n for n in range(2, 9) if want[1][n - 2:n] == pair)   # (a tiny model may repeat itself earlier)
    assert recs[0]["tokens"] == want[1][:first] and recs[0]["finish_reason"] == "stop"


@pytest.mark.gpu
def test_generate_temperature_tiny_b_in_portions(tmp_path):
    """BASELINE's tiny B workload: prompts of 1, 9, 23 and 40 tokens cut into portions
    of 7 beside decoding requests, temperature 0.8 with a seed, 6 new tokens: in 32-bit
    the plain sampler's tokens from the plain implementation's logits; request i is
    seeded with --seed + i."""
    import plain_qwen3 as P
    from velox_b200.sampling.rng import uniform
    root, folder = _write_model(tmp_path, "tiny_b")
    cfg, w = P.load_model_folder(folder)
    lens = (1, 9, 23, 40)
    vocab = cfg["vocab_size"]
    rng = np.random.default_rng(7)   # what --prompt-lens with --prompt-seed 7 draws
    prompts = [[int(t) for t in rng.integers(0, vocab, n)] for n in lens]
    recs, _ = _generate(root, "tiny_b", "--prompt-lens", ",".join(map(str, lens)), "--prompt-seed", "7",
                        "--dtype", "float32", "--max-tokens", "6", "--temperature", "0.8", "--top-p", "0.9",
                        "--seed", "1000", "--page-size", "8", "--max-model-memory", "64MB", "--chunk-size", "7",
                        "--max-batch-tokens", "16", "--max-concurrent", "4", "--max-model-len", "128", "--ignore-eos")
    assert len(recs) == 4
    for i, (p, r) in enumerate(zip(prompts, recs)):
        assert len(r["tokens"]) == 6 and r["prompt_tokens"] == lens[i]
        logits = P.forward_logits(cfg, w, p + r["tokens"])
        for n, tok in enumerate(r["tokens"]):
            probs = P.probabilities(logits[len(p) - 1 + n], 0.8, 0.9)
            assert tok == P.sample_from(probs, uniform(1000 + i, 0, n)), (i, n)
    # bfloat16, the default: runs, and the same command gives the same tokens twice
    a, _ = _generate(root, "tiny_b", "--prompt-lens", "9,23", "--max-tokens", "6", "--temperature", "0.8",
                     "--page-size", "8", "--max-model-len", "128", "--max-model-memory", "1%", "--ignore-eos")
    b, _ = _generate(root, "tiny_b", "--prompt-lens", "9,23", "--max-tokens", "6", "--temperature", "0.8",
                     "--page-size", "8", "--max-model-len", "128", "--max-model-memory", "1%", "--ignore-eos")
    assert a == b and [len(r["tokens"]) for r in a] == [6, 6]
