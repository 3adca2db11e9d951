"""The command line: argument handling (CPU) and generate / inspect / bench smokes (GPU), in the
manner of the reference's scripts/test_mvp.py (run the program, read its output)."""
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import helpers
from mini_llama_cpp_release_b200 import cli

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def run(*args, stdin=None):
    return subprocess.run([sys.executable, "-m", "mini_llama_cpp_release_b200", *args], cwd=ROOT, input=stdin,
                          capture_output=True, text=True, timeout=600)


def test_token_lists():
    assert cli.parse_token_lists("5,17,3;9 9") == [[5, 17, 3], [9, 9]]
    with pytest.raises(SystemExit):
        cli.parse_token_lists(" ; ")


def test_inspect_lists_config_and_tensors_and_flags_problems(tmp_path):
    folder = helpers.model_folder("A")
    p = run("inspect", folder)
    assert p.returncode == 0, p.stderr
    assert "hidden_size: 64" in p.stdout and "model.layers.1.mlp.down_proj.weight" in p.stdout
    assert "cache per token per sequence: 256 B in bfloat16" in p.stdout
    bad = tmp_path / "bad"
    bad.mkdir()
    from safetensors.torch import load_file
    from mini_llama_cpp_release_b200.weights import save_safetensors
    w = load_file(os.path.join(folder, "model.safetensors"))
    del w["model.norm.weight"]
    save_safetensors(str(bad / "model.safetensors"), w)
    helpers.ml.ModelConfig.from_dict(helpers.TINY_A).save(str(bad))
    p = run("inspect", str(bad))
    assert p.returncode == 1 and "PROBLEM: missing tensors (1): model.norm.weight" in p.stdout


def test_unknown_command_and_help():
    assert run("frobnicate").returncode == 2
    assert "generate" in run("--help").stdout


@pytest.mark.gpu
def test_generate_dumps_logits_and_ids_like_the_reference(tmp_path):
    folder = helpers.model_folder("A", std=0.1)
    pm = helpers.plain_model(folder)
    out = str(tmp_path / "dump")
    p = run("--model", folder, "--tokens", "5,17,3,200", "-n", "5", "--dtype", "float32", "--dump-logits", out, "--stop-ids", "511")
    assert p.returncode == 0, p.stderr[-2000:]
    ids = [int(t) for t in open(os.path.join(out, "generation_tokens.txt")).read().split()]
    assert ids == pm.greedy([5, 17, 3, 200], 5) and f"generated ids: {' '.join(map(str, ids))}" in p.stdout
    ref = pm.logits([5, 17, 3, 200] + ids)
    for k in range(3, 8):
        got = torch.from_numpy(np.fromfile(os.path.join(out, f"logits_step{k}.bin"), dtype="<f4").copy())
        assert helpers.rel_err(got, ref[k]) <= helpers.TOL["float32"]
    p = run("generate", "--model", folder, "--tokens", "1,2", "-n", "0")
    assert p.returncode == 0 and "generated 0" in p.stdout                       # scripts/test_mvp.py:58-67
    p = run("generate", "--model", folder, "--tokens", "1," * 250 + "1", "-n", "20")
    assert p.returncode != 0 and "exceeds" in p.stderr                           # context overflow is refused up front


@pytest.mark.gpu
def test_bench_command_prints_the_references_report():
    p = run("bench", helpers.model_folder("B"), "-n", "8", "--prompt-len", "20", "--batch", "3", "--verbose")
    assert p.returncode == 0, p.stderr[-2000:]
    for key in ("prompt tokens:     60", "generated tokens:  24", "decode tokens:     21", "prefill ms:", "tokens/s (decode):",
                "logits shape: [3, 1000]", "GB/s of weights and cache", "limited by", "TFLOP/s"):
        assert key in p.stdout


def test_model_comes_from_a_folder_a_file_or_a_random_configuration(tmp_path, monkeypatch):
    """`--model <path|dir>` and `--config` as the reference resolves them (src/main.cpp:280-281, 452-461), and
    `--random <preset|config.json>`, which writes a model folder from the configuration and a seed."""
    import argparse
    from mini_llama_cpp_release_b200 import measure

    def parse(*argv, positional=False):
        ap = argparse.ArgumentParser()
        cli.add_model_options(ap, positional=positional)
        cli.add_engine_options(ap)
        return ap.parse_args(list(argv))

    assert cli.resolve_model(parse("--model", "some/dir")) == ("some/dir", None)
    assert cli.resolve_model(parse("--model", "w.safetensors", "--config", "c.json")) == ("w.safetensors", "c.json")
    assert cli.resolve_model(parse("some/dir", positional=True)) == ("some/dir", None)
    with pytest.raises(SystemExit, match="--model"):
        cli.resolve_model(parse())
    with pytest.raises(SystemExit, match="not both"):
        cli.resolve_model(parse("--model", "x", "--random", "tiny-a"))
    with pytest.raises(SystemExit, match="neither a preset"):
        cli.resolve_model(parse("--random", "qwen9"))
    monkeypatch.setattr("tempfile.gettempdir", lambda: str(tmp_path))
    folder, cfg_path = cli.resolve_model(parse("--random", "tiny-a", "--weights-seed", "5"))
    assert cfg_path is None and os.path.exists(os.path.join(folder, "model.safetensors"))
    assert helpers.ml.ModelConfig.from_folder(folder).hidden_size == 64
    assert cli.resolve_model(parse("--random", "tiny-a", "--weights-seed", "5"))[0] == folder       # found again, not rewritten
    assert cli.resolve_model(parse("--random", "tiny-a", "--weights-seed", "6"))[0] != folder
    # a configuration of one's own, by the path of its config.json
    helpers.ml.ModelConfig.from_dict(helpers.TINY_B).save(str(tmp_path / "mine"))
    folder_b, _ = cli.resolve_model(parse("--random", str(tmp_path / "mine" / "config.json")))
    assert helpers.ml.ModelConfig.from_folder(folder_b).vocab_size == 1000
    # the five presets are the five configurations the measurements are quoted on
    assert sorted(measure.PRESETS) == ["qwen2-0.5b", "qwen2-1.5b", "qwen2-7b", "tiny-a", "tiny-b"]
    for raw in measure.PRESETS.values():
        helpers.ml.ModelConfig.from_dict(raw)
    # the engine's sizes
    e = cli.engine_config(parse("--model", "x", "--slots", "3", "--dtype", "fp32", "--max-batch-tokens", "100"), need_tokens=640)
    assert (e.max_tokens, e.max_seqs, e.slots, e.dtype, e.max_batch_tokens) == (640, 3, 3, torch.float32, 100)
    with pytest.raises(SystemExit, match="max_batch_tokens"):
        cli.engine_config(parse("--model", "x", "--max-batch-tokens", "0"), need_tokens=64)


def test_engine_configuration_is_checked():
    from mini_llama_cpp_release_b200 import EngineConfig
    e = EngineConfig()
    assert (e.dtype, e.device, e.max_tokens, e.max_seqs, e.max_batch_tokens, e.slots) == (torch.bfloat16, "cuda:0", 8192, None, 16384, 128)
    assert EngineConfig(max_tokens=100, max_seqs=50).slots == 2          # never more slots than pages
    for bad, word in [(dict(device="cpu"), "CUDA"), (dict(dtype="float16"), "dtype"), (dict(max_tokens=0), "max_tokens"),
                      (dict(max_seqs=0), "max_seqs"), (dict(max_batch_tokens=-4), "max_batch_tokens"), (dict(max_tokens=2.5), "max_tokens")]:
        with pytest.raises(ValueError, match=word):
            EngineConfig(**bad)


def test_the_references_backend_option_is_taken_and_cpu_is_refused():
    """`--backend cpu|cuda` is the reference's option (src/main.cpp:291); here only cuda exists, and cpu says so before
    anything is loaded."""
    p = subprocess.run([sys.executable, "-m", "mini_llama_cpp_release_b200", "generate", "--random", "tiny-a", "--tokens", "1,2",
                        "--backend", "cpu"], cwd=ROOT, capture_output=True, text=True, timeout=300)
    assert p.returncode != 0 and "CUDA device only" in p.stderr
    p = run("generate", "--random", "tiny-a", "--prompt", "hello")
    assert p.returncode != 0 and "no tokenizer" in p.stderr


@pytest.mark.gpu
def test_generate_from_random_weights_of_a_preset_with_no_model_on_disk(tmp_path):
    env_tmp = str(tmp_path)
    p = subprocess.run([sys.executable, "-m", "mini_llama_cpp_release_b200", "generate", "--random", "tiny-b", "--tokens", "1,2,3;7",
                        "-n", "8", "--slots", "2", "--backend", "cuda"], cwd=ROOT, capture_output=True, text=True, timeout=600,
                       env=dict(os.environ, TMPDIR=env_tmp))
    assert p.returncode == 0, p.stderr[-2000:]
    lines = [l for l in p.stdout.splitlines() if l.startswith("generated ids:")]
    assert len(lines) == 2 and all(len(l.split()) == 10 for l in lines)
    # the same through a weights file and a config.json that lie apart
    folder = helpers.model_folder("A", std=0.1)
    import shutil
    shutil.copy(os.path.join(folder, "model.safetensors"), str(tmp_path / "w.safetensors"))
    shutil.copy(os.path.join(folder, "config.json"), str(tmp_path / "c.json"))
    p = run("--model", str(tmp_path / "w.safetensors"), "--config", str(tmp_path / "c.json"), "--tokens", "5,17,3,200", "-n", "5",
            "--dtype", "float32", "--stop-ids", "511")
    assert p.returncode == 0, p.stderr[-2000:]
    ids = helpers.plain_model(folder).greedy([5, 17, 3, 200], 5)
    assert f"generated ids: {' '.join(map(str, ids))}" in p.stdout


def test_the_kernel_timing_tool_reads_its_arguments():
    """`python -m mini_llama_cpp_release_b200.kernels.microbench` is the tool the summaries under profiles/ were made
    with; the command lines quoted there must keep parsing."""
    from mini_llama_cpp_release_b200.kernels import microbench
    ap = microbench.parser()
    a = ap.parse_args("gemm --tokens 8 --rows 9728 --k 896 --epilogue silu --copies 1 --once".split())
    assert (a.kernel, a.tokens, a.rows, a.k, a.epilogue, a.copies, a.once, a.rows_form, a.library) == ("gemm", 8, 9728, 896, "silu", 1, True, False, False)
    a = ap.parse_args("gemm --tokens 2048 --rows 1152 --k 896 --epilogue qkv --rows-form".split())
    assert a.rows_form and a.copies == 24
    a = ap.parse_args("attention --seqs 8 --context 4096 --cluster".split())
    assert (a.seqs, a.context, a.q_len, a.cluster, a.impl, a.heads, a.kv_heads, a.head_dim) == (8, 4096, 1, True, "mma", 14, 2, 64)
    a = ap.parse_args("norm --tokens 8 --k 896 --slices 19".split())
    assert a.slices == 19
    assert ap.parse_args("attention --seqs 8 --context 4096 --cluster --phases --copies 8".split()).phases
    for bad in (["conv"], ["gemm", "--epilogue", "relu"], ["attention", "--impl", "library"]):
        with pytest.raises(SystemExit):
            ap.parse_args(bad)
    root = os.path.join(ROOT, "profiles")
    import re, shlex
    for name in os.listdir(root):
        for line in open(os.path.join(root, name)):
            m = re.search(r"kernels\.microbench ((?:gemm|norm|attention)[^`#\"]*)", line)
            if m:
                ap.parse_args(shlex.split(m.group(1).strip()))
