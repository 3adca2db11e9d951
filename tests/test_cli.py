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
                "logits shape: [3, 1000]"):
        assert key in p.stdout
