"""What the benchmark program promises without a GPU: its refusals, its reference arm, and the arithmetic behind the
prefill fraction."""
import importlib.util
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def run(*args):
    return subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), *args], capture_output=True, text=True, timeout=120)


def test_more_than_one_gpu_is_refused_with_one_line_and_exit_code_2():
    r = run("--gpus", "2", "--steps", "2", "--warmup", "1")
    assert r.returncode == 2
    lines = [l for l in r.stdout.splitlines() if l.strip()]
    assert len(lines) == 1 and "one GPU" in lines[0]


def test_reference_arm_says_why_it_is_unavailable():
    r = run("--impl", "reference", "--gpus", "1", "--steps", "2", "--warmup", "1")
    assert r.returncode == 0
    line = json.loads(r.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference" and isinstance(line["unavailable"], str) and "\n" not in line["unavailable"]


def test_prefill_flops_are_the_products_of_the_layers_plus_causal_attention_plus_one_row_of_the_head():
    spec = importlib.util.spec_from_file_location("bench_module", os.path.join(ROOT, "bench.py"))
    bench = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(bench)
    cfg = dict(hidden_size=6, intermediate_size=10, num_attention_heads=4, num_key_value_heads=2, head_dim=3, vocab_size=50)
    T, L = 7, 3
    qkv, o, ffn = (4 + 2 * 2) * 3 * 6, 6 * 4 * 3, 3 * 10 * 6
    want = 2.0 * T * (qkv + o + ffn) * L + L * 4 * 2.0 * T * T * 3 + 2.0 * 50 * 6
    assert bench.prefill_flops(cfg, L, T) == want
    # the sizes the default run names are the ones it builds
    q = bench.QWEN2_0_5B
    assert (q["hidden_size"], q["num_attention_heads"], q["num_key_value_heads"], q["head_dim"], q["intermediate_size"],
            q["vocab_size"], q["num_hidden_layers"]) == (896, 14, 2, 64, 4864, 151936, bench.FULL_LAYERS)
    assert bench.PROMPT_LEN == 2048 and bench.CTX_LEN == 4096
