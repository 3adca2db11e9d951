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


def test_reference_arm_prints_the_contracts_line_or_one_line_that_says_why_not():
    """On a machine without a GPU the reference's program cannot run: the arm then says so in one line and exits 0.
    Where it can run (tests/test_bench_gpu.py) it prints the same keys as the other arm, with `impl: reference`."""
    r = run("--impl", "reference", "--gpus", "1", "--steps", "2", "--warmup", "1")
    assert r.returncode == 0
    line = json.loads(r.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference"
    if "unavailable" in line:
        assert isinstance(line["unavailable"], str) and "\n" not in line["unavailable"] and line["unavailable"]
    else:
        for key in ("metric", "value", "unit", "ms_per_step", "e2e", "config", "dtype", "clocks", "prefill"):
            assert key in line
        assert line["dtype"] == "fp32" and len(line["config"]) <= 20


def test_prefill_flops_are_the_products_of_the_layers_plus_causal_attention_plus_one_row_of_the_head():
    from mini_llama_cpp_release_b200 import measure
    cfg = dict(hidden_size=6, intermediate_size=10, num_attention_heads=4, num_key_value_heads=2, head_dim=3, vocab_size=50)
    T, L = 7, 3
    qkv, o, ffn = (4 + 2 * 2) * 3 * 6, 6 * 4 * 3, 3 * 10 * 6
    want = 2.0 * T * (qkv + o + ffn) * L + L * 4 * 2.0 * T * T * 3 + 2.0 * 50 * 6
    assert measure.prefill_flops(cfg, L, [T]) == want
    # two sequences: the products see all tokens, attention each sequence's own square, the head one row each
    assert measure.prefill_flops(cfg, L, [T, 2]) == 2.0 * (T + 2) * (qkv + o + ffn) * L + L * 4 * 2.0 * (T * T + 4) * 3 + 2 * 2.0 * 50 * 6
    # the sizes the default run names are the ones BASELINE's third configuration gives
    spec = importlib.util.spec_from_file_location("bench_module", os.path.join(ROOT, "bench.py"))
    bench = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(bench)
    work = bench.CONFIGS["qwen2-0.5b"]
    q = measure.PRESETS[work["preset"]]
    assert (q["hidden_size"], q["num_attention_heads"], q["num_key_value_heads"], q["head_dim"], q["intermediate_size"],
            q["vocab_size"], q["num_hidden_layers"], q["tie_word_embeddings"]) == (896, 14, 2, 64, 4864, 151936, 24, True)
    assert work["prompt_len"] == 2048 and work["ctx_len"] == 4096
    assert len(bench.describe(q, 24, 8, work)) + 4 <= 20            # the record keeps at most 20 flat keys of `config`


def test_roofline_names_what_limits_the_step():
    from mini_llama_cpp_release_b200 import measure
    pk = dict(hbm_gbs=1000.0)
    slow = measure.roofline(1e9, 10.0, pk)                         # 100 GB/s of 1000
    assert slow["frac"] == 0.1 and slow["bound"] == "hbm" and "latency" in slow["limited_by"]
    assert measure.roofline(1e9, 1.25, pk)["limited_by"] == "hbm"   # 800 GB/s


def test_ids_of_the_two_decode_loops_are_compared_sequence_by_sequence():
    from mini_llama_cpp_release_b200 import measure
    on_device = [[1, 5], [2, 6], [3, 7], [4, 8]]                   # [step][sequence]
    assert measure.agreement(on_device, [[1, 2, 3, 4], [5, 6, 7, 8]], 32) == dict(steps=4, equal_sequences=2, equal_first_8=2, of=2)
    assert measure.agreement(on_device, [[1, 2, 3, 4], [5, 6, 0, 8]], 32)["equal_sequences"] == 1
    assert measure.agreement(on_device, [[1, 2, 3, 4], [5, 6, 0, 8]], 2)["equal_sequences"] == 2
    long_run = [[7, 9]] * 8 + [[7, 1]] * 24                          # the second sequence parts at its ninth id
    got = measure.agreement(long_run, [[7] * 32, [9] * 32], 32)
    assert (got["equal_sequences"], got["equal_first_8"]) == (1, 2)
