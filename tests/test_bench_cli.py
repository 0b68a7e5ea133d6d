"""The benchmark's command line: what it refuses and what it prints without a GPU."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def run_bench(*args):
    return subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), *args], capture_output=True, text=True,
                          timeout=120)


def test_more_than_one_gpu_is_refused_with_one_line_and_exit_code_2():
    p = run_bench("--gpus", "2")
    assert p.returncode == 2
    lines = [ln for ln in p.stdout.splitlines() if ln.strip()]
    assert len(lines) == 1 and "one GPU" in lines[0]


def test_reference_arm_says_why_it_is_unavailable():
    p = run_bench("--impl", "reference", "--gpus", "1", "--steps", "4", "--warmup", "3")
    assert p.returncode == 0
    line = json.loads(p.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference" and isinstance(line["unavailable"], str) and line["unavailable"]


def test_a_cache_too_small_for_the_prompt_and_the_steps_is_refused():
    p = run_bench("--prompt-tokens", "2048", "--context", "2100", "--steps", "128")
    assert p.returncode == 2 and "holds no prompt" in p.stdout


def test_unknown_preset_is_refused_with_the_names_there_are():
    p = run_bench("--model", "llama-9-900b")
    assert p.returncode == 2 and "no preset 'llama-9-900b'" in p.stdout and "llama-3.1-8b" in p.stdout
