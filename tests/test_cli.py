"""The command line of the torchless runtime (the reference's generate / info / benchmark / chat commands on the
GPU backend).  Without a GPU only ``info`` can run, and every other command has to fail loudly."""
import subprocess
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
CLI = str(ROOT / "litespark-inference_b200" / "torchless" / "__main__.py")


def _run(*argv, stdin=None, timeout=600):
    return subprocess.run([sys.executable, CLI, *argv], capture_output=True, text=True, input=stdin, timeout=timeout)


def test_info_and_argument_errors_without_gpu():
    r = _run("info")
    assert r.returncode == 0 and "kernel   :" in r.stdout and "_lspk_sm100.so" in r.stdout
    assert _run().returncode != 0                                  # a command is required
    assert _run("benchmark", "--embed-dtype", "fp64").returncode != 0


def test_commands_fail_loudly_without_gpu():
    if "GPU      : unavailable" not in _run("info").stdout:
        pytest.skip("a GPU is present")
    r = _run("generate", "1 2 3", "--model", "synthetic-toy")
    assert r.returncode == 2 and "no CPU fallback" in r.stderr


@pytest.mark.gpu
def test_generate_benchmark_chat_on_synthetic_models(tmp_path):
    r = _run("generate", "12 845 9 77", "--model", "synthetic-toy", "--max-tokens", "8", "--raw", "--ignore-eos")
    assert r.returncode == 0, r.stderr
    assert "Prompt (4 tokens)" in r.stdout and "Generated 8 tokens" in r.stdout
    out_line = r.stdout.strip().splitlines()[-1]
    assert len(out_line.split()) == 8 and all(t.isdigit() for t in out_line.split())
    # the same ids through the library's greedy decode
    import importlib
    rt = importlib.import_module("litespark_inference_b200.torchless.runtime")
    synthetic = importlib.import_module("litespark_inference_b200.torchless.synthetic")
    m = synthetic.random_model(synthetic.toy_config(), seed=0, fast=True)
    assert [int(t) for t in out_line.split()] == rt.generate(m, [12, 845, 9, 77], 8)

    r = _run("benchmark", "--model", "synthetic-toy", "--tokens", "8", "--inference")
    assert r.returncode == 0, r.stderr
    assert "Prompt Processing (pp):" in r.stdout and "Token Generation (tg8):" in r.stdout and "±" in r.stdout
    r = _run("benchmark", "--model", "synthetic-falcon-toy", "--tokens", "4")
    assert r.returncode == 0, r.stderr
    assert "TTFT:" in r.stdout and "Throughput:" in r.stdout

    # a Falcon-E checkpoint directory (Hugging Face packing), no tokenizer.json: ids in, ids out
    loader = importlib.import_module("litespark_inference_b200.torchless.loader")
    cfg = synthetic.toy_falcon_config()
    loader.save_falcon_dir(tmp_path, cfg, synthetic.random_falcon_checkpoint_tensors(cfg, seed=9))
    r = _run("chat", "--model", str(tmp_path), "--max-tokens", "4", "--embed-dtype", "int8", stdin="5 6 7\nquit\n")
    assert r.returncode == 0, r.stderr
    assert "Assistant: " in r.stdout and "Goodbye!" in r.stdout
