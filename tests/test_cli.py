"""``bin/firefly`` run as a program."""
import json
import os
import subprocess
import sys

import pytest
import torch

import plain_qwen3 as P

ROOT = os.path.normpath(os.path.join(os.path.dirname(os.path.abspath(__file__)), ".."))
FIREFLY = os.path.join(ROOT, "bin", "firefly")


def _run(*args, timeout=600):
    return subprocess.run([sys.executable, FIREFLY, *args], capture_output=True, text=True, timeout=timeout)


def _write_config(tmp_path, raw):
    path = tmp_path / "cfg.json"
    path.write_text(json.dumps(raw))
    return str(path)


def test_faults_end_with_one_line_not_a_traceback(tmp_path):
    cfg = _write_config(tmp_path, P.TINY_A)
    r = _run("--write-random-model", str(tmp_path / "m"), "--config", cfg, "--seed", "3", "--dtype", "float32")
    assert r.returncode == 0, r.stderr
    assert json.loads(r.stdout)["written"] == str(tmp_path / "m")
    assert os.path.isfile(tmp_path / "m" / "model.safetensors")
    # a folder that is not a model
    r = _run(str(tmp_path / "nothing_here"), "--prompt-ids", "1,2,3")
    assert r.returncode == 1 and r.stderr.startswith("firefly: ") and "Traceback" not in r.stderr
    assert "config.json" in r.stderr
    # no prompt
    r = _run(str(tmp_path / "m"))
    assert r.returncode == 2 and "no prompt given" in r.stderr
    if not torch.cuda.is_available():
        # a machine without a GPU: the engine says so in one line
        r = _run(str(tmp_path / "m"), "--prompt-ids", "1,2,3", "--max-tokens", "2")
        assert r.returncode == 1 and "Traceback" not in r.stderr
        assert r.stderr.strip() == "firefly: firefly_b200 needs a CUDA device and none is available"


@pytest.mark.gpu
def test_generation_as_a_program_matches_the_plain_implementation(tmp_path):
    raw = P.TINY_B
    cfg = _write_config(tmp_path, raw)
    folder = str(tmp_path / "m")
    assert _run("--write-random-model", folder, "--config", cfg, "--seed", "5", "--dtype", "float32").returncode == 0
    from firefly_b200.weights import SafetensorsFile
    f = SafetensorsFile(os.path.join(folder, "model.safetensors"))
    w = {n: f.tensor(n).double() for n in f.names()}
    f.close()
    prompts = [[5, 17, 3, 200, 41, 7, 99], [300, 2], list(range(10, 50))]
    pf = tmp_path / "prompts.jsonl"
    pf.write_text("\n".join(json.dumps(p) for p in prompts[1:]))
    r = _run(folder, "--dtype", "float32", "--prompt-ids", ",".join(map(str, prompts[0])), "--prompts-file", str(pf),
             "--max-tokens", "7", "--max-prefill-chunk-size", "16", "--num-kv-blocks", "64", "--ignore-eos")
    assert r.returncode == 0, r.stderr
    lines = [json.loads(x) for x in r.stdout.strip().splitlines()]
    assert [x["request"] for x in lines] == [0, 1, 2] and [x["prompt_tokens"] for x in lines] == [7, 2, 40]
    for x, p in zip(lines, prompts):
        assert x["tokens"] == P.greedy_generate(raw, w, p, 7)
    # random weights without a folder, synthetic prompts, temperature sampling: the same command twice
    # gives the same tokens
    args = ("--random", cfg, "--seed", "9", "--prompt-len", "33", "--num-prompts", "3", "--max-tokens", "5",
            "--temperature", "0.9", "--num-kv-blocks", "64", "--ignore-eos")
    a, b = _run(*args), _run(*args)
    assert a.returncode == 0 and a.stdout == b.stdout and len(a.stdout.strip().splitlines()) == 3
    assert all(json.loads(x)["prompt_tokens"] == 33 for x in a.stdout.strip().splitlines())
