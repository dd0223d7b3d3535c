"""The command line on a device, as a user runs it: `bin/dllm-b200` as a subprocess on model folders written to a
temporary place; generated ids on standard output and the fingerprint line on standard error, compared with the
plain implementation (float32, so the tokens are exact). Reference: src/etalii_dllm/cli.py:284-297, 771-802."""
import hashlib
import json
import os
import re
import subprocess
import sys

import numpy as np
import pytest
import torch

import plain_llama as P
from helpers import TOL, model_case, prompts_for, rel_error

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
LINE = re.compile(r"^fingerprint: ([0-9a-f]{64})  tokens: (\d+)  finish: (stop|length)$")


@pytest.fixture(scope="module", params=["a", "b"])
def folder(request, tmp_path_factory):
    from etalii.dllm_b200.weights.random_init import write_model

    config, weights = model_case(request.param)
    path = tmp_path_factory.mktemp(f"cli_{request.param}")
    write_model(str(path), config, {k: torch.from_numpy(v).to(torch.bfloat16) for k, v in weights.items()})
    return str(path), config, weights


@pytest.fixture(scope="module")
def folder_b(tmp_path_factory):
    from etalii.dllm_b200.weights.random_init import write_model

    config, weights = model_case("b")
    path = tmp_path_factory.mktemp("cli_only_b")
    write_model(str(path), config, {k: torch.from_numpy(v).to(torch.bfloat16) for k, v in weights.items()})
    return str(path), config, weights


def run(folder, *arguments, dtype="float32", stdin=None, cache_tokens=None):
    command = [sys.executable, os.path.join(ROOT, "bin", "dllm-b200"), "--model", folder, "--dtype", dtype]
    if cache_tokens is not None:
        command += ["--cache-tokens", str(cache_tokens)]
    done = subprocess.run(command + list(arguments), input=stdin, capture_output=True, text=True, timeout=600)
    return done.returncode, done.stdout, done.stderr


def ids(text):
    return ",".join(str(t) for t in text)


def outputs(stdout):
    return [[int(t) for t in line.split()] for line in stdout.splitlines()]


def fingerprints(stderr):
    return [LINE.match(line).groups() for line in stderr.splitlines() if line.startswith("fingerprint:")]


def test_greedy_ids_and_the_fingerprint_line(folder):
    path, config, weights = folder
    prompt = prompts_for(config, (9,), seed=3)[0]
    code, out, err = run(path, "generate", "--prompt-ids", ids(prompt), "--max-tokens", "8", "--ignore-eos")
    assert code == 0, err
    want, _ = P.generate(config, weights, prompt, 8)
    assert outputs(out) == [want]
    (digest, count, finish), = fingerprints(err)
    assert digest == hashlib.sha256(np.asarray(want, dtype="<i4").tobytes()).hexdigest()
    assert (count, finish) == ("8", "length")


def test_choices_draw_from_consecutive_seeds_and_prompts_run_as_one_batch(folder):
    path, config, weights = folder
    prompts = prompts_for(config, (5, 17, 2), seed=4)
    arguments = ["generate", "--max-tokens", "10", "--n", "3", "--temperature", "0.8", "--seed", "5", "--ignore-eos"]
    for prompt in prompts:
        arguments += ["--prompt-ids", ids(prompt)]
    code, out, err = run(path, *arguments)
    assert code == 0, err
    want = [P.generate(config, weights, prompt, 10, temperature=0.8, seed=5 + choice)[0]
            for prompt in prompts for choice in range(3)]
    assert outputs(out) == want
    assert [line for line in err.splitlines() if line.startswith("--- choice")] == \
        [f"--- choice {c} (seed {5 + c})" for _ in prompts for c in range(3)]
    assert len(fingerprints(err)) == 9


def test_prompt_file_stop_ids_and_min_tokens(folder_b, tmp_path):
    path, config, weights = folder_b
    prompts = prompts_for(config, (7, 12), seed=6)
    listing = tmp_path / "prompts.txt"
    listing.write_text("\n".join(" ".join(str(t) for t in p) for p in prompts) + "\n")
    free = [P.generate(config, weights, p, 12)[0] for p in prompts]
    stop = free[0][2]  # the third token the first prompt would produce ends it
    code, out, err = run(path, "generate", "--prompt-file", str(listing), "--max-tokens", "12", "--ignore-eos",
                         "--stop-token-id", str(stop))
    assert code == 0, err
    want = [P.generate(config, weights, p, 12, stop_tokens=[stop]) for p in prompts]
    assert outputs(out) == [w[0] for w in want]
    assert [f[2] for f in fingerprints(err)] == [w[1] for w in want] and want[0][1] == "stop"
    # held back until six tokens are out: the stop token cannot be chosen before
    code, out, err = run(path, "generate", "--prompt-file", str(listing), "--max-tokens", "12", "--ignore-eos",
                         "--stop-token-id", str(stop), "--min-tokens", "6")
    assert code == 0, err
    want = [P.generate(config, weights, p, 12, stop_tokens=[stop], min_tokens=6) for p in prompts]
    assert outputs(out) == [w[0] for w in want] and all(len(w[0]) >= 6 for w in want)


def test_the_models_own_stop_token_ends_unless_ignored(folder_b):
    path, config, weights = folder_b
    prompt = prompts_for(config, (6,), seed=8)[0]
    free = P.generate(config, weights, prompt, 10)[0]
    eos = dict(config, eos_token_id=free[4])
    from etalii.dllm_b200.weights.random_init import write_model
    import tempfile

    with tempfile.TemporaryDirectory() as other:
        write_model(other, eos, {k: torch.from_numpy(v).to(torch.bfloat16) for k, v in weights.items()})
        code, out, err = run(other, "generate", "--prompt-ids", ids(prompt), "--max-tokens", "10")
        assert code == 0, err
        want, reason = P.generate(eos, weights, prompt, 10, stop_tokens=[free[4]])
        assert outputs(out) == [want] and fingerprints(err)[0][2] == reason == "stop"
        code, out, err = run(other, "generate", "--prompt-ids", ids(prompt), "--max-tokens", "10", "--ignore-eos")
        assert code == 0 and outputs(out) == [free]


def test_a_cache_that_is_too_small_is_one_error_line(folder_b):
    path, config, _ = folder_b
    prompt = prompts_for(config, (70,), seed=9)[0]
    code, out, err = run(path, "generate", "--prompt-ids", ids(prompt), "--max-tokens", "8", cache_tokens=64)
    assert code == 2 and out == ""
    lines = [line for line in err.splitlines() if not line.startswith("[dllm_b200]")]
    assert len(lines) == 1 and lines[0].startswith("error:") and "cache" in lines[0] and "Traceback" not in err


def test_bfloat16_through_the_command_line(folder_b):
    path, config, weights = folder_b
    prompt = prompts_for(config, (11,), seed=10)[0]
    code, out, err = run(path, "generate", "--prompt-ids", ids(prompt), "--max-tokens", "6", "--ignore-eos",
                         dtype="bfloat16")
    assert code == 0, err
    context = list(prompt)
    for token in outputs(out)[0]:  # each chosen token is (nearly) the best of the plain logits for its context
        ref = P.forward(config, weights, context)[-1]
        assert ref[token] >= ref.max() - 2 * TOL["bfloat16"] * np.abs(ref).max()
        context.append(token)


def test_replay_subcommand_writes_the_logits_of_wanted_places(folder_b, tmp_path):
    path, config, weights = folder_b
    tokens = prompts_for(config, (20,), seed=12)[0]
    steps = [{"step": 0, "entries": [{"id": "r", "tokens": tokens[:15], "want": [0, 14]}], "end": []},
             {"step": 1, "entries": [{"id": "r", "tokens": tokens[15:], "want": [4]}], "end": ["r"]}]
    code, out, err = run(path, "replay", "--out", str(tmp_path), "--max-tokens", "64",
                         stdin="".join(json.dumps(s) + "\n" for s in steps))
    assert code == 0, err
    assert out.splitlines() == ["done 0", "done 1"]
    plain = P.forward(config, weights, tokens)
    first = np.fromfile(tmp_path / "0.f32", dtype="<f4").reshape(2, -1)
    second = np.fromfile(tmp_path / "1.f32", dtype="<f4").reshape(1, -1)
    assert rel_error(first, plain[[0, 14]]) <= TOL["float32"] and rel_error(second, plain[[19]]) <= TOL["float32"]


def test_bench_subcommand_prints_one_json_line(folder_b):
    path, config, _ = folder_b
    code, out, err = run(path, "bench", "--batch", "3", "--prompt-tokens", "20", "--new-tokens", "12", "--repeats",
                         "2", dtype="bfloat16")
    assert code == 0, err
    line = json.loads(out)
    assert line["batch"] == 3 and line["repeats"] == 2 and line["tokens_per_s"] > 0 and line["sd"] >= 0
    assert abs(line["call_s"] - 3 * 12 / line["tokens_per_s"]) < 0.5 * line["call_s"] + 1e-3
    assert line["prefill_s"] + line["decode_s"] <= line["call_s"] * 1.01
