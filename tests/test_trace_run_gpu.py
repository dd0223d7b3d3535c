"""bin/trace_run as a user runs it: a model folder on disk, steps on standard input, logits in files; compared with
the plain implementation for whole requests, for the last 32 tokens one by one and for batches of unequal lengths
that follow one another in the same cache room."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import plain_llama as P
from helpers import TOL, PlainLogits, model_case, prompts_for, rel_error

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


class Replay:
    def __init__(self, folder, out, dtype, max_tokens):
        self.out = out
        self.process = subprocess.Popen(
            [sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", folder, "--dtype", dtype, "--out", out,
             "--max-tokens", str(max_tokens)], stdin=subprocess.PIPE, stdout=subprocess.PIPE, text=True)
        self.step = 0

    def send(self, entries, end=()):
        record = {"step": self.step, "entries": entries, "end": list(end)}
        self.process.stdin.write(json.dumps(record) + "\n")
        self.process.stdin.flush()
        answer = self.process.stdout.readline().strip()
        assert answer == f"done {self.step}", answer
        path = os.path.join(self.out, f"{self.step}.f32")
        self.step += 1
        wanted = sum(len(e.get("want", [])) for e in entries)
        if wanted == 0:
            assert not os.path.exists(path)
            return None
        return np.fromfile(path, dtype="<f4").reshape(wanted, -1)

    def close(self):
        self.process.stdin.close()
        assert self.process.wait(timeout=60) == 0


@pytest.fixture(scope="module", params=["a", "b"])
def model_folder(request, tmp_path_factory):
    from etalii.dllm_b200.weights.random_init import write_model

    config, weights = model_case(request.param)
    folder = tmp_path_factory.mktemp(f"tiny_{request.param}")
    tensors = {k: torch.from_numpy(v).to(torch.bfloat16) for k, v in weights.items()}  # the values are bf16-exact
    write_model(str(folder), config, tensors)
    return str(folder), config, PlainLogits(config, weights)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_replay_modes(model_folder, dtype, tmp_path):
    folder, config, plain = model_folder
    requests = {name: tokens for name, tokens in zip("abcde", prompts_for(config, (40, 33, 97, 64, 5), seed=44))}
    replay = Replay(folder, str(tmp_path), dtype, max_tokens=64 * 5)
    try:
        # 1. each request alone and whole
        for name, tokens in requests.items():
            got = replay.send([{"id": name, "tokens": tokens, "want": list(range(len(tokens)))}], end=[name])
            assert got.shape == (len(tokens), config["vocab_size"])
            assert rel_error(got, plain(tokens)) <= TOL[dtype], ("whole", name)
        # 2. the last 32 tokens one by one (requests of at least 33 tokens)
        for name, tokens in requests.items():
            if len(tokens) < 33:
                continue
            head = len(tokens) - 32
            rows = [replay.send([{"id": name, "tokens": tokens[:head], "want": [head - 1]}])]
            for index in range(head, len(tokens)):
                last = index == len(tokens) - 1
                rows.append(replay.send([{"id": name, "tokens": [tokens[index]], "want": [0]}],
                                        end=[name] if last else []))
            assert rel_error(np.concatenate(rows), plain(tokens)[head - 1:]) <= TOL[dtype], ("one by one", name)
        # 3. batches of unequal lengths, one after another in the same cache room; shorter requests end earlier
        for batch in (("a", "e", "b"), ("c", "d"), ("e", "a", "d")):
            split = {name: max(1, len(requests[name]) - 4 - 3 * i) for i, name in enumerate(batch)}
            got = replay.send([{"id": n, "tokens": requests[n][:split[n]], "want": list(range(split[n]))}
                               for n in batch])
            offset = 0
            for n in batch:
                assert rel_error(got[offset:offset + split[n]], plain(requests[n])[:split[n]]) <= TOL[dtype], n
                offset += split[n]
            live, position = list(batch), dict(split)
            while live:
                entries = [{"id": n, "tokens": [requests[n][position[n]]], "want": [0]} for n in live]
                ending = [n for n in live if position[n] + 1 == len(requests[n])]
                got = replay.send(entries, end=ending)
                for row, n in enumerate(live):
                    assert rel_error(got[row], plain(requests[n])[position[n]]) <= TOL[dtype], (batch, n, position[n])
                    position[n] += 1
                live = [n for n in live if n not in ending]
        # a step that wants nothing writes no file; an empty want list is allowed
        assert replay.send([{"id": "z", "tokens": requests["e"], "want": []}], end=["z"]) is None
    finally:
        replay.close()
