"""The command line's own decisions, without a device: the random-weights mode writes a folder that `info` reads
back, and what is wrong with an argument comes as one `error:` line and exit code 2, not as a traceback."""
import json

import pytest
import torch

import plain_llama as P
from etalii.dllm_b200.cli import main


@pytest.fixture()
def config_file(tmp_path):
    path = tmp_path / "tiny.json"
    path.write_text(json.dumps(dict(P.TINY_B)))
    return path


def test_random_writes_a_folder_that_info_reads(config_file, tmp_path, capsys):
    out = tmp_path / "model"
    assert main(["random", "--config", str(config_file), "--seed", "3", "--out", str(out)]) == 0
    assert (out / "config.json").is_file() and (out / "model.safetensors").is_file()
    capsys.readouterr()
    assert main(["--model", str(out), "info"]) == 0
    shown = json.loads(capsys.readouterr().out)
    assert shown["hidden_size"] == P.TINY_B["hidden_size"] and shown["vocab_size"] == P.TINY_B["vocab_size"]


@pytest.mark.parametrize("argv,words", [
    (["random", "--config", "/nonexistent/config.json", "--out", "unused"], "No such file"),
    (["info"], "--model is required"),
    (["--model", "/nonexistent/model", "info"], "config.json"),
])
def test_wrong_arguments_are_one_error_line(argv, words, capsys):
    assert main(argv) == 2
    err = capsys.readouterr().err
    assert err.startswith("error:") and words in err and "Traceback" not in err


def test_a_refused_configuration_is_an_error_line(tmp_path, capsys):
    path = tmp_path / "bad.json"
    path.write_text(json.dumps(dict(P.TINY_A, hidden_act="gelu")))
    assert main(["random", "--config", str(path), "--out", str(tmp_path / "m")]) == 2
    assert "gelu" in capsys.readouterr().err


def test_prompts_that_are_not_ids_and_missing_prompts(config_file, tmp_path, capsys):
    out = tmp_path / "model"
    assert main(["random", "--config", str(config_file), "--out", str(out)]) == 0
    assert main(["--model", str(out), "generate", "--prompt-ids", "1,x"]) == 2
    assert "token ids" in capsys.readouterr().err
    assert main(["--model", str(out), "generate"]) == 2
    assert "--prompt-ids" in capsys.readouterr().err
    assert main(["--model", str(out), "generate", "--prompt-ids", "1", "--n", "0"]) == 2
    assert main(["--model", str(out), "generate", "--prompt-ids", "1", "--top-p", "0"]) == 2
    if not torch.cuda.is_available():
        assert main(["--model", str(out), "generate", "--prompt-ids", "1,2"]) == 2
        assert "no CUDA device" in capsys.readouterr().err


def test_generate_options_have_the_reference_names():
    """src/etalii_dllm/cli.py:357-431: the length controls and sampling options of `generate`."""
    from etalii.dllm_b200.cli import build_parser

    args = build_parser().parse_args(
        ["--model", "m", "--dtype", "float32", "generate", "--prompt-ids", "1,2", "--max-tokens", "9", "--temperature",
         "0.7", "--top-k", "5", "--top-p", "0.9", "--min-p", "0.1", "--seed", "4", "--n", "2", "--min-tokens", "3",
         "--ignore-eos", "--stop-token-id", "7", "--stop-token-id", "8"])
    assert (args.max_tokens, args.temperature, args.top_k, args.top_p, args.min_p, args.seed, args.n) == \
        (9, 0.7, 5, 0.9, 0.1, 4, 2)
    assert args.min_tokens == 3 and args.ignore_eos and args.stop_token_id == [7, 8]
