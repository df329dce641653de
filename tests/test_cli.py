"""The command line: option names and defaults (the reference's, tools/cli_args.hpp:57-88), and the commands
that need no GPU."""
import json
import os

import pytest

from ember_b200.cli import _ids, _parser, main
from tests.tiny_configs import tiny_config


def test_option_names_and_defaults():
    a = _parser().parse_intermixed_args(["generate", "-m", "DIR", "-p", "1 2 3"])
    assert (a.model, a.prompt, a.max_tokens, a.temp, a.top_p, a.top_k, a.min_p) == ("DIR", "1 2 3", 512, 0.7, 0.8, 20, 0.0)
    assert (a.max_batch_tokens, a.max_seqs, a.kv_cache_tokens, a.greedy, a.dtype) == (2048, 64, 0, False, "bfloat16")
    a = _parser().parse_intermixed_args(["gen", "--model", "D", "--temperature", "0.5", "--top-k", "5", "--top-p", "0.9",
                                         "--min-p", "0.1", "--seed", "7", "-n", "9", "--greedy", "--no-cuda-graphs"])
    assert (a.temp, a.top_k, a.top_p, a.min_p, a.seed, a.max_tokens, a.greedy, a.no_cuda_graphs) == (0.5, 5, 0.9, 0.1, 7, 9, True, True)


def test_positionals_may_follow_options():
    a = _parser().parse_intermixed_args(["bench", "-m", "DIR", "prompt=512", "gen=32", "batch=1,8"])
    assert a.command == "bench" and a.model == "DIR" and a.rest == ["prompt=512", "gen=32", "batch=1,8"]
    a = _parser().parse_intermixed_args(["gen", "5 6 7", "-m", "DIR"])
    assert a.rest == ["5 6 7"]


def test_token_ids():
    assert _ids("1 2,3\n4 ,5") == [1, 2, 3, 4, 5] and _ids("  ") == []


def test_random_then_info(tmp_path, capsys):
    cfg = tmp_path / "config.json"
    cfg.write_text(json.dumps(tiny_config("a").to_json()))
    out = tmp_path / "model"
    assert main(["random", "--config", str(cfg), "--out", str(out), "--seed", "3"]) == 0
    assert sorted(os.listdir(out)) == ["config.json", "model.safetensors"]
    capsys.readouterr()
    assert main(["info", "-m", str(out)]) == 0
    text = capsys.readouterr().out
    assert "qwen3" in text and "2 layers" in text and "KV cache per token" in text


def test_errors_are_messages_not_tracebacks(tmp_path, capsys):
    assert main(["info", "-m", str(tmp_path / "nothing_here")]) == 1
    assert "error:" in capsys.readouterr().err
    with pytest.raises(SystemExit):
        main(["generate", "-p", "1 2 3"])                      # no model folder
    with pytest.raises(SystemExit):
        main(["random", "--out", str(tmp_path / "x")])         # no configuration
