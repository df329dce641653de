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
    assert (a.gpu_memory, a.kv_cache_mib, a.page_tokens, a.max_context) == (0.92, 0, 64, 0)
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


# ------------------------------------------------------------------- the commands as a user runs them
def _run(argv, timeout=600):
    import subprocess
    import sys
    root = os.path.join(os.path.dirname(os.path.abspath(__file__)), "..")
    return subprocess.run([sys.executable, "-m", "ember_b200"] + argv, capture_output=True, text=True, timeout=timeout,
                          cwd=root)


@pytest.mark.gpu
@pytest.mark.parametrize("name,extra", [("a", []), ("b", ["--page-tokens", "16", "--kv-cache-tokens", "512"]),
                                        ("c", ["--gpu-memory", "0.5", "--max-context", "200", "-v"])])
def test_generate_command_float32_equals_plain(name, extra, tiny_model_dirs):
    """`python -m ember_b200 generate -m DIR -p "ids" --greedy` in a process of its own: the ids it prints are the
    plain implementation's greedy tokens (the reference's cmd_generate: tools/ember_main.cpp:135-158).  With
    --gpu-memory the cache is sized from the device's free memory."""
    import torch
    from tests.plain.qwen3_plain import PlainQwen3
    prompt = [7, 3, 200, 41, 5, 99, 150]
    proc = _run(["generate", "-m", tiny_model_dirs[name], "-p", " ".join(map(str, prompt)), "--greedy", "--dtype", "float32",
                 "-n", "12", "--ignore-eos", "--max-seqs", "4"] + extra)
    assert proc.returncode == 0, proc.stderr[-2000:]
    got = [int(t) for t in proc.stdout.split()]
    assert got == PlainQwen3(tiny_model_dirs[name], torch.float64).greedy(prompt, 12)
    assert "tokens/s" in proc.stderr
    if "-v" in extra:
        assert "cache:" in proc.stderr and "context limit 200" in proc.stderr


@pytest.mark.gpu
def test_generate_command_samples_by_seed(tiny_model_dirs):
    """Sampling options reach the sampler: the same seed gives the same ids, another seed other ids."""
    base = ["generate", "-m", tiny_model_dirs["b"], "-p", "5,6,7,8", "--temp", "0.9", "--top-k", "50", "--top-p", "0.95",
            "-n", "16", "--ignore-eos", "--max-seqs", "2", "--kv-cache-tokens", "256"]
    a, b, c = _run(base + ["--seed", "5"]), _run(base + ["--seed", "5"]), _run(base + ["--seed", "6"])
    assert a.returncode == b.returncode == c.returncode == 0, a.stderr[-2000:]
    assert a.stdout == b.stdout and a.stdout != c.stdout and len(a.stdout.split()) == 16


@pytest.mark.gpu
def test_bench_command(tiny_model_dirs):
    """`bench -m DIR prompt=64 gen=8 batch=1,4`: the reference's table (tools/ember_main.cpp:323-414) with numbers in it."""
    proc = _run(["bench", "-m", tiny_model_dirs["c"], "prompt=64", "gen=8", "batch=1,4", "--max-seqs", "8",
                 "--kv-cache-tokens", "2048"])
    assert proc.returncode == 0, proc.stderr[-2000:]
    out = proc.stdout
    assert "prefill, 64-token prompt" in out and " 1 sequence  x 8 tokens" in out and " 4 sequences x 8 tokens" in out
    rates = [float(x) for x in __import__("re").findall(r"([0-9.]+) t/s", out)]
    assert len(rates) == 4 and all(r > 0 for r in rates)
    assert "steps, 0 preemptions" in out
