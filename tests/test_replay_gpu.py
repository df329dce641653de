"""The engine against the plain implementation under every way of cutting the work,
in float32 and in bfloat16, on the two tiny configurations."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

from tests.plain.qwen3_plain import PlainQwen3
from tests.replay_helpers import (collect, first_mismatch, max_live_tokens, trace_mixed, trace_portions,
                                  trace_tail_decode, trace_whole)
from tests.tiny_configs import TINY

pytestmark = pytest.mark.gpu

TOL = {"float32": 2e-5, "bfloat16": 2.5e-2}
ROOT = os.path.join(os.path.dirname(os.path.abspath(__file__)), "..")


def make_requests(name: str, lengths, seed: int):
    rng = np.random.default_rng(seed)
    vocab = TINY[name]["json"]["vocab_size"]
    return {f"r{i}": rng.integers(0, vocab, size=n).tolist() for i, n in enumerate(lengths)}


@pytest.fixture(scope="module")
def plain_logits(tiny_model_dirs):
    cache = {}

    def get(name, requests):
        out = {}
        for rid, toks in requests.items():
            key = (name, tuple(toks))
            if key not in cache:
                cache[key] = PlainQwen3(tiny_model_dirs[name], torch.float64).logits(toks).numpy()
            out[rid] = cache[key]
        return out

    return get


def replay(model_dir, dtype, steps, capacity, page_tokens=16, max_batch_tokens=512):
    from ember_b200.engine.replay import TraceReplayer
    from ember_b200.engine.runner import ModelRunner
    import tempfile
    runner = ModelRunner.from_dir(model_dir, dtype=dtype, capacity_tokens=capacity, max_batch_tokens=max_batch_tokens,
                                  max_requests=8, page_tokens=page_tokens)
    with tempfile.TemporaryDirectory() as out:
        rp = TraceReplayer(runner, out)
        outputs = {}
        for s in steps:
            got = rp.run_step(s)
            if got is not None:
                outputs[s["step"]] = got.copy()
            assert runner.cache.check() == ""
    assert runner.cache.used_pages() == [0] * len(runner.cache.groups)
    return outputs


LENGTHS = {"a": (5, 17, 33, 100), "b": (1, 31, 64, 100, 130), "c": (3, 70, 200, 333), "d": (2, 65, 129, 260),
           "e": (4, 47, 97, 150), "f": (3, 24, 25, 77, 160)}


@pytest.mark.parametrize("page", [16, 32, 64])          # 16: the reference's block; 64: what the entry point and the benchmark use
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(TINY))
@pytest.mark.parametrize("mode", ["whole", "tail", "portions", "mixed"])
def test_replay_modes(name, dtype, mode, page, tiny_model_dirs, plain_logits):
    requests = make_requests(name, LENGTHS[name], seed=5)
    if mode == "mixed":
        requests = make_requests(name, LENGTHS[name] + (70, 45, 90, 12), seed=6)
    steps = {"whole": trace_whole, "tail": trace_tail_decode, "portions": trace_portions,
             "mixed": lambda r: trace_mixed(r, live=4, seed=3)}[mode](requests)
    capacity = max_live_tokens(steps)          # so few pages that they are used again (whole pages at every size)
    outputs = replay(tiny_model_dirs[name], dtype, steps, capacity, page_tokens=page)
    got = collect(steps, outputs)
    want = plain_logits(name, requests)
    assert set(got) == set(requests)
    for rid, toks in requests.items():
        assert sorted(got[rid]) == list(range(len(toks)))
    first, worst = first_mismatch(got, want, TOL[dtype])
    print(f"{name} {dtype} {mode} page {page}: worst relative error {worst:.3e}")
    assert first is None, f"first wrong position (request, position, error): {first}; worst {worst:.3e}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_run_program(dtype, tiny_model_dirs, plain_logits, tmp_path):
    """The program itself, as a user runs it: stdin lines in, files and 'done' lines out."""
    name = "b"
    requests = make_requests(name, (40, 75, 33), seed=9)
    steps = trace_mixed(requests, live=2, seed=1)
    out = tmp_path / "out"
    proc = subprocess.run(
        [sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", tiny_model_dirs[name], "--dtype", dtype,
         "--out", str(out), "--max-tokens", str(max_live_tokens(steps))],
        input="".join(json.dumps(s) + "\n" for s in steps), capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert [l for l in proc.stdout.splitlines() if l.startswith("done ")] == [f"done {s['step']}" for s in steps]
    vocab = TINY[name]["json"]["vocab_size"]
    outputs = {s["step"]: np.fromfile(out / f"{s['step']}.f32", dtype="<f4").reshape(-1, vocab) for s in steps}
    first, worst = first_mismatch(collect(steps, outputs), plain_logits(name, requests), TOL[dtype])
    assert first is None, f"{first}, worst {worst:.3e}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_replay_odd_records(dtype, tiny_model_dirs, plain_logits):
    """Records at the edges of the format: a step larger than the runner's batch limit (run as several
    batches), a place wanted twice and out of order, nothing wanted, an entry without tokens, a request
    left out of a step, an unknown id in ``end``, an id used again after its end."""
    from ember_b200.engine.replay import TraceReplayer
    from ember_b200.engine.runner import ModelRunner
    import tempfile
    name = "b"
    reqs = make_requests(name, (150, 90), seed=9)
    a, b = reqs["r0"], reqs["r1"]
    want = plain_logits(name, reqs)
    runner = ModelRunner.from_dir(tiny_model_dirs[name], dtype=dtype, capacity_tokens=256, max_batch_tokens=48,
                                  max_requests=4)
    tol = TOL[dtype]

    def close(got, ref):
        assert np.abs(got - ref).max() <= tol * max(1.0, np.abs(ref).max())

    with tempfile.TemporaryDirectory() as out:
        rp = TraceReplayer(runner, out)
        # 190 tokens in one step under a limit of 48; wants out of order, one twice, across the cuts
        got = rp.run_step({"step": 0, "entries": [{"id": "x", "tokens": a[:120], "want": [119, 0, 47, 48, 119]},
                                                  {"id": "y", "tokens": b[:70], "want": [69, 3]}], "end": ["nobody"]})
        assert got.shape[0] == 7 and os.path.getsize(os.path.join(out, "0.f32")) == got.size * 4
        for row, (rid, pos) in enumerate([("r0", 119), ("r0", 0), ("r0", 47), ("r0", 48), ("r0", 119), ("r1", 69),
                                          ("r1", 3)]):
            close(got[row], want[rid][pos])
        # y is left out; x wants nothing; an entry without tokens is skipped
        assert rp.run_step({"step": 1, "entries": [{"id": "x", "tokens": a[120:149], "want": []},
                                                   {"id": "z", "tokens": [], "want": []}], "end": []}) is None
        assert not os.path.exists(os.path.join(out, "1.f32"))
        got = rp.run_step({"step": 2, "entries": [{"id": "y", "tokens": b[70:], "want": [19]},
                                                  {"id": "x", "tokens": a[149:], "want": [0]}], "end": ["x", "y"]})
        close(got[0], want["r1"][89])
        close(got[1], want["r0"][149])
        assert runner.cache.used_pages() == [0]
        # the id comes again: a new request
        got = rp.run_step({"step": 3, "entries": [{"id": "x", "tokens": b[:40], "want": [39]}], "end": ["x"]})
        close(got[0], want["r1"][39])
        from ember_b200.engine.replay import ReplayError
        with pytest.raises(ReplayError):
            rp.run_step({"step": 4, "entries": [{"id": "q", "tokens": [1, 2], "want": [2]}], "end": []})
    assert runner.cache.check() == ""
