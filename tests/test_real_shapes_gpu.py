"""Layers of the published Qwen3 sizes (0.6B, 1.7B, 8B widths; few layers, random weights) against the
plain implementation: the shapes the benchmark times are the shapes whose logits are checked here."""
import numpy as np
import pytest
import torch

from ember_b200.config import Qwen3Config
from ember_b200.weights import write_model_dir
from tests.plain.qwen3_plain import PlainQwen3
from tests.replay_helpers import (collect, first_mismatch, max_live_tokens, trace_mixed, trace_portions,
                                  trace_tail_decode, trace_whole)
from tests.test_replay_gpu import TOL, replay

pytestmark = pytest.mark.gpu


def _json(**kw):
    base = dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", head_dim=128, rope_theta=1000000.0,
                rms_norm_eps=1e-6, max_position_embeddings=4096, attention_bias=False)
    base.update(kw)
    return base


SHAPES = {
    "0.6b": _json(vocab_size=32064, hidden_size=1024, intermediate_size=3072, num_hidden_layers=2,
                  num_attention_heads=16, num_key_value_heads=8, tie_word_embeddings=True),
    "1.7b": _json(vocab_size=151936, hidden_size=2048, intermediate_size=6144, num_hidden_layers=2,
                  num_attention_heads=16, num_key_value_heads=8, tie_word_embeddings=True),
    "8b": _json(vocab_size=32064, hidden_size=4096, intermediate_size=12288, num_hidden_layers=1,
                num_attention_heads=32, num_key_value_heads=8, tie_word_embeddings=False),
}


@pytest.fixture(scope="module")
def shape_dirs(tmp_path_factory):
    made = {}

    def get(name):
        if name not in made:
            d = str(tmp_path_factory.mktemp(f"shape_{name.replace('.', '_')}"))
            write_model_dir(Qwen3Config.from_json(SHAPES[name]), d, seed=7, dtype=torch.bfloat16, std=0.02, norm_std=0.05)
            rng = np.random.default_rng(3)
            reqs = {f"r{i}": rng.integers(0, SHAPES[name]["vocab_size"], size=n).tolist() for i, n in enumerate((97, 40, 66))}
            plain = PlainQwen3(d, torch.float32)
            made[name] = (d, reqs, {rid: plain.logits(t).numpy() for rid, t in reqs.items()})
        return made[name]

    return get


@pytest.mark.parametrize("page", [16, 64])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("mode", ["whole", "tail", "portions", "mixed"])
@pytest.mark.parametrize("name", sorted(SHAPES))
def test_published_layer_sizes(name, mode, dtype, page, shape_dirs):
    model_dir, requests, want = shape_dirs(name)
    steps = {"whole": trace_whole, "tail": trace_tail_decode, "portions": trace_portions,
             "mixed": lambda r: trace_mixed(r, live=3, seed=2)}[mode](requests)
    outputs = replay(model_dir, dtype, steps, max_live_tokens(steps), page_tokens=page)
    got = collect(steps, outputs)
    for rid, toks in requests.items():
        assert sorted(got[rid]) == list(range(len(toks)))
    first, worst = first_mismatch(got, want, TOL[dtype])
    print(f"{name} {dtype} {mode} page {page}: worst relative error {worst:.3e}")
    assert first is None, f"first wrong position (request, position, error): {first}; worst {worst:.3e}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_context_in_portions_then_token_by_token(dtype, shape_dirs):
    """8,224 tokens at the benchmark's layer widths with the entry point's 64-token pages: four portions of 2,048
    (each q/k/v product finishes its heads in the epilogue; every portion's attention reads the pages the earlier
    ones wrote), then 32 single tokens over more than 8,192 keys (the key range cut into the most splits the
    planner makes).  The last row of every portion and every decoded row against the plain implementation (the
    reference's counterpart feeds 300 / 37 / 363 tokens from block 3: tests/test_model.cpp:124-157)."""
    from tests.plain.qwen3_plain import linear, rmsnorm
    from ember_b200.engine.replay import TraceReplayer
    from ember_b200.engine.runner import ModelRunner
    from tests.replay_helpers import rel_err
    import tempfile
    model_dir, _, _ = shape_dirs("1.7b")
    rng = np.random.default_rng(21)
    n, portion, tail = 8224, 2048, 32
    toks = rng.integers(0, SHAPES["1.7b"]["vocab_size"], size=n).tolist()
    plain = PlainQwen3(model_dir, torch.float32)
    rows = [portion * (i + 1) - 1 for i in range((n - tail) // portion)] + list(range(n - tail, n))
    h = plain.hidden_states(toks)[-1][rows]
    ref = linear(rmsnorm(h, plain.w["model.norm.weight"], plain.cfg["eps"]), plain.w["model.embed_tokens.weight"]).numpy()
    steps, at = [], 0
    while at < n - tail:
        steps.append({"step": len(steps), "entries": [{"id": "a", "tokens": toks[at:at + portion], "want": [portion - 1]}],
                      "end": []})
        at += portion
    assert at == n - tail
    for t in range(at, n):
        steps.append({"step": len(steps), "entries": [{"id": "a", "tokens": [toks[t]], "want": [0]}],
                      "end": ["a"] if t == n - 1 else []})
    # the model's position limit in the test folder is 4,096; the long request needs more
    import json, os, shutil
    with tempfile.TemporaryDirectory() as long_dir:
        for f in os.listdir(model_dir):
            if f != "config.json":
                os.symlink(os.path.join(model_dir, f), os.path.join(long_dir, f))
        with open(os.path.join(model_dir, "config.json")) as f:
            cfg = json.load(f)
        cfg["max_position_embeddings"] = 16384
        with open(os.path.join(long_dir, "config.json"), "w") as f:
            json.dump(cfg, f)
        runner = ModelRunner.from_dir(long_dir, dtype=dtype, capacity_tokens=n + 96, max_batch_tokens=portion,
                                      max_requests=2, page_tokens=64)
        with tempfile.TemporaryDirectory() as out:
            rp = TraceReplayer(runner, out)
            got = np.concatenate([rp.run_step(s) for s in steps])
        runner.check_device()
    errs = [rel_err(got[i], ref[i]) for i in range(len(rows))]
    print(f"long context {dtype}: worst relative error {max(errs):.3e} at row {rows[int(np.argmax(errs))]}")
    assert max(errs) <= TOL[dtype], errs


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_prompt_at_the_benchmark_shape(dtype, shape_dirs):
    """2,100 tokens in one step (many attention tiles, split keys afterwards), then single tokens: the last
    prompt position and every decoded position against the plain implementation."""
    from tests.plain.qwen3_plain import linear, rmsnorm
    model_dir, _, _ = shape_dirs("1.7b")
    rng = np.random.default_rng(11)
    toks = rng.integers(0, SHAPES["1.7b"]["vocab_size"], size=2108).tolist()
    head = 2100
    plain = PlainQwen3(model_dir, torch.float32)
    rows = list(range(head - 1, len(toks)))
    h = plain.hidden_states(toks)[-1][rows]
    ref = linear(rmsnorm(h, plain.w["model.norm.weight"], plain.cfg["eps"]), plain.w["model.embed_tokens.weight"]).numpy()
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": toks[:head], "want": [head - 1]}], "end": []}]
    for i, t in enumerate(range(head, len(toks))):
        steps.append({"step": i + 1, "entries": [{"id": "a", "tokens": [toks[t]], "want": [0]}],
                      "end": ["a"] if t == len(toks) - 1 else []})
    from ember_b200.engine.replay import TraceReplayer
    from ember_b200.engine.runner import ModelRunner
    import tempfile
    runner = ModelRunner.from_dir(model_dir, dtype=dtype, capacity_tokens=2176, max_batch_tokens=2176, max_requests=2)
    with tempfile.TemporaryDirectory() as out:
        rp = TraceReplayer(runner, out)
        got = np.concatenate([rp.run_step(s) for s in steps])
    from tests.replay_helpers import rel_err
    errs = [rel_err(got[i], ref[i]) for i in range(len(rows))]
    print(f"long prompt {dtype}: worst relative error {max(errs):.3e}")
    assert max(errs) <= TOL[dtype], errs


def test_portions_with_and_without_the_fused_head_epilogue_agree(shape_dirs):
    """A 700-token prompt in one step (the q/k/v product finishes the heads in its epilogue) and in portions of
    350 and of 600 + 100 (the shorter ones take the separate head kernel): the logits at positions of every
    portion agree with the plain implementation and with each other, whichever path wrote the cache."""
    from ember_b200 import ops
    from ember_b200.engine.replay import TraceReplayer
    from ember_b200.engine.runner import ModelRunner
    from tests.replay_helpers import rel_err
    import tempfile
    model_dir, _, _ = shape_dirs("0.6b")
    rng = np.random.default_rng(5)
    toks = rng.integers(0, SHAPES["0.6b"]["vocab_size"], size=700).tolist()
    rows = [5, 349, 350, 599, 600, 699]
    ref = PlainQwen3(model_dir, torch.float32).logits(toks).numpy()[rows]
    assert ops.QKV_FUSE_MIN_TOKENS <= 600
    results = []
    for cuts in ([700], [350, 350], [600, 100]):
        runner = ModelRunner.from_dir(model_dir, dtype="bfloat16", capacity_tokens=768, max_batch_tokens=768, max_requests=2)
        steps, at = [], 0
        for i, n in enumerate(cuts):
            want = [r - at for r in rows if at <= r < at + n]
            steps.append({"step": i, "entries": [{"id": "a", "tokens": toks[at:at + n], "want": want}],
                          "end": ["a"] if at + n == len(toks) else []})
            at += n
        with tempfile.TemporaryDirectory() as out:
            rp = TraceReplayer(runner, out)
            got = np.concatenate([rp.run_step(s) for s in steps])
        errs = [rel_err(got[i], ref[i]) for i in range(len(rows))]
        assert max(errs) <= TOL["bfloat16"], (cuts, errs)
        results.append(got)
    for other in results[1:]:
        assert max(rel_err(other[i], results[0][i]) for i in range(len(rows))) <= TOL["bfloat16"]


@pytest.mark.parametrize("n_requests", [24, 70])
@pytest.mark.parametrize("name", ["1.7b", "8b"])
def test_many_requests_decode_together_at_published_sizes(name, n_requests, shape_dirs):
    """24 and 70 requests of different lengths decode side by side in bfloat16: steps of 17 to 128 tokens are the
    ones where the q/k/v product leaves fp32 sums for the head kernel, the other products add their parts of K with
    atomics, and the LM head (K in one part) turns its tile in shared memory.  Every request's rows against the
    plain implementation, and the same request alone against itself in the crowd."""
    from ember_b200 import StepEntry
    from ember_b200.engine.runner import ModelRunner
    model_dir, _, _ = shape_dirs(name)
    rng = np.random.default_rng(5 + n_requests)
    vocab = SHAPES[name]["vocab_size"]
    lens = [int(x) for x in rng.integers(9, 80, size=n_requests)]
    seqs = [rng.integers(0, vocab, size=n + 4).tolist() for n in lens]
    plain = PlainQwen3(model_dir, torch.float32)
    check = [0, 1, n_requests // 2, n_requests - 1]                  # requests whose rows are compared
    want = {i: plain.logits(seqs[i]).numpy() for i in check}

    def run(which):
        r = ModelRunner.from_dir(model_dir, dtype="bfloat16", capacity_tokens=64 * (len(which) + 2) * 2, max_batch_tokens=2048,
                                 max_requests=len(which), page_tokens=64)
        for i in which:
            assert r.admit(i) and r.reserve(i, lens[i])
        for a in range(0, len(which), 20):                                      # the prompts, twenty requests a step
            r.step([StepEntry(i, seqs[i][:lens[i]], ()) for i in which[a:a + 20]])
        rows = {i: [] for i in which}
        for t in range(4):
            for i in which:
                assert r.reserve(i, 1)
            lg = r.step([StepEntry(i, [seqs[i][lens[i] + t]], (0,)) for i in which]).float().cpu().numpy()
            for j, i in enumerate(which):
                rows[i].append(lg[j].copy())
        r.check_device()
        return rows

    crowd = run(list(range(n_requests)))
    alone = run([check[2]])
    rel = lambda a, b: float(np.linalg.norm(a - b) / np.linalg.norm(b))          # noqa: E731
    worst = 0.0
    for i in check:
        for t in range(4):
            worst = max(worst, rel(crowd[i][t], want[i][lens[i] + t]))
    print(f"{name}, {n_requests} requests: worst relative error {worst:.3e}")
    assert worst <= TOL["bfloat16"]
    assert max(rel(crowd[check[2]][t], alone[check[2]][t]) for t in range(4)) <= TOL["bfloat16"]
