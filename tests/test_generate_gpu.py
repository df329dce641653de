"""Greedy and sampled generation through the Python entry point, long decoding, first tokens."""
import numpy as np
import pytest
import torch

from tests.plain.qwen3_plain import PlainQwen3
from tests.tiny_configs import TINY

pytestmark = pytest.mark.gpu


def load(tiny_model_dirs, name, dtype, **kw):
    import ember_b200
    opts = dict(kv_cache_tokens=1024, max_batch_tokens=256, max_seqs=8)
    opts.update(kw)
    return ember_b200.load(tiny_model_dirs[name], dtype=dtype, **opts)


@pytest.mark.parametrize("name", sorted(TINY))
def test_greedy_generation_float32_equals_plain(name, tiny_model_dirs):
    plain = PlainQwen3(tiny_model_dirs[name], torch.float64)
    llm = load(tiny_model_dirs, name, "float32")
    rng = np.random.default_rng(0)
    vocab = TINY[name]["json"]["vocab_size"]
    prompts = [rng.integers(0, vocab, size=n).tolist() for n in (1, 5, 17, 33)]
    if name in ("c", "d"):
        prompts = prompts[:2]                                         # the plain implementation is slow at these widths
    outs = llm.generate(prompts, max_tokens=16, ignore_eos=True)      # batched, continuous batching
    for p, o in zip(prompts, outs):
        assert o == plain.greedy(p, 16)
    assert llm.generate(prompts[-1], max_tokens=16, ignore_eos=True) == outs[-1]  # alone: the same tokens
    assert not any(llm.runner.cache.used_pages())          # one count per cache group


def test_greedy_generation_bfloat16_follows_plain_logits(tiny_model_dirs):
    """bfloat16 may pick another token where two logits are close; every token it picks must be
    within bfloat16 reach of the plain implementation's maximum at that position."""
    name = "a"
    plain = PlainQwen3(tiny_model_dirs[name], torch.float64)
    llm = load(tiny_model_dirs, name, "bfloat16")
    prompt = [5, 100, 37, 8, 250, 11]
    out = llm.generate(prompt, max_tokens=12, ignore_eos=True)
    logits = plain.logits(prompt + out).numpy()
    for i, tok in enumerate(out):
        row = logits[len(prompt) - 1 + i]
        assert row.max() - row[tok] < 0.03 * (row.max() - row.min())


def test_long_decoding_float32(tiny_model_dirs):
    """100 decoded tokens one by one after a short prompt: position 101 must still agree."""
    name = "a"          # position limit 128
    from ember_b200 import StepEntry
    plain = PlainQwen3(tiny_model_dirs[name], torch.float64)
    llm = load(tiny_model_dirs, name, "float32")
    toks = np.random.default_rng(4).integers(0, 512, size=120).tolist()
    want = plain.logits(toks).numpy()
    r = llm.runner
    r.admit("x")
    r.reserve("x", 8)
    r.step([StepEntry("x", toks[:8], ())])
    worst = 0.0
    for t in range(8, 120):
        assert r.reserve("x", 1)
        lg = r.step([StepEntry("x", [toks[t]], (0,))])[0].cpu().numpy()
        worst = max(worst, float(np.linalg.norm(lg - want[t]) / np.linalg.norm(want[t])))
    assert worst < 2e-5


def test_first_tokens_of_a_sequence(tiny_model_dirs):
    """Positions 0, 1, 2 fed one at a time (a one-token prompt included)."""
    from ember_b200 import StepEntry
    for name in sorted(TINY):
        plain = PlainQwen3(tiny_model_dirs[name], torch.float64)
        llm = load(tiny_model_dirs, name, "float32")
        toks = [3, 1, 4]
        want = plain.logits(toks).numpy()
        r = llm.runner
        r.admit("f")
        for t in range(3):
            r.reserve("f", 1)
            lg = r.step([StepEntry("f", [toks[t]], (0,))])[0].cpu().numpy()
            assert np.linalg.norm(lg - want[t]) / np.linalg.norm(want[t]) < 2e-5


def test_temperature_sampling_is_a_function_of_seed_and_position(tiny_model_dirs):
    from ember_b200 import SamplingParams
    llm = load(tiny_model_dirs, "b", "float32")
    sp = SamplingParams(temperature=0.8, top_k=50, top_p=0.95, seed=1234)
    rng = np.random.default_rng(2)
    prompts = [rng.integers(0, 1000, size=n).tolist() for n in (1, 31, 64, 100)]
    together = llm.generate(prompts, sampling=sp, max_tokens=24, ignore_eos=True)
    alone = [llm.generate(p, sampling=sp, max_tokens=24, ignore_eos=True) for p in prompts]
    assert together == alone                                   # the batch does not change the draws
    other = llm.generate(prompts[1], sampling=SamplingParams(temperature=0.8, top_k=50, top_p=0.95, seed=99),
                         max_tokens=24, ignore_eos=True)
    assert other != alone[1]


def test_preemption_on_the_device_keeps_the_tokens(tiny_model_dirs):
    """So few pages that requests are preempted and recomputed: the tokens stay the same."""
    name = "a"
    plain = PlainQwen3(tiny_model_dirs[name], torch.float64)
    llm = load(tiny_model_dirs, name, "float32", kv_cache_tokens=96, max_seqs=4, page_tokens=16)
    rng = np.random.default_rng(8)
    prompts = [rng.integers(0, 512, size=n).tolist() for n in (20, 25, 30, 18)]
    outs = llm.generate(prompts, max_tokens=30, ignore_eos=True)
    assert llm.stats.preemptions > 0
    for p, o in zip(prompts, outs):
        assert o == plain.greedy(p, 30)


@pytest.mark.parametrize("name", ["c", "f"])
def test_preemption_on_the_device_bfloat16_at_the_entry_points_page_size(name, tiny_model_dirs):
    """Preemption and recomputation in bfloat16 with 64-token pages: on heads of 128 (the tcgen05 kernels, "c") and
    with a window group whose pages go back while requests run ("f").  Recomputing a request cuts its tokens into
    other steps than the first pass did, so in bfloat16 a token may differ where two logits are close: every
    token that was picked must be within bfloat16 reach of the plain implementation's maximum at its position,
    and a run with pages to spare must pick tokens of the same quality."""
    plain = PlainQwen3(tiny_model_dirs[name], torch.float64)
    vocab = TINY[name]["json"]["vocab_size"]
    rng = np.random.default_rng(18)
    prompts = [rng.integers(0, vocab, size=n).tolist() for n in (70, 45, 100, 30)]
    for tokens_of_cache, expect_preemption in ((384, True), (4096, False)):
        llm = load(tiny_model_dirs, name, "bfloat16", kv_cache_tokens=tokens_of_cache, max_seqs=4, page_tokens=64,
                   prefill_chunk=48)
        outs = llm.generate(prompts, max_tokens=40, ignore_eos=True)
        llm.runner.check_device()
        assert (llm.stats.preemptions > 0) == expect_preemption
        assert llm.runner.cache.check() == "" and not any(llm.runner.cache.used_pages())
        for p, o in zip(prompts, outs):
            assert len(o) == 40
            logits = plain.logits(p + o).numpy()
            for i, tok in enumerate(o):
                row = logits[len(p) - 1 + i]
                assert row.max() - row[tok] < 0.03 * (row.max() - row.min()), (name, tokens_of_cache, i)


def test_state_slots_under_the_engine_with_preemption():
    """A model whose mixers keep per-request state (a running mean in a state slot) beside attention, generated
    from through the engine with so few pages that requests are preempted and admitted again into used slots:
    the tokens equal those of a run that never preempts.  A slot that is not zeroed at re-admission, or shared,
    changes the running mean and with it the tokens."""
    from ember_b200.config import AttentionSpec, GatedMLPSpec, LayerSpec, ModelSpec, RMSNormSpec, RotarySpec, default_schedule
    from ember_b200.engine.engine import Engine
    from ember_b200.engine.runner import ModelRunner
    from ember_b200.parts import register_part
    from ember_b200.weights import WeightStore, random_tensors
    from tests.test_parts_gpu import RunningMeanSpec, make_running_mean
    register_part("mixer", "toy_running_mean", make_running_mean())
    H, V = 48, 300
    norm = RMSNormSpec(size=H, eps=1e-6)
    attn = AttentionSpec(hidden_size=H, num_heads=3, num_kv_heads=1, head_dim=16, qk_norm=True,
                         position=RotarySpec(head_dim=16, rotary_dim=16, theta=1e4))
    mlp = GatedMLPSpec(hidden_size=H, intermediate_size=80)

    def layer(i, mixer):
        p = f"toy.layers.{i}."
        return LayerSpec.prenorm(mixer=mixer, feed_forward=mlp, mixer_norm=norm, feed_forward_norm=norm,
                                 mixer_prefix=p + "mixer.", feed_forward_prefix=p + "mlp.", mixer_norm_prefix=p + "norm_a.",
                                 feed_forward_norm_prefix=p + "norm_b.")

    spec = ModelSpec(architecture="ToyStateForCausalLM", vocab_size=V, hidden_size=H,
                     layers=(layer(0, RunningMeanSpec(hidden_size=H)), layer(1, attn), layer(2, RunningMeanSpec(hidden_size=H))),
                     schedule=default_schedule(3), final_norm=norm, final_norm_prefix="toy.norm.",
                     embedding_name="toy.embed.weight", head_name="toy.head.weight", tie_embeddings=True, max_positions=512,
                     init_std=0.3)
    weights = dict(random_tensors(spec, seed=6, dtype=torch.float32))
    rng = np.random.default_rng(9)
    prompts = [rng.integers(0, V, size=n).tolist() for n in (20, 25, 30, 18, 40, 12)]
    results = {}
    for capacity in (96, 2048):
        runner = ModelRunner(spec, WeightStore.from_tensors(weights), dtype="float32", capacity_tokens=capacity,
                             max_batch_tokens=128, max_requests=4, page_tokens=16)
        # the toy mixer reads the step's host views (slots, run offsets): it does not declare itself graph-safe,
        # so the runner must not capture decode steps (a replayed graph would keep the slots of the captured step)
        assert not runner.cuda_graphs
        eng = Engine(runner, max_prefill_chunk=24)
        results[capacity] = eng.generate(prompts, max_tokens=30, ignore_eos=True)
        runner.check_device()
        assert (eng.stats.preemptions > 0) == (capacity == 96)
        assert runner.cache.check() == "" and runner.cache.free_slots() == 4
    assert results[96] == results[2048]
    assert len({tuple(o) for o in results[96]}) == len(prompts)          # the requests really differ


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_graph_replay_equals_eager_decoding(dtype, tiny_model_dirs):
    """Decode steps through captured graphs give the logits that eager steps give, while the batch
    changes size and contexts grow across a graph's context bucket."""
    from ember_b200 import StepEntry
    name = "b"
    rng = np.random.default_rng(12)
    seqs = {i: rng.integers(0, 1000, size=n).tolist() for i, n in enumerate((90, 140, 200))}

    def run(graphs):
        llm = load(tiny_model_dirs, name, dtype, cuda_graphs=graphs, kv_cache_tokens=1024)
        r = llm.runner
        r.graph_context_bucket = 64
        out = []
        for i, toks in seqs.items():
            r.admit(i), r.reserve(i, 40)
            r.step([StepEntry(i, toks[:40], ())])
        for t in range(40, 90):                       # three runs decode together, then two, then one
            live = [i for i, toks in seqs.items() if t < len(toks)]
            for i in live:
                assert r.reserve(i, 1)
            lg = r.step([StepEntry(i, [seqs[i][t]], (0,)) for i in live])
            out.append(lg.float().cpu().numpy().copy())
        r.check_device()
        return out, r.graph_replays

    eager, n0 = run(False)
    graphed, n1 = run(True)
    assert n0 == 0 and n1 > 30
    for a, b in zip(eager, graphed):
        assert np.array_equal(a, b) if dtype == "float32" else np.allclose(a, b, rtol=0, atol=1e-2 * np.abs(a).max())


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_pipelined_engine_equals_synchronous_engine(dtype, tiny_model_dirs):
    """Steps launched before the ids of the step in flight are read (tokens resolved on the device from the
    sampler's buffer) give the tokens of the synchronous engine: greedy and seeded sampling, a stop token seen
    one step late, requests of different lengths joining and leaving."""
    from ember_b200 import SamplingParams
    from ember_b200.engine.engine import Engine
    llm = load(tiny_model_dirs, "b", dtype, kv_cache_tokens=2048)
    rng = np.random.default_rng(21)
    prompts = [rng.integers(0, 1000, size=n).tolist() for n in (3, 40, 17, 64, 9)]
    for sp in (SamplingParams(temperature=0.0), SamplingParams(temperature=0.9, top_k=40, top_p=0.9, seed=77)):
        results = {}
        for pipeline in (False, True):
            eng = Engine(llm.runner, max_prefill_chunk=32, pipeline=pipeline)
            assert eng.pipeline == pipeline
            free = eng.generate(prompts, sampling=sp, max_tokens=40, ignore_eos=True)
            stop = free[1][7]                       # a token the second request meets early
            stopped = eng.generate(prompts, sampling=sp, max_tokens=40, stop_tokens=(stop,))
            results[pipeline] = (free, stopped)
            assert llm.runner.cache.used_pages() == [0]
            for f, s in zip(free, stopped):
                assert s == (f[:f.index(stop)] if stop in f else f)
        assert results[True] == results[False]
    llm.runner.check_device()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_captured_residuals_follow_the_plain_layers(dtype, tiny_model_dirs):
    """The residual of a step's last token after the embedding and after every layer (the debugging aid of the
    reference's backend, src/backend/backend.hpp:119-122) against the plain implementation's hidden states:
    a prompt portion, then a single token (which would otherwise go through a graph)."""
    from ember_b200 import StepEntry
    name = "b"
    plain = PlainQwen3(tiny_model_dirs[name], torch.float64)
    toks = np.random.default_rng(3).integers(0, 1000, size=41).tolist()
    want = plain.hidden_states(toks)                        # [layers + 1] of [T, hidden]
    llm = load(tiny_model_dirs, name, dtype)
    r = llm.runner
    with pytest.raises(RuntimeError):
        r.captured_hidden()
    r.set_capture_hidden(True)
    r.admit("x"), r.reserve("x", 40)
    r.step([StepEntry("x", toks[:40], (39,))])
    got = r.captured_hidden()
    assert got.shape == (len(want), want[0].shape[1])
    tol = 2e-5 if dtype == "float32" else 2.5e-2
    for l, h in enumerate(want):
        assert float((got[l].double() - h[39]).norm() / h[39].norm()) < tol, l
    r.reserve("x", 1)
    r.step([StepEntry("x", toks[40:], (0,))])
    got = r.captured_hidden()
    for l, h in enumerate(want):
        assert float((got[l].double() - h[40]).norm() / h[40].norm()) < tol, l
    r.set_capture_hidden(False)
    assert r.graph_replays == 0


def test_bfloat16_logits_alone_and_in_a_batch_of_ten(tiny_model_dirs):
    """In bfloat16 a step of up to 8 tokens (and a portion of 512 or more) norms and rotates the heads on the fp32
    accumulator in the q/k/v product's epilogue, while a step of 9 to 511 tokens rounds the product to bfloat16
    first and finishes the heads in a kernel of its own.  The keys a request caches and its logits therefore
    differ by a rounding with the company it keeps; they must stay within bfloat16's tolerance of the plain
    implementation, and of each other, either way."""
    from ember_b200 import StepEntry
    name = "c"                                     # heads of 128: the fused epilogue applies
    plain = PlainQwen3(tiny_model_dirs[name], torch.float64)
    rng = np.random.default_rng(33)
    vocab = TINY[name]["json"]["vocab_size"]
    seqs = [rng.integers(0, vocab, size=40).tolist() for _ in range(10)]
    want = plain.logits(seqs[0]).numpy()

    def decode(n_requests):
        llm = load(tiny_model_dirs, name, "bfloat16", max_seqs=16, kv_cache_tokens=2048)
        r = llm.runner
        for i in range(n_requests):
            r.admit(i), r.reserve(i, 20)
        r.step([StepEntry(i, seqs[i][:20], ()) for i in range(n_requests)])
        rows = []
        for t in range(20, 40):                     # single tokens: 1 run a step (fused) or 10 (separate kernel)
            for i in range(n_requests):
                assert r.reserve(i, 1)
            lg = r.step([StepEntry(i, [seqs[i][t]], (0,)) for i in range(n_requests)])
            rows.append(lg[0].float().cpu().numpy().copy())
        r.check_device()
        return np.stack(rows)

    alone, together = decode(1), decode(10)
    rel = lambda a, b: float(np.linalg.norm(a - b) / np.linalg.norm(b))          # noqa: E731
    assert max(rel(alone[i], want[20 + i]) for i in range(20)) < 2.5e-2
    assert max(rel(together[i], want[20 + i]) for i in range(20)) < 2.5e-2
    assert max(rel(together[i], alone[i]) for i in range(20)) < 2.5e-2


@pytest.mark.parametrize("name", ["c", "d"])
def test_decode_key_splits_merged_in_a_cluster_or_by_the_merge_kernel(name, tiny_model_dirs, monkeypatch):
    """Single tokens after 300 to 500 keys: the planner cuts the keys in two.  Whether the two blocks of a tile
    merge in shared memory as a cluster or through buffers and the merge kernel, the logits follow the plain
    implementation and differ from each other by the merge's rounding only."""
    from ember_b200 import StepEntry
    from ember_b200.parts.attention import Attention
    plain = PlainQwen3(tiny_model_dirs[name], torch.float64)
    rng = np.random.default_rng(77)
    vocab = TINY[name]["json"]["vocab_size"]
    seqs = [rng.integers(0, vocab, size=n).tolist() for n in (330, 470, 505)]
    want = [plain.logits(s).numpy() for s in seqs]

    def decode(in_cluster):
        monkeypatch.setattr(Attention, "CLUSTER_MERGE", in_cluster)
        llm = load(tiny_model_dirs, name, "bfloat16", max_seqs=4, kv_cache_tokens=2048, max_batch_tokens=2048)
        r = llm.runner
        for i, s in enumerate(seqs):
            r.admit(i), r.reserve(i, len(s) - 6)
        r.step([StepEntry(i, s[:-6], ()) for i, s in enumerate(seqs)])
        rows = []
        for t in range(6, 0, -1):
            for i in range(len(seqs)):
                assert r.reserve(i, 1)
            lg = r.step([StepEntry(i, [s[-t]], (0,)) for i, s in enumerate(seqs)])
            rows.append(lg.float().cpu().numpy().copy())
        r.check_device()
        return np.stack(rows)                      # [6 steps, 3 requests, vocab]

    a, b = decode(True), decode(False)
    rel = lambda x, y: float(np.linalg.norm(x - y) / np.linalg.norm(y))          # noqa: E731
    for step in range(6):
        for i, s in enumerate(seqs):
            ref = want[i][len(s) - 6 + step]
            assert rel(a[step, i], ref) < 2.5e-2 and rel(b[step, i], ref) < 2.5e-2
            assert rel(a[step, i], b[step, i]) < 5e-3
