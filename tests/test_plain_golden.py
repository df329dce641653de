"""The plain implementation and the host sampler against the reference's own CPU code (numbers made once by
tests/golden/make_golden.py, with the tiny models' tensors stored beside them) and the plain implementation
against itself in float32."""
import json
import os

import numpy as np
import pytest
import torch

from tests.plain.qwen3_plain import PlainQwen3
from tests.tiny_configs import GOLDEN_CONFIGS, TINY, tiny_prompts

GOLDEN = os.path.join(os.path.dirname(__file__), "golden", "qwen3_reference_logits.npz")


def _rel(a, b):
    a, b = np.asarray(a, dtype=np.float64), np.asarray(b, dtype=np.float64)
    return float(np.linalg.norm(a - b) / max(np.linalg.norm(b), 1e-30))


def golden_model_dir(g, name, out_dir):
    """The model folder the golden logits were made with, rebuilt from the tensors stored beside them."""
    from ember_b200.weights import save_file
    from tests.tiny_configs import tiny_config
    prefix = f"{name}.tensor."
    tensors = {k[len(prefix):]: torch.from_numpy(g[k].copy()).view(torch.bfloat16) for k in g.files if k.startswith(prefix)}
    os.makedirs(out_dir, exist_ok=True)
    with open(os.path.join(out_dir, "config.json"), "w") as f:
        json.dump(tiny_config(name).to_json(), f)
    save_file(tensors, os.path.join(out_dir, "model.safetensors"))
    return out_dir


@pytest.mark.parametrize("name", GOLDEN_CONFIGS)
def test_plain_matches_reference_cpu_backend(name, tmp_path):
    g = np.load(GOLDEN)
    mdir = golden_model_dir(g, name, str(tmp_path / name))
    plain = PlainQwen3(mdir, dtype=torch.float64)
    for pi, prompt in enumerate(tiny_prompts(name)):
        assert list(g[f"{name}.p{pi}.tokens"]) == prompt
        logits = plain.logits(prompt).numpy()
        whole = g[f"{name}.p{pi}.whole"][0]
        assert _rel(logits[-1], whole) < 2e-6
        assert int(np.argmax(logits[-1])) == int(np.argmax(whole))
        # the reference fed in chunks of 7 from physical block 2: row i is the last token of chunk i
        chunked = g[f"{name}.p{pi}.chunk7_block2"]
        ends = [min(len(prompt), s + 7) - 1 for s in range(0, len(prompt), 7)]
        for row, e in zip(chunked, ends):
            assert _rel(logits[e], row) < 2e-6


def test_host_sampler_draws_the_reference_tokens():
    """ember_b200/sampling/host.py against tokens the reference's sample_host drew
    (src/backend/sampling_host.cpp:68-85) for 180 (logits row, parameters, seed, counter) cases, and the size of
    the kept set against its sampling_distribution."""
    from ember_b200.sampling import SamplingParams, sample_host, sampling_distribution
    g = np.load(GOLDEN)
    logits, cases = g["sampler.logits"], g["sampler.cases"]
    assert len(cases) == len(g["sampler.tokens"]) == 180
    for (row, t, tp, tk, mp, seed, counter), tok, kept in zip(cases, g["sampler.tokens"], g["sampler.kept"]):
        p = SamplingParams(temperature=float(t), top_p=float(tp), top_k=int(tk), min_p=float(mp), seed=int(seed))
        assert sample_host(logits[int(row)], p, int(counter)) == int(tok), (row, t, tp, tk, mp, seed, counter)
        assert len(sampling_distribution(logits[int(row)], p)) == int(kept)


@pytest.mark.parametrize("name", sorted(TINY))
def test_plain_float32_close_to_float64(name, tiny_model_dirs):
    mdir = tiny_model_dirs[name]
    p64, p32 = PlainQwen3(mdir, torch.float64), PlainQwen3(mdir, torch.float32)
    prompt = tiny_prompts(name)[-1]
    assert _rel(p32.logits(prompt).numpy(), p64.logits(prompt).numpy()) < 1e-5
    assert p32.greedy(prompt[:9], 4) == p64.greedy(prompt[:9], 4)
