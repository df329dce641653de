"""The plain implementation against the reference's own CPU backend (numbers made once by
tests/golden/make_golden.py) and against itself in float32."""
import hashlib
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


@pytest.mark.parametrize("name", GOLDEN_CONFIGS)
def test_plain_matches_reference_cpu_backend(name, tiny_model_dirs):
    g = np.load(GOLDEN)
    mdir = tiny_model_dirs[name]
    with open(os.path.join(mdir, "model.safetensors"), "rb") as f:
        digest = hashlib.sha256(f.read()).digest()
    if digest != bytes(g[f"{name}.checksum"]):
        pytest.skip("this torch build draws other random weights than the ones the golden logits were made with")
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


@pytest.mark.parametrize("name", sorted(TINY))
def test_plain_float32_close_to_float64(name, tiny_model_dirs):
    mdir = tiny_model_dirs[name]
    p64, p32 = PlainQwen3(mdir, torch.float64), PlainQwen3(mdir, torch.float32)
    prompt = tiny_prompts(name)[-1]
    assert _rel(p32.logits(prompt).numpy(), p64.logits(prompt).numpy()) < 1e-5
    assert p32.greedy(prompt[:9], 4) == p64.greedy(prompt[:9], 4)
