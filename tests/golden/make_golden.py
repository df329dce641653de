"""Makes tests/golden/qwen3_reference_logits.npz: logits of the reference's own CPU backend
(src/backend/cpu/cpu_backend.cpp) on two tiny random Qwen3 models.

Run once, by hand, where the reference's sources are readable and cmake/ninja/g++ exist:

    python tests/golden/make_golden.py --reference /path/to/reference

It builds the reference's CPU library out of tree in a temporary folder, compiles
tests/golden/ref_driver.cpp against it, writes the two tiny models with this repository's
random-weights mode (bfloat16 values, so every reader widens them exactly), and stores the
reference's logits for whole prompts and for chunked feeding from a non-zero first block,
together with the two models' tensors themselves (bfloat16 bit patterns, about 100 KB each), so that the
comparison never depends on a random generator drawing the same numbers again.  It also stores tokens drawn
by the reference's host sampler (src/backend/sampling_host.cpp:68-85) for a list of (logits row, parameters,
seed, counter) cases.  tests/test_plain_golden.py compares the plain implementation and
ember_b200/sampling/host.py with these numbers.
"""
from __future__ import annotations

import argparse
import hashlib
import os
import subprocess
import sys
import tempfile

import numpy as np
import torch

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", ".."))
from tests.tiny_configs import GOLDEN_CONFIGS, TINY, tiny_config, tiny_prompts  # noqa: E402
from ember_b200.weights import write_model_dir  # noqa: E402


def weights_checksum(model_dir: str) -> str:
    with open(os.path.join(model_dir, "model.safetensors"), "rb") as f:
        return hashlib.sha256(f.read()).hexdigest()


def sampler_cases(vocab: int = 1531, rows: int = 6):
    """Logits rows with ties and clusters, and the cases drawn from them: (row, temperature, top_p, top_k,
    min_p, seed, counter)."""
    rng = np.random.default_rng(20240607)
    logits = (rng.normal(size=(rows, vocab)) * 2.0).astype(np.float32)
    logits[1, [7, 900]] = logits[1].max() + 0.5                 # a tie at the top
    logits[2] = np.round(logits[2] * 2) / 2                     # many ties everywhere
    logits[3, :40] += 6.0                                       # a cluster of likely tokens
    variants = [(0.0, 1.0, 0, 0.0), (1.0, 1.0, 0, 0.0), (0.7, 0.8, 20, 0.0), (1.3, 0.7, 0, 0.0), (0.6, 1.0, 5, 0.0),
                (1.0, 1.0, 0, 0.05), (0.9, 0.8, 20, 0.02), (1.0, 1.0, 1, 0.0), (2.0, 0.95, 100, 0.0), (0.5, 0.5, 0, 0.1)]
    cases = []
    for r in range(rows):
        for vi, (t, tp, tk, mp) in enumerate(variants):
            for rep in range(3):
                cases.append((r, t, tp, tk, mp, 1000 + 17 * vi + rep, 5 + 31 * rep + r))
    return logits, cases


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True)
    ap.add_argument("--build-dir", default=None)
    args = ap.parse_args()
    here = os.path.dirname(os.path.abspath(__file__))
    work = args.build_dir or tempfile.mkdtemp(prefix="ember-ref-")
    build = os.path.join(work, "build")
    if not os.path.isfile(os.path.join(build, "libember_core.a")):
        subprocess.check_call(["cmake", "-S", args.reference, "-B", build, "-DEMBER_CUDA=OFF", "-G", "Ninja",
                               "-DCMAKE_BUILD_TYPE=Release"])
        subprocess.check_call(["ninja", "-C", build, "ember_core"])
    driver = os.path.join(work, "ref_driver")
    subprocess.check_call(["g++", "-std=c++20", "-O2", "-I", os.path.join(args.reference, "src"),
                           "-I", os.path.join(args.reference, "tests"), os.path.join(here, "ref_driver.cpp"),
                           os.path.join(build, "libember_core.a"), "-lpthread", "-o", driver])
    out = {}
    for name in GOLDEN_CONFIGS:
        cfg = tiny_config(name)
        mdir = os.path.join(work, f"model_{name}")
        write_model_dir(cfg, mdir, seed=TINY[name]["seed"], dtype=torch.bfloat16, std=TINY[name]["std"],
                        norm_std=TINY[name]["norm_std"])
        # the reference reads model_type, which to_json writes
        out[f"{name}.checksum"] = np.frombuffer(bytes.fromhex(weights_checksum(mdir)), dtype=np.uint8)
        from ember_b200.weights import SafetensorsDir
        sd = SafetensorsDir(mdir)
        for tname in sd.names():                    # the tensors themselves, as bfloat16 bit patterns
            out[f"{name}.tensor.{tname}"] = sd.get(tname).contiguous().view(torch.int16).numpy().copy()
        for pi, prompt in enumerate(tiny_prompts(name)):
            for label, first_block, chunk in (("whole", 0, 0), ("chunk7_block2", 2, 7)):
                binf = os.path.join(work, "logits.bin")
                subprocess.check_call([driver, mdir, binf, str(first_block), str(chunk)] + [str(t) for t in prompt],
                                      stderr=subprocess.DEVNULL)
                rows = np.fromfile(binf, dtype=np.float32).reshape(-1, cfg.vocab_size)
                out[f"{name}.p{pi}.{label}"] = rows
                out[f"{name}.p{pi}.tokens"] = np.asarray(prompt, dtype=np.int32)
    logits, cases = sampler_cases()
    lbin, ctxt, otxt = (os.path.join(work, n) for n in ("sample_logits.bin", "sample_cases.txt", "sample_out.txt"))
    logits.tofile(lbin)
    with open(ctxt, "w") as f:
        for c in cases:
            f.write("%d %.9g %.9g %d %.9g %d %d\n" % c)
    subprocess.check_call([driver, "sample", lbin, str(logits.shape[1]), ctxt, otxt])
    drawn = np.loadtxt(otxt, dtype=np.int64).reshape(-1, 2)
    assert drawn.shape[0] == len(cases)
    out["sampler.logits"] = logits
    out["sampler.cases"] = np.asarray(cases, dtype=np.float64)
    out["sampler.tokens"] = drawn[:, 0].astype(np.int32)
    out["sampler.kept"] = drawn[:, 1].astype(np.int32)
    np.savez_compressed(os.path.join(here, "qwen3_reference_logits.npz"), **out)
    print("wrote", os.path.join(here, "qwen3_reference_logits.npz"), {k: v.shape for k, v in out.items()})


if __name__ == "__main__":
    main()
