"""Makes tests/golden/qwen3_reference_logits.npz: logits of the reference's own CPU backend
(src/backend/cpu/cpu_backend.cpp) on two tiny random Qwen3 models.

Run once, by hand, where the reference's sources are readable and cmake/ninja/g++ exist:

    python tests/golden/make_golden.py --reference /path/to/reference

It builds the reference's CPU library out of tree in a temporary folder, compiles
tests/golden/ref_driver.cpp against it, writes the two tiny models with this repository's
random-weights mode (bfloat16 values, so every reader widens them exactly), and stores the
reference's logits for whole prompts and for chunked feeding from a non-zero first block,
plus a checksum of the weights.  tests/test_plain_golden.py compares the plain implementation
with these numbers.
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
        for pi, prompt in enumerate(tiny_prompts(name)):
            for label, first_block, chunk in (("whole", 0, 0), ("chunk7_block2", 2, 7)):
                binf = os.path.join(work, "logits.bin")
                subprocess.check_call([driver, mdir, binf, str(first_block), str(chunk)] + [str(t) for t in prompt],
                                      stderr=subprocess.DEVNULL)
                rows = np.fromfile(binf, dtype=np.float32).reshape(-1, cfg.vocab_size)
                out[f"{name}.p{pi}.{label}"] = rows
                out[f"{name}.p{pi}.tokens"] = np.asarray(prompt, dtype=np.int32)
    np.savez_compressed(os.path.join(here, "qwen3_reference_logits.npz"), **out)
    print("wrote", os.path.join(here, "qwen3_reference_logits.npz"), {k: v.shape for k, v in out.items()})


if __name__ == "__main__":
    main()
