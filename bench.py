#!/usr/bin/env python3
"""Decode and prefill throughput of the Qwen3-1.7B shape with random weights on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--batch 8] [--impl ours|reference]

Prints ONE JSON line.  ``value`` is decoded tokens a second at the default batch (8), timed on
the device with CUDA events around K decode steps of the step function plus the sampler (the
weights alone, 3.4 GB, exceed the 126 MB L2, so nothing is flushed between steps); ``e2e`` is
the same through the Python entry point (``Engine.step``: host token ids in through pinned
memory, sampled ids back to the host, every step) by wall clock; ``prefill`` is one request of
2,048 tokens in one step; ``points`` holds decode at batch 1 and 64; ``roofline`` divides the
bytes a decode step has to read (every weight once, and the cache of the live requests) by its
time.  A "step" is one decode step.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

QWEN3_1P7B = dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", vocab_size=151936, hidden_size=2048,
                  intermediate_size=6144, num_hidden_layers=28, num_attention_heads=16, num_key_value_heads=8,
                  head_dim=128, rope_theta=1000000.0, rms_norm_eps=1e-6, tie_word_embeddings=True,
                  max_position_embeddings=40960)
CONTEXT = 4096          # decode runs up to this many positions
DECODE_FROM = 3072      # the timed decode steps start here (the middle of 2,048 -> 4,096)
PREFILL_TOKENS = 2048
PAGE_TOKENS = 64          # the engine's default; the reference's block size is 16 (--page-tokens 16: a few per cent slower, more TMA boxes a tile)
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(p):
        try:
            with open(p) as f:
                d = json.load(f)
            out = dict(FALLBACK_PEAKS)
            for k in ("hbm_gbs", "bf16_tflops", "bf16_tflops_sustained"):
                if isinstance(d.get(k), (int, float)) and d[k] > 0:
                    out[k] = float(d[k])
            out["source"] = "measured"
            return out
        except (OSError, ValueError):
            pass
    return dict(FALLBACK_PEAKS)


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.proc, self.lines = None, []

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                                          "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=lambda: self.lines.extend(self.proc.stdout), daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None
        return self

    def __exit__(self, *a):
        if self.proc:
            time.sleep(0.15)
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()
            self.thread.join(timeout=2)

    def summary(self):
        sm, mx, reasons = [], 0, set()
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 6:
                continue
            try:
                sm.append(int(f[0]))
                mx = max(mx, int(f[1]))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": int(statistics.median(sm)) if sm else None, "sm_max_mhz": mx or None,
                "reasons": sorted(reasons), "samples": len(sm)}


def model_bytes_and_flops(cfg, n_layers):
    """Bytes of weights a decode step reads once (bf16) and the flops of a T-token causal prefill."""
    H, I, V, D = cfg.hidden_size, cfg.intermediate_size, cfg.vocab_size, cfg.head_dim
    Q, KV = cfg.q_dim, cfg.kv_dim
    per_layer = H * (Q + 2 * KV) + Q * H + 3 * H * I
    weights = 2 * (n_layers * per_layer + V * H)                       # the head (tied: the embedding) is read once
    norms = 4 * (n_layers * (2 * H + 2 * D) + H)
    kv_per_token = 2 * n_layers * KV * 2                               # K and V, bf16

    def prefill_flops(T):
        linear = 2 * T * n_layers * per_layer + 2 * V * H              # head for one row
        attn = n_layers * cfg.num_attention_heads * 4 * D * (T * (T + 1) // 2)
        return linear + attn

    return weights + norms, kv_per_token, prefill_flops


def build_llm(cfg, n_layers, batch, seed=0, prefill_tokens=PREFILL_TOKENS):
    import ember_b200
    from ember_b200.config import Qwen3Config
    d = dict(cfg.to_json(), num_hidden_layers=n_layers, max_position_embeddings=max(cfg.max_position_embeddings, prefill_tokens))
    c = Qwen3Config.from_json(d)
    cap = max(batch * CONTEXT, prefill_tokens)
    return ember_b200.load_random(c, seed=seed, dtype="bfloat16", kv_cache_tokens=cap, page_tokens=PAGE_TOKENS,
                                  max_batch_tokens=max(prefill_tokens, 2048), max_seqs=max(batch, 1), prefill_chunk=2048)


def fill_cache(llm, batch, context):
    """Admits ``batch`` requests holding ``context`` tokens each without computing them: the pages
    are filled with random values (set-up only; a decode step's time does not depend on them)."""
    import torch
    r = llm.runner
    for t in r.storage._paged.values():
        t.normal_(0.0, 0.5)
    ids = []
    for i in range(batch):
        rid = ("bench", i)
        assert r.admit(rid)
        assert r.cache.ensure(rid, context)
        r.cache.advance(rid, context)
        ids.append(rid)
    return ids


def time_decode(llm, batch, steps, warmup, context):
    """K decode steps of the step function + sampler on the device; returns (ms per step, launches per step)."""
    import torch
    from ember_b200 import SamplingParams, StepEntry, ops
    from ember_b200.sampling import device as dsampler
    r = llm.runner
    ids = fill_cache(llm, batch, context)
    params = [SamplingParams(temperature=0.0)] * batch
    out = torch.empty(batch, dtype=torch.int32, device=r.device)
    vocab = r.spec.vocab_size

    def one(i):
        for rid in ids:
            assert r.reserve(rid, 1)
        entries = [StepEntry(rid, [(1000 + 7 * i + j) % vocab], (0,)) for j, rid in enumerate(ids)]
        logits = r.step(entries)
        dsampler.sample(logits, params, [context + i] * batch, out=out)

    for i in range(warmup):
        one(i)
    torch.cuda.synchronize()
    n0 = ops.launch_count()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(steps):
        one(warmup + i)
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / steps
    launches = (ops.launch_count() - n0) / steps
    r.check_device()
    for rid in ids:
        r.release(rid)
    return ms, launches


def time_e2e(llm, batch, steps, warmup, context):
    """The same decode through Engine.step: host ids in (pinned staging), sampled ids out, each step."""
    import torch
    from ember_b200 import Request, SamplingParams
    eng, r = llm.engine, llm.runner
    vocab = r.spec.vocab_size
    # requests whose prompts are already cached: prefill them for real through the engine
    import random
    rng = random.Random(1234)
    seqs = [eng.submit(Request(prompt=[rng.randrange(1000, min(100000, vocab)) for _ in range(context)],
                               sampling=SamplingParams(temperature=0.0), max_tokens=CONTEXT - context - 8, ignore_eos=True))
            for _ in range(batch)]
    while not all(s.generated >= 1 for s in seqs):
        eng.step()
    for _ in range(warmup):
        eng.step()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for _ in range(steps):
        eng.step()
    torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    for s in seqs:
        s.cancelled = True
    eng.step()
    # bytes per step: the packed int32 arrays of a decode step (tokens, positions, run index, starts, lengths,
    # slots, rows, block table) and the sampler's parameter rows in; sampled ids out
    blocks = (context + steps + warmup + 15) // 16
    ints = 3 * batch + (batch + 1) + 3 * batch + batch * blocks
    return dt * 1000.0 / steps, ints * 4 + 32 * batch, 4 * batch


def time_prefill(llm, tokens, reps, warmup):
    import torch
    from ember_b200 import StepEntry
    r = llm.runner
    vocab = r.spec.vocab_size
    import random
    rng = random.Random(4321)
    times = []
    for i in range(warmup + reps):
        rid = ("prefill", i)
        assert r.admit(rid) and r.reserve(rid, tokens)
        toks = [rng.randrange(1000, min(100000, vocab)) for _ in range(tokens)]
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        r.step([StepEntry(rid, toks, (tokens - 1,))])
        e1.record()
        torch.cuda.synchronize()
        if i >= warmup:
            times.append(e0.elapsed_time(e1))
        r.release(rid)
    r.check_device()
    return statistics.median(times)


def breakdown(cfg, n_layers, batch) -> int:
    """Per-kernel device time of decode steps and of a prefill step, kernels serialised (no programmatic
    dependent launch, no graphs), caches warm: what each kernel costs by itself inside a step."""
    os.environ["EMBER_PDL"] = "0"
    import torch
    from torch.profiler import ProfilerActivity, profile
    from ember_b200 import StepEntry
    import random
    llm = build_llm(cfg, n_layers, max(batch, 1))
    r = llm.runner
    r.cuda_graphs = False
    ids = fill_cache(llm, batch, DECODE_FROM)
    rng = random.Random(1)
    vocab = r.spec.vocab_size

    def decode():
        for rid in ids:
            assert r.reserve(rid, 1)
        r.step([StepEntry(rid, [rng.randrange(1000, min(100000, vocab))], (0,)) for rid in ids])

    def table(title, prof, steps):
        rows = [(e.key, e.self_device_time_total / steps, e.count // steps) for e in prof.key_averages()
                if e.self_device_time_total > 0]
        rows.sort(key=lambda x: -x[1])
        total = sum(x[1] for x in rows)
        print(f"{title}: {total / 1000:.3f} ms of kernels per step")
        for name, us, n in rows[:12]:
            print(f"  {us:9.1f} us {100 * us / total:5.1f} %  x{n:<4d} {name.split('(')[0][-60:]}")

    for _ in range(3):
        decode()
    torch.cuda.synchronize()
    with profile(activities=[ProfilerActivity.CUDA]) as prof:
        for _ in range(3):
            decode()
        torch.cuda.synchronize()
    table(f"decode step, batch {batch}, context {DECODE_FROM}, {n_layers} layers", prof, 3)
    for rid in ids:
        r.release(rid)
    toks = [rng.randrange(1000, min(100000, vocab)) for _ in range(PREFILL_TOKENS)]

    def prefill(i):
        rid = ("prefill", i)
        assert r.admit(rid) and r.reserve(rid, PREFILL_TOKENS)
        r.step([StepEntry(rid, toks, (PREFILL_TOKENS - 1,))])
        torch.cuda.synchronize()
        r.release(rid)

    for i in range(2):
        prefill(i)
    with profile(activities=[ProfilerActivity.CUDA]) as prof:
        prefill(2)
    table(f"prefill step, {PREFILL_TOKENS} tokens, {n_layers} layers", prof, 1)
    return 0


def main() -> int:
    global PAGE_TOKENS, CONTEXT, DECODE_FROM
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--layers", type=int, default=0, help="fewer layers than the configuration has (named in config)")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--skip-points", action="store_true", help="skip the batch 1 / 64 points and the prefill")
    ap.add_argument("--only-prefill", action="store_true", help="profiling aid: run just the 2,048-token prefill")
    ap.add_argument("--breakdown", action="store_true",
                    help="profiling aid: device time per kernel of three decode steps and one 2,048-token prefill step "
                         "(kernels serialised: EMBER_PDL=0 and no CUDA graphs are set by this flag)")
    ap.add_argument("--page-tokens", type=int, default=PAGE_TOKENS, choices=[16, 32, 64], help="tokens per cache page")
    ap.add_argument("--prefill-tokens", type=int, default=PREFILL_TOKENS,
                    help="with --only-prefill: another prompt length (the reported line stays at 2,048)")
    ap.add_argument("--decode-from", type=int, default=DECODE_FROM,
                    help="context length at which the timed decode steps start (other lengths than the default's "
                         "3,072: the cache is sized for it; `config` names it)")
    args = ap.parse_args()
    PAGE_TOKENS = args.page_tokens
    custom_context = None
    if args.decode_from != DECODE_FROM:
        custom_context = DECODE_FROM = max(1, args.decode_from)
        CONTEXT = max(CONTEXT, (DECODE_FROM + args.steps + max(3, args.warmup) + 64 + 63) // 64 * 64)      # whole pages

    if args.impl == "reference":
        # The reference is a C++/CMake program (pip: "neither setup.py nor pyproject.toml found"), so it was built
        # with its own CMake (-DEMBER_CUDA=ON -DCMAKE_CUDA_ARCHITECTURES=100: compiles and links) and driven through
        # create_backend("cuda") -> Backend::forward -> Backend::sample on this workload.  Its first step, a
        # 2,048-token prompt at these layer widths, ended with a memory fault on the B200, so its GPU code is not
        # run again here and this arm stays unavailable.
        print(json.dumps({"impl": "reference", "unavailable":
                          "the reference's CUDA backend, built unmodified with its own CMake for sm_100, faulted on a B200 "
                          "in its first step of this workload (2,048-token prompt, Qwen3-1.7B widths): 'CUDA error at "
                          "src/backend/cuda/cuda_backend.cu:214: an illegal memory access was encountered "
                          "(cudaStreamSynchronize(stream_))'; GPU code that faulted is not run again on this shared pool"}))
        return 0
    if args.gpus != 1:
        print(f"bench.py measures one GPU (this engine is single-GPU); --gpus {args.gpus} is not supported")
        return 2
    warmup = max(3, args.warmup)

    import torch
    from ember_b200.config import Qwen3Config
    cfg = Qwen3Config.from_json(QWEN3_1P7B)
    n_layers = args.layers or cfg.num_hidden_layers
    pk = peaks()
    wbytes, kv_per_token, prefill_flops = model_bytes_and_flops(cfg, n_layers)

    if args.breakdown:
        return breakdown(cfg, n_layers, args.batch)
    if args.only_prefill:
        n_tok = max(2, args.prefill_tokens)
        llm = build_llm(cfg, n_layers, 1, prefill_tokens=n_tok)
        pms = time_prefill(llm, n_tok, reps=max(1, min(5, args.steps)), warmup=min(3, warmup))
        fl = prefill_flops(n_tok)
        print(json.dumps({"prefill": {"value": round(n_tok / (pms * 1e-3), 1), "tokens": n_tok,
                                      "ms": round(pms, 3), "tflops": round(fl / (pms * 1e-3) / 1e12, 1), "layers": n_layers}}))
        return 0

    llm = build_llm(cfg, n_layers, max(args.batch, 1))
    with ClockSampler() as clocks:
        ms, launches = time_decode(llm, args.batch, args.steps, warmup, DECODE_FROM)
    # (the end-to-end loop prefills its prompts through the engine; at other context lengths than the default's the
    # first requests would be done decoding before the last has its prompt in, so it is measured at the default only)
    e2e_ms, h2d, d2h = time_e2e(llm, args.batch, args.steps, warmup, DECODE_FROM) if custom_context is None else (None, 0, 0)
    value = args.batch * 1000.0 / ms
    ctx_mid = DECODE_FROM + warmup + args.steps / 2
    step_bytes = wbytes + args.batch * ctx_mid * kv_per_token
    achieved = step_bytes / (ms * 1e-3) / 1e9

    out = {
        "metric": "decode tok/s at batch 1/8/64; prefill tok/s at 2,048 tokens (Qwen3-1.7B)",
        "value": round(value, 1), "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": warmup,
        "ms_per_step": round(ms, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic (random weights from a seed, random token ids)", "impl": "ours",
        "config": {"model": "Qwen3-1.7B shape", "global_batch": args.batch, "seq_len": CONTEXT,
                   "decode_from": DECODE_FROM, "layers": n_layers, "layers_of_config": cfg.num_hidden_layers,
                   "hidden": cfg.hidden_size, "heads": cfg.num_attention_heads, "kv_heads": cfg.num_key_value_heads,
                   "head_dim": cfg.head_dim, "intermediate": cfg.intermediate_size, "vocab": cfg.vocab_size,
                   "tied": cfg.tie_word_embeddings, "page_tokens": PAGE_TOKENS, "parallelism": "single GPU",
                   "l2": "inputs larger than L2 (3.4 GB of weights per step); no flush",
                   "peaks": pk["source"]},
        "clocks": clocks.summary(),
        "e2e": ({"value": round(args.batch * 1000.0 / e2e_ms, 1), "unit": "tokens/s", "ms_per_step": round(e2e_ms, 4),
                 "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h} if e2e_ms is not None else
                {"skipped": "measured at the default context only"}),
        "gpu_launches": int(round(launches * args.steps)),
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4), "bytes_per_step": int(step_bytes)},
    }
    del llm
    torch.cuda.empty_cache()

    if not args.skip_points:
        llm = build_llm(cfg, n_layers, 1)
        pms = time_prefill(llm, PREFILL_TOKENS, reps=5, warmup=3)
        fl = prefill_flops(PREFILL_TOKENS)
        out["prefill"] = {"value": round(PREFILL_TOKENS / (pms * 1e-3), 1), "tokens": PREFILL_TOKENS, "ms": round(pms, 3),
                          "frac": round(fl / (pms * 1e-3) / (pk["bf16_tflops"] * 1e12), 4), "tflops": round(fl / (pms * 1e-3) / 1e12, 1)}
        points = {}
        ms1, _ = time_decode(llm, 1, args.steps, warmup, DECODE_FROM)
        points["decode_b1"] = round(1000.0 / ms1, 1)
        del llm
        torch.cuda.empty_cache()
        llm = build_llm(cfg, n_layers, 64)
        ms64, _ = time_decode(llm, 64, max(8, args.steps // 2), warmup, DECODE_FROM)
        points["decode_b64"] = round(64 * 1000.0 / ms64, 1)
        points["decode_b8"] = round(value, 1)
        out["points"] = points
        del llm
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    sys.exit(main())
