"""Command line, in the reference's manner (tools/ember_main.cpp:42-79, tools/cli_args.hpp:57-88):

    python -m ember_b200 generate -m DIR -p "12 845 9" [-n 64] [--greedy | --temp T --top-p P --top-k K --min-p P --seed S]
    python -m ember_b200 bench    -m DIR [prompt=512] [gen=128] [batch=1,8,32]
    python -m ember_b200 info     -m DIR
    python -m ember_b200 random   --config CONFIG.json --out DIR [--seed S] [--weights-dtype bfloat16|float32]
    python -m ember_b200 replay   -m DIR --dtype bfloat16 --out DIR --kv-cache-tokens N < trace.jsonl

The engine starts at token ids (there is no tokenizer here): ``-p`` takes ids separated by
spaces or commas, ``--ids-file`` a file of them.  Options keep the reference's names where it
has them: ``-m/--model``, ``--max-batch-tokens`` (2048), ``--max-seqs`` (64), ``--prefill-chunk``
(2048 here, 512 there), ``--gpu-memory`` (0.92), ``--kv-cache-mib``, ``--kv-cache-tokens``, ``-n/--max-tokens`` (512), ``--temp`` (0.7), ``--top-p`` (0.8),
``--top-k`` (20), ``--min-p`` (0), ``--seed``, ``--greedy``, ``--no-cuda-graphs``, ``-v``.  ``--dtype`` (bfloat16 or
float32) stands where the reference has ``--weights``; ``--page-tokens`` (64; the reference's block is 16) and
``--max-context`` are the Python entry point's options of the same names.
"""
from __future__ import annotations

import argparse
import json
import random
import re
import statistics
import sys
import time
from typing import List


def _parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(prog="ember_b200", description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("command", choices=["generate", "gen", "bench", "info", "random", "replay"])
    ap.add_argument("-m", "--model", help="model folder (config.json + safetensors)")
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    ap.add_argument("--device", default="cuda", help="cuda (there is no cpu path)")
    ap.add_argument("--max-batch-tokens", type=int, default=2048)
    ap.add_argument("--max-seqs", type=int, default=64)
    ap.add_argument("--prefill-chunk", type=int, default=2048,
                    help="most prompt tokens of one request in a step (the reference defaults to 512 for a 6 GB GPU; a B200's tensor cores want 2,048)")
    ap.add_argument("--gpu-memory", type=float, default=0.92,
                    help="share of the device's memory to use (weights + cache + buffers); sizes the cache unless one of the next two is given")
    ap.add_argument("--kv-cache-mib", type=int, default=0, help="cache size in MiB")
    ap.add_argument("--kv-cache-tokens", type=int, default=0, help="cache size in tokens (wins over the other two)")
    ap.add_argument("--page-tokens", type=int, default=64, help="tokens per cache page (16, 32 or 64 for the tensor-core attention)")
    ap.add_argument("--max-context", type=int, default=0, help="most tokens a request may reach (0: the model's position limit)")
    ap.add_argument("--strict-weights", action="store_true", help="a tensor in the folder that the model does not use is an error")
    ap.add_argument("-n", "--max-tokens", type=int, default=512)
    ap.add_argument("--temp", "--temperature", dest="temp", type=float, default=0.7)
    ap.add_argument("--top-p", type=float, default=0.8)
    ap.add_argument("--top-k", type=int, default=20)
    ap.add_argument("--min-p", type=float, default=0.0)
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--greedy", action="store_true")
    ap.add_argument("--ignore-eos", action="store_true")
    ap.add_argument("-p", "--prompt", default="", help="token ids separated by spaces or commas")
    ap.add_argument("--ids-file", default="")
    ap.add_argument("--config", default="", help="random: the config.json to make a model for")
    ap.add_argument("--out", default="", help="random / replay: output folder")
    ap.add_argument("--weights-dtype", default="bfloat16", choices=["bfloat16", "float32"])
    ap.add_argument("--no-cuda-graphs", action="store_true", help="launch decode kernels one by one")
    ap.add_argument("-v", "--verbose", action="store_true")
    ap.add_argument("rest", nargs="*", help="bench: prompt=N gen=N batch=a,b,c")
    return ap


def _ids(text: str) -> List[int]:
    return [int(x) for x in re.split(r"[\s,]+", text.strip()) if x]


def _load(args):
    import ember_b200
    if args.device not in ("cuda", "cuda:0"):
        raise SystemExit("error: this engine runs on a CUDA device only (--device cuda)")
    if not args.model:
        raise SystemExit("error: give a model folder with -m DIR")
    llm = ember_b200.load(args.model, dtype=args.dtype, kv_cache_tokens=args.kv_cache_tokens,
                          max_batch_tokens=args.max_batch_tokens, max_seqs=args.max_seqs,
                          prefill_chunk=args.prefill_chunk, cuda_graphs=not args.no_cuda_graphs,
                          gpu_memory=args.gpu_memory, kv_cache_mib=args.kv_cache_mib, page_tokens=args.page_tokens,
                          max_context=args.max_context or None, strict_weights=args.strict_weights)
    if args.verbose:
        r = llm.runner
        print(f"[cache: {r.cache.capacity_tokens()} tokens in pages of {r.cache.page_tokens}, "
              f"{r.storage.bytes() / 2**20:.0f} MiB; context limit {llm.engine.scheduler.max_context}]", file=sys.stderr)
    return llm


def _sampling(args):
    from ember_b200 import SamplingParams
    if args.greedy:
        return SamplingParams(temperature=0.0)
    return SamplingParams(temperature=args.temp, top_p=args.top_p, top_k=args.top_k, min_p=args.min_p, seed=args.seed)


def cmd_generate(args) -> int:
    text = args.prompt or (args.rest[0] if args.rest else "")
    if args.ids_file:
        with open(args.ids_file) as f:
            text = f.read()
    prompt = _ids(text)
    if not prompt:
        raise SystemExit('error: give a prompt of token ids with -p "1 2 3"')
    llm = _load(args)
    t0 = time.perf_counter()
    out = llm.generate(prompt, sampling=_sampling(args), max_tokens=args.max_tokens, ignore_eos=args.ignore_eos)
    dt = time.perf_counter() - t0
    print(" ".join(str(t) for t in out))
    print(f"[{len(prompt)} prompt tokens | {len(out)} tokens in {dt:.2f} s | {len(out) / dt:.1f} tokens/s]", file=sys.stderr)
    return 0


def cmd_info(args) -> int:
    from ember_b200.config import load_config
    if not args.model:
        raise SystemExit("error: give a model folder with -m DIR")
    cfg = load_config(args.model)
    print(cfg.describe())
    for elem, name in ((2, "bfloat16"), (4, "float32")):
        print(f"  KV cache per token, {name}: {cfg.kv_bytes_per_token(elem) / 1024:.1f} KiB")
    return 0


def cmd_random(args) -> int:
    import torch
    from ember_b200.config import config_from_dict
    from ember_b200.weights import write_model_dir
    if not (args.config and args.out):
        raise SystemExit("error: random needs --config CONFIG.json and --out DIR")
    with open(args.config) as f:
        cfg = config_from_dict(json.load(f))
    dt = torch.bfloat16 if args.weights_dtype == "bfloat16" else torch.float32
    write_model_dir(cfg, args.out, seed=args.seed, dtype=dt)
    print(f"wrote {args.out}: {cfg.describe()}")
    return 0


def cmd_replay(args) -> int:
    from ember_b200.engine.replay import TraceReplayer
    from ember_b200.engine.runner import ModelRunner
    if not (args.model and args.out):
        raise SystemExit("error: replay needs -m DIR and --out DIR")
    cap = (max(args.kv_cache_tokens, 64) + 63) // 64 * 64
    runner = ModelRunner.from_dir(args.model, dtype=args.dtype, capacity_tokens=cap,
                                  max_batch_tokens=max(256, min(cap, 16384)), max_requests=16)
    TraceReplayer(runner, args.out).run(sys.stdin)
    return 0


def cmd_bench(args) -> int:
    """Prefill, decode and batched throughput, by the reference's method
    (tools/ember_main.cpp:323-414): random prompts (ids uniform in [1000, 100000] capped by the
    vocabulary), greedy, EOS ignored; prefill = prompt tokens / time of one request with one new
    token; generation = b * (gen - 1) / (time after every request has its first token)."""
    from ember_b200 import Request, SamplingParams
    prompt_len, gen, batches = 512, 128, [1, 8, 32]
    for a in args.rest:
        if a.startswith("prompt="):
            prompt_len = int(a[7:])
        elif a.startswith("gen="):
            gen = int(a[4:])
        elif a.startswith("batch="):
            batches = [int(x) for x in a[6:].split(",") if x]
    llm = _load(args)
    eng = llm.engine
    vocab = llm.spec.vocab_size
    # a model with a short position limit gets shorter prompts and generations than the reference's defaults
    limit = eng.scheduler.max_context
    if prompt_len + 2 > limit or 64 + gen + 1 > limit:
        prompt_len = max(1, min(prompt_len, limit // 2))
        gen = max(2, min(gen, limit - min(64, limit // 2) - 2))
        print(f"(the context limit is {limit}: prompt {prompt_len}, {gen} generated tokens)")
    rng = random.Random(1234)

    def prompt(n):
        lo, hi = min(1000, vocab - 1), min(100000, vocab - 1)
        return [rng.randint(lo, hi) for _ in range(n)]

    def run(n_req, plen, ntok):
        import torch
        seqs = [eng.submit(Request(prompt=prompt(plen), sampling=SamplingParams(temperature=0.0), max_tokens=ntok,
                                   ignore_eos=True, tag="bench")) for _ in range(n_req)]
        t0 = time.perf_counter()
        all_first = None
        while any(s.finished is None for s in seqs):
            eng.step()
            if all_first is None and all(s.generated >= 1 for s in seqs):
                torch.cuda.synchronize()
                all_first = time.perf_counter() - t0
        torch.cuda.synchronize()
        return time.perf_counter() - t0, all_first or 0.0

    print(f"ember_b200 benchmark: {args.model} ({args.dtype}), median of 3 runs")
    run(1, 64, 16)
    run(4, 64, 32)
    pre = [prompt_len / run(1, prompt_len, 1)[0] for _ in range(3)]
    print(f"  prefill, {prompt_len}-token prompt          {statistics.median(pre):10.0f} tokens/s")
    print(f"  {'decode':34s} {'generation':>14s} {'end to end':>14s}")
    for b in batches:
        g, e = [], []
        for _ in range(3):
            total, first = run(b, 32 if b == 1 else 64, gen)
            g.append(b * (gen - 1) / max(total - first, 1e-9))
            e.append(b * gen / total)
        print(f"  {b:2d} sequence{'s' if b > 1 else ' '} x {gen} tokens {'':10s} {statistics.median(g):10.1f} t/s {statistics.median(e):10.1f} t/s")
    st = eng.stats
    print(f"  ({st.steps} steps, {st.preemptions} preemptions)")
    return 0


def main(argv=None) -> int:
    # (intermixed: `bench -m DIR prompt=512 batch=1,8` has positionals after options)
    args = _parser().parse_intermixed_args(argv)
    cmd = {"generate": cmd_generate, "gen": cmd_generate, "bench": cmd_bench, "info": cmd_info,
           "random": cmd_random, "replay": cmd_replay}[args.command]
    try:
        return cmd(args)
    except (ValueError, RuntimeError, FileNotFoundError) as e:
        print(f"error: {e}", file=sys.stderr)
        return 1


if __name__ == "__main__":
    sys.exit(main())
