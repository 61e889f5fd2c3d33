"""llm-serve-llama: the command line, in the reference's manner.

The reference's binary takes ``--model-dir <path-or-hf-id> [--hf-token T] [--host H]
[--port P]`` and then serves HTTP (app/main.cpp:33-70).  Server, tokenizer and
download are outside this engine, so this command takes token ids and prints
token ids: prompts come from ``--prompt-ids FILE`` (a JSON list of lists, or one
prompt per line as space-separated ids) or are drawn at random (``--prompt-len``,
``--num-requests``).  ``--model-dir`` keeps its name and meaning (a local folder
with config.json and safetensors); with ``--random-weights`` the folder needs
only config.json.  ``--host``, ``--port`` and ``--hf-token`` are accepted and
ignored with a note.
"""
from __future__ import annotations

import argparse
import json
import sys
import time

import torch


def _read_prompts(path: str):
    with open(path, "r", encoding="utf-8") as f:
        text = f.read().strip()
    if text.startswith("["):
        data = json.loads(text)
        return [list(map(int, p)) for p in (data if data and isinstance(data[0], list) else [data])]
    return [[int(t) for t in line.split()] for line in text.splitlines() if line.strip()]


def build_parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(prog="llm-serve-llama", description=__doc__.split("\n\n")[0])
    ap.add_argument("--model-dir", required=True, help="folder with config.json and safetensors")
    ap.add_argument("--random-weights", action="store_true",
                    help="draw weights from --seed instead of reading safetensors")
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--dtype", default="bf16", choices=["bf16", "bfloat16", "fp32", "float32"])
    ap.add_argument("--kv-block-size", type=int, default=16)
    ap.add_argument("--num-kv-blocks", type=int, default=1024)
    ap.add_argument("--max-batch-size", type=int, default=256)
    ap.add_argument("--max-tokens-per-batch", type=int, default=2048)
    ap.add_argument("--prefill-chunk", type=int, default=None)
    ap.add_argument("--no-prefix-cache", action="store_true")
    ap.add_argument("--prompt-ids", help="file with prompts as token ids")
    ap.add_argument("--prompt-len", type=int, default=16)
    ap.add_argument("--num-requests", type=int, default=1)
    ap.add_argument("--max-new-tokens", type=int, default=16)
    ap.add_argument("--temperature", type=float, default=0.0)
    ap.add_argument("--top-k", type=int, default=0)
    ap.add_argument("--top-p", type=float, default=1.0)
    ap.add_argument("--repetition-penalty", type=float, default=1.0)
    ap.add_argument("--ignore-eos", action="store_true")
    ap.add_argument("--stats", action="store_true", help="print engine counters at the end")
    ap.add_argument("--bench", choices=["decode", "prefill", "serve"], default=None,
                    help="time instead of printing tokens: 'decode' fills --num-requests contexts of "
                         "--prompt-len and times --max-new-tokens decode steps; 'prefill' times one "
                         "prompt of --prompt-len; 'serve' runs --num-requests prompts of mixed length "
                         "(up to --prompt-len) through continuous batching")
    ap.add_argument("--device", default="cuda:0")
    for flag in ("--host", "--port", "--hf-token"):
        ap.add_argument(flag, default=None, help="accepted for compatibility; not used")
    return ap


def _sync_time(device) -> float:
    torch.cuda.synchronize(device)
    return time.perf_counter()


def run_bench(eng, args) -> dict:
    """Wall-clock timings through the public entry point (host tokens in, host tokens out),
    synchronised on both sides.  Prompts are seeded uniform-random token ids."""
    dev = eng.runner.rt.device
    g = torch.Generator().manual_seed(args.seed)
    V = eng.runner.vocab_size

    def prompt(n):
        return torch.randint(0, V, (n,), generator=g).tolist()

    out = {"bench": args.bench, "dtype": args.dtype, "prompt_len": args.prompt_len,
           "num_requests": args.num_requests}
    if args.bench == "prefill":
        times = []
        for i in range(4):                       # the first run warms up and is dropped
            eng.add_request(prompt(args.prompt_len), 1, ignore_eos=True, seed=i)
            t0 = _sync_time(dev)
            while eng.has_work():
                eng.step()
            times.append(_sync_time(dev) - t0)
        best = min(times[1:])
        out.update(seconds=round(best, 9), prompt_tokens=args.prompt_len, runs=len(times),
                   prompt_tokens_per_s=round(args.prompt_len / best, 1))
    elif args.bench == "decode":
        n_new = max(2, args.max_new_tokens)
        for i in range(args.num_requests):
            eng.add_request(prompt(args.prompt_len), n_new + 8, ignore_eos=True, seed=i)
        while any(not eng.request(r).generated for r in range(args.num_requests)):
            eng.step()                           # prompts in; every request now decodes
        for _ in range(4):
            eng.step()
        t0 = _sync_time(dev)
        made = 0
        for _ in range(n_new - 4):
            made += len(eng.step())
        dt = _sync_time(dev) - t0
        out.update(seconds=round(dt, 9), decode_steps=n_new - 4, generated_tokens=made,
                   generated_tokens_per_s=round(made / dt, 1))
        while eng.has_work():
            eng.step()
    else:
        lens = torch.randint(max(1, args.prompt_len // 16), args.prompt_len + 1,
                             (args.num_requests,), generator=g).tolist()
        for i, n in enumerate(lens):
            eng.add_request(prompt(n), args.max_new_tokens, temperature=args.temperature,
                            ignore_eos=args.ignore_eos, seed=args.seed + i)
        t0 = _sync_time(dev)
        made = 0
        while eng.has_work():
            made += sum(1 for _, tok, _ in eng.step() if tok >= 0)
        dt = _sync_time(dev) - t0
        out.update(seconds=round(dt, 9), prompt_tokens=sum(lens), generated_tokens=made,
                   generated_tokens_per_s=round(made / dt, 1),
                   total_tokens_per_s=round((made + sum(lens)) / dt, 1))
    out["stats"] = eng.stats()
    return out


def main(argv=None) -> int:
    args = build_parser().parse_args(argv)
    for flag in ("host", "port", "hf_token"):
        if getattr(args, flag) is not None:
            print(f"note: --{flag.replace('_', '-')} is ignored (no HTTP server or download here)",
                  file=sys.stderr)
    from .engine.engine import Engine
    eng = Engine(args.model_dir, random_weights=args.random_weights, seed=args.seed,
                 dtype=args.dtype, device=args.device, kv_block_size=args.kv_block_size,
                 num_kv_blocks=args.num_kv_blocks, max_batch_size=args.max_batch_size,
                 max_tokens_per_batch=args.max_tokens_per_batch, prefill_chunk=args.prefill_chunk,
                 prefix_cache=not args.no_prefix_cache, verbose=True)
    if args.bench:
        print(json.dumps(run_bench(eng, args)))
        return 0
    if args.prompt_ids:
        prompts = _read_prompts(args.prompt_ids)
    else:
        g = torch.Generator().manual_seed(args.seed)
        prompts = [torch.randint(0, eng.runner.vocab_size, (args.prompt_len,), generator=g).tolist()
                   for _ in range(args.num_requests)]
    t0 = time.time()
    outs = eng.generate(prompts, max_new_tokens=args.max_new_tokens, temperature=args.temperature,
                        top_k=args.top_k, top_p=args.top_p,
                        repetition_penalty=args.repetition_penalty, seed=args.seed,
                        ignore_eos=args.ignore_eos)
    dt = time.time() - t0
    for i, (p, o) in enumerate(zip(prompts, outs)):
        print(json.dumps({"request": i, "prompt_len": len(p), "tokens": o}))
    if args.stats:
        s = eng.stats()
        s["seconds"] = round(dt, 4)
        s["generated_tokens_per_s"] = round(sum(len(o) for o in outs) / dt, 1) if dt > 0 else None
        print(json.dumps({"stats": s}), file=sys.stderr)
    return 0


if __name__ == "__main__":
    sys.exit(main())
