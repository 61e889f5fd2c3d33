"""Trace replay: feed given token ids through the model step by step and write logits.

It samples nothing and has no forward pass, cache or loader of its own: each
input line becomes one call of :meth:`ModelRunner.step`, the same function the
scheduler drives during generation.  The reference has no such tool (its
tests/debug_dump.cpp runs three fixed prompts whole and prints top-5 values).

Input, one JSON object per line on standard input::

    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}

For a step in which something is wanted, ``<out>/<step>.f32`` holds the logits at
the wanted places, in the order of the entries and of ``want``, as little-endian
32-bit floats ``[wanted, vocab]``.  After every step a line ``done <step>`` is
printed and flushed.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
from typing import IO, Optional

import numpy as np

from .batch import StepEntry
from .runner import ModelRunner

ROUND_TO = 64            # each request's token count is rounded up to this when sizing the pool
MAX_LIVE = 16


def replay(runner: ModelRunner, lines: IO[str], out_dir: str, done: Optional[IO[str]] = None) -> int:
    """Run every step read from ``lines``; returns the number of steps run."""
    os.makedirs(out_dir, exist_ok=True)
    done = done or sys.stdout
    n = 0
    for line in lines:
        line = line.strip()
        if not line:
            continue
        msg = json.loads(line)
        step = msg["step"]
        entries = []
        for e in msg.get("entries", []):
            rid = e["id"]
            if not runner.cache.has(rid):
                if not runner.open(rid):
                    raise RuntimeError(f"step {step}: no free slot for request {rid!r} "
                                       f"({runner.max_requests} are live)")
            entries.append(StepEntry(rid, [int(t) for t in e["tokens"]],
                                     [int(w) for w in e.get("want", [])]))
        if entries:
            logits = runner.step(entries)
            if logits.shape[0]:
                host = logits.detach().to("cpu").numpy().astype("<f4", copy=False)
                with open(os.path.join(out_dir, f"{step}.f32"), "wb") as f:
                    f.write(np.ascontiguousarray(host).tobytes())
            runner.check_kernels()
        for rid in msg.get("end", []):
            if runner.cache.has(rid):
                runner.close(rid)
        print(f"done {step}", file=done, flush=True)
        n += 1
    return n


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="trace_run", description=__doc__.split("\n\n")[0])
    ap.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    ap.add_argument("--dtype", required=True, choices=["bfloat16", "float32"])
    ap.add_argument("--out", required=True, help="folder for <step>.f32 files")
    ap.add_argument("--max-tokens", type=int, required=True,
                    help="most tokens live requests hold at any time (each rounded up to 64)")
    ap.add_argument("--page-size", type=int, default=16)
    ap.add_argument("--device", default="cuda:0")
    args = ap.parse_args(argv)
    if ROUND_TO % args.page_size:
        ap.error(f"--page-size must divide {ROUND_TO}")
    capacity = -(-args.max_tokens // ROUND_TO) * ROUND_TO
    runner = ModelRunner(args.model, dtype=args.dtype, device=args.device, page_size=args.page_size,
                         num_pages=capacity // args.page_size, max_requests=MAX_LIVE,
                         max_model_len=capacity, verbose=True)
    replay(runner, sys.stdin, args.out)
    return 0
