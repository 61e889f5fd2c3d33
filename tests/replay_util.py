"""Driving trace replay from tests: in process, or through bin/trace_run as a user would."""
import io
import json
import os
import subprocess
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def collect(steps, out_dir, vocab):
    """(request, position) -> logits row, from the <step>.f32 files a replay wrote."""
    pos = {}
    rows = {}
    for st in steps:
        n_want = sum(len(e["want"]) for e in st["entries"])
        if n_want:
            data = np.fromfile(os.path.join(out_dir, f"{st['step']}.f32"), dtype="<f4")
            assert data.size == n_want * vocab, f"step {st['step']}: {data.size} floats"
            data = data.reshape(n_want, vocab)
        k = 0
        for e in st["entries"]:
            base = pos.get(e["id"], 0)
            for w in e["want"]:
                rows[(e["id"], base + w)] = data[k]
                k += 1
            pos[e["id"]] = base + len(e["tokens"])
        for rid in st["end"]:
            pos.pop(rid, None)
    return rows


def replay_in_process(runner, steps, out_dir):
    from llm_singularity_b200.engine.trace import replay
    lines = io.StringIO("\n".join(json.dumps(s) for s in steps) + "\n")
    log = io.StringIO()
    n = replay(runner, lines, out_dir, done=log)
    assert log.getvalue().splitlines() == [f"done {s['step']}" for s in steps]
    return n


def track_pages(runner):
    """Wrap ``runner.step`` so that after every step the pages each of its requests holds are
    noted; returns ``{group: {page id: set of requests that held it}}`` (filled as steps run)."""
    held = {}
    inner = runner.step

    def step(entries, *a, **kw):
        out = inner(entries, *a, **kw)
        for e in entries:
            for g in range(len(runner.cache.groups)):
                for page in runner.cache.pages_of(e.request, g):
                    held.setdefault(g, {}).setdefault(int(page), set()).add(e.request)
        return out

    runner.step = step
    return held


def assert_pages_were_used_again(held, seqs, max_tokens, what):
    """The pool was smaller than what all requests need together, and at least one page id of
    every group was held by two different requests over the run."""
    total = sum(-(-len(t) // 64) * 64 for t in seqs.values())
    assert max_tokens < total, f"{what}: pool of {max_tokens} tokens holds all requests ({total})"
    for g, pages in held.items():
        shared = [p for p, who in pages.items() if len(who) > 1]
        assert shared, f"{what}: no page of group {g} was handed out twice"


def replay_subprocess(model_dir, dtype, steps, out_dir, max_tokens, page_size=16, env=None):
    """Feed steps one at a time, waiting for each ``done`` line, as the protocol says."""
    cmd = [sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", model_dir,
           "--dtype", dtype, "--out", out_dir, "--max-tokens", str(max_tokens),
           "--page-size", str(page_size)]
    p = subprocess.Popen(cmd, stdin=subprocess.PIPE, stdout=subprocess.PIPE, text=True, env=env)
    try:
        for s in steps:
            p.stdin.write(json.dumps(s) + "\n")
            p.stdin.flush()
            line = p.stdout.readline().strip()
            assert line == f"done {s['step']}", f"expected 'done {s['step']}', got {line!r}"
        p.stdin.close()
        assert p.wait(timeout=120) == 0
    finally:
        if p.poll() is None:
            p.kill()


def compare(rows, ref_logits, atol, what):
    """``ref_logits``: request -> [n, vocab] tensor of the plain implementation."""
    worst, where = 0.0, None
    for (rid, pos), row in sorted(rows.items(), key=lambda kv: (str(kv[0][0]), kv[0][1])):
        d = float(np.abs(row.astype(np.float64) - ref_logits[rid][pos].numpy()).max())
        if d > worst:
            worst, where = d, (rid, pos)
        assert d <= atol, (f"{what}: first wrong place is request {rid!r} position {pos}: "
                           f"max abs diff {d:.3e} > {atol:.1e}")
    n_expected = sum(r.shape[0] for r in ref_logits.values())
    assert len(rows) == n_expected, f"{what}: {len(rows)} rows compared, {n_expected} expected"
    return worst, where
