#!/usr/bin/env python3
"""Builds model_driver.cpp against the reference's Llama model and writes model_golden.npz.

    python tests/golden/make_model_golden.py --reference <checkout of the reference>

Needs a GPU (the reference's model code is CUDA kernels and cuBLAS calls with no CPU path), nvcc,
and an nlohmann/json header (--json-include; by default the one bundled with the cudnn_frontend
headers of the Python environment is looked for).  The reference is compiled as it is, without
its CMake (which fetches dependencies from the network): models/llama/llama_model.cpp,
kernels/src/cublas_provider.cpp, core/src/safetensors.cpp and kernels/src/*.cu.

The model is the tiny_a configuration of tests/tiny_models.py written in 32-bit by the engine's
random-weights mode (a counter-based stream: the same folder can be made anywhere from the seed).
tiny_a lies inside what the reference can run: eps 1e-5 (fixed there, llama_model.cpp:507), no
rope scaling (only rope_theta is read, :183), pages of 16 (:113), head_dim = hidden / heads (:105).
llama3 rope scaling, another eps or page size and one pass over prompts and decode tokens together
do not exist in the reference and stay pinned by formulas.

What is recorded (the reference returns the last row of a prompt portion and every decode row,
llama_model.cpp:669-698):
  whole    three prompts (5, 17, 33 tokens) in one prefill call: their last rows;
  prefix   the 17-token prompt cut after 1 .. 17 tokens, each as a prompt of its own: every row;
  portions the 33-token prompt as 20 + 13 through prefill_start_pos: the last row;
  decode   after `whole`, eight further tokens per request, the three requests in one decode
           call per step: 24 rows.
tests/test_model_golden.py holds tests/plain_llama.py to these rows.
"""
import argparse
import glob
import os
import pathlib
import subprocess
import sys
import sysconfig
import tempfile

import numpy as np

here = pathlib.Path(__file__).resolve().parent
sys.path.insert(0, str(here.parent))
sys.path.insert(0, str(here.parent.parent))

LENGTHS = (5, 17, 33)
DECODE = 8
SPLIT = 20
BLOCKS = ((3, 0, 5), (9, 14, 8), (22, 17, 30, 16))       # page ids per request, out of order


def cases():
    """(tokens per request incl. the decode tokens, list of (label, command text, row labels))."""
    import tiny_models
    vocab = tiny_models.CONFIGS["tiny_a"]["vocab_size"]
    seqs = [tiny_models.random_tokens(vocab, n + DECODE, 7000 + n) for n in LENGTHS]

    def pre(items):
        lines = [f"prefill {len(items)}"]
        for r, start, n in items:
            lines.append(" ".join(map(str, [start, n, len(BLOCKS[r]), *BLOCKS[r], *seqs[r][start:start + n]])))
        return "\n".join(lines)

    out = []
    for n in range(1, LENGTHS[1] + 1):
        out.append((pre([(1, 0, n)]), [("prefix", 1, n - 1)]))
    out.append((pre([(2, 0, SPLIT)]), [("ignored", 2, SPLIT - 1)]))
    out.append((pre([(2, SPLIT, LENGTHS[2] - SPLIT)]), [("portions", 2, LENGTHS[2] - 1)]))
    out.append((pre([(r, 0, n) for r, n in enumerate(LENGTHS)]),
                [("whole", r, n - 1) for r, n in enumerate(LENGTHS)]))
    for k in range(DECODE):
        lines = [f"decode {len(LENGTHS)}"]
        for r, n in enumerate(LENGTHS):
            lines.append(" ".join(map(str, [n + k + 1, len(BLOCKS[r]), *BLOCKS[r], seqs[r][n + k]])))
        out.append(("\n".join(lines), [("decode", r, n + k) for r, n in enumerate(LENGTHS)]))
    return seqs, out


def find_json_include():
    for base in {sysconfig.get_paths()["purelib"], sysconfig.get_paths()["platlib"]}:
        hits = glob.glob(os.path.join(base, "**", "nlohmann", "json.hpp"), recursive=True)
        if hits:
            return str(pathlib.Path(hits[0]).parent.parent)
    return None


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="root of the reference's source tree")
    ap.add_argument("--json-include", default=None, help="folder that holds nlohmann/json.hpp")
    ap.add_argument("--out", default=str(here / "model_golden.npz"))
    args = ap.parse_args()
    ref = pathlib.Path(args.reference)
    inc = args.json_include or find_json_include()
    if inc is None:
        sys.exit("no nlohmann/json.hpp found; pass --json-include")
    import torch
    import tiny_models
    vocab = tiny_models.CONFIGS["tiny_a"]["vocab_size"]
    seqs, todo = cases()
    with tempfile.TemporaryDirectory() as tmp:
        tmp = pathlib.Path(tmp)
        exe = tmp / "model_driver"
        cmd = ["nvcc", "-O2", "-std=c++17", "-gencode", "arch=compute_100a,code=sm_100a",
               "-I", str(ref / "core" / "include"), "-I", str(ref / "kernels" / "include"),
               "-I", str(ref / "models" / "include"), "-I", str(ref / "models" / "llama"), "-I", inc,
               str(here / "model_driver.cpp"), str(ref / "models" / "llama" / "llama_model.cpp"),
               str(ref / "kernels" / "src" / "cublas_provider.cpp"),
               str(ref / "core" / "src" / "safetensors.cpp"),
               *sorted(glob.glob(str(ref / "kernels" / "src" / "*.cu"))), "-lcublas", "-o", str(exe)]
        print(" ".join(cmd), flush=True)
        subprocess.run(cmd, check=True)
        model = tiny_models.make_model_dir(str(tmp / "tiny_a"), "tiny_a", dtype=torch.float32)
        raw = tmp / "rows.f32"
        text = "\n".join(c for c, _ in todo) + "\n"
        subprocess.run([str(exe), model, str(raw)], input=text, text=True, check=True, timeout=600)
        rows = np.fromfile(raw, dtype="<f4").reshape(-1, vocab)
        probe = weights_probe(model)
    labels = [l for _, ls in todo for l in ls]
    assert len(labels) == rows.shape[0], (len(labels), rows.shape)
    keep = [i for i, l in enumerate(labels) if l[0] != "ignored"]
    np.savez_compressed(
        args.out, logits=rows[keep], kind=np.array([labels[i][0] for i in keep]),
        request=np.array([labels[i][1] for i in keep], dtype=np.int32),
        position=np.array([labels[i][2] for i in keep], dtype=np.int32),
        tokens=np.array([s + [-1] * (max(map(len, seqs)) - len(s)) for s in seqs], dtype=np.int32),
        weights_probe=np.array(probe, dtype=np.float64))
    print(f"wrote {args.out}: {len(keep)} rows of {vocab}")


def weights_probe(model_dir):
    """A few sums over the model's tensors, so that the test can tell 'the weights changed' from
    'the plain implementation disagrees with the reference'."""
    import plain_llama
    _, w = plain_llama.load_model_dir(model_dir)
    names = sorted(w)
    return [float(w[n].double().sum()) for n in names] + [float(sum(w[n].double().abs().sum() for n in names))]


if __name__ == "__main__":
    main()
