#!/usr/bin/env python3
"""Builds sampler_driver.cpp against the reference's sampler and writes sampler_golden.json.

    python tests/golden/make_sampler_golden.py --reference <checkout of the reference>

Only the reference's host-side sampler (core/src/sampling.cpp, core/include/core/sampling.h) can be
run without a GPU; its model code has no CPU path, so the model-level plain implementation rests on
the formulas.  The JSON holds, per case, the histogram of tokens that the reference drew; the test
tests/test_sampler_golden.py checks the plain sampler's distribution against it."""
import argparse
import pathlib
import subprocess
import tempfile

here = pathlib.Path(__file__).resolve().parent


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="root of the reference's source tree")
    args = ap.parse_args()
    ref = pathlib.Path(args.reference)
    with tempfile.TemporaryDirectory() as tmp:
        exe = pathlib.Path(tmp) / "sampler_driver"
        subprocess.run(["g++", "-O2", "-std=c++17", "-I", str(ref / "core" / "include"),
                        str(here / "sampler_driver.cpp"), str(ref / "core" / "src" / "sampling.cpp"),
                        "-o", str(exe)], check=True)
        out = subprocess.run([str(exe)], check=True, capture_output=True, text=True).stdout
    (here / "sampler_golden.json").write_text(out)
    print(f"wrote {here / 'sampler_golden.json'} ({len(out)} bytes)")


if __name__ == "__main__":
    main()
